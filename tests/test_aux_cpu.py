"""Auxiliary components on CPU: pairwise and online datasets, the muP coordinate check, the evaluation-harness
adapter (against a stand-in ``lm_eval``), the S3 mirror of a checkpoint (against a stand-in ``boto3``) and the
weight server's wire protocol."""
import json
import os
import pickle
import socket
import sys
import threading
import types

import numpy as np
import pytest
import torch

from common import ROOT, make_args, run_distributed


class _FakeIndexed:
    def __init__(self, docs):
        self.docs = [np.asarray(d) for d in docs]
        self.sizes = np.asarray([len(d) for d in self.docs], dtype=np.int32)

    def get(self, i):
        return self.docs[i]


def test_pairwise_dataset_keeps_pairs_aligned():
    from gpt_neox_b200.data.pairwise_dataset import PairwiseDataset
    rng = np.random.default_rng(0)
    pos = _FakeIndexed([rng.integers(1, 99, size=n) for n in (5, 9, 3, 12, 7, 4)])
    neg = _FakeIndexed([d + 100 for d in pos.docs])                       # neg doc i = pos doc i + 100
    lab = _FakeIndexed([np.where(np.arange(len(d)) < 2, -100, d) for d in pos.docs])
    ref = _FakeIndexed([np.full(len(d), 0.5, dtype=np.float32) for d in pos.docs])
    ds = PairwiseDataset("t", "p", np.arange(6), pos, neg, num_samples=10, seq_length=15, seed=1,
                         pos_label_dataset=lab, neg_label_dataset=lab, pos_ref_dataset=ref, neg_ref_dataset=ref)
    assert len(ds) == 10
    for i in range(len(ds)):
        s = ds[i]
        assert s["pos"].shape == s["neg"].shape == (16,)
        live = s["pos"] > 0
        assert np.array_equal(s["neg"][live], s["pos"][live] + 100)        # the same document on both sides
        assert (s["pos_label"][~live] == -100).all() and s["pos_ref"].dtype == np.float32
    packed = PairwiseDataset("t", "p", np.arange(6), pos, neg, num_samples=4, seq_length=15, seed=1,
                             pack_impl="pack_until_overflow")
    assert any(len(g) > 1 for g in packed.groups)
    for g in packed.groups:
        assert sum(int(max(pos.sizes[d], neg.sizes[d])) for d in g) <= 16 or len(g) == 1
    with pytest.raises(AssertionError):
        PairwiseDataset("t", "p", np.arange(6), pos, neg, 4, 15, 1, pack_impl="packed")


def test_pairwise_dataset_caches_its_index_beside_the_corpus(tmp_path):
    """With corpora on disk the sample index is written once as ``.npy`` files and loaded afterwards; a dataset built
    only for its document count (the weighting-by-documents first pass) builds no index."""
    import glob
    from gpt_neox_b200.data.indexed_dataset import MMapIndexedDatasetBuilder, make_dataset
    from gpt_neox_b200.data.pairwise_dataset import PairwiseDataset
    rng = np.random.default_rng(0)
    docs = [rng.integers(1, 99, size=n) for n in (5, 9, 3, 12, 7, 4)]
    for side, shift in (("pos", 0), ("neg", 100)):
        b = MMapIndexedDatasetBuilder(str(tmp_path / side) + ".bin", dtype=np.uint16)
        for d in docs:
            b.add_item(np.asarray(d + shift, dtype=np.uint16))
            b.end_document()
        b.finalize(str(tmp_path / side) + ".idx")
    pos, neg = make_dataset(str(tmp_path / "pos"), "mmap"), make_dataset(str(tmp_path / "neg"), "mmap")
    mk = lambda **kw: PairwiseDataset("train_0", str(tmp_path / "pos"), np.arange(6), pos, neg, num_samples=5,
                                      seq_length=15, seed=3, pack_impl="pack_until_overflow", **kw)
    count_only = mk(build_index_mappings=False)
    assert len(count_only) == 0 and count_only.indexed_dataset.sizes.shape[0] == 6
    assert not glob.glob(str(tmp_path / "*pairmap*"))
    first = mk()
    files = sorted(glob.glob(str(tmp_path / "*pairmap*")))
    assert len(files) == 2 and len(first) == 5
    groups = first.groups
    s = first[0]
    live = s["pos"] > 0
    assert np.array_equal(s["neg"][live], s["pos"][live] + 100)
    # the second construction reads the files: swap two samples in the cached boundaries' documents and see it
    doc_file = [f for f in files if f.endswith("_doc_idx.npy")][0]
    saved = np.load(doc_file)
    np.save(doc_file, saved[::-1].copy())
    again = mk()
    assert [d for g in again.groups for d in g] == [d for g in groups for d in g][::-1]


def test_online_dataset_consumes_a_sampling_server():
    from gpt_neox_b200.data.online_dataset import OnlineDataset
    batch = {"prefix": [5, 6, 7], "completions": [[8, 9], [10], [11, 12, 13]], "rewards": [1.0, 0.0, 2.0]}
    srv = socket.socket()
    srv.bind(("127.0.0.1", 0))
    srv.listen(4)
    port = srv.getsockname()[1]

    def serve():
        for _ in range(2):
            conn, _ = srv.accept()
            assert conn.recv(64) == b"train"
            conn.sendall(pickle.dumps(batch))
            conn.close()
    threading.Thread(target=serve, daemon=True).start()
    ds = OnlineDataset(num_samples=6, seq_length=8, leave_one_out=True, dataserver_ips="127.0.0.1", dataserver_ports=port)
    items = [ds[i] for i in range(3)]
    assert [int(x["raw_reward"]) for x in items] == [1, 0, 2]
    # leave-one-out baseline: reward minus the mean of the other completions' rewards
    assert np.allclose([x["reward"][0] for x in items], [1 - 1.0, 0 - 1.5, 2 - 0.5])
    first = items[0]
    assert first["text"][:5].tolist() == [5, 6, 7, 8, 9] and first["label"][:5].tolist() == [-100, -100, -100, 8, 9]
    assert (first["label"][5:] == -100).all()
    assert ds[3]["text"][:3].tolist() == [5, 6, 7]        # second request to the server


def _coord_check(rank, world, out_dir):
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.mup_support import mup_coord_check
    from gpt_neox_b200.utils import Timers
    args = make_args(hidden_size=32, num_attention_heads=4, num_layers=2, use_mup=True, coord_check=True,
                     base_shapes_file=os.path.join(out_dir, "base"), global_num_gpus=world)
    args.configure_distributed_args()
    initialize_megatron(args)
    g = torch.Generator().manual_seed(0)

    def it():
        while True:
            yield {"text": torch.randint(0, args.padded_vocab_size, (2, 33), generator=g)}
    up, sp = mup_coord_check(args, Timers(), it(), widths=[32, 64, 128], nsteps=2, out_dir=out_dir)
    assert set(up.width) == {32, 64, 128} and set(up.t) == {1, 2} and len(up) == len(sp) > 0
    assert np.isfinite(up.l1).all() and np.isfinite(sp.l1).all()
    assert args.hidden_size == 32 and args.use_mup is True          # the run's own settings are restored


def test_mup_coordinate_check_writes_both_tables(tmp_path):
    run_distributed(_coord_check, 1, str(tmp_path))
    for tag in ("up", "sp"):
        assert os.path.getsize(tmp_path / f"coord_check_{tag}.0.csv") > 0


def _adapter(rank, world, out):
    from gpt_neox_b200.eval_tasks.eval_adapter import EvalHarnessAdapter
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.training import forward_step, setup_model_and_optimizer
    args = make_args(global_num_gpus=world, seq_length=32)
    args.configure_distributed_args()
    initialize_megatron(args)
    model, _, _, _ = setup_model_and_optimizer(args)
    ad = EvalHarnessAdapter(model, forward_step, args, batch_size=3)
    reqs = [("the quick brown", " fox"), ("", "hello"), ("abc" * 30, "xyz"), ("q", " a b c")]
    res = ad.loglikelihood(reqs)
    assert len(res) == 4 and all(r[0] < 0 and isinstance(r[1], bool) for r in res)
    # scoring does not depend on how requests are batched
    solo = [ad.loglikelihood([r])[0] for r in reqs]
    assert all(abs(a[0] - b[0]) < 1e-3 for a, b in zip(res, solo)), (res, solo)
    roll = ad.loglikelihood_rolling(["some longer text " * 8])
    assert len(roll) == 1 and roll[0] < 0
    gen = ad.generate_until([("hello", {"until": ["\\n"]})])
    assert len(gen) == 1 and isinstance(gen[0], str)

    # the harness driver, against a stand-in lm_eval package that calls back into the three request types
    calls = {}

    class LM:
        pass

    def evaluate(lm, task_dict, limit=None, bootstrap_iters=0, log_samples=False):
        calls["ll"] = lm.loglikelihood([("ctx", " cont")])
        calls["roll"] = lm.loglikelihood_rolling(["text"])
        calls["gen"] = lm.generate_until([("hi", {"until": ["."]})])
        return {"results": {t: {"acc": 0.5} for t in task_dict}}
    pkg = types.ModuleType("lm_eval")
    pkg.evaluator = types.SimpleNamespace(evaluate=evaluate)
    pkg.tasks = types.SimpleNamespace(TaskManager=lambda: None, get_task_dict=lambda names, tm: {n: object() for n in names})
    pkg.utils = types.SimpleNamespace()
    api = types.ModuleType("lm_eval.api")
    api_model = types.ModuleType("lm_eval.api.model")
    api_model.LM = LM
    sys.modules.update({"lm_eval": pkg, "lm_eval.api": api, "lm_eval.api.model": api_model})
    out_res = ad.run_eval(eval_tasks=["lambada_openai", "piqa"], num_fewshot=0)
    assert set(out_res["results"]) == {"lambada_openai", "piqa"} and out_res["config"]["model"] == "neox"
    assert len(calls["ll"]) == 1 and len(calls["roll"]) == 1 and len(calls["gen"]) == 1
    if rank == 0:
        with open(out, "w") as fh:
            json.dump([r[0] for r in res], fh)


def test_eval_harness_adapter_scores_and_drives_the_harness(tmp_path):
    run_distributed(_adapter, 1, str(tmp_path / "scores.json"))
    assert len(json.load(open(tmp_path / "scores.json"))) == 4


def test_s3_upload_mirrors_the_checkpoint_tree(tmp_path, monkeypatch):
    from gpt_neox_b200 import checkpointing as C
    save = tmp_path / "run1"
    tag = save / "global_step7"
    (tag / "configs").mkdir(parents=True)
    (tag / "mp_rank_00_model_states.pt").write_bytes(b"x" * 10)
    (tag / "configs" / "a.yml").write_text("{}")
    uploaded = []

    class Client:
        def upload_file(self, path, bucket, key, Config=None):
            uploaded.append((os.path.relpath(path, tag), bucket, key, Config.multipart_chunksize))
    boto3 = types.ModuleType("boto3")
    boto3.client = lambda kind: Client()
    s3 = types.ModuleType("boto3.s3")
    transfer = types.ModuleType("boto3.s3.transfer")

    class TransferConfig:
        def __init__(self, **kw):
            self.__dict__.update(kw)
    transfer.TransferConfig = TransferConfig
    monkeypatch.setitem(sys.modules, "boto3", boto3)
    monkeypatch.setitem(sys.modules, "boto3.s3", s3)
    monkeypatch.setitem(sys.modules, "boto3.s3.transfer", transfer)
    args = types.SimpleNamespace(save=str(save), s3_path="s3://bucket/prefix", s3_chunk_size=1 << 20)
    C.upload_checkpoint(7, args)
    assert sorted(u[0] for u in uploaded) == ["configs/a.yml", "mp_rank_00_model_states.pt"]
    assert all(b == "bucket" and k.startswith("prefix/run1/global_step7/") and c == 1 << 20 for _, b, k, c in uploaded)


def test_weight_server_answers_with_a_length_prefixed_map():
    from gpt_neox_b200 import weight_server as W
    model = types.SimpleNamespace(module=torch.nn.Linear(4, 4))       # CPU parameters: nothing to share, empty map
    with socket.socket() as s:
        s.bind(("localhost", 0))
        port = s.getsockname()[1]
    W.start_server(model, ports=port)
    for _ in range(50):
        try:
            c = socket.create_connection(("localhost", port), timeout=2)
            break
        except ConnectionRefusedError:
            import time
            time.sleep(0.1)
    n = int.from_bytes(c.recv(8), "little")
    payload = b""
    while len(payload) < n:
        payload += c.recv(n - len(payload))
    assert pickle.loads(payload) == {}


# ------------------------------------------------------------------ comms logger / flops profiler
def _comms_worker(rank, world, port, q):
    import os
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from gpt_neox_b200.parallel import comms_logger
    stock = dist.all_reduce
    log = comms_logger.configure({"enabled": True, "verbose": False, "prof_all": True})
    x = torch.ones(1024)
    for _ in range(3):
        dist.all_reduce(x)
    out = torch.empty(2048)
    dist.all_gather_into_tensor(out, torch.ones(1024))
    w = dist.all_reduce(torch.ones(256), async_op=True)
    w.wait()
    comms_logger.record_fused("fused_gemm_reduce_scatter", 1 << 20, world)
    rows = log.summary()
    text = log.log_summary(print_fn=lambda s: None)
    log.uninstall()
    assert dist.all_reduce is stock
    dist.destroy_process_group()
    q.put((rank, rows, text))


def test_comms_logger_counts_sizes_and_bandwidth():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29000 + os.getpid() % 2000
    procs = [ctx.Process(target=_comms_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(30)
        assert p.exitcode == 0
    for rank, rows, text in res:
        by = {(op, nbytes): (count, total, mean, alg, bus) for op, nbytes, count, total, mean, alg, bus in rows}
        assert by[("all_reduce", 4096)][0] == 3 and by[("all_reduce", 1024)][0] == 1
        assert by[("all_gather_into_tensor", 8192)][0] == 1
        assert by[("fused_gemm_reduce_scatter", 1 << 20)][0] == 1
        count, total, mean, alg, bus = by[("all_reduce", 4096)]
        assert total > 0 and abs(mean - total / 3) < 1e-9 and abs(bus - alg * 1.0) < 1e-6     # 2 (n-1)/n = 1 at n = 2
        assert "all_reduce" in text and "busbw_avg" in text


def test_comms_logger_disabled_leaves_torch_distributed_alone():
    import torch.distributed as dist
    from gpt_neox_b200.parallel import comms_logger
    before = dist.all_reduce
    log = comms_logger.configure({"enabled": False})
    assert dist.all_reduce is before and not log.enabled
    log = comms_logger.configure({"enabled": True, "prof_all": False, "prof_ops": ["all_reduce"]})
    assert dist.all_reduce is not before and log.wants("all_reduce") and not log.wants("broadcast")
    log.uninstall()
    assert dist.all_reduce is before
    comms_logger.configure(None)


def _flops_worker(rank, world, out_file):
    import torch
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.training import setup_model_and_optimizer, train_step
    from gpt_neox_b200.utils import Timers
    from gpt_neox_b200.utils.flops_profiler import FlopsProfiler
    from common import make_args
    counts = []
    for ckpt in (False, True):
        args = make_args(global_num_gpus=1, checkpoint_activations=ckpt, checkpoint_num_layers=1)
        args.configure_distributed_args()
        if not counts:
            initialize_megatron(args)
        model, opt, sched, _ = setup_model_and_optimizer(args)
        g = torch.Generator().manual_seed(0)
        batch = {"text": torch.randint(0, args.padded_vocab_size, (2, args.seq_length + 1), generator=g)}
        prof = FlopsProfiler.from_config(model.module, {"enabled": True, "profile_step": 1, "module_depth": 2,
                                                        "top_modules": 3, "detailed": True, "output_file": out_file})
        prof.start_profile()
        train_step(args, Timers(), iter([batch]), model, opt, sched)
        prof.stop_profile()
        text = prof.report(batch_size=2)
        T, h, s, L, V = 2 * args.seq_length, args.hidden_size, args.seq_length, args.num_layers, args.padded_vocab_size
        expect = L * (2 * T * h * (3 * h + h + 4 * h + 4 * h) + 4 * 2 * args.num_attention_heads * s * s
                      * (h // args.num_attention_heads) * 0.5) + 2 * T * h * V
        assert abs(prof.total_flops() - expect) / expect < 1e-6, (prof.total_flops(), expect)
        assert "fwd flops per GPU" in text and "depth 1:" in text and open(out_file).read().strip() == text.strip()
        counts.append(prof.total_flops())
    assert counts[0] == counts[1]           # a recomputed forward is not counted a second time


def test_flops_profiler_counts_forward_flops_of_a_small_model(tmp_path):
    from common import run_distributed
    run_distributed(_flops_worker, 1, str(tmp_path / "flops.txt"))


# ------------------------------------------------------------------ autotuner
def _tuning_args(tmp_path, **block):
    from common import make_args
    return make_args(global_num_gpus=1, zero_optimization={"stage": "auto"},
                     autotuning={"enabled": True, "start_profile_step": 1, "end_profile_step": 3,
                                 "num_tuning_micro_batch_sizes": 3, "results_dir": str(tmp_path / "results"),
                                 "exps_dir": str(tmp_path / "exps"), **block})


def test_autotuner_search_with_a_stand_in_runner(tmp_path):
    import json
    from gpt_neox_b200.autotuning import Autotuner
    args = _tuning_args(tmp_path)
    seen = []

    def runner(trial):
        # throughput grows with the micro-batch; stage 1 is a little slower; micro-batch 4 "runs out of memory" at stage 0
        mb, stage = trial.train_micro_batch_size_per_gpu, trial.zero_optimization["stage"]
        seen.append((stage, mb, trial.train_iters, trial.save, trial.autotuning_run))
        assert trial.train_batch_size == mb * trial.gradient_accumulation_steps
        if stage == 0 and mb == 4:
            return 1
        with open(trial.autotuning_metric_path, "w") as fh:
            json.dump({"throughput": 100.0 * mb - 10 * stage, "latency": 1.0 / mb, "tokens_per_sec": 1.0}, fh)
        return 0

    tuner = Autotuner(args, runner=runner)
    assert tuner.micro_batch_sizes() == [1, 2, 4] and tuner.zero_stages() == [0, 1, 2, 3]
    best = tuner.tune()
    # five trials in a row without an improvement (the default patience) end the search one trial early
    assert [s[:2] for s in seen] == [(z, mb) for z in (0, 1, 2, 3) for mb in (1, 2, 4)][:-1]
    assert all(s[2] == 4 and s[3] is None and s[4] is None for s in seen)
    assert best["zero_stage"] == 1 and best["micro_batch"] == 4 and best["throughput"] == 390.0
    summary = json.load(open(tmp_path / "results" / "summary.json"))
    assert summary["best"]["name"] == "z1_mbs4" and len(summary["experiments"]) == 11
    assert "failed (1)" in open(tmp_path / "results" / "summary.txt").read()
    final = tuner.apply_best(best)
    assert final.train_micro_batch_size_per_gpu == 4 and final.zero_optimization["stage"] == 1
    assert final.autotuning_run is None
    # latency as the metric: lower is better; early stopping after one non-improving trial
    tuner = Autotuner(_tuning_args(tmp_path, metric="latency", tuner_early_stopping=1, tune_zero_stage=False),
                      runner=runner)
    assert tuner.tune()["micro_batch"] == 2          # stage 0: 1, 2 ok, 4 fails


def test_autotuner_runs_a_real_trial_through_the_launcher(tmp_path):
    """One trial end to end on CPU: the launcher starts the training script, the training loop writes the metric."""
    import json
    from gpt_neox_b200.autotuning import Autotuner
    args = _tuning_args(tmp_path, num_tuning_micro_batch_sizes=1)
    args.update_values({"user_script": os.path.join(ROOT, "train.py"), "zero_optimization": {"stage": 0},
                        "num_gpus": 1, "master_port": 29000 + os.getpid() % 2000})
    best = Autotuner(args).tune()
    assert best is not None and best["exit_code"] == 0 and best["throughput"] > 0 and best["latency"] > 0
    assert json.load(open(tmp_path / "exps" / "z0_mbs1" / "metric.json"))["tokens_per_sec"] > 0


def test_csv_monitor_sink_and_comet_settings(tmp_path, monkeypatch):
    """``csv_monitor`` writes one ``step,value`` file per metric; the Comet experiment gets its name, tags, other
    fields and the non-default configuration (against a stand-in ``comet_ml``)."""
    from gpt_neox_b200 import logging as L
    mon = L.configure_csv_monitor({"enabled": True, "output_path": str(tmp_path), "job_name": "job"})
    try:
        for it, v in ((1, 2.5), (2, 2.25)):
            L.tb_wandb_log("train/lm_loss", v, it, use_wandb=False)
        L.tb_wandb_log("runtime/tokens_per_sec", 1000.0, 2, use_wandb=False)
    finally:
        mon.close()
        L.configure_csv_monitor(None)
    rows = open(tmp_path / "job" / "train_lm_loss.csv").read().split()
    assert rows == ["step,train/lm_loss", "1,2.5", "2,2.25"]
    assert os.path.exists(tmp_path / "job" / "runtime_tokens_per_sec.csv")
    L.tb_wandb_log("train/lm_loss", 1.0, 3, use_wandb=False)                 # disabled again: nothing is appended
    assert len(open(tmp_path / "job" / "train_lm_loss.csv").read().split()) == 3

    calls = {}

    class Experiment:
        def __init__(self, **kw):
            calls["init"] = kw

        def log_parameters(self, d):
            calls["params"] = d

        def set_name(self, n):
            calls["name"] = n

        def add_tags(self, t):
            calls["tags"] = t

        def log_others(self, o):
            calls["others"] = o
    monkeypatch.setitem(sys.modules, "comet_ml", types.SimpleNamespace(Experiment=Experiment))
    args = make_args(use_comet=True, comet_workspace="ws", comet_project="proj", comet_experiment_name="run-7",
                     comet_tags=["b200", "125M"], comet_others={"note": "x"})
    args.rank = 0
    args.initialize_comet()
    assert calls["init"] == {"workspace": "ws", "project_name": "proj"} and calls["name"] == "run-7"
    assert calls["tags"] == ["b200", "125M"] and calls["others"] == {"note": "x"}
    assert calls["params"]["comet_project"] == "proj"


def _dump_state(rank, world):
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.training import setup_model_and_optimizer
    args = make_args(global_num_gpus=world, dump_state=True, zero_optimization={"stage": 1})
    args.configure_distributed_args()
    initialize_megatron(args)
    engine, *_ = setup_model_and_optimizer(args)
    from gpt_neox_b200.training import dump_engine_state
    rows = dump_engine_state(engine, args)
    assert rows["engine"] == "NeoXEngine" and rows["zero_stage"] == 1 and rows["buckets"] >= 1
    assert rows["optimizer"] == "FusedAdam" and rows["total_params"] == engine.total_params


def test_dump_state_prints_the_engine_configuration(capfd):
    run_distributed(_dump_state, 1)
    assert "engine state:" in capfd.readouterr().out
