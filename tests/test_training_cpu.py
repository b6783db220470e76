"""End-to-end training on CPU (gloo): loss decreases, ZeRO-1 == ZeRO-0, pipeline 1F1B trains, checkpoints
round-trip bit-exactly (the reference's own -- skipped -- model tests define these contracts:
tests/model/test_model_train.py:72-93, test_model_checkpoint.py:80-127)."""
import json
import os

import pytest
import torch

from common import make_args, run_distributed, run_distributed_many


def _setup(cfg):
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.training import setup_model_and_optimizer
    args = make_args(**cfg)
    args.configure_distributed_args()
    initialize_megatron(args)
    model, opt, sched, _ = setup_model_and_optimizer(args)
    return args, model, opt, sched


def _fixed_batches(args, n=4):
    from gpt_neox_b200.parallel import mpu
    g = torch.Generator().manual_seed(100 + mpu.get_data_parallel_rank())
    batches = [{"text": torch.randint(0, args.padded_vocab_size, (args.train_micro_batch_size_per_gpu,
                                                                   args.seq_length + 1), generator=g)}
               for _ in range(n)]

    def it():
        i = 0
        while True:
            yield batches[i % n]
            i += 1
    return it()


def _train(args, model, opt, sched, steps, it=None):
    from gpt_neox_b200.training import train_step
    from gpt_neox_b200.utils import Timers
    it = it or _fixed_batches(args)
    losses = []
    for _ in range(steps):
        d, _ = train_step(args, Timers(), it, model, opt, sched)
        losses.append(float(d["lm_loss"]))
    return losses


def _loss_decreases(rank, world, cfg, out):
    args, model, opt, sched = _setup({**cfg, "global_num_gpus": world})
    losses = _train(args, model, opt, sched, 12)
    assert min(losses) < losses[0], losses
    if rank == 0 and out:
        with open(out, "w") as fh:
            json.dump(losses, fh)


@pytest.mark.parametrize("cfg", [
    {},                                                                      # GPT-NeoX style: rotary, parallel residual
    {"gpt_j_residual": False, "norm": "rmsnorm", "activation": "swiglu", "use_bias_in_mlp": False,
     "use_bias_in_attn_linear": False, "rotary_pct": 1.0, "num_kv_heads": 2, "intermediate_size": 192},   # llama style
    {"pos_emb": "alibi", "no_weight_tying": False},                          # ALiBi + tied embeddings
    {"pos_emb": "learned", "checkpoint_activations": True, "gradient_accumulation_steps": 2,
     "hidden_dropout": 0.1, "attention_dropout": 0.1},
    {"pos_emb": "rpe", "gpt_j_residual": False},
    {"precision": "bfloat16", "zero_optimization": {"stage": 1}},
    {"precision": "fp16", "fp16": {"enabled": True, "loss_scale": 0, "initial_scale_power": 8}},
    {"use_bnb_optimizer": True},                                             # block-wise 8-bit Adam states + stable embedding
    {"checkpoint_activations": True, "checkpoint_in_cpu": True},
])
def test_loss_decreases_single_process(cfg):
    run_distributed(_loss_decreases, 1, cfg, None)


def test_zero1_matches_zero0(tmp_path):
    a, b = str(tmp_path / "z0.json"), str(tmp_path / "z1.json")
    run_distributed_many((_loss_decreases, 2, {"zero_optimization": {"stage": 0}}, a),
                         (_loss_decreases, 2, {"zero_optimization": {"stage": 1}}, b))
    l0, l1 = json.load(open(a)), json.load(open(b))
    assert all(abs(x - y) < 1e-4 for x, y in zip(l0, l1)), (l0, l1)


@pytest.mark.parametrize("extra", [
    {"zero_optimization": {"stage": 1, "cpu_offload": True}},
    {"zero_optimization": {"stage": 2, "offload_optimizer": {"device": "cpu", "pin_memory": True},
                           "reduce_bucket_size": 20000}, "precision": "bfloat16"},
    {"zero_optimization": {"stage": 3, "cpu_offload": True, "reduce_bucket_size": 20000}},
    {"zero_optimization": {"stage": 3, "cpu_offload": True, "offload_param": {"device": "cpu"},
                           "reduce_bucket_size": 20000}, "precision": "bfloat16"},
    {"zero_optimization": {"stage": 1}, "weight_decay": 0.0,
     "optimizer": {"type": "cpu_torch_adam", "params": {"lr": 1e-3, "betas": [0.9, 0.95], "eps": 1e-8}}},
])
def test_optimizer_state_offload_matches_device_states(extra, tmp_path):
    """Masters and Adam states in host memory, updated by the C++ host kernel (or torch's Adam): the same losses as
    the device-resident optimizer at every ZeRO stage, in fp32 and bf16 (where the host kernel also produces the
    rounded 16-bit shard that is copied back)."""
    a, b = str(tmp_path / "dev.json"), str(tmp_path / "host.json")
    base = {k: v for k, v in extra.items() if k != "optimizer"}
    zero = dict(base.get("zero_optimization", {}))
    zero.pop("cpu_offload", None)
    zero.pop("offload_optimizer", None)
    zero.pop("offload_param", None)
    if "optimizer" in extra:              # torch's Adam on host masters against the device Adam, same settings
        base["optimizer"] = {"type": "Adam", "params": extra["optimizer"]["params"]}
    run_distributed_many((_loss_decreases, 2, {**base, "zero_optimization": zero}, a),
                         (_loss_decreases, 2, extra, b))
    l0, l1 = json.load(open(a)), json.load(open(b))
    tol = 2e-2 if extra.get("precision") == "bfloat16" else 1e-4
    assert all(abs(x - y) < tol for x, y in zip(l0, l1)), (l0, l1)


def _offload_layout(rank, world):
    """Where things live with offload on: masters, gradients-for-the-step and optimizer states on the host."""
    args, model, opt, sched = _setup({"global_num_gpus": world, "precision": "bfloat16",
                                      "zero_optimization": {"stage": 1, "cpu_offload": True}})
    from gpt_neox_b200.optim.cpu_adam import CPUAdam
    assert opt.offload_optimizer and isinstance(opt.optimizer, CPUAdam)
    _train(args, model, opt, sched, 2)
    for b in opt.buckets:
        assert b.offload and b.master.device.type == "cpu" and b.host_out.dtype == torch.bfloat16
        st = opt.optimizer.state[b.master]
        assert st["exp_avg"].device.type == "cpu" and "host_param" not in st     # updated in place
        # the parameter buffer holds exactly the bf16 rounding of the host master shard
        assert torch.equal(b.flat_param[b.lo:b.hi].cpu(), b.master.data.bfloat16())


def test_optimizer_state_offload_layout():
    run_distributed(_offload_layout, 2)


def _host_staged_construction(rank, world):
    """Stage 3 with parameter offload: layers are parked on the host as they are built, and the optimizer reduces
    every bucket to this rank's shard before it lays out the next one."""
    from gpt_neox_b200.engine import pipe_module
    parked = []
    real_to = torch.nn.Module.to

    def spy(self, *a, **kw):
        if pipe_module.LayerSpec._post_build is not None and a and a[0] == "cpu":
            parked.append(type(self).__name__)
        return real_to(self, *a, **kw)
    torch.nn.Module.to = spy
    try:
        args, model, opt, sched = _setup({"global_num_gpus": world, "precision": "bfloat16",
                                          "zero_optimization": {"stage": 3, "cpu_offload": True,
                                                                "offload_param": {"device": "cpu"},
                                                                "reduce_bucket_size": 20000}})
    finally:
        torch.nn.Module.to = real_to
    assert pipe_module.LayerSpec._post_build is None                 # the hook does not outlive the construction
    assert len(parked) >= args.num_layers + 2, parked               # embedding, every block, the final layers
    sharded = [b for b in opt.buckets if b.partition_grads]
    assert len(sharded) > 2 and opt.max_resident_at_build == 1
    assert all(b.flat_param is None and b.partition_params and b.param_shard.device.type == "cpu" for b in sharded)
    losses = _train(args, model, opt, sched, 6)
    assert min(losses) < losses[0]


def test_zero3_param_offload_builds_the_model_through_the_host():
    run_distributed(_host_staged_construction, 2)


def _overlap_losses(rank, world, cfg, out):
    args, model, opt, sched = _setup({**cfg, "global_num_gpus": world})
    losses = _train(args, model, opt, sched, 8)
    if rank == 0:
        with open(out, "w") as fh:
            json.dump({"losses": losses, "overlapped": getattr(opt, "overlapped_reductions", 0),
                       "buckets": len(getattr(opt, "buckets", []))}, fh)


def test_zero1_overlapped_reduction_matches_plain(tmp_path):
    """Bucketed gradient reduce-scatter started from backward hooks + asynchronous parameter all-gather give the
    same losses as the reduce-at-step form, and the early path is really taken."""
    a, b = str(tmp_path / "plain.json"), str(tmp_path / "overlap.json")
    base = {"gradient_accumulation_steps": 2}
    run_distributed_many((_overlap_losses, 2, {**base, "zero_optimization": {"stage": 1}}, a),
                         (_overlap_losses, 2, {**base, "zero_optimization": {"stage": 1, "overlap_comm": True,
                                                                             "reduce_bucket_size": 20000}}, b))
    ra, rb = json.load(open(a)), json.load(open(b))
    assert all(abs(x - y) < 1e-4 for x, y in zip(ra["losses"], rb["losses"])), (ra, rb)
    assert rb["buckets"] > ra["buckets"] and rb["overlapped"] > 0, rb


@pytest.mark.parametrize("world,cfg", [
    (4, {"model_parallel_size": 2, "sequence_parallel": True}),        # norm gradients are all-reduced after backward
    (2, {"no_weight_tying": False}),                                   # the embedding weight is used twice
    (4, {"pipe_parallel_size": 2, "num_layers": 4, "no_weight_tying": False}),   # tied across pipeline stages
])
def test_overlapped_reduction_leaves_late_gradients_alone(tmp_path, world, cfg):
    """Gradients that are completed only after backward (sequence-parallel norm gradients, weights tied across
    layers or stages) must not be part of an early data-parallel reduction: the run with overlap reproduces
    the losses of the run without it, and other buckets are still reduced early."""
    a, b = str(tmp_path / "plain.json"), str(tmp_path / "overlap.json")
    base = {"gradient_accumulation_steps": 2, **cfg}
    run_distributed_many((_overlap_losses, world, {**base, "zero_optimization": {"stage": 1}}, a),
                         (_overlap_losses, world, {**base, "zero_optimization": {"stage": 1, "overlap_comm": True,
                                                                                 "reduce_bucket_size": 20000}}, b))
    ra, rb = json.load(open(a)), json.load(open(b))
    assert all(abs(x - y) < 1e-5 for x, y in zip(ra["losses"], rb["losses"])), (ra, rb)
    assert rb["overlapped"] > 0, rb


def _recompute_losses(rank, world, cfg, skip, out):
    from gpt_neox_b200.parallel import rng
    rng.set_recompute_skip(skip)
    args, model, opt, sched = _setup({**cfg, "global_num_gpus": world, "checkpoint_activations": True})
    losses = _train(args, model, opt, sched, 6)
    if rank == 0:
        with open(out, "w") as fh:
            json.dump(losses, fh)


@pytest.mark.parametrize("world,cfg", [
    (1, {}),                                                              # parallel residual: dense and linear2 skipped
    (1, {"gpt_j_residual": False, "use_bias_in_mlp": False}),             # sequential residual: linear2 skipped
    (2, {"model_parallel_size": 2}),                                      # ... and the tensor-parallel all-reduce
    (2, {"model_parallel_size": 2, "sequence_parallel": True, "checkpoint_num_layers": 2}),
    (2, {"pipe_parallel_size": 2, "num_layers": 4, "gradient_accumulation_steps": 2}),
])
def test_recomputation_skips_the_block_tail_without_changing_the_training(tmp_path, world, cfg):
    """When a checkpointed block is re-run in backward the output of its last layer is never read; the GEMMs (and
    the reduction) that only produce it are skipped.  Losses must be identical to the full recomputation."""
    a, b = str(tmp_path / "full.json"), str(tmp_path / "skip.json")
    run_distributed_many((_recompute_losses, world, cfg, False, a),
                         (_recompute_losses, world, cfg, True, b))
    la, lb = json.load(open(a)), json.load(open(b))
    assert la == lb, (la, lb)
    assert lb[-1] < lb[0]


def test_tensor_and_data_parallel_training():
    run_distributed(_loss_decreases, 4, {"model_parallel_size": 2, "sequence_parallel": True,
                                         "zero_optimization": {"stage": 1}}, None)


def test_pipeline_parallel_training():
    run_distributed(_loss_decreases, 2, {"pipe_parallel_size": 2, "gradient_accumulation_steps": 4,
                                         "num_layers": 4}, None)


def test_pipeline_with_tied_embeddings_and_tp():
    run_distributed(_loss_decreases, 4, {"pipe_parallel_size": 2, "model_parallel_size": 2,
                                         "gradient_accumulation_steps": 2, "num_layers": 4,
                                         "no_weight_tying": False}, None)


def _wall_clock_breakdown(rank, world, cfg):
    """``wall_clock_breakdown``: the engine publishes per-phase milliseconds every ``steps_per_print`` steps."""
    args, model, opt, sched = _setup({**cfg, "global_num_gpus": world, "wall_clock_breakdown": True,
                                      "steps_per_print": 2})
    assert model.wall_clock_breakdown() and model.steps_per_print() == 2 and model.timer_values is None
    _train(args, model, opt, sched, 1)
    assert model.timer_values is None                         # published at multiples of steps_per_print only
    _train(args, model, opt, sched, 1)
    vals = model.timer_values
    want = ({"train_batch", "forward_microstep", "backward_microstep", "batch_input", "step"}
            if args.is_pipe_parallel else {"forward", "backward", "step"})
    assert want <= set(vals), vals
    assert all(v >= 0.0 for v in vals.values()) and vals["step"] > 0.0
    if args.is_pipe_parallel:
        assert vals["train_batch"] >= vals["forward_microstep"]
    # the training log forwards them to the metric sinks as timers/<phase>
    from gpt_neox_b200 import logging as L
    from gpt_neox_b200.utils import Timers
    seen = {}

    class Writer:
        def add_scalar(self, key, value, it):
            seen[key] = value
    args.tensorboard_writer = Writer()
    timers = Timers()
    timers("interval time").start()
    L.training_log(args, timers, {"lm_loss": torch.tensor(1.0)}, {}, 1e-4, model.global_steps, 1.0, False, 0, model,
                   opt, None)
    if rank == 0:
        assert "timers/step" in seen and "train/lm_loss" in seen


@pytest.mark.parametrize("world,cfg", [(1, {}), (2, {"pipe_parallel_size": 2, "gradient_accumulation_steps": 2,
                                                      "num_layers": 4})])
def test_wall_clock_breakdown(world, cfg):
    run_distributed(_wall_clock_breakdown, world, cfg)


def _curriculum(rank, world, cfg):
    """Sequence-length curriculum: the length the model actually sees ramps from min to max difficulty, on the
    sequential engine (driven by the engine's forward) and on the pipeline engine (driven by its batch function)."""
    from gpt_neox_b200.models import gpt as G
    cl = {"enabled": True, "curriculum_type": "seqlen", "min_difficulty": 8, "max_difficulty": 32,
          "schedule_type": "fixed_linear", "schedule_config": {"total_curriculum_step": 6, "difficulty_step": 8}}
    args, model, opt, sched = _setup({**cfg, "global_num_gpus": world, "curriculum_learning": cl})
    seen = []
    if not args.is_pipe_parallel:
        inner = model.module.sequential[0]
        inner.register_forward_pre_hook(lambda m, a: seen.append(a[0][0].shape[1]) if m.training else None)
    it = _fixed_batches(args)
    losses = []
    if args.is_pipe_parallel and rank == 0:
        first = model.module.forward_funcs[0]
        first.register_forward_pre_hook(lambda m, a: seen.append(a[0][0].shape[1]) if m.training else None)
    for step in range(8):
        args.iteration = step                               # what the training loop maintains
        losses += _train(args, model, opt, sched, 1, it)
    assert all(l == l for l in losses)
    if seen and (not args.is_pipe_parallel or rank == 0):
        assert seen[0] == 8 and seen[-1] == 32 and sorted(seen) == seen, seen
    model.eval()                                            # evaluation always sees whole sequences
    if not args.is_pipe_parallel:
        from gpt_neox_b200.training import forward_step
        loss, _ = forward_step(it, model, args, None)
        assert loss == loss


def test_sequence_length_curriculum():
    run_distributed_many((_curriculum, 1, {}),
                         (_curriculum, 2, {"pipe_parallel_size": 2, "num_layers": 4, "gradient_accumulation_steps": 2}))


def _post_training(rank, world, cfg):
    """``train_step`` with a post-training objective: batches of the shape that objective's data loader yields, a
    reference model where one is needed, finite metrics, and a loss that moves."""
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.parallel import mpu
    from gpt_neox_b200.training import setup_model_and_optimizer, train_step
    from gpt_neox_b200.utils import Timers
    args = make_args(**{**cfg, "global_num_gpus": world})
    args.configure_distributed_args()
    initialize_megatron(args)
    model, opt, sched, ref = setup_model_and_optimizer(args)
    impl = args.train_impl
    assert (ref is not None) == (impl in ("dpo", "kto") and not args.dpo_reference_free
                                 and args.precompute_model_name is None)
    g = torch.Generator().manual_seed(100 + mpu.get_data_parallel_rank())
    mb, L, V = args.train_micro_batch_size_per_gpu, args.seq_length + 1, args.padded_vocab_size
    tok = lambda: torch.randint(1, V, (mb, L), generator=g)

    def batch():
        if impl == "rm":                       # one labelled position per sequence: where the reward is read
            lab = torch.full((mb, L), -100)
            lab[:, -1] = 5
            return {"pos": tok(), "neg": tok(), "pos_label": lab.clone(), "neg_label": lab.clone()}
        if impl == "dpo":
            return {"pos": tok(), "neg": tok()}
        if impl == "kto":
            return {"text": tok(), "reward": (torch.rand(mb, L, generator=g) > 0.5).float() * 2 - 1,
                    "ref": torch.zeros(mb, L)}
        return {"text": tok(), "reward": torch.rand(mb, generator=g), "raw_reward": torch.rand(mb, generator=g)}
    fixed = [batch() for _ in range(2)]

    def it():
        i = 0
        while True:
            yield fixed[i % 2]
            i += 1
    itr, losses = it(), []
    for _ in range(6):
        d, _ = train_step(args, Timers(), itr, model, opt, sched, reference_model=ref)
        assert all(float(v) == float(v) for v in d.values()), d
        losses.append(float(d["lm_loss"]))
    assert min(losses[2:]) < max(losses[:2]), losses
    return losses


_POST_TRAINING_CASES = [
    (2, {"train_impl": "dpo", "model_parallel_size": 2, "dpo_beta": 0.1}),                       # with a reference model
    (4, {"train_impl": "dpo", "dpo_reference_free": True, "model_parallel_size": 2, "sequence_parallel": True,
         "zero_optimization": {"stage": 2, "reduce_bucket_size": 30000}}),
    (2, {"train_impl": "rm", "model_parallel_size": 2, "no_weight_tying": True,
         "pos_train_label_data_paths": ["x"], "neg_train_label_data_paths": ["x"]}),
    (2, {"train_impl": "kto", "model_parallel_size": 2}),                                        # reference model
    (2, {"train_impl": "kto", "precompute_model_name": "ref"}),                                  # stored reference log-probs
    (2, {"train_impl": "reinforce", "model_parallel_size": 2}),
]


def test_post_training_objectives_train_end_to_end():
    # the six jobs are independent: side by side, three at a time
    jobs = [(_post_training, world, {"train_micro_batch_size_per_gpu": 2, **cfg}) for world, cfg in _POST_TRAINING_CASES]
    run_distributed_many(*jobs[:3])
    run_distributed_many(*jobs[3:])


def _pipeline_with_middle_stages(rank, world, cfg):
    """More than two stages: a middle stage both receives and sends the one-time shape header; training and
    evaluation run through every stage."""
    args, model, opt, sched = _setup({**cfg, "global_num_gpus": world})
    it = _fixed_batches(args)
    losses = _train(args, model, opt, sched, 8, it)
    assert min(losses) < losses[0], losses
    ev = model.eval_batch(it)
    assert torch.isfinite(ev).all() and abs(float(ev) - losses[-1]) < 1.0
    losses += _train(args, model, opt, sched, 2, it)          # and back to training
    assert all(l == l for l in losses)


def test_pipeline_with_middle_stages():
    run_distributed_many(
        (_pipeline_with_middle_stages, 4, {"pipe_parallel_size": 4, "num_layers": 6, "gradient_accumulation_steps": 6,
                                           "no_weight_tying": False}),
        (_pipeline_with_middle_stages, 3, {"pipe_parallel_size": 3, "num_layers": 5,
                                           "gradient_accumulation_steps": 2}))      # fewer micro-batches than stages


def test_tensor4_pipeline2_layout_trains():
    """The 8-rank layout of the headline benchmark (tensor parallel 4 x pipeline 2, activation checkpointing,
    ZeRO-1, bf16) through the host-side code paths: grouping, 1F1B schedule, tied / late gradients."""
    run_distributed(_loss_decreases, 8, {"pipe_parallel_size": 2, "model_parallel_size": 4,
                                         "gradient_accumulation_steps": 4, "num_layers": 4, "num_attention_heads": 8,
                                         "checkpoint_activations": True, "zero_optimization": {"stage": 1},
                                         "precision": "bfloat16"}, None, timeout=600)


def _checkpoint(rank, world, cfg, save_dir):
    from gpt_neox_b200.checkpointing import load_checkpoint, save_checkpoint
    from gpt_neox_b200.parallel import mpu
    base = {**cfg, "global_num_gpus": world, "save": save_dir, "load": save_dir,
            "checkpoint_validation_with_forward_pass": True}
    args, model, opt, sched = _setup({**base, "load": None})
    it = _fixed_batches(args)
    _train(args, model, opt, sched, 3, it)
    save_checkpoint(args, 42, model, opt, sched)
    want = {k: v.detach().clone() for k, v in model.module.state_dict().items()}
    next_losses = _train(args, model, opt, sched, 2, it)
    # a fresh model restored from disk must reproduce parameters bit-exactly and continue identically
    mpu.destroy_model_parallel()
    args2, model2, opt2, sched2 = _setup(base)
    assert args2.iteration == 42
    got = model2.module.state_dict()
    assert set(got) == set(want)
    for k in want:
        assert torch.equal(got[k], want[k]), k
    it2 = _fixed_batches(args2)
    for _ in range(3 * args2.gradient_accumulation_steps):
        next(it2)
    again = _train(args2, model2, opt2, sched2, 2, it2)
    assert all(abs(x - y) < 1e-5 for x, y in zip(next_losses, again)), (next_losses, again)
    if rank == 0:
        tag = os.path.join(save_dir, "global_step42")
        assert open(os.path.join(save_dir, "latest")).read().strip() == "global_step42"
        assert os.path.isdir(tag)


def test_checkpoint_round_trip_sequential(tmp_path):
    run_distributed(_checkpoint, 1, {}, str(tmp_path))
    files = os.listdir(tmp_path / "global_step42")
    assert "mp_rank_00_model_states.pt" in files
    sd = torch.load(tmp_path / "global_step42" / "mp_rank_00_model_states.pt", weights_only=False)
    assert any(k.startswith("sequential.0.word_embeddings") for k in sd["module"])
    assert sd["iteration"] == 42 and "args" in sd


def _cross_layout(rank, world, cfg_save, cfg_load, d):
    from gpt_neox_b200.checkpointing import save_checkpoint
    from gpt_neox_b200.parallel import mpu
    args, model, opt, sched = _setup({**cfg_save, "global_num_gpus": world, "save": d, "load": None})
    _train(args, model, opt, sched, 2, _fixed_batches(args))
    save_checkpoint(args, 7, model, opt, sched)
    strip = lambda k: k.split(".", 1)[-1] if k.startswith("sequential.") else k
    want = {strip(k): v.detach().clone() for k, v in model.module.state_dict().items()}
    mpu.destroy_model_parallel()
    args2, model2, opt2, sched2 = _setup({**cfg_load, "global_num_gpus": world, "save": d, "load": d})
    assert args2.iteration == 7
    got = {strip(k): v for k, v in model2.module.state_dict().items()}
    shared = set(got) & set(want)
    assert len(shared) > 10 and all(torch.equal(got[k], want[k]) for k in shared)
    _train(args2, model2, opt2, sched2, 1, _fixed_batches(args2))


@pytest.mark.parametrize("save,load", [(1, 0), (0, 1)])
def test_checkpoint_moves_between_the_pipeline_and_the_sequential_layout(tmp_path, save, load):
    """Per-layer files (a pipeline engine with one stage) load into the sequential model and the sequential state
    dict loads into a pipeline module: same weights, training continues."""
    run_distributed(_cross_layout, 1, {"pipe_parallel_size": save}, {"pipe_parallel_size": load}, str(tmp_path))


def test_checkpoint_round_trip_data_parallel_without_zero(tmp_path):
    """ZeRO stage 0 on two data-parallel ranks: only rank 0 writes the (replicated) optimizer state and both read it."""
    run_distributed(_checkpoint, 2, {"zero_optimization": {"stage": 0}}, str(tmp_path))
    files = os.listdir(tmp_path / "global_step42")
    assert "zero_pp_rank_0_mp_rank_00_optim_states.pt" in files
    assert "zero_pp_rank_1_mp_rank_00_optim_states.pt" not in files


def test_checkpoint_round_trip_onebit_adam_compression_phase(tmp_path):
    """Saved while the momentum is already exchanged as sign bits: the per-rank error-feedback buffers are part of
    every rank's own optimizer file, so the continuation is exact."""
    run_distributed(_checkpoint, 2, {"zero_optimization": {"stage": 0},
                                     "optimizer": {"type": "OneBitAdam", "params": {"lr": 1e-3, "freeze_step": 2}}},
                    str(tmp_path))
    files = os.listdir(tmp_path / "global_step42")
    assert sum(f.endswith("optim_states.pt") for f in files) == 2


@pytest.mark.parametrize("world,zero", [(2, 0), (4, 1)])
def test_checkpoint_round_trip_expert_parallel(tmp_path, world, zero):
    """Experts split over two expert-parallel ranks (times two expert-data-parallel ranks in the second case): every
    expert-parallel rank writes its own experts and optimizer state, and gets them back."""
    run_distributed(_checkpoint, world, {"moe_num_experts": 4, "moe_top_k": 2, "expert_interval": 2,
                                         "moe_expert_parallel_size": 2, "gpt_j_residual": False,
                                         "zero_optimization": {"stage": zero}}, str(tmp_path))
    files = os.listdir(tmp_path / "global_step42")
    assert {"expert_ep_rank_00_mp_rank_00_model_states.pt", "expert_ep_rank_01_mp_rank_00_model_states.pt"} <= set(files)
    a = torch.load(tmp_path / "global_step42" / "expert_ep_rank_00_mp_rank_00_model_states.pt", weights_only=False)
    b = torch.load(tmp_path / "global_step42" / "expert_ep_rank_01_mp_rank_00_model_states.pt", weights_only=False)
    assert set(a) == set(b) and a and any(not torch.equal(a[k], b[k]) for k in a)      # different experts
    assert sum(f.endswith("optim_states.pt") for f in files) == world


def test_checkpoint_round_trip_zero1_two_ranks(tmp_path):
    run_distributed(_checkpoint, 2, {"zero_optimization": {"stage": 1}, "precision": "bfloat16"}, str(tmp_path))
    files = os.listdir(tmp_path / "global_step42")
    assert "bf16_zero_pp_rank_0_mp_rank_00_optim_states.pt" in files
    assert "bf16_zero_pp_rank_1_mp_rank_00_optim_states.pt" in files


def test_checkpoint_round_trip_pipeline_layout(tmp_path):
    run_distributed(_checkpoint, 2, {"pipe_parallel_size": 2, "num_layers": 4, "gradient_accumulation_steps": 2},
                    str(tmp_path))
    files = sorted(os.listdir(tmp_path / "global_step42"))
    # layer files: 00 embedding, 02..05 transformer layers, 07 final norm, 08 output projection
    for idx in (0, 2, 3, 4, 5, 7, 8):
        assert f"layer_{idx:02d}-model_00-model_states.pt" in files, files
    assert "layer_01-model_00-model_states.pt" not in files       # _pre_transformer_block has no parameters


def test_keep_last_n_checkpoints(tmp_path):
    from gpt_neox_b200.checkpointing import delete_old_checkpoints
    for i in (1, 2, 10, 20):
        os.makedirs(tmp_path / f"global_step{i}")
    delete_old_checkpoints(str(tmp_path), 2)
    assert sorted(os.listdir(tmp_path)) == ["global_step10", "global_step20"]


# ------------------------------------------------------------------ 1-bit Adam: compressed momentum communication
def _onebit_collective(rank, world):
    import torch.distributed as dist
    from gpt_neox_b200.optim.onebit_adam import compressed_allreduce, pack_signs, unpack_signs
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x = torch.randn(64)
    assert torch.equal(unpack_signs(pack_signs(x)), torch.where(x >= 0, 1.0, -1.0))
    n = 8 * world * 50
    g = torch.Generator().manual_seed(11 + rank)
    werr, serr = torch.zeros(n), torch.zeros(n // world)
    sum_out, sum_true = torch.zeros(n), torch.zeros(n)
    for step in range(40):
        local = torch.randn(n, generator=g) + 0.3            # a common drift plus rank-specific noise
        true = local.clone()
        dist.all_reduce(true)
        true /= world
        out = compressed_allreduce(local.clone(), werr, serr)
        ref = out.clone()
        dist.broadcast(ref, 0)
        assert torch.equal(out, ref)                          # every rank reconstructs the same tensor
        sum_out += out
        sum_true += true
    # error feedback: what one step loses is re-sent later, so the running sums stay within a few quantisation steps
    drift = (sum_out - sum_true).abs().max().item()
    assert drift < 6.0, drift
    assert (sum_out - sum_true).abs().mean().item() < 0.05 * sum_true.abs().mean().item() + 1.5


def test_onebit_compressed_allreduce_error_feedback():
    run_distributed(_onebit_collective, 2)


def _onebit_training(rank, world):
    import torch.distributed as dist
    from gpt_neox_b200.parallel import comms_logger
    cfg = {"optimizer": {"type": "OneBitAdam", "params": {"lr": 2e-3, "betas": [0.9, 0.95], "eps": 1e-8,
                                                          "freeze_step": 4}},
           "zero_optimization": {"stage": 0}, "global_num_gpus": world, "train_iters": 20, "lr_decay_iters": 20}
    args, model, opt, sched = _setup(cfg)
    log = comms_logger.configure({"enabled": True})
    grad_bytes = {b.flat_grad.numel() * 4 for b in opt.buckets}
    it = _fixed_batches(args)
    from gpt_neox_b200.training import train_step
    from gpt_neox_b200.utils import Timers
    losses, grad_reductions = [], []
    for _ in range(14):
        d, _ = train_step(args, Timers(), it, model, opt, sched)
        losses.append(float(d["lm_loss"]))
        grad_reductions.append(sum(c for (op, nbytes, c, *_r) in log.summary() if op == "all_reduce" and nbytes in grad_bytes))
    log.uninstall()
    comms_logger.configure(None)
    # warm-up steps all-reduce the gradients; afterwards only sign bits and scales travel
    assert grad_reductions[3] > grad_reductions[0] and grad_reductions[-1] == grad_reductions[3], grad_reductions
    assert min(losses[6:]) < losses[0], losses
    for p in model.module.parameters():
        ref = p.detach().clone()
        dist.broadcast(ref, 0)
        assert torch.equal(ref, p.detach())                   # the ranks never drift apart


def test_onebit_adam_trains_with_compressed_momentum():
    run_distributed(_onebit_training, 2)


# ------------------------------------------------------------------ ZeRO stage 2: gradient partitioning
def _zero2_losses(rank, world, cfg, out):
    from gpt_neox_b200.training import train_step
    from gpt_neox_b200.utils import Timers
    args, model, opt, sched = _setup({**cfg, "global_num_gpus": world})
    it = _fixed_batches(args)
    losses = []
    for _ in range(6):
        d, _ = train_step(args, Timers(), it, model, opt, sched)
        losses.append(float(d["lm_loss"]))
        if opt.zero_stage >= 2:
            # between steps no full-size gradient buffer is alive, only the fp32 shard accumulators
            assert opt.partition_grads and all(b.flat_grad is None for b in opt.buckets if b.partition_grads)
            assert all(b.grad_acc.numel() == b.padded // b.world for b in opt.buckets if b.partition_grads)
            assert all(getattr(p, "main_grad", 0) is None for b in opt.buckets if b.partition_grads for p in b.params)
    if rank == 0 and out:
        with open(out, "w") as fh:
            json.dump({"losses": losses, "buckets": len(opt.buckets)}, fh)


@pytest.mark.parametrize("extra", [
    {},                                                     # data parallel 2
    {"model_parallel_size": 2, "sequence_parallel": True},  # tensor parallel 2 x data parallel 2, late norm-gradient sync
])
def test_zero2_gradient_partitioning_matches_zero1(tmp_path, extra):
    world = 4 if extra else 2
    base = {"gradient_accumulation_steps": 2, "train_micro_batch_size_per_gpu": 2, **extra}
    a, b = str(tmp_path / "z1.json"), str(tmp_path / "z2.json")
    run_distributed_many((_zero2_losses, world, {**base, "zero_optimization": {"stage": 1}}, a),
                         (_zero2_losses, world, {**base, "zero_optimization": {"stage": 2, "reduce_bucket_size": 40000}}, b))
    ra, rb = json.load(open(a)), json.load(open(b))
    assert rb["buckets"] > ra["buckets"]                    # stage 2 bounds its transient memory by bucketing
    for x, y in zip(ra["losses"], rb["losses"]):
        assert abs(x - y) < 2e-4, (ra["losses"], rb["losses"])


def _zero2_pp_worker(rank, world):
    with pytest.raises((SystemExit, ValueError)):
        _setup({"global_num_gpus": 2, "pipe_parallel_size": 2, "zero_optimization": {"stage": 2}})


def test_zero2_refuses_pipeline_parallelism():
    run_distributed(_zero2_pp_worker, 2)


# ------------------------------------------------------------------ ZeRO stage 3: parameter partitioning
def _zero3_worker(rank, world, cfg, out, ckpt_dir):
    from gpt_neox_b200.training import train_step
    from gpt_neox_b200.utils import Timers
    args, model, opt, sched = _setup({**cfg, "global_num_gpus": world})
    it = _fixed_batches(args)
    losses = []
    part = getattr(opt, "param_partitioner", None)
    for step in range(6):
        d, _ = train_step(args, Timers(), it, model, opt, sched)
        losses.append(float(d["lm_loss"]))
        if opt.zero_stage >= 3:
            assert part is not None and part.gathers > 0
            # between steps only shards are held: no full parameter or gradient buffer
            assert all(b.flat_param is None and b.flat_grad is None for b in part.buckets)
            assert all(b.param_shard.numel() == b.padded // b.world for b in part.buckets)
            assert all(p.numel() > 0 and p.data.stride() == (0,) * p.dim() for b in part.buckets for p in b.params)
    if opt.zero_stage >= 3 and ckpt_dir:
        # checkpoint round trip: the full weights are written and read back through the partitioner
        from gpt_neox_b200.checkpointing import load_checkpoint, save_checkpoint
        args.save = args.load = ckpt_dir
        save_checkpoint(args, 6, model, opt, sched)
        with part.all_resident():
            before = [p.detach().clone() for p in model.module.parameters()]
        for b in part.buckets:
            b.param_shard.zero_()
            b.master.data.zero_()
        load_checkpoint(args, model, opt, sched)
        with part.all_resident():
            for x, p in zip(before, model.module.parameters()):
                assert torch.equal(x, p.detach())
        d, _ = train_step(args, Timers(), it, model, opt, sched)
        losses.append(float(d["lm_loss"]))
    if rank == 0 and out:
        with open(out, "w") as fh:
            json.dump(losses, fh)


@pytest.mark.parametrize("extra", [{}, {"checkpoint_activations": True, "checkpoint_num_layers": 1},
                                   {"precision": "bfloat16"}])
def test_zero3_parameter_partitioning_matches_zero1(tmp_path, extra):
    base = {"gradient_accumulation_steps": 2, "train_micro_batch_size_per_gpu": 2, **extra}
    a, b = str(tmp_path / "z1.json"), str(tmp_path / "z3.json")
    run_distributed_many((_zero3_worker, 2, {**base, "zero_optimization": {"stage": 1}}, a, None),
                         (_zero3_worker, 2, {**base, "zero_optimization": {"stage": 3, "reduce_bucket_size": 40000}}, b,
                          str(tmp_path / "ckpt")))
    la, lb = json.load(open(a)), json.load(open(b))
    tol = 2e-4 if extra.get("precision") != "bfloat16" else 3e-2
    for x, y in zip(la, lb):
        assert abs(x - y) < tol, (la, lb)
    assert lb[6] < lb[0]                      # training continues after the checkpoint round trip


@pytest.mark.parametrize("precision", ["fp32", "bfloat16"])
def test_zero3_offload_checkpoint_round_trip(tmp_path, precision):
    """Stage 3 with optimizer states and parameter shards in host memory: save, wipe, load gives the same
    parameters back and training continues (the worker asserts it)."""
    cfg = {"gradient_accumulation_steps": 2, "train_micro_batch_size_per_gpu": 2, "precision": precision,
           "zero_optimization": {"stage": 3, "reduce_bucket_size": 40000, "cpu_offload": True,
                                 "offload_param": {"device": "cpu"}}}
    out = str(tmp_path / "z3.json")
    run_distributed(_zero3_worker, 2, cfg, out, str(tmp_path / "ckpt"))
    losses = json.load(open(out))
    assert len(losses) == 7 and losses[6] < losses[0]


def test_zero3_with_tensor_and_sequence_parallelism(tmp_path):
    base = {"gradient_accumulation_steps": 2, "train_micro_batch_size_per_gpu": 2, "model_parallel_size": 2,
            "sequence_parallel": True}
    a, b = str(tmp_path / "z1.json"), str(tmp_path / "z3.json")
    run_distributed_many((_zero3_worker, 4, {**base, "zero_optimization": {"stage": 1}}, a, None),
                         (_zero3_worker, 4, {**base, "zero_optimization": {"stage": 3, "reduce_bucket_size": 40000}}, b, None))
    for x, y in zip(json.load(open(a)), json.load(open(b))):
        assert abs(x - y) < 2e-4
