"""Failure handling, exercised on the host only: a rank that dies takes the job down with its exit code, damaged
or half-written checkpoints fall back to the last completed one (or fail with a message naming the file), a save
interrupted by SIGTERM leaves the previous checkpoint loadable, and data-pipeline errors carry rank and iteration."""
import os
import signal
import subprocess
import sys
import textwrap
import time

import pytest
import torch

from common import ROOT, make_args, run_distributed


def test_launcher_takes_the_job_down_when_a_rank_dies(tmp_path):
    from gpt_neox_b200 import launcher
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent("""
        import os, sys, time
        rank = int(os.environ["RANK"])
        time.sleep(0.5)                  # "between steps"
        if rank == 1:
            sys.exit(7)                  # this rank dies
        time.sleep(120)                  # the others would wait for it in their next collective
    """))
    t0 = time.time()
    rc = launcher.spawn_local([str(script)], [0, 1, 2], 0, [0], 3, "127.0.0.1", 29599)
    assert rc == 7
    assert time.time() - t0 < 30, "the surviving ranks were not stopped"


def test_launcher_kills_ranks_that_ignore_sigterm(tmp_path, monkeypatch):
    from gpt_neox_b200 import launcher
    monkeypatch.setattr(launcher, "TEARDOWN_GRACE_S", 1.0)
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent("""
        import os, signal, sys, time
        signal.signal(signal.SIGTERM, signal.SIG_IGN)      # e.g. stuck inside a native call
        if int(os.environ["RANK"]) == 0:
            time.sleep(0.3); sys.exit(3)
        time.sleep(120)
    """))
    t0 = time.time()
    assert launcher.spawn_local([str(script)], [0, 1], 0, [0], 2, "127.0.0.1", 29598) == 3
    assert time.time() - t0 < 30


def _save_two(rank, world, save_dir):
    from gpt_neox_b200.checkpointing import save_checkpoint
    from test_training_cpu import _fixed_batches, _setup, _train
    args, model, opt, sched = _setup({"global_num_gpus": world, "save": save_dir, "load": None,
                                      "zero_optimization": {"stage": 1}, "precision": "bfloat16"})
    it = _fixed_batches(args)
    _train(args, model, opt, sched, 2, it)
    save_checkpoint(args, 10, model, opt, sched)
    _train(args, model, opt, sched, 2, it)
    save_checkpoint(args, 20, model, opt, sched)


def _load(rank, world, load_dir, expect_iter, out):
    from test_training_cpu import _setup
    try:
        args, model, opt, sched = _setup({"global_num_gpus": world, "save": load_dir, "load": load_dir,
                                          "zero_optimization": {"stage": 1}, "precision": "bfloat16"})
        got = args.iteration
        err = ""
    except Exception as exc:
        got, err = -1, f"{type(exc).__name__}: {exc}"
    if rank == 0:
        with open(out, "w") as fh:
            fh.write(f"{got}\\n{err}")
    if expect_iter is not None:
        assert got == expect_iter, (got, err)


def test_truncated_shard_falls_back_to_the_last_complete_checkpoint(tmp_path):
    d = str(tmp_path / "ckpt")
    run_distributed(_save_two, 2, d)
    assert open(os.path.join(d, "latest")).read().strip() == "global_step20"
    victim = os.path.join(d, "global_step20", "bf16_zero_pp_rank_1_mp_rank_00_optim_states.pt")   # rank 1's own shard
    size = os.path.getsize(victim)
    with open(victim, "r+b") as fh:
        fh.truncate(size // 2)
    run_distributed(_load, 2, d, 10, str(tmp_path / "r.txt"))      # both ranks agree on the older tag


def test_missing_latest_uses_the_newest_completed_checkpoint(tmp_path):
    d = str(tmp_path / "ckpt")
    run_distributed(_save_two, 1, d)
    os.remove(os.path.join(d, "latest"))
    run_distributed(_load, 1, d, 20, str(tmp_path / "r.txt"))


def test_only_checkpoint_damaged_fails_with_the_file_name(tmp_path):
    d = str(tmp_path / "ckpt")
    run_distributed(_save_two, 1, d)
    import shutil
    shutil.rmtree(os.path.join(d, "global_step10"))
    victim = os.path.join(d, "global_step20", "mp_rank_00_model_states.pt")
    with open(victim, "r+b") as fh:
        fh.truncate(100)
    out = str(tmp_path / "r.txt")
    run_distributed(_load, 1, d, None, out)
    got, err = open(out).read().split("\\n", 1)
    assert got == "-1" and "mp_rank_00_model_states.pt" in err and "truncated or corrupt" in err, err


def test_sigterm_during_save_keeps_the_previous_checkpoint(tmp_path):
    """A child process writes checkpoint 10, then starts writing checkpoint 20 with a slowed-down writer and is
    killed in the middle: ``latest`` still names 10, no file under a final name is partial, and 10 loads."""
    d = str(tmp_path / "ckpt")
    child = tmp_path / "child.py"
    child.write_text(textwrap.dedent(f"""
        import os, sys, time
        sys.path.insert(0, {ROOT!r}); sys.path.insert(0, os.path.join({ROOT!r}, "tests"))
        os.environ.update(RANK="0", LOCAL_RANK="0", WORLD_SIZE="1", MASTER_ADDR="127.0.0.1", MASTER_PORT="29597")
        import torch
        from gpt_neox_b200 import checkpointing as C
        from test_training_cpu import _fixed_batches, _setup, _train
        args, model, opt, sched = _setup({{"save": {d!r}, "load": None}})
        it = _fixed_batches(args)
        _train(args, model, opt, sched, 1, it)
        C.save_checkpoint(args, 10, model, opt, sched)
        real = torch.save
        def slow(obj, path, *a, **k):
            real(obj, path, *a, **k)
            print("WROTE", flush=True)
            time.sleep(30)
        torch.save = slow
        C.save_checkpoint(args, 20, model, opt, sched)
    """))
    p = subprocess.Popen([sys.executable, str(child)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    deadline = time.time() + 240
    seen = False
    while time.time() < deadline:
        line = p.stdout.readline()
        if not line:
            break
        if line.startswith("WROTE"):
            seen = True
            break
    assert seen, "the child never reached the second save"
    p.send_signal(signal.SIGTERM)
    p.wait(timeout=30)
    assert open(os.path.join(d, "latest")).read().strip() == "global_step10"
    step20 = os.path.join(d, "global_step20")
    assert not os.path.exists(os.path.join(step20, ".complete"))
    for name in os.listdir(step20) if os.path.isdir(step20) else []:
        if name.endswith(".pt"):
            torch.load(os.path.join(step20, name), map_location="cpu", weights_only=False)   # whole, never partial
    run_distributed(_load, 1, d, 10, str(tmp_path / "r.txt"))


def test_data_loader_error_names_rank_and_iteration():
    from gpt_neox_b200.training import _next_batch
    args = make_args()
    args.rank, args.iteration = 5, 123

    def broken():
        yield {"text": torch.zeros(1, 4, dtype=torch.long)}
        raise OSError("index file is truncated")
    it = broken()
    assert _next_batch(it, args) is not None
    with pytest.raises(RuntimeError, match=r"rank 5 at iteration 123.*index file is truncated"):
        _next_batch(it, args)
    with pytest.raises(RuntimeError, match=r"exhausted on rank 5"):
        _next_batch(iter(()), args)
