"""Process launcher (what ``deepspeed.launcher.runner`` does for the reference, ``deepy.py:37``).

Single node (default): spawn one worker per visible GPU (or ``num_gpus``) with ``RANK``, ``LOCAL_RANK``,
``WORLD_SIZE``, ``MASTER_ADDR=127.0.0.1`` and ``MASTER_PORT`` set, forward their output, and tear the group
down if any worker fails.

Multi node: read the hostfile (``host slots=N``), apply ``--include`` / ``--exclude`` / ``--num_nodes`` /
``--num_gpus``, and build the per-host command for the configured ``launcher`` (``pdsh``, ``openmpi``,
``mvapich``, ``slurm``).  Each remote host runs this module again with ``--node_rank``, which starts that
host's workers.  Environment variables with the usual prefixes (``NCCL``, ``PYTHON``, ``CUDA`` ...) and
``WANDB_API_KEY`` are exported to the workers.
"""
from __future__ import annotations

import base64
import json
import os
import shlex
import signal
import subprocess
import sys
import time

EXPORT_PREFIXES = ("NCCL", "PYTHON", "MV2", "UCX", "CUDA", "NEOX", "TORCH", "WANDB")


def _world_info(neox_args):
    """Ordered ``{host: [device ids]}`` for the job."""
    from .config.args import DLTS_HOSTFILE, resource_pool
    hostfile = neox_args.hostfile or (DLTS_HOSTFILE if os.path.exists(DLTS_HOSTFILE) else None)
    if hostfile is None:
        import torch
        n = neox_args.num_gpus if neox_args.num_gpus and neox_args.num_gpus > 0 else \
            (neox_args.global_num_gpus or torch.cuda.device_count() or 1)
        return {"localhost": list(range(n))}
    pool = resource_pool(hostfile, neox_args.include or "", neox_args.exclude or "")
    if neox_args.num_nodes and neox_args.num_nodes > 0:
        pool = dict(list(pool.items())[: neox_args.num_nodes])
    if neox_args.num_gpus and neox_args.num_gpus > 0:
        pool = {h: ids[: neox_args.num_gpus] for h, ids in pool.items()}
    return pool


def _exports():
    env = {}
    for k, v in os.environ.items():
        if k.startswith(EXPORT_PREFIXES):
            env[k] = v
    return env


def worker_argv(neox_args):
    """``[script, --deepspeed_config b64, --megatron_config b64]``."""
    argv = neox_args.get_deepspeed_main_args()
    i = argv.index(neox_args.user_script)
    return argv[i:]


TEARDOWN_GRACE_S = 15.0     # between SIGTERM and SIGKILL when a failed rank takes the job down


def spawn_local(script_argv, local_ids, node_rank, nnodes_offsets, world_size, master_addr, master_port,
                extra_env=None):
    """Start this host's workers and wait; returns the first non-zero exit code (0 if all succeeded)."""
    procs = []
    base_rank = nnodes_offsets[node_rank]
    for local_rank, dev in enumerate(local_ids):
        env = dict(os.environ)
        env.update(extra_env or {})
        env.update(RANK=str(base_rank + local_rank), LOCAL_RANK=str(local_rank), WORLD_SIZE=str(world_size),
                   MASTER_ADDR=master_addr, MASTER_PORT=str(master_port))
        procs.append(subprocess.Popen([sys.executable, "-u", *script_argv], env=env))
    rc = 0
    deadline = float("inf")
    try:
        alive = set(range(len(procs)))
        while alive:
            for i in list(alive):
                r = procs[i].poll()
                if r is None:
                    continue
                alive.discard(i)
                if r != 0 and rc == 0:
                    rc = r
                    for j in alive:                 # one rank failed: stop the others
                        procs[j].send_signal(signal.SIGTERM)
                    deadline = time.time() + TEARDOWN_GRACE_S
            if rc != 0 and alive and time.time() > deadline:
                for j in alive:                     # a rank stuck in a collective may ignore SIGTERM
                    procs[j].kill()
            time.sleep(0.2)
    except KeyboardInterrupt:
        for p in procs:
            p.send_signal(signal.SIGTERM)
        rc = 130
    return rc


def multinode_command(neox_args, world, script_argv, master_addr):
    """Command line that fans the job out to every host with the configured launcher."""
    hosts = list(world.keys())
    enc_world = base64.urlsafe_b64encode(json.dumps(world).encode()).decode()
    exports = " ".join(f"export {k}={shlex.quote(v)};" for k, v in _exports().items())
    inner = (f"{sys.executable} -u -m gpt_neox_b200.launcher --world_info={enc_world} --master_addr={master_addr} "
             f"--master_port={neox_args.master_port} --node_rank=%n -- " + " ".join(shlex.quote(a) for a in script_argv))
    kind = neox_args.launcher
    if kind == "pdsh":
        return ["pdsh", "-S", "-f", "1024", "-w", ",".join(hosts), f"{exports} cd {shlex.quote(os.getcwd())}; {inner}"]
    if kind in ("openmpi", "mvapich"):
        total = sum(len(v) for v in world.values())
        cmd = ["mpirun", "-n", str(total), "-hostfile", neox_args.hostfile or "/job/hostfile"]
        if kind == "openmpi":
            cmd += ["--mca", "btl", "^openib", "--mca", "btl_tcp_if_include", "eth0"]
            for k, v in _exports().items():
                cmd += ["-x", f"{k}={v}"]
        return cmd + [sys.executable, "-u", *script_argv]
    if kind == "slurm":
        total = sum(len(v) for v in world.values())
        cmd = ["srun", "-n", str(total)]
        if neox_args.comment:
            cmd += ["--comment", neox_args.comment]
        if neox_args.account:
            cmd += ["--account", neox_args.account]
        if neox_args.include:
            cmd += ["--include", neox_args.include]
        if neox_args.exclude:
            cmd += ["--exclude", neox_args.exclude]
        return cmd + [sys.executable, "-u", *script_argv]
    raise ValueError(f"unknown launcher {kind}")


def launch(neox_args):
    if neox_args.autotuning_run in ("tune", "run"):
        from .autotuning import Autotuner
        tuner = Autotuner(neox_args)
        best = tuner.tune()
        if neox_args.autotuning_run == "tune" or best is None:
            return 0 if best is not None else 1
        neox_args = tuner.apply_best(best)
    world = _world_info(neox_args)
    script_argv = worker_argv(neox_args)
    extra = {}
    if neox_args.use_wandb and "WANDB_API_KEY" not in os.environ:
        from .utils.wandb import get_wandb_api_key
        key = get_wandb_api_key(neox_args)
        if key:
            extra["WANDB_API_KEY"] = key
    total = sum(len(v) for v in world.values())
    multi = len(world) > 1 or neox_args.force_multi or neox_args.deepspeed_slurm or neox_args.deepspeed_mpi
    master_addr = neox_args.master_addr or ("127.0.0.1" if not multi else list(world.keys())[0])
    if not multi:
        ids = list(world.values())[0]
        return spawn_local(script_argv, ids, 0, [0], total, master_addr, neox_args.master_port, extra)
    cmd = multinode_command(neox_args, world, script_argv, master_addr)
    print("launching:", " ".join(cmd), flush=True)
    return subprocess.call(cmd, env={**os.environ, **extra})


def _node_main(argv=None):
    """Entry used on each host of a multi-node pdsh launch."""
    import argparse
    p = argparse.ArgumentParser()
    p.add_argument("--world_info", required=True)
    p.add_argument("--master_addr", required=True)
    p.add_argument("--master_port", type=int, default=29500)
    p.add_argument("--node_rank", default="%n")
    p.add_argument("rest", nargs=argparse.REMAINDER)
    a = p.parse_args(argv)
    world = json.loads(base64.urlsafe_b64decode(a.world_info).decode())
    hosts = list(world.keys())
    if a.node_rank.isdigit():
        node_rank = int(a.node_rank)
    else:
        import socket
        me = socket.gethostname()
        node_rank = next((i for i, h in enumerate(hosts) if h == me or h.split(".")[0] == me.split(".")[0]), 0)
    offsets, acc = [], 0
    for h in hosts:
        offsets.append(acc)
        acc += len(world[h])
    rest = a.rest[1:] if a.rest and a.rest[0] == "--" else a.rest
    return spawn_local(rest, world[hosts[node_rank]], node_rank, offsets, acc, a.master_addr, a.master_port)


if __name__ == "__main__":
    sys.exit(_node_main())
