"""Which call sites launch eager torch kernels during one training step.

    python -m gpt_neox_b200.utils.step_profile --layers 2 --micro-batches 2 [--out eager_ops.txt]

Builds the benchmark's GPT-NeoX-20B-shaped model with ``--layers`` layers on one GPU, runs three warm-up steps, then
one step under ``torch.profiler`` (CPU + CUDA activities, python stacks) and lists every ``aten::`` element-wise /
copy / fill / reduction operator with its device time, call count, input shapes and the innermost frames of this
package that issued it.  The framework's own kernels are launched through ctypes and do not appear as ``aten::`` ops,
so the table is exactly the work that has NOT been folded into a kernel yet -- the list to shrink.
"""
import argparse
import os
import sys
import types

import torch

EAGER = ("copy_", "add", "add_", "fill_", "zero_", "sum", "cat", "contiguous", "clone", "mul", "mul_", "to", "_to_copy",
         "index_select", "div_", "div", "stack", "index_add_", "masked_fill", "masked_fill_", "where", "mean")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--micro-batches", type=int, default=2)
    ap.add_argument("--min-us", type=float, default=20.0, help="hide operators below this total device time")
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, root)
    for k, v in (("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29641"), ("RANK", "0"), ("WORLD_SIZE", "1"),
                 ("LOCAL_RANK", "0")):
        os.environ.setdefault(k, v)
    import bench
    from ..config import NeoXArgs
    from ..initialize import initialize_megatron
    from ..training import setup_model_and_optimizer, train_step
    from . import Timers
    flags = types.SimpleNamespace(gpus=1, tp=None, pp=None, model="neox-20b", layers=a.layers, micro_batch=4,
                                  seq_per_gpu=4 * a.micro_batches, global_batch=128, no_act_ckpt=False, fp8=None)
    cfg, vocab, _ = bench.build_config(flags)
    args = NeoXArgs.from_dict(cfg)
    args.configure_distributed_args()
    args.build_tokenizer()
    args.padded_vocab_size = vocab
    initialize_megatron(args)
    model, opt, sched, _ = setup_model_and_optimizer(args)
    g = torch.Generator().manual_seed(0)
    batches = [torch.randint(0, vocab, (4, args.seq_length + 1), generator=g).cuda() for _ in range(4)]

    def stream():
        i = 0
        while True:
            yield {"text": batches[i % 4]}
            i += 1
    data = stream()
    for _ in range(3):
        train_step(args, Timers(), data, model, opt, sched)
    torch.cuda.synchronize()
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA], with_stack=True, record_shapes=True,
                 experimental_config=torch._C._profiler._ExperimentalConfig(verbose=True)) as prof:
        train_step(args, Timers(), data, model, opt, sched)
        torch.cuda.synchronize()
    rows, total = [], 0.0
    for e in prof.key_averages(group_by_input_shape=True, group_by_stack_n=12):
        if not e.key.startswith("aten::") or e.key.split("::")[1] not in EAGER:
            continue
        t = getattr(e, "device_time_total", None) or getattr(e, "cuda_time_total", 0)
        if t < a.min_us:
            continue
        frames = [s for s in e.stack if "gpt_neox_b200" in s][:4] or [s for s in e.stack][:2]
        rows.append((t, e.count, e.key, str(e.input_shapes)[:70], frames))
    rows.sort(key=lambda r: -r[0])
    lines = [f"{t:10.0f} us  x{c:<4} {k:<18} {shp}\n" + "".join(f"            {f}\n" for f in fr)
             for t, c, k, shp, fr in rows]
    text = "".join(lines)
    print(text)
    if a.out:
        with open(a.out, "w") as fh:
            fh.write(text)


if __name__ == "__main__":
    main()
