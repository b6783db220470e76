"""One-GPU fp16 training run with dynamic loss scaling (launched by tests/test_training_gpu.py).

The initial loss scale is far too large on purpose: the first steps overflow in fp16, must be skipped (parameters
untouched, scale halved), and training must then proceed on the native fp16 kernels without any fallback to library
or eager paths.  Prints ``FP16_SMOKE_OK``.
"""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))


def main():
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    torch.cuda.set_device(0)
    from common import make_args
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.ops import linear as L
    from gpt_neox_b200.ops import native
    from gpt_neox_b200.training import setup_model_and_optimizer, train_step
    from gpt_neox_b200.utils import Timers
    args = make_args(hidden_size=256, num_attention_heads=4, num_layers=2, seq_length=128, max_position_embeddings=128,
                     precision="fp16", fp16={"enabled": True, "loss_scale": 0, "initial_scale_power": 26,
                                             "loss_scale_window": 1000, "hysteresis": 1, "min_loss_scale": 1},
                     global_num_gpus=1, distributed_backend="nccl", zero_optimization={"stage": 1},
                     train_micro_batch_size_per_gpu=4, gradient_accumulation_steps=1,
                     attention_config=[[["flash"], "all"]], train_iters=100, lr_decay_iters=100)
    args.configure_distributed_args()
    initialize_megatron(args)
    model, opt, sched, _ = setup_model_and_optimizer(args)
    assert next(model.module.parameters()).dtype == torch.float16
    g = torch.Generator().manual_seed(3)
    batch = {"text": torch.randint(0, args.padded_vocab_size, (4, 129), generator=g)}

    def it():
        while True:
            yield batch
    data = it()
    before = [p.detach().clone() for p in list(model.module.parameters())[:3]]
    scale0 = opt.cur_scale
    losses, skipped = [], []
    launches = native.launch_count
    for _ in range(24):
        d, skip = train_step(args, Timers(), data, model, opt, sched)
        losses.append(float(d["lm_loss"]))
        skipped.append(int(skip))
        if skip and sum(skipped) == 1:
            for a, b in zip(before, list(model.module.parameters())[:3]):
                assert torch.equal(a, b.detach()), "a skipped step changed parameters"
    status = native.read_status()
    good = [l for l, s in zip(losses, skipped) if not s]
    ok = (status == 0 and sum(skipped) >= 1 and opt.cur_scale < scale0 and len(good) >= 4 and good[-1] < good[0]
          and all(l == l for l in good) and native.launch_count > launches and not L._warned)
    print(f"losses {losses}\nskipped {skipped} scale {scale0} -> {opt.cur_scale} status {status} fallbacks {L._warned}",
          flush=True)
    if ok:
        print("FP16_SMOKE_OK", flush=True)
    torch.distributed.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
