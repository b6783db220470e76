"""Multi-process (gloo, CPU) tests of the parallel primitives: every mapping's forward/backward against a
single-process dense computation, vocab-parallel cross entropy, tensor-parallel model equivalence."""
import pytest
import torch

from common import make_args, run_distributed


def _mappings(rank, world):
    import torch.distributed as dist
    from gpt_neox_b200.parallel import mappings as M, mpu
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mpu.initialize_model_parallel(world)
    torch.manual_seed(0)
    full = torch.randn(8, 4, 12)
    # copy -> all-reduce in backward
    x = full.clone().requires_grad_()
    M.copy_to_model_parallel_region(x).sum().backward()
    assert torch.allclose(x.grad, torch.full_like(x, float(world)))
    # reduce forward
    y = M.reduce_from_model_parallel_region(full.clone() * (rank + 1))
    assert torch.allclose(y, full * sum(range(1, world + 1)))
    # scatter / gather last dim are inverse
    x = full.clone().requires_grad_()
    part = M.scatter_to_model_parallel_region(x)
    assert part.shape[-1] == 12 // world
    back = M.gather_from_model_parallel_region(part)
    assert torch.equal(back, full)
    back.sum().backward()
    assert torch.allclose(x.grad, torch.ones_like(x))
    # sequence-parallel: reduce-scatter(seq) then gather(seq) == all-reduce
    for seq_dim in (0, 1):
        x = (full.clone() * (rank + 1)).requires_grad_()
        rs = M.reduce_scatter_to_sequence_parallel_region(x, seq_dim)
        ag = M.gather_from_sequence_parallel_region(rs, seq_dim)
        assert torch.allclose(ag, full * sum(range(1, world + 1)), atol=1e-5)
        ag.sum().backward()
        assert torch.allclose(x.grad, torch.full_like(x, float(world)))
        sc = M.scatter_to_sequence_parallel_region(full.clone(), seq_dim)
        assert sc.shape[seq_dim] == full.shape[seq_dim] // world


def test_mappings_two_ranks():
    run_distributed(_mappings, 2)


def _vocab_ce(rank, world):
    import torch.distributed as dist
    from gpt_neox_b200.parallel import mpu
    from gpt_neox_b200.parallel.cross_entropy import vocab_parallel_cross_entropy
    dist.init_process_group("gloo", rank=rank, world_size=world)
    assert mpu.is_unitialized()
    mpu.initialize_model_parallel(world)
    # the Megatron-LM spellings name the same group
    assert not mpu.is_unitialized() and mpu.get_tensor_model_parallel_group() is mpu.get_model_parallel_group()
    assert mpu.get_tensor_model_parallel_rank() == rank and mpu.get_tensor_model_parallel_world_size() == world
    assert mpu.get_tensor_model_parallel_src_rank() == 0
    torch.manual_seed(0)
    V = 64
    logits = torch.randn(3, 5, V) * 2
    tgt = torch.randint(0, V, (3, 5))
    w = torch.rand(3, 5)
    ref_in = logits.clone().requires_grad_()
    ref = torch.nn.functional.cross_entropy(ref_in.view(-1, V), tgt.view(-1), reduction="none").view(3, 5)
    (ref * w).sum().backward()
    shard = logits[..., rank * V // world:(rank + 1) * V // world].clone().requires_grad_()
    loss = vocab_parallel_cross_entropy(shard, tgt)
    (loss * w).sum().backward()
    assert torch.allclose(loss, ref, atol=1e-5)
    assert torch.allclose(shard.grad, ref_in.grad[..., rank * V // world:(rank + 1) * V // world], atol=1e-5)


def test_vocab_parallel_cross_entropy_two_ranks():
    run_distributed(_vocab_ce, 2)


def _tp_model(rank, world, sequence_parallel, gpt_j):
    """Logits and a loss of the TP=2 model equal those of the TP=1 model built from the same full weights."""
    import torch.distributed as dist
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.models import GPT2ModelPipe, cross_entropy
    from gpt_neox_b200.parallel import mpu
    cfg = dict(use_cpu_initialization=True, model_parallel_size=world, global_num_gpus=world,
               sequence_parallel=sequence_parallel, gpt_j_residual=gpt_j, num_layers=2)
    args = make_args(**cfg)
    args.configure_distributed_args()
    initialize_megatron(args)
    torch.manual_seed(1)
    model = GPT2ModelPipe(args, parallel_output=False).to_sequential()
    torch.manual_seed(7)
    tokens = torch.randint(0, args.padded_vocab_size, (2, args.seq_length))
    pos = torch.arange(args.seq_length).unsqueeze(0).expand_as(tokens)
    logits, _ = model((tokens, pos, None))
    # dense twin: same seeds, TP degree 1 (host initialisation draws the full matrices identically)
    mpu.set_model_parallel_world_size(1)
    mpu.set_model_parallel_rank(0)
    args1 = make_args(**{**cfg, "model_parallel_size": 1, "global_num_gpus": 1, "sequence_parallel": False})
    torch.manual_seed(1)
    dense = GPT2ModelPipe(args1, parallel_output=False).to_sequential()
    ref, _ = dense((tokens, pos, None))
    assert logits.shape == ref.shape
    assert torch.allclose(logits, ref, atol=2e-4, rtol=1e-3), (logits - ref).abs().max()


@pytest.mark.parametrize("sequence_parallel,gpt_j", [(False, True), (True, True), (True, False)])
def test_tensor_parallel_model_matches_dense(sequence_parallel, gpt_j):
    run_distributed(_tp_model, 2, sequence_parallel, gpt_j)


def _partitioned_checkpoint(rank, world, _cfg, _out):
    """Activation checkpointing with the saved inputs sliced over the TP group (and parked on the host) reproduces
    plain checkpointing exactly."""
    import torch
    from gpt_neox_b200.parallel import mpu, rng
    mpu.initialize_model_parallel(world)
    torch.manual_seed(3)
    lin = torch.nn.Linear(16, 16)
    x0 = torch.randn(6, 4, 16)            # replicated input, as between transformer layers without sequence parallelism

    def run(partition, cpu):
        rng.configure_checkpointing(partition, cpu)
        x = x0.clone().requires_grad_(True)
        y = rng.checkpoint(lambda t: torch.tanh(lin(t)) * t, x)
        lin.zero_grad()
        y.square().sum().backward()
        return y.detach().clone(), x.grad.clone(), lin.weight.grad.clone()

    base = run(False, False)
    for mode in ((True, False), (True, True), (False, True)):
        got = run(*mode)
        for a, b in zip(base, got):
            assert torch.allclose(a, b, atol=1e-6), mode
    rng.configure_checkpointing(False, False)


def test_partitioned_activation_checkpointing():
    run_distributed(_partitioned_checkpoint, 2, None, None)


# ------------------------------------------------------------------ flag-protocol replay (stands in for a device race detector)
@pytest.mark.parametrize("world", [2, 4, 8])
def test_flag_protocols_are_race_and_deadlock_free_under_random_interleavings(world):
    from gpt_neox_b200.parallel import protocol_model as PM
    seeds = range(60 if world < 8 else 20)
    PM.check(PM.gemm_all_reduce_program, world, seeds=seeds, epochs=6)
    PM.check(PM.gemm_all_reduce_program, world, seeds=seeds, epochs=6, deferred_tail=True)
    PM.check(PM.zero_peer_program, world, seeds=seeds, steps=5)


def test_protocol_checker_notices_a_missing_guard():
    """The checker has teeth: drop one wait and some interleaving produces a stale or overwritten read."""
    from gpt_neox_b200.parallel import protocol_model as PM
    for kw in ({"program": PM.gemm_all_reduce_program, "epochs": 6, "wait_ready": False},
               {"program": PM.gemm_all_reduce_program, "epochs": 6, "wait_ready": False, "deferred_tail": True},
               {"program": PM.zero_peer_program, "steps": 5, "wait_done_before_zero": False}):
        program = kw.pop("program")
        with pytest.raises(PM.ProtocolViolation):
            PM.check(program, 4, seeds=range(300), **kw)
    # the "buffer is free again" guards of the all-reduce are implied by stream order in this call sequence
    PM.check(PM.gemm_all_reduce_program, 4, seeds=range(100), epochs=6, guard_recv=False, guard_gathered=False)
    # and a circular wait is reported as a deadlock, not as a hang
    sim = PM.Simulator(2)
    sim.add(0, "main", [("wait", "x", 1, 1), ("signal", 1, "x", 1)])
    sim.add(1, "main", [("wait", "x", 0, 1), ("signal", 0, "x", 1)])
    with pytest.raises(PM.ProtocolViolation, match="deadlock"):
        sim.run(0)
