"""Tensor-parallel layers: vocabulary-sharded embedding, column- and row-sharded linears and a
head-sharded T5 relative position bias (API of ``megatron/mpu/layers.py:98-794``).

Sharding rules:

* ``ColumnParallelLinear``  W is ``[out/tp, in]``; with sequence parallelism the input arrives sharded
  along ``seq_dim`` and is all-gathered before the GEMM, otherwise it is an identity whose backward
  all-reduces.  ``gather_output`` all-gathers the last dim.  ``skip_bias_add`` returns the bias to the
  caller so it can be fused into the next op.
* ``RowParallelLinear``  W is ``[out, in/tp]``; the partial products are reduce-scattered (sequence
  parallel) or all-reduced, unless ``parallel_output`` defers the reduction to the caller (GPT-J
  residual sums attention and MLP partials first).

The GEMMs run through ``ops.linear`` (tcgen05 kernel, fused epilogue).  When the fused peer-memory
collectives are enabled (``parallel/fused_comm.py``) the all-gather / reduce-scatter around the
GEMM is replaced by the fused kernel.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.nn import init
from torch.nn.parameter import Parameter

from ..ops import embedding as fused_embedding
from ..ops.linear import output_is_dead
from ..ops.linear import linear as fused_linear
from ..ops.mxfp8 import mx_linear
from ..ops import fp8 as F8
from . import fused_comm
from . import mappings as M
from . import mpu
from .rng import get_cuda_rng_tracker


def _device(neox_args=None):
    if torch.cuda.is_available() and not (neox_args is not None and getattr(neox_args, "use_cpu_initialization", False)
                                          and False):
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def _mark(weight, partition_dim, stride=1):
    weight.model_parallel = True
    weight.partition_dim = partition_dim
    weight.partition_stride = stride


def init_sharded_weight(neox_args, weight, full_rows, full_cols, partition_dim, init_method, stride=1):
    """Initialise a sharded weight.

    Device path: draw under the tensor-parallel RNG stream so every shard differs.  Host path
    (``use_cpu_initialization``): draw the full fp32 matrix with the default stream (identical on all
    ranks) and keep this rank's slice, which makes the result independent of the TP degree.
    """
    _mark(weight, partition_dim, stride)
    if getattr(neox_args, "use_cpu_initialization", False):
        master = torch.empty(full_rows, full_cols, dtype=torch.float)
        init_method(master)
        tp, r = mpu.get_model_parallel_world_size(), mpu.get_model_parallel_rank()
        per = weight.shape[partition_dim] // stride
        pieces = torch.split(master, per, dim=partition_dim)[r::tp]
        with torch.no_grad():
            weight.copy_(torch.cat(pieces, dim=partition_dim).to(weight.dtype))
        return
    with get_cuda_rng_tracker().fork():
        if weight.dtype in (torch.bfloat16, torch.float16) and not weight.is_cuda:
            tmp = torch.empty(weight.shape, dtype=torch.float)
            init_method(tmp)
            with torch.no_grad():
                weight.copy_(tmp.to(weight.dtype))
        else:
            init_method(weight)


class VocabParallelEmbedding(nn.Module):
    """Embedding sharded along the vocabulary; out-of-range ids contribute zeros, then all-reduce."""

    def __init__(self, neox_args, num_embeddings, embedding_dim, init_method=init.xavier_normal_):
        super().__init__()
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self.model_parallel_size = mpu.get_model_parallel_world_size()
        self.vocab_start_index, self.vocab_end_index = mpu.VocabUtility.vocab_range_from_global_vocab_size(
            num_embeddings, mpu.get_model_parallel_rank(), self.model_parallel_size)
        self.num_embeddings_per_partition = self.vocab_end_index - self.vocab_start_index
        self.init_method = init_method
        self.weight = Parameter(torch.empty(self.num_embeddings_per_partition, embedding_dim, device=_device(neox_args),
                                            dtype=neox_args.params_dtype))
        init_sharded_weight(neox_args, self.weight, num_embeddings, embedding_dim, 0, init_method)

    def forward(self, input_):
        if fused_embedding.kernel_ok(input_, self.weight):
            # gather kernel: rows of ids owned by another rank come out as zeros; backward scatter-adds in fp32
            out = fused_embedding.embedding(input_, self.weight, self.vocab_start_index)
            return M.reduce_from_model_parallel_region(out)
        if self.model_parallel_size > 1:
            mask = (input_ < self.vocab_start_index) | (input_ >= self.vocab_end_index)
            local = (input_ - self.vocab_start_index).masked_fill(mask, 0)
        else:
            mask, local = None, input_
        out = F.embedding(local, self.weight)
        if mask is not None:
            out = out.masked_fill(mask.unsqueeze(-1), 0.0)
        return M.reduce_from_model_parallel_region(out)


class ParallelRelativePositionBias(nn.Module):
    """T5 bucketed relative position bias with heads sharded over tensor-parallel ranks."""

    def __init__(self, neox_args, scale, causal=True, num_buckets=32, max_distance=128, heads=8,
                 init_method=init.xavier_normal_):
        super().__init__()
        self.scale, self.causal, self.num_buckets, self.max_distance, self.heads = scale, causal, num_buckets, \
            max_distance, heads
        tp, r = mpu.get_model_parallel_world_size(), mpu.get_model_parallel_rank()
        self.num_heads_per_partition = mpu.divide(heads, tp)
        self.head_start_index = r * self.num_heads_per_partition
        self.head_end_index = self.head_start_index + self.num_heads_per_partition
        self.weight = Parameter(torch.empty(num_buckets, self.num_heads_per_partition, device=_device(neox_args),
                                            dtype=neox_args.params_dtype))
        init_sharded_weight(neox_args, self.weight, num_buckets, heads, 1, init_method)
        self._cache = None

    def _bucket(self, rel):
        nb = self.num_buckets
        ret = torch.zeros_like(rel)
        n = -rel
        if not self.causal:
            nb //= 2
            ret = ret + (n < 0).long() * nb
            n = n.abs()
        else:
            n = n.clamp(min=0)
        max_exact = nb // 2
        small = n < max_exact
        large = max_exact + (torch.log(n.float().clamp(min=1) / max_exact) / math.log(self.max_distance / max_exact)
                             * (nb - max_exact)).long()
        large = large.clamp(max=nb - 1)
        return ret + torch.where(small, n, large)

    def forward(self, q_len, k_len):
        if self._cache is None or self._cache[0] != (q_len, k_len) or self._cache[1].device != self.weight.device:
            q = torch.arange(q_len, dtype=torch.long, device=self.weight.device)
            k = torch.arange(k_len, dtype=torch.long, device=self.weight.device)
            self._cache = ((q_len, k_len), self._bucket(k[None, :] - q[:, None]))
        values = F.embedding(self._cache[1], self.weight)        # [q, k, heads/tp]
        return values.movedim(2, 0).unsqueeze(0) * self.scale     # [1, heads/tp, q, k]


def _fp8_setup(layer, neox_args, enabled):
    """``enabled``: whether this layer runs in fp8.  The transformer block decides that from the ``te_*`` switches
    (the keys with which the reference swaps Transformer Engine layers into attention and MLP,
    megatron/model/transformer.py:93-140, 395-420); every other user of these classes (output projection, MoE
    experts, reward head) stays in bf16, as there.  The remaining ``te_fp8_*`` keys fill the per-layer recipe."""
    layer.fp8 = bool(enabled)
    layer.fp8_hybrid = getattr(neox_args, "te_fp8_format", "hybrid") == "hybrid"
    layer.fp8_wgrad = bool(getattr(neox_args, "te_fp8_wgrad", True))
    kind = getattr(neox_args, "te_fp8_recipe", "current") or "current"
    layer.fp8_block_scaled = kind == "mxfp8"
    layer.fp8_recipe = F8.Fp8Recipe(
        recipe=kind if kind != "mxfp8" else "current", hybrid=layer.fp8_hybrid, fp8_wgrad=layer.fp8_wgrad,
        margin=int(getattr(neox_args, "te_fp8_margin", 0) or 0),
        history_len=max(1, int(getattr(neox_args, "te_fp8_amax_history_len", 1) or 1)),
        most_recent=getattr(neox_args, "te_fp8_amax_compute_algo", "most_recent") != "max")


class _GeluGradOnInput(torch.autograd.Function):
    """Identity whose backward multiplies by GeLU'(aux): the contract of ``dgelu_aux`` for a layer that cannot fold
    it into its dgrad GEMM."""

    @staticmethod
    def forward(ctx, x, aux):
        ctx.save_for_backward(aux)
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        from ..ops.functional import dgelu_mul
        (aux,) = ctx.saved_tensors
        return dgelu_mul(g.contiguous(), aux), None


def _fp8_matmul(layer, x, bias, residual=None, act=None, dgelu_aux=None, split_pre=False):
    """``act(x W^T + bias) + residual`` through the layer's fp8 recipe; the epilogue fusions of ``ops.linear`` apply
    on the tensor-core fp8 path, the block-scaled path composes them from separate ops."""
    n_out, n_in = layer.weight.shape
    if layer.fp8_block_scaled or not F8.shapes_ok(x.numel() // n_in, n_out, n_in) or \
            (x.numel() // n_in) % 16 or x.dtype != torch.bfloat16 or (bias is not None and bias.dtype != x.dtype):
        if dgelu_aux is not None:
            x = _GeluGradOnInput.apply(x, dgelu_aux)
        out = mx_linear(x, layer.weight, bias, layer.fp8_hybrid, layer.fp8_wgrad)
        if act == "gelu":
            out = F.gelu(out, approximate="tanh")          # autograd owns GeLU': no pre-activation is handed out
        if residual is not None:
            out = out + residual
        return (out, None) if split_pre else out
    return F8.fp8_linear(x, layer.weight, bias, layer.fp8_recipe, residual, act, dgelu_aux, split_pre)


class ColumnParallelLinear(nn.Module):
    """``Y = X A + b`` with ``A`` split along its output (column) dimension."""

    def __init__(self, neox_args, input_size, output_size, bias=True, gather_output=True,
                 init_method=init.xavier_normal_, stride=1, keep_master_weight_for_test=False, skip_bias_add=False,
                 MOE=False, MoE_mp_size=1, mup_rescale_parameters=False, seq_dim=0, fp8=False):
        super().__init__()
        self.input_size, self.output_size, self.gather_output = input_size, output_size, gather_output
        world = MoE_mp_size if MOE else mpu.get_model_parallel_world_size()
        self.tp = world
        self.output_size_per_partition = mpu.divide(output_size, world)
        self.skip_bias_add = skip_bias_add
        self.sequence_parallel = bool(getattr(neox_args, "sequence_parallel", False)) and world > 1
        self.seq_dim = seq_dim
        self.init_method, self.stride = init_method, stride
        self.mup_rescale_parameters = mup_rescale_parameters
        self.use_mup = getattr(neox_args, "use_mup", False)
        self.width_mult_val = 1.0
        _fp8_setup(self, neox_args, fp8)
        dev = _device(neox_args)
        self.weight = Parameter(torch.empty(self.output_size_per_partition, input_size, device=dev,
                                            dtype=neox_args.params_dtype))
        init_sharded_weight(neox_args, self.weight, output_size, input_size, 0, init_method, stride)
        if bias:
            self.bias = Parameter(torch.zeros(self.output_size_per_partition, device=dev, dtype=neox_args.params_dtype))
            _mark(self.bias, 0, stride)
        else:
            self.register_parameter("bias", None)

    def set_parallel_output(self, value: bool):
        self.gather_output = not value

    def width_mult(self):
        return self.width_mult_val

    def matmul(self, input_, bias, act=None, split_pre=False):
        """Region mapping + GEMM: ``act(gather_or_copy(input_) W^T + bias)``.  Uses the kernel that overlaps the
        collective with the GEMM when the shapes allow it, the NCCL mapping otherwise.  ``split_pre``: return
        ``(out, pre_activation)`` and take the gradient w.r.t. the pre-activation in backward (the consumer applies
        GeLU' in its own dgrad GEMM, see ``ops.linear._LinearFn``)."""
        K = input_.shape[-1]
        if self.fp8:
            x = M.gather_from_sequence_parallel_region(input_, self.seq_dim) if self.sequence_parallel else \
                M.copy_to_model_parallel_region(input_)
            return _fp8_matmul(self, x, bias, act=act, split_pre=split_pre)
        if self.tp > 1 and self.tp == mpu.get_model_parallel_world_size() and not mpu.get_fp32_allreduce():
            tokens = input_.numel() // K
            rows = tokens if self.sequence_parallel else tokens // self.tp
            ok = (self.seq_dim == 0 or input_.shape[0] == 1 or not self.sequence_parallel) and \
                (self.sequence_parallel or tokens % self.tp == 0)
            if ok and (bias is None or bias.dtype == torch.bfloat16) and \
                    fused_comm.eligible(input_, self.weight, self.tp, rows):
                if self.sequence_parallel and self.seq_dim != 0:
                    assert not split_pre
                    out = fused_comm.column_linear(input_[0], self.weight, bias, act, True)
                    return out.unsqueeze(0)
                return fused_comm.column_linear(input_, self.weight, bias, act, self.sequence_parallel, split_pre)
        if self.sequence_parallel:
            x = M.gather_from_sequence_parallel_region(input_, self.seq_dim)
        else:
            x = M.copy_to_model_parallel_region(input_)
        return fused_linear(x, self.weight, bias, act=act, split_pre=split_pre)

    def forward(self, input_, act=None):
        if self.use_mup and self.mup_rescale_parameters:
            input_ = input_ / self.width_mult()
        bias = None if self.skip_bias_add else self.bias
        out = self.matmul(input_, bias, act)
        if self.gather_output:
            # after the sequence all-gather every rank holds the full sequence, so gathering the output
            # features is well defined (the reference asserts here, which rules out inference under SP)
            out = M.gather_from_model_parallel_region(out)
        return out, (self.bias if self.skip_bias_add else None)


class RowParallelLinear(nn.Module):
    """``Y = X A + b`` with ``A`` split along its input (row) dimension and ``X`` along its last dim."""

    def __init__(self, neox_args, input_size, output_size, bias=True, input_is_parallel=False,
                 init_method=init.xavier_normal_, stride=1, keep_master_weight_for_test=False, skip_bias_add=False,
                 MOE=False, MoE_mp_size=1, parallel_output=False, mup_rescale_parameters=False, fp8=False):
        super().__init__()
        self.input_size, self.output_size, self.input_is_parallel = input_size, output_size, input_is_parallel
        world = MoE_mp_size if MOE else mpu.get_model_parallel_world_size()
        self.tp = world
        self.input_size_per_partition = mpu.divide(input_size, world)
        self.skip_bias_add = skip_bias_add
        self.parallel_output = parallel_output
        self.sequence_parallel = bool(getattr(neox_args, "sequence_parallel", False)) and world > 1
        assert not (self.sequence_parallel and not input_is_parallel), \
            "Cannot have self.input_is_parallel=False and self.sequence_parallel=True."
        self.init_method, self.stride = init_method, stride
        self.mup_rescale_parameters = mup_rescale_parameters
        self.use_mup = getattr(neox_args, "use_mup", False)
        _fp8_setup(self, neox_args, fp8)
        dev = _device(neox_args)
        self.weight = Parameter(torch.empty(output_size, self.input_size_per_partition, device=dev,
                                            dtype=neox_args.params_dtype))
        init_sharded_weight(neox_args, self.weight, output_size, input_size, 1, init_method, stride)
        if bias:
            self.bias = Parameter(torch.zeros(output_size, device=dev, dtype=neox_args.params_dtype))
            if self.sequence_parallel and not parallel_output:
                # replicated parameter whose gradient is computed from this rank's sequence shard only
                self.bias.sequence_parallel_grad_sync = True
        else:
            self.register_parameter("bias", None)

    def set_parallel_output(self, value: bool):
        self.parallel_output = value

    def _fusable(self, x):
        if self.fp8:
            return False
        if self.tp == 1 or self.tp != mpu.get_model_parallel_world_size() or mpu.get_fp32_allreduce():
            return False
        tokens = x.numel() // x.shape[-1]
        return tokens % self.tp == 0 and fused_comm.eligible(x, self.weight, self.tp, tokens // self.tp) and \
            (self.bias is None or self.bias.dtype == torch.bfloat16)

    def forward(self, input_, residual=None, dgelu_aux=None, fuse_bias=False):
        """``residual`` (optional) is added to the layer's output: after the cross-rank reduction when this layer
        performs it, to this rank's partial product when the caller defers it (``parallel_output``).
        ``dgelu_aux``: pre-activation of the layer that produced ``input_`` through a GeLU (see ``matmul``).
        ``fuse_bias``: add the bias here (GEMM epilogue) even if the layer was built with ``skip_bias_add``; the
        returned bias is then ``None``."""
        x = input_ if self.input_is_parallel else M.scatter_to_model_parallel_region(input_)
        skip = self.skip_bias_add and not fuse_bias
        bias = None if skip else self.bias
        if not self.parallel_output and self._fusable(x):
            # GEMM -> reduce-scatter / all-reduce in one pass; bias and residual are added after the reduction
            out = fused_comm.row_linear(x, self.weight, bias, residual, self.sequence_parallel, dgelu_aux=dgelu_aux)
            return out, (self.bias if skip else None)
        local = self.tp == 1 or self.parallel_output
        if self.fp8:
            out = _fp8_matmul(self, x, bias if local else None, residual=residual if local else None,
                              dgelu_aux=dgelu_aux)
        else:
            out = fused_linear(x, self.weight, bias if local else None, residual=residual if local else None,
                               dgelu_aux=dgelu_aux)
        if not local:
            if output_is_dead() and not self.fp8:
                # recomputed block tail: the reduced values are never read, keep only shape and autograd edge
                if self.sequence_parallel:
                    out = M.reduce_scatter_to_sequence_parallel_region(out, values_unused=True)
            elif self.sequence_parallel:
                out = M.reduce_scatter_to_sequence_parallel_region(out)
            else:
                out = M.reduce_from_model_parallel_region(out)
            if bias is not None:
                out = out + bias
            if residual is not None:
                out = out + residual
        return out, (self.bias if skip else None)

    def forward_reduced(self, input_, partial_add, post_residual, dgelu_aux=None):
        """``reduce_over_tp(input_ W^T + bias + partial_add) + post_residual`` regardless of ``parallel_output``:
        the GPT-J style residual, where attention and MLP partial sums share one reduction.  Every rank's bias is
        added to its own partial product (they are distinct parameters, as in the reference's
        ``megatron/model/transformer.py:1283-1331``)."""
        x = input_ if self.input_is_parallel else M.scatter_to_model_parallel_region(input_)
        if self._fusable(x):
            return fused_comm.row_linear(x, self.weight, self.bias, post_residual, self.sequence_parallel,
                                         partial_add=partial_add, bias_partial=True, dgelu_aux=dgelu_aux)
        if self.fp8:
            out = _fp8_matmul(self, x, self.bias, residual=partial_add, dgelu_aux=dgelu_aux)
        else:
            out = fused_linear(x, self.weight, self.bias, residual=partial_add, dgelu_aux=dgelu_aux)
        if self.tp > 1:
            if output_is_dead() and not self.fp8:
                if self.sequence_parallel:
                    out = M.reduce_scatter_to_sequence_parallel_region(out, values_unused=True)
            elif self.sequence_parallel:
                out = M.reduce_scatter_to_sequence_parallel_region(out)
            else:
                out = M.reduce_from_model_parallel_region(out)
        return out + post_residual
