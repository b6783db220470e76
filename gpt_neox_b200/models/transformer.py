"""Transformer building blocks: MLP, self-attention, the residual layer and the LM head
(behaviour of ``megatron/model/transformer.py`` of the reference).

Activations are ``[s, b, h]`` inside the stack (sequence-parallel regions hold ``[s/tp, b, h]``).
Parameter names and weight layouts are checkpoint-compatible with the reference:
``attention.query_key_value`` (per-head interleaved ``[np, 3*hn]`` for MHA, contiguous ``[Q|K|V]`` for
GQA), ``attention.dense``, ``mlp.linear1`` (gated activations: ``[up ; gate]`` halves), ``mlp.linear2``,
``input_layernorm``, ``post_attention_layernorm``.

B200-first differences in mechanism: bias, GeLU and both residual additions are folded into GEMM
epilogues whenever no dropout or cross-rank reduction sits in between; attention always runs the
fused flash kernel (masks are generated in-kernel, no ``[1,1,s,s]`` mask tensor is consumed) unless a
feature needs explicit scores (T5 relative position bias, block-sparse patterns).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as OF
from ..ops.sparse_attention import block_sparse_attention
from ..ops.attention import flash_attention, packed_qkv_attention, packed_qkv_ok
from ..ops.linear import dead_outputs, linear as fused_linear
from ..parallel import mappings as M
from ..parallel import mpu
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear
from ..parallel.rng import get_cuda_rng_tracker, recompute_tail
from .norms import LayerNorm, get_norm
from .positional import AliBi, RotaryEmbedding, apply_rotary_pos_emb

GATED = ("geglu", "reglu", "swiglu", "bilinear", "glu")


def mlp_dims(neox_args, multiple_of=None):
    """(linear1 output size, linear2 input size) following the reference sizing rules
    (``transformer.py:121-147``): gated activations shrink the width to 2/3 and consume half."""
    mult = multiple_of if multiple_of is not None else neox_args.mlp_multiple_of
    if neox_args.intermediate_size:
        ffn = neox_args.intermediate_size
    elif neox_args.expansion_factor:
        ffn = int(neox_args.expansion_factor * neox_args.hidden_size)
    else:
        ffn = 4 * neox_args.hidden_size
    ffn_in = ffn
    if neox_args.activation in GATED:
        ffn = int(ffn * 2 / 3)
        ffn_in = ffn // 2
    ffn = int((2 * mult) * ((ffn + 2 * mult - 1) // (2 * mult)))
    ffn_in = int(mult * ((ffn_in + mult - 1) // mult))
    return ffn, ffn_in


class ParallelMLP(nn.Module):
    """h -> ffn -> h.  linear1 is column-parallel, linear2 row-parallel."""

    def __init__(self, neox_args, init_method, output_layer_init_method, parallel_output=False, multiple_of=None,
                 MOE=False, MoE_mp_size=1):
        super().__init__()
        self.activation_type = neox_args.activation
        self.is_gated = neox_args.activation in GATED
        ffn, ffn_in = mlp_dims(neox_args, multiple_of)
        self.ffn_dim, self.ffn_dim_in = ffn, ffn_in
        self.linear1 = ColumnParallelLinear(neox_args, neox_args.hidden_size, ffn, gather_output=False,
                                            init_method=init_method, skip_bias_add=True, MOE=MOE,
                                            MoE_mp_size=MoE_mp_size, bias=neox_args.use_bias_in_mlp,
                                            fp8=not MOE and (neox_args.te_columnparallel or neox_args.te_layernorm_mlp))
        self.linear2 = RowParallelLinear(neox_args, ffn_in, neox_args.hidden_size, input_is_parallel=True,
                                         init_method=output_layer_init_method, parallel_output=parallel_output,
                                         skip_bias_add=True, MOE=MOE, MoE_mp_size=MoE_mp_size,
                                         bias=neox_args.use_bias_in_mlp,
                                         fp8=not MOE and (neox_args.te_rowparallel or neox_args.te_layernorm_mlp))
        if not self.is_gated and self.activation_type != "gelu":
            self.act = OF.get_activation(self.activation_type)

    def forward(self, hidden_states, residual=None, partial_add=None, post_residual=None, fuse_bias=False,
                dead_output=False):
        """Returns ``(output, output_bias)``; ``residual`` is added by linear2 (see ``RowParallelLinear.forward``).
        With ``post_residual`` it returns ``reduce(mlp + bias + partial_add) + post_residual`` as one tensor.
        ``dead_output``: the result is not going to be read (recomputation of a checkpointed block's last layer), so
        linear2 only records its inputs for backward."""
        with dead_outputs(False):
            return self._forward(hidden_states, residual, partial_add, post_residual, fuse_bias, dead_output)

    def _forward(self, hidden_states, residual, partial_add, post_residual, fuse_bias, dead_output):
        l1 = self.linear1
        if self.activation_type == "gelu":
            # bias + GeLU in linear1's epilogue; GeLU' in linear2's data-gradient epilogue
            inter, pre = l1.matmul(hidden_states, l1.bias, act="gelu", split_pre=True)
            with dead_outputs(dead_output):
                if post_residual is not None:
                    return self.linear2.forward_reduced(inter, partial_add, post_residual, dgelu_aux=pre)
                return self.linear2(inter, residual=residual, dgelu_aux=pre, fuse_bias=fuse_bias)
        else:
            inter, bias = l1(hidden_states)
            if self.is_gated:
                inter = OF.gated_act(inter, self.activation_type, bias)
            else:
                inter = self.act(inter + bias if bias is not None else inter)
        with dead_outputs(dead_output):
            if post_residual is not None:
                return self.linear2.forward_reduced(inter, partial_add, post_residual)
            return self.linear2(inter, residual=residual, fuse_bias=fuse_bias)


class ParallelLinear(nn.Module):
    """hidden -> padded vocab (column-parallel, sequence dim 1), or hidden -> 1 for reward models."""

    def __init__(self, neox_args, parallel_output=True, init_method=nn.init.xavier_normal_, is_last_layer=False):
        super().__init__()
        self.is_rm = neox_args.train_impl == "rm"
        if not self.is_rm:
            self.final_linear = ColumnParallelLinear(neox_args, neox_args.hidden_size, neox_args.padded_vocab_size,
                                                     bias=False, init_method=init_method,
                                                     gather_output=not parallel_output, skip_bias_add=False,
                                                     mup_rescale_parameters=is_last_layer, seq_dim=1)
        else:
            self.rm_linear = RowParallelLinear(neox_args, neox_args.hidden_size, 1, bias=False,
                                               input_is_parallel=False, init_method=init_method,
                                               parallel_output=False, skip_bias_add=False,
                                               mup_rescale_parameters=is_last_layer)

    def forward(self, hidden_states):
        return self.final_linear(hidden_states) if not self.is_rm else self.rm_linear(hidden_states)


def sparse_layout_mask(kind, sq, sk, cfg, device):
    """Dense boolean mask (True = masked) equivalent to the block-sparse layouts of the reference's
    sparse attention types (``megatron/model/utils.py:253-353``): ``local`` (sliding window of blocks),
    ``sparse_fixed`` (local blocks + a global column per stride), ``sparse_variable``, ``bigbird``
    (window + global + random blocks) and ``bslongformer`` (window + global blocks)."""
    block = int(cfg.get("block", 16))
    nq, nk = (sq + block - 1) // block, (sk + block - 1) // block
    qi = torch.arange(nq, device=device)[:, None]
    ki = torch.arange(nk, device=device)[None, :]
    if kind == "local":
        w = int(cfg.get("num_sliding_window_blocks", 3))
        keep = (qi - ki).abs() <= w // 2
    elif kind in ("sparse_fixed", "sparse_variable"):
        local = int(cfg.get("num_local_blocks", 4))
        nglob = int(cfg.get("num_global_blocks", 1))
        keep = (qi // local) == (ki // local)
        keep = keep | ((ki % local) >= (local - nglob))
    elif kind == "bigbird":
        w = int(cfg.get("num_sliding_window_blocks", 3))
        nglob = int(cfg.get("num_global_blocks", 1))
        nrand = int(cfg.get("num_random_blocks", 1))
        keep = ((qi - ki).abs() <= w // 2) | (ki < nglob) | (qi < nglob)
        g = torch.Generator().manual_seed(0)
        rnd = torch.rand(nq, nk, generator=g).to(device)
        keep = keep | (rnd >= torch.topk(rnd, min(nrand, nk), dim=-1).values[:, -1:])
    elif kind == "bslongformer":
        w = int(cfg.get("num_sliding_window_blocks", 3))
        glob = cfg.get("global_block_indices", [0])
        keep = (qi - ki).abs() <= w // 2
        for gidx in glob:
            keep = keep | (ki == gidx) | (qi == gidx)
    else:
        raise ValueError(f"unknown sparse attention type {kind}")
    keep = keep.repeat_interleave(block, 0).repeat_interleave(block, 1)[:sq, :sk]
    return ~keep


class ParallelSelfAttention(nn.Module):
    """[s, b, h] -> [s, b, h] self-attention with heads sharded over tensor-parallel ranks."""

    def __init__(self, neox_args, attention_mask_func, init_method, output_layer_init_method, layer_number,
                 rpe=None, rotary=False, use_cache=False, parallel_output=False):
        super().__init__()
        self.fp16 = neox_args.precision == "fp16"
        self.bf16 = neox_args.precision == "bfloat16"
        self.attention_mask_func = attention_mask_func
        self.apply_query_key_layer_scaling = neox_args.apply_query_key_layer_scaling
        self.use_cache = use_cache
        self.attention_softmax_in_fp32 = neox_args.attention_softmax_in_fp32 or self.apply_query_key_layer_scaling
        self.layer_number = layer_number
        tp = mpu.get_model_parallel_world_size()
        self.hidden_size_per_partition = mpu.divide(neox_args.hidden_size, tp)
        self.hidden_size_per_attention_head = mpu.divide(neox_args.hidden_size, neox_args.num_attention_heads)
        self.num_attention_heads_per_partition = mpu.divide(neox_args.num_attention_heads, tp)
        self.pos_emb = neox_args.pos_emb
        self.sliding_window_width = neox_args.sliding_window_width
        hn = self.hidden_size_per_attention_head

        kv = neox_args.num_kv_heads
        if kv is not None and kv != neox_args.num_attention_heads:
            self.gqa = True
            self.num_kv_heads_per_partition = mpu.divide(kv, tp)
            self.kv_hidden_size = kv * hn
        else:
            self.gqa = False
            self.num_kv_heads_per_partition = self.num_attention_heads_per_partition
            self.kv_hidden_size = neox_args.hidden_size
        out_features = neox_args.hidden_size + 2 * self.kv_hidden_size
        self.query_key_value = ColumnParallelLinear(neox_args, neox_args.hidden_size, out_features,
                                                    gather_output=False, init_method=init_method,
                                                    bias=neox_args.use_bias_in_attn_linear,
                                                    fp8=neox_args.te_columnparallel or neox_args.te_mha)

        coeff = None
        self.norm_factor = math.sqrt(hn)
        if self.apply_query_key_layer_scaling:
            coeff = max(1, self.layer_number)
            self.norm_factor *= coeff
        if neox_args.use_mup:
            self.norm_factor = hn
        self.coeff = coeff

        self.use_qk_layernorm = neox_args.use_qk_layernorm
        if self.use_qk_layernorm:
            norm, eps = get_norm(neox_args)
            dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else None
            self.qk_layernorm = LayerNorm([self.num_attention_heads_per_partition, hn][-1], eps=eps, device=dev,
                                          dtype=neox_args.params_dtype)

        self.rpe = rpe
        if self.pos_emb == "alibi":
            self.alibi_embed = AliBi(neox_args.num_attention_heads, mp_size=tp, mp_rank=mpu.get_model_parallel_rank())
        if rotary:
            if neox_args.rotary_pct == 1:
                self.rotary_ndims = None
            else:
                assert neox_args.rotary_pct < 1
                self.rotary_ndims = int(hn * neox_args.rotary_pct)
            dim = self.rotary_ndims if self.rotary_ndims is not None else hn
            self.rotary_emb = RotaryEmbedding(dim, base=neox_args.rotary_emb_base,
                                              max_seq_len=neox_args.max_position_embeddings or neox_args.seq_length,
                                              precision=neox_args.params_dtype,
                                              save_inv_freqs=neox_args.rotary_save_freqs_buffer)
        else:
            self.rotary_emb = None

        # fixed-capacity key/value cache for graph-replayed decoding (text_generation.GraphDecoder sets these)
        self.static_kv, self.static_pos, self.static_filled = None, None, False
        self.attention_type = neox_args.attention_config[layer_number]
        self.sparse = self.attention_type not in ("global", "flash")
        self.sparsity_config = neox_args.sparsity_config or {}
        self.dropout_p = neox_args.attention_dropout
        self.attention_dropout = nn.Dropout(self.dropout_p)
        self.dense = RowParallelLinear(neox_args, neox_args.hidden_size, neox_args.hidden_size,
                                       input_is_parallel=True, init_method=output_layer_init_method,
                                       skip_bias_add=True, parallel_output=parallel_output,
                                       bias=neox_args.use_bias_in_attn_linear,
                                       fp8=neox_args.te_rowparallel or neox_args.te_mha)

    # ------------------------------------------------------------------ projections
    def _project(self, hidden_states):
        mixed, _ = self.query_key_value(hidden_states)
        np_, kvp, hn = self.num_attention_heads_per_partition, self.num_kv_heads_per_partition, \
            self.hidden_size_per_attention_head
        if not self.gqa:
            mixed = mixed.view(*mixed.shape[:-1], np_, 3 * hn)
            return mixed[..., :hn], mixed[..., hn:2 * hn], mixed[..., 2 * hn:]
        q, k, v = torch.split(mixed, (np_ * hn, kvp * hn, kvp * hn), dim=-1)
        return (q.reshape(*q.shape[:-1], np_, hn), k.reshape(*k.shape[:-1], kvp, hn),
                v.reshape(*v.shape[:-1], kvp, hn))

    # ------------------------------------------------------------------ explicit-score attention
    def _scores_attention(self, q, k, v, attention_mask):
        """Unfused path: QK^T -> (+rpe/alibi) -> scaled masked softmax -> dropout -> PV.  Needed for T5
        relative position bias, block-sparse layouts, attention dropout and fp32 softmax."""
        sq, b, np_, hn = q.shape
        sk = k.shape[0]
        if (self.sparse and sq == sk and attention_mask is None and self.rpe is None and self.pos_emb != "alibi"
                and self.sliding_window_width is None):
            # block-sparse layouts: only the kept tiles of the score matrix are computed (ops/sparse_attention.py)
            drop = None
            if self.dropout_p > 0 and self.training:
                def drop(p):
                    with get_cuda_rng_tracker().fork():
                        return self.attention_dropout(p)
            scale = (float(self.coeff) if self.coeff is not None else 1.0) / self.norm_factor
            return block_sparse_attention(q, k, v, self.attention_type, self.sparsity_config, scale, dropout=drop)
        if k.shape[2] != np_:
            rep = np_ // k.shape[2]
            k = k.repeat_interleave(rep, dim=2)
            v = v.repeat_interleave(rep, dim=2)
        qf = q.permute(1, 2, 0, 3)
        kf = k.permute(1, 2, 3, 0)
        scores = torch.matmul(qf, kf) * (1.0 / self.norm_factor)        # [b, np, sq, sk]
        if self.rpe is not None:
            scores = scores + self.rpe(sq, sk).to(scores.dtype)
        if self.pos_emb == "alibi":
            scores = self.alibi_embed(scores)
        if attention_mask is None:
            qi = torch.arange(sq, device=q.device)[:, None] + (sk - sq)
            ki = torch.arange(sk, device=q.device)[None, :]
            attention_mask = (ki > qi)
            if self.sliding_window_width is not None:
                attention_mask = attention_mask | (ki < qi - self.sliding_window_width)
            attention_mask = attention_mask[None, None]
        else:
            attention_mask = attention_mask[..., -sq:, :sk] if attention_mask.shape[-2] >= sq else attention_mask
        if self.sparse:
            attention_mask = attention_mask | sparse_layout_mask(self.attention_type, sq, sk, self.sparsity_config,
                                                                 q.device)[None, None]
        scale = float(self.coeff) if self.coeff is not None else 1.0
        if self.attention_softmax_in_fp32:
            scores = scores.float()
        probs = OF.scaled_masked_softmax(scores, attention_mask.expand(-1, 1, sq, sk) if attention_mask.shape[1] == 1
                                         else attention_mask, scale).to(q.dtype)
        if self.dropout_p > 0 and self.training:
            with get_cuda_rng_tracker().fork():
                probs = self.attention_dropout(probs)
        ctx = torch.matmul(probs, v.permute(1, 2, 0, 3))                  # [b, np, sq, hn]
        return ctx.permute(2, 0, 1, 3).contiguous()

    def static_cache_supported(self):
        """Static-cache decoding covers rotary / learned / no positional scheme with plain causal attention."""
        return (self.rpe is None and not self.sparse and self.pos_emb != "alibi" and self.sliding_window_width is None
                and not self.use_qk_layernorm)

    def _static_decode(self, q, k, v):
        """One new token against the fixed-capacity cache: write its key / value at ``static_pos``, attend to every
        slot up to that position (a mask computed on the device), all shapes independent of the position."""
        buf, pos = self.static_kv, self.static_pos
        buf[0].index_copy_(0, pos, k.to(buf.dtype))
        buf[1].index_copy_(0, pos, v.to(buf.dtype))
        keys, vals = buf[0], buf[1]
        np_ = q.shape[2]
        if keys.shape[2] != np_:
            rep = np_ // keys.shape[2]
            keys, vals = keys.repeat_interleave(rep, dim=2), vals.repeat_interleave(rep, dim=2)
        scale = (float(self.coeff) if self.coeff is not None else 1.0) / self.norm_factor
        scores = torch.einsum("qbhd,kbhd->bhqk", q, keys).float() * scale
        future = torch.arange(keys.shape[0], device=q.device)[None, None, None, :] > pos
        probs = torch.softmax(scores.masked_fill(future, float("-inf")), dim=-1).to(q.dtype)
        return torch.einsum("bhqk,kbhd->qbhd", probs, vals)

    def _packed_path(self, hidden_states, layer_past):
        """rotary + flash attention on the packed QKV projection, in place (training / no kv-cache)."""
        if self.gqa or self.use_qk_layernorm or self.use_cache or self.rpe is not None or self.sparse or \
                (self.dropout_p > 0 and self.training) or (layer_past is not None and layer_past[0].numel() > 0):
            return None
        mixed, _ = self.query_key_value(hidden_states)
        np_, hn = self.num_attention_heads_per_partition, self.hidden_size_per_attention_head
        mixed = mixed.view(*mixed.shape[:-1], np_, 3 * hn)
        if not packed_qkv_ok(mixed, hn):
            return (mixed,)
        cos = sin = None
        if self.rotary_emb is not None:
            cos, sin = self.rotary_emb(mixed, seq_len=mixed.shape[0])
            cos, sin = cos[:mixed.shape[0]], sin[:mixed.shape[0]]
        slopes = self.alibi_embed.slopes if self.pos_emb == "alibi" else None
        return packed_qkv_attention(mixed, cos, sin, causal=True, softmax_scale=(self.coeff or 1.0) / self.norm_factor,
                                    window=self.sliding_window_width, alibi_slopes=slopes)

    def forward(self, hidden_states, attention_mask=None, layer_past=None, residual=None, fuse_bias=False,
                dead_dense=False):
        packed = self._packed_path(hidden_states, layer_past)
        if packed is not None and not isinstance(packed, tuple):
            ctx = packed.reshape(packed.shape[0], packed.shape[1], self.hidden_size_per_partition)
            with dead_outputs(dead_dense):
                return self.dense(ctx, residual=residual, fuse_bias=fuse_bias)
        if isinstance(packed, tuple):
            mixed, hn = packed[0], self.hidden_size_per_attention_head
            q, k, v = mixed[..., :hn], mixed[..., hn:2 * hn], mixed[..., 2 * hn:]
        else:
            q, k, v = self._project(hidden_states)
        if self.use_qk_layernorm:
            q, k = self.qk_layernorm(q), self.qk_layernorm(k)
        static_step = self.static_kv is not None and self.use_cache and k.shape[0] == 1 and self.static_filled
        if self.rotary_emb is not None and static_step:
            # decoding against the fixed-capacity cache: the position lives on the device (``static_pos``), so the
            # same launch sequence serves every step and can be replayed from a CUDA graph
            cos, sin = self.rotary_emb(v, seq_len=self.static_kv.shape[1])
            cos_q, sin_q = cos.index_select(0, self.static_pos), sin.index_select(0, self.static_pos)
            q, k = OF.rope(q, cos_q, sin_q), OF.rope(k, cos_q, sin_q)
        elif self.rotary_emb is not None:
            offset = layer_past[0].shape[0] if layer_past is not None and layer_past[0].numel() > 0 else 0
            seq_len = k.shape[0] + offset
            cos, sin = self.rotary_emb(v, seq_len=seq_len)
            if self.rotary_ndims is not None:
                rd = self.rotary_ndims
                cos_q, sin_q = cos[offset:seq_len], sin[offset:seq_len]
                q = OF.rope(q, cos_q, sin_q)        # kernels rotate the first `rd` dims and copy the rest
                k = OF.rope(k, cos_q, sin_q)
            else:
                q, k = apply_rotary_pos_emb(q, k, cos, sin, offset=offset)
        if static_step:
            ctx = self._static_decode(q, k, v)
            ctx = ctx.reshape(ctx.shape[0], ctx.shape[1], self.hidden_size_per_partition)
            out, bias = self.dense(ctx, residual=residual, fuse_bias=fuse_bias)
            return [out, self.static_kv], bias
        if self.use_cache and self.static_kv is not None:
            # prompt pass of a static-cache generation: the usual causal attention over the prompt, whose keys and
            # values also go into the fixed-capacity buffer
            n = k.shape[0]
            self.static_kv[0, :n].copy_(k)
            self.static_kv[1, :n].copy_(v)
            self.static_filled = True
            present = self.static_kv
        elif self.use_cache:
            # keys and values live in one buffer with spare rows behind the filled part: a decoding step writes its
            # new rows in place and hands out views, instead of re-copying the whole cache with cat + stack
            present = _extend_kv_cache(layer_past, k, v)
            k, v = present[0], present[1]
        else:
            if layer_past is not None and layer_past[0].numel() > 0:
                k = torch.cat((layer_past[0].type_as(k), k), dim=0)
                v = torch.cat((layer_past[1].type_as(v), v), dim=0)
            present = None

        need_scores = self.rpe is not None or self.sparse or (self.dropout_p > 0 and self.training)
        if need_scores:
            ctx = self._scores_attention(q, k, v, attention_mask)
        else:
            slopes = self.alibi_embed.slopes if self.pos_emb == "alibi" else None
            ctx = flash_attention(q, k, v, causal=True, softmax_scale=(self.coeff or 1.0) / self.norm_factor,
                                  window=self.sliding_window_width, alibi_slopes=slopes)
        ctx = ctx.reshape(ctx.shape[0], ctx.shape[1], self.hidden_size_per_partition)
        with dead_outputs(dead_dense and not self.use_cache):
            out, bias = self.dense(ctx, residual=residual, fuse_bias=fuse_bias)
        if self.use_cache:
            out = [out, present]
        return out, bias


_ZEROS = {}


def _zero_scalar(device, dtype):
    """A shared 0-d zero on ``device`` (read-only by convention): the auxiliary loss of a layer without experts.
    Creating it per call would cost a host-to-device copy per layer and micro-batch."""
    key = (device, dtype)
    z = _ZEROS.get(key)
    if z is None:
        z = _ZEROS[key] = torch.zeros((), device=device, dtype=dtype)
    return z


def _extend_kv_cache(layer_past, k, v):
    """``[2, n + s, b, heads, d]`` view holding the cached keys / values followed by the new ones.  The view carries
    its backing buffer (``_kv_buf``, capacity grown geometrically), so the next step appends in place when there is
    room: O(s) per step instead of the O(n) of concatenating (reference: ``torch.cat`` + ``torch.stack`` per step,
    ``megatron/model/transformer.py:1003-1012``)."""
    s = k.shape[0]
    n = layer_past[0].shape[0] if layer_past is not None and layer_past[0].numel() > 0 else 0
    buf = getattr(layer_past, "_kv_buf", None) if n else None
    # ``_filled``: rows written so far; a second consumer continuing from the same past (branching) must not overwrite
    # what the first one appended, so it gets a buffer of its own
    usable = (buf is not None and buf.dtype == k.dtype and buf.shape[2:] == k.shape[1:] and buf.shape[1] >= n + s
              and buf.device == k.device and getattr(buf, "_filled", -1) == n)
    if not usable:
        cap = max(2 * (n + s), 64)
        new = torch.empty((2, cap) + tuple(k.shape[1:]), dtype=k.dtype, device=k.device)
        if n:
            new[0, :n].copy_(layer_past[0])
            new[1, :n].copy_(layer_past[1])
        buf = new
    buf[0, n:n + s].copy_(k)
    buf[1, n:n + s].copy_(v)
    buf._filled = n + s
    present = buf[:, :n + s]
    present._kv_buf = buf
    return present


class ParallelTransformerLayer(nn.Module):
    """One pre-norm residual block.  ``forward(x, attention_mask, layer_past=None)`` returns
    ``(output, moe_loss)``."""

    def __init__(self, neox_args, attention_mask_func, init_method, output_layer_init_method, layer_number, rpe=None,
                 rotary=False, use_cache=False):
        super().__init__()
        self.layer_number = layer_number
        self.neox_args = neox_args
        norm, eps = get_norm(neox_args)
        self.input_layernorm = norm(neox_args.hidden_size, eps=eps)
        self.use_cache = use_cache
        self.hidden_dropout = neox_args.hidden_dropout
        self.gpt_j_residual = neox_args.gpt_j_residual
        self.gpt_j_tied = neox_args.gpt_j_tied
        self.mlp_type = "regular"
        self.moe_type = neox_args.moe_type
        self.activation = neox_args.activation
        self.num_experts = neox_args.moe_num_experts if (layer_number % neox_args.expert_interval == 0
                                                         and neox_args.moe_num_experts > 1) else 1
        self.tp = mpu.get_model_parallel_world_size()
        self.sequence_parallel = neox_args.sequence_parallel and self.tp > 1
        self.layer_past = None
        self.attention = ParallelSelfAttention(neox_args, attention_mask_func, init_method, output_layer_init_method,
                                               layer_number, rpe=rpe, rotary=rotary, use_cache=use_cache,
                                               parallel_output=self.gpt_j_residual)
        if not (self.gpt_j_residual and self.gpt_j_tied):
            self.post_attention_layernorm = norm(neox_args.hidden_size, eps=eps)
        if self.num_experts <= 1:
            self.mlp = ParallelMLP(neox_args, init_method, output_layer_init_method,
                                   parallel_output=self.gpt_j_residual)
        else:
            from .moe import ParallelMoE, ResidualMoE
            if neox_args.moe_type == "deepspeed" and neox_args.moe_use_residual:
                dense = ParallelMLP(neox_args, init_method, output_layer_init_method, parallel_output=False)
                self.mlp = ResidualMoE(neox_args, init_method, output_layer_init_method, self.num_experts, dense)
            else:
                self.mlp = ParallelMoE(neox_args, init_method, output_layer_init_method, self.num_experts)
            self.mlp_type = "moe"

    def _reduce(self, x):
        if self.sequence_parallel:
            return M.reduce_scatter_to_sequence_parallel_region(x)
        return M.reduce_from_model_parallel_region(x)

    def forward(self, x, attention_mask=None, layer_past=None):
        layer_past = layer_past if layer_past is not None else self.layer_past
        p = self.hidden_dropout
        fuse = (p == 0.0 or not self.training)
        moe_loss = _zero_scalar(x.device, x.dtype).view(())     # a fresh tensor object over the shared zero
        if self.gpt_j_residual:
            # both norms and the residual connection read x: one autograd node, whose backward adds the three
            # gradient contributions inside the norm-backward kernels (ops/functional.py::norm_fan_out)
            if self.gpt_j_tied:
                x1, residual = OF.norm_fan_out(x, [self.input_layernorm])
                x2 = x1
            else:
                x1, x2, residual = OF.norm_fan_out(x, [self.input_layernorm, self.post_attention_layernorm])
            if fuse and self.mlp_type == "regular" and not self.use_cache:
                # attention partial (+ its bias) [+ residual when no reduction follows] accumulated by the
                # GEMM epilogues:  out = residual + attn + b_a + mlp + b_m
                attn_res = residual if self.tp == 1 else None
                # Recomputation of a checkpointed block's last layer: the layer output is never read, and both
                # output projections (attention dense, MLP linear2) feed nothing else, so they only record their
                # inputs for backward -- no GEMM, no tensor-parallel reduction.
                dead = recompute_tail()
                # the attention output bias rides in the dense GEMM's epilogue (every rank adds its own to its partial)
                a_out, a_bias = self.attention(x1, attention_mask, layer_past=layer_past, residual=attn_res,
                                               fuse_bias=True, dead_dense=dead)
                if a_bias is not None:
                    a_out = a_out + a_bias
                if self.tp == 1:
                    m_out, m_bias = self.mlp(x2, residual=a_out, fuse_bias=True, dead_output=dead)
                    if m_bias is not None:
                        m_out = m_out + m_bias
                    return m_out, moe_loss
                # one reduction for both partial sums, fused with the last GEMM:  reduce(mlp + b_m + attn + b_a) + x
                return self.mlp(x2, partial_add=a_out, post_residual=residual, dead_output=dead), moe_loss
            a_out, a_bias = self.attention(x1, attention_mask, layer_past=layer_past)
            if self.use_cache:
                a_out, presents = a_out
                self.layer_past = presents
            a_out = F.dropout(a_out + a_bias if a_bias is not None else a_out, p=p, training=self.training)
            if self.mlp_type == "moe":
                m_out, moe_loss = self.mlp(x2)
                m_bias = None
            else:
                m_out, m_bias = self.mlp(x2)
            m_out = F.dropout(m_out + m_bias if m_bias is not None else m_out, p=p, training=self.training)
            out = residual + self._reduce(m_out + a_out) if self.tp > 1 else residual + m_out + a_out
            return out, moe_loss

        # sequential residual
        h1, residual = OF.norm_fan_out(x, [self.input_layernorm])
        can_fuse_res = fuse and not self.use_cache
        a_out, a_bias = self.attention(h1, attention_mask, layer_past=layer_past,
                                       residual=residual if (can_fuse_res and self.attention.dense.bias is None) else None)
        if self.use_cache:
            a_out, presents = a_out
            self.layer_past = presents
        if can_fuse_res and self.attention.dense.bias is None:
            x = a_out
        else:
            x = OF.bias_dropout_add(a_out, a_bias, residual, p, self.training)
        ln2, x = OF.norm_fan_out(x, [self.post_attention_layernorm])
        if self.mlp_type == "moe":
            m_out, moe_loss = self.mlp(ln2)
            out = OF.bias_dropout_add(m_out, None, x, p, self.training)
        else:
            fuse_m = can_fuse_res and self.mlp.linear2.bias is None
            # (see the parallel-residual branch: in a recomputed block tail only linear2's inputs are needed)
            m_out, m_bias = self.mlp(ln2, residual=x if fuse_m else None, dead_output=fuse_m and recompute_tail())
            out = m_out if fuse_m else OF.bias_dropout_add(m_out, m_bias, x, p, self.training)
        return out, moe_loss


class ParallelTransformerLayerPipe(ParallelTransformerLayer):
    """Pipeline form: takes and returns ``(hidden_states, attention_mask)``."""

    def forward(self, args):
        assert len(args) == 2, "ParallelTransformerLayerPipe expects 2 arguments - hidden_states and attention_mask"
        hidden_states, attention_mask = args
        output, moe_loss = super().forward(hidden_states, attention_mask)
        self.last_moe_loss = moe_loss
        return output, attention_mask


class ParallelLinearPipe(ParallelLinear):
    def forward(self, args):
        assert isinstance(args, torch.Tensor), "ParallelLinearPipe expects a single argument - hidden_states"
        logits, _ = super().forward(args)
        return logits


class NormPipe(nn.Module):
    def __init__(self, norm_class, hidden_size, eps):
        super().__init__()
        self.norm = norm_class(hidden_size, eps=eps)

    def forward(self, args):
        assert not isinstance(args, tuple), "NormPipe should only receive a single tensor as input"
        return self.norm(args)


def parallel_lm_logits(input_, word_embeddings_weight, parallel_output, seq_parallel=False, seq_dim=1, bias=None):
    """LM logits with the (tied) embedding matrix as the projection."""
    if seq_parallel:
        x = M.gather_from_sequence_parallel_region(input_, seq_dim)
    else:
        x = M.copy_to_model_parallel_region(input_)
    logits = fused_linear(x, word_embeddings_weight, bias)
    return logits if parallel_output else M.gather_from_model_parallel_region(logits)
