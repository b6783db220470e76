"""The GPT model as a flat list of layer specs (API of ``megatron/model/gpt2_model.py`` and the
``SequentialWrapper`` of ``megatron/model/utils.py:90-221``).

Spec list (index = checkpoint layer id): ``0`` embedding, ``1`` ``_pre_transformer_block``
([b,s,h] -> [s,b,h], no parameters), ``2 .. L+1`` the L mixer layers (transformer / gMLP / RWKV /
Mamba according to ``attention_config``), ``L+2`` ``_post_transformer_block`` (drop the mask,
[s,b,h] -> [b,s,h]), ``L+3`` final norm, ``L+4`` output projection (tied to the embedding unless
``no_weight_tying``).

``GPT2ModelPipe`` is the stage-partitioned form consumed by the pipeline engine;
``to_sequential()`` re-wraps the very same modules (no second allocation) for ``pipe_parallel_size: 0``.
"""
from __future__ import annotations

import math
from functools import partial

import torch
import torch.nn as nn

from ..engine.pipe_module import LayerSpec, PipelineModule, TiedLayerSpec
from ..parallel import mpu
from ..parallel.rng import set_block_tail
from ..parallel.cross_entropy import vocab_parallel_cross_entropy
from ..parallel.layers import ParallelRelativePositionBias
from .embeddings import EmbeddingPipe
from .init_functions import get_init_methods
from .norms import get_norm
from .transformer import NormPipe, ParallelLinearPipe, ParallelTransformerLayerPipe, parallel_lm_logits


def gpt2_attention_mask_func(attention_scores, ltor_mask):
    """Fill masked positions with the most negative finite value of the dtype (in place)."""
    mask_value = torch.finfo(attention_scores.dtype).min
    return attention_scores.masked_fill_(ltor_mask, mask_value)


def cross_entropy(output, labels, _fp16=False):
    """LM loss: vocab-parallel CE on fp32-cast logits, masked mean (``gpt2_model.py:60-78``).
    The kernels read the logits in their storage dtype and accumulate in fp32, which is what the
    fp32 cast of the reference buys without materialising a ``[b, s, V]`` fp32 copy."""
    labels, loss_mask = labels[0], labels[1]
    losses = vocab_parallel_cross_entropy(output.contiguous(), labels)
    loss_mask = loss_mask.reshape(-1)
    return torch.sum(losses.reshape(-1) * loss_mask) / loss_mask.sum()


def _pre_transformer_block(args):
    assert len(args) == 2, "Incorrect number of arguments to _pre_transformer_block"
    return args[0].transpose(0, 1).contiguous(), args[1]


def _post_transformer_block(args):
    assert len(args) == 2, "Incorrect number of arguments to _post_transformer_block"
    return args[0].transpose(0, 1).contiguous()


class Lambda(nn.Module):
    def __init__(self, func):
        super().__init__()
        self.func = func

    def forward(self, x):
        return self.func(x)


def recursive_setattr(m, attr, value, assert_type=None, type_filter=None):
    if assert_type is not None:
        assert isinstance(value, assert_type), "Value is not the correct type."
    if isinstance(m, (list, tuple, nn.Sequential, nn.ModuleList)):
        for i in m:
            recursive_setattr(i, attr, value, assert_type, type_filter)
    elif isinstance(m, nn.Module):
        if hasattr(m, attr) and (type_filter is None or isinstance(getattr(m, attr), type_filter)):
            setattr(m, attr, value)
        for child in m.children():
            recursive_setattr(child, attr, value, assert_type, type_filter)


class SequentialWrapper(nn.Module):
    """nn.Sequential + interval activation checkpointing + curriculum truncation + MoE loss collection."""

    def __init__(self, layers, activation_checkpoint_interval, activation_checkpoint_func, parent_class_name=None):
        super().__init__()
        self.sequential = nn.Sequential(*layers)
        self.activation_checkpoint_interval = activation_checkpoint_interval
        self.parent_class_name = parent_class_name
        self.activation_checkpoint_func = activation_checkpoint_func
        self.batch_fn = None

    def _is_checkpointable(self, funcs):
        if self.parent_class_name == "GPT2ModelPipe":
            return all("ParallelTransformerLayerPipe" in f.__class__.__name__ for f in funcs)
        return any(len(list(f.parameters())) > 0 for f in funcs if isinstance(f, nn.Module))

    def set_batch_fn(self, fn):
        self.batch_fn = fn

    def _set_parallel_output(self, value):
        last = self.sequential[-1]
        if hasattr(last, "final_linear"):
            last.final_linear.set_parallel_output(value)
        self.parallel_output = value
        for owner in getattr(self, "_owner", []):
            owner.parallel_output = value     # read by the tied-embedding logits helper

    def inference_mode(self, use_cache=True):
        recursive_setattr(self.sequential, "use_cache", use_cache, assert_type=bool)
        self._set_parallel_output(False)
        recursive_setattr(self.sequential, "training", False)

    def train_mode(self):
        recursive_setattr(self.sequential, "use_cache", False)
        self._set_parallel_output(True)
        recursive_setattr(self.sequential, "training", True)

    def clear_cache(self):
        recursive_setattr(self.sequential, "layer_past", None)

    def forward(self, forward_input, curriculum_seqlen=None, labels=None, neox_args=None):
        if self.batch_fn:
            forward_input = self.batch_fn(forward_input)
        if curriculum_seqlen is not None and isinstance(forward_input, tuple) and len(forward_input) == 3:
            neox_args.update_value("curriculum_seqlen", curriculum_seqlen)
            tokens, position_ids, attention_mask = forward_input
            if curriculum_seqlen < position_ids.size(1):
                tokens = tokens[:, :curriculum_seqlen].contiguous()
                position_ids = position_ids[:, :curriculum_seqlen].contiguous()
                if labels is not None:
                    labels = labels[:, :curriculum_seqlen].contiguous()
                if attention_mask is not None:
                    attention_mask = attention_mask[:, :, :curriculum_seqlen, :curriculum_seqlen].contiguous()
            forward_input = (tokens, position_ids, attention_mask)
        moe_losses = []
        layers = list(self.sequential)      # slicing the container itself would build a new nn.Sequential each time

        def exec_range(start, end):
            def run(*inputs):
                x = inputs[0] if len(inputs) == 1 else inputs
                block = layers[start:end]
                for i, layer in enumerate(block):
                    set_block_tail(i == len(block) - 1)
                    x = layer(x)
                    if hasattr(layer, "last_moe_loss"):
                        moe_losses.append(layer.last_moe_loss)
                return x
            return run

        n = len(layers)
        if self.activation_checkpoint_interval == 0 or not torch.is_grad_enabled():
            x = exec_range(0, n)(forward_input)
        else:
            x = forward_input
            for start in range(0, n, self.activation_checkpoint_interval):
                end = min(start + self.activation_checkpoint_interval, n)
                if not isinstance(x, tuple):
                    x = (x,)
                if self._is_checkpointable(layers[start:end]):
                    x = self.activation_checkpoint_func(exec_range(start, end), *x)
                else:
                    x = exec_range(start, end)(*x)
        return x, moe_losses


class GPT2ModelPipe(PipelineModule):
    """GPT as a pipeline of layer specs.

    :param num_tokentypes: number of token types (0 = none)
    :param parallel_output: keep the logits sharded over tensor-parallel ranks (training) or gather them
    :param topology: rank grid (``parallel.mpu.Topology``); defaults to the initialised one
    :param use_cache: keep key/value caches on the layers (generation)
    """

    def __init__(self, neox_args, num_tokentypes=0, parallel_output=True, topology=None, use_cache=False):
        self.neox_args = neox_args
        self.use_cache = use_cache
        self.parallel_output = parallel_output
        self.hidden_size = neox_args.hidden_size
        self.num_tokentypes = num_tokentypes
        self.init_method, self.output_layer_init_method = get_init_methods(neox_args)
        self.__topology__ = topology
        self.specs = []
        self.init_specs()
        num_stages = max(1, neox_args.pipe_parallel_size) if mpu.get_pipe_parallel_world_size() > 1 else 1
        super().__init__(layers=self.specs, loss_fn=partial(cross_entropy, _fp16=neox_args.fp16_lm_cross_entropy),
                         num_stages=num_stages, topology=topology,
                         activation_checkpoint_interval=neox_args.checkpoint_num_layers
                         if neox_args.checkpoint_activations else 0,
                         partition_method=neox_args.pipe_partition_method,
                         checkpointable_layers=["GMLPBlock", "ParallelTransformerLayerPipe",
                                                "ParallelMambaResidualLayerPipe", "RWKVResidualLayerPipe"])

    def insert_layers(self, layers, idx):
        """Insert layer(s) at spec index ``idx`` and rebuild (used by soft-prompt tuning)."""
        if isinstance(layers, (nn.Module, LayerSpec)) or callable(layers) and not isinstance(layers, list):
            layers = [layers]
        self.specs[idx:idx] = list(layers)
        PipelineModule.__init__(self, layers=self.specs, loss_fn=self.loss_fn, num_stages=self.num_stages,
                                activation_checkpoint_interval=self.activation_checkpoint_interval,
                                partition_method=self.neox_args.pipe_partition_method,
                                checkpointable_layers=self.checkpointable_layers)

    def init_specs(self):
        a = self.neox_args
        tied = not a.no_weight_tying
        emb_args = (a, self.hidden_size, a.padded_vocab_size, a.max_position_embeddings, a.hidden_dropout,
                    self.init_method, self.num_tokentypes)
        self.specs = []
        if tied:
            self.specs.append(TiedLayerSpec("embed", EmbeddingPipe, *emb_args,
                                            tied_weight_attr="word_embeddings_weight"))
        else:
            self.specs.append(LayerSpec(EmbeddingPipe, *emb_args))
        self.specs.append(_pre_transformer_block)
        rpe_emb = None
        if a.pos_emb == "rpe":
            hn = mpu.divide(a.hidden_size, a.num_attention_heads)
            rpe_emb = ParallelRelativePositionBias(a, scale=math.sqrt(hn), causal=True, num_buckets=a.rpe_num_buckets,
                                                   max_distance=a.rpe_max_distance, heads=a.num_attention_heads)
        for i in range(a.num_layers):
            kind = a.attention_config[i]
            if kind in ("gmlp", "amlp"):
                from .gmlp import GMLPBlock
                self.specs.append(LayerSpec(GMLPBlock, init_method=self.init_method, layer_number=i,
                                            output_layer_init_method=self.output_layer_init_method, neox_args=a,
                                            mask_fn=gpt2_attention_mask_func))
            elif kind == "rwkv":
                from .rwkv import RWKVResidualLayerPipe
                self.specs.append(LayerSpec(RWKVResidualLayerPipe, neox_args=a, layer_number=i))
            elif kind == "mamba":
                from .mamba import ParallelMambaResidualLayerPipe
                self.specs.append(LayerSpec(ParallelMambaResidualLayerPipe, neox_args=a, init_method=self.init_method,
                                            output_layer_init_method=self.output_layer_init_method, layer_number=i))
            else:
                self.specs.append(LayerSpec(ParallelTransformerLayerPipe, neox_args=a,
                                            attention_mask_func=gpt2_attention_mask_func,
                                            init_method=self.init_method,
                                            output_layer_init_method=self.output_layer_init_method, layer_number=i,
                                            rpe=rpe_emb, rotary=a.pos_emb == "rotary", use_cache=self.use_cache))
        self.specs.append(_post_transformer_block)
        norm, eps = get_norm(a)
        self.specs.append(LayerSpec(NormPipe, norm, a.hidden_size, eps=eps))

        def _logits_helper(embedding, lm_output):
            if a.use_mup:
                lm_output = lm_output / getattr(embedding.word_embeddings.weight, "mup_width_mult", 1.0)
            return parallel_lm_logits(lm_output, embedding.word_embeddings_weight, self.parallel_output,
                                      seq_parallel=a.sequence_parallel and mpu.get_model_parallel_world_size() > 1)

        if tied:
            self.specs.append(TiedLayerSpec("embed", EmbeddingPipe, *emb_args, forward_fn=_logits_helper,
                                            tied_weight_attr="word_embeddings_weight"))
        else:
            self.specs.append(LayerSpec(ParallelLinearPipe, neox_args=a, init_method=self.init_method,
                                        parallel_output=self.parallel_output, is_last_layer=True))

    def _set_parallel_output(self, value):
        final = list(self.forward_funcs)[-1]
        if isinstance(final, ParallelLinearPipe) and hasattr(final, "final_linear"):
            final.final_linear.set_parallel_output(value)
        self.parallel_output = value

    def inference_mode(self, use_cache=True):
        recursive_setattr(list(self.forward_funcs), "use_cache", use_cache, assert_type=bool)
        self._set_parallel_output(False)
        recursive_setattr(list(self.forward_funcs), "training", False)

    def train_mode(self):
        recursive_setattr(list(self.forward_funcs), "use_cache", False)
        self._set_parallel_output(True)
        recursive_setattr(list(self.forward_funcs), "training", True)

    def clear_cache(self):
        recursive_setattr(list(self.forward_funcs), "layer_past", None)

    def to_sequential(self):
        """Plain sequential form over the already-built modules (requires a single pipeline stage)."""
        assert self.num_stages == 1, "to_sequential() needs every layer on this rank (one pipeline stage)"
        layers, owners = [], {}
        for n, spec in enumerate(self.specs):
            if isinstance(spec, TiedLayerSpec):
                mod = self.tied_modules[spec.key]
                if spec.key in owners:
                    fn = spec.forward_fn
                    layers.append(Lambda(lambda x, _m=mod, _f=fn: _f(_m, x)))
                else:
                    owners[spec.key] = mod
                    layers.append(mod)
            elif isinstance(spec, LayerSpec) or isinstance(spec, nn.Module):
                layers.append(self.layer_module(n))
            elif callable(spec):
                layers.append(Lambda(spec))
            else:
                raise ValueError(f"Layer number {n} ({spec}) Not recognized")
        seq = SequentialWrapper(layers, self.activation_checkpoint_interval, self.activation_checkpoint_func,
                                parent_class_name=self.__class__.__name__)
        seq.parallel_output = self.parallel_output
        seq._owner = [self]          # a list so the pipe container is not registered as a sub-module
        return seq
