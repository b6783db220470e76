"""Declarative schema of every configuration key.

The configuration surface (key names, defaults, accepted values) is the one documented in
``configs/neox_arguments.md`` of the reference and declared there as eleven dataclass mix-ins
(``megatron/neox_arguments/neox_args.py:55-1682``, ``deepspeed_args.py:29-369``).  Here it is a single
text table parsed at import time into ``FIELDS``; ``NeoXArgs`` (``args.py``) is generated from it.

Line format:   ``name : type = default   # one-line description``
Types:         ``int float str bool list dict any``, ``lit[a|b|c]`` (closed set of strings) and
               unions written ``int|list``.  Every key also accepts ``None``.
"""
from __future__ import annotations

import ast
from dataclasses import dataclass
from typing import Any

_TABLE = r"""
[parallelism]
pipe_parallel_size : int = 0                       # pipeline stages; 0 runs the plain sequential module, >=1 the pipeline engine
model_parallel_size : int = 1                      # tensor (Megatron) parallel degree
pipe_partition_method : str = 'type:transformer|mlp'   # how layers are split over stages: 'uniform', 'parameters' or 'type:<regex>'
world_size : int = None                            # total ranks, filled in from the environment
is_pipe_parallel : bool = False                    # derived: pipe_parallel_size >= 1
sequence_parallel : bool = False                   # Megatron sequence parallelism over the tensor-parallel group
expert_interval : int = 2                          # place an MoE block every N-th layer

[model]
precision : lit[fp16|fp32|bfloat16] = None         # parameter / compute dtype
num_layers : int = None                            # transformer depth
hidden_size : int = None                           # model width
intermediate_size : int = None                     # MLP width (before gating); overrides expansion_factor
mlp_multiple_of : int = 1                          # round the MLP width up to a multiple of this
expansion_factor : float = None                    # MLP width = expansion_factor * hidden_size
num_attention_heads : int = None                   # query heads
num_kv_heads : int = None                          # key/value heads (grouped-query attention); None = num_attention_heads
seq_length : int = None                            # training sequence length
sliding_window_width : int = None                  # local attention window; None = full causal attention
max_position_embeddings : int = None               # longest position the model supports
norm : lit[layernorm|rmsnorm|scalenorm|te_rmsnorm|te_layernorm] = 'layernorm'   # normalisation layer
layernorm_fusion : bool = False                    # use the fused LayerNorm kernel
rmsnorm_fusion : bool = False                      # use the fused RMSNorm kernel
use_qk_layernorm : bool = False                    # LayerNorm on per-head queries and keys
layernorm_epsilon : float = 1e-05                  # LayerNorm epsilon
rms_norm_epsilon : float = 1e-08                   # RMSNorm epsilon
scalenorm_epsilon : float = 1e-08                  # ScaleNorm epsilon
pos_emb : lit[learned|rotary|sinusoidal|rpe|alibi|none] = 'learned'   # positional information
rpe_num_buckets : int = 32                         # T5 relative-position buckets
rpe_max_distance : int = 128                       # T5 relative-position maximum distance
opt_pos_emb_offset : int = 0                       # OPT-style offset added to learned position ids
no_weight_tying : bool = False                     # untie input embedding and output projection
attention_config : list = None                     # per-layer attention kinds, e.g. [[["flash"], "all"]]
sparsity_config : dict = None                      # block-sparse attention options
num_unique_layers : int = None                     # parameter sharing: number of distinct layers
param_sharing_style : str = 'grouped'              # 'grouped' or 'spaced' parameter sharing
make_vocab_size_divisible_by : int = 128           # pad the vocabulary to a multiple of this (times TP)
activation : lit[gelu|geglu|relu|softsign|swish|mish|silu|reglu|swiglu|bilinear|glu] = 'gelu'   # MLP non-linearity
use_flashattn_swiglu : bool = False                # use the fused SwiGLU kernel
scaled_upper_triang_masked_softmax_fusion : bool = False   # fused causal softmax kernel
scaled_masked_softmax_fusion : bool = False        # fused masked softmax kernel
bias_gelu_fusion : bool = False                    # fuse bias add and GeLU
bias_dropout_fusion : bool = False                 # fuse bias add, dropout and residual add
rope_fusion : bool = False                         # fused rotary embedding kernel
fp16_lm_cross_entropy : bool = False               # keep logits in fp16 for the loss
init_method_std : float = 0.02                     # std of the normal initialiser
apply_query_key_layer_scaling : bool = False       # scale QK^T by 1/layer_number (forces fp32 softmax)
use_cpu_initialization : bool = False              # initialise weights on the host
attention_softmax_in_fp32 : bool = False           # compute softmax in fp32
rotary_pct : float = 1.0                           # fraction of each head that is rotated
rotary_emb_base : int = 10000                      # rotary frequency base
rotary_save_freqs_buffer : bool = False            # keep inv_freq in the state dict
init_method : lit[normal|scaled_normal|orthogonal|scaled_orthogonal|xavier_uniform|xavier_normal|wang_init|small_init|single_residual_scaled_normal] = 'normal'   # weight initialiser
output_layer_init_method : lit[normal|scaled_normal|orthogonal|scaled_orthogonal|xavier_uniform|xavier_normal|wang_init|small_init|single_residual_scaled_normal] = 'scaled_normal'   # initialiser of residual-output projections
gmlp_attn_dim : int = 64                           # tiny-attention width inside aMLP blocks
gpt_j_residual : bool = False                      # parallel attention + MLP residual
gpt_j_tied : bool = False                          # share one LayerNorm between the parallel branches
use_bias_in_norms : bool = True                    # norms carry a bias
use_bias_in_attn_linear : bool = True              # attention projections carry biases
use_bias_in_mlp : bool = True                      # MLP projections carry biases
soft_prompt_tuning : dict = None                   # {'enabled', 'num_tokens', 'init_string', 'init_range'}
mamba_selective_scan_fusion : bool = False         # fused selective-scan kernel
mamba_causal_conv_fusion : bool = False            # fused causal conv1d kernel
mamba_inner_func_fusion : bool = False             # fully fused Mamba inner function
mamba_selective_fp32_params : bool = True          # keep A_log and D in fp32
mamba_use_bias_in_conv : bool = True               # bias in the Mamba conv1d
mamba_use_bias_in_linears : bool = False           # bias in the Mamba projections
output_layer_parallelism : lit[column] = 'column'  # sharding of the output projection
serve_model_weights : bool = False                 # export CUDA IPC handles of the weights over TCP
weight_server_port : int|list = 6000               # base port of the weight server
online_dataserver_ips : str|list = 'localhost'     # hosts of the online data servers
online_dataserver_ports : int|list = 10000         # ports of the online data servers
te_columnparallel : bool = False                   # run column-parallel linears on the fp8 tensor cores
te_rowparallel : bool = False                      # run row-parallel linears on the fp8 tensor cores
te_fp8_recipe : lit[current|delayed|mxfp8] = 'current'   # per-tensor scale from this tensor's amax / from an amax history / 32-element E8M0 block scales fed to the block-scaled tcgen05 GEMM (csrc/gemm_mxfp8_sm100.cu)
te_layernorm_mlp : bool = False                    # both MLP linears in fp8 (whatever te_columnparallel / te_rowparallel say)
te_mha : bool = False                              # QKV and output projections of attention in fp8
te_fp8_format : lit[e4m3|hybrid] = 'hybrid'        # 'hybrid' = E4M3 forward, E5M2 gradients
te_fp8_wgrad : bool = True                         # weight gradients in fp8 too
te_fp8_amax_history_len : int = 1                  # delayed-scaling history length
te_fp8_amax_compute_algo : str = 'most_recent'     # delayed-scaling amax rule: 'max' over the history or 'most_recent'
te_fp8_margin : int = 0                            # scaling margin
te_fp8_mha : bool = False                          # accepted; the attention core (QK^T, PV) stays bf16
dim_att : int = None                               # RWKV attention width
head_size : int = None                             # RWKV head size
ffn_dim : int = None                               # RWKV channel-mix width

[optimizer]
optimizer_type : lit[adam|onebitadam|cpu_adam|cpu_torch_adam|sm3|madgrad_wd|sgd|lion] = 'adam'   # derived from optimizer.type
use_bnb_optimizer : bool = False                   # 8-bit optimizer states
zero_stage : int|list|lit[all] = None              # derived from zero_optimization.stage
zero_reduce_scatter : bool = None                  # derived
zero_contiguous_gradients : bool = None            # derived
zero_reduce_bucket_size : int = None               # derived
zero_allgather_bucket_size : int = None            # derived
lr : float = None                                  # derived from optimizer.params.lr

[lr_scheduler]
lr_decay_style : lit[constant|linear|cosine|exponential] = 'linear'   # decay curve
lr_decay_iters : int = None                        # decay horizon; None = train_iters
lr_decay_fraction : float = None                   # decay horizon as a fraction of train_iters
min_lr : float = 0.0                               # floor of the schedule
warmup : float = 0.01                              # warm-up fraction of the decay horizon
override_lr_scheduler : bool = False               # ignore scheduler state found in a checkpoint
use_checkpoint_lr_scheduler : bool = False         # take all scheduler values from the checkpoint

[logging]
use_wandb : bool = None                            # log to Weights & Biases
wandb_group : str = None
wandb_run_name : str = None
wandb_team : str = None
wandb_project : str = 'neox'
wandb_host : str = 'https://api.wandb.ai'
wandb_init_all_ranks : bool = False
git_hash : str = None                              # commit of the code that ran
log_dir : str = None                               # directory of the per-host stdout/stderr tee
tensorboard_dir : str = None
use_comet : bool = None
comet_workspace : str = None
comet_project : str = None
comet_experiment_name : str = None
comet_tags : list = None
comet_others : dict = None
comet_experiment : any = None
peak_theoretical_tflops : float = None             # denominator for MFU / HFU
log_interval : int = 100
log_grad_pct_zeros : bool = False
log_param_norm : bool = False
log_grad_norm : bool = False
log_optimizer_states : bool = False
log_gradient_noise_scale : bool = False
gradient_noise_scale_n_batches : int = 5
gradient_noise_scale_cpu_offload : bool = False
memory_profiling : bool = False
memory_profiling_path : str = None
profile : bool = False
profile_step_start : int = 10
profile_step_stop : int = 12

[other]
distributed_backend : str = 'nccl'
local_rank : int = None
rank : int = None
lazy_mpu_init : bool = False
short_seq_prob : float = 0.1
eod_mask_loss : bool = False
adlr_autoresume : bool = False
adlr_autoresume_interval : int = 1000
seed : int = 1234
onnx_safe : bool = False
deepscale : bool = False
deepscale_config : str = None
deepspeed_mpi : bool = False
deepspeed_slurm : bool = False
user_script : str = None
iteration : int = None
do_train : bool = None
do_valid : bool = None
do_test : bool = None
global_num_gpus : int = None

[tokenizer]
tokenizer_type : lit[GPT2BPETokenizer|HFTokenizer|HFGPT2Tokenizer|SPMTokenizer|CharLevelTokenizer|TiktokenTokenizer] = 'GPT2BPETokenizer'
padded_vocab_size : int = None

[training]
data_path : str = None
autotuning_metric_path : str = None             # set by the autotuner for a trial run: file that receives the measured throughput
use_shared_fs : bool = True
train_data_paths : list = None
train_label_data_paths : list = None
train_reward_data_paths : list = None
test_data_paths : list = None
test_label_data_paths : list = None
test_reward_data_paths : list = None
valid_data_paths : list = None
valid_label_data_paths : list = None
valid_reward_data_paths : list = None
pos_train_data_paths : list = None
neg_train_data_paths : list = None
pos_train_label_data_paths : list = None
neg_train_label_data_paths : list = None
pos_valid_data_paths : list = None
neg_valid_data_paths : list = None
pos_valid_label_data_paths : list = None
neg_valid_label_data_paths : list = None
pos_test_data_paths : list = None
neg_test_data_paths : list = None
pos_test_label_data_paths : list = None
neg_test_label_data_paths : list = None
train_data_weights : list = None
valid_data_weights : list = None
test_data_weights : list = None
weight_by_num_documents : bool = False
weighted_sampler_alpha : float = 1.0
data_impl : lit[infer|mmap|cached] = 'infer'
pack_impl : lit[packed|pack_until_overflow|unpacked] = 'packed'
dataset_impl : lit[gpt2|pairwise|online] = 'gpt2'
train_impl : lit[normal|dpo|rm|kto|reinforce] = 'normal'
dpo_fp32 : bool = True
dpo_reference_free : bool = False
dpo_beta : float = 0.1
kto_fp32 : bool = True
kto_desirable_weight : float = 1.0
kto_undesirable_weight : float = 1.0
z_loss : float = 0.0
kto_beta : float = 0.1
fp32_reinforce : bool = True
kl_impl : lit[abs|mse|kl|full] = 'mse'
kl_div_beta : float = 0.1
reinforce_leave_one_out : bool = False
allow_chopped : bool = True
mmap_warmup : bool = False
save : str = None
s3_path : str = None
s3_chunk_size : int = 104857600
config_files : dict = None
load : str = None
checkpoint_validation_with_forward_pass : bool = False
checkpoint_scale : lit[linear|log] = 'linear'
checkpoint_factor : int|float = None
extra_save_iters : list = None
no_save_optim : bool = False
no_save_rng : bool = False
no_load_optim : bool = False
no_load_rng : bool = False
finetune : bool = False
batch_size : int = None
train_iters : int = None
train_epochs : int = None
eval_iters : int = 100
keep_last_n_checkpoints : int = None
eval_interval : int = 1000
split : str = '969, 30, 1'
vocab_file : str = None
merge_file : str = None
num_workers : int = 2
exit_interval : int = None
attention_dropout : float = 0.0
hidden_dropout : float = 0.0
weight_decay : float = 0.1
checkpoint_activations : bool = False
checkpoint_num_layers : int = 1
deepspeed_activation_checkpointing : bool = True
contiguous_checkpointing : bool = False
checkpoint_in_cpu : bool = False
synchronize_each_layer : bool = False
profile_backward : bool = False
partition_activations : bool = False
clip_grad : float = 1.0
hysteresis : int = 2
dynamic_loss_scale : bool = None
loss_scale : float = None
loss_scale_window : float = 1000.0
min_scale : float = 1.0
char_level_ppl : bool = False
use_mup : bool = False
coord_check : bool = False
save_base_shapes : bool = False
base_shapes_file : str = None
mup_init_scale : float = 1.0
mup_attn_temp : float = 1.0
mup_output_temp : float = 1.0
mup_embedding_mult : float = 1.0
mup_rp_embedding_mult : float = 1.0
mup_width_scale : int = 2

[textgen]
cuda_graph_decode : bool = False                   # decode against fixed-capacity key/value caches and replay each step from a CUDA graph (single GPU, rotary / learned positions)
text_gen_type : str = None
precompute_model_name : str = None
temperature : float = 0.0
top_p : float = 0.0
top_k : int = 0
return_logits : bool = False
maximum_tokens : int = 64
prompt_end : str = '\n'
sample_input_file : str = None
sample_output_file : str = 'samples.txt'
num_samples : int = 1
recompute : bool = False
eval_results_prefix : str = ''
eval_tasks : list = None
moe_top_k : int = 1
use_tutel : bool = False
moe_num_experts : int = 1
moe_loss_coeff : float = 0.1
moe_train_capacity_factor : float = 1.0
moe_eval_capacity_factor : float = 1.0
moe_min_capacity : int = 4
moe_token_dropping : bool = False
create_moe_param_group : bool = True
moe_use_residual : bool = True
moe_expert_parallel_size : int = 1
moe_type : str = 'megablocks'
moe_glu : bool = False
moe_lbl_in_fp32 : bool = False
moe_jitter_eps : float = None
enable_expert_tensor_parallelism : bool = False

[engine]
deepspeed : bool = True
train_batch_size : int = None
train_micro_batch_size_per_gpu : int = None
gradient_accumulation_steps : int = 1
optimizer : dict = None
scheduler : dict = None
fp32_allreduce : bool = False
prescale_gradients : bool = False
gradient_predivide_factor : float = 1.0
sparse_gradients : bool = False
fp16 : dict = None
bf16 : dict = None
amp : dict = None
gradient_clipping : float = 1.0
zero_optimization : dict = None
curriculum_learning : dict = None
curriculum_seqlen : int = 0
steps_per_print : int = 10
wall_clock_breakdown : bool = False
dump_state : bool = False
flops_profiler : dict = None
communication_data_type : bool = None
autotuning : dict = None
activation_checkpointing : dict = None
sparse_attention : dict = None
data_efficiency : dict = None
tensorboard : dict = None
wandb : dict = None
csv_monitor : dict = None
elasticity : dict = None
comms_logger : dict = None
compression_training : dict = None
checkpoint : dict = None
data_types : dict = None
deepspeed_extra_args : dict = None

[runner]
hostfile : str = None
include : str = None
exclude : str = None
num_nodes : int = -1
num_gpus : int = None
master_port : int = 29500
master_addr : str = None
launcher : lit[pdsh|openmpi|mvapich|slurm] = 'pdsh'
force_multi : bool = False
detect_nvlink_pairs : bool = False
autotuning_run : str = None
no_ssh_check : bool = False
comment : str = None
account : str = None
"""


@dataclass(frozen=True)
class Field:
    name: str
    group: str
    types: tuple          # python types accepted (besides None)
    choices: tuple        # allowed literal strings ('' = unrestricted)
    default: Any
    doc: str

    def accepts(self, value) -> bool:
        if value is None or not self.types and not self.choices:
            return True
        if self.choices and isinstance(value, str) and value.lower() in {c.lower() for c in self.choices}:
            return True
        if value == "auto":   # autotuning placeholder
            return True
        for t in self.types:
            if t is Any:
                return True
            if t is float and isinstance(value, (int, float)) and not isinstance(value, bool):
                return True
            if t is int and isinstance(value, bool):
                continue
            if isinstance(value, t):
                return True
        return False

    def type_str(self) -> str:
        parts = [t.__name__ if t is not Any else "any" for t in self.types]
        if self.choices:
            parts.append("one of " + ", ".join(repr(c) for c in self.choices))
        return " | ".join(parts)


_PY = {"int": int, "float": float, "str": str, "bool": bool, "list": list, "dict": dict, "any": Any}


def _parse_type(spec: str):
    types, choices = [], []
    depth, cur, parts = 0, "", []
    for ch in spec:
        if ch == "[":
            depth += 1
        elif ch == "]":
            depth -= 1
        if ch == "|" and depth == 0:
            parts.append(cur)
            cur = ""
        else:
            cur += ch
    parts.append(cur)
    for p in parts:
        p = p.strip()
        if p.startswith("lit["):
            choices.extend(x.strip() for x in p[4:-1].split("|"))
        else:
            types.append(_PY[p])
    return tuple(types), tuple(choices)


def _parse_table(text: str):
    fields, group = {}, None
    for raw in text.splitlines():
        line = raw.rstrip()
        if not line.strip():
            continue
        if line.startswith("["):
            group = line.strip()[1:-1]
            continue
        doc = ""
        # the description starts at the last " # " that is outside quotes
        if "   #" in line:
            line, doc = line.split("   #", 1)
        name, rest = line.split(":", 1)
        tspec, default = rest.split("=", 1)
        types, choices = _parse_type(tspec.strip())
        fields[name.strip()] = Field(name.strip(), group, types, choices, ast.literal_eval(default.strip()),
                                     doc.strip())
    return fields


FIELDS: dict[str, Field] = _parse_table(_TABLE)
GROUPS: dict[str, list[str]] = {}
for _f in FIELDS.values():
    GROUPS.setdefault(_f.group, []).append(_f.name)

# keys that make up the engine ("deepspeed") configuration dict and the launcher flags
ENGINE_KEYS = tuple(GROUPS["engine"])
RUNNER_KEYS = tuple(GROUPS["runner"])

ATTENTION_TYPE_CHOICES = ("global", "local", "sparse_fixed", "sparse_variable", "bigbird", "bslongformer", "gmlp",
                          "amlp", "flash", "rwkv", "mamba")

ZERO_DEFAULTS = {"stage": 0, "allgather_partitions": True, "reduce_scatter": True, "allgather_bucket_size": int(5e8),
                 "overlap_comm": False, "reduce_bucket_size": int(5e8), "contiguous_gradients": False}
OPT_DEFAULT = "Adam"
OPT_PARAMS_DEFAULTS = {"lr": 0.001, "betas": [0.9, 0.999], "eps": 1.0e-8, "weight_decay": 0,
                       "freeze_step": 400, "momentum": 0.0, "cuda_aware": False}
