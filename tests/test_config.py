"""Configuration system: YAML merging, derived values, validation, launcher argument round trip."""
import base64
import glob
import json
import os

import pytest
import yaml

from gpt_neox_b200.config import FIELDS, NeoXArgs, expand_attention_types

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CONFIGS = os.path.join(ROOT, "configs")

MINIMAL = {"num_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "max_position_embeddings": 128,
           "seq_length": 128, "train_micro_batch_size_per_gpu": 2, "global_num_gpus": 1,
           "optimizer": {"type": "Adam", "params": {"lr": 1e-3}}}


def _write(tmp_path, name, obj):
    p = tmp_path / name
    p.write_text(json.dumps(obj))
    return str(p)


def test_schema_is_consistent():
    assert len(FIELDS) > 300
    for f in FIELDS.values():
        assert f.accepts(f.default), f"default of {f.name} violates its own type"


def test_batch_triple_is_solved():
    a = NeoXArgs.from_dict({**MINIMAL, "global_num_gpus": 8, "model_parallel_size": 2,
                            "train_batch_size": 64, "gradient_accumulation_steps": None})
    assert a.dp_world_size == 4
    assert (a.train_batch_size, a.train_micro_batch_size_per_gpu, a.gradient_accumulation_steps) == (64, 2, 8)
    with pytest.raises(AssertionError):
        NeoXArgs.from_dict({**MINIMAL, "train_batch_size": 7, "gradient_accumulation_steps": 2})


def test_precision_and_zero_are_derived():
    a = NeoXArgs.from_dict({**MINIMAL, "bf16": {"enabled": True}, "zero_optimization": {"stage": 1}})
    assert a.precision == "bfloat16" and a.zero_stage == 1
    import torch
    assert a.params_dtype == torch.bfloat16
    b = NeoXArgs.from_dict({**MINIMAL, "fp16": {"enabled": True, "loss_scale": 0}})
    assert b.precision == "fp16" and b.fp16["enabled"] is True
    c = NeoXArgs.from_dict(MINIMAL)
    assert c.precision == "fp32" and c.zero_stage == 0 and c.lr == 1e-3 and c.optimizer_type == "Adam"


def test_attention_config_expansion():
    assert expand_attention_types([[["global", "local"], 2], [["flash"], 1]], 5) == \
        ["global", "local", "global", "local", "flash"]
    assert expand_attention_types([[["flash"], "all"]], 3) == ["flash"] * 3
    a = NeoXArgs.from_dict({**MINIMAL, "attention_config": [[["flash"], "all"]]})
    assert a.attention_config == ["flash", "flash"]


def test_yaml_merge_rules(tmp_path):
    f1 = _write(tmp_path, "model.yml", {k: v for k, v in MINIMAL.items() if k != "optimizer"} | {"pos-emb": "rotary"})
    f2 = _write(tmp_path, "opt.yml", {"optimizer": MINIMAL["optimizer"]})
    a = NeoXArgs.from_ymls([f1, f2])
    assert a.pos_emb == "rotary"                        # '-' and '_' are interchangeable
    assert set(a.config_files) == {"model.yml", "opt.yml"}
    f3 = _write(tmp_path, "dup.yml", {"hidden_size": 128})
    with pytest.raises(ValueError):
        NeoXArgs.from_ymls([f1, f2, f3])                # duplicate key across files
    with pytest.raises(TypeError):
        NeoXArgs.from_dict({**MINIMAL, "definitely_not_a_key": 1})


def test_type_and_value_validation():
    with pytest.raises(ValueError):
        NeoXArgs.from_dict({**MINIMAL, "hidden_size": "big"})
    with pytest.raises(ValueError):
        NeoXArgs.from_dict({**MINIMAL, "hidden_size": 65})                  # not divisible by heads
    with pytest.raises(ValueError):
        NeoXArgs.from_dict({**MINIMAL, "seq_length": 256})                  # exceeds max positions
    with pytest.raises(ValueError):
        NeoXArgs.from_dict({**MINIMAL, "norm": "batchnorm"})                # not in the closed set
    with pytest.raises(AssertionError):
        NeoXArgs.from_dict({**MINIMAL, "num_kv_heads": 3})                  # must divide the head count
    with pytest.raises(AssertionError):
        NeoXArgs.from_dict({**MINIMAL, "moe_num_experts": 4, "sequence_parallel": True})


def test_worker_argument_round_trip(tmp_path):
    f1 = _write(tmp_path, "a.yml", {**MINIMAL, "global_num_gpus": 1})
    script = tmp_path / "train.py"
    script.write_text("")
    a = NeoXArgs.consume_deepy_args([str(script), f1])
    argv = a.get_deepspeed_main_args()
    assert argv[argv.index(str(script)) + 1] == "--deepspeed_config"
    blob = argv[argv.index("--megatron_config") + 1]
    decoded = json.loads(base64.urlsafe_b64decode(blob).decode())
    assert decoded["hidden_size"] == 64
    b = NeoXArgs.consume_neox_args(input_args=argv[argv.index(str(script)) + 1:])
    for key in ("hidden_size", "num_layers", "train_batch_size", "lr", "precision", "attention_config"):
        assert getattr(a, key) == getattr(b, key)
    ds = a.deepspeed_config
    assert ds["train_batch_size"] == a.train_batch_size and "hidden_size" not in ds


def test_conf_dir_and_missing_suffix(tmp_path):
    _write(tmp_path, "small.yml", MINIMAL)
    script = tmp_path / "train.py"
    script.write_text("")
    a = NeoXArgs.consume_deepy_args([str(script), "-d", str(tmp_path), "small"])
    assert a.hidden_size == 64


def test_hostfile_resource_pool(tmp_path):
    from gpt_neox_b200.config import resource_pool
    hf = tmp_path / "hostfile"
    hf.write_text("node1 slots=4\nnode2 slots=4\n# comment\n")
    assert resource_pool(str(hf)) == {"node1": [0, 1, 2, 3], "node2": [0, 1, 2, 3]}
    assert resource_pool(str(hf), include="node1:0,2") == {"node1": [0, 2]}
    assert resource_pool(str(hf), exclude="node2") == {"node1": [0, 1, 2, 3]}
    a = NeoXArgs.from_dict({**{k: v for k, v in MINIMAL.items() if k != "global_num_gpus"}, "hostfile": str(hf),
                            "train_micro_batch_size_per_gpu": 1})
    assert a.global_num_gpus == 8


def _config_keys(path):
    with open(path) as fh:
        return {k.replace("-", "_") for k in (yaml.load(fh, Loader=yaml.FullLoader) or {})}


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(CONFIGS, "**", "*.yml"), recursive=True)),
                         ids=lambda p: os.path.relpath(p, CONFIGS))
def test_every_shipped_config_loads(path):
    """Model files load (with the overlays they are meant to be combined with); overlays only contain declared keys."""
    keys = _config_keys(path)
    if "num_layers" not in keys:
        unknown = keys - set(NeoXArgs.known_keys())
        assert not unknown, f"{path}: undeclared keys {sorted(unknown)}"
        return
    files = [path]
    if "optimizer" not in keys and os.path.basename(os.path.dirname(path)) == "llama":
        files.append(os.path.join(CONFIGS, "llama", "train_config.yml"))
    have = set().union(*[_config_keys(f) for f in files])
    if not have & {"data_path", "train_data_paths", "vocab_file", "save", "load"}:
        files.append(os.path.join(CONFIGS, "local_setup.yml"))
        have |= _config_keys(files[-1])
    over = {} if "global_num_gpus" in have else {"global_num_gpus": 8}
    if not have & {"train_micro_batch_size_per_gpu", "train_batch_size"}:
        over["train_micro_batch_size_per_gpu"] = 1
    if not have & {"checkpoint_factor", "extra_save_iters"}:
        over["checkpoint_factor"] = 1000
    a = NeoXArgs.from_ymls(files, overwrite_values=over)
    assert a.num_layers > 0 and a.train_batch_size > 0
    # the precision named in the file is the one the run gets
    want = "fp16" if (keys & {"fp16"}) and not (keys & {"bf16"}) and "precision" not in keys else None
    if want:
        assert a.precision == "fp16", (path, a.precision)


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(CONFIGS, "**", "*.json"), recursive=True)),
                         ids=lambda p: os.path.relpath(p, CONFIGS))
def test_json_configs_parse(path):
    import json
    with open(path) as fh:
        assert isinstance(json.load(fh), dict)


def test_every_argument_used_in_code_is_declared():
    """Scan the package for ``neox_args.<name>`` / ``args.<name>`` reads and check each name against the schema
    (the check the reference runs in tests/neox_args/test_neoxargs_usage.py:24-85)."""
    import re
    # attributes attached at run time (objects, not configuration)
    runtime = {"tokenizer", "tensorboard_writer", "comet_experiment", "py"}
    known = set(NeoXArgs.known_keys()) | set(dir(NeoXArgs)) | runtime
    pat = re.compile(r"\bneox_args\.([a-zA-Z_][a-zA-Z0-9_]*)")
    root = os.path.join(os.path.dirname(CONFIGS), "gpt_neox_b200")
    missing = {}
    for dirpath, _, files in os.walk(root):
        for f in files:
            if not f.endswith(".py"):
                continue
            with open(os.path.join(dirpath, f)) as fh:
                for name in pat.findall(fh.read()):
                    if name not in known:
                        missing.setdefault(name, []).append(os.path.relpath(os.path.join(dirpath, f), root))
    assert not missing, missing


def test_elastic_batch_configuration():
    from gpt_neox_b200.config.elasticity import ElasticityError, compute_elastic_config, valid_gpu_counts
    block = {"enabled": True, "max_train_batch_size": 2000, "micro_batch_sizes": [2, 4, 6], "min_gpus": 1,
             "max_gpus": 64}
    batch, gpus, micro = compute_elastic_config(block, world_size=8)
    assert batch <= 2000 and gpus == valid_gpu_counts(batch, [2, 4, 6], 1, 64) and 8 in gpus
    assert micro in (2, 4, 6) and batch % (micro * 8) == 0
    # no other batch size admits more GPU counts, and among equals the largest was taken
    for other in range(2, 2001, 2):
        n = len(valid_gpu_counts(other, [2, 4, 6], 1, 64))
        assert n < len(gpus) or (n == len(gpus) and other <= batch)
    small, _, _ = compute_elastic_config({**block, "prefer_larger_batch": False})
    assert small <= batch and len(valid_gpu_counts(small, [2, 4, 6], 1, 64)) == len(gpus)
    with pytest.raises(ElasticityError):
        compute_elastic_config({"micro_batch_sizes": [8], "max_train_batch_size": 4})
    with pytest.raises(ElasticityError):
        compute_elastic_config({"micro_batch_sizes": [3], "max_train_batch_size": 9, "min_gpus": 1, "max_gpus": 4}, 2)


def test_elasticity_block_sets_the_batch_triple():
    cfg = {k: v for k, v in MINIMAL.items() if k != "train_micro_batch_size_per_gpu"}
    cfg.update(global_num_gpus=4, elasticity={"enabled": True, "max_train_batch_size": 96, "micro_batch_sizes": [2, 3],
                                              "min_gpus": 1, "max_gpus": 8})
    args = NeoXArgs.from_dict(cfg)
    assert args.train_batch_size == args.train_micro_batch_size_per_gpu * args.gradient_accumulation_steps * 4
    assert args.train_batch_size <= 96 and args.train_micro_batch_size_per_gpu in (2, 3)
    with pytest.raises(AssertionError):
        NeoXArgs.from_dict(dict(cfg, train_batch_size=args.train_batch_size + 4))
