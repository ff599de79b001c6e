"""Configuration, registry, safetensors reader and the weight loader's single error."""
import json
import os
import struct

import pytest
import torch

import helpers
from lia_rs_b200 import ConfigError, LlamaConfig, WeightError, write_random_model
from lia_rs_b200.config import known_architectures, resolve_architecture
from lia_rs_b200.weights import (SafetensorsError, load_weights, parse_header, storage_dtype,
                                 write_safetensors)

BASE = helpers.TINY["tiny-A"]["config"]


def test_config_reads_every_key_and_derives_scales():
    cfg = LlamaConfig.from_dict(BASE)
    assert (cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (64, 4, 2, 16)
    assert cfg.embedding_scale == 12 and abs(cfg.residual_scale - 1.4 / 2 ** 0.5) < 1e-12
    assert cfg.logit_scale == 32 / 64 and cfg.tie_word_embeddings
    plain = dict(BASE)
    for key in ("scale_emb", "scale_depth", "dim_model_base", "head_dim"):
        plain.pop(key)
    cfg = LlamaConfig.from_dict(plain)       # absent scalars: the reference's plain Llama
    assert (cfg.embedding_scale, cfg.residual_scale, cfg.logit_scale, cfg.head_dim) == (1.0, 1.0, 1.0, 16)
    assert LlamaConfig.from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("change, message", [
    ({"hidden_act": "gelu"}, "hidden_act"), ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"type": "linear"}}, "rope_scaling"), ({"quantization_config": {"bits": 4}}, "quantized"),
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 7}, "even"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"), ({"rope_theta": -1}, "rope_theta"), ({"vocab_size": None}, "vocab_size"),
    ({"layer_types": ["sliding_attention", "full_attention"]}, "sliding_window"),
    ({"layer_types": ["full_attention"]}, "layer_types"), ({"scale_depth": float("inf")}, "scale_depth"),
])
def test_config_refusals(change, message):
    with pytest.raises(ConfigError, match=message):
        LlamaConfig.from_dict({**BASE, **change})


def test_sizes_the_kernels_cannot_take_are_refused_when_the_model_is_described():
    """The configuration class knows the architecture, not the kernels: a head size that the attention kernels do
    not take passes `LlamaConfig` and is refused by the attention part when the model's description is put
    together (on the CPU, before any tensor is read), with the kernels' reason."""
    for head_dim in (24, 272):
        config = LlamaConfig.from_dict({**BASE, "head_dim": head_dim})
        with pytest.raises(ValueError, match="multiple of 16 of at most 256"):
            resolve_architecture(config.to_dict()).build(config)
    config = LlamaConfig.from_dict({**BASE, "head_dim": 48})
    assert len(resolve_architecture(config.to_dict()).build(config).layers) == config.num_hidden_layers


def test_registry():
    assert "LlamaForCausalLM" in known_architectures() and "llama" in known_architectures()
    assert resolve_architecture({"model_type": "llama"}).config_class is LlamaConfig
    with pytest.raises(ConfigError, match="unsupported model architecture.*known"):
        resolve_architecture({"architectures": ["Mystery"], "model_type": "mystery"})
    with pytest.raises(ConfigError, match="capacity"):
        LlamaConfig.from_dict(BASE).validate_capacity(257)


def test_safetensors_header_checks():
    ok = {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}
    assert parse_header(json.dumps(ok).encode(), 8)["a"].shape == (2,)
    cases = [
        ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, 4, "extent"),
        ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]},
          "b": {"dtype": "F32", "shape": [1], "data_offsets": [8, 12]}}, 12, "gap"),
        ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]},
          "b": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}}, 4, "gap or overlapping"),
        ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}}, 8, "unindexed"),
        ({"a": {"dtype": "F8", "shape": [1], "data_offsets": [0, 1]}}, 1, "unsupported safetensors dtype"),
        ({"__metadata__": {"k": 1}}, 0, "metadata"),
    ]
    for header, size, message in cases:
        with pytest.raises(SafetensorsError, match=message):
            parse_header(json.dumps(header).encode(), size)
    with pytest.raises(SafetensorsError, match="start with an object"):
        parse_header(b"[1]", 0)


def test_random_model_folder_roundtrip_and_storage_types(tmp_path):
    cfg = LlamaConfig.from_dict(helpers.TINY["tiny-B"]["config"])
    folder = write_random_model(cfg, str(tmp_path / "m"), seed=3)
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    raw = json.load(open(os.path.join(folder, "config.json")))
    arch = resolve_architecture(raw)
    assert arch.config_class.from_dict(raw) == cfg
    specs = arch.build(cfg).tensor_specs()
    weights = load_weights(folder, specs)
    assert set(weights) == {s.name for s in specs} and "lm_head.weight" in weights
    assert all(t.dtype == torch.bfloat16 for t in weights.values())
    again = write_random_model(cfg, str(tmp_path / "n"), seed=3)
    same = load_weights(again, specs)
    assert all(torch.equal(weights[k], same[k]) for k in weights)
    other = load_weights(write_random_model(cfg, str(tmp_path / "o"), seed=4), specs)
    assert not torch.equal(weights["model.embed_tokens.weight"], other["model.embed_tokens.weight"])
    assert torch.equal(weights["model.norm.weight"], torch.ones(96, dtype=torch.bfloat16))
    # storage rule: 16-bit floats -> bfloat16, 32-bit floats stay, integer tables -> int32
    assert storage_dtype(torch.float16) == torch.bfloat16 and storage_dtype(torch.float32) == torch.float32
    assert storage_dtype(torch.int64) == torch.int32
    weights["model.norm.weight"] = weights["model.norm.weight"].float()
    write_safetensors(os.path.join(folder, "model.safetensors"), weights)
    assert load_weights(folder, specs)["model.norm.weight"].dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = LlamaConfig.from_dict(BASE)
    folder = write_random_model(cfg, str(tmp_path / "m"), seed=0)
    specs = resolve_architecture(cfg.to_dict()).build(cfg).tensor_specs()
    weights = load_weights(folder, specs)
    del weights["model.layers.1.mlp.up_proj.weight"]
    del weights["model.norm.weight"]
    weights["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32, dtype=torch.bfloat16)
    weights["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)       # tied: not expected
    weights["stray.bias"] = torch.zeros(3, dtype=torch.bfloat16)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights)
    with pytest.raises(WeightError) as info:
        load_weights(folder, specs)
    error = info.value
    assert error.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert error.unexpected == ["lm_head.weight", "stray.bias"]
    assert [(n, tuple(e), tuple(f)) for n, e, f in error.wrong_shape] == [
        ("model.layers.0.self_attn.q_proj.weight", (64, 64), (64, 32))]
    text = str(error)
    for piece in ("missing tensors (2)", "unexpected tensors (2)", "wrong shapes (1)", "stray.bias",
                  "expected [64, 64], found [64, 32]"):
        assert piece in text


def test_truncated_file_and_non_finite_values(tmp_path):
    cfg = LlamaConfig.from_dict(BASE)
    folder = write_random_model(cfg, str(tmp_path / "m"), seed=0)
    specs = resolve_architecture(cfg.to_dict()).build(cfg).tensor_specs()
    path = os.path.join(folder, "model.safetensors")
    weights = load_weights(folder, specs)
    weights["model.norm.weight"][3] = float("nan")
    write_safetensors(path, weights)
    with pytest.raises(WeightError, match="non-finite values in model.norm.weight"):
        load_weights(folder, specs)
    blob = open(path, "rb").read()
    open(path, "wb").write(blob[:-10])
    with pytest.raises(SafetensorsError, match="extent|unindexed"):
        load_weights(folder, specs)
    open(path, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        load_weights(folder, specs)
