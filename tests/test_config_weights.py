"""Configuration, registry and checkpoint checks (no GPU)."""
import json
import os
import struct

import pytest
import torch

import harness as H  # noqa: F401
from tiny_configs import TINY_A, TINY_B, TINY_C, TINY_D

from lastengine_b200.config import ConfigError, Lfm3Config
from lastengine_b200.registry import ARCHITECTURES, RegistryError, plan_from_config
from lastengine_b200.weights import WeightsError, check_names, write_model_dir
from lastengine_b200.weights.safetensors_io import SafetensorsFile, open_checkpoint, save_file


def test_tiny_configs_parse_and_differ():
    a, b, c = (Lfm3Config.from_dict(x) for x in (TINY_A, TINY_B, TINY_C))
    assert (a.ffn_dim, b.ffn_dim) == (128, 160)           # 240 -> int(2*240/3)=160 -> multiple of 32
    assert a.head_dim == 16 and b.head_dim == 32 and c.rope_dim == 32
    assert b.layer_is_moe(1) and not b.layer_is_moe(0) and not a.layer_is_moe(3)
    assert c.layer_types[0] == "sliding_attention" and c.sliding_window == 24
    for f in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
              "head_dim", "ffn_dim", "rope_theta", "conv_L_cache", "norm_eps", "tie_embedding"):
        assert getattr(a, f) != getattr(b, f), f


def test_baseline_ffn_width_rule():
    cfg = dict(TINY_A, intermediate_size=8192, block_auto_adjust_ff_dim=True, block_multiple_of=256)
    assert Lfm3Config.from_dict(cfg).ffn_dim == 5632


def test_defaults_follow_the_reference():
    cfg = {k: v for k, v in TINY_A.items() if k not in ("norm_eps", "rope_theta", "head_dim", "tie_embedding")}
    c = Lfm3Config.from_dict(cfg)
    assert c.norm_eps == 1e-5 and c.rope_theta == 10000.0 and c.head_dim == 16 and c.tie_embedding


@pytest.mark.parametrize("change,needle", [
    ({"hidden_size": None}, "hidden_size"),
    ({"layer_types": ["conv"]}, "layer_types"),
    ({"layer_types": ["conv", "mamba", "conv", "attention"]}, "mamba"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"conv_L_cache": None}, "conv_L_cache"),
    ({"conv_L_cache": 1}, "conv_L_cache"),
    ({"rope_dim": 18}, "rope_dim"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"num_experts": 4}, "num_experts_per_tok"),
    ({"layer_types": ["conv", "sliding_attention", "conv", "attention"]}, "sliding_window"),
])
def test_config_errors_name_the_key(change, needle):
    cfg = {k: v for k, v in {**TINY_A, **change}.items() if v is not None}
    with pytest.raises(ConfigError) as e:
        Lfm3Config.from_dict(cfg)
    assert needle in str(e.value)


def test_registry_chooses_by_config_and_lists_known_names():
    plan = plan_from_config(TINY_B)
    assert [l.mixer.kind for l in plan.layers] == ["shortconv", "shortconv", "attention", "shortconv", "shortconv", "attention"]
    assert [l.ffn.kind for l in plan.layers] == ["swiglu"] + ["sigmoid_topk_moe"] * 5
    assert plan_from_config(dict(TINY_A, architectures=["Lfm2ForCausalLM"])).vocab_size == 256
    with pytest.raises(RegistryError) as e:
        plan_from_config(dict(TINY_A, architectures=["GptNeoXForCausalLM"]))
    assert "GptNeoXForCausalLM" in str(e.value) and "Lfm3ForCausalLM" in str(e.value)
    assert "lfm3" in ARCHITECTURES


def test_plan_schedule_is_checked():
    from lastengine_b200.parts.base import ScheduleEntry
    import dataclasses
    plan = plan_from_config(TINY_A)
    with pytest.raises(ValueError):
        dataclasses.replace(plan, schedule=[ScheduleEntry(9)])
    with pytest.raises(ValueError):
        dataclasses.replace(plan, schedule=[ScheduleEntry(1, cache=1, writes_cache=False)])


def specs_of(cfg):
    from lastengine_b200.engine.model import Model
    from lastengine_b200.parts.base import BuildEnv
    return Model(plan_from_config(cfg), BuildEnv(torch.device("cpu"), torch.bfloat16)).tensor_specs()


def test_model_folder_roundtrip(tmp_path):
    d = write_model_dir(TINY_B, str(tmp_path / "m"), seed=5)
    assert json.load(open(os.path.join(d, "config.json")))["hidden_size"] == 96
    ck = open_checkpoint(d)
    specs = specs_of(TINY_B)
    assert len(ck) == len([s for s in specs.values() if not s.optional]) == 172
    f, n = ck["model.layers.1.feed_forward.expert_bias"]
    assert f.dtype(n) == torch.float32                                  # biases are stored in 32-bit
    assert ck["model.embed_tokens.weight"][0].dtype("model.embed_tokens.weight") == torch.bfloat16
    assert "lm_head.weight" in ck and "model.lm_head.weight" not in ck
    w = ck["model.layers.0.conv.conv.weight"][0].tensor("model.layers.0.conv.conv.weight")
    assert tuple(w.shape) == (96, 1, 4)
    d2 = write_model_dir(TINY_B, str(tmp_path / "m2"), seed=5)
    a = open_checkpoint(d2)["lm_head.weight"][0].tensor("lm_head.weight")
    assert torch.equal(a, ck["lm_head.weight"][0].tensor("lm_head.weight"))   # same seed, same values
    d3 = write_model_dir(TINY_B, str(tmp_path / "m3"), seed=6)
    assert not torch.equal(a, open_checkpoint(d3)["lm_head.weight"][0].tensor("lm_head.weight"))
    norm = ck["model.embedding_norm.weight"][0].tensor("model.embedding_norm.weight")
    assert torch.all(norm == 1)                                          # norm weights are 1 by default


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    specs = specs_of(TINY_A)
    found = {n: s.shape for n, s in specs.items()}
    del found["layers.1.self_attn.q_proj.weight"], found["embedding_norm.weight"]
    found["layers.0.conv.extra.weight"] = (3,)
    found["layers.2.conv.conv.weight"] = (64, 3)
    with pytest.raises(WeightsError) as e:
        check_names(specs, found, "dir")
    msg = str(e.value)
    for needle in ("missing tensors (2)", "layers.1.self_attn.q_proj.weight", "embedding_norm.weight",
                   "unexpected tensors (1)", "layers.0.conv.extra.weight", "wrong shapes (1)",
                   "layers.2.conv.conv.weight: expected [64, 1, 3], found [64, 3]"):
        assert needle in msg, needle
    check_names(specs, {n: s.shape for n, s in specs.items()}, "dir")


def test_optional_tensors_frequency_factors_and_conv_bias(tmp_path):
    """The model's rotary frequency factors are one optional tensor that every attention layer
    without a window names; a checkpoint fits with it and without it.  `conv_bias` adds a bias
    tensor per convolution, which a checkpoint must then have."""
    specs = specs_of(TINY_D)
    ff = specs["rope_freqs.weight"]
    assert ff.optional and ff.shape == (8,) and specs["layers.0.conv.conv.bias"].shape == (72,)
    found = {n: s.shape for n, s in specs.items()}
    check_names(specs, found, "dir")
    del found["rope_freqs.weight"]
    check_names(specs, found, "dir")
    del found["layers.3.conv.conv.bias"]
    with pytest.raises(WeightsError, match=r"missing tensors \(1\): layers.3.conv.conv.bias"):
        check_names(specs, found, "dir")
    assert "rope_freqs.weight" in specs_of(TINY_A) and "layers.0.conv.conv.bias" not in specs_of(TINY_A)
    # only layers without a window take the factors (src/dense.rs:125)
    plan = plan_from_config(TINY_D)
    assert [l.mixer.params["position"].params["freq_factors"] for l in plan.layers if l.mixer.kind == "attention"] == [True, False]
    # a model whose attention layers all have a window names no such tensor; its plan says that a
    # checkpoint may carry it all the same (the loader then skips it instead of calling it unexpected)
    only_windows = dict(TINY_D, layer_types=["conv", "sliding_attention", "sliding_attention", "conv"])
    assert "rope_freqs.weight" not in specs_of(only_windows)
    assert "rope_freqs.weight" in plan_from_config(only_windows).unused_tensors
    # a written folder leaves the optional tensor out; the test helper adds it
    d = H.make_model_dir(TINY_D, 3, str(tmp_path / "d"), freq_factors=True)
    ck = open_checkpoint(d)
    assert "model.rope_freqs.weight" in ck and len(ck) == len(specs)
    b = ck["model.layers.0.conv.conv.bias"][0].tensor("model.layers.0.conv.conv.bias")
    assert b.dtype == torch.float32 and float(b.abs().max()) > 0


def test_tied_model_rejects_an_output_matrix():
    specs = specs_of(TINY_A)
    found = {n: s.shape for n, s in specs.items()}
    found["lm_head.weight"] = (256, 64)
    with pytest.raises(WeightsError, match="unexpected tensors.*lm_head.weight"):
        check_names(specs, found, "dir")


def test_broken_files_are_reported(tmp_path):
    p = str(tmp_path / "model.safetensors")
    with pytest.raises(WeightsError, match="no model.safetensors"):
        open_checkpoint(str(tmp_path))
    open(p, "wb").write(b"\x01\x02")
    with pytest.raises(WeightsError, match="truncated"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(WeightsError, match="truncated"):
        SafetensorsFile(p)
    save_file({"x": torch.arange(6, dtype=torch.float32).view(2, 3), "i": torch.arange(4, dtype=torch.int64)}, p)
    sf = SafetensorsFile(p)
    assert torch.equal(sf.tensor("x"), torch.arange(6, dtype=torch.float32).view(2, 3))
    data = open(p, "rb").read()
    open(p, "wb").write(data[:-8])
    with pytest.raises(WeightsError, match="truncated"):
        SafetensorsFile(p)


def test_kept_dtypes():
    from lastengine_b200.parts.base import BIAS, MATRIX, NORM, VECTOR, TensorSpec
    from lastengine_b200.weights.loader import kept_dtype
    bf, f32 = torch.bfloat16, torch.float32
    assert kept_dtype(TensorSpec((1,), MATRIX), bf, bf) == bf
    assert kept_dtype(TensorSpec((1,), MATRIX), bf, f32) == f32
    assert kept_dtype(TensorSpec((1,), NORM), bf, bf) == f32
    assert kept_dtype(TensorSpec((1,), VECTOR), f32, bf) == f32
    assert kept_dtype(TensorSpec((1,), BIAS), f32, bf) == f32
    assert kept_dtype(TensorSpec((1,), MATRIX), torch.int64, bf) == torch.int32


def test_engine_options():
    from lastengine_b200 import EngineOptions
    o = EngineOptions.of(None, dtype=torch.float32, max_tokens=100)
    assert o.dtype == "float32" and o.max_tokens == 100 and o.max_batch_tokens == 16384 and o.use_graphs
    assert EngineOptions.of(o, max_seqs=3).max_tokens == 100
    with pytest.raises(TypeError, match="max_token"):
        EngineOptions.of(None, max_token=5)
    with pytest.raises(ValueError):
        EngineOptions(dtype="float16")
    with pytest.raises(ValueError):
        EngineOptions(max_tokens=0)


def test_engine_refuses_to_run_without_cuda():
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from lastengine_b200 import Engine
    with pytest.raises(RuntimeError, match="CUDA device only"):
        Engine(plan_from_config(TINY_A), dtype="float32")
