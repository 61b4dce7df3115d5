"""Configuration, registry, weight loading errors and the random-weights mode (no device)."""

from __future__ import annotations

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

import helpers as H
from lockstep_b200.config import (ConfigError, Qwen3Config, config_from_dict, known_architectures,
                                  load_config, register_architecture, unregister_architecture)
from lockstep_b200.engine.model import expected_weights
from lockstep_b200.weights import WeightError, load_weights, write_random_model


def read_tensors(folder):
    """Copies, so that the file can be rewritten while the tensors are in use."""
    return {k: v.clone() for k, v in load_file(str(folder / "model.safetensors")).items()}


def test_registry_maps_architecture_name_to_config():
    assert "Qwen3ForCausalLM" in known_architectures()
    cfg = config_from_dict(H.TINY_B)
    assert isinstance(cfg, Qwen3Config)
    assert (cfg.hidden_size, cfg.num_key_value_heads, cfg.head_dim, cfg.vocab_size) == (80, 1, 32, 500)
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 1e6 and cfg.tie_word_embeddings is False
    by_type = config_from_dict({k: v for k, v in H.TINY_A.items() if k != "architectures"})
    assert isinstance(by_type, Qwen3Config)
    with pytest.raises(ConfigError, match="unknown architecture"):
        config_from_dict({**H.TINY_A, "architectures": ["NopeForCausalLM"]})


def test_config_errors_are_clear():
    with pytest.raises(ConfigError, match="lacks the keys.*rope_theta"):
        config_from_dict({k: v for k, v in H.TINY_A.items() if k != "rope_theta"})
    with pytest.raises(ConfigError, match="multiple of"):
        config_from_dict({**H.TINY_A, "num_key_value_heads": 3})
    with pytest.raises(ConfigError, match="attention_bias"):
        config_from_dict({**H.TINY_A, "attention_bias": True})
    with pytest.raises(ConfigError, match="rope_scaling"):
        config_from_dict({**H.TINY_A, "rope_scaling": {"type": "yarn", "factor": 2}})
    with pytest.raises(ConfigError, match="hidden_act"):
        config_from_dict({**H.TINY_A, "hidden_act": "gelu"})
    with pytest.raises(ConfigError, match="sliding_window"):
        config_from_dict({**H.TINY_A, "use_sliding_window": True})


def test_head_dim_defaults_to_width_over_heads():
    raw = {k: v for k, v in H.TINY_A.items() if k != "head_dim"}
    assert config_from_dict(raw).head_dim == 16


def test_spec_is_data_layer_by_layer():
    spec = config_from_dict(H.TINY_C).model_spec()
    assert [l.mixer["window"] for l in spec.layers] == [0, 40, 40]
    assert [r.layer for r in spec.schedule] == [0, 1, 2] and spec.cache_entries == 3
    assert spec.layers[0].mixer_norm["eps"] == 3e-6
    assert spec.layers[2].mixer["num_kv_heads"] == 3 and spec.layers[2].mixer["head_dim"] == 48


def test_expected_weights_names_and_shapes():
    w = expected_weights(config_from_dict(H.TINY_B).model_spec())
    assert w["model.layers.2.self_attn.q_proj.weight"].shape == (128, 80)
    assert w["model.layers.0.self_attn.o_proj.weight"].shape == (80, 128)
    assert w["model.layers.1.self_attn.k_norm.weight"].shape == (32,)
    assert w["model.layers.1.mlp.down_proj.weight"].shape == (80, 200)
    assert w["lm_head.weight"].shape == (500, 80)
    tied = expected_weights(config_from_dict(H.TINY_A).model_spec())
    assert "lm_head.weight" not in tied and "model.embed_tokens.weight" in tied


def test_random_weights_mode_is_seeded(tmp_path):
    a = write_random_model(tmp_path / "a", H.TINY_A, seed=3, dtype="bfloat16")
    b = write_random_model(tmp_path / "b", H.TINY_A, seed=3, dtype="bfloat16")
    c = write_random_model(tmp_path / "c", H.TINY_A, seed=4, dtype="float32")
    wa, wb, wc = (load_file(str(p / "model.safetensors")) for p in (a, b, c))
    assert set(wa) == set(expected_weights(config_from_dict(H.TINY_A).model_spec()))
    assert all(torch.equal(wa[k], wb[k]) for k in wa)
    assert wa["model.norm.weight"].dtype == torch.bfloat16 and wc["model.norm.weight"].dtype == torch.float32
    assert not torch.equal(wa["model.norm.weight"].float(), wc["model.norm.weight"])
    assert isinstance(load_config(a), Qwen3Config)
    assert json.loads((a / "config.json").read_text())["architectures"] == ["Qwen3ForCausalLM"]


def test_loader_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_random_model(tmp_path / "m", H.TINY_B, seed=1, dtype="float32")
    spec = config_from_dict(H.TINY_B).model_spec()
    expected = expected_weights(spec)
    tensors = read_tensors(folder)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(4)
    tensors["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(16, 80)
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightError) as e:
        load_weights(folder, expected, torch.float32, "cpu")
    msg = str(e.value)
    assert "missing (2): model.layers.1.mlp.up_proj.weight, model.norm.weight" in msg
    assert "unexpected (1): model.layers.0.self_attn.rotary.inv_freq" in msg
    assert "model.layers.2.self_attn.k_proj.weight: file has [16, 80], model needs [32, 80]" in msg


def test_loader_keeps_dtypes_as_stored(tmp_path):
    folder = write_random_model(tmp_path / "m", H.TINY_A, seed=1, dtype="bfloat16")
    tensors = read_tensors(folder)
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float() + 1e-4   # stored in 32-bit
    save_file(tensors, str(folder / "model.safetensors"))
    expected = expected_weights(config_from_dict(H.TINY_A).model_spec())
    got = load_weights(folder, expected, torch.bfloat16, "cpu")
    assert got["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert got["model.norm.weight"].dtype == torch.float32       # a tensor stored in 32-bit stays so
    assert got["model.layers.0.input_layernorm.weight"].dtype == torch.bfloat16
    wide = load_weights(folder, expected, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in wide.values())
    assert torch.equal(wide["model.embed_tokens.weight"], tensors["model.embed_tokens.weight"].float())


def test_cast_report_measures_what_the_rounding_cost(tmp_path):
    """A float32 folder read by the bfloat16 engine: the report counts the elements that changed
    and the largest errors; read by the float32 engine, or stored in bfloat16, nothing changes."""
    from lockstep_b200.engine.model import Model
    from lockstep_b200.parts import Runtime

    folder = write_random_model(tmp_path / "m", H.TINY_A, seed=3, dtype="float32")
    spec = config_from_dict(H.TINY_A).model_spec()
    model = Model(spec, Runtime(torch.device("cpu"), torch.float32, 16, 8, torch.zeros(2, dtype=torch.int32)))
    tensors = read_tensors(folder)
    tensors["model.layers.0.mlp.down_proj.weight"][0, 0] = 1.0 + 2.0 ** -9      # needs 9 bits: rounds to 1.0
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()      # the tied head stored as well
    save_file(tensors, str(folder / "model.safetensors"))
    expected = model.weight_specs()
    report: dict = {}
    got = load_weights(folder, expected, torch.bfloat16, "cpu", aliases=model.aliases(), report=report)
    total = sum(t.numel() for n, t in tensors.items() if n != "lm_head.weight")
    assert report["distinct_elements"] == total and report["stored_elements_by_dtype"] == {"torch.float32": total}
    gains = sum(t.numel() for n, t in tensors.items() if n.endswith("norm.weight"))
    assert report["kept_elements_by_dtype"] == {"torch.bfloat16": total - gains, "torch.float32": gains}
    assert report["tied_names_dropped"] == ["lm_head.weight"]
    assert report["duplicate_elements_dropped"] == tensors["lm_head.weight"].numel()
    changed = sum(int((t != t.bfloat16().float()).sum()) for n, t in tensors.items()
                  if n != "lm_head.weight" and not n.endswith("norm.weight"))
    assert report["elements_not_exactly_representable"] == changed > 0
    assert 2.0 ** -9 <= report["max_abs_error"] < 2.0 ** -6 and 2.0 ** -10 < report["max_rel_error"] <= 2.0 ** -8
    assert got["model.layers.0.mlp.down_proj.weight"][0, 0] == 1.0
    exact: dict = {}
    load_weights(folder, expected, torch.float32, "cpu", aliases=model.aliases(), report=exact)
    assert exact["elements_not_exactly_representable"] == 0 and exact["max_abs_error"] == 0.0


def test_tied_head_stored_twice_must_agree(tmp_path):
    from lockstep_b200.engine.model import Model
    from lockstep_b200.parts import Runtime

    folder = write_random_model(tmp_path / "m", H.TINY_A, seed=1, dtype="float32")
    spec = config_from_dict(H.TINY_A).model_spec()
    rt = Runtime(torch.device("cpu"), torch.float32, 16, 8, torch.zeros(2, dtype=torch.int32))
    model = Model(spec, rt)
    tensors = read_tensors(folder)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    save_file(tensors, str(folder / "model.safetensors"))
    load_weights(folder, model.weight_specs(), torch.float32, "cpu", aliases=model.aliases())
    tensors["lm_head.weight"][0, 0] += 1
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightError, match="ties lm_head.weight"):
        load_weights(folder, model.weight_specs(), torch.float32, "cpu", aliases=model.aliases())


def test_sharded_folder(tmp_path):
    folder = write_random_model(tmp_path / "m", H.TINY_A, seed=1, dtype="float32")
    tensors = read_tensors(folder)
    names = sorted(tensors)
    half = len(names) // 2
    save_file({k: tensors[k] for k in names[:half]}, str(folder / "model-00001-of-00002.safetensors"))
    save_file({k: tensors[k] for k in names[half:]}, str(folder / "model-00002-of-00002.safetensors"))
    (folder / "model.safetensors").unlink()
    weight_map = {k: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                  for i, k in enumerate(names)}
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    got = load_weights(folder, expected_weights(config_from_dict(H.TINY_A).model_spec()), torch.float32, "cpu")
    assert all(torch.equal(got[k], tensors[k]) for k in names)


def test_another_architecture_can_be_registered():
    @register_architecture("ToyForCausalLM", model_type="toy")
    class ToyConfig:
        @classmethod
        def from_dict(cls, raw):
            return cls()

    try:
        assert isinstance(config_from_dict({"architectures": ["ToyForCausalLM"]}), ToyConfig)
        assert isinstance(config_from_dict({"model_type": "toy"}), ToyConfig)
    finally:
        unregister_architecture("ToyForCausalLM")
    assert "ToyForCausalLM" not in known_architectures()


def test_no_device_means_a_loud_error(tmp_path):
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from lockstep_b200.engine import ModelRunner
    from lockstep_b200.kernels import KernelError

    folder = write_random_model(tmp_path / "m", H.TINY_A, seed=1, dtype="float32")
    with pytest.raises(KernelError, match="no CPU fallback"):
        ModelRunner(folder, dtype="float32")
