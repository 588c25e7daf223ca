"""Configuration and registry (no GPU)."""
import json

import pytest

from conftest import TINY_A, TINY_B
from nanoinfer_b200.config import ConfigError, GPT2Config
from nanoinfer_b200.registry import UnknownArchitecture, get_architecture, load_config


def test_reads_every_key():
    a, b = GPT2Config.from_dict(TINY_A), GPT2Config.from_dict(TINY_B)
    assert (a.vocab_size, a.n_positions, a.n_embd, a.n_layer, a.n_head) == (512, 128, 64, 2, 4)
    assert (a.head_dim, a.inner_dim, a.gelu_kind, a.tie_word_embeddings) == (16, 256, "tanh", True)
    assert (b.head_dim, b.inner_dim, b.gelu_kind, b.tie_word_embeddings) == (24, 200, "erf", False)
    assert b.layer_norm_epsilon == 1e-6 and b.scale_attn_by_inverse_layer_idx


def test_n_inner_null_means_four_times_width():
    raw = dict(TINY_A, n_inner=None)
    assert GPT2Config.from_dict(raw).inner_dim == 4 * 64


def test_param_count_matches_reference_formula():
    # crates/core/src/config.rs:29-39 gives 124,439,808 for GPT-2 small
    raw = dict(architectures=["GPT2LMHeadModel"], vocab_size=50257, n_positions=1024, n_embd=768, n_layer=12,
               n_head=12, layer_norm_epsilon=1e-5, activation_function="gelu_new")
    assert GPT2Config.from_dict(raw).n_params() == 124_439_808


@pytest.mark.parametrize("patch, word", [
    ({"n_head": 5}, "divisible"), ({"vocab_size": 0}, "positive"), ({"activation_function": "relu"}, "activation"),
    ({"layer_norm_epsilon": 0.0}, "epsilon"), ({"n_embd": "64"}, "expected int"), ({"n_layer": None}, "missing"),
])
def test_bad_values_are_refused(patch, word):
    with pytest.raises(ConfigError) as e:
        GPT2Config.from_dict(dict(TINY_A, **patch))
    assert word in str(e.value)


def test_all_problems_in_one_error():
    raw = {k: v for k, v in TINY_A.items() if k not in ("n_embd", "n_head")}
    with pytest.raises(ConfigError) as e:
        GPT2Config.from_dict(raw)
    assert "n_embd" in str(e.value) and "n_head" in str(e.value)


def test_registry_by_architecture_name(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    cfg = load_config(str(tmp_path))
    assert isinstance(cfg, GPT2Config) and cfg.n_embd == 120
    assert get_architecture("GPT2LMHeadModel").config_cls is GPT2Config
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY_B, architectures=["NoSuchModel"])))
    with pytest.raises(UnknownArchitecture):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))


def test_spec_is_built_from_the_configuration_only():
    cfg = GPT2Config.from_dict(TINY_B)
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    m0, m2 = spec.layers[0].mixer.args, spec.layers[2].mixer.args
    assert m0["head_dim"] == 24 and m0["n_head"] == 5
    assert abs(m0["scale"] - 24 ** -0.5) < 1e-12 and abs(m2["scale"] - 24 ** -0.5 / 3) < 1e-12
    assert spec.layers[1].feed_forward.args == dict(width=120, inner=200, activation="erf", bias=True)
    assert spec.head.tensors["weight"].name == "lm_head.weight"
    assert spec.layers[0].mixer.tensors["qkv_weight"].transposed
