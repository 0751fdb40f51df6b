"""Configuration and registry (no GPU): every size comes from config.json; what the engine
cannot honour is refused with the key's name (model/config.go:132-312, model/model.go:95-192)."""
import copy

import pytest

import tiny
from tgo_b200.config.qwen3 import ConfigError, Qwen3Config, qwen3_model_spec
from tgo_b200.registry import ARCHITECTURES, Registry, model_spec_from_config


def test_tiny_configs_differ_in_every_size_and_option():
    a, b = Qwen3Config.from_dict(tiny.TINY_A), Qwen3Config.from_dict(tiny.TINY_B)
    for f in ("hidden_size", "num_hidden_layers", "num_attention_heads", "head_dim",
              "intermediate_size", "vocab_size", "rms_norm_eps", "rope_theta",
              "tie_word_embeddings", "max_position_embeddings", "kv_group", "q_width"):
        assert getattr(a, f) != getattr(b, f), f
    assert a.layer_windows == (None, None) and b.layer_windows == (None, 24, None)
    assert b.q_width != b.hidden_size          # head_dim from the file, not hidden/heads
    assert tiny.TINY_A_RUN["page_size"] != tiny.TINY_B_RUN["page_size"]


def test_spec_carries_the_files_numbers():
    spec = qwen3_model_spec(tiny.TINY_B)
    assert spec.architecture == "Qwen3ForCausalLM" and spec.hidden_size == 96
    assert len(spec.layers) == 3 and [c.layer for c in spec.run_order] == [0, 1, 2]
    m = spec.layers[1].mixer
    assert (m.num_heads, m.num_kv_heads, m.head_dim, m.window, m.qk_norm) == (6, 2, 32, 24, True)
    assert m.position.theta == 1e6 and m.position.rotary_dim == 32 and m.norm_eps == 1e-5
    assert spec.layers[0].mixer.window is None
    assert spec.layers[2].feed_forward.intermediate_size == 224
    assert spec.head_name == "lm_head.weight" and spec.tied_head_alias is None
    tied = qwen3_model_spec(tiny.TINY_A)
    assert tied.head_name is None and tied.tied_head_alias == "lm_head.weight"


def test_defaults_head_dim_and_kv_heads():
    raw = copy.deepcopy(tiny.TINY_A)
    del raw["head_dim"], raw["num_key_value_heads"]
    c = Qwen3Config.from_dict(raw)
    assert c.head_dim == 16 and c.num_key_value_heads == 4


@pytest.mark.parametrize("edit,needle", [
    (lambda r: r.pop("hidden_size"), "hidden_size is required"),
    (lambda r: r.update(num_hidden_layers=0), "num_hidden_layers is 0"),
    (lambda r: r.update(vocab_size=-3), "vocab_size"),
    (lambda r: r.pop("rms_norm_eps"), "rms_norm_eps is required"),
    (lambda r: r.update(rope_theta=1e60), "rope_theta"),
    (lambda r: r.update(rms_norm_eps=1e-60), "rms_norm_eps"),
    (lambda r: r.update(head_dim=15), "head_dim is 15"),
    (lambda r: r.update(num_key_value_heads=3), "num_key_value_heads"),
    (lambda r: r.update(rope_scaling={"rope_type": "yarn", "factor": 4}), "rope_scaling is set (yarn)"),
    (lambda r: r.update(attention_bias=True), "attention_bias"),
    (lambda r: r.update(hidden_act="gelu"), "hidden_act"),
    (lambda r: r.update(sliding_window=64, use_sliding_window=None) or r.pop("use_sliding_window"),
     "sliding_window is 64"),
    (lambda r: r.update(use_sliding_window=True, sliding_window=None), "use_sliding_window"),
    (lambda r: r.update(layer_types=["full_attention"]), "layer_types"),
    (lambda r: r.update(layer_types=["full_attention", "sliding_attention"], sliding_window=None),
     "sliding_window is not set"),
    (lambda r: r.update(layer_types=["full_attention", "linear_attention"]), "known kinds"),
    (lambda r: r.update(max_position_embeddings=None), "max_position_embeddings is required"),
    (lambda r: r.update(architectures=[]), "architectures[0]"),
])
def test_refusals_name_the_key(edit, needle):
    raw = copy.deepcopy(tiny.TINY_A)
    edit(raw)
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(raw)
    assert needle in str(e.value)


def test_head_dim_default_must_divide():
    raw = copy.deepcopy(tiny.TINY_A)
    del raw["head_dim"]
    raw["num_attention_heads"] = 6
    raw["num_key_value_heads"] = 2
    with pytest.raises(ConfigError, match="head_dim is absent"):
        Qwen3Config.from_dict(raw)


def test_use_sliding_window_with_max_window_layers():
    raw = copy.deepcopy(tiny.TINY_B)
    del raw["layer_types"]
    raw.update(use_sliding_window=True, max_window_layers=2, sliding_window=10)
    assert Qwen3Config.from_dict(raw).layer_windows == (None, None, 10)


def test_null_rope_scaling_and_qwen_window_keys_pass():
    raw = dict(tiny.TINY_A, rope_scaling=None, sliding_window=None, use_sliding_window=False)
    assert Qwen3Config.from_dict(raw).layer_windows == (None, None)


def test_registry_unknown_lists_known_and_duplicates_raise():
    with pytest.raises(KeyError) as e:
        model_spec_from_config({"architectures": ["NoSuchModel"]})
    assert "Qwen3ForCausalLM" in str(e.value) and "NoSuchModel" in str(e.value)
    r = Registry("thing")
    r.register("a", object)
    with pytest.raises(ValueError, match="twice"):
        r.register("a", object)
    with pytest.raises(ValueError, match="needs a name"):
        r.register("", object)
    with pytest.raises(ValueError, match="no constructor"):
        r.register("b", None)
    assert "Qwen3ForCausalLM" in ARCHITECTURES.names()


def test_run_order_is_validated():
    from tgo_b200.config.spec import LayerCall
    spec = qwen3_model_spec(tiny.TINY_A)
    spec.run_order = [LayerCall(0), LayerCall(5)]
    with pytest.raises(ValueError, match="names layer 5"):
        spec.validate()
    spec.run_order = [LayerCall(0, cache_from=0)]
    with pytest.raises(ValueError, match="does not run before"):
        spec.validate()
    spec.run_order = [LayerCall(0), LayerCall(1, cache_from=0), LayerCall(0, cache_from=1)]
    with pytest.raises(ValueError, match="owns none"):
        spec.validate()
    spec.run_order = [LayerCall(0), LayerCall(1), LayerCall(0, cache_from=0)]
    spec.validate()


def test_build_folder_is_one_for_all_threads():
    """Several libraries compile side by side: every thread must get the same folder (a
    probe file shared by name once sent some of them to the fallback folder)."""
    from concurrent.futures import ThreadPoolExecutor

    from tgo_b200.kernels import build as kb
    kb._build_dir_found = None
    with ThreadPoolExecutor(max_workers=8) as pool:
        got = set(pool.map(lambda _: kb._build_dir(), range(64)))
    assert len(got) == 1
    # and the host library, which needs no CUDA compiler, builds and loads
    lib = kb.load_library("host_runtime")
    assert lib.tgo_cache_create
