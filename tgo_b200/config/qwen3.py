"""Typed reading of a Qwen3 dense config.json, and its translation to a ModelSpec.

Every size and constant of the model comes from the file; a key the engine
cannot honour is refused with the key's name in the message, never approximated
(model/config.go:132-215 for the rules, :224-271 for the refusals).

Beyond the reference: `attention_bias` and `hidden_act` are read and refused when
they ask for what the layers do not compute (the reference never reads them and
fails later, at the weight check); and a per-layer `layer_types` list with
"sliding_attention" entries is accepted, because the engine's attention and
cache handle a window. `use_sliding_window: true` without that list is turned into
one with `max_window_layers`; a bare `sliding_window` with no switch beside it is
refused as in the reference, since it does not say which layers it means.
"""
from __future__ import annotations

import json
import math
import struct
from dataclasses import dataclass
from typing import Optional

from .spec import (FeedForwardSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec, NormSpec,
                   PositionSpec)

ARCHITECTURE = "Qwen3ForCausalLM"


class ConfigError(ValueError):
    """A config.json the engine refuses. The message names the key."""


def _f32(x: float) -> float:
    return struct.unpack("<f", struct.pack("<f", x))[0]


def _positive_int(raw: dict, key: str, required: bool = True) -> Optional[int]:
    v = raw.get(key)
    if v is None:
        if required:
            raise ConfigError(f"config: {key} is required")
        return None
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config: {key} is {v!r}; it must be an integer")
    if v <= 0:
        raise ConfigError(f"config: {key} is {v}; it must be positive")
    return v


def _positive_float(raw: dict, key: str) -> float:
    v = raw.get(key)
    if v is None:
        raise ConfigError(f"config: {key} is required")
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config: {key} is {v!r}; it must be a number")
    if not v > 0:
        raise ConfigError(f"config: {key} is {v}; it must be positive")
    try:
        f = _f32(float(v))
    except OverflowError:
        f = math.inf
    if math.isinf(f):
        raise ConfigError(f"config: {key} is {v}, which is not finite as a 32-bit float")
    if f == 0.0:
        raise ConfigError(f"config: {key} is {v}, which rounds to zero as a 32-bit float")
    return float(v)


@dataclass(frozen=True)
class Qwen3Config:
    """config.json of a Qwen3 dense model, checked (model/config.go:20-87)."""
    architecture: str
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    layer_windows: tuple             # per layer: None or the window length

    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def kv_group(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @staticmethod
    def from_dict(raw: dict) -> "Qwen3Config":
        archs = raw.get("architectures")
        if not archs or not isinstance(archs, list) or not archs[0]:
            raise ConfigError("config: architectures[0] is required; it is the registry key")
        d = _positive_int(raw, "hidden_size")
        L = _positive_int(raw, "num_hidden_layers")
        H = _positive_int(raw, "num_attention_heads")
        f = _positive_int(raw, "intermediate_size")
        V = _positive_int(raw, "vocab_size")
        maxpos = _positive_int(raw, "max_position_embeddings")
        eps = _positive_float(raw, "rms_norm_eps")
        if raw.get("rope_theta") is None and isinstance(raw.get("rope_parameters"), dict):
            rp = raw["rope_parameters"]
            if rp.get("rope_type", "default") != "default":
                raise ConfigError(f"config: rope_parameters.rope_type is {rp.get('rope_type')!r} "
                                  "and no scaling is supported")
            theta = _positive_float(rp, "rope_theta")
        else:
            theta = _positive_float(raw, "rope_theta")

        if raw.get("head_dim") is not None:
            dh = raw["head_dim"]
            if isinstance(dh, bool) or not isinstance(dh, int) or dh <= 0:
                raise ConfigError(f"config: head_dim is {dh!r}; it must be a positive integer")
        elif d % H != 0:
            raise ConfigError("config: head_dim is absent and its default "
                              f"hidden_size/num_attention_heads is not an integer ({d}/{H})")
        else:
            dh = d // H
        if dh % 2 != 0:
            raise ConfigError(f"config: head_dim is {dh}; the rotation pairs channels and "
                              "refuses an odd width")

        Hkv = _positive_int(raw, "num_key_value_heads", required=False) or H
        if H % Hkv != 0:
            raise ConfigError(f"config: num_attention_heads ({H}) is not a multiple of "
                              f"num_key_value_heads ({Hkv})")

        scaling = raw.get("rope_scaling")
        if scaling is not None:
            name = "unnamed"
            if isinstance(scaling, dict):
                name = scaling.get("rope_type") or scaling.get("type") or "unnamed"
            raise ConfigError(f"config: rope_scaling is set ({name}) and no scaling is supported")

        if raw.get("attention_bias"):
            raise ConfigError("config: attention_bias is true; the projections here have no bias")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config: hidden_act is {act!r}; the feed-forward here is SiLU-gated")

        windows = _layer_windows(raw, L)
        tie = raw.get("tie_word_embeddings", False)
        if not isinstance(tie, bool):
            raise ConfigError(f"config: tie_word_embeddings is {tie!r}; it must be true or false")
        return Qwen3Config(archs[0], d, L, H, Hkv, dh, f, V, eps, theta, tie, maxpos, windows)

    @staticmethod
    def from_json(text: str) -> "Qwen3Config":
        try:
            raw = json.loads(text)
        except json.JSONDecodeError as e:
            raise ConfigError(f"config: not JSON: {e}") from None
        if not isinstance(raw, dict):
            raise ConfigError("config: the top level must be an object")
        return Qwen3Config.from_dict(raw)


def _layer_windows(raw: dict, L: int) -> tuple:
    window = raw.get("sliding_window")
    use = raw.get("use_sliding_window")
    kinds = raw.get("layer_types")
    if window is not None and (isinstance(window, bool) or not isinstance(window, int)
                               or window <= 0):
        raise ConfigError(f"config: sliding_window is {window!r}; it must be a positive integer "
                          "or null")
    if kinds is not None:
        if not isinstance(kinds, list) or len(kinds) != L:
            raise ConfigError(f"config: layer_types must list num_hidden_layers ({L}) entries")
        out = []
        for i, kd in enumerate(kinds):
            if kd == "full_attention":
                out.append(None)
            elif kd == "sliding_attention":
                if window is None:
                    raise ConfigError(f"config: layer_types[{i}] is sliding_attention and "
                                      "sliding_window is not set")
                out.append(window)
            else:
                raise ConfigError(f"config: layer_types[{i}] is {kd!r}; known kinds are "
                                  "full_attention, sliding_attention")
        if use is False and any(w is not None for w in out):
            raise ConfigError("config: use_sliding_window is false and layer_types has "
                              "sliding_attention layers")
        return tuple(out)
    if use:
        if window is None:
            raise ConfigError("config: use_sliding_window is true and sliding_window is not set")
        first = raw.get("max_window_layers")
        if isinstance(first, bool) or not isinstance(first, int) or first < 0:
            raise ConfigError("config: use_sliding_window is true and max_window_layers does not "
                              "say which layers have the window")
        return tuple(window if i >= first else None for i in range(L))
    if window is not None and use is None:
        raise ConfigError(f"config: sliding_window is {window} with neither use_sliding_window "
                          "nor layer_types beside it; it does not say which layers it means")
    return tuple([None] * L)


# The checkpoint's tensor names below a layer's prefix, by the role each part asks for
# (model/qwen3.go:57-67 is the reference's table for this architecture).
ATTENTION_TENSORS = (("q", "self_attn.q_proj.weight"), ("k", "self_attn.k_proj.weight"),
                     ("v", "self_attn.v_proj.weight"), ("o", "self_attn.o_proj.weight"),
                     ("q_norm", "self_attn.q_norm.weight"), ("k_norm", "self_attn.k_norm.weight"))
FEED_FORWARD_TENSORS = (("gate", "mlp.gate_proj.weight"), ("up", "mlp.up_proj.weight"),
                        ("down", "mlp.down_proj.weight"))
BLOCK_TENSORS = (("mixer_norm", "input_layernorm.weight"),
                 ("ffn_norm", "post_attention_layernorm.weight"))


def qwen3_model_spec(raw: dict) -> ModelSpec:
    """config.json (as a dict) -> ModelSpec. The weight names are the checkpoint's own
    (model/qwen3.go:18-26, :76-148): per layer input_layernorm, self_attn.{q,k,v,o}_proj,
    self_attn.{q,k}_norm, post_attention_layernorm, mlp.{gate,up,down}_proj."""
    c = Qwen3Config.from_dict(raw)
    attention_tensors, ffn_tensors, block_tensors = \
        ATTENTION_TENSORS, FEED_FORWARD_TENSORS, BLOCK_TENSORS
    norm = NormSpec("rmsnorm", c.rms_norm_eps)
    pos = PositionSpec("rope_half_split", rotary_dim=c.head_dim, theta=c.rope_theta)
    layers = []
    for i in range(c.num_hidden_layers):
        mixer = MixerSpec("gqa_attention", num_heads=c.num_attention_heads,
                          num_kv_heads=c.num_key_value_heads, head_dim=c.head_dim,
                          qk_norm=True, window=c.layer_windows[i], position=pos,
                          norm_eps=c.rms_norm_eps, tensors=attention_tensors)
        ffn = FeedForwardSpec("swiglu", intermediate_size=c.intermediate_size,
                              tensors=ffn_tensors)
        layers.append(LayerSpec("prenorm_residual", f"model.layers.{i}.", mixer, ffn, norm,
                                block_tensors))
    spec = ModelSpec(
        architecture=c.architecture, hidden_size=c.hidden_size, vocab_size=c.vocab_size,
        layers=layers, run_order=[LayerCall(i) for i in range(c.num_hidden_layers)],
        final_norm=norm, embedding_name="model.embed_tokens.weight",
        final_norm_name="model.norm.weight",
        head_name=None if c.tie_word_embeddings else "lm_head.weight",
        tied_head_alias="lm_head.weight" if c.tie_word_embeddings else None,
        max_positions=c.max_position_embeddings, source=dict(raw))
    spec.validate()
    return spec
