"""Architecture-neutral description of a model: what the engine builds from.

An architecture's config reader (for instance `config/qwen3.py`) turns its own
config.json keys into these records. Everything below the reader (parts, cache,
step function, kernels) sees only these records, never a model's name, so another
architecture is another reader plus, where needed, new part kinds.

The reference keeps the same split between a typed `Config` and the blocks that
take their constants as parameters (model/config.go:20-87, nn/attention.go:60-94,
model/layerkind.go:21-59).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, Optional


def tensor_names(tensors, prefix: str, roles: Iterable[str], what: str) -> Dict[str, str]:
    """The checkpoint names a part asks for: `tensors` is the (role, name) table its spec
    carries (names relative to the layer's prefix), `roles` the roles the part needs. A role
    the table does not name is an error of the architecture's config reader, which owns the
    table (model/qwen3.go:57-67 keeps it per architecture in the same way)."""
    table = dict(tensors)
    out = {}
    for role in roles:
        if role not in table:
            raise ValueError(f"{what}: the spec names no tensor for the role {role!r}; "
                             f"it names {sorted(table) or 'none'}")
        out[role] = prefix + table[role]
    return out


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last axis. kind names a registered norm part."""
    kind: str
    eps: float


@dataclass(frozen=True)
class PositionSpec:
    """How positions enter a mixer. kind names a registered position encoding.
    `rotary_dim` channels of each head are rotated; the rest are left alone."""
    kind: str
    rotary_dim: int = 0
    theta: float = 0.0


@dataclass(frozen=True)
class MixerSpec:
    """The token-mixing part of a layer. kind names a registered mixer.

    For attention kinds: `window` is None when a query reads every earlier key,
    else the number of most recent keys (its own included) that it reads.
    `tensors` is the (role, checkpoint name relative to the layer's prefix) table of the
    mixer's weights; the roles are the mixer kind's own (attention: q, k, v or qkv joined, o,
    q_norm, k_norm). `extra` carries what a mixer kind outside this package needs.
    """
    kind: str
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    qk_norm: bool = False
    window: Optional[int] = None
    scale: Optional[float] = None        # None: 1/sqrt(head_dim)
    position: Optional[PositionSpec] = None
    norm_eps: float = 0.0                # eps of the per-head q/k norm
    tensors: tuple = ()
    extra: tuple = ()


@dataclass(frozen=True)
class FeedForwardSpec:
    """The per-token part of a layer. kind names a registered feed-forward. `tensors` as in
    MixerSpec (gated feed-forward: gate, up or gate_up joined, down)."""
    kind: str
    intermediate_size: int = 0
    tensors: tuple = ()
    extra: tuple = ()


@dataclass(frozen=True)
class LayerSpec:
    """One layer: which block arrangement, and the parts inside it.
    `prefix` is the tensor-name prefix of the layer's weights ("model.layers.3."); every
    part of the layer gets it and adds the names of its own spec's `tensors` table.
    `tensors` names the block's own weights (pre-norm block: mixer_norm, ffn_norm)."""
    block: str
    prefix: str
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    norm: NormSpec
    tensors: tuple = ()


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    `layer` indexes ModelSpec.layers (a layer may be named by several calls, which
    then share weights). `cache_from` is None when the call owns a cache of its
    own, else the index of an earlier call whose cache it reads without writing.
    """
    layer: int
    cache_from: Optional[int] = None


@dataclass
class ModelSpec:
    """A whole decoder: embedding, layers, their run order, final norm and head."""
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: list                     # list[LayerSpec]
    run_order: list                  # list[LayerCall]
    final_norm: NormSpec
    embedding_name: str
    final_norm_name: str
    head_name: Optional[str]         # None: the head is the embedding table (tied)
    tied_head_alias: Optional[str] = None   # name a tied checkpoint may ship anyway
    max_positions: int = 0           # advisory, as in the reference
    source: dict = field(default_factory=dict)   # the config.json it came from

    @property
    def tied_head(self) -> bool:
        return self.head_name is None

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("model spec: no layers")
        for i, call in enumerate(self.run_order):
            if not (0 <= call.layer < len(self.layers)):
                raise ValueError(f"model spec: run_order[{i}] names layer {call.layer}, "
                                 f"there are {len(self.layers)}")
            if call.cache_from is not None:
                if not (0 <= call.cache_from < i):
                    raise ValueError(f"model spec: run_order[{i}] reads the cache of call "
                                     f"{call.cache_from}, which does not run before it")
                if self.run_order[call.cache_from].cache_from is not None:
                    raise ValueError(f"model spec: run_order[{i}] reads the cache of call "
                                     f"{call.cache_from}, which owns none")
