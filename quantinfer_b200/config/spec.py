"""Descriptions of a model as data: parts with their sizes and constants, the
layers they form, and the order in which layers run.

An architecture's config class turns its config.json into a :class:`ModelSpec`.
Nothing below the spec knows which architecture it came from: parts are built
from their spec alone (`parts.registry.build_*`). The reference keeps the same
split between a config and an architecture-neutral description
(crates/quantinfer-model/src/semantic.rs:39-57,91-103: per-layer attention,
normalisation, activation and positional specs).

Each spec carries `kind`, the key under which the part's class is registered,
and `prefix`, prepended to the part's local tensor names to give the names in
the weight files.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class NormSpec:
    """`kind` "rmsnorm": gain per coordinate, tensor `prefix + "weight"`. "rmsnorm_scalar": one gain for all
    coordinates, the tensor named `prefix` itself, of shape []."""

    size: int
    eps: float
    prefix: str = ""
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class PositionSpec:
    """Rotary encoding over the first `rotary_dim` dimensions of each head, angle of pair p =
    position * theta^(-2p / rotary_dim). `pairing` says which two elements pair p is:
    "half_split" (p, p + rotary_dim / 2) or "interleaved" (2p, 2p + 1)."""

    head_dim: int
    rotary_dim: int
    theta: float
    max_positions: int
    kind: str = "rope_half_split"
    pairing: str = "half_split"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a paged key/value cache."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    position: Optional[PositionSpec]
    qk_norm: bool = False
    qk_norm_eps: float = 1e-6
    window: Optional[int] = None      # None: all earlier keys; n: the last n keys
    scale: Optional[float] = None     # None: head_dim ** -0.5
    prefix: str = ""
    kind: str = "attention"


@dataclass(frozen=True)
class FeedForwardSpec:
    """Gated feed-forward: down(act(gate(x)) * up(x))."""

    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    prefix: str = ""
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class RotarySpec:
    """Rotary encoding whose angles are computed where they are used (no table, so no limit on
    positions): pair i of the first `rotary_dim` coordinates of a part turns by position *
    theta^(-2i / rotary_dim). `pairing` as for :class:`PositionSpec`."""

    rotary_dim: int
    theta: float
    pairing: str = "interleaved"
    kind: str = "rope_direct"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention over a cached low-rank latent: a position caches `kv_rank` numbers (normalised,
    gain per coordinate) and a rotated key part of `rot_dim` numbers that all heads share; per head the
    key's plain part (`head_dim` numbers) and the value (`value_dim`) are projections of the latent.
    `shares_latent`: the layer has no latent projection and reads the cache entry of another layer.
    `sink`: the softmax's denominator holds one more learned term per head."""

    hidden_size: int
    num_heads: int
    head_dim: int
    rot_dim: int
    value_dim: int
    kv_rank: int
    position: Optional[RotarySpec]
    norm_eps: float
    scale: float
    window: Optional[int] = None
    sink: bool = False
    shares_latent: bool = False
    prefix: str = ""
    kind: str = "latent_attention"


@dataclass(frozen=True)
class DenseFeedForwardSpec:
    """Feed-forward without a gate: down(act(up(x)))."""

    hidden_size: int
    intermediate_size: int
    activation: str = "gelu_tanh"
    prefix: str = ""
    kind: str = "dense_mlp"


@dataclass(frozen=True)
class ShortConvSpec:
    """A bank of short causal convolutions over time that read one input: filter k has `taps` weights per
    channel, stored as the tensor `names[k]` of shape [width, taps]; out_k = (input if `residual`) +
    filter_k(input). The last taps - 1 inputs are a request's state."""

    width: int
    taps: int
    names: tuple
    residual: bool = True
    kind: str = "short_conv"


@dataclass(frozen=True)
class ParallelLayerSpec:
    """One block with one norm whose output feeds the mixer and the feed-forward side by side:
    h = norm(x); x += gate_m * mixer(conv_m(h)) + gate_f * ffn(conv_f(h)). `conv` (optional) is the bank
    of input convolutions, one filter per sublayer; `gate_names` (optional) are the prefixes of the sigmoid
    gates' projections of h, one per sublayer ("<name>" the matrix, "<name>.b" the bias). `ffn` may be None."""

    norm: NormSpec
    mixer: object
    ffn: object
    conv: Optional[ShortConvSpec] = None
    gate_names: Optional[tuple] = None
    kind: str = "parallel_gated"

    # what the model reads of any layer spec
    @property
    def mixer_norm(self):
        return self.norm


@dataclass(frozen=True)
class BigramEmbeddingSpec:
    """Token embedding plus a row of a hashed bigram table [buckets + 1, hidden]: row (previous * mul_prev +
    current * mul_cur) mod buckets, the last row for a sequence's first token."""

    vocab_size: int
    hidden_size: int
    buckets: int
    mul_prev: int
    mul_cur: int
    table_name: str = "embed"
    bigram_name: str = "bigram"
    prefix: str = ""
    kind: str = "bigram_embedding"


@dataclass(frozen=True)
class LayerSpec:
    """One block: x += mixer(norm(x)); x += ffn(norm(x)) for kind `prenorm`."""

    mixer_norm: NormSpec
    mixer: object          # a mixer spec (AttentionSpec or any registered kind)
    ffn_norm: NormSpec
    ffn: object            # a feed-forward spec
    kind: str = "prenorm"


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run `layer` with cache entry `cache`.

    Naming a layer twice reuses its weights. `writes_cache=False` makes the
    call read a cache entry that an earlier call filled, without adding to it.
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class EmbeddingSpec:
    vocab_size: int
    hidden_size: int
    prefix: str = ""
    kind: str = "embedding"
    weight_name: Optional[str] = None   # the tensor's full name when it is not prefix + "weight"


@dataclass(frozen=True)
class HeadSpec:
    vocab_size: int
    hidden_size: int
    tied: bool              # True: the head is the embedding table
    prefix: str = ""
    kind: str = "lm_head"
    softcap: Optional[float] = None     # c: logits = c * tanh(logits / c)
    weight_name: Optional[str] = None   # the tensor's full name when it is not prefix + "weight"


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: EmbeddingSpec
    layers: tuple
    order: tuple
    final_norm: NormSpec
    head: HeadSpec
    eos_token_id: Optional[int] = None
    extra: dict = field(default_factory=dict, compare=False)

    def cache_entries(self) -> int:
        return 1 + max(call.cache for call in self.order) if self.order else 0

    def validate(self) -> None:
        from ..errors import ConfigError

        if not self.layers or not self.order:
            raise ConfigError("a model needs at least one layer and one entry in its run order")
        written = set()
        for i, call in enumerate(self.order):
            if not 0 <= call.layer < len(self.layers):
                raise ConfigError(f"run order entry {i} names layer {call.layer}, the model has {len(self.layers)}")
            if call.cache < 0:
                raise ConfigError(f"run order entry {i} has a negative cache entry")
            if call.writes_cache:
                if call.cache in written:
                    raise ConfigError(f"run order entry {i}: cache entry {call.cache} already has a writer")
                written.add(call.cache)
            elif call.cache not in written:
                raise ConfigError(f"run order entry {i} reads cache entry {call.cache} before any layer wrote it")
        if written != set(range(self.cache_entries())):
            raise ConfigError("cache entries must be numbered 0..n-1 and each needs a writer")
