"""Typed configuration of the Bebuvik design, read from the keys of its config.json.

A small decoder-only model: token embedding plus a hashed bigram embedding; layers
with ONE scalar-gain RMS norm whose output feeds a latent-attention mixer and a dense
feed-forward side by side, each behind a short causal convolution added to its input
and each scaled by a sigmoid gate computed from the normalised stream; some layers
read another layer's cached latent instead of projecting their own; soft-capped logits.

config.json keys (every size and every constant that can differ between models):

    architecture            "Bebuvik"
    vocab, width
    norm.eps
    canon.taps              taps of the input convolutions (absent: no input convolution)
    embedding.bigram        {buckets, mul_prev, mul_cur} (absent: no bigram table)
    logit_softcap           c in c * tanh(logits / c) (absent or null: none)
    layers[i]               {type: "latent_attention",
                             mixer: {heads, dim, rot_dim, vdim, kv_rank, scale, rot: {base, dims},
                                     mask: {size} (absent: every earlier position), kv_from: j (optional)},
                             mlp: {kind: "dense", ff} or null}

Tensor names: `embed`, `bigram`, `l<i>.norm1`, `l<i>.mix.{q,dkv,dkv.norm,uk,uv,sink,o}`,
`l<i>.mlp.{up,down}`, `l<i>.canon1`, `l<i>.canon2`, `l<i>.rg1`, `l<i>.rg1.b`, `l<i>.rg2`,
`l<i>.rg2.b`, `final.norm`, `head`. The design sets no limit on positions.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field

from ..errors import ConfigError
from .spec import (BigramEmbeddingSpec, DenseFeedForwardSpec, EmbeddingSpec, HeadSpec, LatentAttentionSpec, LayerCall,
                   ModelSpec, NormSpec, ParallelLayerSpec, RotarySpec, ShortConvSpec)

ARCHITECTURE = "Bebuvik"

# The design has no position limit; block tables and the like are sized by the engine's own limits.
UNLIMITED_POSITIONS = 1 << 30


def _get(d, key, kind, where, required=True, default=None):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        if required:
            raise ConfigError(f"config.json has no `{where}{key}`")
        return default
    v = d[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int) or v < 0:
            raise ConfigError(f"config.json `{where}{key}` must be a non-negative integer, got {v!r}")
        return v
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
            raise ConfigError(f"config.json `{where}{key}` must be a finite number, got {v!r}")
        return float(v)
    if kind is dict:
        if not isinstance(v, dict):
            raise ConfigError(f"config.json `{where}{key}` must be an object")
        return v
    return v


@dataclass(frozen=True)
class BebuvikMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    window: object = None      # None: every earlier position
    kv_from: object = None     # None: the layer projects its own latent


@dataclass(frozen=True)
class BebuvikLayer:
    mixer: BebuvikMixer
    ff: object = None          # intermediate size of the dense feed-forward, None: the layer has none


@dataclass(frozen=True)
class BebuvikConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple
    taps: object = None                # None: no input convolution
    bigram: object = None              # (buckets, mul_prev, mul_cur) or None
    logit_softcap: object = None
    raw: dict = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, d: dict) -> "BebuvikConfig":
        if not isinstance(d, dict):
            raise ConfigError("config.json must hold a JSON object")
        if d.get("architecture", ARCHITECTURE) != ARCHITECTURE and ARCHITECTURE not in (d.get("architectures") or []):
            raise ConfigError(f"this is not a {ARCHITECTURE} configuration")
        layers_in = d.get("layers")
        if not isinstance(layers_in, list) or not layers_in:
            raise ConfigError("config.json `layers` must be a non-empty list")
        layers = []
        for i, entry in enumerate(layers_in):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json `layers[{i}]` must be an object")
            if entry.get("type") != "latent_attention":
                raise ConfigError(f"config.json `{where}type` is {entry.get('type')!r}; this design's mixer is 'latent_attention'")
            m = _get(entry, "mixer", dict, where)
            mw = where + "mixer."
            rot = _get(m, "rot", dict, mw)
            mask = _get(m, "mask", dict, mw, required=False)
            mixer = BebuvikMixer(
                heads=_get(m, "heads", int, mw), dim=_get(m, "dim", int, mw), rot_dim=_get(m, "rot_dim", int, mw),
                vdim=_get(m, "vdim", int, mw), kv_rank=_get(m, "kv_rank", int, mw), scale=_get(m, "scale", float, mw),
                rot_base=_get(rot, "base", float, mw + "rot."), rot_dims=_get(rot, "dims", int, mw + "rot."),
                window=_get(mask, "size", int, mw + "mask.") if mask is not None else None,
                kv_from=_get(m, "kv_from", int, mw, required=False))
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json `{where}mlp.kind` must be 'dense' (or `mlp` null)")
                ff = _get(mlp, "ff", int, where + "mlp.")
            layers.append(BebuvikLayer(mixer, ff))
        canon = _get(d, "canon", dict, "", required=False)
        emb = _get(d, "embedding", dict, "", required=False)
        big = _get(emb, "bigram", dict, "embedding.", required=False) if emb is not None else None
        cfg = cls(
            vocab=_get(d, "vocab", int, ""), width=_get(d, "width", int, ""),
            norm_eps=_get(_get(d, "norm", dict, ""), "eps", float, "norm."),
            layers=tuple(layers),
            taps=_get(canon, "taps", int, "canon.") if canon is not None else None,
            bigram=(_get(big, "buckets", int, "embedding.bigram."), _get(big, "mul_prev", int, "embedding.bigram."),
                    _get(big, "mul_cur", int, "embedding.bigram.")) if big is not None else None,
            logit_softcap=_get(d, "logit_softcap", float, "", required=False),
            raw=copy.deepcopy(d))
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        if self.raw:
            return copy.deepcopy(self.raw)
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps}, "layers": []}
        if self.taps is not None:
            d["canon"] = {"taps": self.taps}
        if self.bigram is not None:
            d["embedding"] = {"bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), self.bigram))}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        for layer in self.layers:
            m = layer.mixer
            mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale,
                     "rot": {"base": m.rot_base, "dims": m.rot_dims}}
            if m.window is not None:
                mixer["mask"] = {"size": m.window}
            if m.kv_from is not None:
                mixer["kv_from"] = m.kv_from
            d["layers"].append({"type": "latent_attention", "mixer": mixer,
                                "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}})
        return d

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("Bebuvik `vocab` and `width` must be greater than zero")
        if self.norm_eps <= 0.0:
            raise ConfigError("Bebuvik `norm.eps` must be positive")
        if self.taps is not None and not 1 <= self.taps <= 16:
            raise ConfigError(f"Bebuvik `canon.taps` must be between 1 and 16, got {self.taps}")
        if self.bigram is not None and (self.bigram[0] <= 0 or max(self.bigram[1:]) >= 1 << 31):
            raise ConfigError("Bebuvik `embedding.bigram` needs a positive number of buckets and multipliers below 2^31")
        if self.logit_softcap is not None and self.logit_softcap <= 0.0:
            raise ConfigError("Bebuvik `logit_softcap` must be positive")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if min(m.heads, m.dim, m.vdim, m.kv_rank) <= 0:
                raise ConfigError(f"Bebuvik layer {i}: heads, dim, vdim and kv_rank must be greater than zero")
            if m.rot_dims % 2 or m.rot_dims > m.rot_dim:
                raise ConfigError(f"Bebuvik layer {i}: rot.dims ({m.rot_dims}) must be even and within rot_dim ({m.rot_dim})")
            if m.rot_base <= 0.0 or m.scale <= 0.0:
                raise ConfigError(f"Bebuvik layer {i}: rot.base and scale must be positive")
            if m.window is not None and m.window <= 0:
                raise ConfigError(f"Bebuvik layer {i}: mask.size must be positive")
            if layer.ff is not None and layer.ff <= 0:
                raise ConfigError(f"Bebuvik layer {i}: mlp.ff must be greater than zero")
            if m.kv_from is not None:
                if not 0 <= m.kv_from < i:
                    raise ConfigError(f"Bebuvik layer {i}: kv_from ({m.kv_from}) must name an earlier layer")
                src = self.layers[m.kv_from].mixer
                if src.kv_from is not None:
                    raise ConfigError(f"Bebuvik layer {i}: kv_from names layer {m.kv_from}, which has no latent projection of its own")
                if (src.kv_rank, src.rot_dim, src.rot_base, src.rot_dims) != (m.kv_rank, m.rot_dim, m.rot_base, m.rot_dims):
                    raise ConfigError(f"Bebuvik layer {i}: its latent size and rotation differ from those of layer {m.kv_from}, whose cache it reads")

    # ---- the model as data --------------------------------------------------

    def to_model_spec(self) -> ModelSpec:
        layers, order, entry_of = [], [], {}
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}.", layer.mixer
            mixer = LatentAttentionSpec(
                hidden_size=self.width, num_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim,
                kv_rank=m.kv_rank, position=RotarySpec(m.rot_dims, m.rot_base, "interleaved") if m.rot_dims else None,
                norm_eps=self.norm_eps, scale=m.scale, window=m.window, sink=True, shares_latent=m.kv_from is not None,
                prefix=p + "mix.")
            ffn = DenseFeedForwardSpec(self.width, layer.ff, "gelu_tanh", p + "mlp.") if layer.ff is not None else None
            names = (p + "canon1",) + ((p + "canon2",) if ffn is not None else ())
            gates = (p + "rg1",) + ((p + "rg2",) if ffn is not None else ())
            layers.append(ParallelLayerSpec(
                norm=NormSpec(self.width, self.norm_eps, p + "norm1", "rmsnorm_scalar"), mixer=mixer, ffn=ffn,
                conv=ShortConvSpec(self.width, self.taps, names) if self.taps is not None else None, gate_names=gates))
            if m.kv_from is None:
                entry_of[i] = len(entry_of)
                order.append(LayerCall(i, entry_of[i], True))
            else:
                order.append(LayerCall(i, entry_of[m.kv_from], False))
        if self.bigram is not None:
            embedding = BigramEmbeddingSpec(self.vocab, self.width, *self.bigram, table_name="embed", bigram_name="bigram")
        else:
            embedding = EmbeddingSpec(self.vocab, self.width, "", weight_name="embed")
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, max_positions=UNLIMITED_POSITIONS,
            embedding=embedding, layers=tuple(layers), order=tuple(order),
            final_norm=NormSpec(self.width, self.norm_eps, "final.norm", "rmsnorm_scalar"),
            head=HeadSpec(self.vocab, self.width, False, "", softcap=self.logit_softcap, weight_name="head"),
            eos_token_id=None)
        spec.validate()
        return spec
