"""Typed configuration of the Kiruvik design, read from the keys of its config.json.

A small decoder-only model normalised by dynamic tanh instead of statistics: every layer has a norm before and
after each of its two sublayers and a multiplier on what joins the 32-bit stream. A layer's mixer is either
grouped-query attention (biased projections, rotation over part of each head, chunked visibility, an output gate)
or a Mamba-2 state-space mixer; its feed-forward is a gated dense one (tanh-form gelu), a routed mixture of small
clamped experts with a shared expert, or absent. A stretch of layers may run several times in a row with the same
weights, each pass with cache entries of its own and begun by mixing the embedding's output back into the stream.

config.json keys (every size, and every constant that can differ between models):

    architecture            "Kiruvik"
    vocab, width, residual_mult
    norm.eps                eps of the RMS norms inside mixers (the dynamic-tanh norms use none)
    loop                    {start, stop, times}: layers start .. stop - 1 run `times` times (absent: once)
    layers[i]               {type: "attention" | "mamba2", mixer: {...}, mlp: {...} or null}
      attention mixer       {heads, kv_heads, dim, vdim, scale, rot: {base, dims}, mask: {size}}
      mamba2 mixer          {heads, vdim, state, groups, conv, norm_groups}
      mlp dense             {kind: "dense", ff}
      mlp moe               {kind: "moe", router: {experts, top, scale}, expert: {ff, limit}, shared: {ff, limit}}

Tensor names: `embed`, `loop.in`, `l<i>.norm1|norm1b|norm2|norm2b` (each with `.b`, `.alpha`),
`l<i>.mix.{q,k,v,o}` (each with `.b`) and `l<i>.mix.g`, or `l<i>.mix.{in,conv,conv.b,dt_bias,A_log,D,norm,o}`,
`l<i>.mlp.{gate,up,down}` or `l<i>.mlp.{router,correction,e<k>.gate|up|down,shared.gate|up|down}`, `final.norm`
(`.b`, `.alpha`), `head`. The design sets no limit on positions.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field

from ..errors import ConfigError
from .bebuvik import UNLIMITED_POSITIONS, _get
from .spec import (ClampedGLUSpec, EmbeddingSpec, FeedForwardSpec, GatedAttentionSpec, HeadSpec, LayerCall, ModelSpec, MoESpec,
                   NormSpec, ReentrySpec, RotarySpec, SandwichLayerSpec, StateSpaceSpec)

ARCHITECTURE = "Kiruvik"

# constants the design fixes
EXPERT_SIGMOID_SLOPE = 1.702        # g * sigmoid(1.702 g) in an expert
DENSE_ACTIVATION = "gelu_tanh"


@dataclass(frozen=True)
class KiruvikAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float = 10000.0
    rot_dims: int = 0
    chunk: object = None           # mask.size; None: every earlier position


@dataclass(frozen=True)
class KiruvikMamba:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class KiruvikDense:
    ff: int


@dataclass(frozen=True)
class KiruvikMoE:
    experts: int
    top: int
    scale: float
    ff: int
    limit: float
    shared_ff: object = None       # None: no shared expert
    shared_limit: object = None


@dataclass(frozen=True)
class KiruvikLayer:
    mixer: object                  # KiruvikAttention or KiruvikMamba
    mlp: object = None             # KiruvikDense, KiruvikMoE or None


@dataclass(frozen=True)
class KiruvikConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: tuple
    loop: object = None            # (start, stop, times) or None
    raw: dict = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, d: dict) -> "KiruvikConfig":
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
            m = _get(entry, "mixer", dict, where)
            mw = where + "mixer."
            kind = entry.get("type")
            if kind == "attention":
                rot = _get(m, "rot", dict, mw, required=False)
                mask = _get(m, "mask", dict, mw, required=False)
                mixer = KiruvikAttention(
                    heads=_get(m, "heads", int, mw), kv_heads=_get(m, "kv_heads", int, mw), dim=_get(m, "dim", int, mw),
                    vdim=_get(m, "vdim", int, mw), scale=_get(m, "scale", float, mw),
                    rot_base=_get(rot, "base", float, mw + "rot.") if rot is not None else 10000.0,
                    rot_dims=_get(rot, "dims", int, mw + "rot.") if rot is not None else 0,
                    chunk=_get(mask, "size", int, mw + "mask.") if mask is not None else None)
            elif kind == "mamba2":
                mixer = KiruvikMamba(
                    heads=_get(m, "heads", int, mw), vdim=_get(m, "vdim", int, mw), state=_get(m, "state", int, mw),
                    groups=_get(m, "groups", int, mw), conv=_get(m, "conv", int, mw), norm_groups=_get(m, "norm_groups", int, mw))
            else:
                raise ConfigError(f"config.json `{where}type` is {kind!r}; this design's mixers are 'attention' and 'mamba2'")
            mlp_in, mlp = entry.get("mlp"), None
            if mlp_in is not None:
                lw = where + "mlp."
                if not isinstance(mlp_in, dict):
                    raise ConfigError(f"config.json `{where}mlp` must be an object or null")
                if mlp_in.get("kind") == "dense":
                    mlp = KiruvikDense(_get(mlp_in, "ff", int, lw))
                elif mlp_in.get("kind") == "moe":
                    r, e = _get(mlp_in, "router", dict, lw), _get(mlp_in, "expert", dict, lw)
                    sh = _get(mlp_in, "shared", dict, lw, required=False)
                    mlp = KiruvikMoE(
                        experts=_get(r, "experts", int, lw + "router."), top=_get(r, "top", int, lw + "router."),
                        scale=_get(r, "scale", float, lw + "router."), ff=_get(e, "ff", int, lw + "expert."),
                        limit=_get(e, "limit", float, lw + "expert."),
                        shared_ff=_get(sh, "ff", int, lw + "shared.") if sh is not None else None,
                        shared_limit=_get(sh, "limit", float, lw + "shared.") if sh is not None else None)
                else:
                    raise ConfigError(f"config.json `{lw}kind` must be 'dense' or 'moe' (or `mlp` null)")
            layers.append(KiruvikLayer(mixer, mlp))
        loop_in = _get(d, "loop", dict, "", required=False)
        loop = None
        if loop_in is not None:
            loop = (_get(loop_in, "start", int, "loop."), _get(loop_in, "stop", int, "loop."), _get(loop_in, "times", int, "loop."))
        cfg = cls(vocab=_get(d, "vocab", int, ""), width=_get(d, "width", int, ""),
                  norm_eps=_get(_get(d, "norm", dict, ""), "eps", float, "norm."),
                  residual_mult=_get(d, "residual_mult", float, "", required=False, default=1.0),
                  layers=tuple(layers), loop=loop, raw=copy.deepcopy(d))
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        if self.raw:
            return copy.deepcopy(self.raw)
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "residual_mult": self.residual_mult, "layers": []}
        if self.loop is not None:
            d["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        for layer in self.layers:
            m = layer.mixer
            if isinstance(m, KiruvikAttention):
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
                if m.rot_dims:
                    mixer["rot"] = {"base": m.rot_base, "dims": m.rot_dims}
                if m.chunk is not None:
                    mixer["mask"] = {"size": m.chunk}
                kind = "attention"
            else:
                mixer = {"heads": m.heads, "vdim": m.vdim, "state": m.state, "groups": m.groups, "conv": m.conv,
                         "norm_groups": m.norm_groups}
                kind = "mamba2"
            f = layer.mlp
            if f is None:
                mlp = None
            elif isinstance(f, KiruvikDense):
                mlp = {"kind": "dense", "ff": f.ff}
            else:
                mlp = {"kind": "moe", "router": {"experts": f.experts, "top": f.top, "scale": f.scale},
                       "expert": {"ff": f.ff, "limit": f.limit}}
                if f.shared_ff is not None:
                    mlp["shared"] = {"ff": f.shared_ff, "limit": f.shared_limit}
            d["layers"].append({"type": kind, "mixer": mixer, "mlp": mlp})
        return d

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("Kiruvik `vocab` and `width` must be greater than zero")
        if self.norm_eps <= 0.0:
            raise ConfigError("Kiruvik `norm.eps` must be positive")
        n = len(self.layers)
        if self.loop is not None:
            a, b, times = self.loop
            if not 0 <= a < b <= n or times < 1:
                raise ConfigError(f"Kiruvik `loop` {self.loop} must name a stretch of the {n} layers and run it at least once")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if isinstance(m, KiruvikAttention):
                if min(m.heads, m.kv_heads, m.dim, m.vdim) <= 0 or m.heads % m.kv_heads:
                    raise ConfigError(f"Kiruvik layer {i}: heads must be a positive multiple of kv_heads, dim and vdim positive")
                if m.rot_dims % 2 or m.rot_dims > m.dim:
                    raise ConfigError(f"Kiruvik layer {i}: rot.dims ({m.rot_dims}) must be even and within dim ({m.dim})")
                if (m.rot_dims and m.rot_base <= 0.0) or m.scale <= 0.0:
                    raise ConfigError(f"Kiruvik layer {i}: rot.base and scale must be positive")
                if m.chunk is not None and m.chunk <= 0:
                    raise ConfigError(f"Kiruvik layer {i}: mask.size must be positive")
            else:
                if min(m.heads, m.vdim, m.state, m.groups, m.conv, m.norm_groups) <= 0:
                    raise ConfigError(f"Kiruvik layer {i}: every size of a mamba2 mixer must be greater than zero")
                if m.heads % m.groups or (m.heads * m.vdim) % m.norm_groups:
                    raise ConfigError(f"Kiruvik layer {i}: heads must be a multiple of groups, and heads * vdim of norm_groups")
            f = layer.mlp
            if isinstance(f, KiruvikDense) and f.ff <= 0:
                raise ConfigError(f"Kiruvik layer {i}: mlp.ff must be greater than zero")
            if isinstance(f, KiruvikMoE):
                if not 0 < f.top <= f.experts or f.ff <= 0 or f.limit <= 0.0:
                    raise ConfigError(f"Kiruvik layer {i}: a mixture needs 0 < top <= experts, ff > 0 and limit > 0")
                if f.shared_ff is not None and (f.shared_ff <= 0 or f.shared_limit is None or f.shared_limit <= 0.0):
                    raise ConfigError(f"Kiruvik layer {i}: the shared expert needs ff > 0 and limit > 0")

    # ---- the model as data --------------------------------------------------

    def run_order(self) -> list:
        """(layer, first of a pass) in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        a, b, times = self.loop
        order = [(i, False) for i in range(a)]
        for _ in range(times):
            order += [(i, i == a) for i in range(a, b)]
        return order + [(i, False) for i in range(b, n)]

    def to_model_spec(self) -> ModelSpec:
        w = self.width

        def norm(name):
            return NormSpec(w, self.norm_eps, name, "dyt")

        layers = []
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}.", layer.mixer
            if isinstance(m, KiruvikAttention):
                mixer = GatedAttentionSpec(
                    hidden_size=w, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim,
                    position=RotarySpec(m.rot_dims, m.rot_base, "half_split") if m.rot_dims else None, scale=m.scale,
                    chunk=m.chunk, window=None, bias=True, out_gate=True, prefix=p + "mix.")
            else:
                mixer = StateSpaceSpec(hidden_size=w, heads=m.heads, head_dim=m.vdim, state=m.state, groups=m.groups,
                                       conv_taps=m.conv, norm_groups=m.norm_groups, norm_eps=self.norm_eps, prefix=p + "mix.")
            f, ffn = layer.mlp, None
            if isinstance(f, KiruvikDense):
                ffn = FeedForwardSpec(w, f.ff, DENSE_ACTIVATION, p + "mlp.", names=("gate", "up", "down"))
            elif isinstance(f, KiruvikMoE):
                shared = (ClampedGLUSpec(w, f.shared_ff, f.shared_limit, EXPERT_SIGMOID_SLOPE, p + "mlp.shared.")
                          if f.shared_ff is not None else None)
                ffn = MoESpec(hidden_size=w, experts=f.experts, top=f.top, router_scale=f.scale,
                              expert=ClampedGLUSpec(w, f.ff, f.limit, EXPERT_SIGMOID_SLOPE, p + "mlp."), shared=shared,
                              prefix=p + "mlp.")
            layers.append(SandwichLayerSpec(
                mixer_norm=norm(p + "norm1"), mixer_post_norm=norm(p + "norm1b"), mixer=mixer,
                ffn_norm=norm(p + "norm2") if ffn is not None else None,
                ffn_post_norm=norm(p + "norm2b") if ffn is not None else None, ffn=ffn, residual_mult=self.residual_mult))
        order = tuple(LayerCall(layer, entry, True, reenter) for entry, (layer, reenter) in enumerate(self.run_order()))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=w, max_positions=UNLIMITED_POSITIONS,
            embedding=EmbeddingSpec(self.vocab, w, "", weight_name="embed"), layers=tuple(layers), order=order,
            final_norm=norm("final.norm"), head=HeadSpec(self.vocab, w, False, "", weight_name="head"), eos_token_id=None,
            reentry=ReentrySpec(w, "loop.in") if self.loop is not None else None)
        spec.validate()
        return spec
