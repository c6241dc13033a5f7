"""Shared by the Kiruvik tests: small configurations that differ from one another in every size and option, weights
drawn so that activations are of order one (attention far from uniform, tanh norms neither linear nor saturated,
decays slow enough for a state to last, routers with clear winners), model folders, and the plain implementation's logits."""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def attn(heads, kv_heads, dim, vdim, rot_dims, chunk=None, base=10000.0, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    return {"type": "attention", "mixer": m}


def ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, scale, ff, limit, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale}, "expert": {"ff": ff, "limit": limit}}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


CONFIGS = {
    # no size a power of two or a multiple of eight; values smaller than keys; three kv heads; a chunk that is no
    # multiple of the page; a layer without chunks and without feed-forward; two groups and three norm parts in the
    # recurrent layer; a loop that starts after the first layer
    "P": {"architecture": "Kiruvik", "vocab": 131, "width": 40, "norm": {"eps": 3e-6}, "residual_mult": 0.7,
          "loop": {"start": 1, "stop": 3, "times": 3},
          "layers": [layer(attn(3, 3, 10, 6, 4, chunk=9, base=300.0), dense(56)),
                     layer(ssm(4, 6, 5, 2, 4, 3), moe(5, 3, 1.7, 12, 0.8, shared=(20, 1.3))),
                     layer(attn(6, 2, 6, 14, 6, chunk=21), moe(3, 3, 0.9, 10, 2.0)),
                     layer(attn(2, 1, 12, 12, 0), None)]},
    # sizes that are multiples of 16; one kv head; the whole head rotated; one expert a token and no shared expert;
    # two taps; no loop
    "Q": {"architecture": "Kiruvik", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 1.0,
          "layers": [layer(ssm(2, 32, 64, 1, 2, 1), dense(96)),
                     layer(attn(4, 1, 32, 16, 32, chunk=16, base=250000.0), moe(8, 1, 2.0, 32, 1.0)),
                     layer(attn(4, 4, 16, 32, 8, chunk=48), dense(128))]},
    # one tap (a convolution without state); a state of more rows than a warp; every layer looped twice;
    # a chunk of one page; two rotated coordinates
    "R": {"architecture": "Kiruvik", "vocab": 97, "width": 48, "norm": {"eps": 1e-6}, "residual_mult": 0.8,
          "loop": {"start": 0, "stop": 2, "times": 2},
          "layers": [layer(ssm(3, 8, 33, 3, 1, 2), moe(6, 2, 1.3, 16, 1.5, shared=(8, 0.5))),
                     layer(attn(2, 2, 8, 8, 2, chunk=8, base=50.0), dense(40))]},
}
PAGE_SIZES = {"P": 8, "Q": 16, "R": 8}
SEEDS = {"P": 21, "Q": 22, "R": 23}


def draw_weights(cfg: dict, seed: int, dtype=torch.bfloat16) -> dict:
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def mat(out, inp, gain=1.0):
        return (torch.randn(out, inp, generator=g) * gain / math.sqrt(inp)).to(dtype)

    def vec(n, std, mean=0.0):
        return (mean + std * torch.randn(n, generator=g)).to(dtype)

    def norm(name):
        return {name: vec(W, 0.2, 1.0), name + ".b": vec(W, 0.1), name + ".alpha": (0.4 + 0.8 * torch.rand((), generator=g)).to(dtype)}

    w = {"embed": torch.randn(cfg["vocab"], W, generator=g).to(dtype), "head": mat(cfg["vocab"], W, 2.0)}
    w.update(norm("final.norm"))
    if cfg.get("loop"):
        w["loop.in"] = mat(W, 2 * W, 1.4)
    for i, entry in enumerate(cfg["layers"]):
        p, m = f"l{i}.", entry["mixer"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if entry["mlp"] is not None else ()):
            w.update(norm(p + n))
        if entry["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"] = mat(H * d, W, 2.5), mat(G * d, W, 2.5), mat(G * dv, W)
            w[p + "mix.g"], w[p + "mix.o"] = mat(H * dv, W, 1.5), mat(W, H * dv)
            for n, size in (("q", H * d), ("k", G * d), ("v", G * dv), ("o", W)):
                w[p + f"mix.{n}.b"] = vec(size, 0.3)
        else:
            nh, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, ch = nh * P, nh * P + 2 * G * N
            w[p + "mix.in"] = mat(inner + ch + nh, W, 1.5)
            w[p + "mix.conv"] = (0.6 * torch.randn(ch, m["conv"], generator=g)).to(dtype)
            w[p + "mix.conv.b"] = vec(ch, 0.2)
            w[p + "mix.dt_bias"] = vec(nh, 0.5, -0.5)
            w[p + "mix.A_log"] = (torch.rand(nh, generator=g) * 2.0 - 3.0).to(dtype)     # decays of 0.8 to 0.98 a step
            w[p + "mix.D"] = vec(nh, 0.3, 1.0)
            w[p + "mix.norm"] = vec(inner, 0.2, 1.0)
            w[p + "mix.o"] = mat(W, inner)
        f = entry["mlp"]
        if f is None:
            continue
        if f["kind"] == "dense":
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(f["ff"], W, 1.5), mat(f["ff"], W), mat(W, f["ff"])
        else:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            w[p + "mlp.router"] = mat(E, W, 3.0)
            w[p + "mlp.correction"] = vec(E, 0.1)
            for e in range(E):
                w[p + f"mlp.e{e}.gate"], w[p + f"mlp.e{e}.up"] = mat(ff, W, 1.5), mat(ff, W, 1.5)
                w[p + f"mlp.e{e}.down"] = mat(W, ff)
            if f.get("shared"):
                sf = f["shared"]["ff"]
                w[p + "mlp.shared.gate"], w[p + "mlp.shared.up"] = mat(sf, W, 1.5), mat(sf, W, 1.5)
                w[p + "mlp.shared.down"] = mat(W, sf)
    return w


def write_folder(path, cfg: dict, weights: dict) -> Path:
    from quantinfer_b200.weights import write_safetensors

    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg, indent=1))
    write_safetensors(path / "model.safetensors", {k: v.contiguous() for k, v in weights.items()})
    return path


def make(path, name: str):
    """(folder, config, weights) of the named configuration."""
    cfg = CONFIGS[name]
    w = draw_weights(cfg, SEEDS[name])
    return write_folder(path, cfg, w), cfg, w


def plain_rows(cfg: dict, weights: dict, requests: dict) -> dict:
    """{(request, position): logits row} from the plain implementation."""
    from plain import plain_kiruvik

    rows = {}
    for rid, toks in requests.items():
        logits = plain_kiruvik.forward(cfg, weights, toks).to(torch.float32).numpy()
        for p in range(len(toks)):
            rows[(rid, p)] = logits[p]
    return rows
