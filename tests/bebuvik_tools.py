"""Shared by the Bebuvik tests: small configurations that differ from one another in every size and option,
weights drawn so that activations are of order one (attention is far from uniform, gates are not all 1/2, sinks
matter), model folders, and the plain implementation's logits."""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def _mixer(heads, dim, rot_dim, vdim, kv_rank, window=None, kv_from=None, base=10000.0, rot_dims=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims},
         "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim)}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _layer(mixer, ff):
    return {"type": "latent_attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


CONFIGS = {
    # no size a power of two or a multiple of eight; three heads; a reader whose window is wider than its writer's;
    # a layer without feed-forward; a layer that sees every earlier position; three taps
    "P": {"architecture": "Bebuvik", "vocab": 211, "width": 44, "norm": {"eps": 3e-6}, "canon": {"taps": 3},
          "embedding": {"bigram": {"buckets": 97, "mul_prev": 31, "mul_cur": 5}}, "logit_softcap": 7.5,
          "layers": [_layer(_mixer(3, 10, 4, 12, 18, window=9), 60),
                     _layer(_mixer(3, 10, 4, 12, 18, window=21, kv_from=0), None),
                     _layer(_mixer(2, 6, 6, 14, 22, base=500.0, rot_dims=4), 36),
                     _layer(_mixer(5, 6, 6, 4, 22, window=5, kv_from=2, base=500.0, rot_dims=4), 52)]},
    # one head, two taps, a window of one page, sizes that are multiples of 16 (what tensor-core kernels take)
    "Q": {"architecture": "Bebuvik", "vocab": 320, "width": 64, "norm": {"eps": 1e-5}, "canon": {"taps": 2},
          "embedding": {"bigram": {"buckets": 509, "mul_prev": 1, "mul_cur": 3}}, "logit_softcap": 30.0,
          "layers": [_layer(_mixer(1, 32, 16, 32, 64, window=16, base=250000.0), 96),
                     _layer(_mixer(4, 16, 16, 16, 32, window=33), 128),
                     _layer(_mixer(8, 16, 16, 32, 32, window=64, kv_from=1), 64)]},
    # what the configuration may leave out: no input convolution, no bigram table, no soft cap, no window
    "R": {"architecture": "Bebuvik", "vocab": 150, "width": 40, "norm": {"eps": 1e-6},
          "layers": [_layer(_mixer(2, 8, 8, 8, 16), 48), _layer(_mixer(4, 8, 8, 8, 16, kv_from=0), 48)]},
    # one tap (a filter without state), five taps, long windows over small pages
    "S": {"architecture": "Bebuvik", "vocab": 190, "width": 48, "norm": {"eps": 2e-6}, "canon": {"taps": 5},
          "embedding": {"bigram": {"buckets": 64, "mul_prev": 7, "mul_cur": 7}}, "logit_softcap": 12.0,
          "layers": [_layer(_mixer(2, 16, 8, 24, 24, window=44), 80), _layer(_mixer(2, 16, 8, 24, 24, window=44, kv_from=0), 80),
                     _layer(_mixer(3, 8, 2, 8, 40, window=7), None)]},
}
CONFIGS["T"] = dict(CONFIGS["S"], canon={"taps": 1})
PAGE_SIZES = {"P": 8, "Q": 16, "R": 16, "S": 8, "T": 32}
SEEDS = {"P": 11, "Q": 12, "R": 13, "S": 14, "T": 15}


def draw_weights(cfg: dict, seed: int, dtype=torch.bfloat16) -> dict:
    """Weights by tensor name. Matrices N(0, 1 / fan-in) scaled up so that scores spread over several units,
    filters and biases of order one, sinks N(0, 1), scalar gains near one."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def mat(out, inp, gain=1.0):
        return (torch.randn(out, inp, generator=g) * gain / math.sqrt(inp)).to(dtype)

    w = {"embed": torch.randn(cfg["vocab"], W, generator=g).to(dtype), "head": mat(cfg["vocab"], W, 2.0),
         "final.norm": (1.0 + 0.2 * torch.randn((), generator=g)).to(dtype)}
    big = (cfg.get("embedding") or {}).get("bigram")
    if big:
        w["bigram"] = torch.randn(big["buckets"] + 1, W, generator=g).to(dtype)
    taps = (cfg.get("canon") or {}).get("taps")
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, d, r, e, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        w[p + "norm1"] = (1.0 + 0.2 * torch.randn((), generator=g)).to(dtype)
        w[p + "mix.q"] = mat(H * (d + r), W, 2.5)
        if m.get("kv_from") is None:
            w[p + "mix.dkv"] = mat(R + r, W, 2.0)
            w[p + "mix.dkv.norm"] = (1.0 + 0.3 * torch.randn(R, generator=g)).to(dtype)
        w[p + "mix.uk"] = mat(H * d, R, 1.5)
        w[p + "mix.uv"] = mat(H * e, R)
        w[p + "mix.sink"] = torch.randn(H, generator=g).to(dtype)
        w[p + "mix.o"] = mat(W, H * e)
        w[p + "rg1"] = mat(W, W)
        w[p + "rg1.b"] = (0.5 * torch.randn(W, generator=g)).to(dtype)
        if taps:
            w[p + "canon1"] = (0.4 * torch.randn(W, taps, generator=g)).to(dtype)
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            w[p + "mlp.up"], w[p + "mlp.down"] = mat(ff, W), mat(W, ff)
            w[p + "rg2"] = mat(W, W)
            w[p + "rg2.b"] = (0.5 * torch.randn(W, generator=g)).to(dtype)
            if taps:
                w[p + "canon2"] = (0.4 * torch.randn(W, taps, generator=g)).to(dtype)
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


def plain_rows(cfg: dict, weights: dict, requests: dict, dtype=torch.float64) -> dict:
    """{(request, position): logits row} from the plain implementation."""
    from plain import plain_bebuvik

    rows = {}
    for rid, toks in requests.items():
        logits = plain_bebuvik.forward(cfg, weights, toks, dtype).to(torch.float32).numpy()
        for p in range(len(toks)):
            rows[(rid, p)] = logits[p]
    return rows
