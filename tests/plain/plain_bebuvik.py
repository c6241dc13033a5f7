"""A plain, slow implementation of the Bebuvik design on the CPU: whole sequences,
no cache, no state, one function per mechanism. It is the yardstick the engine
is compared with and shares no code with it: it takes config.json as a
dictionary and the weights as a {name: tensor} dictionary.

The design in short. Tokens are embedded as a table row plus a row of a hashed
bigram table. Every layer normalises the stream once (RMS norm with a single
gain), hands that to a mixer and to a feed-forward side by side, each behind a
short causal convolution over time that is added to its input, and adds both
results, each scaled by a sigmoid gate computed from the normalised stream. The
mixer is attention over a low-rank latent: keys and values are expanded per head
from one cached vector per position, a small rotated part of the key is shared
by all heads, positions see a sliding window, and the softmax's denominator
holds one extra learned term per head that has no value. Some layers have no
latent projection of their own and read another layer's. The logits are
squashed by a scaled tanh.

Arithmetic is in `dtype` (float32 or float64) throughout.
"""

from __future__ import annotations

import math

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def scalar_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose gain is one number for all coordinates."""
    return rms_unit(x, eps) * gain.reshape(())


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def bigram_rows(tokens, buckets: int, mul_prev: int, mul_cur: int) -> list:
    """Row of the bigram table for every token of one sequence: a hash of (previous, current);
    the first token, which has no previous one, takes the table's last row."""
    rows = []
    for i, t in enumerate(tokens):
        rows.append(buckets if i == 0 else (int(tokens[i - 1]) * mul_prev + int(t) * mul_cur) % buckets)
    return rows


def embed(tokens, table: torch.Tensor, bigram, hash_cfg) -> torch.Tensor:
    x = table[torch.tensor(list(tokens), dtype=torch.long)]
    if bigram is not None:
        rows = bigram_rows(tokens, hash_cfg["buckets"], hash_cfg["mul_prev"], hash_cfg["mul_cur"])
        x = x + bigram[torch.tensor(rows, dtype=torch.long)]
    return x


def causal_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h [T, C], w [C, taps]: out_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the start."""
    T, taps = h.shape[0], w.shape[1]
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def rotate_interleaved(v: torch.Tensor, positions, base: float, dims: int) -> torch.Tensor:
    """v [T, ..., D]: the first `dims` coordinates are rotated in pairs (2i, 2i + 1) by the angle
    position * base^(-2i / dims); the rest pass."""
    out = v.clone()
    for n, p in enumerate(positions):
        for i in range(dims // 2):
            f = torch.tensor(float(base), dtype=v.dtype) ** (-2.0 * i / dims)
            a = torch.tensor(float(p), dtype=v.dtype) * f
            c, s = torch.cos(a), torch.sin(a)
            a0, a1 = v[n, ..., 2 * i].clone(), v[n, ..., 2 * i + 1].clone()
            out[n, ..., 2 * i] = a0 * c - a1 * s
            out[n, ..., 2 * i + 1] = a1 * c + a0 * s
    return out


def latent_of(u: torch.Tensor, w_dkv: torch.Tensor, gain: torch.Tensor, eps: float, rank: int,
              positions, base: float, rot_dims: int):
    """The cached pair of one layer: the normalised latent [T, rank] and the rotated shared key part
    [T, rot_dim]."""
    z = u @ w_dkv.t()
    c = rms_unit(z[:, :rank], eps) * gain
    kr = rotate_interleaved(z[:, rank:], positions, base, rot_dims)
    return c, kr


def windowed_sink_attention(q_plain, q_rot, k_plain, k_rot, v, sink, scale: float, window):
    """q_plain [T, H, d], q_rot [T, H, r], k_plain [T, H, d], k_rot [T, r], v [T, H, e], sink [H].
    Position i sees j with 0 <= i - j < window (window None: every j <= i). The weights of a row
    are exp(score) / (sum of exp(score) + exp(sink))."""
    T, H, _ = q_plain.shape
    out = torch.zeros((T, H, v.shape[-1]), dtype=v.dtype)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        for h in range(H):
            s = (k_plain[lo:i + 1, h] @ q_plain[i, h] + k_rot[lo:i + 1] @ q_rot[i, h]) * scale
            m = torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            out[i, h] = (e / (e.sum() + torch.exp(sink[h] - m))) @ v[lo:i + 1, h]
    return out


def latent_attention(u, w, prefix: str, m: dict, eps: float, positions, shared):
    """The mixer on its input u [T, width]. `shared` is (latent, rotated key part) of the layer that
    `kv_from` names, or None when this layer projects its own. Returns (output, (latent, key part))."""
    H, d, r, e, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base, rot_dims = m["rot"]["base"], m["rot"]["dims"]
    T = u.shape[0]
    q = (u @ w[prefix + "q"].t()).reshape(T, H, d + r)
    q_plain = q[..., :d]
    q_rot = rotate_interleaved(q[..., d:], positions, base, rot_dims)
    if shared is None:
        shared = latent_of(u, w[prefix + "dkv"], w[prefix + "dkv.norm"], eps, rank, positions, base, rot_dims)
    c, kr = shared
    k_plain = (c @ w[prefix + "uk"].t()).reshape(T, H, d)
    v = (c @ w[prefix + "uv"].t()).reshape(T, H, e)
    window = (m.get("mask") or {}).get("size")
    o = windowed_sink_attention(q_plain, q_rot, k_plain, kr, v, w[prefix + "sink"], m["scale"], window)
    return o.reshape(T, H * e) @ w[prefix + "o"].t(), shared


def dense_ff(u, w_up, w_down):
    return gelu_tanh(u @ w_up.t()) @ w_down.t()


def layer(x, w, i: int, spec: dict, cfg: dict, positions, latents: dict):
    """One layer on the stream x [T, width]; `latents` collects every layer's cached pair."""
    p = f"l{i}."
    eps = cfg["norm"]["eps"]
    h = scalar_norm(x, w[p + "norm1"], eps)
    canon = "canon" in cfg
    u1 = h + causal_conv(h, w[p + "canon1"]) if canon else h
    m = spec["mixer"]
    shared = latents[m["kv_from"]] if m.get("kv_from") is not None else None
    y, latents[i] = latent_attention(u1, w, p + "mix.", m, eps, positions, shared)
    total = torch.sigmoid(h @ w[p + "rg1"].t() + w[p + "rg1.b"]) * y
    if spec.get("mlp") is not None:
        u2 = h + causal_conv(h, w[p + "canon2"]) if canon else h
        f = dense_ff(u2, w[p + "mlp.up"], w[p + "mlp.down"])
        total = total + torch.sigmoid(h @ w[p + "rg2"].t() + w[p + "rg2.b"]) * f
    return x + total


def forward(cfg: dict, weights: dict, tokens, dtype=torch.float32, streams=None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence. `streams`, a list, receives the stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    positions = list(range(len(tokens)))
    x = embed(tokens, w["embed"], w.get("bigram"), (cfg.get("embedding") or {}).get("bigram"))
    latents = {}
    for i, spec in enumerate(cfg["layers"]):
        x = layer(x, w, i, spec, cfg, positions, latents)
        if streams is not None:
            streams.append(x.clone())
    z = scalar_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].t()
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z
