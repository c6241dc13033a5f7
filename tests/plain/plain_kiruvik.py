"""A plain, slow restatement of the Kiruvik design in float64, one function per mechanism, for whole
sequences at once (no cache, no state carried between calls, no batching). It reads the design's config
dictionary and a dictionary of tensors by name and shares nothing with the engine.

Notation: T tokens, positions 0 .. T - 1; matrices are stored [out, in] and applied as x @ W.T.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def f64(t):
    return t.to(F)


def dyt(x, w, b, alpha):
    """Dynamic tanh: tanh(alpha x) w + b, elementwise; no statistics of x."""
    return torch.tanh(f64(alpha) * x) * f64(w) + f64(b)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotate_half_split(x, positions, dims, base):
    """x [T, heads, d]; the first `dims` coordinates of a head turn: coordinate i pairs with i + dims / 2,
    by the angle position * base^(-2 i / dims); the rest pass."""
    if not dims:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=F)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(F)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def visible(T, chunk=None, window=None):
    """Boolean [T, T]: query i sees key j."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if chunk:
        ok &= (i // chunk) == (j // chunk)
    if window:
        ok &= j > i - window
    return ok


def gated_attention(h, m, w, p):
    """m: the mixer's config; w: tensors; p: the prefix of its tensor names ('l3.mix.')."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    lin = lambda name: h @ f64(w[p + name]).T + f64(w[p + name + ".b"])
    q = lin("q").view(T, H, d)
    k = lin("k").view(T, G, d)
    v = lin("v").view(T, G, dv)
    pos = torch.arange(T)
    rot = m.get("rot") or {}
    q = rotate_half_split(q, pos, rot.get("dims", 0), rot.get("base", 1.0))
    k = rotate_half_split(k, pos, rot.get("dims", 0), rot.get("base", 1.0))
    mask = visible(T, chunk=(m.get("mask") or {}).get("size"))
    out = torch.zeros(T, H, dv, dtype=F)
    for hq in range(H):
        g = hq // (H // G)
        s = (q[:, hq] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~mask, float("-inf"))
        out[:, hq] = torch.softmax(s, dim=-1) @ v[:, g]
    gate = torch.sigmoid(h @ f64(w[p + "g"]).T)
    return (out.reshape(T, H * dv) * gate) @ f64(w[p + "o"]).T + f64(w[p + "o.b"])


def causal_conv(x, filt, bias):
    """x [T, C]; filt [C, taps], the last column weighs the current token; zeros before the start."""
    T, C = x.shape
    taps = filt.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=F), x])
    y = f64(bias)[None, :].repeat(T, 1)
    for j in range(taps):
        y = y + pad[j:j + T] * f64(filt)[:, j][None, :]
    return y


def mamba2(h, m, w, p, eps):
    T = h.shape[0]
    nh, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = nh * P
    proj = h @ f64(w[p + "in"]).T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(T, nh, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + f64(w[p + "dt_bias"]))
    A = -torch.exp(f64(w[p + "A_log"]))
    D = f64(w[p + "D"])
    y = torch.zeros(T, nh, P, dtype=F)
    for hd in range(nh):
        g = hd // (nh // G)
        S = torch.zeros(N, P, dtype=F)
        for t in range(T):
            S = torch.exp(A[hd] * dt[t, hd]) * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + D[hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    yg = y.view(T, parts, inner // parts)
    yg = yg / torch.sqrt((yg ** 2).mean(dim=-1, keepdim=True) + eps)
    y = yg.reshape(T, inner) * f64(w[p + "norm"])
    return y @ f64(w[p + "o"]).T


def dense_ffn(h, w, p):
    return (gelu_tanh(h @ f64(w[p + "gate"]).T) * (h @ f64(w[p + "up"]).T)) @ f64(w[p + "down"]).T


def clamped_expert(h, w, p, limit):
    g = torch.clamp(h @ f64(w[p + "gate"]).T, max=limit)
    u = torch.clamp(h @ f64(w[p + "up"]).T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ f64(w[p + "down"]).T


def moe(h, mlp, w, p):
    r = mlp["router"]
    E, top = r["experts"], r["top"]
    s = torch.softmax(h @ f64(w[p + "router"]).T, dim=-1)
    choice = s + f64(w[p + "correction"])
    idx = torch.topk(choice, top, dim=-1).indices
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        sel = s[t, idx[t]]
        wt = sel / (sel.sum() + 1e-20) * r["scale"]
        for j in range(top):
            e = int(idx[t, j])
            out[t] += wt[j] * clamped_expert(h[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + clamped_expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


def layer(x, cfg, i, w):
    e = cfg["layers"][i]
    p = f"l{i}."
    m = cfg["residual_mult"]
    norm = lambda name, v: dyt(v, w[p + name], w[p + name + ".b"], w[p + name + ".alpha"])
    h = norm("norm1", x)
    if e["type"] == "attention":
        y = gated_attention(h, e["mixer"], w, p + "mix.")
    elif e["type"] == "mamba2":
        y = mamba2(h, e["mixer"], w, p + "mix.", cfg["norm"]["eps"])
    else:
        raise ValueError(e["type"])
    x = x + m * norm("norm1b", y)
    if e.get("mlp") is not None:
        h = norm("norm2", x)
        y = dense_ffn(h, w, p + "mlp.") if e["mlp"]["kind"] == "dense" else moe(h, e["mlp"], w, p + "mlp.")
        x = x + m * norm("norm2b", y)
    return x


def run_order(cfg):
    """Layer indices in the order they run; True marks the first layer of a pass of the loop."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for _ in range(times):
        order += [(i, i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(cfg, w, tokens, want_layers=False):
    """Logits [T, vocab] of one sequence from its first token on."""
    x0 = f64(w["embed"])[torch.as_tensor(tokens, dtype=torch.long)]
    x = x0
    after = []
    for i, reenter in run_order(cfg):
        if reenter:
            x = torch.cat([x, x0], dim=-1) @ f64(w["loop.in"]).T
        x = layer(x, cfg, i, w)
        after.append(x)
    h = dyt(x, w["final.norm"], w["final.norm.b"], w["final.norm.alpha"])
    logits = h @ f64(w["head"]).T
    return (logits, after) if want_layers else logits
