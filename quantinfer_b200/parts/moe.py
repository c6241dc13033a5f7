"""Feed-forwards of the clamped gated form, alone and as a routed mixture.

    expert(x) = down(g * sigmoid(alpha g) * (u + 1)),   g = min(gate(x), limit),  u = clamp(up(x), -limit, limit)

`ClampedGLU` is one such feed-forward for every token (gate and up stacked into one product). `MoE` routes:

    s       = softmax(router(x))                        over all experts, 32-bit
    chosen  = the `top` largest of s + correction       (the correction steers the choice only)
    w_k     = s_k / (sum of the chosen s + 1e-20) * router_scale
    y       = sum_k w_k expert_k(x)  (+ shared(x))

The tokens are grouped by expert on the device: the (token, choice) pairs are sorted by expert, each expert's rows
form tiles of their own, and ONE grouped launch per projection runs every expert over exactly its rows; no count
crosses to the host, so the step can sit in a CUDA graph. The experts' matrices are stacked [experts, out, in] at
load. A row's result does not depend on what else the expert got, so a token's output is the same in any batch.

A step of many tokens (a prompt or a long portion; never a step that is being captured) instead reads the experts'
row counts on the host, once, gathers the rows into the experts' order and runs each expert's rows through the
framework's tcgen05 product, which is several times faster than the grouped mma.sync kernel at such sizes.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..errors import ConfigError
from ..weights.loader import TensorNeed
from .base import Part, register_part
from .linear import Linear


class ClampedGLU(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        h, i = spec.hidden_size, spec.intermediate_size
        self.gate_up = Linear(runtime, 2 * i, h, spec.prefix + "gate+up")
        self.down = Linear(runtime, h, i, spec.prefix + "down")

    @classmethod
    def needs_of_spec(cls, spec):
        h, i, p = spec.hidden_size, spec.intermediate_size, spec.prefix
        return {p + "gate": TensorNeed((i, h)), p + "up": TensorNeed((i, h)), p + "down": TensorNeed((h, i))}

    def load(self, tensors):
        p = self.spec.prefix
        g, u = tensors[p + "gate"], tensors[p + "up"]
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        self.gate_up.load(torch.cat([g, u], dim=0))
        self.down.load(tensors[p + "down"])

    def forward(self, x):
        gu = self.gate_up(x)
        a = torch.empty((x.shape[0], self.spec.intermediate_size), dtype=x.dtype, device=x.device)
        kernels.glu_clamped(gu, a, self.spec.limit, self.spec.alpha)
        return self.down(a)

    __call__ = forward


class MoE(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        s = spec
        if not 0 < s.top <= s.experts:
            raise ConfigError(f"moe: {s.top} of {s.experts} experts a token")
        self.router = Linear(runtime, s.experts, s.hidden_size, s.prefix + "router")
        self.shared = ClampedGLU(s.shared, runtime) if s.shared is not None else None
        self.w_gate_up = self.w_down = self.correction = None

    @classmethod
    def needs_of_spec(cls, s):
        p, h, i = s.prefix, s.hidden_size, s.expert.intermediate_size
        needs = {}
        for e in range(s.experts):
            needs.update({f"{p}e{e}.gate": TensorNeed((i, h)), f"{p}e{e}.up": TensorNeed((i, h)), f"{p}e{e}.down": TensorNeed((h, i))})
        needs[p + "router"] = TensorNeed((s.experts, h))
        needs[p + "correction"] = TensorNeed((s.experts,), "matrix", "zeros")
        if s.shared is not None:
            needs.update(ClampedGLU.needs_of_spec(s.shared))
        return needs

    def load(self, tensors):
        s, p, rt = self.spec, self.spec.prefix, self.runtime
        self.router.load(tensors[p + "router"])
        self.correction = self._gain(tensors[p + "correction"])
        gu = torch.stack([torch.cat([tensors[f"{p}e{e}.gate"], tensors[f"{p}e{e}.up"]], dim=0) for e in range(s.experts)])
        down = torch.stack([tensors[f"{p}e{e}.down"] for e in range(s.experts)])
        if rt.dtype == torch.float32:
            gu, down = gu.to(torch.float32), down.to(torch.float32)
        self.w_gate_up, self.w_down = gu.to(rt.device).contiguous(), down.to(rt.device).contiguous()
        if self.shared is not None:
            self.shared.load(tensors)

    ROWS_AN_EXPERT = 128      # from this many rows an expert (on average) a step goes expert by expert

    def _by_expert(self, x, pairs: int) -> bool:
        s = self.spec
        return (x.dtype == torch.bfloat16 and self.w_gate_up.dtype == torch.bfloat16 and not kernels.knock_out
                and pairs >= self.ROWS_AN_EXPERT * s.experts and s.hidden_size % 8 == 0 and s.expert.intermediate_size % 8 == 0
                and not torch.cuda.is_current_stream_capturing())

    def forward(self, x):
        s = self.spec
        n, dev = x.shape[0], x.device
        pairs, ff = n * s.top, s.expert.intermediate_size
        logits = self.router(x, out_dtype=torch.float32)
        ids = torch.empty((n, s.top), dtype=torch.int32, device=dev)
        weights = torch.empty((n, s.top), dtype=torch.float32, device=dev)
        kernels.moe_route(logits, self.correction, ids, weights, s.router_scale)
        offsets = torch.empty(s.experts + 1, dtype=torch.int32, device=dev)
        order = torch.empty(pairs, dtype=torch.int32, device=dev)
        place = torch.empty(pairs, dtype=torch.int32, device=dev)
        tiles = torch.empty((min(pairs, pairs // kernels.moe_tile_rows() + s.experts), 3), dtype=torch.int32, device=dev)
        kernels.moe_group(ids, s.experts, offsets, order, place, tiles)
        gu = torch.empty((pairs, 2 * ff), dtype=x.dtype, device=dev)
        a = torch.empty((pairs, ff), dtype=x.dtype, device=dev)
        y = torch.empty((pairs, s.hidden_size), dtype=x.dtype, device=dev)
        if self._by_expert(x, pairs):
            bounds = offsets.tolist()          # the one place where such a step waits for the device
            xs = torch.empty((pairs, s.hidden_size), dtype=x.dtype, device=dev)
            kernels.moe_gather(x, order, s.top, xs)
            kernels.moe_gemm_by_expert(xs, self.w_gate_up, gu, bounds, self.runtime.status)
            kernels.glu_clamped(gu, a, s.expert.limit, s.expert.alpha)
            kernels.moe_gemm_by_expert(a, self.w_down, y, bounds, self.runtime.status)
        else:
            kernels.moe_gemm(x, self.w_gate_up, gu, tiles, order, s.top, gather=True)
            kernels.glu_clamped(gu, a, s.expert.limit, s.expert.alpha)
            kernels.moe_gemm(a, self.w_down, y, tiles, order, s.top, gather=False)
        shared = self.shared.forward(x) if self.shared is not None else None
        out = torch.empty((n, s.hidden_size), dtype=x.dtype, device=dev)
        kernels.moe_combine(y, place, weights, shared, out)
        return out

    __call__ = forward


register_part("ffn", "clamped_glu", ClampedGLU)
register_part("ffn", "moe", MoE)
