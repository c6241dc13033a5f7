"""A bank of short causal convolutions over time that read one input.

    out_k[t] = (x[t] if residual) + sum_j w_k[:, j] * x[t - taps + 1 + j]        per channel, j = 0 .. taps - 1

over each request's own time axis, zeros before its start. Each filter is a tensor [width, taps]; the
request's last taps - 1 inputs are its state of fixed size (`state_need`), which the kernel reads for a step's
first tokens and advances, so a step may cut a sequence anywhere. The input is the 32-bit output of a norm;
the sums are 32-bit; the outputs come in the activation type (they feed projections).
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache.needs import StateNeed
from ..errors import ConfigError
from ..weights.loader import TensorNeed
from .base import Part, register_part


class ShortConv(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if not 1 <= len(spec.names) <= 2:
            raise ConfigError("short_conv: one or two filters over one input")
        if spec.taps < 1:
            raise ConfigError("short_conv: a filter needs at least one tap")
        self.weights = None      # float32 [filters, taps, width]

    @classmethod
    def needs_of_spec(cls, spec):
        return {name: TensorNeed((spec.width, spec.taps)) for name in spec.names}

    def load(self, tensors):
        w = torch.stack([tensors[n].to(torch.float32).t() for n in self.spec.names])
        self.weights = w.to(self.runtime.device).contiguous()

    def state_need(self):
        return StateNeed((self.spec.taps - 1, self.spec.width), torch.float32) if self.spec.taps > 1 else None

    def forward(self, x, batch, state, want_copy: bool = False):
        """x float32 [tokens, width]. Returns (outputs, one per filter, in the activation type; x in that type or
        None)."""
        outs = [torch.empty(x.shape, dtype=self.runtime.dtype, device=x.device) for _ in self.spec.names]
        copy = torch.empty(x.shape, dtype=self.runtime.dtype, device=x.device) if want_copy else None
        kernels.short_conv(x, self.weights, state, outs, copy, batch.token_req, batch.q_start, batch.start_pos,
                           batch.slot_ids, residual=self.spec.residual)
        return outs, copy


register_part("conv", "short_conv", ShortConv)
