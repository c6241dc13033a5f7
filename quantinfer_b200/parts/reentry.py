"""What a pass over a looped stretch of layers begins with: the stream is mixed with the embedding's output,

    x <- [x ; x0] . W^T          W [hidden, 2 hidden], x first

The two 32-bit streams are written side by side in the activation type (one small kernel) and projected back to a
32-bit stream; whatever the layer before left pending is added to the stream first.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorNeed
from .base import Part, register_part
from .linear import Linear
from .norm import PostNormed


class ConcatProjection(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.proj = Linear(runtime, spec.hidden_size, 2 * spec.hidden_size, spec.weight_name)

    @classmethod
    def needs_of_spec(cls, spec):
        return {spec.weight_name: TensorNeed((spec.hidden_size, 2 * spec.hidden_size))}

    def load(self, tensors):
        self.proj.load(tensors[self.spec.weight_name])

    def forward(self, resid, delta, x0):
        if isinstance(delta, PostNormed):
            delta = delta.apply(resid)
        if delta is not None:
            kernels.dyt(resid, delta)
        both = torch.empty((resid.shape[0], 2 * self.spec.hidden_size), dtype=self.runtime.dtype, device=resid.device)
        kernels.concat_cast(resid, x0, both)
        return self.proj(both, out_dtype=torch.float32)


register_part("reentry", "concat_proj", ConcatProjection)
