from . import attention, block, embedding, ffn, gated_attention, latent_attention, mamba2, moe, norm, position, reentry, short_conv  # noqa: F401  (registers the built-in kinds)
from .base import Part, Runtime, build_part, part_class, register_part
from .linear import Linear

__all__ = ["Part", "Runtime", "build_part", "part_class", "register_part", "Linear"]
