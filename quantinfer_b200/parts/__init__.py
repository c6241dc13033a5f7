from . import attention, block, embedding, ffn, latent_attention, norm, position, short_conv  # noqa: F401  (registers the built-in kinds)
from .base import Part, Runtime, build_part, part_class, register_part
from .linear import Linear

__all__ = ["Part", "Runtime", "build_part", "part_class", "register_part", "Linear"]
