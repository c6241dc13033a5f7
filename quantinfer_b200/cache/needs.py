"""What a mixer asks of the cache manager for one cache entry."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every position (window None) or of the last `window`
    positions, in pages [num_pages, num_kv_heads, page_size, head_dim]."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


    def pools(self, page_size: int) -> tuple:
        """Shapes of a page in the key pool and in the value pool."""
        shape = (self.num_kv_heads, page_size, self.head_dim)
        return shape, shape

    def merged(self, other):
        """The need of an entry that `other` reads too, or None when the two cannot share one."""
        if not isinstance(other, PagedKVNeed) or (other.num_kv_heads, other.head_dim) != (self.num_kv_heads, self.head_dim):
            return None
        return PagedKVNeed(self.num_kv_heads, self.head_dim, _wider(self.window, other.window))


@dataclass(frozen=True)
class PagedLatentNeed:
    """One row of `width` numbers per position (a latent and what rides with it), shared by every
    head, in pages [num_pages, page_size, width]; there is no second pool. `window` as above."""

    width: int
    window: Optional[int] = None

    def pools(self, page_size: int) -> tuple:
        return (page_size, self.width), None

    def merged(self, other):
        if not isinstance(other, PagedLatentNeed) or other.width != self.width:
            return None
        return PagedLatentNeed(self.width, _wider(self.window, other.window))


def _wider(a, b):
    """The window that keeps what both readers see (None: everything)."""
    return None if a is None or b is None else max(a, b)


@dataclass(frozen=True)
class StateNeed:
    """A state of fixed size per request, in a slot: [num_slots, *shape].
    `dtype` None means the activation type. A slot is zeroed when a request opens."""

    shape: tuple
    dtype: object = None
