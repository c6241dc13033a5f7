"""What a mixer asks of the cache manager for one cache entry."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every position (window None) or of the last `window`
    positions, in pages [num_pages, num_kv_heads, page_size, head_dim] (values
    [..., value_dim] when that is given). `chunk`: queries see only the keys of
    their own chunk of that many positions (counted from the sequence's start),
    so the pages of earlier chunks go back as soon as a request has passed them."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    value_dim: Optional[int] = None
    chunk: Optional[int] = None

    def pools(self, page_size: int) -> tuple:
        """Shapes of a page in the key pool and in the value pool."""
        return ((self.num_kv_heads, page_size, self.head_dim),
                (self.num_kv_heads, page_size, self.value_dim or self.head_dim))

    def merged(self, other):
        """The need of an entry that `other` reads too, or None when the two cannot share one."""
        if not isinstance(other, PagedKVNeed) or (other.num_kv_heads, other.head_dim, other.value_dim or other.head_dim) != (
                self.num_kv_heads, self.head_dim, self.value_dim or self.head_dim):
            return None
        if self.chunk != other.chunk:      # readers with other chunks: keep what any of them may see
            return PagedKVNeed(self.num_kv_heads, self.head_dim, None, self.value_dim, None)
        return PagedKVNeed(self.num_kv_heads, self.head_dim, _wider(self.window, other.window), self.value_dim, self.chunk)


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
