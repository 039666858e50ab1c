"""What a mixer keeps for each request, as plain data.

`PagedKV`: keys and values that grow by one row per token, stored in pages.
`window`, when set, means that only the last `window` tokens are ever read, so
pages that lie wholly before the window may be given back.  `chunk`, when set,
means that positions form blocks of that many from the request's first token and
no query reads a key of an earlier block, so pages that lie wholly before the
block of the next query may be given back too.
`PagedLatent`: one row per token from which keys and values are both derived (a
compressed latent); paged and windowed like `PagedKV`, but stored once.
`FixedState`: a tensor of fixed shape per request, stored in a slot.
`Several`: a mixer that keeps more than one of these (two mixers side by side); every part is placed as if it
were a call's only need, and the call's cache holds them in order (`CallCache.parts`).
Calls of the running order whose needs are equal share one group: one pool of
pages (or slots) and one block table per request.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class PagedKV:
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    chunk: Optional[int] = None

    planes = 2                      # keys and values are stored apart

    def bytes_per_token(self, itemsize: int) -> int:
        return 2 * self.num_kv_heads * self.head_dim * itemsize


@dataclass(frozen=True)
class PagedLatent:
    """A row of `width` numbers per token, read both as the key and as the value of one shared head."""
    width: int
    window: Optional[int] = None
    chunk: Optional[int] = None

    planes = 1                      # one tensor serves as keys and as values
    num_kv_heads = 1

    @property
    def head_dim(self) -> int:
        return self.width

    def bytes_per_token(self, itemsize: int) -> int:
        return self.width * itemsize


def first_needed_position(need, num_tokens: int) -> int:
    """The first position that a query at position `num_tokens` or later of a request can still read."""
    first = 0
    if need.window is not None:
        first = max(first, num_tokens - need.window + 1)
    if getattr(need, "chunk", None):
        first = max(first, num_tokens // need.chunk * need.chunk)
    return first


@dataclass(frozen=True)
class FixedState:
    shape: Tuple[int, ...]
    dtype: str = "float32"


@dataclass(frozen=True)
class Several:
    parts: Tuple[object, ...]
