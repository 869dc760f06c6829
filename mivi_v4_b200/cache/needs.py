"""What a mixer asks of the cache.  A mixer that keeps nothing returns None; one that keeps
several things (keys and values AND a state, two states of different shape or dtype) returns a
list of needs and gets a list of views, one for each, in the same order."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch


@dataclass(frozen=True)
class KVNeed:
    """Keys and values that grow by one row per token.  ``window`` > 0: only the
    last ``window`` tokens are ever read, so pages that lie wholly before them
    are given back while the sequence is still running; ``keep_first`` tokens at the start of the sequence
    stay readable for good, so the pages that hold any of them are never given back.  ``v_dim`` > 0: values
    of another size than the keys' ``head_dim``; a page is then one flat row, the keys [kv head][row][head_dim]
    followed by the values [kv head][row][v_dim].  ``chunk`` > 0 (instead of a window): a token reads only the
    keys of its own chunk of ``chunk`` positions, counted from the sequence's start, so the pages that lie wholly
    before the chunk of the next token are given back.  ``values_in_keys``: the values are the first ``v_dim``
    elements of the keys' rows (a compressed cache that all heads read), so a page holds rows only:
    [kv head][row][head_dim]."""
    n_kv_heads: int
    head_dim: int
    window: int = 0
    v_dim: int = 0
    keep_first: int = 0
    chunk: int = 0
    values_in_keys: bool = False

    @property
    def value_dim(self) -> int:
        return self.v_dim or self.head_dim

    @property
    def uneven(self) -> bool:
        return self.values_in_keys or self.value_dim != self.head_dim

    def page_elements(self, page_size: int) -> int:
        """Elements of one layer's page when it is one flat row (``uneven``)."""
        per_row = self.head_dim if self.values_in_keys else self.head_dim + self.value_dim
        return self.n_kv_heads * page_size * per_row


@dataclass(frozen=True)
class StateNeed:
    """State of a fixed size per sequence, zero when a sequence starts (the short
    convolution's last k-1 inputs; any recurrent state).  ``dtype``: what it is stored in."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32
