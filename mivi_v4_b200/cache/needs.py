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
    are given back while the sequence is still running."""
    n_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateNeed:
    """State of a fixed size per sequence, zero when a sequence starts (the short
    convolution's last k-1 inputs; any recurrent state).  ``dtype``: what it is stored in."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32
