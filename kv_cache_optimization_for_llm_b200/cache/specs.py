"""What a mixer asks of the cache, and what it is handed back at each step."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values that grow with the sequence, kept in pages.  ``window``: only
    the newest ``window`` keys are ever read, older pages may be given back.
    ``keep_first``: with a window, the sequence's first ``keep_first`` keys are read for good as
    well, so the pages that hold them stay.
    ``planes``: 2 keeps keys and values; 1 keeps a single row per token and head (a mixer
    whose keys and values are both read from one cached latent, or one that lays a token's key
    and value side by side in a row of ``head_dim`` = key size + value size)."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    planes: int = 2
    keep_first: int = 0


@dataclass(frozen=True)
class SlotStateSpec:
    """State of fixed size per request, kept in the request's state slot."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class PagedWithStateSpec:
    """Both: rows that grow with the sequence, in pages, and a state of fixed size in the request's
    slot (a mixer that attends over cached keys and also carries the last inputs of a short
    convolution from step to step)."""
    paged: PagedKVSpec
    state: SlotStateSpec


def paged_part(spec) -> Optional[PagedKVSpec]:
    """What a mixer's wish asks of the page pools (None: nothing)."""
    if isinstance(spec, PagedKVSpec):
        return spec
    return spec.paged if isinstance(spec, PagedWithStateSpec) else None


def state_part(spec) -> Optional[SlotStateSpec]:
    """What a mixer's wish asks of the state slots (None: nothing)."""
    if isinstance(spec, SlotStateSpec):
        return spec
    return spec.state if isinstance(spec, PagedWithStateSpec) else None


@dataclass
class PagedKVBinding:
    """A schedule entry's view of its pages: ``k`` and ``v`` are
    [num_pages, num_kv_heads, page_size, head_dim] (``v`` is None for a group that keeps one
    plane); the block tables of the step's
    requests are ``batch.block_tables[group]``.  ``write`` is False for an entry that
    reads another entry's cache.  ``state``: the per-request state ``state[slot]`` of a mixer that
    asked for one beside its pages (:class:`PagedWithStateSpec`), else None."""
    k: torch.Tensor
    v: Optional[torch.Tensor]
    group: int
    page_size: int
    write: bool = True
    state: Optional[torch.Tensor] = None


@dataclass
class SlotStateBinding:
    """A schedule entry's per-request state: ``state[slot]`` with the step's slots in
    ``batch.slots``.  A request whose portion starts at position 0 has to be reset
    by the mixer (``batch.req_start``)."""
    state: torch.Tensor
    write: bool = True
