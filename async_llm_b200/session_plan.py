"""Write planning of the cache-view session: which slots the new tokens go to.

Restates the two integer-only helpers of the reference session that the attention planner and
the kernels depend on (bit-exact index code):

* ``plan_decode_writes``  -- SharedCacheSession._plan_decode_writes (session.py:1102-1141)
* ``alloc_token_storage`` -- SharedCacheSession._alloc_token_storage (session.py:1078-1100)
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .blocks import CacheBlock, WorkerGroup


def plan_decode_writes(group: WorkerGroup, page_allocator, page_size: int, device) -> Tuple[
        Dict[int, Optional[int]], torch.Tensor, List[int]]:
    """Destination of every worker's new token for one decode step.

    Returns ``(new_page_for_block, new_token_slots, write_pos)``: ``id(block) ->`` page-start slot
    of a freshly borrowed page (or None), the ``[W]`` int32 destination slots, and the
    block-relative RoPE position of each write (the block's mRoPE span).  All blocks whose last
    page is full share ONE allocation; an allocator that keeps a host copy of its free list
    (``alloc_page_list``) answers it without a device-to-host readback, which would wait for
    everything queued on the stream.
    """
    pending: Dict[int, Optional[int]] = {}
    full: List[CacheBlock] = []
    for target in group.write_to:
        if id(target) in pending:
            raise ValueError("WorkerGroup has two workers writing the same block in one step")
        pending[id(target)] = None
        if not target.has_capacity:
            full.append(target)
    if full:
        take = getattr(page_allocator, "alloc_page_list", None)
        fresh = take(len(full)) if take is not None else page_allocator.alloc_pages(len(full)).cpu().tolist()
        for target, start in zip(full, fresh):
            pending[id(target)] = start
    slots: List[int] = []
    positions: List[int] = []
    for target in group.write_to:
        page = pending[id(target)]
        base = target.page_starts[-1] if page is None else page
        slots.append(base + target.num_tokens % page_size)
        positions.append(target.mrope_span)
    return pending, torch.tensor(slots, dtype=torch.int32, device=device), positions


def alloc_token_storage(page_allocator, page_size: int, device, seq_len: int,
                        write_to: Optional[CacheBlock] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Borrow the pages needed to append ``seq_len`` tokens to ``write_to``.

    Returns ``(new_page_starts, token_slots)``: the free tail of the block's last page is used
    first, then the fresh pages, in block order.
    """
    tail = 0 if write_to is None else write_to.free_tail
    fresh = -(-max(0, seq_len - tail) // page_size)
    starts = page_allocator.alloc_pages(fresh)
    slots = page_allocator.pages_to_tokens(starts)
    if tail == 0:
        return starts, slots[:seq_len]
    first = write_to.page_starts[-1] + write_to.last_page_len
    head = torch.arange(first, first + tail, dtype=slots.dtype, device=device)
    return starts, torch.cat((head, slots))[:seq_len]
