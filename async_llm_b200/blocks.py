"""Host-side request model of the cache-view path: blocks, contexts and worker groups.

These classes keep the public names, constructor arguments, attributes and error
behaviour of the reference request model so user code written against it runs
unchanged:

* ``CacheBlock``   -- minisgl/shared_cache/shared_block.py:24-195
* ``AsyncContext`` -- minisgl/shared_cache/async_context.py:12-40
* ``WorkerGroup``  -- minisgl/shared_cache/worker_group.py:9-97

A block is an ordered list of pool pages plus a token count.  Block-relative token
``i`` lives in physical slot ``page_starts[i // P] + i % P``.  Keys in the pool are
rotated at block-relative positions; nothing here touches device memory.
"""

from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Dict, Iterator, List, Optional, Sequence, Tuple, Union

import torch


class _TrackedDict(dict):
    """dict that bumps its owner's revision before any mutation.

    Mirrors the invalidation contract of the reference ``StateDict``
    (minisgl/shared_cache/gdn_state.py:15-58): planners may cache per-block
    address tables and must notice when a state tensor is replaced.

    A publisher that replaces every entry at once (one decode step writes all layers of a block) may
    hand the entries over as a producer (``defer``): the per-layer tensor views are then only built
    when somebody reads the dictionary -- the kernels work from the cached addresses and never do.
    """

    def __init__(self, owner: "CacheBlock", values=()):
        super().__init__(values)
        self._owner = owner
        self._deferred = None      # zero-argument callable returning the (key, value) pairs still to be merged
        self._deferred_keys = frozenset()

    def _touch(self) -> None:
        self._owner._gdn_revision += 1

    def _sync(self) -> None:
        producer = self._deferred
        if producer is not None:
            self._deferred, self._deferred_keys = None, frozenset()
            super().update(producer())

    def defer(self, producer, keys) -> None:
        """Replace-or-add the entries ``producer()`` yields (their keys are ``keys``), lazily.  Counts
        as a mutation now.  An earlier deferred update that this one overwrites completely is dropped
        unbuilt; otherwise it goes in first, so that later entries win."""
        self._touch()
        keys = frozenset(keys)
        if self._deferred is not None and not self._deferred_keys <= keys:
            self._sync()
        self._deferred, self._deferred_keys = producer, keys

    def known_keys(self) -> set:
        """The dictionary's keys, pending ones included, without building anything."""
        return set(dict.keys(self)) | self._deferred_keys

    # -- reads: merge what is pending first
    def __getitem__(self, key):
        self._sync()
        return super().__getitem__(key)

    def get(self, key, default=None):
        self._sync()
        return super().get(key, default)

    def __contains__(self, key):
        self._sync()
        return super().__contains__(key)

    def __iter__(self):
        self._sync()
        return super().__iter__()

    def __len__(self):
        self._sync()
        return super().__len__()

    def keys(self):
        self._sync()
        return super().keys()

    def values(self):
        self._sync()
        return super().values()

    def items(self):
        self._sync()
        return super().items()

    def copy(self):
        self._sync()
        return dict(super().items())

    def __eq__(self, other):
        self._sync()
        return super().__eq__(other)

    def __ne__(self, other):
        return not self.__eq__(other)

    __hash__ = None

    def __repr__(self):
        self._sync()
        return super().__repr__()

    # -- mutations
    def __setitem__(self, key, value):
        self._touch()
        self._sync()
        super().__setitem__(key, value)

    def __delitem__(self, key):
        self._touch()
        self._sync()
        super().__delitem__(key)

    def clear(self):
        self._touch()
        self._deferred, self._deferred_keys = None, frozenset()
        super().clear()

    def pop(self, key, *default):
        self._touch()
        self._sync()
        return super().pop(key, *default)

    def popitem(self):
        self._touch()
        self._sync()
        return super().popitem()

    def update(self, *args, **kwargs):
        self._touch()
        self._sync()
        super().update(*args, **kwargs)

    def setdefault(self, key, default=None):
        self._sync()
        if not super().__contains__(key):
            self._touch()
        return super().setdefault(key, default)

    def __ior__(self, other):
        self.update(other)
        return self


class _PageList(list):
    """``CacheBlock.page_starts``: a plain list to its users (the reference appends to it, extends
    it, slices it, replaces it) that counts its mutations, so that planners can keep the page
    numbers of a block as an array between steps and notice when the list changed."""

    __slots__ = ("rev",)

    def __init__(self, values=()):
        super().__init__(values)
        self.rev = 0

    def _wrap(name):  # noqa: N805 - class-body helper
        base = getattr(list, name)

        def method(self, *args, **kwargs):
            self.rev += 1
            return base(self, *args, **kwargs)

        method.__name__ = name
        return method

    for _name in ("append", "extend", "insert", "pop", "remove", "clear", "sort", "reverse",
                  "__setitem__", "__delitem__", "__iadd__", "__imul__"):
        locals()[_name] = _wrap(_name)
    del _wrap, _name


class CacheBlock:
    """A paged, shareable run of KV cache (and GDN summaries) written by one coroutine.

    Attributes kept from the reference: ``block_id``, ``device``, ``page_size``,
    ``page_starts`` (page-start token slots, multiples of ``page_size``),
    ``num_tokens``, ``token_ids``, ``mrope_span_override``, ``linear_affine``
    (``{layer: (A_hat [1,H,dk,dk], B_hat [1,H,dv,dk])}``) and ``linear_conv_state``
    (``{layer: [conv_dim, k]}``).
    """

    _ids = itertools.count()

    def __init__(self, device: torch.device, page_size: int = 1):
        self.block_id = next(CacheBlock._ids)
        self.device = device
        self.page_size = int(page_size)
        self._page_starts = _PageList()
        self._page_cache = None       # (list identity, revision, page size, page numbers as int64 array)
        self.num_tokens = 0
        self.token_ids: List[int] = []
        self.mrope_span_override: Optional[int] = None
        self._gdn_revision = 0
        self._gdn_ptr_cache = None    # (revision, device, [layers, 2] summary addresses, tensors kept alive)
        self._gdn_conv_cache = None   # (revision, device, [layers] conv-state addresses, tensors kept alive)
        self._linear_affine: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = _TrackedDict(self)
        self._linear_conv_state: Dict[int, torch.Tensor] = _TrackedDict(self)

    # -- page list --------------------------------------------------------------
    @property
    def page_starts(self) -> List[int]:
        return self._page_starts

    @page_starts.setter
    def page_starts(self, values) -> None:
        self._page_starts = values if isinstance(values, _PageList) else _PageList(values)

    def page_numbers(self):
        """Page numbers (``page_start // page_size``) as an int64 array, cached until the list changes."""
        import numpy as np

        lst = self._page_starts
        c = self._page_cache
        if c is None or c[0] is not lst or c[1] != lst.rev or c[2] != self.page_size:
            arr = np.asarray(lst, dtype=np.int64) // self.page_size if len(lst) else np.zeros(0, np.int64)
            c = self._page_cache = (lst, lst.rev, self.page_size, arr)
        return c[3]

    # -- GDN state dictionaries -------------------------------------------------
    @property
    def linear_affine(self):
        return self._linear_affine

    @linear_affine.setter
    def linear_affine(self, value):
        self._gdn_revision += 1
        self._linear_affine = value

    @property
    def linear_conv_state(self):
        return self._linear_conv_state

    @linear_conv_state.setter
    def linear_conv_state(self, value):
        self._gdn_revision += 1
        self._linear_conv_state = value

    def _replace_linear_states(self, affine, conv) -> None:
        """Install new state dictionaries whose later mutations are tracked
        (minisgl/shared_cache/shared_block.py:96-99)."""
        self._gdn_revision += 1
        self._linear_affine = _TrackedDict(self, affine)
        self._linear_conv_state = _TrackedDict(self, conv)

    def invalidate_gdn_state(self) -> None:
        self._gdn_revision += 1

    # -- paging arithmetic ------------------------------------------------------
    @property
    def mrope_span(self) -> int:
        ov = self.mrope_span_override
        return self.num_tokens if ov is None else ov

    @property
    def num_pages(self) -> int:
        return len(self.page_starts)

    @property
    def last_page_len(self) -> int:
        if self.num_tokens == 0:
            return 0
        return self.num_tokens - (len(self.page_starts) - 1) * self.page_size

    @property
    def free_tail(self) -> int:
        return len(self.page_starts) * self.page_size - self.num_tokens

    @property
    def has_capacity(self) -> bool:
        return self.free_tail > 0

    def pages_needed(self, num_new_tokens: int) -> int:
        spill = num_new_tokens - self.free_tail
        return 0 if spill <= 0 else -(-spill // self.page_size)

    def slot_of(self, i: int) -> int:
        """Physical token slot of block-relative token ``i``."""
        return self.page_starts[i // self.page_size] + i % self.page_size

    def page_starts_tensor(self) -> torch.Tensor:
        return torch.tensor(self.page_starts, dtype=torch.int32, device=self.device)

    def page_numbers_tensor(self) -> torch.Tensor:
        return self.page_starts_tensor() // self.page_size

    def token_slots_tensor(self) -> torch.Tensor:
        if self.num_tokens == 0:
            return torch.empty(0, dtype=torch.int32, device=self.device)
        lane = torch.arange(self.page_size, dtype=torch.int32, device=self.device)
        grid = self.page_starts_tensor().unsqueeze(1) + lane.unsqueeze(0)
        return grid.reshape(-1)[: self.num_tokens]

    # -- writes -----------------------------------------------------------------
    def grow_pages(self, page_starts: torch.Tensor, num_new_tokens: int) -> None:
        """Record a prefill write of ``num_new_tokens`` tokens (tail of the last page
        first, then the fresh ``page_starts``)."""
        assert num_new_tokens > 0, "grow_pages needs at least one token"
        want = self.pages_needed(num_new_tokens)
        assert page_starts.numel() == want, (
            f"grow_pages got {page_starts.numel()} pages for {num_new_tokens} tokens "
            f"(free tail {self.free_tail}, page_size {self.page_size}); expected {want}"
        )
        self.page_starts += [int(s) for s in page_starts.tolist()]
        self.num_tokens += num_new_tokens

    def append_token(self, new_page_start: Optional[int]) -> None:
        """Record one decode write; ``new_page_start`` is given iff the last page is full."""
        if new_page_start is None:
            assert self.has_capacity, "append_token needs a new page but none was given"
        else:
            assert not self.has_capacity, "append_token got a new page but last page has room"
            self.page_starts.append(int(new_page_start))
        self.num_tokens += 1
        if self.mrope_span_override is not None:
            self.mrope_span_override += 1

    def clear(self) -> List[int]:
        """Empty the block; returns the page-start slots the caller must free."""
        released = list(self.page_starts)
        self.page_starts.clear()
        self.token_ids.clear()
        self.num_tokens = 0
        self.mrope_span_override = None
        self._linear_affine.clear()
        self._linear_conv_state.clear()
        self._gdn_revision += 1
        return released

    def __repr__(self) -> str:
        return (
            f"CacheBlock(id={self.block_id}, tokens={self.num_tokens}, "
            f"pages={self.num_pages}, page_size={self.page_size})"
        )


def block_page_numbers(block):
    """Page numbers (``page_start // page_size``) of any block-like object as an int64 array.

    Blocks of this package keep the array between steps (``CacheBlock.page_numbers``); any other
    object with the reference's public attributes (``page_starts``, ``page_size`` --
    minisgl/shared_cache/shared_block.py:24-60) is read through those, so the planners also take
    the reference's own ``CacheBlock``."""
    cached = getattr(block, "page_numbers", None)
    if cached is not None:
        return cached()
    import numpy as np

    starts = block.page_starts
    return np.asarray(starts, dtype=np.int64) // int(block.page_size) if len(starts) else np.zeros(0, np.int64)


SharedBlock = CacheBlock
CacheView = List[CacheBlock]


@dataclass
class AsyncContext:
    """One coroutine's decoding context: the view it reads and the block it writes.

    ``output_block`` defaults to the last block of ``cache_view``; a write block
    outside the view is allowed (the coroutine still attends to its own new token).
    """

    cache_view: CacheView = field(default_factory=list)
    output_block: CacheBlock = None  # type: ignore[assignment]
    next_input_id: Optional[int] = None

    def __post_init__(self) -> None:
        if self.output_block is None:
            assert self.cache_view, "AsyncContext needs a cache_view or an explicit output_block"
            self.output_block = self.cache_view[-1]

    @property
    def num_cached_tokens(self) -> int:
        return sum(b.num_tokens for b in self.cache_view)


class WorkerGroup:
    """The coroutines decoded together in one step.

    Accepts either a sequence of ``AsyncContext`` or the keyword pair
    ``cache_structure=`` / ``write_to=``.  Two workers writing one block in the
    same step raise ``ValueError`` (minisgl/shared_cache/worker_group.py:53-57).
    """

    def __init__(
        self,
        workers: Optional[Sequence[AsyncContext]] = None,
        *,
        cache_structure: Optional[Sequence[Sequence[CacheBlock]]] = None,
        write_to: Optional[Sequence[CacheBlock]] = None,
    ):
        if workers is None:
            assert cache_structure is not None, "WorkerGroup needs workers or cache_structure"
            views = [list(v) for v in cache_structure]
            targets = [v[-1] for v in views] if write_to is None else list(write_to)
            assert len(targets) == len(views)
            workers = [AsyncContext(cache_view=v, output_block=t) for v, t in zip(views, targets)]
        else:
            assert cache_structure is None and write_to is None, (
                "pass either workers or cache_structure/write_to, not both"
            )
        self.workers: List[AsyncContext] = list(workers)
        writers = [id(c.output_block) for c in self.workers]
        if len(set(writers)) != len(writers):
            raise ValueError("WorkerGroup has two workers writing the same block in one step")

    def __getitem__(self, key: Union[int, slice]):
        picked = self.workers[key]
        return WorkerGroup(picked) if isinstance(key, slice) else picked

    def __len__(self) -> int:
        return len(self.workers)

    def __iter__(self) -> Iterator[AsyncContext]:
        return iter(self.workers)

    @property
    def num_workers(self) -> int:
        return len(self.workers)

    @property
    def cache_structure(self) -> List[List[CacheBlock]]:
        return [list(c.cache_view) for c in self.workers]

    @property
    def write_to(self) -> List[CacheBlock]:
        return [c.output_block for c in self.workers]

    def worker_cache_length(self, worker_idx: int) -> int:
        return self.workers[worker_idx].num_cached_tokens

    def max_cache_length(self) -> int:
        return max((c.num_cached_tokens for c in self.workers), default=0)

    def __repr__(self) -> str:
        distinct = {id(b) for c in self.workers for b in c.cache_view}
        return f"WorkerGroup(workers={self.num_workers}, blocks={len(distinct)})"
