"""Plain (view-less) paged attention behind the host framework's attention-backend plugin interface.

The reference routes every forward that carries no cache view -- ``prefill_block`` without context,
ordinary scheduler batches -- through ``ctx.attn_backend`` (minisgl/layers/attention.py:62-65,
minisgl/shared_cache/session.py:1153-1170), an object implementing ``BaseAttnBackend``
(minisgl/attention/base.py:18-35) that is chosen by name from ``SUPPORTED_ATTENTION_BACKENDS``
(minisgl/attention/__init__.py:15-68).  Its stock implementations construct FlashInfer / TensorRT-LLM
wrappers (minisgl/attention/fi.py:80-188).  ``B200AttnBackend`` implements the same interface on
the kernels of this package, so that an engine started with ``attention_backend="b200"`` constructs
no third-party attention object at all:

* queries and keys arrive ROTATED (the layer applied its rotary embedding), so nothing is rotated
  here: the attention op below is built without a cos/sin table and the kernels multiply by the
  identity row;
* a request's keys sit at arbitrary token slots ``page_table[table_idx, :device_len]`` -- paging
  with page size 1, exactly how the stock backends read the pool (fi.py:176-180);
* a prefill / extend / mixed batch is a batched view prefill whose requests have no context block
  (causal, end-aligned over prefix + new tokens: dense tcgen05 tiles); a decode batch is a decode
  step whose views hold one block each (streaming split-K lanes).

The page table is read on the host once per ``prepare_metadata`` (one device-to-host copy of the
rows in use): the planners of this package are host planners.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from .attention_base import BaseAttnBackend, BaseAttnMetadata
from .blocks import AsyncContext, WorkerGroup
from .view_attention import (PrefillSpec, SharedCacheAttention, SharedCacheAttnMetadata,
                             SharedDecodeAttentionBuffers)


class _SlotPool:
    """The pool seen with page size 1: ``[num_slots, 1, Hkv, D]`` views of the same memory."""

    def __init__(self, kv_cache):
        self._inner = kv_cache
        self._pool_structs: Dict = {}
        self.device, self.dtype, self.num_layers = kv_cache.device, kv_cache.dtype, kv_cache.num_layers

    def _flat(self, cache: torch.Tensor) -> torch.Tensor:
        return cache.view(-1, 1, cache.shape[-2], cache.shape[-1])

    def k_cache(self, index: int) -> torch.Tensor:
        return self._flat(self._inner.k_cache(index))

    def v_cache(self, index: int) -> torch.Tensor:
        return self._flat(self._inner.v_cache(index))

    def store_kv(self, k, v, out_loc, layer_id) -> None:
        self._inner.store_kv(k, v, out_loc, layer_id)


class _SlotRun:
    """A request's cached tokens as a block of one-token pages (what the planners read of a block)."""

    __slots__ = ("page_starts", "num_tokens", "page_size", "mrope_span_override")

    def __init__(self, slots: np.ndarray, num_tokens: int):
        self.page_starts = slots
        self.num_tokens = int(num_tokens)
        self.page_size = 1
        self.mrope_span_override = None

    @property
    def mrope_span(self) -> int:
        return self.num_tokens


@dataclass
class B200AttnMetadata(BaseAttnMetadata):
    inner: SharedCacheAttnMetadata
    last: torch.Tensor

    def get_last_indices(self, bs: int) -> torch.Tensor:
        return self.last[:bs]


class B200AttnBackend(BaseAttnBackend):
    """``BaseAttnBackend`` on the cache-view kernels (see the module docstring).

    ``config`` needs ``num_qo_heads``, ``num_kv_heads`` and ``head_dim``; ``kv_cache`` is the engine's
    pool (``BaseKVCachePool`` accessors) and ``page_table`` its ``[tables, max_len]`` int32 token-slot
    table.  ``page_table`` may also be a zero-argument callable returning the table (the engine
    creates it after the backend).
    """

    def __init__(self, config, kv_cache, page_table, *, dense_engine: Optional[str] = None) -> None:
        self.config = config
        self.kvcache = kv_cache
        self._page_table = page_table
        self.device = torch.device(kv_cache.device)
        self.num_qo_heads = int(config.num_qo_heads)
        self.num_kv_heads = int(config.num_kv_heads)
        self.head_dim = int(config.head_dim)
        self.op = SharedCacheAttention(_SlotPool(kv_cache), None, self.num_qo_heads, self.num_kv_heads,
                                       self.head_dim, 1, kv_cache.dtype, self.device, dense_engine=dense_engine)
        self.capture_bs: List[int] = []
        self.max_seq_len = 0
        self.graph_buffers: Dict[int, SharedDecodeAttentionBuffers] = {}

    # ------------------------------------------------------------------ planning
    def _table(self) -> torch.Tensor:
        return self._page_table() if callable(self._page_table) else self._page_table

    def _slot_rows(self, reqs) -> List[np.ndarray]:
        """Token slots ``page_table[table_idx, :device_len]`` of every request, on the host."""
        table = self._table()
        longest = max(int(r.device_len) for r in reqs)
        idx = torch.tensor([int(r.table_idx) for r in reqs], dtype=torch.int64, device=table.device)
        rows = table.index_select(0, idx)[:, :longest].to("cpu").numpy().astype(np.int64, copy=False)
        return [rows[i, : int(r.device_len)] for i, r in enumerate(reqs)]

    def _plan(self, batch, graph_buffers=None) -> B200AttnMetadata:
        reqs = batch.padded_reqs
        rows = self._slot_rows(reqs)
        if all(int(r.extend_len) == 1 for r in reqs) and batch.is_decode:
            runs = [_SlotRun(s[: int(r.cached_len)], int(r.cached_len)) for s, r in zip(rows, reqs)]
            group = WorkerGroup([AsyncContext(cache_view=[b], output_block=b) for b in runs])
            new_slots = torch.tensor([int(s[int(r.cached_len)]) for s, r in zip(rows, reqs)], dtype=torch.int32)
            pending = {id(b): int(slot) for b, slot in zip(runs, new_slots.tolist())}   # page size 1: always a new page
            inner = self.op.prepare(group, pending, new_slots, graph_buffers=graph_buffers)
            last = torch.arange(len(reqs), device=self.device)
        else:
            specs = [PrefillSpec([], torch.from_numpy(s), int(r.extend_len), int(r.cached_len), None)
                     for s, r in zip(rows, reqs)]
            inner = self.op.prepare_prefill_batch(specs)
            last = inner.last_indices
        return B200AttnMetadata(inner=inner, last=last)

    def prepare_metadata(self, batch) -> None:
        batch.attn_metadata = self._plan(batch)

    # ------------------------------------------------------------------ forward
    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layer_id: int, batch) -> torch.Tensor:
        """``q [rows, Hq, D]`` (or ``[rows, Hq*D]``), ``k``/``v [rows, Hkv*D]``, all rotated by the caller;
        stores k/v at ``batch.out_loc`` and returns ``[rows, Hq*D]`` (minisgl/attention/fi.py:176-188)."""
        meta = batch.attn_metadata
        assert isinstance(meta, B200AttnMetadata)
        if not q.is_cuda:
            raise RuntimeError("the B200 attention backend needs CUDA tensors: there is no CPU fallback")
        self.kvcache.store_kv(k, v, batch.out_loc, layer_id)
        return self.op._attend(q.reshape(q.shape[0], -1), meta.inner, layer_id)

    # ------------------------------------------------------------------ CUDA-graph hooks
    def init_capture_graph(self, max_seq_len: int, bs_list: List[int]) -> None:
        """Fixed-capacity decode tables for every batch size a graph will be captured for
        (minisgl/attention/fi.py:222-229; driven by minisgl/engine/graph.py:118-212)."""
        assert not self.capture_bs, "Capture already initialized."
        self.capture_bs = sorted(bs_list)
        self.max_seq_len = int(max_seq_len)
        for bs in self.capture_bs:
            self.graph_buffers[bs] = SharedDecodeAttentionBuffers(self.op, bs, 1, bs * self.max_seq_len)
        self.op.prepare_workspace(tuple(self.graph_buffers.values()))

    def prepare_for_capture(self, batch) -> None:
        bs = batch.size
        assert bs in self.graph_buffers, f"no graph buffers for batch size {bs}"
        batch.attn_metadata = self._plan(batch, graph_buffers=self.graph_buffers[bs])

    def prepare_for_replay(self, batch) -> None:
        bs = batch.padded_size
        assert bs in self.graph_buffers, f"no graph buffers for batch size {bs}"
        batch.attn_metadata = self._plan(batch, graph_buffers=self.graph_buffers[bs])


def register(name: str = "b200") -> bool:
    """Register ``B200AttnBackend`` under ``name`` in the host framework's backend registry
    (``SUPPORTED_ATTENTION_BACKENDS``, minisgl/attention/__init__.py:15-40), taking the pool and the
    page table from its global context as the stock backends do (minisgl/attention/fi.py:88,197).
    Returns False when the host framework is not importable."""
    try:
        from minisgl.attention import SUPPORTED_ATTENTION_BACKENDS
        from minisgl.core import get_global_ctx
    except Exception:   # noqa: BLE001 -- the host framework is optional
        return False

    if name in SUPPORTED_ATTENTION_BACKENDS.supported_names():
        return True

    def create_b200_backend(config):
        ctx = get_global_ctx()
        return B200AttnBackend(config, ctx.kv_cache, lambda: get_global_ctx().page_table)

    SUPPORTED_ATTENTION_BACKENDS.register(name)(create_b200_backend)
    return True


__all__ = ["B200AttnBackend", "B200AttnMetadata", "register"]
