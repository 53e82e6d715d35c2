"""Cache-view attention: host planner + the one-call-per-layer forward.

Drop-in for the reference ``SharedCacheAttention`` (minisgl/shared_cache/attention.py:135-752):
same constructor, ``prepare`` / ``prepare_prefill_batch`` / ``forward`` / ``_rope`` signatures,
same metadata fields (``sub_worker``, ``sub_loc``, ``pad_slot``, ``n_main``, ``n_aux``, ...), so a
model layer that calls ``batch.attn_metadata.shared_cache_op.forward(q, k, v, layer_id, batch)``
(minisgl/layers/attention.py:57-60) runs unchanged.

What differs is below the seam.  The reference materialises one rotated query copy per
(worker, segment), runs one paged-attention call per wrapper and merges with a third kernel;
here the planner emits a device work list and ``forward`` makes two C calls per layer:
``va_store_kv`` (rotate K at its block-relative position, scatter K and V) and ``va_view_decode``
(walk the view's page tables, rotate Q per segment inside the kernel, merge).

The planner still computes the reference's per-sub-request tables -- they define the semantics
(post-append lengths, pending pages, implicit self segment) and are what the bit-exact index
tests compare -- and derives the device work list from them.
"""

from __future__ import annotations

import ctypes as C
import itertools
import os
from types import SimpleNamespace
from dataclasses import dataclass, field
from typing import Dict, List, Literal, Optional, Sequence

import numpy as np
import torch

from . import _lib
from .attention_base import BaseAttnMetadata
from .blocks import CacheBlock, WorkerGroup, block_page_numbers
from .kvpool import pool_struct, store_rows

DENSE_ENGINES = {"mma_sync": 0, "tcgen05": 1}
_NO_PAGES = np.zeros(0, np.int64)
_NO_PAGES32 = np.zeros(0, np.int32)
MIN_ITEM_KEYS = 128   # a lane's quota never drops below this many keys
CUT_SLACK_KEYS = 48   # a lane cut this close to a segment boundary is dropped


@dataclass
class HostTables:
    """The integer tables the reference hands to its paged-attention planner, kept on the host.

    ``main_*`` describe the paged sub-requests in reference order (worker-major), ``aux_*`` the
    single-token implicit-self sub-requests (minisgl/shared_cache/attention.py:326-368).
    """

    main_indices: List[int] = field(default_factory=list)
    main_indptr: List[int] = field(default_factory=lambda: [0])
    main_seq_lens: List[int] = field(default_factory=list)
    main_last_page_len: List[int] = field(default_factory=list)
    aux_slots: List[int] = field(default_factory=list)
    # prefill: (ctx, self) x (qo_indptr, kv_indptr, kv_indices, seq_lens, last_page_len)
    extra: Dict[str, List[int]] = field(default_factory=dict)


@dataclass
class SharedCacheAttnMetadata(BaseAttnMetadata):
    shared_cache_op: "SharedCacheAttention"
    sub_worker_list: Optional[Sequence[int]]   # None until first read for a batched prefill
    sub_loc_list: Optional[Sequence[int]]
    pad_slot_list: Optional[Sequence[int]]
    num_workers: int
    max_segments: int
    n_main: int = 0
    n_aux: int = 0
    n_ctx_rows: int = 0
    last_indices: Optional[torch.Tensor] = None
    phase: Literal["decode", "prefill_batch"] = "decode"
    _tables: Optional[HostTables] = field(default=None, repr=False)
    _table_recipe: object = field(default=None, repr=False)
    plan: object = field(default=None, repr=False)
    graph_buffers: object = field(default=None, repr=False)
    _pos32: Optional[torch.Tensor] = field(default=None, repr=False)
    _loc32: Optional[torch.Tensor] = field(default=None, repr=False)
    _lists_recipe: object = field(default=None, repr=False)

    def _ensure_prefill_lists(self) -> None:
        """Per-row tables of a batched prefill in the reference's shape (attention.py:505-547):
        one (row, segment) sub-request per new token and segment, context segments of all
        requests first, then the self segments.  Built on first access; the kernels read the tile /
        segment tables instead."""
        if self._lists_recipe is None or self.sub_worker_list is not None:
            return
        snapshot, page_pool, widest, P, q_pos3 = self._lists_recipe
        ex: Dict[str, List[int]] = {k: [] for k in (
            "ctx_qo_indptr", "ctx_kv_indptr", "ctx_kv_indices", "ctx_seq_lens", "ctx_last_page_len",
            "self_qo_indptr", "self_kv_indptr", "self_kv_indices", "self_seq_lens", "self_last_page_len")}
        for key in ("ctx_qo_indptr", "ctx_kv_indptr", "self_qo_indptr", "self_kv_indptr"):
            ex[key].append(0)
        ctx_rows, ctx_slot, ctx_loc, self_rows, self_slot, self_loc, tok = [], [], [], [], [], [], []
        offset = 0
        for S, T, T_span, start, ctx_snap, own_off, own_n in snapshot:
            rows = range(offset, offset + S)
            tok.extend(range(S))
            before = 0
            for j, (run, n_pages, n_tokens, last_len, span) in enumerate(ctx_snap):
                shift = start - before
                ctx_rows.extend(rows)
                ctx_slot.extend([j] * S)
                ctx_loc.extend(range(shift, shift + S))
                ex["ctx_kv_indices"].extend(page_pool[run: run + n_pages].tolist())
                ex["ctx_kv_indptr"].append(ex["ctx_kv_indptr"][-1] + n_pages)
                ex["ctx_qo_indptr"].append(ex["ctx_qo_indptr"][-1] + S)
                ex["ctx_seq_lens"].append(n_tokens)
                ex["ctx_last_page_len"].append(last_len)
                before += span
            total = T + S
            self_rows.extend(rows)
            self_slot.extend([len(ctx_snap)] * S)
            self_loc.extend(range(T_span, T_span + S))
            ex["self_kv_indices"].extend(page_pool[own_off: own_off + own_n].tolist())
            ex["self_kv_indptr"].append(ex["self_kv_indptr"][-1] + own_n)
            ex["self_qo_indptr"].append(ex["self_qo_indptr"][-1] + S)
            ex["self_seq_lens"].append(total)
            ex["self_last_page_len"].append(total - (own_n - 1) * P)
            offset += S
        gather = ctx_rows + self_rows
        slot = ctx_slot + self_slot
        sub_loc = ctx_loc + self_loc
        if q_pos3 is not None:
            # the reference's [3, n] form: per-axis position + the segment's offset, where the
            # scalar list holds token index + offset
            rows_np = np.asarray(gather, np.int64)
            tok_np = np.asarray(tok, np.int64)
            sub_loc = q_pos3[:, rows_np].astype(np.int64) + (np.asarray(sub_loc, np.int64) - tok_np[rows_np])[None, :]
        self.sub_worker_list = gather
        self.sub_loc_list = sub_loc
        self.pad_slot_list = [r * widest + s_ for r, s_ in zip(gather, slot)]
        self._tables = HostTables(extra=ex)

    @property
    def tables(self) -> HostTables:
        """The reference's paged-attention tables of this step (built on first access: the
        kernels read the work list instead)."""
        self._ensure_prefill_lists()
        if self._tables is None:
            t = HostTables()
            if self._table_recipe is not None:
                sub_blk, sub_len, run_len, page_pool, aux_kv, P = self._table_recipe
                run_off = np.concatenate(([0], np.cumsum(run_len)))
                for bi, length in zip(sub_blk.tolist(), sub_len.tolist()):
                    pages = page_pool[run_off[bi]: run_off[bi + 1]].tolist()
                    t.main_indices.extend(pages)
                    t.main_indptr.append(t.main_indptr[-1] + len(pages))
                    t.main_seq_lens.append(length)
                    t.main_last_page_len.append(length - (len(pages) - 1) * P)
                t.aux_slots = aux_kv.tolist()
            self._tables = t
        return self._tables

    # The reference exposes these as device int64 tensors; the kernels here never read them, so
    # they are built on first access only.
    def _dev(self, values) -> torch.Tensor:
        return torch.tensor(values, dtype=torch.int64, device=self.shared_cache_op.device)

    @property
    def sub_worker(self) -> torch.Tensor:
        self._ensure_prefill_lists()
        return self._dev(self.sub_worker_list)

    @property
    def sub_loc(self) -> torch.Tensor:
        self._ensure_prefill_lists()
        return self._dev(self.sub_loc_list)

    @property
    def pad_slot(self) -> torch.Tensor:
        self._ensure_prefill_lists()
        return self._dev(self.pad_slot_list)

    def get_last_indices(self, bs: int) -> torch.Tensor:
        if self.phase == "prefill_batch":
            assert self.last_indices is not None
            return self.last_indices
        return torch.arange(bs, device=self.shared_cache_op.device)


@dataclass
class PrefillSpec:
    """One request of a batched view-conditioned prefill (same fields as the reference's
    ``PrefillSpec``, minisgl/shared_cache/attention.py:98-115)."""

    context: List[CacheBlock]
    self_page_starts: torch.Tensor
    num_new: int
    self_prefix_len: int = 0
    self_prefix_span: Optional[int] = None
    mrope_rel: Optional[torch.Tensor] = None


@dataclass
class DecodePlan:
    """Device work list of one decode step (see ``VaDecodePlan`` in the C header)."""

    blob: torch.Tensor            # int32 device tensor holding every table
    host_blob: torch.Tensor       # pinned source of the async upload (kept alive)
    struct: _lib.VaDecodePlan
    num_items: int
    host: Dict[str, np.ndarray]   # host copies of the tables (tests, debugging)
    num_partials: int = 0
    groups: Optional["DensePlan"] = None   # dense tiles of blocks read by many workers


@dataclass
class DensePlan:
    """Device tables of a dense-tile launch (see ``VaDensePlan`` in the C header)."""

    blob: torch.Tensor
    host_blob: torch.Tensor
    struct: _lib.VaDensePlan
    host: Dict[str, np.ndarray]


# VIEWATTN_FORK_DENSE=0 keeps the dense tiles of a decode step behind the store kernel (comparisons)
FORK_DENSE_EARLY = os.environ.get("VIEWATTN_FORK_DENSE", "1") != "0"


class _ViewTopology:
    """Flattened structure of a worker group's views: valid while the same blocks sit in the same
    views with the same write blocks, whatever their lengths and page lists do meanwhile."""

    __slots__ = ("key", "blocks", "index", "targets", "view_blk", "view_start", "aux_w", "aux_w_np",
                 "written_flag", "subs", "written_max_readers")

    def __init__(self, key, workers, written):
        self.key = key
        blocks: List[CacheBlock] = []
        index: Dict[int, int] = {}
        view_blk: List[int] = []
        view_start = [0]
        aux_w: List[int] = []
        for w, ctx in enumerate(workers):
            target = ctx.output_block
            inside = False
            for b in ctx.cache_view:
                bi = index.get(id(b))
                if bi is None:
                    bi = index[id(b)] = len(blocks)
                    blocks.append(b)
                view_blk.append(bi)
                inside = inside or b is target
            view_start.append(len(view_blk))
            if not inside:
                aux_w.append(w)
        self.blocks, self.index = blocks, index
        self.targets = [ctx.output_block for ctx in workers]   # keeps the ids in `key` alive
        self.view_blk = np.asarray(view_blk, np.int32)
        self.view_start = np.asarray(view_start, np.int32)
        self.aux_w = aux_w
        self.aux_w_np = np.asarray(aux_w, np.int32)
        self.written_flag = np.fromiter((id(b) in written for b in blocks), np.int32, len(blocks))
        # how many views read the most widely read block that is written this step: the dense tiles of
        # a step only depend on the step's new keys if such a block is read widely enough to be tiled
        readers = np.bincount(self.view_blk, minlength=len(blocks)) if len(view_blk) else np.zeros(len(blocks), np.int64)
        self.written_max_readers = int((readers * self.written_flag).max()) if len(blocks) else 0
        self.subs = np.empty((5, max(len(view_blk) + len(aux_w), 1)), np.int32)   # filled by the planner


class SharedDecodeAttentionBuffers:
    """Fixed-capacity, address-stable decode plan for CUDA-graph replay.

    The counterpart of the reference's graph variant (minisgl/shared_cache/attention_graph.py:14-121):
    one capacity (``workers`` rows, views of at most ``depth`` blocks, ``max_pages`` page indices),
    every table at a fixed device address with fixed extents, so a graph captured once keeps
    working while the topology behind it changes.  ``prepare(..., graph_buffers=self)`` re-plans on
    the host and copies the new tables INTO these buffers; unused lanes, tiles and rows are empty
    ranges the kernels step over.  The split of the SMs between the streaming pass and the dense
    tiles is frozen at construction (``dense_fraction``), because the grid sizes are part of the
    captured launches.  Exceeding a capacity raises ``ValueError`` before anything is copied.
    """

    def __init__(self, attention: "SharedCacheAttention", workers: int, depth: int, max_pages: int,
                 dummy_slots=None, *, dense_fraction: float = 0.0):
        # positional arguments as the reference's class takes them (attention_graph.py:15; call site
        # minisgl/shared_cache/graph.py:90-91).  `dummy_slots` (the reference's padding targets) is
        # accepted and not needed: padding rows are empty ranges here and are never stored.
        a = self.attention = attention
        self.dummy_slots = dummy_slots
        self.workers, self.depth, self.max_pages = workers, depth, max_pages
        H = a.num_kv_heads
        if a.device.type == "cuda":
            lanes_max = a.lanes()
            width = _lib.lib().va_decode_lane_width(a.head_dim)
        else:
            lanes_max, width = getattr(a, "_lanes", None) or 592, getattr(a, "_lane_width", 1)
        n_sms = max(1, lanes_max // width)
        self.dense_sms = min(n_sms - 1, int(round(n_sms * dense_fraction))) if dense_fraction > 0 else 0
        self.stream_lanes = (n_sms - self.dense_sms) * width
        per_tile = a.tile_rows() // a.gqa
        self.cap_pages = max_pages + workers
        self.cap_items = workers * (depth + 1) * H + self.stream_lanes + 8
        self.cap_tiles = 4 * self.dense_sms + H * workers * max(2, depth) if self.dense_sms else 0
        self.cap_entries = self.cap_tiles * per_tile
        self.cap_partials = self.cap_items + self.cap_entries
        self.n_groups = workers * H
        sizes = [self.cap_pages, self.cap_items * _lib.VA_ITEM_WORDS, self.stream_lanes + 1, self.n_groups + 1,
                 self.cap_tiles * 8, self.cap_entries * 4, self.cap_tiles * 8]
        self.offs = [0]
        for sz in sizes:
            self.offs.append(self.offs[-1] + (-(-sz // 4) * 4))
        self.sizes = sizes
        on_gpu = a.device.type == "cuda"
        self.host = torch.zeros(max(self.offs[-1], 4), dtype=torch.int32, pin_memory=on_gpu)
        self.blob = self.host.to(a.device) if on_gpu else self.host
        base = self.blob.data_ptr()
        ptr = lambda i: base + 4 * self.offs[i]
        self.dense_struct = _lib.VaDensePlan()
        d = self.dense_struct
        d.page_indices, d.tiles, d.entries, d.segments = ptr(0), ptr(4), ptr(5), ptr(6)
        d.num_page_indices, d.num_tiles, d.num_entries, d.num_segments = (
            self.cap_pages, self.cap_tiles, self.cap_entries, self.cap_tiles)
        d.num_partials, d.num_rows, d.num_ctas = self.cap_partials, workers, self.dense_sms
        d.engine = DENSE_ENGINES[a.dense_engine]
        self.struct = _lib.VaDecodePlan()
        st = self.struct
        st.page_indices, st.items, st.lane_off, st.row_part_off = ptr(0), ptr(1), ptr(2), ptr(3)
        st.num_items, st.num_lanes, st.num_rows = self.cap_items, self.stream_lanes, workers
        st.num_partials, st.num_page_indices, st.phase_mask = self.cap_partials, self.cap_pages, 0
        st.groups = C.addressof(d) if self.cap_tiles else None
        if on_gpu:
            a._reserve_partials(self.cap_partials)
        self.event = torch.cuda.Event() if on_gpu else None

    def load(self, pages, items, lane_off, row_part_off, W, n_partials, dense, work) -> "DecodePlan":
        if W > self.workers:
            raise ValueError(f"decode batch of {W} workers exceeds the prepared capacity {self.workers}")
        if pages.size > self.cap_pages:
            raise ValueError(f"{pages.size} page indices exceed the prepared capacity {self.cap_pages}")
        if items.shape[0] > self.cap_items or n_partials > self.cap_partials:
            raise ValueError("decode plan exceeds the prepared item / partial capacity")
        if dense is not None and (dense[0].shape[0] > self.cap_tiles or dense[1].shape[0] > self.cap_entries):
            raise ValueError("shared-block tiles exceed the prepared capacity")
        if self.event is not None:
            self.event.synchronize()   # the previous upload has been consumed by the copy engine
        hv, o = self.host.numpy(), self.offs
        hv[o[0]: o[0] + pages.size] = pages
        hv[o[1]: o[1] + items.size] = items.reshape(-1)
        hv[o[2]: o[2] + lane_off.size] = lane_off
        full = np.full(self.n_groups + 1, row_part_off[-1], np.int32)   # rows beyond W: empty ranges
        full[: row_part_off.size] = row_part_off
        hv[o[3]: o[3] + full.size] = full
        hv[o[4]: o[5]] = 0                                               # unused tiles: zero entries
        if dense is not None:
            tiles, ent, seg = dense
            hv[o[4]: o[4] + tiles.size] = tiles.reshape(-1)
            hv[o[5]: o[5] + ent.size] = ent.reshape(-1)
            hv[o[6]: o[6] + seg.size] = seg.reshape(-1)
        if self.blob is not self.host:
            self.blob.copy_(self.host, non_blocking=True)
            self.event.record()
        # host-side record of what was loaded, read back from the staging buffer itself
        n_items = items.shape[0]
        work = dict(work, items=hv[o[1]: o[1] + n_items * _lib.VA_ITEM_WORDS].reshape(n_items, -1).copy(),
                    lane_off=hv[o[2]: o[2] + self.stream_lanes + 1].copy(),
                    row_part_off=hv[o[3]: o[3] + self.n_groups + 1].copy(),
                    page_indices=hv[o[0]: o[0] + pages.size].copy())
        groups = None
        if dense is not None:
            nt, ne = dense[0].shape[0], dense[1].shape[0]
            groups = SimpleNamespace(host={
                "tiles": hv[o[4]: o[4] + nt * 8].reshape(nt, 8).copy(),
                "entries": hv[o[5]: o[5] + ne * 4].reshape(ne, 4).copy(),
                "segments": hv[o[6]: o[6] + dense[2].size].reshape(-1, 8).copy(),
                "page_indices": work["page_indices"]})
        return DecodePlan(blob=self.blob, host_blob=self.host, struct=self.struct, num_items=n_items,
                          host=work, num_partials=n_partials, groups=groups)


class SharedPrefillAttentionBuffers:
    """Fixed-capacity, address-stable tables of a batched view prefill for CUDA-graph replay.

    Same constructor as the reference's class (minisgl/shared_cache/attention_graph.py:124-167):
    ``workers`` requests at most, each reading at most ``depth`` context blocks, ``rows`` query rows
    in total, ``max_pages`` page indices.  ``prepare_prefill_batch(specs, graph_buffers=self)``
    plans on the host and copies the tile / entry / segment tables INTO these buffers; unused
    tiles have no entries and are stepped over, and output rows beyond the planned batch are not
    written.  ``dummy_slots`` (the reference's padding targets) is accepted and not needed: rows
    without a tile are never stored through the attention tables.
    """

    def __init__(self, attention: "SharedCacheAttention", workers: int, depth: int, rows: int, max_pages: int,
                 dummy_slots=None):
        a = self.attention = attention
        self.workers, self.depth, self.rows, self.max_pages = workers, depth, rows, max_pages
        per_tile = a.tile_rows() // a.gqa
        self.cap_tiles = (-(-rows // per_tile) + workers) * a.num_kv_heads
        self.cap_entries = rows
        self.cap_segments = workers * (depth + 1)
        self.cap_pages = max_pages
        # with interleaved mRoPE the captured launch is the per-axis instantiation: the rows' (time, height,
        # width) positions live in a fixed [3, rows] region (token index on all axes for text batches)
        self.with_axes = a.mrope_section is not None and a.dense_engine == "tcgen05"
        self.sizes = [self.cap_pages, self.cap_tiles * 8, self.cap_entries * 4, self.cap_segments * 8,
                      3 * rows if self.with_axes else 0]
        self.offs = [0]
        for sz in self.sizes:
            self.offs.append(self.offs[-1] + (-(-sz // 4) * 4))
        on_gpu = a.device.type == "cuda"
        self.host = torch.zeros(max(self.offs[-1], 4), dtype=torch.int32, pin_memory=on_gpu)
        self.blob = self.host.to(a.device) if on_gpu else self.host
        base = self.blob.data_ptr()
        st = self.struct = _lib.VaDensePlan()
        st.page_indices, st.tiles, st.entries, st.segments = (base + 4 * o for o in self.offs[:4])
        st.num_page_indices, st.num_tiles, st.num_entries, st.num_segments = (
            self.cap_pages, self.cap_tiles, self.cap_entries, self.cap_segments)
        st.num_partials, st.num_rows, st.num_ctas = 0, rows, 0
        st.engine = DENSE_ENGINES[a.dense_engine]
        if self.with_axes:
            st.q_pos3 = base + 4 * self.offs[4]
            st.mrope_lim_h, st.mrope_lim_w = a._mrope_lims
        self.event = torch.cuda.Event() if on_gpu else None

    def load(self, pages, tile_arr, entries, seg_arr, n_rows, q_pos3=None) -> "DensePlan":
        if n_rows > self.rows:
            raise ValueError(f"{n_rows} query rows exceed the prepared capacity {self.rows}")
        if pages.size > self.cap_pages:
            raise ValueError(f"{pages.size} page indices exceed the prepared capacity {self.cap_pages}")
        if tile_arr.shape[0] > self.cap_tiles or seg_arr.shape[0] > self.cap_segments:
            raise ValueError("prefill plan exceeds the prepared tile / segment capacity")
        if self.event is not None:
            self.event.synchronize()   # the previous upload has left the staging buffer
        hv, o = self.host.numpy(), self.offs
        hv[o[1]: o[2]] = 0             # unused tiles: zero entries
        for off, arr in zip(o, (pages, tile_arr, entries, seg_arr)):
            hv[off: off + arr.size] = arr.reshape(-1)
        if self.with_axes:
            axes = hv[o[4]: o[4] + 3 * self.rows].reshape(3, self.rows)   # [3, rows] with the capacity's row stride
            axes[:] = 0
            axes[:, :n_rows] = q_pos3 if q_pos3 is not None else entries[:n_rows, 1][None, :]
        elif q_pos3 is not None:
            raise NotImplementedError("these buffers were built without per-axis query positions")
        if self.blob is not self.host:
            self.blob.copy_(self.host, non_blocking=True)
            self.event.record()
        return DensePlan(blob=self.blob, host_blob=self.host, struct=self.struct,
                         host={"page_indices": pages, "tiles": tile_arr, "entries": entries, "segments": seg_arr})


class SharedCacheAttention:
    """Owns the scratch buffers and runs cache-view attention through the C ABI."""

    def __init__(
        self,
        kv_cache,
        cos_sin_cache: torch.Tensor,
        num_qo_heads: int,
        num_kv_heads: int,
        head_dim: int,
        page_size: int,
        dtype: torch.dtype,
        device: torch.device,
        rotary_dim: Optional[int] = None,
        mrope_section: Optional[tuple] = None,
        rope_base: Optional[float] = None,
        *,
        dense_engine: Optional[str] = None,
    ) -> None:
        if mrope_section is not None and rope_base is None:
            raise ValueError("mrope_section needs rope_base (the rotation is defined by its frequencies)")
        if dtype != torch.bfloat16:
            raise ValueError("the B200 view-attention kernels compute in bfloat16")
        self.kv_cache = kv_cache
        self.num_qo_heads = num_qo_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        # Interleaved mRoPE (minisgl/shared_cache/attention.py:164-174): keys are rotated with 3-axis
        # positions and the reference's bf16 arithmetic (va_store_kv_mrope / va_mrope_rotate);
        # queries only ever carry one position for all axes (a segment distance) and are rotated
        # inside the attention kernels from the table below, in fp32.
        self.mrope_section = tuple(mrope_section) if mrope_section is not None else None
        self._mrope_lims = (0, 0)
        if self.mrope_section is not None:
            assert len(self.mrope_section) == 3 and sum(self.mrope_section) == self.rotary_dim // 2, \
                "mrope_section must split the rotary half into (time, height, width)"
            self._mrope_lims = (3 * int(self.mrope_section[1]), 3 * int(self.mrope_section[2]))
        self.page_size = page_size
        self.dtype = dtype
        self.device = torch.device(device)
        self.cos_sin_cache = cos_sin_cache
        self._cos_sin = None
        if mrope_section is not None:
            # row p = cos | sin of p * inv_freq, the angles the reference computes on the fly; as many
            # rows as the model's own table has positions
            max_pos = int(cos_sin_cache.shape[0]) if cos_sin_cache is not None else 32768
            rd = head_dim if rotary_dim is None else rotary_dim
            inv_freq = 1.0 / (rope_base ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))
            freqs = torch.arange(max_pos, dtype=torch.float32)[:, None] * inv_freq[None, :]
            self._cos_sin = torch.cat((freqs.cos(), freqs.sin()), dim=-1).to(self.device).contiguous()
        elif cos_sin_cache is not None:
            self._cos_sin = cos_sin_cache.to(device=self.device, dtype=torch.float32).contiguous()
            assert self._cos_sin.shape[1] == self.rotary_dim, "cos_sin_cache must be [max_pos, rotary_dim]"
        # which tensor-core path runs dense tiles (prefill, shared-block decode): the keyword argument,
        # else the VIEWATTN_DENSE_ENGINE environment variable, else tcgen05
        self.dense_engine = dense_engine or os.environ.get("VIEWATTN_DENSE_ENGINE", "tcgen05")
        if self.dense_engine not in DENSE_ENGINES:
            raise ValueError(f"dense_engine must be one of {sorted(DENSE_ENGINES)}")
        self._lanes: Optional[int] = None
        self._sm_count: Optional[int] = None
        self._topology: Optional[_ViewTopology] = None   # flattened views of the last planned group
        self._plan_params = _lib.VaPlanParams()
        self._plan_layout = _lib.VaPlanLayout()
        self._plan_step = _lib.VaViewStep()
        self._plan_subs = _lib.VaViewSubs()
        self._plan_dense_words = 0                       # most tile/entry/segment words a step needed
        self._partial_o: Optional[torch.Tensor] = None
        self._partial_ml: Optional[torch.Tensor] = None
        self._status: Optional[torch.Tensor] = None
        # kept for callers that read it (the reference exposes its FlashInfer workspace here)
        self._workspace = None

    # ------------------------------------------------------------------ utilities
    @property
    def gqa(self) -> int:
        return self.num_qo_heads // self.num_kv_heads

    def tile_rows(self) -> int:
        """Query rows one dense tile holds: the tcgen05 engine runs two 128-row streams per CTA at
        head_dim 128, every other case is one 128-row tile."""
        return 256 if (self.dense_engine == "tcgen05" and self.head_dim == 128) else 128

    def lanes(self) -> int:
        if self._lanes is None:
            n = _lib.lib().va_decode_lanes(self.head_dim)
            if n <= 0:
                _lib.check(n, "va_decode_lanes")
            self._lanes = n
        return self._lanes

    def status(self) -> torch.Tensor:
        if self._status is None:
            self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
        return self._status

    def check_status(self) -> None:
        """Read the device status word (synchronises); raises on a recorded device fault."""
        code = int(self.status().item())
        if code != 0:
            self._status.zero_()
            raise RuntimeError(f"view attention kernel reported {_lib.DEVICE_CODES.get(code, code)}")

    def prepare_workspace(self, profiles) -> None:
        """Reserve the split-K scratch of the largest profile before graph capture (no-op if none).

        A profile is a fixed-capacity buffer object (``SharedDecodeAttentionBuffers`` /
        ``SharedPrefillAttentionBuffers``), as in the reference
        (minisgl/shared_cache/attention.py:212-239): it must belong to this instance, and the call
        must come before capture."""
        profiles = tuple(profiles)
        if not profiles:
            return
        if self.device.type == "cuda" and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("Attention workspace must be prepared once before capture")
        if any(getattr(p, "attention", self) is not self for p in profiles):
            raise ValueError("Attention workspace profiles must belong to this instance")
        need = max(int(getattr(p, "cap_partials", 0) or getattr(p, "max_items", 0) or 0) for p in profiles)
        if need:
            self._reserve_partials(need)

    def _reserve_partials(self, n_items: int) -> None:
        cap = 0 if self._partial_o is None else self._partial_o.shape[0]
        if n_items > cap:
            if self.device.type == "cuda" and torch.cuda.is_current_stream_capturing():
                raise RuntimeError("Attention workspace must be prepared once before capture")
            new_cap = max(n_items, int(cap * 1.5), 1024)
            self._partial_o = torch.empty(new_cap, self.gqa, self.head_dim, dtype=torch.float32, device=self.device)
            self._partial_ml = torch.empty(new_cap, self.gqa, 2, dtype=torch.float32, device=self.device)

    def _rope(self, x: torch.Tensor, corrections: torch.Tensor) -> torch.Tensor:
        """RoPE delta rotation of ``x [N, heads, head_dim]`` by ``corrections [N]`` (signed)."""
        if not x.is_cuda:
            raise RuntimeError("_rope runs the CUDA rotation kernel; there is no CPU fallback")
        n, heads, d = x.shape
        out = torch.empty((n, heads, d), dtype=x.dtype, device=x.device)
        if n == 0:
            return out
        src = x.contiguous()
        if src.dtype != torch.bfloat16:
            # fp32/fp16 inputs (block merge re-rotation): rotate in bf16 storage is not the
            # reference's behaviour, so refuse rather than silently change precision
            raise NotImplementedError("_rope kernel handles bfloat16 activations")
        delta = corrections.to(device=x.device, dtype=torch.int32).contiguous()
        if self.mrope_section is not None:
            # [N] (one position for all axes) or [3, N]; the reference's bf16 arithmetic
            axes = 3 if delta.dim() == 2 else 1
            assert delta.shape[-1] == n and (axes == 1 or delta.shape[0] == 3)
            rc = _lib.lib().va_mrope_rotate(
                src.data_ptr(), out.data_ptr(), delta.data_ptr(), axes, n, heads, d, self.rotary_dim,
                self._cos_sin.data_ptr(), self._cos_sin.shape[0], *self._mrope_lims, _lib.stream_ptr(),
            )
            _lib.check(rc, "va_mrope_rotate")
            return out
        rc = _lib.lib().va_rope_rotate(
            src.data_ptr(), out.data_ptr(), delta.data_ptr(), n, heads, d, self.rotary_dim,
            self._cos_sin.data_ptr(), self._cos_sin.shape[0], _lib.stream_ptr(),
        )
        _lib.check(rc, "va_rope_rotate")
        return out

    # ------------------------------------------------------------------ decode planner
    def prepare(
        self,
        group: WorkerGroup,
        new_page_for_block: Dict[int, Optional[int]],
        new_token_slots: torch.Tensor,
        graph_buffers=None,
    ) -> SharedCacheAttnMetadata:
        """Plan one decode step.

        ``new_page_for_block`` maps ``id(write_block)`` to the page-start slot of a page
        allocated for this step's token (or None); its keys are the blocks written this step.
        ``new_token_slots [W]`` is each worker's destination slot.  Segment lengths are counted
        post-append, a pending page is visible to every reader of the block, empty blocks are
        skipped, and a worker whose write block is outside its view gets a one-token segment
        at distance 0 (minisgl/shared_cache/attention.py:282-448).
        """
        workers = group.workers
        W = len(workers)
        assert W > 0
        P = self.page_size
        written = new_page_for_block.keys()

        # The structure of the views (which blocks, in which order, who writes where) changes
        # rarely between decode steps; it is flattened once and reused while it stays the same.
        views = [c.cache_view for c in workers]
        key = (tuple(map(id, itertools.chain.from_iterable(views))), tuple(map(len, views)),
               tuple([id(c.output_block) for c in workers]), frozenset(written))
        topo = self._topology
        if topo is None or topo.key != key:
            topo = self._topology = _ViewTopology(key, workers, written)
        blocks = topo.blocks
        nb = len(blocks)
        for b in blocks:
            assert b.page_size == P, "blocks of one pool share its page size"

        # post-append token count and span of every distinct block
        tok = np.fromiter([b.num_tokens for b in blocks], np.int32, nb)
        overrides = [b.mrope_span_override for b in blocks]
        span = tok
        if overrides.count(None) != nb:
            span = np.fromiter([t if o is None else o for t, o in zip(tok.tolist(), overrides)], np.int32, nb)
        blk_len = tok + topo.written_flag
        blk_span = span + topo.written_flag

        # a worker whose write block is outside its view: one key at its new slot, distance = the
        # write block's span (minisgl/shared_cache/attention.py:326-368)
        aux_w = topo.aux_w
        n_aux = len(aux_w)
        if n_aux:
            slots_host = new_token_slots.cpu().tolist()
            aux_loc = np.asarray([topo.targets[w].mrope_span for w in aux_w], np.int32)
            aux_kv = np.asarray([int(slots_host[w]) for w in aux_w], np.int64)
        else:
            aux_loc, aux_kv = _NO_PAGES32, _NO_PAGES

        # page numbers of every non-empty distinct block, each block once, in one flat array (a
        # block keeps its page numbers as an array until its page list changes); a page allocated
        # for this step's token is the last page of its block's run
        lens = blk_len.tolist()
        runs = [block_page_numbers(b) if n else _NO_PAGES for b, n in zip(blocks, lens)]
        run_len = np.fromiter([r.size for r in runs], np.int32, nb)
        index = topo.index
        pending_page = None
        for bid, slot in new_page_for_block.items():
            if slot is not None:
                bi = index.get(bid)
                if bi is not None and lens[bi]:
                    if pending_page is None:
                        pending_page = np.full(nb, -1, np.int32)
                    pending_page[bi] = slot // P
        pages = np.concatenate(runs).astype(np.int32) if nb else _NO_PAGES32

        step = self._plan_step
        step.num_workers, step.num_blocks, step.num_aux, step.page_size = W, nb, n_aux, P
        step.view_start, step.view_block = topo.view_start.ctypes.data, topo.view_blk.ctypes.data
        step.block_len, step.block_span = blk_len.ctypes.data, blk_span.ctypes.data
        step.block_pages, step.pages = run_len.ctypes.data, pages.ctypes.data
        step.block_pending_page = pending_page.ctypes.data if pending_page is not None else None
        step.aux_worker, step.aux_loc, step.aux_slot = (topo.aux_w_np.ctypes.data, aux_loc.ctypes.data,
                                                        aux_kv.ctypes.data)
        subs = topo.subs
        info = self._plan_subs
        plan_fn = _lib.lib().va_plan_views
        plan = self._run_planner(
            lambda pp, blob_ptr, cap, lay: plan_fn(C.byref(pp), C.byref(step), blob_ptr, cap, C.byref(lay),
                                                   subs.ctypes.data, subs.shape[1], C.byref(info)),
            subs.shape[1], pages.size + nb + n_aux, W, graph_buffers)

        n_main, widest = info.num_main, info.max_segments
        n_sub = n_main + n_aux
        sub_out = subs[:, :n_sub].astype(np.int64)       # a copy: the next step reuses the buffer
        self._check_positions(int(sub_out[1].max()) if n_sub else 0, "a query's distance to a view block")
        meta = SharedCacheAttnMetadata(
            shared_cache_op=self,
            sub_worker_list=sub_out[0],
            sub_loc_list=sub_out[1],
            pad_slot_list=sub_out[0] * widest + sub_out[2],
            num_workers=W,
            max_segments=widest,
            n_main=n_main,
            n_aux=n_aux,
        )
        # the reference's paged-attention tables are only built when somebody reads them
        if pending_page is not None:
            run_len = run_len + (pending_page >= 0)
        meta._table_recipe = (sub_out[4, :n_main], sub_out[3, :n_main], run_len, plan.host["page_indices"], aux_kv, P)
        meta.plan = plan
        meta.graph_buffers = graph_buffers
        # the dense tiles may be launched before the step's keys are stored when no block they could
        # cover is written in the step; a plan that is re-made behind a captured graph keeps the
        # conservative order, because the launch order is part of the capture
        meta.fork_dense_early = (graph_buffers is None and plan.groups is not None
                                 and topo.written_max_readers < self.GROUP_MIN_READERS)
        if graph_buffers is not None:
            meta.num_workers = graph_buffers.workers
        return meta

    def _check_positions(self, largest: int, what: str) -> None:
        """The kernels clamp a rotation distance to the last row of the cos/sin table, as
        ``apply_rope_correction`` does (minisgl/shared_cache/rope_correction.py:36); a view longer
        than the table would be rotated wrongly without any signal, so the planners refuse it."""
        if self._cos_sin is not None and largest >= self._cos_sin.shape[0]:
            raise ValueError(f"{what} ({largest}) reaches beyond the RoPE table ({self._cos_sin.shape[0]} positions)")

    # Planner constants of the streaming / dense-tile split (per-SM key rates, keys per microsecond
    # for one (reader, kv head) unit resp. one (reader group, kv head) tile row), by head_dim.
    GROUP_MIN_READERS = 4
    GROUP_MIN_KEYS = 256     # shorter shared blocks are not worth a tile of their own
    DENSE_TILES_PER_CTA = 1  # key chunks are sized so that every dense CTA runs this many tiles
    STREAM_RATE = {256: 31.0, 128: 60.0}
    DENSE_RATE = {256: 10.0, 128: 25.0}          # mma.sync tiles
    DENSE_RATE_TCGEN05 = {256: 16.0, 128: 30.0}  # tcgen05 tiles, K/V rows gathered (pages of fewer than 8 tokens)
    DENSE_RATE_TCGEN05_TMA = {256: 20.0, 128: 30.0}  # tcgen05 tiles, whole pages fetched as TMA boxes

    def _run_planner(self, call, n_sub_bound: int, n_pages: int, W: int, buffers=None) -> DecodePlan:
        """Run a native planner entry point (``call(params, blob_ptr, blob_words, layout)``) into
        one pinned int32 blob and start its upload; ``n_sub_bound`` bounds the sub-requests."""
        H = self.num_kv_heads
        on_gpu = self.device.type == "cuda"
        if on_gpu:
            G_max = self.lanes()
            width = _lib.lib().va_decode_lane_width(self.head_dim)
        else:
            G_max = getattr(self, "_lanes", None) or 592
            width = getattr(self, "_lane_width", 1)
        if self.dense_engine != "tcgen05":
            rates = self.DENSE_RATE
        elif self.page_size % 8 == 0 and self.page_size <= 64:
            rates = self.DENSE_RATE_TCGEN05_TMA
        else:
            rates = self.DENSE_RATE_TCGEN05
        pp = self._plan_params
        pp.num_workers, pp.num_kv_heads = W, H
        pp.readers_per_tile = self.tile_rows() // self.gqa
        pp.num_sms, pp.lane_width = max(1, G_max // width), width
        pp.group_min_readers, pp.group_min_keys = self.GROUP_MIN_READERS, self.GROUP_MIN_KEYS
        pp.dense_tiles_per_cta = self.DENSE_TILES_PER_CTA
        pp.min_item_keys, pp.cut_slack_keys = MIN_ITEM_KEYS, CUT_SLACK_KEYS
        pp.fixed_stream_lanes = buffers.stream_lanes if buffers is not None else 0
        pp.fixed_dense_sms = buffers.dense_sms if buffers is not None else 0
        pp.stream_rate = self.STREAM_RATE.get(self.head_dim, 30.0)
        pp.dense_rate = rates.get(self.head_dim, 30.0)

        lanes_cap = pp.fixed_stream_lanes or G_max
        cap = n_pages + 8 * (n_sub_bound * H + lanes_cap) + lanes_cap + W * H + 64 + self._plan_dense_words
        lay = self._plan_layout
        while True:
            if buffers is None:
                host = torch.empty(cap, dtype=torch.int32, pin_memory=on_gpu)
                hv = host.numpy()
            else:
                host, hv = None, np.empty(cap, np.int32)   # staged again into the fixed tables below
            rc = call(pp, hv.ctypes.data, cap, lay)
            if rc != _lib.VA_ERR_CAPACITY or cap >= lay.total_words:
                break
            cap = int(lay.total_words)
        _lib.check(rc, "decode planner")
        dense_words = int(lay.total_words) - lay.off_tiles
        if dense_words > self._plan_dense_words:
            self._plan_dense_words = dense_words + dense_words // 2

        n_items, n_tiles, G = lay.num_items, lay.num_tiles, lay.num_lanes
        n_partials = lay.num_partials
        view = lambda off, n, cols=0: (hv[off: off + n] if not cols else hv[off: off + n * cols].reshape(n, cols))
        work = {
            "items": view(lay.off_items, n_items, _lib.VA_ITEM_WORDS),
            "lane_off": view(lay.off_lane_off, G + 1),
            "row_part_off": view(lay.off_row_part_off, lay.num_groups + 1),
            "page_indices": view(lay.off_pages, lay.num_pages),
            "quota": np.array([lay.quota]), "total_keys": np.array([lay.total_keys]),
            "dense_sms": np.array([lay.dense_sms]),
        }
        dense = None
        if n_tiles:
            dense = (view(lay.off_tiles, n_tiles, 8), view(lay.off_entries, lay.num_entries, 4),
                     view(lay.off_segments, lay.num_segments, 8))
        if buffers is not None:
            return buffers.load(work["page_indices"], work["items"], work["lane_off"], work["row_part_off"], W,
                                n_partials, dense, work)

        total = int(lay.total_words)
        blob = host[:total].to(self.device, non_blocking=True) if on_gpu else host
        base_ptr = blob.data_ptr()
        groups_plan = None
        if dense is not None:
            d = _lib.VaDensePlan()
            d.page_indices = base_ptr + 4 * lay.off_pages
            d.tiles = base_ptr + 4 * lay.off_tiles
            d.entries = base_ptr + 4 * lay.off_entries
            d.segments = base_ptr + 4 * lay.off_segments
            d.num_page_indices, d.num_tiles = lay.num_pages, n_tiles
            d.num_entries, d.num_segments = lay.num_entries, lay.num_segments
            d.num_partials, d.num_rows, d.num_ctas = n_partials, W, lay.dense_sms
            d.engine = DENSE_ENGINES[self.dense_engine]
            groups_plan = DensePlan(blob=blob, host_blob=host, struct=d,
                                    host={"page_indices": work["page_indices"], "tiles": dense[0],
                                          "entries": dense[1], "segments": dense[2]})
        st = _lib.VaDecodePlan()
        st.page_indices = base_ptr + 4 * lay.off_pages
        st.items = base_ptr + 4 * lay.off_items
        st.lane_off = base_ptr + 4 * lay.off_lane_off
        st.row_part_off = base_ptr + 4 * lay.off_row_part_off
        st.num_items, st.num_lanes, st.num_rows = n_items, G, W
        st.num_partials, st.num_page_indices, st.phase_mask = n_partials, lay.num_pages, 0
        st.groups = C.addressof(groups_plan.struct) if groups_plan is not None else None
        return DecodePlan(blob=blob, host_blob=host, struct=st, num_items=n_items, host=work,
                          num_partials=n_partials, groups=groups_plan)

    # ------------------------------------------------------------------ forward
    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layer_id: int, batch) -> torch.Tensor:
        """``q [rows, Hq*D]``, ``k``/``v [rows, Hkv*D]`` unrotated; returns ``[rows, Hq*D]``.

        ``batch.positions`` are the block-relative write positions, ``batch.out_loc`` the
        physical slots of the new tokens (minisgl/shared_cache/attention.py:624-703).
        """
        meta = batch.attn_metadata
        assert isinstance(meta, SharedCacheAttnMetadata)
        if not q.is_cuda:
            raise RuntimeError("view attention needs CUDA tensors: there is no CPU fallback")
        mrope_positions = getattr(batch, "mrope_positions", None)
        if mrope_positions is not None and self.mrope_section is None:
            raise ValueError("batch.mrope_positions needs an attention op built with mrope_section")
        if meta._pos32 is None:
            # [rows], or [3, rows] when the write does not sit at one position on all three axes
            pos = batch.positions if mrope_positions is None else mrope_positions
            meta._pos32 = (pos if pos.dtype == torch.int32 else pos.to(torch.int32)).contiguous()
        status = self.status()
        forked = False
        if meta.phase != "prefill_batch" and getattr(meta, "fork_dense_early", False) and FORK_DENSE_EARLY:
            # the tiles of the widely read blocks start now, beside the store kernel
            q = self._decode_queries(q, meta)
            plan = meta.plan
            self._reserve_partials(plan.num_partials)
            pool = pool_struct(self.kv_cache, layer_id, self.num_qo_heads, self._cos_sin, self.rotary_dim)
            rc = _lib.lib().va_view_decode_fork_groups(
                C.byref(pool), C.byref(plan.struct), q.data_ptr(), q.stride(0), self._partial_o.data_ptr(),
                self._partial_ml.data_ptr(), status.data_ptr(), _lib.stream_ptr())
            _lib.check(rc, "va_view_decode_fork_groups")
            forked = True
        store_rows(self.kv_cache, k, v, batch.out_loc, layer_id, meta._pos32, self._cos_sin,
                   self.rotary_dim, status=status,
                   mrope_lims=self._mrope_lims if self.mrope_section is not None else None)
        return self._attend(q, meta, layer_id, forked=forked)

    @staticmethod
    def _decode_queries(q: torch.Tensor, meta: SharedCacheAttnMetadata) -> torch.Tensor:
        q2 = q.reshape(meta.num_workers, -1)
        return q2 if q2.stride(1) == 1 else q2.contiguous()

    def _attend(self, q: torch.Tensor, meta: SharedCacheAttnMetadata, layer_id: int, forked: bool = False) -> torch.Tensor:
        """The attention of a planned step over keys that are already in the pool (``forked``: the
        step's dense tiles were launched before the store and only have to be joined)."""
        if meta.phase == "prefill_batch":
            return self._forward_prefill_batch(q, meta, layer_id)

        rows = meta.num_workers
        status = self.status()
        plan: DecodePlan = meta.plan
        self._reserve_partials(plan.num_partials)
        q2 = self._decode_queries(q, meta)
        out = torch.empty(rows, self.num_qo_heads * self.head_dim, dtype=q.dtype, device=q.device)
        pool = pool_struct(self.kv_cache, layer_id, self.num_qo_heads, self._cos_sin, self.rotary_dim)
        mask = plan.struct.phase_mask
        if forked:
            plan.struct.phase_mask = mask | _lib.VA_PHASE_GROUPS_FORKED
        try:
            rc = _lib.lib().va_view_decode(
                C.byref(pool), C.byref(plan.struct), q2.data_ptr(), q2.stride(0), out.data_ptr(),
                out.stride(0), self._partial_o.data_ptr(), self._partial_ml.data_ptr(),
                status.data_ptr(), _lib.stream_ptr(),
            )
        finally:
            plan.struct.phase_mask = mask
        _lib.check(rc, "va_view_decode")
        return out

    # ------------------------------------------------------------------ prefill planner
    def prepare_prefill_batch(self, specs: Sequence[PrefillSpec], graph_buffers=None) -> SharedCacheAttnMetadata:
        """Plan several view-conditioned prefills as one forward, request-major.

        Request ``r`` owns output rows ``[offset_r, offset_r + num_new_r)``.  Its new tokens
        attend non-causally to every context block (sized from the block's pre-write token
        count) and causally, end-aligned, to their own block including its prefix
        (minisgl/shared_cache/attention.py:450-622).  Query rotation per segment:
        ``rel + (self_offset - prefix_j)`` for context block ``j``, ``rel + T_span`` for self.
        """
        assert specs, "prepare_prefill_batch needs at least one request"
        use_3d = any(spec.mrope_rel is not None for spec in specs)
        if use_3d:
            # new tokens with genuine (time, height, width) positions (attention.py:118-127)
            if self.mrope_section is None:
                raise ValueError("PrefillSpec.mrope_rel needs an attention op built with mrope_section")
            if self.dense_engine != "tcgen05":
                raise NotImplementedError("3-axis query positions run on the tcgen05 engine")
        rel3_parts: List[np.ndarray] = []
        P = self.page_size
        widest = max(len(spec.context) + 1 for spec in specs)
        last: List[int] = []
        page_parts: List[np.ndarray] = []   # page numbers, every distinct block once, then own pages
        n_pages = 0
        block_run: Dict[int, int] = {}
        segments: List[List[int]] = []     # dense-plan segment rows
        req_segments: List[tuple] = []     # (seg_begin, seg_count, row offset, S) per request
        # what the reference-shaped tables are rebuilt from, should somebody read them:
        # per request (S, T, T_span, [(run offset, pages, tokens, last page len, span)], own pages)
        snapshot: List[tuple] = []
        n_ctx_rows = 0
        offset = 0
        for spec in specs:
            S = int(spec.num_new)
            assert S > 0
            T = int(spec.self_prefix_len)
            T_span = T if spec.self_prefix_span is None else int(spec.self_prefix_span)
            spans = [b.mrope_span for b in spec.context]
            start = sum(spans) + T_span          # running position of the first new token
            self._check_positions(start + S - 1, "a new token's position in its view")
            seg_begin = len(segments)
            before = 0
            if use_3d:
                if spec.mrope_rel is None:
                    rel3 = np.broadcast_to(np.arange(S, dtype=np.int64), (3, S))
                else:
                    rel3 = spec.mrope_rel.to(dtype=torch.int64, device="cpu").numpy()
                    assert rel3.shape == (3, S), f"mrope_rel must be [3, {S}], got {tuple(rel3.shape)}"
                rel3_parts.append(rel3)
            ctx_snap = []
            for block, span in zip(spec.context, spans):
                assert block.num_tokens > 0, "context blocks must be non-empty"
                key = id(block)
                run = block_run.get(key)
                if run is None:
                    run = block_run[key] = n_pages
                    pages = block_page_numbers(block)
                    page_parts.append(pages)
                    n_pages += pages.size
                ctx_snap.append((run, block.num_pages, block.num_tokens, block.last_page_len, span))
                segments.append([run, 0, block.num_tokens, start - before, -1, 0, 0, 0])
                before += span
            n_ctx_rows += S * len(spec.context)
            own = np.asarray(spec.self_page_starts.cpu().tolist(), np.int64) // P
            own_off = n_pages
            page_parts.append(own)
            n_pages += own.size
            segments.append([own_off, 0, T + S, T_span, T, 0, 0, 0])
            req_segments.append((seg_begin, len(segments) - seg_begin, offset, S))
            snapshot.append((S, T, T_span, start, ctx_snap, own_off, own.size))
            last.append(offset + S - 1)
            offset += S

        n_rows = offset
        page_pool = np.concatenate(page_parts).astype(np.int32) if page_parts else np.zeros(0, np.int32)
        q_pos3 = np.ascontiguousarray(np.concatenate(rel3_parts, axis=1), np.int32) if use_3d else None
        meta = SharedCacheAttnMetadata(
            shared_cache_op=self,
            sub_worker_list=None,
            sub_loc_list=None,
            pad_slot_list=None,
            num_workers=n_rows,
            max_segments=widest,
            n_ctx_rows=n_ctx_rows,
            last_indices=torch.tensor(last, dtype=torch.int64, device=self.device),
            phase="prefill_batch",
        )
        meta._lists_recipe = (snapshot, page_pool, widest, P, q_pos3)
        meta.plan = self._upload_dense_plan(page_pool, segments, req_segments, n_rows, buffers=graph_buffers,
                                            q_pos3=q_pos3)
        meta.graph_buffers = graph_buffers
        if graph_buffers is not None:
            meta.num_workers = graph_buffers.rows
        return meta

    def _upload_dense_plan(self, page_pool, segments, req_segments, n_rows, buffers=None, q_pos3=None):
        """Tiles of tile_rows/G consecutive new tokens per (request, kv head), heaviest first, every
        other round of the CTA stride reversed: the native planner ``va_plan_prefill_tiles`` (CTA c
        runs tiles c, c + n, ...; heaviest-first order alone hands CTA 0 the heaviest tile of every
        round -- config 3: heaviest CTA 2.5 % above the mean instead of 6.6 %, 780 -> 805 TFLOP/s; a
        least-loaded-CTA assignment balances better on paper (1.5 %) but measured slower (795): it
        separates in time the tiles that share a request's K/V in L2)."""
        per_tile = self.tile_rows() // self.gqa
        seg_arr = np.asarray(segments, np.int32).reshape(-1, 8)
        req_arr = np.asarray(req_segments, np.int32).reshape(-1, 4)
        H = self.num_kv_heads
        cap = int(sum(-(-int(S) // per_tile) for _, _, _, S in req_segments)) * H
        entries = np.empty((n_rows, 4), np.int32)
        tile_arr = np.empty((max(cap, 1), 8), np.int32)
        n_ctas = self._dense_ctas(cap if buffers is None else buffers.cap_tiles)
        n_tiles = C.c_int32(0)
        rc = _lib.lib().va_plan_prefill_tiles(seg_arr.ctypes.data, seg_arr.shape[0], req_arr.ctypes.data,
                                              req_arr.shape[0], per_tile, H, n_ctas, entries.ctypes.data, n_rows,
                                              tile_arr.ctypes.data, cap, C.byref(n_tiles))
        _lib.check(rc, "va_plan_prefill_tiles")
        tile_arr = tile_arr[: n_tiles.value]
        pages = np.asarray(page_pool, np.int32)
        if buffers is not None:
            return buffers.load(pages, tile_arr, entries, seg_arr, n_rows, q_pos3=q_pos3)
        return self._pack_dense(pages, tile_arr, entries, seg_arr, n_rows, 0, q_pos3=q_pos3)

    def _dense_ctas(self, num_tiles: int) -> int:
        """CTAs a dense-tile launch of ``num_tiles`` table rows runs (one per SM at most)."""
        if self._sm_count is None:
            n = _lib.lib().va_sm_count() if self.device.type == "cuda" else 0
            self._sm_count = n if n > 0 else 148
        return max(1, min(self._sm_count, num_tiles))

    def _pack_dense(self, pages, tile_arr, entries, seg_arr, n_rows, n_partials, n_ctas=0, q_pos3=None):
        parts = [pages, tile_arr, entries, seg_arr] + ([q_pos3] if q_pos3 is not None else [])
        sizes = [a.size for a in parts]
        offs = [0]
        for sz in sizes:
            offs.append(offs[-1] + (-(-sz // 4) * 4))
        on_gpu = self.device.type == "cuda"
        host = torch.empty(max(offs[-1], 4), dtype=torch.int32, pin_memory=on_gpu)
        hv = host.numpy()
        for off, sz, arr in zip(offs, sizes, parts):
            hv[off: off + sz] = arr.reshape(-1)
        blob = host.to(self.device, non_blocking=True) if on_gpu else host
        st = _lib.VaDensePlan()
        base = blob.data_ptr()
        if q_pos3 is not None:
            st.q_pos3 = base + 4 * offs[4]
            st.mrope_lim_h, st.mrope_lim_w = self._mrope_lims
        st.page_indices = base + 4 * offs[0]
        st.tiles = base + 4 * offs[1]
        st.entries = base + 4 * offs[2]
        st.segments = base + 4 * offs[3]
        st.num_page_indices = int(pages.size)
        st.num_tiles = int(tile_arr.shape[0])
        st.num_entries = int(entries.shape[0])
        st.num_segments = int(seg_arr.shape[0])
        st.num_partials = int(n_partials)
        st.num_rows = int(n_rows)
        st.num_ctas = int(n_ctas)
        st.engine = DENSE_ENGINES[self.dense_engine]
        return DensePlan(blob=blob, host_blob=host, struct=st,
                         host={"page_indices": pages, "tiles": tile_arr, "entries": entries,
                               "segments": seg_arr})

    def _forward_prefill_batch(self, q, meta, layer_id):
        plan: DensePlan = meta.plan
        rows = meta.num_workers
        q2 = q.reshape(rows, -1)
        if q2.stride(1) != 1:
            q2 = q2.contiguous()
        out = torch.empty(rows, self.num_qo_heads * self.head_dim, dtype=q.dtype, device=q.device)
        pool = pool_struct(self.kv_cache, layer_id, self.num_qo_heads, self._cos_sin, self.rotary_dim)
        rc = _lib.lib().va_view_dense(
            C.byref(pool), C.byref(plan.struct), q2.data_ptr(), q2.stride(0), out.data_ptr(),
            out.stride(0), None, None, self.status().data_ptr(), _lib.stream_ptr(),
        )
        _lib.check(rc, "va_view_dense")
        return out
