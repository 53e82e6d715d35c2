"""CUDA-graph contract of the cache-view path: preparation hooks for the host framework's GraphRunner.

Counterpart of the reference's ``SharedGraphIO`` (minisgl/shared_cache/graph.py:68-227), driven by
``GraphRunner`` (minisgl/engine/graph.py:118-212) through the same calls:

    init_capture_graph(max_seq_len, bs_list)   fixed-capacity tables for every batch size (and, with
                                               ``prefill_rows``, every prefill row count)
    prepare_for_capture(batch)                 plan a dummy topology of the batch's size into the tables
    finish_capture(batch)                      drop what the warm-up forward produced
    pad_inputs(batch)                          pad a real decode batch to its captured size
    prepare_for_replay(batch)                  check that the session planned into the captured tables
    select_prefill(jobs) / prefill_capture_batch(rows) / destroy_capture_graph() / retire_completed()

What makes a forward capturable here: ``SharedCacheAttention.prepare(..., graph_buffers=)`` and
``SharedCacheGDN.prepare_decode(..., buffers=)`` plan on the host and copy the step's tables into
device tensors whose addresses never change; every kernel of the forward is launched with the same
arguments and grid whatever the topology; padding rows are empty ranges / zero addresses.  Nothing
is allocated and no host value is read inside the captured region.

``session`` is the object that owns the pieces; the attributes read are the reference session's:
``sc_attn``, ``sc_gdn`` (or None), ``page_allocator``, ``page_size``, ``device``, ``kv_cache``,
``_model_config.num_linear_layers``, ``engine.dtype``, ``engine.stream``.  Multimodal prefill inputs
(image embeddings) are not staged here; text and per-axis positions are.
"""

from __future__ import annotations

from types import SimpleNamespace
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from .blocks import CacheBlock, WorkerGroup
from .view_attention import PrefillSpec, SharedDecodeAttentionBuffers, SharedPrefillAttentionBuffers
from .view_gdn import GDNDecodeBuffers, GDNPrefillBuffers


def _set_gdn_ar(value) -> None:
    """Publish the GDN seam object where the host framework's layers look for it
    (``get_global_ctx().gdn_ar``, minisgl/core.py); a no-op without the host framework."""
    try:
        from minisgl.core import get_global_ctx

        get_global_ctx().gdn_ar = value
    except Exception:   # noqa: BLE001 -- stand-alone use: the caller hands the object to its layers
        pass


class _PrefillInputs:
    """Stable model inputs of a captured prefill: rows beyond the planned batch are zero tokens with
    slot -1 (never stored)."""

    def __init__(self, device, rows: int, workers: int, vocab_size: Optional[int], with_mrope: bool):
        self.input_ids = torch.zeros(rows, device=device, dtype=torch.int32)
        self.positions = torch.zeros(rows, device=device, dtype=torch.int64)
        self.out_loc = torch.full((rows,), -1, device=device, dtype=torch.int32)
        self.mrope = torch.zeros(3, rows, device=device, dtype=torch.int64) if with_mrope else None
        self.logits = (torch.empty(workers, vocab_size, device=device, dtype=torch.float32)
                       if vocab_size else None)

    def bind(self, batch, rows: int) -> None:
        batch.input_ids, batch.positions, batch.out_loc = (
            t[:rows] for t in (self.input_ids, self.positions, self.out_loc))
        if self.mrope is not None:
            batch.mrope_positions = self.mrope[:, :rows]

    def copy_from(self, batch, rows: int) -> None:
        n = batch.input_ids.numel()
        self.input_ids[:rows].zero_()
        self.positions[:rows].zero_()
        self.out_loc[:rows].fill_(-1)
        self.input_ids[:n].copy_(batch.input_ids)
        self.positions[:n].copy_(batch.positions)
        self.out_loc[:n].copy_(batch.out_loc)
        if self.mrope is not None:
            self.mrope[:, :rows].zero_()
            positions = getattr(batch, "mrope_positions", None)
            self.mrope[:, :n].copy_(batch.positions.expand(3, -1) if positions is None else positions)


class SharedGraphIO:
    def __init__(self, session, depth: int, prefill_rows: Sequence[int] = (), *, dense_fraction: float = 0.0):
        # dense_fraction: share of the SMs the captured decode launches reserve for the tensor-core
        # tiles of blocks read by many workers (grid sizes are part of a captured graph, so the split
        # between those tiles and the streaming lanes is frozen per profile)
        self.session, self.depth = session, int(depth)
        self.dense_fraction = float(dense_fraction)
        self.attention: Dict[int, SharedDecodeAttentionBuffers] = {}
        self.gdn: Dict[int, GDNDecodeBuffers] = {}
        self.dummy_slots: Optional[torch.Tensor] = None
        self.prefill_rows: List[int] = sorted(set(prefill_rows))
        self.prefill_attention: Dict[int, SharedPrefillAttentionBuffers] = {}
        self.prefill_gdn: Dict[int, GDNPrefillBuffers] = {}
        self.prefill_batches: Dict[int, object] = {}
        self.prefill_inputs: Optional[_PrefillInputs] = None

    # ------------------------------------------------------------------ session accessors
    def _linear_layers(self) -> int:
        s = self.session
        cfg = getattr(s, "_model_config", None)
        return int(cfg.num_linear_layers if cfg is not None else s.num_linear_layers)

    def _dtype(self):
        s = self.session
        engine = getattr(s, "engine", None)
        return engine.dtype if engine is not None else s.dtype

    def _sync(self) -> None:
        engine = getattr(self.session, "engine", None)
        stream = getattr(engine, "stream", None)
        if stream is not None:
            stream.synchronize()
        elif torch.device(self.session.device).type == "cuda":
            torch.cuda.current_stream(self.session.device).synchronize()

    # ------------------------------------------------------------------ the contract
    def retire_completed(self) -> None:
        # a profile may not be selected again for many steps: its completed references must not
        # keep an old topology's tensors alive
        for buffers in (*self.gdn.values(), *self.prefill_gdn.values()):
            buffers.retire_completed()

    def init_capture_graph(self, max_seq_len: int, bs_list: Sequence[int]) -> None:
        s = self.session
        P = s.page_size
        # a reserved page per padded worker: padding rows never write to a live block's pages and
        # never collide with one another
        self.dummy_slots = s.page_allocator.alloc_pages(max(bs_list))
        for bs in bs_list:
            max_pages = bs * ((max_seq_len + P - 1) // P + self.depth)
            self.attention[bs] = SharedDecodeAttentionBuffers(s.sc_attn, bs, self.depth, max_pages, self.dummy_slots[:bs],
                                                              dense_fraction=self.dense_fraction)
            if s.sc_gdn is not None:
                self.gdn[bs] = GDNDecodeBuffers(s.sc_gdn, self._linear_layers(), bs, self.depth, self._dtype())
        if self.prefill_rows:
            model_cfg = getattr(getattr(getattr(s, "engine", None), "config", None), "model_config", None)
            vocab = getattr(model_cfg, "vocab_size", None) or getattr(s, "vocab_size", None)
            self.prefill_inputs = _PrefillInputs(s.device, max(self.prefill_rows), max(bs_list), vocab,
                                                 s.sc_attn.mrope_section is not None)
            dummy_pages = self.dummy_slots.long() // P
            for layer in range(s.kv_cache.num_layers):
                s.kv_cache.k_cache(layer).index_fill_(0, dummy_pages, 0)
                s.kv_cache.v_cache(layer).index_fill_(0, dummy_pages, 0)
            for rows in self.prefill_rows:
                workers = min(rows, max(bs_list))
                max_pages = workers * ((max_seq_len + P - 1) // P + self.depth)
                self.prefill_attention[rows] = SharedPrefillAttentionBuffers(
                    s.sc_attn, workers, self.depth, rows, max_pages, self.dummy_slots[:workers])
                if s.sc_gdn is not None:
                    self.prefill_gdn[rows] = GDNPrefillBuffers(s.sc_gdn, self._linear_layers(), workers, self.depth,
                                                               self._dtype(), rows)
        # reserve the split-K scratch of the whole catalogue before the first capture
        s.sc_attn.prepare_workspace((*self.attention.values(), *self.prefill_attention.values()))

    def select_prefill(self, jobs):
        """The smallest captured prefill profile a batch of prefill jobs fits (each job: ``input_ids``,
        ``context`` blocks, write ``block``); ``ValueError`` when none does."""
        P = self.session.page_size
        workers, rows = len(jobs), sum(job.input_ids.numel() for job in jobs)
        contexts = [[b for b in (job.context or []) if b.num_tokens > 0] for job in jobs]
        depth = max((len(c) + 1 for c in contexts), default=1)
        if depth > self.depth:
            raise ValueError("Shared prefill exceeds graph depth capacity")
        distinct = {id(b): b for c in contexts for b in c}       # the planner lists every block's pages once
        pages = sum(b.num_pages for b in distinct.values())
        pages += sum((job.block.num_tokens + job.input_ids.numel() + P - 1) // P for job in jobs)
        for capacity in self.prefill_rows:
            buffers = self.prefill_attention[capacity]
            if rows <= capacity and workers <= buffers.workers and pages <= buffers.max_pages:
                return buffers
        raise ValueError("Shared prefill exceeds graph request/token-row/page capacity")

    def prefill_capture_batch(self, rows: int):
        """A batch object bound to the stable prefill inputs of the ``rows`` profile."""
        buffers = self.prefill_attention[rows]
        engine = getattr(self.session, "engine", None)
        try:
            from minisgl.core import Batch

            batch = Batch(reqs=[engine.dummy_req] * buffers.workers, phase="prefill")
            batch.padded_reqs = batch.reqs
        except Exception:   # noqa: BLE001 -- stand-alone use
            batch = SimpleNamespace(reqs=[None] * buffers.workers, padded_reqs=[None] * buffers.workers,
                                    phase="prefill", is_prefill=True, is_decode=False, size=buffers.workers,
                                    padded_size=buffers.workers, mrope_positions=None, attn_metadata=None)
        self.prefill_inputs.bind(batch, rows)
        self.prefill_batches[rows] = batch
        logits = self.prefill_inputs.logits
        return batch, (logits[: buffers.workers] if logits is not None else None)

    def prepare_for_capture(self, batch) -> None:
        s, bs = self.session, batch.size
        P = s.page_size
        layers = self._linear_layers() if s.sc_gdn is not None else 0
        slots = self.dummy_slots[:bs].cpu().tolist()
        if batch.is_prefill:
            rows = batch.input_ids.numel()
            batch.input_ids.zero_()
            batch.positions.zero_()
            batch.out_loc.fill_(-1)
            lengths = [rows // bs + (i < rows % bs) for i in range(bs)]
            blocks = [CacheBlock(s.device, P) for _ in range(bs)]
            contexts = [CacheBlock(s.device, P) for _ in range(bs)]
            for block, slot in zip(contexts, slots):
                block.page_starts, block.num_tokens = [slot], 1
            # the captured launches are sized by the profile, not by this dummy batch; no KV is written
            specs = [PrefillSpec([contexts[i]] * (self.depth - 1),
                                 self.dummy_slots[i:i + 1].repeat((n + P - 1) // P), n)
                     for i, n in enumerate(lengths) if n > 0]
            batch.attn_metadata = s.sc_attn.prepare_prefill_batch(specs, self.prefill_attention[rows])
            if s.sc_gdn is not None:
                live = [(b, n) for b, n in zip(blocks, lengths) if n > 0]
                s.sc_gdn.set_context([[b] for b, _ in live], [b for b, _ in live], prefill_segments=[n for _, n in live])
                s.sc_gdn.prepare_prefill(layers, self._dtype(), rows, buffers=self.prefill_gdn[rows])
                _set_gdn_ar(s.sc_gdn)
            return
        batch.input_ids.zero_()
        batch.positions.zero_()
        batch.out_loc.copy_(self.dummy_slots[:bs])
        blocks = [CacheBlock(s.device, P) for _ in range(bs)]
        for block, slot in zip(blocks, slots):
            block.page_starts = [slot]
        group = WorkerGroup(cache_structure=[[b] for b in blocks], write_to=blocks)
        batch.attn_metadata = s.sc_attn.prepare(group, {id(b): None for b in blocks}, self.dummy_slots[:bs],
                                                self.attention[bs])
        if s.sc_gdn is not None:
            s.sc_gdn.set_context([[b] for b in blocks], blocks)
            s.sc_gdn.prepare_decode(layers, self._dtype(), buffers=self.gdn[bs])
            _set_gdn_ar(s.sc_gdn)

    def finish_capture(self, batch) -> None:
        gdn = self.session.sc_gdn
        if gdn is not None:
            if batch.is_prefill:
                gdn.finish_prefill(False)
                buffers = self.prefill_gdn[batch.input_ids.numel()]
            else:
                gdn.finish_decode(False)
                buffers = self.gdn[batch.size]
            # the warm-up's output slabs are not persistent state: retire them now, and leave the
            # tables without output addresses until a real step is planned
            self._sync()
            buffers.retire_completed()
            buffers.write_ptrs.zero_()
        _set_gdn_ar(None)

    def prepare_for_replay(self, batch) -> None:
        # the session has planned its real group into the captured tables before entering the forward
        meta = batch.attn_metadata
        if batch.is_prefill:
            rows = meta.graph_buffers.rows
            assert meta.graph_buffers is self.prefill_attention[rows], "prefill was not planned into the captured tables"
            self.prefill_inputs.copy_from(batch, rows)
            return
        assert meta.graph_buffers is self.attention[batch.padded_size], "decode was not planned into the captured tables"

    def pad_inputs(self, batch) -> None:
        n, padded = batch.size, batch.padded_size
        batch.input_ids = F.pad(batch.input_ids, (0, padded - n))
        batch.positions = F.pad(batch.positions, (0, padded - n))
        batch.out_loc = torch.cat([batch.out_loc, self.dummy_slots[n:padded].to(batch.out_loc.dtype)])

    def destroy_capture_graph(self) -> None:
        if self.dummy_slots is not None:
            self._sync()
            self.session.page_allocator.free_pages(self.dummy_slots)
            self.dummy_slots = None
        for buffers in (*self.gdn.values(), *self.prefill_gdn.values()):
            buffers.retire_completed()
        ar = self.session.sc_gdn
        if ar is not None and ar.decode_buffers in self.gdn.values():
            ar.decode_buffers = None
        if ar is not None and ar.prefill_buffers in self.prefill_gdn.values():
            ar.prefill_buffers = None
        self.attention.clear()
        self.gdn.clear()
        self.prefill_gdn.clear()
        self.prefill_attention.clear()
        self.prefill_batches.clear()
        self.prefill_inputs = None


__all__ = ["SharedGraphIO"]
