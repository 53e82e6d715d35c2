"""Gated DeltaNet state over an ordered block list: host side of the GDN seam.

Drop-in for the reference ``SharedCacheGDN`` (minisgl/shared_cache/gdn.py:28-282): the model's
GDN layer finds this object at ``get_global_ctx().gdn_ar`` and the session drives it with
``set_context`` / ``prepare_decode`` / ``finish_decode`` (session.py:1195-1227).  Each
``CacheBlock`` carries, per linear layer, an affine summary ``(A_hat [1,H,dk,dk], B_hat [1,H,dv,dk])``
of its tokens and a conv window; a worker's initial recurrent state is the fold of its chain.

Two ways in:

* the reference's call sequence -- ``compose_initial_recurrent_state`` then the recurrence then
  ``capture_token_affines`` -- is served by ``va_gdn_compose`` and the capture mode of
  ``va_gdn_prefill``;
* the fused calls ``decode_step`` / ``prefill_scan`` replace that whole sequence by one kernel per
  layer (``va_gdn_step``: no state is materialised for a one-token step; ``va_gdn_prefill``: the
  output rows and the block's new summary from one joint scan).

New summaries are always written to fresh tensors and published into the write blocks only by
``finish_decode(True)`` / ``finish_prefill(True)``, so a failed forward leaves every block as it was
and readers of the previous summary are never disturbed (gdn_decode.py:112-121, 172-188).
"""

from __future__ import annotations

import ctypes as C
import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from . import _lib
from .blocks import CacheBlock, _TrackedDict

GDN_ENGINES = {"scan": 0, "chunk": 1, "chunk_tc": 2}   # VA_GDN_ENGINE_* of the C header


# rows of the per-step address table [8, layers, workers, depth]
ROW_CHAIN_A, ROW_CHAIN_B, ROW_READ_A, ROW_READ_B, ROW_CONV_READ, ROW_WRITE_A, ROW_WRITE_B, ROW_CONV_WRITE = range(8)


class GDNDecodeBuffers:
    """Fixed-capacity, address-stable address tables of a GDN decode step, for CUDA-graph replay.

    The counterpart of the reference's class of the same name (minisgl/shared_cache/gdn_decode.py:62-214):
    one capacity -- ``layers`` linear layers, ``workers`` rows, chains of at most ``depth`` blocks --
    whose device tables never move.  ``SharedCacheGDN.prepare_decode(..., buffers=self)`` plans on the
    host and copies the step's addresses INTO these tables; the kernels of ``decode_pre`` /
    ``decode_step`` are always launched over ``workers`` rows with the same arguments, so a graph
    captured once keeps working while topology and block summaries change behind it.  Rows beyond
    the planned batch carry zero addresses: they read the identity, write nothing and their output
    rows are ignored.  New summaries still go to FRESH slabs allocated on the host at prepare time
    (never inside a capture), so readers of the previous summary are never disturbed
    (gdn_decode.py:112-121).  Exceeding a capacity raises ``ValueError`` before anything is copied.
    """

    def __init__(self, ar: "SharedCacheGDN", layers: int, workers: int, depth: int, dtype: torch.dtype):
        self.ar, self.layers, self.workers, self.depth, self.dtype = ar, int(layers), int(workers), max(1, int(depth)), dtype
        self.device = ar.device
        on_gpu = self.device.type == "cuda"
        shape = (8, self.layers, self.workers, self.depth)
        self.host_tab = torch.zeros(shape, dtype=torch.int64, pin_memory=on_gpu)
        self.host_rw = torch.zeros(self.layers, 6, self.workers, dtype=torch.int64, pin_memory=on_gpu)
        self.tab = self.host_tab.to(self.device) if on_gpu else self.host_tab
        self.rw = self.host_rw.to(self.device) if on_gpu else self.host_rw
        self.event = torch.cuda.Event() if on_gpu else None
        self.prepare_count = 0

    @property
    def write_ptrs(self) -> torch.Tensor:
        """``[layers, 3, workers]`` view of the output addresses (A_hat, B_hat, conv window); zeroing it
        turns a replay into a step that publishes nothing (gdn_decode.py: ``write_ptrs``)."""
        return self.rw[:, 3:6]

    def retire_completed(self) -> None:
        self.ar._retire()

    def load(self, tab: np.ndarray) -> None:
        """Copy a step's table ``[8, layers, W, depth]`` (W, depth within capacity) into the fixed tables."""
        _, layers, W, depth = tab.shape
        if layers != self.layers:
            raise ValueError(f"GDN buffers were prepared for {self.layers} layers, not {layers}")
        if W > self.workers:
            raise ValueError(f"GDN batch of {W} workers exceeds the prepared capacity {self.workers}")
        if depth > self.depth:
            raise ValueError(f"GDN chain depth {depth} exceeds the prepared capacity {self.depth}")
        if self.event is not None:
            self.event.synchronize()   # the previous upload has left the staging buffers
        hv = self.host_tab.numpy()
        hv[...] = 0
        hv[:, :, :W, :depth] = tab
        self.host_rw.numpy()[...] = hv[2:8, :, :, 0].transpose(1, 0, 2)
        if self.tab is not self.host_tab:
            self.tab.copy_(self.host_tab, non_blocking=True)
            self.rw.copy_(self.host_rw, non_blocking=True)
            self.event.record()
        self.prepare_count += 1


class GDNPrefillBuffers(GDNDecodeBuffers):
    """Fixed-capacity tables of a batched GDN prefill (minisgl/shared_cache/gdn_prefill.py:11-61):
    on top of the decode tables, ``rows`` token rows at most, the requests' row offsets at a fixed
    device address and the chunk engine's scratch reserved for ``rows`` tokens.  Requests beyond the
    planned batch are empty ranges."""

    def __init__(self, ar: "SharedCacheGDN", layers: int, workers: int, depth: int, dtype: torch.dtype, rows: int):
        super().__init__(ar, layers, workers, depth, dtype)
        self.rows = int(rows)
        on_gpu = self.device.type == "cuda"
        self.host_seg = torch.zeros(self.workers + 1, dtype=torch.int32, pin_memory=on_gpu)
        self.seg = self.host_seg.to(self.device) if on_gpu else self.host_seg
        self.scratch = None
        if on_gpu:
            need = int(_lib.lib().va_gdn_prefill_scratch_bytes(self.rows, ar.num_heads))
            self.scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=self.device)

    def check_segments(self, segments: Sequence[int]) -> None:
        if len(segments) > self.workers or any(int(t) <= 0 for t in segments) or sum(segments) > self.rows:
            raise ValueError("Prefill exceeds prepared request/token capacity")

    def load_segments(self, segments: Sequence[int]) -> None:
        self.check_segments(segments)
        off = np.zeros(self.workers + 1, np.int32)
        off[1: len(segments) + 1] = np.cumsum(np.asarray(segments, np.int64))
        off[len(segments) + 1:] = off[len(segments)]
        self.host_seg.numpy()[...] = off
        if self.seg is not self.host_seg:
            self.seg.copy_(self.host_seg, non_blocking=True)
            self.event.record()


class SharedCacheGDN:
    """Per-forward composer / capturer of GDN block summaries over worker chains."""

    def __init__(
        self,
        *,
        num_heads: int,
        head_k_dim: int,
        head_v_dim: int,
        conv_dim: int,
        conv_kernel: int,
        device: torch.device,
        state_dtype: torch.dtype = torch.float32,
        num_k_heads: Optional[int] = None,
        prefill_engine: Optional[str] = None,
    ) -> None:
        # summaries are stored in ``state_dtype``; the kernels widen them when read, work in fp32 and
        # round once when a new summary is stored (minisgl/shared_cache/gdn.py:40-45,249-269)
        if state_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("Shared GDN state dtype must be float32 or bfloat16")
        self._summary_code = _lib.summary_code(state_dtype)
        # fused prefill: "chunk_tc" = 64-token chunks, the state walked with tcgen05 products (state in
        # TMEM; bf16 operands, fp32 state), "chunk" = the same on mma.sync, "scan" = token-by-token
        # fp32 recurrence (also what capture_token_affines always runs)
        self.prefill_engine = prefill_engine or os.environ.get("VIEWATTN_GDN_ENGINE", "chunk_tc")
        if self.prefill_engine not in GDN_ENGINES:
            raise ValueError(f"prefill_engine must be one of {sorted(GDN_ENGINES)}")
        self._chunk_scratch: Optional[torch.Tensor] = None
        self._status: Optional[torch.Tensor] = None
        self._init_row_index: Optional[torch.Tensor] = None
        self.decode_buffers: Optional[GDNDecodeBuffers] = None
        self.prefill_buffers: Optional[GDNPrefillBuffers] = None
        self.device = torch.device(device)
        self.state_dtype = state_dtype
        self.num_heads = num_heads              # value heads (post GQA repeat)
        self.num_k_heads = num_k_heads or num_heads
        self.head_k_dim = head_k_dim
        self.head_v_dim = head_v_dim
        self.conv_dim = conv_dim
        self.conv_kernel = conv_kernel
        self.cache_structure: List[List[CacheBlock]] = []
        self.write_to: List[CacheBlock] = []
        self.prefill_segments: Optional[List[int]] = None
        self._prepared_decode = False
        self._prepared_prefill = False
        self._step = None      # tables + outputs of the prepared forward
        self._pending = []     # (event, references) kept until the GPU is done with raw pointers
        self.prepare_count = 0

    def status(self) -> torch.Tensor:
        """Device word the kernels report findings into (a bounded wait that ran out)."""
        if self._status is None:
            self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
        return self._status

    def check_status(self) -> None:
        """Raise if a kernel of this object reported a device-side finding (synchronises)."""
        if self._status is not None:
            code = int(self._status.item())
            if code:
                self._status.zero_()
                raise RuntimeError(f"GDN kernel reported device status {code}")

    # ------------------------------------------------------------------ context
    def set_context(self, cache_structure, write_to, prefill_segments=None) -> None:
        self.cache_structure = [list(c) for c in cache_structure]
        self.write_to = list(write_to)
        self.prefill_segments = None if prefill_segments is None else list(prefill_segments)
        self._prepared_decode = False
        self._prepared_prefill = False

    @property
    def num_workers(self) -> int:
        return len(self.cache_structure)

    def has_previous_affine(self, lin_idx: int) -> bool:
        return any(lin_idx in b.linear_affine for chain in self.cache_structure for b in chain)

    # ------------------------------------------------------------------ pointer tables
    def _pair_ptrs(self, block: CacheBlock, layer: int, keep: list):
        pair = block.linear_affine.get(layer)
        if pair is None:
            return 0, 0
        a, b = pair
        H, dk, dv = self.num_heads, self.head_k_dim, self.head_v_dim
        if tuple(a.shape) != (1, H, dk, dk) or tuple(b.shape) != (1, H, dv, dk):
            raise ValueError(f"Unexpected GDN state shape {tuple(a.shape)} / {tuple(b.shape)}")
        a2 = a.to(device=self.device, dtype=self.state_dtype).contiguous()
        b2 = b.to(device=self.device, dtype=self.state_dtype).contiguous()
        keep += [a2, b2]
        return a2.data_ptr(), b2.data_ptr()

    def _block_ptrs(self, block: CacheBlock, layers: int, keep: list) -> np.ndarray:
        """Device addresses ``[layers, 2]`` of a block's (A_hat, B_hat) per layer, 0 where it has
        none.  Kept on the block until one of its state dictionaries changes (the reference caches
        the same addresses behind its StateDict, minisgl/shared_cache/gdn_state.py:15-58)."""
        rev = getattr(block, "_gdn_revision", None)
        c = getattr(block, "_gdn_ptr_cache", None) if rev is not None else None
        if c is None or c[0] != rev or c[1] != (self.device, self.state_dtype) or c[2].shape[0] < layers:
            held: list = []
            ptrs = np.zeros((layers, 2), np.int64)
            for layer in range(layers):
                ptrs[layer] = self._pair_ptrs(block, layer, held)
            c = (rev, (self.device, self.state_dtype), ptrs, held)
            if rev is not None:   # a block without a revision counter (the reference's own class) is re-read
                block._gdn_ptr_cache = c
        keep.append(c[3])
        return c[2][:layers]

    def _block_conv_ptrs(self, block: CacheBlock, layers: int, keep: list) -> np.ndarray:
        """Device addresses ``[layers]`` of a block's conv windows (bf16 ``[conv_dim, k]``), 0 where
        it has none; kept on the block like the summary addresses."""
        rev = getattr(block, "_gdn_revision", None)
        c = getattr(block, "_gdn_conv_cache", None) if rev is not None else None
        if c is None or c[0] != rev or c[1] != self.device or c[2].shape[0] < layers:
            held: list = []
            ptrs = np.zeros(layers, np.int64)
            for layer, state in block.linear_conv_state.items():
                if 0 <= layer < layers:
                    if tuple(state.shape) != (self.conv_dim, self.conv_kernel):
                        raise ValueError(f"Unexpected GDN conv state shape {tuple(state.shape)}")
                    t = state.to(device=self.device, dtype=torch.bfloat16).contiguous()
                    held.append(t)
                    ptrs[layer] = t.data_ptr()
            c = (rev, self.device, ptrs, held)
            if rev is not None:
                block._gdn_conv_cache = c
        keep.append(c[3])
        return c[2][:layers]

    def _build_tables(self, layers: int, with_outputs: bool, buffers: Optional[GDNDecodeBuffers] = None):
        """Address tables of every layer in one upload: ``[8, L, W, depth]`` (rows ``ROW_*``); the read /
        write rows use ``[..., 0]`` only.  With ``buffers`` the tables are copied into its fixed device
        tensors and the step runs over its ``workers`` rows."""
        chains, targets = self.cache_structure, self.write_to
        if len(chains) != len(targets) or len({id(t) for t in targets}) != len(targets):
            raise ValueError("GDN forward needs one distinct write target per worker")
        W = len(chains)
        depth = max(1, max((len(c) for c in chains), default=0))
        if buffers is not None and (W > buffers.workers or depth > buffers.depth or layers != buffers.layers):
            buffers.load(np.zeros((8, layers, W, depth), np.int64))   # raises the capacity error
        keep: list = []
        # every distinct block once; row 0 of the address table stands for "no block here"
        index: Dict[int, int] = {}
        rows = [np.zeros((layers, 2), np.int64)]
        conv_rows = [np.zeros(layers, np.int64)]
        chain_idx = np.zeros((W, depth), np.int64)
        target_idx = np.zeros(W, np.int64)

        def number(block) -> int:
            i = index.get(id(block))
            if i is None:
                i = index[id(block)] = len(rows)
                rows.append(self._block_ptrs(block, layers, keep))
                if with_outputs:
                    conv_rows.append(self._block_conv_ptrs(block, layers, keep))
            return i

        for w, chain in enumerate(chains):
            for j, block in enumerate(chain):
                chain_idx[w, j] = number(block)
            target_idx[w] = number(targets[w])
        addr = np.ascontiguousarray(np.stack(rows))               # [blocks + 1, L, 2]
        conv_addr = np.ascontiguousarray(np.stack(conv_rows)) if with_outputs else None   # [blocks + 1, L]
        chain32 = np.ascontiguousarray(chain_idx, dtype=np.int32)
        target32 = np.ascontiguousarray(target_idx, dtype=np.int32)
        out_a = out_b = conv_out = None
        bases = [None, None, None]          # per-worker addresses of layer 0: write a, write b, conv write
        strides = [0, 0, 0]                 # bytes between a worker's layers
        if with_outputs:
            H, dk, dv = self.num_heads, self.head_k_dim, self.head_v_dim
            conv_out = [torch.empty(layers, self.conv_dim, self.conv_kernel, dtype=torch.bfloat16,
                                    device=self.device) for _ in targets]
            bases[2] = np.fromiter((t.data_ptr() for t in conv_out), np.int64, W)
            strides[2] = self.conv_dim * self.conv_kernel * 2
            # one all-layer allocation per worker: a stopped worker must not pin a whole batch
            if dk == dv:
                # A_hat and B_hat of all layers of one worker in one allocation: [2 * layers, 1, H, d, d]
                out_a = [torch.empty(2 * layers, 1, H, dk, dk, dtype=self.state_dtype, device=self.device)
                         for _ in targets]
                out_b = None
                stride = H * dk * dk * out_a[0].element_size() if W else 0
                bases[0] = np.fromiter((t.data_ptr() for t in out_a), np.int64, W)
                bases[1] = bases[0] + layers * stride
                strides[0] = strides[1] = stride
            else:
                out_a = [torch.empty(layers, 1, H, dk, dk, dtype=self.state_dtype, device=self.device) for _ in targets]
                out_b = [torch.empty(layers, 1, H, dv, dk, dtype=self.state_dtype, device=self.device) for _ in targets]
                esz = out_a[0].element_size() if W else 0
                bases[0] = np.fromiter((t.data_ptr() for t in out_a), np.int64, W)
                bases[1] = np.fromiter((t.data_ptr() for t in out_b), np.int64, W)
                strides[0], strides[1] = H * dk * dk * esz, H * dv * dk * esz
        # the tables themselves (chain rows, read / write rows, most recent conv window along each
        # chain -- minisgl/shared_cache/gdn.py:182-207) are laid out by the native planner
        tab = np.zeros((8, layers, W, depth), dtype=np.int64)
        ptr = lambda a: a.ctypes.data if a is not None else None
        rc = _lib.VA_OK if W == 0 else _lib.lib().va_gdn_plan_tables(
            ptr(addr), ptr(conv_addr), ptr(chain32), ptr(target32), ptr(bases[0]), strides[0], ptr(bases[1]),
            strides[1], ptr(bases[2]), strides[2], len(rows) - 1, layers, W, depth, ptr(tab))
        _lib.check(rc, "va_gdn_plan_tables")
        if buffers is not None:
            buffers.load(tab)
            dev, rw, run_W, run_depth = buffers.tab, buffers.rw, buffers.workers, buffers.depth
        else:
            on_gpu = self.device.type == "cuda"
            host = torch.from_numpy(tab)
            if on_gpu:
                host = host.pin_memory()
            dev = host.to(self.device, non_blocking=True)
            keep.append(host)
            # per-layer rows of the six [W] address lists (read a/b/conv, write a/b/conv), compact
            rw = dev[2:8, :, :, 0].transpose(0, 1).contiguous()            # [L, 6, W]
            run_W, run_depth = W, depth
        return {"tab": dev, "rw": rw, "host": tab, "depth": run_depth, "W": run_W, "real_W": W, "layers": layers,
                "out_a": out_a, "out_b": out_b, "conv_out": conv_out,
                # layers whose conv window this forward writes: recorded by decode_pre / prefill_pre as they
                # run; a forward replayed from a graph runs no host code, so with fixed tables every layer counts
                "conv_layers": set(range(layers)) if (buffers is not None and with_outputs) else set(),
                "keep": keep, "targets": list(targets), "buffers": buffers}

    def _retire(self) -> None:
        self._pending = [(ev, refs) for ev, refs in self._pending if not ev.query()]

    # ------------------------------------------------------------------ decode
    def prepare_decode(self, layers: int, dtype: torch.dtype, *, buffers=None) -> None:
        """Snapshot every layer's chain / write-block addresses and allocate the output slabs."""
        if self._step is not None:
            raise RuntimeError("Previous GDN forward has not been published")
        if self.device.type == "cuda":
            self._retire()
        self._step = self._build_tables(layers, with_outputs=True, buffers=buffers)
        self.decode_buffers = buffers
        self._prepared_decode = True
        self.prepare_count += 1

    def _publish(self, success: bool) -> None:
        st = self._step
        if st is None:
            return
        if success:
            layers = st["layers"]
            # the new summaries' addresses are known without touching the tensors again: [W, L, 2]
            new_ptrs = np.ascontiguousarray(st["host"][ROW_WRITE_A:ROW_WRITE_B + 1, :, :, 0].transpose(2, 1, 0))
            conv_layers = sorted(st["conv_layers"])
            for w, target in enumerate(st["targets"]):
                slab_a = st["out_a"][w]
                slab_b = slab_a if st["out_b"] is None else st["out_b"][w]
                conv_slab = st["conv_out"][w]

                def affine_items(slab_a=slab_a, slab_b=slab_b):
                    if slab_b is slab_a:
                        rows = slab_a.unbind(0)
                        return zip(range(layers), zip(rows[:layers], rows[layers:]))
                    return zip(range(layers), zip(slab_a.unbind(0), slab_b.unbind(0)))

                def conv_items(conv_slab=conv_slab):
                    rows = conv_slab.unbind(0)
                    return [(layer, rows[layer]) for layer in conv_layers]

                affine, conv = target.linear_affine, target.linear_conv_state
                lazy = isinstance(affine, _TrackedDict) and isinstance(conv, _TrackedDict)
                if lazy:
                    # the per-layer views (48 + 24 tensor objects per worker) are only built if somebody
                    # reads the dictionaries; the kernels work from the addresses cached below
                    affine.defer(affine_items, range(layers))
                    if conv_layers:
                        conv.defer(conv_items, conv_layers)
                    full_a = affine.known_keys() == set(range(layers))
                    full_c = conv.known_keys() == set(range(layers))
                else:
                    affine.update(affine_items())
                    if conv_layers:
                        conv.update(conv_items())
                    full_a = len(affine) == layers
                    full_c = len(conv) == layers
                if not hasattr(target, "_gdn_revision"):
                    continue
                if full_a:
                    target._gdn_ptr_cache = (target._gdn_revision, (self.device, self.state_dtype), new_ptrs[w],
                                             [slab_a, slab_b])
                if len(conv_layers) == layers and full_c:
                    target._gdn_conv_cache = (target._gdn_revision, self.device,
                                              np.ascontiguousarray(st["host"][ROW_CONV_WRITE, :, w, 0]), [conv_slab])
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._pending.append((ev, st["keep"]))
        self._step = None

    def finish_decode(self, success: bool) -> None:
        if self._prepared_decode:
            self._publish(success)
            self._prepared_decode = False

    def decode_step(self, lin_idx: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                    g: torch.Tensor, beta: torch.Tensor, l2norm_eps: float = 1e-6) -> torch.Tensor:
        """One fused GDN decode step for layer ``lin_idx``.

        ``q,k [W, Hk or H, dk]``, ``v [W, H, dv]`` bf16 (post conv, NOT normalised), ``g,beta [W, H]``
        fp32.  Returns the core output ``[W, H, dv]``; the write blocks' new summaries go to the
        slabs allocated by ``prepare_decode`` and become visible at ``finish_decode(True)``.
        """
        if not self._prepared_decode:
            raise RuntimeError("decode_step needs prepare_decode first")
        if not q.is_cuda:
            raise RuntimeError("the GDN step kernel needs CUDA tensors: there is no CPU fallback")
        st = self._step
        W = st["W"]
        # rows of q / k / v are read where they lie (slices of a layer's [q | k | v] conv output)
        q, k, v = (t if (t.stride(2) == 1 and t.stride(1) == t.shape[2]) else t.contiguous() for t in (q, k, v))
        g32, b32 = g.float().contiguous(), beta.float().contiguous()
        out = torch.empty(W, self.num_heads, self.head_v_dim, dtype=q.dtype, device=q.device)
        tab = st["tab"]
        a = _lib.VaGdnStep()
        a.q, a.k, a.v, a.g, a.beta, a.out = (t.data_ptr() for t in (q, k, v, g32, b32, out))
        a.q_row_stride, a.k_row_stride, a.v_row_stride = q.stride(0), k.stride(0), v.stride(0)
        a.summary_dtype = self._summary_code
        a.chain_a = tab[0, lin_idx].data_ptr()
        a.chain_b = tab[1, lin_idx].data_ptr()
        row = st["rw"].data_ptr() + lin_idx * 6 * W * 8                # [6, W] int64 rows of this layer
        a.read_a, a.read_b, a.write_a, a.write_b = (row + i * W * 8 for i in (0, 1, 3, 4))
        a.num_workers, a.depth = W, st["depth"]
        a.num_k_heads, a.num_v_heads = q.shape[1], self.num_heads
        a.head_k_dim, a.head_v_dim = self.head_k_dim, self.head_v_dim
        a.l2_eps, a.q_scale = l2norm_eps, self.head_k_dim ** -0.5
        a.status = None
        _lib.check(_lib.lib().va_gdn_step(C.byref(a), _lib.stream_ptr()), "va_gdn_step")
        st["keep"] += [q, k, v, g32, b32]
        return out

    def decode_pre(self, lin_idx: int, qkv: torch.Tensor, conv_weight: torch.Tensor, a: torch.Tensor,
                   b: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor):
        """Conv window + SiLU + gates of layer ``lin_idx`` for every worker's new token, reading each
        chain's most recent conv window and writing the write block's next one in place (no gather /
        scatter): what ``prior_conv_states`` + ``_decode_conv_silu`` + ``_gates`` + ``set_conv_states``
        do in the reference's eager path (minisgl/models/qwen3_5_delta.py:453-461,486; the prepared
        path's gather_rows / scatter_rows, minisgl/shared_cache/gdn_decode.py).  Returns
        ``(qkv_conv [W, conv_dim] bf16, beta [W, Hv] fp32, g [W, Hv] fp32)``; the new conv states
        become visible at ``finish_decode(True)``."""
        if not self._prepared_decode:
            raise RuntimeError("decode_pre needs prepare_decode first")
        if not qkv.is_cuda:
            raise RuntimeError("the GDN layer kernels need CUDA tensors: there is no CPU fallback")
        st = self._step
        W = st["W"]
        assert qkv.shape == (W, self.conv_dim) and qkv.dtype == torch.bfloat16
        if qkv.stride(1) != 1:
            qkv = qkv.contiguous()
        weight = conv_weight.reshape(self.conv_dim, -1).to(torch.bfloat16).contiguous()
        assert weight.shape[1] == self.conv_kernel
        Hv = self.num_heads
        # a / b are read where they lie (columns of the fused input projection)
        a2, b2 = (t if (t.dtype == torch.bfloat16 and t.dim() == 2 and t.shape == (W, Hv) and t.stride(1) == 1)
                  else t.reshape(W, Hv).to(torch.bfloat16).contiguous() for t in (a, b))
        a_log = A_log.to(device=self.device, dtype=torch.float32).contiguous()
        bias = dt_bias.to(device=self.device, dtype=torch.float32).contiguous()
        qkv_out = torch.empty(W, self.conv_dim, dtype=torch.bfloat16, device=self.device)
        beta16 = torch.empty(W, Hv, dtype=torch.bfloat16, device=self.device)
        beta = torch.empty(W, Hv, dtype=torch.float32, device=self.device)
        g = torch.empty(W, Hv, dtype=torch.float32, device=self.device)
        row = st["rw"].data_ptr() + lin_idx * 6 * W * 8
        args = _lib.VaGdnDecodePre()
        args.qkv, args.qkv_row_stride = qkv.data_ptr(), qkv.stride(0)
        args.prior_conv, args.conv_out = None, None
        args.prior_conv_ptrs, args.conv_out_ptrs = row + 2 * W * 8, row + 5 * W * 8
        args.conv_weight, args.a, args.b = weight.data_ptr(), a2.data_ptr(), b2.data_ptr()
        args.a_row_stride, args.b_row_stride = a2.stride(0), b2.stride(0)
        args.a_log, args.dt_bias = a_log.data_ptr(), bias.data_ptr()
        args.qkv_out, args.beta_out, args.beta_f32_out, args.g_out = (qkv_out.data_ptr(), beta16.data_ptr(),
                                                                      beta.data_ptr(), g.data_ptr())
        args.num_workers, args.conv_dim, args.conv_kernel, args.num_v_heads = W, self.conv_dim, self.conv_kernel, Hv
        _lib.check(_lib.lib().va_gdn_decode_pre(C.byref(args), _lib.stream_ptr()), "va_gdn_decode_pre")
        st["conv_layers"].add(lin_idx)
        st["keep"] += [qkv, weight, a2, b2, a_log, bias, beta16]
        return qkv_out, beta, g

    # ------------------------------------------------------------------ reference call sequence
    def compose_initial_recurrent_state(self, lin_idx: int, dtype: torch.dtype) -> Optional[torch.Tensor]:
        """``[W, H, dk, dv]`` initial state of every worker (None if no block has a summary)."""
        if not self.has_previous_affine(lin_idx):
            return None
        if self.device.type != "cuda":
            raise RuntimeError("the GDN compose kernel needs a CUDA device: there is no CPU fallback")
        st = self._step if self._step is not None else self._build_tables(lin_idx + 1, with_outputs=False)
        W = st["W"]
        state = torch.empty(W, self.num_heads, self.head_k_dim, self.head_v_dim, dtype=torch.float32,
                            device=self.device)
        rc = _lib.lib().va_gdn_compose(st["tab"][0, lin_idx].data_ptr(), st["tab"][1, lin_idx].data_ptr(),
                                       state.data_ptr(), W, st["depth"], self.num_heads,
                                       self.head_k_dim, self.head_v_dim, self._summary_code, _lib.stream_ptr())
        _lib.check(rc, "va_gdn_compose")
        if st is not self._step:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._pending.append((ev, st["keep"] + [st["tab"]]))
        return state.to(dtype=dtype)

    def prior_conv_states(self, lin_idx: int) -> Optional[torch.Tensor]:
        """Most recent conv window along each chain ``[W, conv_dim, k]`` (zeros where a chain has
        none; None when every chain is empty) -- minisgl/shared_cache/gdn.py:182-207."""
        found: List[Optional[torch.Tensor]] = []
        sample = None
        for chain in self.cache_structure:
            hit = None
            for block in reversed(chain):
                hit = block.linear_conv_state.get(lin_idx)
                if hit is not None:
                    break
            sample = hit if hit is not None else sample
            found.append(hit)
        if sample is None:
            return None
        zero = torch.zeros(self.conv_dim, self.conv_kernel, device=self.device, dtype=sample.dtype)
        return torch.stack([(c if c is not None else zero).to(self.device) for c in found], dim=0)

    def set_conv_states(self, lin_idx: int, conv: torch.Tensor, workers: Optional[Sequence[int]] = None) -> None:
        targets = self.write_to if workers is None else [self.write_to[w] for w in workers]
        for w, target in enumerate(targets):
            target.linear_conv_state[lin_idx] = conv[w].detach().clone()

    def capture_token_affines(self, lin_idx: int, key: torch.Tensor, value: torch.Tensor,
                              alpha: torch.Tensor, beta: torch.Tensor, l2norm_eps: float = 1e-6,
                              workers: Optional[Sequence[int]] = None) -> None:
        """Fold ``key/value [W, seq, H, d]``, ``alpha/beta [W, seq, H]`` into the write blocks'
        summaries (minisgl/shared_cache/gdn.py:213-269); published immediately, like the
        reference's eager path."""
        targets = self.write_to if workers is None else [self.write_to[w] for w in workers]
        W, seq, H, dk = key.shape
        keep: list = []
        init = np.zeros((4, W), dtype=np.int64)
        H_, dv = self.num_heads, self.head_v_dim
        out_a = [torch.empty(1, H_, dk, dk, dtype=self.state_dtype, device=self.device) for _ in targets]
        out_b = [torch.empty(1, H_, dv, dk, dtype=self.state_dtype, device=self.device) for _ in targets]
        for w, target in enumerate(targets):
            init[0, w], init[1, w] = self._pair_ptrs(target, lin_idx, keep)
            init[2, w], init[3, w] = out_a[w].data_ptr(), out_b[w].data_ptr()
        self._scan(key.reshape(W * seq, H, dk), key.reshape(W * seq, H, dk), value.reshape(W * seq, H, dv),
                   alpha.float().log().reshape(W * seq, H), beta.float().reshape(W * seq, H),
                   [seq] * W, None, init, l2norm_eps, want_out=False, keep=keep)
        for w, target in enumerate(targets):
            target.linear_affine[lin_idx] = (out_a[w], out_b[w])

    # ------------------------------------------------------------------ prefill
    def prepare_prefill(self, layers: int, dtype: torch.dtype, rows: int, *, buffers=None) -> None:
        if self._step is not None:
            raise RuntimeError("Previous GDN forward has not been published")
        if self.device.type == "cuda":
            self._retire()
        segments = list(self.prefill_segments or [rows])
        if buffers is not None:
            buffers.check_segments(segments)
        self._step = self._build_tables(layers, with_outputs=True, buffers=buffers)
        self._step["segments"] = segments
        if buffers is not None:
            buffers.load_segments(segments)
        else:
            # once per forward, from pinned memory: a copy from pageable memory would wait for the
            # stream's earlier kernels and serialise the host behind the GPU
            self._step["seg_d"] = self._upload_i32(np.concatenate(([0], np.cumsum(segments))))
        self.prefill_buffers = buffers
        self._prepared_prefill = True
        self.prepare_count += 1

    def finish_prefill(self, success: bool) -> None:
        if self._prepared_prefill:
            self._publish(success)
            self._prepared_prefill = False

    def _upload_i32(self, values) -> torch.Tensor:
        """A small host array as an int32 device tensor, staged through pinned memory."""
        host = torch.from_numpy(np.ascontiguousarray(values, dtype=np.int32))
        if self.device.type != "cuda":
            return host
        return host.pin_memory().to(self.device, non_blocking=True)

    def _init_rows(self) -> torch.Tensor:
        """Rows (read a, read b, write a, write b) of a layer's ``[6, W]`` address list."""
        if self._init_row_index is None:
            self._init_row_index = torch.tensor([0, 1, 3, 4], dtype=torch.int64, device=self.device)
        return self._init_row_index

    def _scan(self, q, k, v, g, beta, segments, state0, init, eps, want_out=True, keep=None,
              final_state=None, engine="scan", buffers=None):
        if not q.is_cuda:
            raise RuntimeError("the GDN scan kernel needs CUDA tensors: there is no CPU fallback")
        # dense rows, fetched by the chunk engines as 16-byte pieces
        q, k, v = (t if t.data_ptr() % 16 == 0 else t.clone() for t in (q.contiguous(), k.contiguous(), v.contiguous()))
        g32, b32 = g.float().contiguous(), beta.float().contiguous()
        N = q.shape[0]
        out = torch.empty(N, self.num_heads, self.head_v_dim, dtype=v.dtype, device=v.device)
        if buffers is not None:
            # fixed capacity: the offsets sit at a fixed address, requests beyond the batch are empty
            # ranges, rows beyond the last request are left alone
            if N > buffers.rows:
                raise ValueError(f"{N} token rows exceed the prepared capacity {buffers.rows}")
            seg_d = buffers.seg
        else:
            st = self._step
            if st is not None and segments is st.get("segments") and st.get("seg_d") is not None:
                seg_d = st["seg_d"]          # the prepared forward's own offsets, uploaded once
            else:
                seg_d = self._upload_i32(np.concatenate(([0], np.cumsum(segments))))
        if isinstance(init, torch.Tensor):
            init_t = init
        else:
            init_t = torch.from_numpy(init)
            if self.device.type == "cuda":
                init_t = init_t.pin_memory().to(self.device, non_blocking=True)
        a = _lib.VaGdnPrefill()
        a.q, a.k, a.v, a.g, a.beta, a.out = (t.data_ptr() for t in (q, k, v, g32, b32, out))
        a.seg_off = seg_d.data_ptr()
        a.state0 = state0.data_ptr() if state0 is not None else None
        a.init_a, a.init_b, a.write_a, a.write_b = (init_t[i].data_ptr() for i in range(4))
        a.final_state = final_state.data_ptr() if final_state is not None else None
        a.num_requests = len(segments) if buffers is None else buffers.workers
        a.num_k_heads, a.num_v_heads = q.shape[1], self.num_heads
        a.head_k_dim, a.head_v_dim = self.head_k_dim, self.head_v_dim
        a.l2_eps, a.q_scale = eps, self.head_k_dim ** -0.5
        a.engine = GDN_ENGINES[engine]
        a.summary_dtype = self._summary_code
        a.status = self.status().data_ptr()
        a.num_tokens = N
        a.max_segment_tokens = (int(max(segments)) if len(segments) else 0) if buffers is None else N
        if engine != "scan" and buffers is not None:
            a.scratch, a.scratch_bytes = buffers.scratch.data_ptr(), buffers.scratch.numel()
        elif engine != "scan" and N > 0:
            # scratch of the chunk pre-pass (K, Q, -W, U, P rows per token and head), kept and grown
            need = int(_lib.lib().va_gdn_prefill_scratch_bytes(N, self.num_heads))
            if self._chunk_scratch is None or self._chunk_scratch.numel() < need:
                self._chunk_scratch = torch.empty(max(need, 1), dtype=torch.uint8, device=self.device)
            a.scratch, a.scratch_bytes = self._chunk_scratch.data_ptr(), self._chunk_scratch.numel()
        _lib.check(_lib.lib().va_gdn_prefill(C.byref(a), _lib.stream_ptr()), "va_gdn_prefill")
        if keep is not None:
            keep += [q, k, v, g32, b32, seg_d, init_t]
        return out if want_out else None

    def prefill_pre(self, lin_idx: int, qkv: torch.Tensor, conv_weight: torch.Tensor) -> torch.Tensor:
        """Causal conv + SiLU of layer ``lin_idx`` over the prepared requests' rows, each request
        preceded by its chain's most recent conv window, and the write blocks' next windows -- what
        ``_forward_ar_prefill_one`` does request by request with ``prior_conv_states`` /
        ``_prefill_conv_silu`` / ``set_conv_states`` (minisgl/models/qwen3_5_delta.py:399-437), and
        ``GDNPrefillBuffers.convolve`` in the prepared path (minisgl/shared_cache/gdn_prefill.py:63-65).
        ``qkv [N, conv_dim]`` bf16, rows request-major.  Returns ``qkv_conv [N, conv_dim]``; the new
        windows become visible at ``finish_prefill(True)``."""
        if not self._prepared_prefill:
            raise RuntimeError("prefill_pre needs prepare_prefill first")
        if not qkv.is_cuda:
            raise RuntimeError("the GDN layer kernels need CUDA tensors: there is no CPU fallback")
        st = self._step
        W = st["W"]
        N = qkv.shape[0]
        assert qkv.shape[1] == self.conv_dim and qkv.dtype == torch.bfloat16
        if qkv.stride(1) != 1:
            qkv = qkv.contiguous()
        weight = conv_weight.reshape(self.conv_dim, -1).to(torch.bfloat16).contiguous()
        assert weight.shape[1] == self.conv_kernel
        buffers = st["buffers"]
        if buffers is not None:
            seg_d = buffers.seg
        else:
            assert sum(st["segments"]) == N, "prefill segments do not cover the batch"
            seg_d = st["seg_d"]
        qkv_out = torch.empty(N, self.conv_dim, dtype=torch.bfloat16, device=self.device)
        if buffers is not None:
            qkv_out.zero_()    # rows beyond the planned batch are not written by the kernel
        row = st["rw"].data_ptr() + lin_idx * 6 * W * 8
        args = _lib.VaGdnPrefillConv()
        args.qkv, args.qkv_row_stride = qkv.data_ptr(), qkv.stride(0)
        args.prior_conv, args.conv_out = None, None
        args.prior_conv_ptrs, args.conv_out_ptrs = row + 2 * W * 8, row + 5 * W * 8
        args.conv_weight, args.seg_off = weight.data_ptr(), seg_d.data_ptr()
        args.qkv_out = qkv_out.data_ptr()
        args.num_requests, args.num_tokens, args.conv_dim, args.conv_kernel = W, N, self.conv_dim, self.conv_kernel
        _lib.check(_lib.lib().va_gdn_prefill_conv(C.byref(args), _lib.stream_ptr()), "va_gdn_prefill_conv")
        st["conv_layers"].add(lin_idx)
        st["keep"] += [qkv, weight, seg_d]
        return qkv_out

    def prefill_scan(self, lin_idx: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     g: torch.Tensor, beta: torch.Tensor, l2norm_eps: float = 1e-6,
                     final_state: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Fused GDN prefill of layer ``lin_idx`` over the prepared requests.

        ``q,k [N, Hk or H, dk]``, ``v [N, H, dv]``, ``g,beta [N, H]`` with rows request-major
        (``prefill_segments``).  Composes every request's initial state from its chain, scans its
        tokens, returns the core output ``[N, H, dv]`` and leaves each write block's new summary in
        the slabs published by ``finish_prefill(True)``.
        """
        if not self._prepared_prefill:
            raise RuntimeError("prefill_scan needs prepare_prefill first")
        st = self._step
        state0 = None
        # (a fixed-capacity step always composes: whether any chain carries a summary may change
        # between replays; a chain without one composes to zeros)
        if st["buffers"] is not None or self.has_previous_affine(lin_idx):
            state0 = torch.empty(st["W"], self.num_heads, self.head_k_dim, self.head_v_dim,
                                 dtype=torch.float32, device=self.device)
            rc = _lib.lib().va_gdn_compose(st["tab"][0, lin_idx].data_ptr(), st["tab"][1, lin_idx].data_ptr(),
                                           state0.data_ptr(), st["W"], st["depth"], self.num_heads,
                                           self.head_k_dim, self.head_v_dim, self._summary_code, _lib.stream_ptr())
            _lib.check(rc, "va_gdn_compose")
        init = st["rw"][lin_idx].index_select(0, self._init_rows())    # read a/b, write a/b: [4, W]
        return self._scan(q, k, v, g, beta, st["segments"], state0, init, l2norm_eps, keep=st["keep"],
                          final_state=final_state, engine=self.prefill_engine, buffers=st["buffers"])


__all__ = ["SharedCacheGDN", "GDNDecodeBuffers", "GDNPrefillBuffers"]
