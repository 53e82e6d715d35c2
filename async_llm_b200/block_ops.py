"""Block merge and append: the KV copy, the key re-rotation and the GDN summary composition.

Drop-in for ``SharedCacheSession.merge_blocks`` / ``append_block`` / ``create_block`` /
``free_block`` (minisgl/shared_cache/session.py:317-528), as a small class a session delegates
to.  The block bookkeeping (page allocation, token ids, span override, which summaries are cloned
and which are kept) is the reference's; the data movement is two C calls instead of Python loops
over the layers: ``va_block_copy`` (K/V rows of every layer, right-hand keys rotated by the left
block's span on the way) and ``va_gdn_compose_pairs`` (``A = A1 A2``, ``B = B1 A2 + B2`` of every
layer that both blocks summarise).
"""

from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from .blocks import CacheBlock
from .kvpool import pool_struct


def _div_ceil(a: int, b: int) -> int:
    return -(-a // b)


class BlockOps:
    """``kv_cache``: a pool with ``k_cache(layer)`` / ``v_cache(layer)`` / ``num_layers``;
    ``page_allocator``: ``alloc_pages(n) -> int32 tensor of page starts`` and ``free_pages``;
    ``sc_attn``: the ``SharedCacheAttention`` of the session (its cos/sin table and rotary_dim
    drive the key rotation)."""

    def __init__(self, kv_cache, page_allocator, sc_attn, page_size: int, device,
                 state_dtype: torch.dtype = torch.float32) -> None:
        # storage type of the GDN summaries; composed in fp32, bf16 results rounded once after the
        # fp32 add (minisgl/shared_cache/gdn_affine.py:113-122)
        self._summary_code = _lib.summary_code(state_dtype)
        self.state_dtype = state_dtype
        self.kv_cache = kv_cache
        self.page_allocator = page_allocator
        self.sc_attn = sc_attn
        self.page_size = int(page_size)
        self.device = torch.device(device)
        self._layers: Optional[Tuple[int, int]] = None   # (num_layers per call, layer stride)

    # ------------------------------------------------------------------ blocks
    def create_block(self) -> CacheBlock:
        return CacheBlock(self.device, page_size=self.page_size)

    def free_block(self, block: CacheBlock) -> None:
        """Return a block's pages to the page allocator and reset it."""
        self._validate_block(block)
        page_starts = block.clear()
        if page_starts:
            self.page_allocator.free_pages(torch.tensor(page_starts, dtype=torch.int32, device=self.device))

    def _validate_block(self, block: CacheBlock) -> None:
        if torch.device(block.device) != self.device:
            raise ValueError("block must belong to this session's device")
        if block.page_size != self.page_size:
            raise ValueError("block must use this session's page size")

    # ------------------------------------------------------------------ merge / append
    @torch.inference_mode()
    def merge_blocks(self, left: CacheBlock, right: CacheBlock) -> CacheBlock:
        """Copy ``left + right`` into a new compact block; both inputs stay valid and unchanged
        (minisgl/shared_cache/session.py:330-376)."""
        self._validate_block(left)
        self._validate_block(right)
        left_tokens, right_tokens = left.num_tokens, right.num_tokens
        left_span, right_span = left.mrope_span, right.mrope_span
        total = left_tokens + right_tokens

        merged = self.create_block()
        num_pages = _div_ceil(total, self.page_size)
        if num_pages:
            merged.page_starts = self.page_allocator.alloc_pages(num_pages).tolist()
        merged.num_tokens = total
        if total:
            parts = [b.token_slots_tensor() for b in (left, right) if b.num_tokens]
            source = parts[0] if len(parts) == 1 else torch.cat(parts)
            self._copy_slots(source, merged.token_slots_tensor(), shift_begin=left_tokens,
                             shift=left_span if right_tokens else 0)
        self._finish_block_merge(merged, left, right, left_span, right_span, keep_left_state=False)
        return merged

    @torch.inference_mode()
    def append_block(self, left: CacheBlock, right: CacheBlock) -> CacheBlock:
        """Append a copy of ``right`` to ``left`` and return ``left``; free slots of ``left``'s last
        page are filled first.  ``append_block(block, block)`` duplicates ``block`` in place
        (minisgl/shared_cache/session.py:378-420)."""
        self._validate_block(left)
        self._validate_block(right)
        left_tokens, right_tokens = left.num_tokens, right.num_tokens
        left_span, right_span = left.mrope_span, right.mrope_span
        if right_tokens:
            # the source layout is captured before ``left`` grows: with left is right, growing
            # changes the slots token_slots_tensor returns
            source = right.token_slots_tensor()
            new_pages = self.page_allocator.alloc_pages(left.pages_needed(right_tokens))
            left.grow_pages(new_pages, right_tokens)
            dest = left.token_slots_tensor()[left_tokens: left_tokens + right_tokens]
            self._copy_slots(source, dest, shift_begin=0, shift=left_span)
        self._finish_block_merge(left, left, right, left_span, right_span, keep_left_state=True)
        return left

    # ------------------------------------------------------------------ data movement
    def _layer_layout(self) -> Tuple[int, int]:
        """(layers one call covers, elements between layers): all layers at once when the pool is
        one evenly strided buffer, else layer by layer."""
        if self._layers is None:
            n = self.kv_cache.num_layers
            k0, v0 = self.kv_cache.k_cache(0), self.kv_cache.v_cache(0)
            layout = (1, k0.numel())
            if n > 1:
                esz = k0.element_size()
                dk = self.kv_cache.k_cache(1).data_ptr() - k0.data_ptr()
                dv = self.kv_cache.v_cache(1).data_ptr() - v0.data_ptr()
                even = dk == dv and dk >= k0.numel() * esz and dk % (8 * esz) == 0 and all(
                    self.kv_cache.k_cache(i).data_ptr() == k0.data_ptr() + i * dk
                    and self.kv_cache.v_cache(i).data_ptr() == v0.data_ptr() + i * dv for i in range(2, n))
                if even:
                    layout = (n, dk // esz)
            self._layers = layout
        return self._layers

    def _copy_slots(self, source: torch.Tensor, dest: torch.Tensor, shift_begin: int, shift: int) -> None:
        """K/V rows of every layer from ``source`` slots to ``dest`` slots; keys of tokens
        ``[shift_begin, n)`` rotated by ``shift`` positions."""
        n = int(source.numel())
        assert int(dest.numel()) == n
        if n == 0:
            return
        if not source.is_cuda:
            raise RuntimeError("block merge runs the CUDA copy kernel: there is no CPU fallback")
        src = source.to(torch.int32).contiguous()
        dst = dest.to(torch.int32).contiguous()
        a = self.sc_attn
        per_call, stride = self._layer_layout()
        status = a.status()
        for layer in range(0, self.kv_cache.num_layers, per_call):
            pool = pool_struct(self.kv_cache, layer, a.num_qo_heads, a._cos_sin, a.rotary_dim)
            rc = _lib.lib().va_block_copy(C.byref(pool), per_call, stride, src.data_ptr(), dst.data_ptr(), n,
                                          shift_begin, shift, status.data_ptr(), _lib.stream_ptr())
            _lib.check(rc, "va_block_copy")

    def _compose_pairs(self, pairs):
        """``[(A1, B1, A2, B2)] -> [(A, B)]`` with ``A = A1 A2``, ``B = B1 A2 + B2``, one launch."""
        if not pairs:
            return []
        outs, keep = [], []
        rows = [[], [], [], [], [], []]
        heads, dv, dk = pairs[0][1].shape[-3:]
        for a1, b1, a2, b2 in pairs:
            tensors = [t.to(device=self.device, dtype=self.state_dtype).contiguous() for t in (a1, b1, a2, b2)]
            if not tensors[0].is_cuda:
                raise RuntimeError("block merge runs the CUDA compose kernel: there is no CPU fallback")
            out_a, out_b = torch.empty_like(tensors[0]), torch.empty_like(tensors[1])
            keep.append(tensors)
            outs.append((out_a, out_b))
            for row, t in zip(rows, (*tensors, out_a, out_b)):
                row.append(t.data_ptr())
        table = torch.tensor(rows, dtype=torch.int64).to(self.device)
        rc = _lib.lib().va_gdn_compose_pairs(*(table[i].data_ptr() for i in range(6)), len(pairs), heads, dk, dv,
                                             self._summary_code, _lib.stream_ptr())
        _lib.check(rc, "va_gdn_compose_pairs")
        return outs

    def _finish_block_merge(self, destination: CacheBlock, left: CacheBlock, right: CacheBlock,
                            left_span: int, right_span: int, keep_left_state: bool) -> None:
        """Token ids, span override and recurrent state of the result
        (minisgl/shared_cache/session.py:422-480)."""
        left_token_ids = list(left.token_ids)
        destination.token_ids = [*left_token_ids, *right.token_ids]
        merged_span = left_span + right_span
        destination.mrope_span_override = None if merged_span == destination.num_tokens else merged_span

        merged_affine: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        both = []
        for layer in sorted(set(left.linear_affine) | set(right.linear_affine)):
            lp, rp = left.linear_affine.get(layer), right.linear_affine.get(layer)
            if lp is None:
                merged_affine[layer] = (rp[0].clone(), rp[1].clone())
            elif rp is None:
                merged_affine[layer] = lp if keep_left_state else (lp[0].clone(), lp[1].clone())
            else:
                both.append((layer, lp, rp))
        composed = self._compose_pairs([(lp[0], lp[1], rp[0], rp[1]) for _, lp, rp in both])
        for (layer, lp, _), (out_a, out_b) in zip(both, composed):
            merged_affine[layer] = (out_a.view_as(lp[0]), out_b.view_as(lp[1]))

        merged_conv: Dict[int, torch.Tensor] = {}
        for layer in sorted(set(left.linear_conv_state) | set(right.linear_conv_state)):
            right_state = right.linear_conv_state.get(layer)
            left_state = left.linear_conv_state.get(layer)
            state = right_state if right_state is not None else left_state
            merged_conv[layer] = state if keep_left_state and right_state is None else state.clone()
        destination._replace_linear_states(merged_affine, merged_conv)
