"""KV pool and page allocator behind the reference's pool interface.

* ``BaseKVCachePool`` / ``MHAKVCache`` -- minisgl/kvcache/base.py:10-37, mha_pool.py:10-68
* ``PageAllocator``                    -- minisgl/kvcache/page_allocator.py:6-62

Layout in HBM: one allocation ``[2, layers, num_pages, page_size, Hkv, D]`` bf16, so
``k_cache(i)`` / ``v_cache(i)`` are contiguous ``[num_pages, page_size, Hkv, D]`` views that callers
may reshape to ``[-1, Hkv, D]`` or index_copy_ into, exactly as with the reference pool.  A token
row (one head) is ``D*2`` contiguous bytes; the kernels fetch it in 16-byte pieces.
``store_kv`` runs the rotate-and-store CUDA kernel; there is no torch fallback.
"""

from __future__ import annotations

import ctypes as C
from abc import ABC, abstractmethod
from typing import List, Optional

import numpy as np
import torch

from . import _lib


class BaseKVCachePool(ABC):
    @abstractmethod
    def k_cache(self, index: int) -> torch.Tensor: ...

    @abstractmethod
    def v_cache(self, index: int) -> torch.Tensor: ...

    @abstractmethod
    def store_kv(self, k: torch.Tensor, v: torch.Tensor, out_loc: torch.Tensor, layer_id: int) -> None: ...

    @property
    @abstractmethod
    def device(self) -> torch.device: ...

    @property
    @abstractmethod
    def dtype(self) -> torch.dtype: ...

    @property
    @abstractmethod
    def num_layers(self) -> int: ...


class MHAKVCache(BaseKVCachePool):
    """Paged multi-head KV pool (same constructor arguments as the reference pool)."""

    def __init__(
        self,
        num_kv_heads: int,
        num_layers: int,
        head_dim: int,
        num_pages: int,
        page_size: int,
        dtype: torch.dtype,
        device: torch.device,
    ) -> None:
        if dtype != torch.bfloat16:
            raise ValueError("the B200 view-attention kernels store the KV pool in bfloat16")
        self._buf = torch.empty(
            (2, num_layers, num_pages, page_size, num_kv_heads, head_dim), dtype=dtype, device=device
        )
        self._layers = num_layers
        self._device = torch.device(device)
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.num_pages = num_pages
        self.page_size = page_size
        self._status: Optional[torch.Tensor] = None
        self._pool_structs = {}   # C descriptions of the layers, see pool_struct

    def k_cache(self, index: int) -> torch.Tensor:
        return self._buf[0, index]

    def v_cache(self, index: int) -> torch.Tensor:
        return self._buf[1, index]

    def store_kv(self, k: torch.Tensor, v: torch.Tensor, out_loc: torch.Tensor, layer_id: int) -> None:
        """Scatter ``k``/``v`` rows ``[n, Hkv*D]`` to slots ``out_loc`` (negative slot = skip).

        Keys are stored as given (already rotated by the caller), as in the reference's
        ``store_cache`` (minisgl/kernel/store.py:30-42).
        """
        store_rows(self, k, v, out_loc, layer_id, positions=None, cos_sin=None, rotary_dim=None)

    @property
    def device(self) -> torch.device:
        return self._device

    @property
    def dtype(self) -> torch.dtype:
        return self._buf.dtype

    @property
    def num_layers(self) -> int:
        return self._layers


_DUMMY_COS_SIN = {}


def pool_struct(kv_cache, layer_id: int, num_q_heads: int, cos_sin: Optional[torch.Tensor],
                rotary_dim: Optional[int], sm_scale: Optional[float] = None) -> _lib.VaPool:
    """Describe one layer of a pool (any object with ``k_cache``/``v_cache``) to the C ABI.

    An ``MHAKVCache`` keeps the descriptions of its layers between calls (its buffer never moves)."""
    cache = getattr(kv_cache, "_pool_structs", None)
    if cache is None:
        return _describe_pool(kv_cache, layer_id, num_q_heads, cos_sin, rotary_dim, sm_scale)
    key = (layer_id, num_q_heads, id(cos_sin), rotary_dim, sm_scale)
    hit = cache.get(key)
    if hit is not None and hit[1] is cos_sin:
        return hit[0]
    p = _describe_pool(kv_cache, layer_id, num_q_heads, cos_sin, rotary_dim, sm_scale)
    cache[key] = (p, cos_sin)
    return p


def _describe_pool(kv_cache, layer_id, num_q_heads, cos_sin, rotary_dim, sm_scale) -> _lib.VaPool:
    kc = kv_cache.k_cache(layer_id)
    vc = kv_cache.v_cache(layer_id)
    assert kc.is_contiguous() and vc.is_contiguous(), "per-layer pool views must be contiguous"
    pages, page_size, hkv, d = kc.shape
    if cos_sin is None:
        key = (kc.device, d)
        if key not in _DUMMY_COS_SIN:
            row = torch.zeros(1, d, dtype=torch.float32, device=kc.device)
            row[:, : d // 2] = 1.0
            _DUMMY_COS_SIN[key] = row
        cos_sin = _DUMMY_COS_SIN[key]
        rotary_dim = d
    assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
    rd = int(rotary_dim if rotary_dim is not None else d)
    assert cos_sin.shape[1] == rd, "cos_sin_cache must be [max_pos, rotary_dim]"
    p = _lib.VaPool()
    p.k = kc.data_ptr()
    p.v = vc.data_ptr()
    p.num_slots = pages * page_size
    p.page_size = page_size
    p.num_q_heads = num_q_heads
    p.num_kv_heads = hkv
    p.head_dim = d
    p.rotary_dim = rd
    p.max_pos = cos_sin.shape[0]
    p.cos_sin = cos_sin.data_ptr()
    p.sm_scale = float(sm_scale if sm_scale is not None else d ** -0.5)
    return p


def store_rows(kv_cache, k, v, out_loc, layer_id, positions, cos_sin, rotary_dim,
               status: Optional[torch.Tensor] = None, mrope_lims=None) -> None:
    """Rotate ``k`` at ``positions`` (or not, when ``positions`` is None) and scatter k, v.

    With ``mrope_lims = (3*section[1], 3*section[2])`` the rotation is the interleaved 3-axis
    mRoPE and ``positions`` is ``[n]`` or ``[3, n]``."""
    n = k.shape[0]
    if n == 0:
        return
    if not k.is_cuda:
        raise RuntimeError("store_kv needs CUDA tensors: the cache-view path has no CPU fallback")
    k2 = k.reshape(n, -1)
    v2 = v.reshape(n, -1)
    if k2.stride(1) != 1:
        k2 = k2.contiguous()
    if v2.stride(1) != 1:
        v2 = v2.contiguous()
    loc = out_loc if out_loc.dtype == torch.int32 else out_loc.to(torch.int32)
    pos_ptr = None
    if positions is not None:
        pos = positions if positions.dtype == torch.int32 else positions.to(torch.int32)
        pos_ptr = pos.data_ptr()
    hkv = getattr(kv_cache, "num_kv_heads", None) or kv_cache.k_cache(layer_id).shape[2]
    pool = pool_struct(kv_cache, layer_id, hkv, cos_sin, rotary_dim)
    status_ptr = status.data_ptr() if status is not None else None
    if mrope_lims is not None and positions is not None:
        axes = 3 if pos.dim() == 2 else 1
        assert pos.is_contiguous() and pos.shape[-1] == n and (axes == 1 or pos.shape[0] == 3)
        rc = _lib.lib().va_store_kv_mrope(
            C.byref(pool), k2.data_ptr(), k2.stride(0), v2.data_ptr(), v2.stride(0), pos_ptr, axes,
            loc.data_ptr(), n, mrope_lims[0], mrope_lims[1], status_ptr, _lib.stream_ptr(),
        )
        _lib.check(rc, "va_store_kv_mrope")
        return
    rc = _lib.lib().va_store_kv(
        C.byref(pool), k2.data_ptr(), k2.stride(0), v2.data_ptr(), v2.stride(0), pos_ptr,
        loc.data_ptr(), n, status_ptr, _lib.stream_ptr(),
    )
    _lib.check(rc, "va_store_kv")


class PageAllocator:
    """Free list of page-start slots ``[0, P, 2P, ...]`` kept as a device int32 tensor
    (minisgl/kvcache/page_allocator.py:6-62), with a host copy of the same list beside it.

    ``alloc_pages(n)`` takes the first ``n`` entries, ``free_pages`` appends; exhaustion raises
    ``RuntimeError`` before anything is handed out.  ``alloc_page_list(n)`` is the same allocation
    answered from the host copy: the write planner needs the page numbers as Python ints, and
    reading them back from the device tensor waits for everything queued on the stream (a decode
    step that crossed a page boundary lost the overlap of its planning with the previous step).
    """

    def __init__(self, num_pages: int, page_size: int, device: torch.device) -> None:
        self.num_pages = num_pages
        self.page_size = page_size
        self.device = device
        self._free_host = np.arange(num_pages, dtype=np.int32) * page_size
        self._free = torch.from_numpy(self._free_host.copy()).to(device)

    @property
    def num_free_pages(self) -> int:
        return self._free.numel()

    @property
    def free_page_starts(self) -> torch.Tensor:
        return self._free

    def pages_to_tokens(self, page_starts: torch.Tensor) -> torch.Tensor:
        if self.page_size == 1:
            return page_starts
        lane = torch.arange(self.page_size, dtype=page_starts.dtype, device=page_starts.device)
        return (page_starts.unsqueeze(1) + lane.unsqueeze(0)).reshape(-1)

    def _take(self, num_pages: int):
        have = self.num_free_pages
        if num_pages > have:
            raise RuntimeError(
                f"PageAllocator out of pages: requested {num_pages}, only {have} free"
            )
        taken, self._free = self._free[:num_pages], self._free[num_pages:]
        host, self._free_host = self._free_host[:num_pages], self._free_host[num_pages:]
        return taken, host

    def alloc_pages(self, num_pages: int) -> torch.Tensor:
        return self._take(num_pages)[0].clone()

    def alloc_page_list(self, num_pages: int) -> List[int]:
        """``alloc_pages(num_pages)`` as a list of ints, without touching the device."""
        return self._take(num_pages)[1].tolist()

    def free_pages(self, page_starts) -> None:
        """Give pages back: a tensor (device or host) or a sequence of page-start slots."""
        if isinstance(page_starts, torch.Tensor):
            if page_starts.numel() == 0:
                return
            host = page_starts.detach().to("cpu", torch.int32).numpy()
            back = page_starts.to(device=self._free.device, dtype=self._free.dtype)
        else:
            host = np.asarray(list(page_starts), dtype=np.int32)
            if host.size == 0:
                return
            back = torch.from_numpy(host).to(self._free.device)
        self._free = torch.cat((self._free, back))
        self._free_host = np.concatenate((self._free_host, host))
