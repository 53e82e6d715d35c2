"""The gated full-attention layer around the view attention: counterpart of ``Qwen3_5Attention.forward``
on the shared-cache path (minisgl/models/qwen3_5_attn.py:100-137).

The projections stay plain GEMMs.  Between them the reference runs a split, two ``contiguous`` copies,
two per-head RMSNorm calls (FlashInfer ``gemma_rmsnorm``), the attention op, and the sigmoid output
gate as three eager ops; here ``qk_norm`` (one launch: q and k normalised straight out of the fused
projection rows) and ``output_gate`` (one launch, the gate read where the projection left it) stand
either side of ``SharedCacheAttention.forward``.
"""

from __future__ import annotations

import ctypes as C
from typing import Tuple

import torch

from . import _lib


def _need_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} runs a CUDA kernel: there is no CPU fallback")


def qk_norm(qkv: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor, num_q_heads: int, num_kv_heads: int,
            head_dim: int, eps: float, weight_plus_one: bool = True) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``qkv [n, (2*Hq + 2*Hkv) * D]`` bf16 rows of the fused projection, laid out
    ``[head: q | gate] * Hq, k heads, v heads``.  Returns ``(q [n, Hq*D], k [n, Hkv*D], v)`` with q and k
    RMS-normalised per head (``weight`` fp32 ``[D]``, ``1 + weight`` when ``weight_plus_one``); ``v`` is a
    view of the rows."""
    _need_cuda(qkv, "qk_norm")
    if qkv.dtype != torch.bfloat16:
        raise NotImplementedError("the attention layer kernels take bfloat16 activations")
    n = qkv.shape[0]
    width = (2 * num_q_heads + 2 * num_kv_heads) * head_dim
    assert qkv.shape[1] == width, f"qkv rows must be {width} wide"
    if qkv.stride(1) != 1:
        qkv = qkv.contiguous()
    q = torch.empty(n, num_q_heads * head_dim, dtype=torch.bfloat16, device=qkv.device)
    k = torch.empty(n, num_kv_heads * head_dim, dtype=torch.bfloat16, device=qkv.device)
    a = _lib.VaAttnQkNorm()
    a.qkv, a.qkv_row_stride = qkv.data_ptr(), qkv.stride(0)
    a.q_weight, a.k_weight = q_weight.data_ptr(), k_weight.data_ptr()
    assert q_weight.dtype == torch.float32 and k_weight.dtype == torch.float32 and q_weight.is_cuda
    a.q_out, a.k_out = q.data_ptr(), k.data_ptr()
    a.n, a.num_q_heads, a.num_kv_heads, a.head_dim = n, num_q_heads, num_kv_heads, head_dim
    a.eps, a.weight_plus_one = float(eps), int(bool(weight_plus_one))
    _lib.check(_lib.lib().va_attn_qk_norm(C.byref(a), _lib.stream_ptr()), "va_attn_qk_norm")
    v = qkv[:, (2 * num_q_heads + num_kv_heads) * head_dim:]
    return q, k, v


def output_gate(o: torch.Tensor, qkv: torch.Tensor, num_q_heads: int, head_dim: int) -> torch.Tensor:
    """``bf16(float(o) * sigmoid(float(gate)))`` with ``o [n, Hq*D]`` and the gate read in place from the
    projection rows ``qkv`` (``_sigmoid_output_gate``, minisgl/models/qwen3_5_attn.py:21-23)."""
    _need_cuda(o, "output_gate")
    n = o.shape[0]
    o2 = o.reshape(n, num_q_heads * head_dim).contiguous()
    out = torch.empty_like(o2)
    rc = _lib.lib().va_attn_output_gate(o2.data_ptr(), qkv.data_ptr(), qkv.stride(0), out.data_ptr(), n, num_q_heads,
                                        head_dim, _lib.stream_ptr())
    _lib.check(rc, "va_attn_output_gate")
    return out


class GatedAttentionLayer:
    """``forward(x, batch)``: fused projection GEMM -> ``qk_norm`` -> the batch's view attention op
    (unrotated q / k, as the reference passes them) -> ``output_gate`` -> output projection.

    ``w_qkv [(2*Hq + 2*Hkv) * D, hidden]``, ``w_o [hidden, Hq*D]`` bf16; ``q_norm``, ``k_norm`` ``[D]`` in the
    checkpoint's ``weight`` form (the layer computes with ``1 + weight``)."""

    def __init__(self, kv_idx: int, num_q_heads: int, num_kv_heads: int, head_dim: int, w_qkv: torch.Tensor,
                 w_o: torch.Tensor, q_norm: torch.Tensor, k_norm: torch.Tensor, eps: float = 1e-6,
                 weight_plus_one: bool = True) -> None:
        self.kv_idx, self.num_q_heads, self.num_kv_heads, self.head_dim = kv_idx, num_q_heads, num_kv_heads, head_dim
        self.w_qkv, self.w_o = w_qkv, w_o
        self.q_norm = q_norm.to(device=w_qkv.device, dtype=torch.float32).contiguous()
        self.k_norm = k_norm.to(device=w_qkv.device, dtype=torch.float32).contiguous()
        self.eps, self.weight_plus_one = float(eps), bool(weight_plus_one)

    def forward(self, x: torch.Tensor, batch) -> torch.Tensor:
        qkv = torch.nn.functional.linear(x, self.w_qkv)
        q, k, v = qk_norm(qkv, self.q_norm, self.k_norm, self.num_q_heads, self.num_kv_heads, self.head_dim, self.eps,
                          self.weight_plus_one)
        o = batch.attn_metadata.shared_cache_op.forward(q, k, v, self.kv_idx, batch)
        return torch.nn.functional.linear(output_gate(o, qkv, self.num_q_heads, self.head_dim), self.w_o)


__all__ = ["qk_norm", "output_gate", "GatedAttentionLayer"]
