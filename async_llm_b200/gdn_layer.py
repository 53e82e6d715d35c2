"""The elementwise steps of a Gated DeltaNet layer either side of the recurrent core, fused.

``decode_conv_gates`` and ``gated_rmsnorm`` are what ``Qwen3_5GatedDeltaNet._forward_ar_decode``
(minisgl/models/qwen3_5_delta.py:443-489) computes between its projections and the recurrent step
and between the step and the output projection; each is one C call here
(``va_gdn_decode_pre``, ``va_gdn_gated_rmsnorm``) instead of a chain of eager torch launches.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib


def _need_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} runs a CUDA kernel: there is no CPU fallback")


def decode_conv_gates(qkv: torch.Tensor, prior_conv: Optional[torch.Tensor], conv_weight: torch.Tensor,
                      a: torch.Tensor, b: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor,
                      beta_f32: bool = False) -> Tuple[torch.Tensor, ...]:
    """One decode token per worker.

    ``qkv [W, conv_dim]`` bf16 (rows may be strided), ``prior_conv [W, conv_dim, k]`` bf16 or None
    (zeros), ``conv_weight [conv_dim, 1, k]`` (the checkpoint layout) or ``[conv_dim, k]``,
    ``a, b [W, Hv]`` bf16, ``A_log, dt_bias [Hv]``.
    Returns ``(qkv_conv [W, conv_dim] bf16, new_conv_state [W, conv_dim, k] bf16,
    beta [W, Hv] bf16, g [W, Hv] fp32)``; with ``beta_f32`` a fifth tensor, ``beta`` widened to fp32
    (what ``SharedCacheGDN.decode_step`` consumes without a conversion launch).
    """
    _need_cuda(qkv, "decode_conv_gates")
    if qkv.dtype != torch.bfloat16:
        raise NotImplementedError("the GDN layer kernels take bfloat16 activations")
    W, conv_dim = qkv.shape
    if qkv.stride(1) != 1:
        qkv = qkv.contiguous()
    weight = conv_weight.reshape(conv_dim, -1).to(torch.bfloat16).contiguous()
    k = weight.shape[1]
    if prior_conv is not None:
        assert prior_conv.shape == (W, conv_dim, k)
        prior_conv = prior_conv.to(torch.bfloat16).contiguous()
    Hv = a.shape[-1]
    a2 = a.reshape(W, Hv).to(torch.bfloat16).contiguous()
    b2 = b.reshape(W, Hv).to(torch.bfloat16).contiguous()
    a_log = A_log.to(device=qkv.device, dtype=torch.float32).contiguous()
    bias = dt_bias.to(device=qkv.device, dtype=torch.float32).contiguous()
    qkv_out = torch.empty(W, conv_dim, dtype=torch.bfloat16, device=qkv.device)
    conv_out = torch.empty(W, conv_dim, k, dtype=torch.bfloat16, device=qkv.device)
    beta = torch.empty(W, Hv, dtype=torch.bfloat16, device=qkv.device)
    g = torch.empty(W, Hv, dtype=torch.float32, device=qkv.device)
    beta32 = torch.empty(W, Hv, dtype=torch.float32, device=qkv.device) if beta_f32 else None
    args = _lib.VaGdnDecodePre()
    args.qkv, args.qkv_row_stride = qkv.data_ptr(), qkv.stride(0)
    args.prior_conv = prior_conv.data_ptr() if prior_conv is not None else None
    args.conv_weight, args.a, args.b = weight.data_ptr(), a2.data_ptr(), b2.data_ptr()
    args.a_log, args.dt_bias = a_log.data_ptr(), bias.data_ptr()
    args.qkv_out, args.conv_out = qkv_out.data_ptr(), conv_out.data_ptr()
    args.beta_out, args.g_out = beta.data_ptr(), g.data_ptr()
    args.beta_f32_out = beta32.data_ptr() if beta32 is not None else None
    args.num_workers, args.conv_dim, args.conv_kernel, args.num_v_heads = W, conv_dim, k, Hv
    _lib.check(_lib.lib().va_gdn_decode_pre(C.byref(args), _lib.stream_ptr()), "va_gdn_decode_pre")
    return (qkv_out, conv_out, beta, g, beta32) if beta_f32 else (qkv_out, conv_out, beta, g)


def gated_rmsnorm(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``weight * x * rsqrt(mean(x^2) + eps) * silu(gate)`` over the last dim, fp32 inside;
    ``x``, ``gate`` bf16 of one shape, ``weight [dim]``."""
    _need_cuda(x, "gated_rmsnorm")
    if x.dtype != torch.bfloat16:
        raise NotImplementedError("the GDN layer kernels take bfloat16 activations")
    dim = x.shape[-1]
    xc = x.contiguous()
    assert gate.shape == xc.shape
    # the gate may be a slice of a wider projection output ``[tokens, ..., dim]``: its rows are read
    # where they lie when everything but the token dimension is dense
    rows_per_token, token_stride = 0, 0
    gc = gate
    inner = 1
    dense_inner = gate.dtype == torch.bfloat16 and gate.dim() >= 2
    for d in range(gate.dim() - 1, 0, -1):
        dense_inner = dense_inner and gate.stride(d) == inner
        inner *= gate.shape[d]
    if dense_inner and gate.stride(0) >= inner:
        rows_per_token, token_stride = inner // dim, gate.stride(0)
    else:
        gc = gate.to(torch.bfloat16).contiguous()
    w = weight.to(device=x.device, dtype=torch.float32).contiguous()
    out = torch.empty_like(xc)
    rc = _lib.lib().va_gdn_gated_rmsnorm(xc.data_ptr(), gc.data_ptr(), w.data_ptr(), out.data_ptr(),
                                         xc.numel() // dim, dim, float(eps), rows_per_token, token_stride,
                                         _lib.stream_ptr())
    _lib.check(rc, "va_gdn_gated_rmsnorm")
    return out


def prefill_conv(qkv: torch.Tensor, prior_conv: Optional[torch.Tensor], conv_weight: torch.Tensor,
                 segments) -> Tuple[torch.Tensor, torch.Tensor]:
    """Causal depthwise conv + SiLU of a batch of prefills in one launch.

    ``qkv [T, conv_dim]`` bf16 rows of all requests, ``segments`` their token counts (a list, or a
    device int32 tensor of ``R + 1`` offsets), ``prior_conv [R, conv_dim, k]`` or None.  Returns
    ``(qkv_conv [T, conv_dim], new_conv_states [R, conv_dim, k])`` -- what the per-request loop of
    ``_forward_ar_prefill`` (minisgl/models/qwen3_5_delta.py:360-419) computes request by request.
    """
    _need_cuda(qkv, "prefill_conv")
    if qkv.dtype != torch.bfloat16:
        raise NotImplementedError("the GDN layer kernels take bfloat16 activations")
    T, conv_dim = qkv.shape
    if qkv.stride(1) != 1:
        qkv = qkv.contiguous()
    weight = conv_weight.reshape(conv_dim, -1).to(torch.bfloat16).contiguous()
    k = weight.shape[1]
    if isinstance(segments, torch.Tensor):
        seg_off = segments.to(device=qkv.device, dtype=torch.int32).contiguous()
        R = seg_off.numel() - 1
    else:
        offs = [0]
        for n in segments:
            offs.append(offs[-1] + int(n))
        assert offs[-1] == T, "prefill segments do not cover the batch"
        R = len(offs) - 1
        seg_off = torch.tensor(offs, dtype=torch.int32).to(qkv.device)
    if prior_conv is not None:
        assert prior_conv.shape == (R, conv_dim, k)
        prior_conv = prior_conv.to(torch.bfloat16).contiguous()
    qkv_out = torch.empty(T, conv_dim, dtype=torch.bfloat16, device=qkv.device)
    conv_out = torch.empty(R, conv_dim, k, dtype=torch.bfloat16, device=qkv.device)
    args = _lib.VaGdnPrefillConv()
    args.qkv, args.qkv_row_stride = qkv.data_ptr(), qkv.stride(0)
    args.prior_conv = prior_conv.data_ptr() if prior_conv is not None else None
    args.conv_weight, args.seg_off = weight.data_ptr(), seg_off.data_ptr()
    args.qkv_out, args.conv_out = qkv_out.data_ptr(), conv_out.data_ptr()
    args.num_requests, args.num_tokens, args.conv_dim, args.conv_kernel = R, T, conv_dim, k
    _lib.check(_lib.lib().va_gdn_prefill_conv(C.byref(args), _lib.stream_ptr()), "va_gdn_prefill_conv")
    return qkv_out, conv_out


class GatedDeltaNetLayer:
    """One Gated DeltaNet layer over worker chains: the counterpart of the async-reasoning entry
    points of ``Qwen3_5GatedDeltaNet`` (minisgl/models/qwen3_5_delta.py:349-490).

    The projections stay plain GEMMs (``torch.nn.functional.linear`` on the weights given here);
    everything between them runs on this package's kernels through the prepared ``SharedCacheGDN``
    object (``ar``) of the forward:

      decode   ``ar.decode_pre`` (conv window + SiLU + gates + next window, one launch)
               -> ``ar.decode_step`` (chain fold + one recurrent token + summary update, one launch)
               -> ``gated_rmsnorm``
      prefill  ``ar.prefill_pre`` (causal conv of all requests + next windows, one launch), gates
               -> ``ar.prefill_scan`` (chain fold, joint scan: outputs + the write blocks' summaries)
               -> ``gated_rmsnorm``

    The caller brackets a model forward with ``ar.set_context`` / ``ar.prepare_decode`` (or
    ``prepare_prefill``) and ``ar.finish_decode(ok)`` (``finish_prefill``), exactly as the reference
    session does (minisgl/shared_cache/session.py:1195-1227); new summaries and conv windows become
    visible to the blocks only then.

    Weights: ``w_qkv [2*Hk*dk + Hv*dv, hidden]``, ``w_z [Hv*dv, hidden]``, ``w_a``, ``w_b [Hv, hidden]``,
    ``w_out [hidden, Hv*dv]`` bf16; ``conv_weight [conv_dim, 1, k]``; ``A_log``, ``dt_bias [Hv]``;
    ``norm_weight [dv]``.
    """

    def __init__(self, lin_idx: int, num_k_heads: int, num_v_heads: int, head_k_dim: int, head_v_dim: int,
                 w_qkv: torch.Tensor, w_z: torch.Tensor, w_a: torch.Tensor, w_b: torch.Tensor, w_out: torch.Tensor,
                 conv_weight: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor, norm_weight: torch.Tensor,
                 eps: float = 1e-6) -> None:
        self.lin_idx = lin_idx
        self.num_k_heads, self.num_v_heads = num_k_heads, num_v_heads
        self.head_k_dim, self.head_v_dim = head_k_dim, head_v_dim
        self.key_dim, self.value_dim = num_k_heads * head_k_dim, num_v_heads * head_v_dim
        self.conv_dim = 2 * self.key_dim + self.value_dim
        self.w_qkv, self.w_z, self.w_a, self.w_b, self.w_out = w_qkv, w_z, w_a, w_b, w_out
        # one GEMM for the four input projections: rows [qkv | z | a | b]
        self.w_in = torch.cat((w_qkv, w_z, w_a, w_b), dim=0).contiguous()
        self.conv_weight = conv_weight.reshape(self.conv_dim, -1).to(torch.bfloat16).contiguous()
        self.A_log = A_log.to(device=w_qkv.device, dtype=torch.float32).contiguous()
        self.dt_bias = dt_bias.to(device=w_qkv.device, dtype=torch.float32).contiguous()
        self.norm_weight = norm_weight.to(device=w_qkv.device, dtype=torch.float32).contiguous()
        self.eps = float(eps)

    def _project(self, x: torch.Tensor):
        y = torch.nn.functional.linear(x, self.w_in)
        return torch.split(y, [self.conv_dim, self.value_dim, self.num_v_heads, self.num_v_heads], dim=-1)

    def _split_heads(self, qkv: torch.Tensor):
        n = qkv.shape[0]
        q, k, v = torch.split(qkv, [self.key_dim, self.key_dim, self.value_dim], dim=-1)
        return (q.reshape(n, self.num_k_heads, self.head_k_dim), k.reshape(n, self.num_k_heads, self.head_k_dim),
                v.reshape(n, self.num_v_heads, self.head_v_dim))

    def _finish(self, core: torch.Tensor, z: torch.Tensor) -> torch.Tensor:
        n = core.shape[0]
        normed = gated_rmsnorm(core.reshape(n, self.num_v_heads, self.head_v_dim),
                               z.reshape(n, self.num_v_heads, self.head_v_dim), self.norm_weight, self.eps)
        return torch.nn.functional.linear(normed.reshape(n, self.value_dim), self.w_out)

    def forward_ar_decode(self, x: torch.Tensor, ar) -> torch.Tensor:
        """``x [W, hidden]``: one token per worker (``_forward_ar_decode``, qwen3_5_delta.py:443-490)."""
        qkv, z, a, b = self._project(x)
        qkv2, beta, g = ar.decode_pre(self.lin_idx, qkv, self.conv_weight, a, b, self.A_log, self.dt_bias)
        q, k, v = self._split_heads(qkv2)
        core = ar.decode_step(self.lin_idx, q, k, v, g, beta)
        return self._finish(core, z)

    def forward_ar_prefill(self, x: torch.Tensor, ar) -> torch.Tensor:
        """``x [N, hidden]``: the rows of all requests of a batched prefill, request-major
        (``_forward_ar_prefill``, qwen3_5_delta.py:349-441)."""
        qkv, z, a, b = self._project(x)
        qkv2 = ar.prefill_pre(self.lin_idx, qkv, self.conv_weight)
        q, k, v = self._split_heads(qkv2)
        beta = b.sigmoid()                                                     # _gates, :296-299
        g = -self.A_log.exp() * torch.nn.functional.softplus(a.float() + self.dt_bias)
        core = ar.prefill_scan(self.lin_idx, q, k, v, g, beta)
        return self._finish(core, z)


__all__ = ["decode_conv_gates", "gated_rmsnorm", "prefill_conv", "GatedDeltaNetLayer"]
