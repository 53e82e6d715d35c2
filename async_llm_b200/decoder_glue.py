"""Elementwise glue between the sub-layers of a decoder layer: the fused residual add + RMSNorm and
the SwiGLU gate, one launch each (the reference's ``RMSNormFused`` / ``silu_and_mul`` calls,
minisgl/layers/norm.py:25-43, minisgl/layers/activation.py:9-12)."""

from __future__ import annotations

from typing import Optional

import torch

from . import _lib


def _check(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} runs a CUDA kernel: there is no CPU fallback")
    if t.dtype != torch.bfloat16:
        raise NotImplementedError(f"{what} takes bfloat16 tensors")


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                weight_plus_one: bool = False) -> torch.Tensor:
    """``residual += delta`` in place (fp32 sum, stored as bf16), returns the RMS-normalised fp32 sum
    times ``weight`` (``1 + weight`` when ``weight_plus_one``), rounded once.  ``delta=None``: plain norm
    of ``residual``.  ``residual``/``delta [n, dim]`` contiguous bf16, ``weight [dim]`` bf16."""
    _check(residual, "add_rmsnorm")
    n, dim = residual.shape
    assert residual.is_contiguous() and weight.shape == (dim,) and weight.dtype == torch.bfloat16
    if delta is not None:
        assert delta.shape == residual.shape and delta.dtype == torch.bfloat16
        delta = delta.contiguous()
    out = torch.empty_like(residual)
    rc = _lib.lib().va_add_rmsnorm(residual.data_ptr(), delta.data_ptr() if delta is not None else None,
                                   weight.contiguous().data_ptr(), out.data_ptr(), n, dim, float(eps),
                                   int(bool(weight_plus_one)), _lib.stream_ptr())
    _lib.check(rc, "va_add_rmsnorm")
    return out


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` of rows ``[gate | up]`` (``[n, 2 * inter]`` bf16, the fused gate/up projection);
    fp32 inside, one rounding.  Returns ``[n, inter]``."""
    _check(gate_up, "silu_mul")
    n, two = gate_up.shape
    assert two % 2 == 0
    if gate_up.stride(1) != 1:
        gate_up = gate_up.contiguous()
    inter = two // 2
    out = torch.empty(n, inter, dtype=torch.bfloat16, device=gate_up.device)
    rc = _lib.lib().va_silu_mul(gate_up.data_ptr(), gate_up.stride(0), out.data_ptr(), n, inter, _lib.stream_ptr())
    _lib.check(rc, "va_silu_mul")
    return out


__all__ = ["add_rmsnorm", "silu_mul"]
