"""ctypes binding of the C ABI declared in ``include/view_attn_b200.h``.

There is no CPU fallback: if the shared library is missing, ``lib()`` raises.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Optional

import os

_PKG = Path(__file__).resolve().parent
# VIEWATTN_B200_LIB points at another build of the same C ABI (e.g. an instrumented one)
LIB_PATH = Path(os.environ.get("VIEWATTN_B200_LIB", _PKG / "libviewattn_b200.so"))

VA_OK = 0
VA_ERR_CAPACITY = -3
VA_ITEM_WORDS = 8
ERRORS = {
    -1: "VA_ERR_BAD_ARG",
    -2: "VA_ERR_UNSUPPORTED",
    -3: "VA_ERR_CAPACITY",
    -4: "VA_ERR_LAUNCH",
}
DEVICE_CODES = {1: "VA_DEV_BAD_PAGE", 2: "VA_DEV_BAD_ROW", 3: "VA_DEV_WAIT_EXPIRED"}


class VaPool(C.Structure):
    _fields_ = [
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("num_slots", C.c_int64),
        ("page_size", C.c_int32),
        ("num_q_heads", C.c_int32),
        ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("rotary_dim", C.c_int32),
        ("max_pos", C.c_int32),
        ("cos_sin", C.c_void_p),
        ("sm_scale", C.c_float),
    ]


class VaDecodePlan(C.Structure):
    _fields_ = [
        ("page_indices", C.c_void_p),
        ("items", C.c_void_p),
        ("lane_off", C.c_void_p),
        ("row_part_off", C.c_void_p),
        ("num_items", C.c_int32),
        ("num_lanes", C.c_int32),
        ("num_rows", C.c_int32),
        ("num_partials", C.c_int32),
        ("num_page_indices", C.c_int32),
        ("phase_mask", C.c_int32),
        ("groups", C.c_void_p),
    ]


class VaDensePlan(C.Structure):
    _fields_ = [
        ("page_indices", C.c_void_p),
        ("tiles", C.c_void_p),
        ("entries", C.c_void_p),
        ("segments", C.c_void_p),
        ("num_page_indices", C.c_int32),
        ("num_tiles", C.c_int32),
        ("num_entries", C.c_int32),
        ("num_segments", C.c_int32),
        ("num_partials", C.c_int32),
        ("num_rows", C.c_int32),
        ("num_ctas", C.c_int32),
        ("engine", C.c_int32),
        ("q_pos3", C.c_void_p),
        ("mrope_lim_h", C.c_int32),
        ("mrope_lim_w", C.c_int32),
    ]


class VaGdnStep(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("g", C.c_void_p),
        ("beta", C.c_void_p), ("out", C.c_void_p), ("chain_a", C.c_void_p), ("chain_b", C.c_void_p),
        ("read_a", C.c_void_p), ("read_b", C.c_void_p), ("write_a", C.c_void_p), ("write_b", C.c_void_p),
        ("num_workers", C.c_int32), ("depth", C.c_int32), ("num_k_heads", C.c_int32),
        ("num_v_heads", C.c_int32), ("head_k_dim", C.c_int32), ("head_v_dim", C.c_int32),
        ("l2_eps", C.c_float), ("q_scale", C.c_float), ("status", C.c_void_p),
        ("q_row_stride", C.c_int64), ("k_row_stride", C.c_int64), ("v_row_stride", C.c_int64),
        ("summary_dtype", C.c_int32),
    ]


class VaGdnPrefill(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("g", C.c_void_p),
        ("beta", C.c_void_p), ("out", C.c_void_p), ("seg_off", C.c_void_p), ("state0", C.c_void_p),
        ("init_a", C.c_void_p), ("init_b", C.c_void_p), ("write_a", C.c_void_p), ("write_b", C.c_void_p),
        ("final_state", C.c_void_p),
        ("num_requests", C.c_int32), ("num_k_heads", C.c_int32), ("num_v_heads", C.c_int32),
        ("head_k_dim", C.c_int32), ("head_v_dim", C.c_int32), ("l2_eps", C.c_float), ("q_scale", C.c_float),
        ("engine", C.c_int32), ("max_segment_tokens", C.c_int32), ("scratch", C.c_void_p),
        ("scratch_bytes", C.c_int64), ("num_tokens", C.c_int64), ("summary_dtype", C.c_int32),
        ("status", C.c_void_p),
    ]


class VaPlanParams(C.Structure):
    _fields_ = [
        ("num_workers", C.c_int32), ("num_kv_heads", C.c_int32), ("readers_per_tile", C.c_int32),
        ("num_sms", C.c_int32), ("lane_width", C.c_int32), ("group_min_readers", C.c_int32),
        ("group_min_keys", C.c_int32), ("dense_tiles_per_cta", C.c_int32), ("min_item_keys", C.c_int32),
        ("cut_slack_keys", C.c_int32), ("fixed_stream_lanes", C.c_int32), ("fixed_dense_sms", C.c_int32),
        ("stream_rate", C.c_double), ("dense_rate", C.c_double),
    ]


class VaPlanLayout(C.Structure):
    _fields_ = [
        ("total_words", C.c_int64), ("quota", C.c_int64), ("total_keys", C.c_int64),
        ("off_pages", C.c_int32), ("num_pages", C.c_int32),
        ("off_items", C.c_int32), ("num_items", C.c_int32),
        ("off_lane_off", C.c_int32), ("num_lanes", C.c_int32),
        ("off_row_part_off", C.c_int32), ("num_groups", C.c_int32),
        ("off_tiles", C.c_int32), ("num_tiles", C.c_int32),
        ("off_entries", C.c_int32), ("num_entries", C.c_int32),
        ("off_segments", C.c_int32), ("num_segments", C.c_int32),
        ("num_partials", C.c_int32), ("dense_sms", C.c_int32),
    ]


class VaViewStep(C.Structure):
    _fields_ = [
        ("num_workers", C.c_int32), ("num_blocks", C.c_int32), ("num_aux", C.c_int32), ("page_size", C.c_int32),
        ("view_start", C.c_void_p), ("view_block", C.c_void_p), ("block_len", C.c_void_p),
        ("block_span", C.c_void_p), ("block_pages", C.c_void_p), ("block_pending_page", C.c_void_p),
        ("pages", C.c_void_p),
        ("aux_worker", C.c_void_p), ("aux_loc", C.c_void_p), ("aux_slot", C.c_void_p),
    ]


class VaViewSubs(C.Structure):
    _fields_ = [("num_main", C.c_int32), ("num_aux", C.c_int32), ("max_segments", C.c_int32)]


class VaGdnDecodePre(C.Structure):
    _fields_ = [
        ("qkv", C.c_void_p), ("qkv_row_stride", C.c_int64), ("prior_conv", C.c_void_p),
        ("conv_weight", C.c_void_p), ("a", C.c_void_p), ("b", C.c_void_p), ("a_log", C.c_void_p),
        ("dt_bias", C.c_void_p), ("qkv_out", C.c_void_p), ("conv_out", C.c_void_p), ("beta_out", C.c_void_p),
        ("g_out", C.c_void_p), ("beta_f32_out", C.c_void_p), ("prior_conv_ptrs", C.c_void_p),
        ("conv_out_ptrs", C.c_void_p), ("num_workers", C.c_int32), ("conv_dim", C.c_int32),
        ("conv_kernel", C.c_int32),
        ("num_v_heads", C.c_int32), ("a_row_stride", C.c_int64), ("b_row_stride", C.c_int64),
    ]


class VaGdnPrefillConv(C.Structure):
    _fields_ = [
        ("qkv", C.c_void_p), ("qkv_row_stride", C.c_int64), ("prior_conv", C.c_void_p),
        ("conv_weight", C.c_void_p), ("seg_off", C.c_void_p), ("qkv_out", C.c_void_p), ("conv_out", C.c_void_p),
        ("prior_conv_ptrs", C.c_void_p), ("conv_out_ptrs", C.c_void_p),
        ("num_requests", C.c_int32), ("num_tokens", C.c_int32), ("conv_dim", C.c_int32), ("conv_kernel", C.c_int32),
    ]


class VaAttnQkNorm(C.Structure):
    _fields_ = [
        ("qkv", C.c_void_p), ("qkv_row_stride", C.c_int64), ("q_weight", C.c_void_p), ("k_weight", C.c_void_p),
        ("q_out", C.c_void_p), ("k_out", C.c_void_p), ("n", C.c_int32), ("num_q_heads", C.c_int32),
        ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("eps", C.c_float), ("weight_plus_one", C.c_int32),
    ]


SUMMARY_F32, SUMMARY_BF16 = 0, 1   # VA_SUMMARY_*
VA_PHASE_GROUPS_FORKED = 8


def summary_code(dtype) -> int:
    """VA_SUMMARY_* of a torch dtype of block summaries."""
    import torch
    if dtype == torch.float32:
        return SUMMARY_F32
    if dtype == torch.bfloat16:
        return SUMMARY_BF16
    raise ValueError("Shared GDN state dtype must be float32 or bfloat16")


# name -> (restype, argtypes); every symbol the header declares is listed here
SIGNATURES = {
    "va_abi_version": (C.c_int, []),
    "va_last_cuda_error": (C.c_char_p, []),
    "va_sm_count": (C.c_int, []),
    "va_store_kv": (C.c_int, [C.POINTER(VaPool), C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                              C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "va_rope_rotate": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                 C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]),
    "va_decode_lanes": (C.c_int, [C.c_int32]),
    "va_decode_lane_width": (C.c_int, [C.c_int32]),
    "va_view_decode": (C.c_int, [C.POINTER(VaPool), C.POINTER(VaDecodePlan), C.c_void_p, C.c_int64,
                                 C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_void_p]),
    "va_view_decode_fork_groups": (C.c_int, [C.POINTER(VaPool), C.POINTER(VaDecodePlan), C.c_void_p, C.c_int64,
                                             C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "va_view_dense": (C.c_int, [C.POINTER(VaPool), C.POINTER(VaDensePlan), C.c_void_p, C.c_int64,
                                C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p,
                                C.c_void_p]),
    "va_view_decode_static": (C.c_int, [C.POINTER(VaPool), C.POINTER(VaDecodePlan), C.c_void_p, C.c_int64,
                                        C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "va_gdn_step": (C.c_int, [C.POINTER(VaGdnStep), C.c_void_p]),
    "va_gdn_compose": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                 C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "va_gdn_prefill_scratch_bytes": (C.c_int64, [C.c_int64, C.c_int32]),
    "va_gdn_prefill": (C.c_int, [C.POINTER(VaGdnPrefill), C.c_void_p]),
    "va_plan_decode": (C.c_int, [C.POINTER(VaPlanParams), C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
                                 C.c_int64, C.POINTER(VaPlanLayout)]),
    "va_gdn_plan_tables": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                     C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int32, C.c_int32,
                                     C.c_int32, C.c_int32, C.c_void_p]),
    "va_plan_prefill_tiles": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                        C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.POINTER(C.c_int32)]),
    "va_block_copy": (C.c_int, [C.POINTER(VaPool), C.c_int32, C.c_int64, C.c_void_p, C.c_void_p, C.c_int32,
                                C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "va_gdn_compose_pairs": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "va_mrope_rotate": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                  C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "va_store_kv_mrope": (C.c_int, [C.POINTER(VaPool), C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p,
                                    C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                    C.c_void_p]),
    "va_gdn_decode_pre": (C.c_int, [C.POINTER(VaGdnDecodePre), C.c_void_p]),
    "va_gdn_gated_rmsnorm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32,
                                       C.c_float, C.c_int32, C.c_int64, C.c_void_p]),
    "va_gdn_prefill_conv": (C.c_int, [C.POINTER(VaGdnPrefillConv), C.c_void_p]),
    "va_add_rmsnorm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_float,
                                 C.c_int32, C.c_void_p]),
    "va_silu_mul": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "va_attn_qk_norm": (C.c_int, [C.POINTER(VaAttnQkNorm), C.c_void_p]),
    "va_attn_output_gate": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                      C.c_void_p]),
    "va_plan_views": (C.c_int, [C.POINTER(VaPlanParams), C.POINTER(VaViewStep), C.c_void_p, C.c_int64,
                                C.POINTER(VaPlanLayout), C.c_void_p, C.c_int64, C.POINTER(VaViewSubs)]),
}

_LIB: Optional[C.CDLL] = None


def lib() -> C.CDLL:
    """Load the extension once; raise if it has not been built."""
    global _LIB
    if _LIB is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m async_llm_b200.build` "
                "(there is no CPU fallback for the cache-view kernels)"
            )
        handle = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = handle
    return _LIB


def check(rc: int, what: str) -> None:
    """Turn a negative return code into the reference's exception types."""
    if rc == VA_OK:
        return
    name = ERRORS.get(rc, str(rc))
    detail = ""
    if rc == -4:
        detail = ": " + lib().va_last_cuda_error().decode()
    if rc in (-1, -2, -3):
        raise ValueError(f"{what} failed with {name}{detail}")
    raise RuntimeError(f"{what} failed with {name}{detail}")


def stream_ptr(stream=None, device_index: Optional[int] = None) -> int:
    """Raw handle of ``stream`` (default: the current stream of ``device_index`` / the current device)."""
    import torch

    if stream is not None:
        return stream.cuda_stream
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is not None:
        # the raw query skips building a torch.cuda.Stream object on every kernel launch
        return raw(torch.cuda.current_device() if device_index is None else device_index)
    return torch.cuda.current_stream().cuda_stream
