"""The decode entry point that brings its own scratch (va_view_decode_static).

It exists for callers that cannot allocate device memory once they are running -- for example a
serving process that handed all free HBM to its KV pool at start-up, or a host binding the C ABI
without a device allocator.  The split-K scratch then comes from a fixed array inside the library
instead of from the caller.  The test drives the entry point through the C ABI, twice in a row on
one stream (the array is shared by all calls and keeps the previous call's contents), and checks
the rows against the regular entry point, which is itself checked against the CPU oracle.
"""
import ctypes as C

import pytest
import torch

from async_llm_b200 import _lib
import benchcases as wl
from async_llm_b200.kvpool import pool_struct
from helpers import assert_close_bf16

pytestmark = pytest.mark.gpu


def call_static(dv, plan_struct, out):
    pool = pool_struct(dv.pool, 0, dv.case.num_q_heads, dv.attn._cos_sin, dv.attn.rotary_dim)
    return _lib.lib().va_view_decode_static(
        C.byref(pool), C.byref(plan_struct), dv.q.data_ptr(), dv.q.stride(0), out.data_ptr(),
        out.stride(0), dv.attn.status().data_ptr(), _lib.stream_ptr())


@pytest.mark.parametrize("shape", ["three_block_views", "shared_prefix_tiles"])
def test_static_scratch_decode_matches_regular_entry_point(cuda_device, shape):
    if shape == "three_block_views":
        case = wl.config1_decode(page_size=16)
    else:  # a block read by many requests: dense tiles + streaming lanes + merge
        case = wl.config2_decode(page_size=16, requests=12, shared_len=600, private_len=150)
    dv = wl.DeviceView(case, cuda_device)
    batch = dv.plan()
    want = dv.decode(batch).clone()          # regular entry point (caller-supplied scratch)
    torch.cuda.synchronize()
    plan = batch.attn_metadata.plan
    assert (shape == "shared_prefix_tiles") == (plan.groups is not None)
    outs = [torch.full_like(want, float("nan")) for _ in range(2)]
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for attempt in range(2):                 # second call starts from the first call's leftovers
        rc = call_static(dv, plan.struct, outs[attempt])
        assert rc == 0, f"va_view_decode_static returned {rc} on call {attempt}"
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    # the reason the entry point exists: the driver handed out no device memory for these calls
    assert free_after == free_before, f"device memory changed by {free_before - free_after} bytes"
    dv.attn.check_status()
    for attempt, out in enumerate(outs):
        assert_close_bf16(out, want.float(), f"static-scratch decode, call {attempt}")
        assert torch.equal(out, want)        # same kernels, same order of operations


def test_static_scratch_refuses_plans_beyond_its_capacity(cuda_device):
    case = wl.config1_decode(page_size=16)
    dv = wl.DeviceView(case, cuda_device)
    batch = dv.plan()
    want = dv.decode(batch).clone()
    big = _lib.VaDecodePlan()
    C.memmove(C.byref(big), C.byref(batch.attn_metadata.plan.struct), C.sizeof(big))
    limit = 2048 * 8 // (case.num_q_heads // case.num_kv_heads)
    out = torch.zeros(len(case.views), case.num_q_heads * case.head_dim, dtype=torch.bfloat16,
                      device=cuda_device)
    big.num_partials = limit + 1
    assert call_static(dv, big, out) == -3   # VA_ERR_CAPACITY, nothing launched
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0
    big.num_partials = limit                 # a plan that claims exactly the whole array is served
    assert call_static(dv, big, out) == 0
    torch.cuda.synchronize()
    dv.attn.check_status()
    assert torch.equal(out, want)


def test_static_scratch_refuses_shared_block_tiles_beyond_its_capacity(cuda_device):
    # the dense tiles of a shared block bound their writes by their own partial count: one that
    # exceeds the static array (or the step's own count) must be refused before anything runs
    case = wl.config2_decode(page_size=16, requests=12, shared_len=600, private_len=150)
    dv = wl.DeviceView(case, cuda_device)
    batch = dv.plan()
    plan = batch.attn_metadata.plan
    assert plan.groups is not None
    dv.decode(batch)                                   # sizes the caller-side scratch used further down
    gqa = case.num_q_heads // case.num_kv_heads
    tiles = _lib.VaDensePlan()
    C.memmove(C.byref(tiles), C.byref(plan.groups.struct), C.sizeof(tiles))
    step = _lib.VaDecodePlan()
    C.memmove(C.byref(step), C.byref(plan.struct), C.sizeof(step))
    step.groups = C.addressof(tiles)
    out = torch.zeros(len(case.views), case.num_q_heads * case.head_dim, dtype=torch.bfloat16,
                      device=cuda_device)
    tiles.num_partials = 2048 * 8 // gqa + 1           # beyond the static array
    assert call_static(dv, step, out) == -3
    tiles.num_partials = step.num_partials + 1         # within the array, beyond the step's own count
    assert call_static(dv, step, out) == -3
    pool = pool_struct(dv.pool, 0, case.num_q_heads, dv.attn._cos_sin, dv.attn.rotary_dim)
    rc = _lib.lib().va_view_decode(C.byref(pool), C.byref(step), dv.q.data_ptr(), dv.q.stride(0), out.data_ptr(),
                                   out.stride(0), dv.attn._partial_o.data_ptr(), dv.attn._partial_ml.data_ptr(),
                                   dv.attn.status().data_ptr(), _lib.stream_ptr())
    assert rc == -3                                    # the regular entry point refuses it too
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0
