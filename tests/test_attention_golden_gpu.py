"""The CUDA attention kernels against output rows of the REFERENCE implementation on the same seeded
inputs (tests/golden/attention_golden.npz: the unmodified reference ``SharedCacheAttention`` with its
FlashInfer kernels, run on a GPU by tests/golden/make_attention_golden.py).  Tolerance: the stated
2e-2 max-abs / 1e-3 mean-abs; whether the reference's own one-bf16-step gate (atol 2e-3,
tests/core/test_shared_decode_attention_graph.py:104) also holds is printed."""
import os

import numpy as np
import pytest
import torch

import benchcases as wl
from attention_cases import DECODE_CASES, PREFILL_CASES
from helpers import assert_close_bf16

GOLD = os.path.join(os.path.dirname(__file__), "golden", "attention_golden.npz")
pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not os.path.exists(GOLD), reason="tests/golden/attention_golden.npz not generated")]

ENGINES = ["tcgen05", "mma_sync"]


def bits_to_bf16(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


def report(kind, name, engine, got, ref):
    diff = (got.float().cpu() - ref.float()).abs()
    print(f"[{kind}/{name}/{engine}] kernels vs reference rows: max-abs {float(diff.max()):.3e} mean-abs "
          f"{float(diff.mean()):.3e} within 2e-3: {bool(diff.max() <= 2e-3)}")


@pytest.mark.parametrize("engine", ENGINES)
@pytest.mark.parametrize("name", list(DECODE_CASES))
def test_decode_kernels_match_reference_rows(cuda_device, name, engine):
    z = np.load(GOLD)
    case = DECODE_CASES[name]()
    dv = wl.DeviceView(case, cuda_device, dense_engine=engine)
    out = dv.decode()
    torch.cuda.synchronize()
    dv.attn.check_status()
    rows = torch.from_numpy(z[f"decode/{name}/rows"])
    ref = bits_to_bf16(z[f"decode/{name}/out"])
    got = out.cpu()[rows]
    assert_close_bf16(got, ref.float(), f"kernels vs reference, decode/{name}")
    report("decode", name, engine, got, ref)
    _, slots, _ = case.plan_writes()
    stored = dv.pool.k_cache(0).view(-1, case.num_kv_heads * case.head_dim)[slots.to(cuda_device).long()].cpu()
    assert torch.equal(stored.view(torch.int16), torch.from_numpy(z[f"decode/{name}/new_keys"]))


@pytest.mark.parametrize("engine", ENGINES)
@pytest.mark.parametrize("name", list(PREFILL_CASES))
def test_prefill_kernels_match_reference_rows(cuda_device, name, engine):
    z = np.load(GOLD)
    case = PREFILL_CASES[name]()
    dp = wl.DevicePrefill(case, cuda_device, dense_engine=engine)
    out = dp.forward()
    torch.cuda.synchronize()
    dp.attn.check_status()
    rows = torch.from_numpy(z[f"prefill/{name}/rows"])
    ref = bits_to_bf16(z[f"prefill/{name}/out"])
    got = out.cpu()[rows]
    assert_close_bf16(got, ref.float(), f"kernels vs reference, prefill/{name}")
    report("prefill", name, engine, got, ref)
