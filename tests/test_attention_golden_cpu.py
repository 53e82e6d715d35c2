"""The CPU oracle of the attention core against output rows of the REFERENCE implementation.

tests/golden/attention_golden.npz holds what the unmodified reference ``SharedCacheAttention``
(FlashInfer paged decode / prefill kernels + ``merge_states``, minisgl/shared_cache/attention.py:
282-752) produced on a GPU for the seeded cases of tests/attention_cases.py
(tests/golden/make_attention_golden.py generated it).  This pins ``oracle/view_oracle.view_decode``
/ ``view_prefill``: the oracle accumulates in fp32, the reference kernels round their output to
bf16, so the two agree to bf16 resolution.
"""
import json
import os

import numpy as np
import pytest
import torch

from attention_cases import DECODE_CASES, PREFILL_CASES
from helpers import assert_close_bf16, oracle_decode, oracle_prefill

GOLD = os.path.join(os.path.dirname(__file__), "golden", "attention_golden.npz")
pytestmark = pytest.mark.skipif(not os.path.exists(GOLD), reason="tests/golden/attention_golden.npz not generated")


def golden():
    return np.load(GOLD)


def bits_to_bf16(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


def test_fixture_says_where_it_came_from():
    info = json.loads(bytes(golden()["info"]).decode())
    assert info["flashinfer"] and info["gpu"]
    assert set(info["cases"]) >= {f"decode/{n}" for n in DECODE_CASES} | {f"prefill/{n}" for n in PREFILL_CASES}


# the full-size cases cost the oracle seconds; the rest are small
@pytest.mark.parametrize("name", list(DECODE_CASES))
def test_oracle_decode_matches_reference_rows(name):
    z = golden()
    case = DECODE_CASES[name]()
    want, k_ref, _ = oracle_decode(case)
    rows = torch.from_numpy(z[f"decode/{name}/rows"])
    ref = bits_to_bf16(z[f"decode/{name}/out"])
    assert_close_bf16(ref, want[rows], f"reference vs oracle, decode/{name}")
    # one bf16 step at these magnitudes: the reference's own graph-vs-eager gate (atol 2e-3,
    # tests/core/test_shared_decode_attention_graph.py:104) is reported, not asserted
    diff = (ref.float() - want[rows]).abs()
    print(f"[decode/{name}] reference vs fp32 oracle: max-abs {float(diff.max()):.3e} mean-abs {float(diff.mean()):.3e} "
          f"within 2e-3: {bool(diff.max() <= 2e-3)}")
    # the rotated keys the reference stored are the oracle's, bit for bit
    _, slots, _ = case.plan_writes()
    mine = k_ref.view(-1, case.num_kv_heads * case.head_dim)[slots.long()]
    assert torch.equal(mine.view(torch.int16), torch.from_numpy(z[f"decode/{name}/new_keys"]))


@pytest.mark.parametrize("name", list(PREFILL_CASES))
def test_oracle_prefill_matches_reference_rows(name):
    z = golden()
    case = PREFILL_CASES[name]()
    want, _, _ = oracle_prefill(case)
    rows = torch.from_numpy(z[f"prefill/{name}/rows"])
    ref = bits_to_bf16(z[f"prefill/{name}/out"])
    assert_close_bf16(ref, want[rows], f"reference vs oracle, prefill/{name}")
    diff = (ref.float() - want[rows]).abs()
    print(f"[prefill/{name}] reference vs fp32 oracle: max-abs {float(diff.max()):.3e} mean-abs {float(diff.mean()):.3e} "
          f"within 2e-3: {bool(diff.max() <= 2e-3)}")
