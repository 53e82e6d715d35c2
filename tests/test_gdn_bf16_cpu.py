"""bf16 storage of GDN block summaries: the CPU oracle's rounding points against the fixture generated
from the reference's ``SharedCacheGDN(state_dtype=torch.bfloat16)`` eager path
(minisgl/shared_cache/gdn.py:127-269, gdn_affine.py:113-122)."""
import os
import sys

import numpy as np
import torch

from oracle import gdn_oracle as go

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden  # noqa: E402  (seeded input builder only)

GOLDEN = np.load(os.path.join(HERE, "golden", "gdn_bf16_golden.npz"))
BF16 = torch.bfloat16


def from_bits(a):
    return torch.from_numpy(a.copy()).view(BF16)


def assert_same_rounding(got, want, what):
    """Same values rounded at the same points: fp32 sums that associate differently may flip the last
    bit of a few bf16 results, nothing more."""
    assert got.dtype == BF16 and want.dtype == BF16
    flipped = (got.view(torch.int16) != want.view(torch.int16)).float().mean().item()
    assert flipped < 2e-3, f"{what}: {flipped:.2%} of the stored values differ"
    torch.testing.assert_close(got.float(), want.float(), atol=1e-3, rtol=1.6e-2)


def build_blocks():
    """Block summaries by the oracle, block by block, stored as bf16."""
    c = make_golden.BF16_CASE
    data = make_golden.gdn_bf16_inputs()
    pairs = {}
    for name, T in c["block_tokens"].items():
        pairs[name] = None
        if T:
            k, v, alpha, beta = data[name]
            pairs[name] = go.capture_tokens(None, k, v, alpha, beta, state_dtype=BF16)
    return c, data, pairs


def test_captured_summaries_round_once_per_call():
    c, data, pairs = build_blocks()
    for name, pair in pairs.items():
        if pair is None:
            assert f"{name}_A" not in GOLDEN.files
            continue
        assert_same_rounding(pair[0], from_bits(GOLDEN[f"{name}_A"]), name)
        assert_same_rounding(pair[1], from_bits(GOLDEN[f"{name}_B"]), name)


def test_chain_fold_rounds_every_link():
    c, data, pairs = build_blocks()
    H, dk, dv = c["H"], c["dk"], c["dv"]
    want = torch.from_numpy(GOLDEN["S0"])
    for w, chain in enumerate(c["chains"]):
        got = go.chain_initial_state([pairs[n] for n in chain], H, dk, dv, BF16)
        # same operands and rounding points; the fp32 matmuls may associate differently
        torch.testing.assert_close(got, want[w], atol=2e-2, rtol=2e-2)
        assert (got - want[w]).abs().mean().item() < 1e-3
    # the fold in fp32 differs from the rounded one by more than that somewhere: the rounding is real
    full = go.chain_initial_state([pairs[n] for n in c["chains"][0]], H, dk, dv, torch.float32)
    assert not torch.equal(full, want[0])


def test_new_tokens_fold_into_rounded_summaries():
    c, data, pairs = build_blocks()
    H, dk, dv = c["H"], c["dk"], c["dv"]
    k, v, alpha, beta = data["new"]
    W, n = len(c["targets"]), c["new_tokens"]
    for w, name in enumerate(c["targets"]):
        A, Bm = go.capture_tokens(pairs[name], k.view(W, n, H, dk)[w], v.view(W, n, H, dv)[w],
                                  alpha.view(W, n, H)[w], beta.view(W, n, H)[w], state_dtype=BF16)
        assert_same_rounding(A, from_bits(GOLDEN[f"new{w}_A"]), name)
        assert_same_rounding(Bm, from_bits(GOLDEN[f"new{w}_B"]), name)
