"""GPU parity of the GDN kernels with bf16 summary storage (``SharedCacheGDN(state_dtype=bfloat16)``):
against the fixture generated from the reference's bf16 eager path and against the CPU oracle, through
the seam object.  The kernels widen stored summaries, work in fp32 and round once per stored summary;
the chain fold keeps its intermediate in fp32 where the reference rounds every link, so the composed
state is compared with the reference's within bf16 resolution."""
import os
import sys

import numpy as np
import pytest
import torch

from async_llm_b200.blocks import CacheBlock
from async_llm_b200.view_gdn import SharedCacheGDN
from helpers import assert_close_bf16
from oracle import gdn_oracle as go

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden  # noqa: E402  (seeded input builder only)

pytestmark = pytest.mark.gpu

GOLDEN = np.load(os.path.join(HERE, "golden", "gdn_bf16_golden.npz"))
BF16 = torch.bfloat16


def from_bits(a):
    return torch.from_numpy(a.copy()).view(BF16)


def assert_same_rounding(got, want, what, flips=5e-3):
    got, want = got.cpu(), want.cpu()
    assert got.dtype == BF16 and want.dtype == BF16, what
    flipped = (got.view(torch.int16) != want.view(torch.int16)).float().mean().item()
    assert flipped < flips, f"{what}: {flipped:.2%} of the stored values differ"
    torch.testing.assert_close(got.float(), want.float(), atol=2e-3, rtol=1.6e-2)


def make_ar(device, H, hk=None, engine=None):
    return SharedCacheGDN(num_heads=H, head_k_dim=128, head_v_dim=128, conv_dim=2 * (hk or H) * 128 + H * 128,
                          conv_kernel=4, device=device, num_k_heads=hk or H, state_dtype=BF16, prefill_engine=engine)


def golden_blocks(device):
    c = make_golden.BF16_CASE
    blocks = {}
    for name in c["block_tokens"]:
        b = CacheBlock(device, 16)
        if f"{name}_A" in GOLDEN.files:
            b.linear_affine[0] = (from_bits(GOLDEN[f"{name}_A"]).to(device), from_bits(GOLDEN[f"{name}_B"]).to(device))
        blocks[name] = b
    return c, blocks


def test_capture_and_compose_match_the_reference_rows(cuda_device):
    c, blocks = golden_blocks(cuda_device)
    data = make_golden.gdn_bf16_inputs()
    H, dk, dv = c["H"], c["dk"], c["dv"]
    ar = make_ar(cuda_device, H)
    # block summaries from their tokens (the reference's eager capture call)
    for name, T in c["block_tokens"].items():
        if T == 0:
            continue
        fresh = CacheBlock(cuda_device, 16)
        k, v, alpha, beta = (t.to(cuda_device) for t in data[name])
        ar.set_context([[fresh]], [fresh])
        ar.capture_token_affines(0, k[None], v[None], alpha[None], beta[None])
        A, Bm = fresh.linear_affine[0]
        assert_same_rounding(A, from_bits(GOLDEN[f"{name}_A"]), f"{name} A_hat")
        assert_same_rounding(Bm, from_bits(GOLDEN[f"{name}_B"]), f"{name} B_hat")
    # chain fold over the reference's stored summaries
    chains = [[blocks[n] for n in ch] for ch in c["chains"]]
    targets = [blocks[n] for n in c["targets"]]
    ar.set_context(chains, targets)
    S0 = ar.compose_initial_recurrent_state(0, torch.float32).cpu()
    want = torch.from_numpy(GOLDEN["S0"])
    scale = float(want.abs().max())
    assert float((S0 - want).abs().max()) <= 2e-2 * max(scale, 1.0)
    assert float((S0 - want).abs().mean()) <= 1e-3 * max(scale, 1.0)
    # and against the fp32 fold of the same stored summaries (what the kernel computes)
    for w, ch in enumerate(c["chains"]):
        exact = go.chain_initial_state([None if 0 not in blocks[n].linear_affine else
                                        tuple(t.cpu().float() for t in blocks[n].linear_affine[0]) for n in ch], H, dk, dv)
        torch.testing.assert_close(S0[w], exact, atol=2e-5, rtol=1e-4)
    # two more tokens per worker into the write blocks
    k, v, alpha, beta = (t.to(cuda_device) for t in data["new"])
    W, n = len(targets), c["new_tokens"]
    ar.capture_token_affines(0, k.view(W, n, H, dk), v.view(W, n, H, dv), alpha.view(W, n, H), beta.view(W, n, H))
    torch.cuda.synchronize()
    for w, t in enumerate(targets):
        A, Bm = t.linear_affine[0]
        assert_same_rounding(A, from_bits(GOLDEN[f"new{w}_A"]), f"worker {w} A_hat")
        assert_same_rounding(Bm, from_bits(GOLDEN[f"new{w}_B"]), f"worker {w} B_hat")


def cpu_pair(block):
    pair = block.linear_affine.get(0)
    return None if pair is None else (pair[0].cpu(), pair[1].cpu())


def test_fused_decode_step_bf16_summaries(cuda_device):
    # the fused step over bf16 summaries: output against the oracle run on the same stored values, new
    # summaries rounded once; q / k / v handed over as slices of one wider row (read in place)
    c, blocks = golden_blocks(cuda_device)
    H, dk, dv = c["H"], c["dk"], c["dv"]
    chains = [[blocks[n] for n in ch] for ch in c["chains"]]
    targets = [blocks[n] for n in c["targets"]]
    W = len(chains)
    g = torch.Generator().manual_seed(91)
    row = torch.randn(W, 3 * H * dk + 40, generator=g).to(BF16)
    gate = torch.nn.functional.logsigmoid(torch.randn(W, H, generator=g))
    beta = torch.sigmoid(torch.randn(W, H, generator=g))
    q, k, v = (row[:, i * H * dk: (i + 1) * H * dk].view(W, H, dk) for i in range(3))
    # fp32 fold of the stored values, fp32 update, one rounding: what the kernel does
    want_o, _ = go.decode_step([[None if p is None else (p[0].float(), p[1].float()) for p in map(cpu_pair, ch)]
                                for ch in chains], [None] * W, q, k, v, gate, beta)
    want_new = [go.capture_tokens(cpu_pair(t), k[w][None], v[w][None], gate[w].exp()[None], beta[w][None],
                                  state_dtype=BF16) for w, t in enumerate(targets)]
    ar = make_ar(cuda_device, H)
    ar.set_context(chains, targets)
    ar.prepare_decode(1, BF16)
    row_d = row.to(cuda_device)
    qd, kd, vd = (row_d[:, i * H * dk: (i + 1) * H * dk].view(W, H, dk) for i in range(3))
    assert not qd.is_contiguous()
    o = ar.decode_step(0, qd, kd, vd, gate.to(cuda_device), beta.to(cuda_device))
    ar.finish_decode(True)
    torch.cuda.synchronize()
    assert_close_bf16(o.reshape(W, -1), want_o.float().reshape(W, -1), "gdn decode step, bf16 summaries")
    for w, t in enumerate(targets):
        A, Bm = t.linear_affine[0]
        assert A.dtype == BF16 and Bm.dtype == BF16
        assert_same_rounding(A, want_new[w][0], f"worker {w} A_hat")
        assert_same_rounding(Bm, want_new[w][1], f"worker {w} B_hat")


@pytest.mark.parametrize("engine", ["scan", "chunk", "chunk_tc"])
def test_prefill_bf16_summaries(cuda_device, engine):
    # two blocks written in order: the second starts from the (bf16) summary of the first; outputs
    # against one uninterrupted scan, summaries against the oracle's rounded capture
    H, hk = 4, 2
    g = torch.Generator().manual_seed(97)
    lens = [70, 45]

    def tokens(T):
        q = torch.randn(T, hk, 128, generator=g).to(BF16)
        k = torch.randn(T, hk, 128, generator=g).to(BF16)
        v = torch.randn(T, H, 128, generator=g).to(BF16)
        return q, k, v, torch.nn.functional.logsigmoid(torch.randn(T, H, generator=g)), torch.sigmoid(torch.randn(T, H, generator=g))

    data = [tokens(T) for T in lens]
    rep = lambda x: x.repeat_interleave(H // hk, dim=1)
    ar = make_ar(cuda_device, H, hk, engine)
    written, outs = [], []
    for j, T in enumerate(lens):
        new = CacheBlock(cuda_device, 16)
        ar.set_context([written + [new]], [new], prefill_segments=[T])
        ar.prepare_prefill(1, BF16, T)
        o = ar.prefill_scan(0, *(t.to(cuda_device) for t in data[j]))
        ar.finish_prefill(True)
        torch.cuda.synchronize()
        ar.check_status()
        outs.append(o.cpu())
        written.append(new)
    q, k, v, gate, beta = (torch.cat([d[i] for d in data]) for i in range(5))
    want, _ = go.recurrent_delta_rule(rep(q)[None], rep(k)[None], v[None], gate[None], beta[None],
                                      torch.zeros(1, H, 128, 128))
    got = torch.cat(outs)
    assert_close_bf16(got.reshape(got.shape[0], -1), want[0].float().reshape(got.shape[0], -1), f"bf16 summaries / {engine}")
    off = 0
    for j, T in enumerate(lens):
        A, Bm = go.capture_tokens(None, rep(k[off: off + T]), v[off: off + T], gate[off: off + T].exp(),
                                  beta[off: off + T], state_dtype=BF16)
        gotA, gotB = cpu_pair(written[j])
        assert gotA.dtype == BF16
        if engine == "scan":
            assert_same_rounding(gotA, A, f"block {j} A_hat")
            assert_same_rounding(gotB, Bm, f"block {j} B_hat")
        else:   # bf16 operands inside the chunks
            torch.testing.assert_close(gotA.float(), A.float(), atol=1.5e-2, rtol=2e-2)
            torch.testing.assert_close(gotB.float(), Bm.float(), atol=1.5e-2, rtol=2e-2)
        off += T


def test_block_merge_composes_bf16_pairs(cuda_device):
    from async_llm_b200.block_ops import BlockOps

    c, blocks = golden_blocks(cuda_device)
    ops = BlockOps.__new__(BlockOps)
    ops.device, ops.state_dtype = cuda_device, BF16
    from async_llm_b200 import _lib
    ops._summary_code = _lib.summary_code(BF16)
    a, b = blocks["a"].linear_affine[0], blocks["b"].linear_affine[0]
    (A, Bm), = ops._compose_pairs([(a[0], a[1], b[0], b[1])])
    torch.cuda.synchronize()
    wantA, wantB = go.affine_compose(a[0].cpu(), a[1].cpu(), b[0].cpu(), b[1].cpu(), BF16)
    assert_same_rounding(A, wantA, "merged A_hat")
    assert_same_rounding(Bm, wantB, "merged B_hat")
