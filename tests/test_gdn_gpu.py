"""GPU parity of the Gated DeltaNet kernels (fused decode step, compose, prefill scan) against the
CPU oracle, through the SharedCacheGDN seam object."""
import pytest
import torch

from async_llm_b200.blocks import CacheBlock
from async_llm_b200.view_gdn import SharedCacheGDN
from helpers import assert_close_bf16
from oracle import gdn_oracle as go

pytestmark = pytest.mark.gpu

H, HK, DK, DV = 4, 2, 128, 128
AFFINE_ATOL = 5e-6   # the reference's own tolerance for captured summaries (fp32)


def rand_tokens(g, T):
    q = torch.randn(T, HK, DK, generator=g).to(torch.bfloat16)
    k = torch.randn(T, HK, DK, generator=g).to(torch.bfloat16)
    v = torch.randn(T, H, DV, generator=g).to(torch.bfloat16)
    gate = torch.nn.functional.logsigmoid(torch.randn(T, H, generator=g))
    beta = torch.sigmoid(torch.randn(T, H, generator=g))
    return q, k, v, gate, beta


def rep(x):
    """key heads repeated to value heads, as the model layer does before the reference kernels"""
    return x.repeat_interleave(H // HK, dim=1)


def block_with_summary(g, T, device):
    """A block whose layer-0 summary folds T random tokens (built with the oracle)."""
    b = CacheBlock(device, 16)
    if T:
        _, k, v, gate, beta = rand_tokens(g, T)
        A, Bm = go.capture_tokens(None, rep(k), v, gate.exp(), beta)
        b.linear_affine[0] = (A.to(device), Bm.to(device))
    return b


def cpu_pair(block):
    pair = block.linear_affine.get(0)
    return None if pair is None else (pair[0].cpu(), pair[1].cpu())


def make_gdn(device):
    return SharedCacheGDN(num_heads=H, head_k_dim=DK, head_v_dim=DV, conv_dim=2 * HK * DK + H * DV,
                          conv_kernel=4, device=device, num_k_heads=HK)


def test_fused_decode_step(cuda_device):
    g = torch.Generator().manual_seed(41)
    shared = block_with_summary(g, 40, cuda_device)
    mid = block_with_summary(g, 9, cuda_device)
    bare = block_with_summary(g, 0, cuda_device)        # a block without a summary
    priv = [block_with_summary(g, 5 + i, cuda_device) for i in range(3)]
    fresh = block_with_summary(g, 0, cuda_device)       # written for the first time
    outside = block_with_summary(g, 7, cuda_device)     # write block outside its worker's view
    chains = [[shared, priv[0]], [shared, bare, mid, priv[1]], [priv[2]], [shared, fresh], [shared, mid], []]
    targets = [priv[0], priv[1], priv[2], fresh, outside, block_with_summary(g, 0, cuda_device)]
    W = len(chains)
    q, k, v, gate, beta = rand_tokens(g, W)
    want_o, want_new = go.decode_step([[cpu_pair(b) for b in c] for c in chains],
                                      [cpu_pair(t) for t in targets], rep(q), rep(k), v, gate, beta)
    ar = make_gdn(cuda_device)
    ar.set_context(chains, targets)
    ar.prepare_decode(1, torch.bfloat16)
    old = [cpu_pair(t) for t in targets]
    o = ar.decode_step(0, q.to(cuda_device), k.to(cuda_device), v.to(cuda_device),
                       gate.to(cuda_device), beta.to(cuda_device))
    torch.cuda.synchronize()
    # nothing is visible before publish; a failed forward publishes nothing
    for t, before in zip(targets, old):
        now = cpu_pair(t)
        assert (now is None) == (before is None)
        if now is not None:
            assert torch.equal(now[0], before[0]) and torch.equal(now[1], before[1])
    ar.finish_decode(True)
    assert_close_bf16(o.reshape(W, -1), want_o.float().reshape(W, -1), "gdn decode step")
    for w, t in enumerate(targets):
        A, Bm = cpu_pair(t)
        torch.testing.assert_close(A, want_new[w][0], atol=AFFINE_ATOL, rtol=1e-5)
        torch.testing.assert_close(Bm, want_new[w][1], atol=AFFINE_ATOL, rtol=1e-5)


def test_compose_and_capture_reference_sequence(cuda_device):
    g = torch.Generator().manual_seed(43)
    a, b, c = (block_with_summary(g, n, cuda_device) for n in (12, 30, 0))
    w0, w1 = block_with_summary(g, 3, cuda_device), block_with_summary(g, 0, cuda_device)
    chains = [[a, c, b, w0], [b, w1], [c]]
    targets = [w0, w1, block_with_summary(g, 0, cuda_device)]
    ar = make_gdn(cuda_device)
    ar.set_context(chains, targets)
    S0 = ar.compose_initial_recurrent_state(0, torch.float32)
    want = torch.stack([go.chain_initial_state([cpu_pair(x) for x in ch], H, DK, DV) for ch in chains])
    torch.testing.assert_close(S0.cpu(), want, atol=2e-5, rtol=1e-4)
    # per-token capture (the reference's eager call), two tokens per worker
    _, k, v, gate, beta = rand_tokens(g, 6)
    before = [cpu_pair(t) for t in targets]
    ar.capture_token_affines(0, rep(k).view(3, 2, H, DK).to(cuda_device), v.view(3, 2, H, DV).to(cuda_device),
                             gate.exp().view(3, 2, H).to(cuda_device), beta.view(3, 2, H).to(cuda_device))
    torch.cuda.synchronize()
    for w, t in enumerate(targets):
        A, Bm = go.capture_tokens(before[w], rep(k).view(3, 2, H, DK)[w], v.view(3, 2, H, DV)[w],
                                  gate.exp().view(3, 2, H)[w], beta.view(3, 2, H)[w])
        got = cpu_pair(t)
        torch.testing.assert_close(got[0], A, atol=AFFINE_ATOL, rtol=1e-5)
        torch.testing.assert_close(got[1], Bm, atol=AFFINE_ATOL, rtol=1e-5)
    assert ar.compose_initial_recurrent_state(1, torch.float32) is None


@pytest.mark.parametrize("engine", ["scan", "chunk", "chunk_tc"])
def test_prefill_scan_carries_state_across_blocks(cuda_device, engine):
    # three blocks written in order by two requests: block j starts from the fold of blocks < j,
    # so the outputs equal one uninterrupted scan, and every block gets its own summary
    g = torch.Generator().manual_seed(47)
    R, lens = 2, [37, 64, 21]
    data = [[rand_tokens(g, T) for T in lens] for _ in range(R)]
    ar = make_gdn(cuda_device)
    ar.prefill_engine = engine
    # the chunked engine rounds its operands to bf16 (fp32 accumulation and state)
    s_atol, s_rtol = (2e-5, 1e-4) if engine == "scan" else (1.5e-2, 2e-2)
    written = [[] for _ in range(R)]
    outs = [[] for _ in range(R)]
    for j, T in enumerate(lens):
        new = [CacheBlock(cuda_device, 16) for _ in range(R)]
        ar.set_context([written[r] + [new[r]] for r in range(R)], new, prefill_segments=[T] * R)
        ar.prepare_prefill(1, torch.bfloat16, R * T)
        cat = [torch.cat([data[r][j][i] for r in range(R)]).to(cuda_device) for i in range(5)]
        o = ar.prefill_scan(0, *cat)
        ar.finish_prefill(True)
        torch.cuda.synchronize()
        ar.check_status()
        for r in range(R):
            outs[r].append(o[r * T: (r + 1) * T].cpu())
            written[r].append(new[r])
    for r in range(R):
        q, k, v, gate, beta = (torch.cat([data[r][j][i] for j in range(len(lens))]) for i in range(5))
        want, S_end = go.recurrent_delta_rule(rep(q)[None], rep(k)[None], v[None], gate[None], beta[None],
                                              torch.zeros(1, H, DK, DV))
        got = torch.cat(outs[r])
        assert_close_bf16(got.reshape(got.shape[0], -1), want[0].float().reshape(got.shape[0], -1), "gdn prefill")
        off = 0
        for j, T in enumerate(lens):
            A, Bm = go.capture_tokens(None, rep(k[off: off + T]), v[off: off + T], gate[off: off + T].exp(),
                                      beta[off: off + T])
            gotA, gotB = cpu_pair(written[r][j])
            torch.testing.assert_close(gotA, A, atol=s_atol, rtol=s_rtol)
            torch.testing.assert_close(gotB, Bm, atol=s_atol, rtol=s_rtol)
            off += T
        # the fold of all three summaries is the final state of the uninterrupted scan (the
        # recurrence normalises k in bf16, the capture in fp32, hence the looser bound)
        S_fold = go.chain_initial_state([cpu_pair(b) for b in written[r]], H, DK, DV)
        torch.testing.assert_close(S_fold, S_end[0], atol=4e-3 if engine == "scan" else 2e-2, rtol=1e-2 if engine == "scan" else 3e-2)


# ------------------------------------------------------------------ benchmark-size cases
def tokens_for(g, T, hk, h):
    q = torch.randn(T, hk, DK, generator=g).to(torch.bfloat16)
    k = torch.randn(T, hk, DK, generator=g).to(torch.bfloat16)
    v = torch.randn(T, h, DV, generator=g).to(torch.bfloat16)
    gate = torch.nn.functional.logsigmoid(torch.randn(T, h, generator=g))
    beta = torch.sigmoid(torch.randn(T, h, generator=g))
    return q, k, v, gate, beta


MULTI_CHUNK_SHAPES = {
    # name: (value heads, key heads, block lengths, requests)
    "h4_200": (4, 2, [200], 2),                     # 4 chunks, the last one ragged
    "h4_2048_then_130": (4, 2, [2048, 130], 2),     # 32 chunks, then a block that starts from their fold
    "hv32_4x2048": (32, 16, [2048] * 4, 1),         # the benchmark's chunked-prefill shape, one request
}


@pytest.mark.parametrize("engine", ["scan", "chunk", "chunk_tc"])
@pytest.mark.parametrize("shape", list(MULTI_CHUNK_SHAPES))
def test_prefill_blocks_of_many_chunks(cuda_device, engine, shape):
    # Blocks far longer than one 64-token chunk: inside a launch the chunked engine carries the state
    # from chunk to chunk, between launches it is carried by the fold of the blocks' summaries.  The
    # outputs must equal one uninterrupted token-by-token scan, every block's summary the fold of
    # its own tokens; the errors are printed so that the drift over 8192 tokens is on record.
    h, hk, lens, R = MULTI_CHUNK_SHAPES[shape]
    g = torch.Generator().manual_seed(53)
    data = [[tokens_for(g, T, hk, h) for T in lens] for _ in range(R)]
    ar = SharedCacheGDN(num_heads=h, head_k_dim=DK, head_v_dim=DV, conv_dim=2 * hk * DK + h * DV,
                        conv_kernel=4, device=cuda_device, num_k_heads=hk, prefill_engine=engine)
    written = [[] for _ in range(R)]
    outs = [[] for _ in range(R)]
    for j, T in enumerate(lens):
        new = [CacheBlock(cuda_device, 16) for _ in range(R)]
        ar.set_context([written[r] + [new[r]] for r in range(R)], new, prefill_segments=[T] * R)
        ar.prepare_prefill(1, torch.bfloat16, R * T)
        cat = [torch.cat([data[r][j][i] for r in range(R)]).to(cuda_device) for i in range(5)]
        o = ar.prefill_scan(0, *cat)
        ar.finish_prefill(True)
        torch.cuda.synchronize()
        ar.check_status()
        for r in range(R):
            outs[r].append(o[r * T: (r + 1) * T].cpu())
            written[r].append(new[r])
    rep_h = lambda x: x.repeat_interleave(h // hk, dim=1)
    worst_sum, worst_out, mean_out = 0.0, 0.0, 0.0
    for r in range(R):
        q, k, v, gate, beta = (torch.cat([data[r][j][i] for j in range(len(lens))]) for i in range(5))
        want, S_end = go.recurrent_delta_rule(rep_h(q)[None], rep_h(k)[None], v[None], gate[None], beta[None],
                                              torch.zeros(1, h, DK, DV))
        got = torch.cat(outs[r])
        n = got.shape[0]
        assert_close_bf16(got.reshape(n, -1), want[0].float().reshape(n, -1), f"gdn prefill {shape}/{engine}")
        diff = (got.float().reshape(n, -1) - want[0].float().reshape(n, -1)).abs()
        worst_out, mean_out = max(worst_out, float(diff.max())), max(mean_out, float(diff.mean()))
        off = 0
        for j, T in enumerate(lens):
            A, Bm = go.capture_tokens(None, rep_h(k[off: off + T]), v[off: off + T], gate[off: off + T].exp(),
                                      beta[off: off + T])
            gotA, gotB = cpu_pair(written[r][j])
            worst_sum = max(worst_sum, float((gotA - A).abs().max()), float((gotB - Bm).abs().max()))
            off += T
        S_fold = go.chain_initial_state([cpu_pair(b) for b in written[r]], h, DK, DV)
        fold_err = float((S_fold - S_end[0]).abs().max())
        print(f"[gdn prefill {shape}/{engine}] request {r}: out max-abs {float(diff.max()):.3e} mean-abs "
              f"{float(diff.mean()):.3e}; summary max-abs {worst_sum:.3e}; folded final state max-abs {fold_err:.3e} "
              f"(|S| max {float(S_end.abs().max()):.3f})")
        # the scan engine is exact fp32 arithmetic (its k is normalised in fp32, the recurrence's in
        # bf16: hence not 5e-6); the chunked engine rounds operands to bf16 once per chunk
        assert worst_sum <= (AFFINE_ATOL if engine == "scan" else 1e-2)
        assert fold_err <= (8e-3 if engine == "scan" else 1.5e-2)


@pytest.mark.parametrize("depth", [2, 4])
def test_fused_decode_step_at_benchmark_size(cuda_device, depth):
    # the GDN decode configuration of the benchmark: 128 workers, 16 key / 32 value heads, chains of
    # `depth` blocks whose first block is shared by every worker
    import benchcases as wl

    W, h, hk = 128, 32, 16
    g = torch.Generator().manual_seed(59)
    shared = CacheBlock(cuda_device, 16)
    shared.linear_affine[0] = wl.gdn_random_summary(h, DK, DV, 1, cuda_device)
    mids = []
    for j in range(depth - 2):
        b = CacheBlock(cuda_device, 16)
        b.linear_affine[0] = wl.gdn_random_summary(h, DK, DV, 2 + j, cuda_device)
        mids.append(b)
    privs = []
    for w in range(W):
        b = CacheBlock(cuda_device, 16)
        b.linear_affine[0] = wl.gdn_random_summary(h, DK, DV, 100 + w, cuda_device)
        privs.append(b)
    chains = [[shared] + mids + [privs[w]] for w in range(W)]
    q, k, v, gate, beta = tokens_for(g, W, hk, h)
    rep_h = lambda x: x.repeat_interleave(h // hk, dim=1)
    want_o, want_new = go.decode_step([[cpu_pair(b) for b in c] for c in chains], [cpu_pair(t) for t in privs],
                                      rep_h(q), rep_h(k), v, gate, beta)
    ar = SharedCacheGDN(num_heads=h, head_k_dim=DK, head_v_dim=DV, conv_dim=2 * hk * DK + h * DV,
                        conv_kernel=4, device=cuda_device, num_k_heads=hk)
    ar.set_context(chains, privs)
    ar.prepare_decode(1, torch.bfloat16)
    o = ar.decode_step(0, *(t.to(cuda_device) for t in (q, k, v, gate, beta)))
    torch.cuda.synchronize()
    ar.finish_decode(True)
    assert_close_bf16(o.reshape(W, -1), want_o.float().reshape(W, -1), f"gdn decode step W=128 depth {depth}")
    for w in (0, 1, 63, 127):
        A, Bm = cpu_pair(privs[w])
        torch.testing.assert_close(A, want_new[w][0], atol=AFFINE_ATOL, rtol=1e-5)
        torch.testing.assert_close(Bm, want_new[w][1], atol=AFFINE_ATOL, rtol=1e-5)
