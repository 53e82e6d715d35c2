"""GPU parity of view-conditioned prefill (store + dense tiles through the C ABI) vs the oracle."""
import pytest
import torch

import benchcases as wl
from helpers import assert_close_bf16, oracle_prefill

pytestmark = pytest.mark.gpu


ENGINES = ["tcgen05", "mma_sync"]   # the two tensor-core paths of the dense tiles


def run_case(case, device, dense_engine=None):
    dp = wl.DevicePrefill(case, device, dense_engine=dense_engine)
    assert dense_engine is None or dp.attn.dense_engine == dense_engine
    out = dp.forward()
    torch.cuda.synchronize()
    dp.attn.check_status()
    want, k_ref, v_ref = oracle_prefill(case)
    assert torch.equal(dp.pool.k_cache(0).cpu(), k_ref)
    assert torch.equal(dp.pool.v_cache(0).cpu(), v_ref)
    assert_close_bf16(out, want, "view prefill")


@pytest.mark.parametrize("engine", ENGINES)
@pytest.mark.parametrize("page_size", [1, 16, 64])
def test_small_view_prefill(cuda_device, page_size, engine):
    # ragged chunk sizes, a request without context, a write block that already holds a prefix
    lengths = {"a": 70, "b": 129, "c": 5, "w0": 0, "w1": 37, "w2": 0}
    reqs = [{"context": ["a", "b"], "write": "w0", "num_new": 45},
            {"context": ["b", "c", "a"], "write": "w1", "num_new": 33},
            {"context": [], "write": "w2", "num_new": 70}]
    for D, hq, hkv in ((128, 8, 2), (256, 8, 1)):
        case = wl.make_prefill_case(lengths=lengths, requests=reqs, num_q_heads=hq, num_kv_heads=hkv,
                                    head_dim=D, page_size=page_size, rope_base=1e6, seed=5)
        run_case(case, cuda_device, engine)


@pytest.mark.parametrize("engine", ENGINES)
def test_config3_reduced(cuda_device, engine):
    # the benchmark topology (shared pool of context blocks, 2-6 blocks per request) at a size the
    # CPU oracle finishes in seconds
    case = wl.config3_prefill(requests=4, chunk=96, pool_blocks=6, min_len=100, max_len=400,
                              max_context=1400)
    run_case(case, cuda_device, engine)


def test_config3_four_requests_at_full_chunk_size(cuda_device):
    # the benchmark's own request shape -- 512 new tokens against 2-6 context blocks of 1K-8K tokens,
    # Hq32/Hkv8/D128 -- for the first 4 of its 16 requests (the CPU oracle needs seconds per request)
    case = wl.config3_prefill(requests=4)
    assert all(r["num_new"] == 512 for r in case.requests)
    run_case(case, cuda_device)


def test_graph_replay_after_replanning_prefill_buffers(cuda_device):
    # a CUDA graph captured around forward() on one batch keeps producing the oracle's rows after a
    # different batch (other requests, other lengths) is planned into the same fixed-capacity
    # buffers (the reference's SharedPrefillAttentionBuffers, attention_graph.py:124-167)
    import dataclasses
    from types import SimpleNamespace
    from async_llm_b200 import SharedPrefillAttentionBuffers

    lengths = {"a": 70, "b": 129, "c": 5, "w0": 0, "w1": 37, "w2": 0}
    reqs = [{"context": ["a", "b"], "write": "w0", "num_new": 45},
            {"context": ["b", "c", "a"], "write": "w1", "num_new": 33},
            {"context": [], "write": "w2", "num_new": 70}]
    full = wl.make_prefill_case(lengths=lengths, requests=reqs, num_q_heads=8, num_kv_heads=2, head_dim=128,
                                page_size=16, rope_base=1e6, seed=5)
    offs = [0, 45, 78, 148]

    def sub_case(idx):   # the batch made of requests idx (rows stay request-major)
        rows = torch.cat([torch.arange(offs[i], offs[i + 1]) for i in idx])
        return dataclasses.replace(full, requests=[full.requests[i] for i in idx],
                                   self_pages=[full.self_pages[i] for i in idx], q=full.q[rows],
                                   k_new=full.k_new[rows], v_new=full.v_new[rows],
                                   positions=full.positions[rows], out_loc=full.out_loc[rows])

    dp = wl.DevicePrefill(full, cuda_device)
    cap = 160
    bufs = SharedPrefillAttentionBuffers(dp.attn, workers=3, depth=3, rows=cap, max_pages=full.num_pages)
    q = torch.zeros(cap, full.q.shape[1], dtype=torch.bfloat16, device=cuda_device)
    k = torch.zeros(cap, full.k_new.shape[1], dtype=torch.bfloat16, device=cuda_device)
    v = torch.zeros_like(k)
    pos = torch.zeros(cap, dtype=torch.int32, device=cuda_device)
    loc = torch.full((cap,), -1, dtype=torch.int32, device=cuda_device)   # negative slot: row is not stored

    def stage(case):
        n = case.q.shape[0]
        q[:n], k[:n], v[:n] = case.q.to(cuda_device), case.k_new.to(cuda_device), case.v_new.to(cuda_device)
        pos.zero_(); loc.fill_(-1)
        pos[:n], loc[:n] = case.positions.to(cuda_device), case.out_loc.to(cuda_device)
        return dp.attn.prepare_prefill_batch(case.specs(), graph_buffers=bufs), n

    first = sub_case([0, 2])
    meta, _ = stage(first)
    batch = SimpleNamespace(attn_metadata=meta, positions=pos, out_loc=loc, mrope_positions=None)
    dp.attn.forward(q, k, v, 0, batch)        # warm-up outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = dp.attn.forward(q, k, v, 0, batch)
    for case in (first, sub_case([1]), full):
        _, n = stage(case)
        graph.replay()
        torch.cuda.synchronize()
        dp.attn.check_status()
        want, _, _ = oracle_prefill(case)
        assert_close_bf16(out[:n], want, "prefill graph replay")
