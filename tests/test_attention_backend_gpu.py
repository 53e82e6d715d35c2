"""GPU parity of the attention-backend plugin (ordinary prefill / extend / decode batches, and decode
replayed from a CUDA graph after re-planning) against the CPU oracle's causal paged attention."""
import pytest
import torch

from async_llm_b200 import B200AttnBackend, MHAKVCache
from attention_backend_cases import make_batch, make_plain_case, oracle_rows
from helpers import assert_close_bf16

pytestmark = pytest.mark.gpu


def gpu_backend(case, device, dense_engine=None):
    pool = MHAKVCache(case.hkv, 1, case.d, case.k_pool.shape[0], case.page_size, torch.bfloat16, device)
    pool.k_cache(0).copy_(case.k_pool)
    pool.v_cache(0).copy_(case.v_pool)
    return B200AttnBackend(case.config, pool, case.table.to(device), dense_engine=dense_engine), pool


def run(case, phase, device, dense_engine=None):
    be, pool = gpu_backend(case, device, dense_engine)
    batch = make_batch(case, phase, device)
    be.prepare_metadata(batch)
    out = be.forward(case.q.to(device).view(-1, case.hq, case.d), case.k.to(device), case.v.to(device), 0, batch)
    torch.cuda.synchronize()
    be.op.check_status()
    want, k_ref, v_ref = oracle_rows(case)
    assert torch.equal(pool.k_cache(0).cpu(), k_ref) and torch.equal(pool.v_cache(0).cpu(), v_ref)
    assert_close_bf16(out, want, f"plain {phase}")


@pytest.mark.parametrize("engine", ["tcgen05", "mma_sync"])
@pytest.mark.parametrize("d,hq,hkv", [(128, 8, 2), (256, 8, 1)])
def test_plain_prefill_and_extend(cuda_device, d, hq, hkv, engine):
    # a fresh prompt, a request extending a cached prefix, a long fresh prompt: one causal batch
    run(make_plain_case([(0, 45), (37, 33), (0, 200)], hq=hq, hkv=hkv, d=d), "prefill", cuda_device, engine)


@pytest.mark.parametrize("d,hq,hkv", [(128, 16, 4), (256, 16, 2)])
def test_plain_decode(cuda_device, d, hq, hkv):
    run(make_plain_case([(300, 1), (37, 1), (1, 1), (129, 1), (64, 1)], hq=hq, hkv=hkv, d=d), "decode", cuda_device)


def test_decode_graph_replay_after_replanning(cuda_device):
    # the graph hooks of the plugin interface: fixed-capacity tables per batch size, a graph captured
    # on one batch keeps answering correctly after another batch is planned into the same tables
    first = make_plain_case([(300, 1), (37, 1), (1, 1), (129, 1)], seed=5, min_slots=1024)
    second = make_plain_case([(12, 1), (400, 1), (77, 1), (250, 1)], seed=5, min_slots=1024)
    be, pool = gpu_backend(first, cuda_device)
    be.init_capture_graph(512, [4])
    q = first.q.to(cuda_device).clone()
    k, v = first.k.to(cuda_device).clone(), first.v.to(cuda_device).clone()
    batch = make_batch(first, "decode", cuda_device)
    be.prepare_for_capture(batch)
    be.forward(q, k, v, 0, batch)          # warm-up outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = be.forward(q, k, v, 0, batch)
    for case in (first, second, first):
        pool.k_cache(0).copy_(case.k_pool)
        pool.v_cache(0).copy_(case.v_pool)
        be._page_table = case.table.to(cuda_device)
        nxt = make_batch(case, "decode", cuda_device)
        be.prepare_for_replay(nxt)
        q.copy_(case.q); k.copy_(case.k); v.copy_(case.v)
        batch.out_loc.copy_(nxt.out_loc)
        graph.replay()
        torch.cuda.synchronize()
        be.op.check_status()
        want, _, _ = oracle_rows(case)
        assert_close_bf16(out, want, "plain decode graph replay")
