"""GPU parity of the view-decode path (store + decode through the C ABI) against the CPU oracle."""
import pytest
import torch

import benchcases as wl
from helpers import assert_close_bf16, oracle_decode

pytestmark = pytest.mark.gpu


ENGINES = ["tcgen05", "mma_sync"]   # the two tensor-core paths behind the shared-block tiles


def run_case(case, device, dense_engine=None):
    dv = wl.DeviceView(case, device, dense_engine=dense_engine)
    out = dv.decode()
    torch.cuda.synchronize()
    dv.attn.check_status()
    want, k_ref, v_ref = oracle_decode(case)
    # the rotated new keys and the values land in the pool bit-exactly
    assert torch.equal(dv.pool.k_cache(0).cpu(), k_ref)
    assert torch.equal(dv.pool.v_cache(0).cpu(), v_ref)
    assert_close_bf16(out, want, "view decode")
    return dv, out


@pytest.mark.parametrize("page_size", [1, 4, 16, 64])
def test_config1_three_block_views(cuda_device, page_size):
    run_case(wl.config1_decode(page_size=page_size), cuda_device)


@pytest.mark.parametrize("engine", ENGINES)
@pytest.mark.parametrize("page_size", [1, 16])
def test_shared_prefix_small(cuda_device, page_size, engine):
    # the shared-prefix topology of the roofline configuration at a size the oracle finishes fast
    case = wl.config2_decode(page_size=page_size, requests=6, shared_len=700, private_len=333)
    dv, _ = run_case(case, cuda_device, engine)
    assert dv.attn.dense_engine == engine


@pytest.mark.parametrize("engine", ENGINES)
def test_config2_full_size(cuda_device, engine):
    # the benchmark configuration itself: 64 requests x [shared 8192 | private 2048], Hq16/Hkv2/D256,
    # streaming lanes for the private blocks, dense tiles for the shared block, one merge
    case = wl.config2_decode(page_size=16)
    dv, out = run_case(case, cuda_device, engine)
    assert out.shape == (64, 16 * 256)


def test_edge_topologies(cuda_device):
    # empty blocks, a block read twice, cross readers of a block written this step, a write block
    # outside the view (implicit self segment), lengths around page and stage edges
    lengths = {"common": 17, "left": 16, "right": 0, "empty": 0, "solo": 1, "tail": 33, "out": 5}
    views = [["common", "empty", "right", "left"], ["common", "left", "common"], ["solo"],
             ["tail", "common"], ["common"]]
    writes = ["left", "right", "solo", "tail", "out"]
    for D, hq, hkv in ((128, 8, 2), (256, 8, 1), (128, 4, 4)):
        case = wl.make_view_case(lengths=lengths, views=views, writes=writes, num_q_heads=hq,
                                 num_kv_heads=hkv, head_dim=D, page_size=16, rope_base=1e6, seed=7)
        run_case(case, cuda_device)


def test_repeated_forward_is_deterministic(cuda_device):
    case = wl.config1_decode(page_size=16)
    dv = wl.DeviceView(case, cuda_device)
    batch = dv.plan()
    a = dv.decode(batch).clone()
    b = dv.decode(batch).clone()
    torch.cuda.synchronize()
    assert torch.equal(a, b)


@pytest.mark.parametrize("engine", ENGINES)
def test_scratch_left_poisoned_does_not_reach_the_output(cuda_device, engine):
    # the split-K scratch keeps whatever an earlier step left in it: every slot the merge pass reads
    # must have been written by this step's items / tiles.  Poison it with NaN and decode a step that
    # uses both the streaming lanes and the dense tiles of a shared block.
    case = wl.config2_decode(page_size=16, requests=12, shared_len=700, private_len=90,
                             num_q_heads=8, num_kv_heads=2, head_dim=128)
    dv = wl.DeviceView(case, cuda_device, dense_engine=engine)
    batch = dv.plan()
    assert batch.attn_metadata.plan.groups is not None
    clean = dv.decode(batch).clone()
    dv.attn._partial_o.fill_(float("nan"))
    dv.attn._partial_ml.fill_(float("nan"))
    poisoned = dv.decode(batch)
    torch.cuda.synchronize()
    dv.attn.check_status()
    assert torch.isfinite(poisoned.float()).all()
    assert torch.equal(poisoned, clean)


@pytest.mark.parametrize("dense_fraction", [0.0, 0.25])
def test_graph_replay_after_replanning_into_fixed_buffers(cuda_device, dense_fraction):
    # a CUDA graph captured on one topology keeps producing the oracle's result after another
    # topology is planned into the same fixed-capacity buffers (the reference's graph variant,
    # minisgl/shared_cache/attention_graph.py): addresses and grid sizes never change
    import dataclasses
    from types import SimpleNamespace
    from async_llm_b200.view_attention import SharedDecodeAttentionBuffers

    lengths = {"sys": 600, "a": 40, "b": 77, "c": 130, "d": 9, "e": 300, "f": 0}
    writes = ["a", "b", "c", "d", "e", "f"]
    views_a = [["sys", "a"], ["sys", "b"], ["sys", "c"], ["sys", "d"], ["sys", "e"], ["f"]]
    views_b = [["sys", "e", "a"], ["b"], ["c", "sys"], ["sys", "d", "c"], ["e"], ["sys", "f"]]
    case_a = wl.make_view_case(lengths=lengths, views=views_a, writes=writes, num_q_heads=8,
                               num_kv_heads=2, head_dim=128, page_size=16, rope_base=1e6, seed=11)
    case_b = dataclasses.replace(case_a, views=views_b)
    dv = wl.DeviceView(case_a, cuda_device)
    bufs = SharedDecodeAttentionBuffers(dv.attn, workers=6, depth=3, max_pages=case_a.num_pages,
                                        dense_fraction=dense_fraction)
    pending, slots, positions = case_a.plan_writes()
    pos_dev, loc_dev = positions.to(cuda_device), slots.to(cuda_device)
    meta = dv.attn.prepare(case_a.group, pending, slots, graph_buffers=bufs)
    batch = SimpleNamespace(attn_metadata=meta, positions=pos_dev, out_loc=loc_dev, mrope_positions=None)
    dv.attn.forward(dv.q, dv.k_new, dv.v_new, 0, batch)      # warm-up outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = dv.attn.forward(dv.q, dv.k_new, dv.v_new, 0, batch)
    for case in (case_a, case_b, case_a):
        pending, slots, positions = case.plan_writes()
        dv.attn.prepare(case.group, pending, slots, graph_buffers=bufs)
        pos_dev.copy_(positions)
        loc_dev.copy_(slots)
        graph.replay()
        torch.cuda.synchronize()
        dv.attn.check_status()
        want, _, _ = oracle_decode(case)
        assert_close_bf16(out, want, "graph replay")


def test_dense_tiles_launch_order_follows_what_the_step_writes(cuda_device):
    # The tiles of a widely read block start before the step's keys are stored unless that block
    # is itself written in the step: then its new key is one of the keys the tiles must see, and
    # they stay behind the store.  Both orders give the oracle's rows.
    lengths = {"shared": 700}
    views, writes = [], []
    for r in range(6):
        lengths[f"p{r}"] = 40 + r
        views.append(["shared", f"p{r}"])
        writes.append(f"p{r}")
    early = wl.make_view_case(lengths=lengths, views=views, writes=writes, num_q_heads=16, num_kv_heads=2,
                              head_dim=256, page_size=16, rope_base=1e7, seed=21)
    dv = wl.DeviceView(early, cuda_device)
    batch = dv.plan()
    assert batch.attn_metadata.plan.groups is not None and batch.attn_metadata.fork_dense_early
    run_case(early, cuda_device)
    # worker 0 appends to the block everybody reads
    late = wl.make_view_case(lengths=lengths, views=views, writes=["shared"] + writes[1:], num_q_heads=16,
                             num_kv_heads=2, head_dim=256, page_size=16, rope_base=1e7, seed=22)
    dv = wl.DeviceView(late, cuda_device)
    batch = dv.plan()
    assert batch.attn_metadata.plan.groups is not None and not batch.attn_metadata.fork_dense_early
    run_case(late, cuda_device)
