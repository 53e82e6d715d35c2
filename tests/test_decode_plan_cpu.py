"""The decode work list, replayed on the CPU: executing the items exactly as the kernel does
(item -> partial, partials of (row, kv head) -> merged output) must reproduce the oracle."""
import numpy as np
import pytest
import torch

import benchcases as wl
from async_llm_b200.view_attention import SharedCacheAttention
from helpers import oracle_decode
from oracle import view_oracle as vo


def replay(case, plan, k_pool, v_pool):
    P, Hkv, D, Hq = case.page_size, case.num_kv_heads, case.head_dim, case.num_q_heads
    g = Hq // Hkv
    h = plan.host
    items, pages = h["items"], h["page_indices"]
    kf, vf = k_pool.view(-1, Hkv, D).float(), v_pool.view(-1, Hkv, D).float()
    W = len(case.views)
    n_part = plan.num_partials
    part_o = torch.zeros(n_part, g, D)
    part_m = torch.full((n_part, g), float("-inf"))
    part_l = torch.zeros(n_part, g)
    written = np.zeros(n_part, int)
    q = case.q.view(W, Hq, D)
    covered = np.zeros(len(items), bool)
    for lane in range(len(h["lane_off"]) - 1):
        for it in range(h["lane_off"][lane], h["lane_off"][lane + 1]):
            poff, tok0, n, row, loc, part, kvh, _ = items[it]
            covered[it] = True
            toks = tok0 + np.arange(n)
            slots = torch.from_numpy(pages[poff + toks // P].astype(np.int64) * P + toks % P)
            qr = vo.rope_delta(q[row: row + 1], torch.tensor([int(loc)]), case.cos_sin)[0]
            qg = qr[kvh * g: (kvh + 1) * g].float()
            s = qg @ kf[slots, kvh].T * D ** -0.5
            m = s.max(dim=-1).values
            p = torch.exp(s - m[:, None])
            part_o[part] = p @ vf[slots, kvh]
            part_m[part], part_l[part] = m, p.sum(-1)
            written[part] += 1
    assert covered.all(), "every item must belong to exactly one lane"
    if plan.groups is not None:
        gh = plan.groups.host
        for e0, ecnt, seg0, nseg, kvh, mode, _, _ in gh["tiles"]:
            assert mode == 1 and nseg == 1
            poff, tok0, n, loc_base, causal, _, _, _ = gh["segments"][seg0]
            toks = tok0 + np.arange(n)
            slots = torch.from_numpy(gh["page_indices"][poff + toks // P].astype(np.int64) * P + toks % P)
            for row, rel, part, _ in gh["entries"][e0: e0 + ecnt]:
                qr = vo.rope_delta(q[row: row + 1], torch.tensor([int(rel + loc_base)]), case.cos_sin)[0]
                qg = qr[kvh * g: (kvh + 1) * g].float()
                s = qg @ kf[slots, kvh].T * D ** -0.5
                m = s.max(dim=-1).values
                p = torch.exp(s - m[:, None])
                part_o[part] = p @ vf[slots, kvh]
                part_m[part], part_l[part] = m, p.sum(-1)
                written[part] += 1
    assert (written == 1).all(), "every partial slot is written exactly once"
    out = torch.zeros(W, Hq, D)
    rpo = h["row_part_off"]
    for row in range(W):
        for kvh in range(Hkv):
            sl = slice(rpo[row * Hkv + kvh], rpo[row * Hkv + kvh + 1])
            m = part_m[sl].max(dim=0).values
            wgt = torch.exp(part_m[sl] - m)
            num = (part_o[sl] * wgt[..., None]).sum(0)
            den = (part_l[sl] * wgt).sum(0)
            out[row, kvh * g: (kvh + 1) * g] = num / den[:, None]
    return out.view(W, -1)


def cpu_plan(case, lanes, width=1):
    a = SharedCacheAttention(None, case.cos_sin, case.num_q_heads, case.num_kv_heads, case.head_dim,
                             case.page_size, torch.bfloat16, torch.device("cpu"))
    a._lanes = lanes
    a._lane_width = width
    pending, slots, _ = case.plan_writes()
    return a.prepare(case.group, pending, slots)


@pytest.mark.parametrize("page_size,lanes", [(1, 592), (16, 888), (4, 7), (64, 1)])
def test_config1_plan_replay(page_size, lanes):
    case = wl.config1_decode(page_size=page_size)
    want, k_pool, v_pool = oracle_decode(case)
    meta = cpu_plan(case, lanes)
    got = replay(case, meta.plan, k_pool, v_pool)
    torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-4)
    h = meta.plan.host
    per_lane = np.add.reduceat(h["items"][:, 2], h["lane_off"][:-1].clip(max=len(h["items"]) - 1))
    assert h["items"][:, 2].sum() == h["total_keys"][0]
    assert (h["items"][:, 2] > 0).all()


def test_edge_topology_plan_replay():
    lengths = {"common": 17, "left": 16, "right": 0, "empty": 0, "solo": 1, "tail": 33, "out": 5}
    views = [["common", "empty", "right", "left"], ["common", "left", "common"], ["solo"],
             ["tail", "common"], ["common"]]
    writes = ["left", "right", "solo", "tail", "out"]
    case = wl.make_view_case(lengths=lengths, views=views, writes=writes, num_q_heads=8,
                             num_kv_heads=2, head_dim=128, page_size=16, rope_base=1e6, seed=7)
    want, k_pool, v_pool = oracle_decode(case)
    meta = cpu_plan(case, 64)
    assert meta.n_aux == 2 and meta.max_segments == 4
    got = replay(case, meta.plan, k_pool, v_pool)
    torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("readers,page_size", [(6, 16), (37, 4)])
def test_shared_prefix_goes_to_dense_tiles(readers, page_size):
    # a block read by many workers is planned as dense tiles (one pass over its keys for all
    # readers); the private blocks stay on the streaming lanes; both feed one merge
    case = wl.config2_decode(page_size=page_size, requests=readers, shared_len=300, private_len=70,
                             num_q_heads=8, num_kv_heads=2, head_dim=128)
    want, k_pool, v_pool = oracle_decode(case)
    meta = cpu_plan(case, 64, 4)
    assert meta.plan.groups is not None
    assert meta.plan.struct.num_lanes % 4 == 0 and meta.plan.struct.num_lanes < 64
    got = replay(case, meta.plan, k_pool, v_pool)
    torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-4)


def _two_topologies():
    import dataclasses
    lengths = {"sys": 600, "a": 40, "b": 77, "c": 130, "d": 9, "e": 300, "f": 0}
    writes = ["a", "b", "c", "d", "e", "f"]
    views_a = [["sys", "a"], ["sys", "b"], ["sys", "c"], ["sys", "d"], ["sys", "e"], ["f"]]
    views_b = [["sys", "e", "a"], ["b"], ["c", "sys"], ["sys", "d", "c"], ["e"], ["sys", "f"]]
    case_a = wl.make_view_case(lengths=lengths, views=views_a, writes=writes, num_q_heads=8,
                               num_kv_heads=2, head_dim=128, page_size=16, rope_base=1e6, seed=11)
    return case_a, dataclasses.replace(case_a, views=views_b)


@pytest.mark.parametrize("dense_fraction", [0.0, 0.25])
def test_fixed_capacity_buffers_replan(dense_fraction):
    # two topologies planned one after the other into the same fixed-capacity tables: the
    # addresses and extents in the C structs stay put, the loaded work replays to the oracle
    from async_llm_b200.view_attention import SharedDecodeAttentionBuffers
    case_a, case_b = _two_topologies()
    a = SharedCacheAttention(None, case_a.cos_sin, 8, 2, 128, 16, torch.bfloat16, torch.device("cpu"))
    a._lanes, a._lane_width = 64, 4
    bufs = SharedDecodeAttentionBuffers(a, workers=6, depth=3, max_pages=case_a.num_pages,
                                        dense_fraction=dense_fraction)
    frozen = None
    for case in (case_a, case_b, case_a):
        pending, slots, _ = case.plan_writes()
        meta = a.prepare(case.group, pending, slots, graph_buffers=bufs)
        st = meta.plan.struct
        snap = (st.page_indices, st.items, st.lane_off, st.row_part_off, st.num_items, st.num_lanes,
                st.num_rows, st.num_partials, st.num_page_indices)
        frozen = frozen or snap
        assert snap == frozen
        assert (meta.plan.groups is not None) == (dense_fraction > 0)
        want, k_pool, v_pool = oracle_decode(case)
        got = replay(case, meta.plan, k_pool, v_pool)
        torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-4)


def test_fixed_capacity_buffers_reject_overflow():
    from async_llm_b200.view_attention import SharedDecodeAttentionBuffers
    case_a, _ = _two_topologies()
    a = SharedCacheAttention(None, case_a.cos_sin, 8, 2, 128, 16, torch.bfloat16, torch.device("cpu"))
    a._lanes, a._lane_width = 64, 4
    pending, slots, _ = case_a.plan_writes()
    with pytest.raises(ValueError, match="workers"):
        a.prepare(case_a.group, pending, slots, graph_buffers=SharedDecodeAttentionBuffers(a, 4, 3, 1000))
    with pytest.raises(ValueError, match="page indices"):
        a.prepare(case_a.group, pending, slots, graph_buffers=SharedDecodeAttentionBuffers(a, 6, 3, 8))


def test_replanning_consecutive_steps_reuses_the_view_structure():
    # consecutive decode steps of one worker group: the same views, blocks that grow by a token and
    # now and then by a page.  The planner keeps the flattened view structure between steps; the
    # lengths, spans and page runs it plans with must be those of the current step.
    case = wl.make_view_case(
        lengths={"sys": 300, "a": 15, "b": 31, "c": 0, "out": 16}, num_q_heads=8, num_kv_heads=2, head_dim=128,
        views=[["sys", "a"], ["sys", "b"], ["c", "sys"], ["sys"]], writes=["a", "b", "c", "out"],
        page_size=16, rope_base=1e6, seed=23, spare_pages=8)
    a = SharedCacheAttention(None, case.cos_sin, 8, 2, 128, 16, torch.bfloat16, torch.device("cpu"))
    a._lanes, a._lane_width = 16, 1
    group = case.group
    structures = set()
    for step in range(4):
        pending, slots, positions = case.plan_writes()
        want, k_pool, v_pool = oracle_decode(case)
        meta = a.prepare(group, pending, slots)
        structures.add(id(a._topology))
        got = replay(case, meta.plan, k_pool, v_pool)
        torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-4)
        # commit the step: the pool keeps the stored token, the write blocks grow
        case.k_pool, case.v_pool = k_pool, v_pool
        for name in case.writes:
            b = case.blocks[name]
            page = pending[id(b)]
            if page is not None:
                b.page_starts.append(page)
                case.free_pages.remove(page)
            b.num_tokens += 1
    assert len(structures) == 1, "the same views are flattened once"
    # a changed view is noticed
    group.workers[3].cache_view.append(case.blocks["a"])
    case.views[3].append("a")
    pending, slots, _ = case.plan_writes()
    want, k_pool, v_pool = oracle_decode(case)
    got = replay(case, a.prepare(group, pending, slots).plan, k_pool, v_pool)
    torch.testing.assert_close(got, want, atol=2e-5, rtol=1e-4)
    assert len(a._topology.view_blk) == 8


def test_planners_refuse_views_longer_than_the_rope_table():
    # a rotation distance beyond the cos/sin table would be clamped silently by the kernels (and by
    # the reference's apply_rope_correction): both planners raise instead
    case = wl.config2_decode(page_size=16, requests=3, shared_len=300, private_len=70,
                             num_q_heads=8, num_kv_heads=2, head_dim=128)
    short = case.cos_sin[:200]
    a = SharedCacheAttention(None, short, 8, 2, 128, 16, torch.bfloat16, torch.device("cpu"))
    a._lanes, a._lane_width = 64, 4
    pending, slots, _ = case.plan_writes()
    with pytest.raises(ValueError, match="RoPE table"):
        a.prepare(case.group, pending, slots)
    from async_llm_b200 import PrefillSpec
    spec = PrefillSpec([case.blocks["shared"]], torch.tensor([0, 16], dtype=torch.int32), 20, 0, None)
    with pytest.raises(ValueError, match="RoPE table"):
        a.prepare_prefill_batch([spec])
