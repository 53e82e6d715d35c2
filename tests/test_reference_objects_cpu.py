"""The planners and the GDN seam object take the REFERENCE's own request objects.

The reference's ``CacheBlock`` / ``WorkerGroup`` / ``AsyncContext``
(minisgl/shared_cache/{shared_block,worker_group,async_context}.py) are imported from a reference
checkout -- the directory named by ``ASYNC_LLM_REFERENCE_PYTHON``, else the usual places -- and fed
to this package's ``SharedCacheAttention.prepare`` / ``prepare_prefill_batch`` and
``SharedCacheGDN.set_context``: the emitted tables must equal the ones planned from this package's
own block class.  Skipped where no checkout is present.
"""
import os
import sys

import numpy as np
import pytest
import torch

import benchcases as wl
from async_llm_b200 import PrefillSpec, SharedCacheAttention
from async_llm_b200.view_attention import SharedDecodeAttentionBuffers

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# the reference's python tree: named by the environment, a checkout beside this repository, or the
# unmodified install under baseline/_ref
CANDIDATES = [os.environ.get("ASYNC_LLM_REFERENCE_PYTHON"),
              os.path.join(os.path.dirname(ROOT), "reference", "python"),
              os.path.join(ROOT, "baseline", "_ref")]


@pytest.fixture(scope="module")
def ref():
    for path in CANDIDATES:
        if path and os.path.isdir(os.path.join(path, "minisgl", "shared_cache")):
            if path not in sys.path:
                sys.path.insert(0, path)
            try:
                from minisgl.shared_cache import async_context, shared_block, worker_group
            except Exception as exc:   # noqa: BLE001
                pytest.skip(f"reference checkout at {path} does not import here: {exc}")
            return shared_block, worker_group, async_context
    pytest.skip("no reference checkout on this machine")


def mirror(case, ref_block_cls):
    out = {}
    for name, b in case.blocks.items():
        rb = ref_block_cls(torch.device("cpu"), case.page_size)
        rb.page_starts = list(b.page_starts)
        rb.num_tokens = b.num_tokens
        out[name] = rb
    return out


def cpu_attention(case):
    a = SharedCacheAttention(None, case.cos_sin, case.num_q_heads, case.num_kv_heads, case.head_dim,
                             case.page_size, torch.bfloat16, torch.device("cpu"))
    a._lanes, a._lane_width = 64, 4
    return a


def plan_tables(meta):
    h = meta.plan.host
    t = meta.tables
    return (h["items"].copy(), h["lane_off"].copy(), h["row_part_off"].copy(), h["page_indices"].copy(),
            list(meta.sub_worker_list), list(meta.sub_loc_list), list(meta.pad_slot_list),
            t.main_indices, t.main_indptr, t.main_seq_lens, t.main_last_page_len, t.aux_slots,
            meta.n_main, meta.n_aux, meta.max_segments)


def test_decode_planner_takes_reference_blocks_and_groups(ref):
    shared_block, worker_group, _ = ref
    lengths = {"common": 17, "left": 16, "right": 0, "empty": 0, "solo": 1, "tail": 33, "out": 5}
    views = [["common", "empty", "right", "left"], ["common", "left", "common"], ["solo"],
             ["tail", "common"], ["common"]]
    writes = ["left", "right", "solo", "tail", "out"]
    case = wl.make_view_case(lengths=lengths, views=views, writes=writes, num_q_heads=8, num_kv_heads=2,
                             head_dim=128, page_size=16, rope_base=1e6, seed=7)
    pending, slots, _ = case.plan_writes()
    own = plan_tables(cpu_attention(case).prepare(case.group, pending, slots))

    blocks = mirror(case, shared_block.CacheBlock)
    group = worker_group.WorkerGroup(cache_structure=[[blocks[n] for n in v] for v in views],
                                     write_to=[blocks[n] for n in writes])
    by_id = {id(b): n for n, b in case.blocks.items()}
    ref_pending = {id(blocks[by_id[k]]): v for k, v in pending.items()}
    a = cpu_attention(case)
    theirs = plan_tables(a.prepare(group, ref_pending, slots))
    for x, y in zip(own, theirs):
        assert np.array_equal(np.asarray(x), np.asarray(y))
    # the reference's positional call of the fixed-capacity buffers (graph.py:90-91): the fifth
    # positional argument is its dummy-slot tensor
    bufs = SharedDecodeAttentionBuffers(a, 5, 4, case.num_pages, torch.zeros(5, dtype=torch.int32))
    a.prepare_workspace((bufs,))
    fixed = a.prepare(group, ref_pending, slots, graph_buffers=bufs)
    assert fixed.n_main == own[12] and fixed.n_aux == own[13]


def test_prefill_planner_takes_reference_blocks(ref):
    shared_block, _, _ = ref
    lengths = {"a": 70, "b": 129, "c": 5, "w0": 0, "w1": 37, "w2": 0}
    reqs = [{"context": ["a", "b"], "write": "w0", "num_new": 45},
            {"context": ["b", "c", "a"], "write": "w1", "num_new": 33},
            {"context": [], "write": "w2", "num_new": 70}]
    case = wl.make_prefill_case(lengths=lengths, requests=reqs, num_q_heads=8, num_kv_heads=2, head_dim=128,
                                page_size=16, rope_base=1e6, seed=5)
    a = cpu_attention(case)
    own = a.prepare_prefill_batch(case.specs())
    blocks = mirror(case, shared_block.CacheBlock)
    specs = [PrefillSpec([blocks[n] for n in r["context"]], pages, r["num_new"], blocks[r["write"]].num_tokens, None)
             for r, pages in zip(case.requests, case.self_pages)]
    theirs = a.prepare_prefill_batch(specs)
    for key in ("page_indices", "tiles", "entries", "segments"):
        assert np.array_equal(own.plan.host[key], theirs.plan.host[key]), key
    assert own.sub_loc_list == theirs.sub_loc_list and own.pad_slot_list == theirs.pad_slot_list
    assert own.tables.extra == theirs.tables.extra


def test_gdn_tables_take_reference_blocks(ref):
    from async_llm_b200.blocks import CacheBlock
    from async_llm_b200.view_gdn import ROW_CONV_READ, SharedCacheGDN

    shared_block, _, _ = ref
    H, dk, dv, conv_dim, kw = 2, 128, 128, 512, 4
    g = torch.Generator().manual_seed(3)

    def fill(block, layers):
        for layer in layers:
            block.linear_affine[layer] = (torch.randn(1, H, dk, dk, generator=g), torch.randn(1, H, dv, dk, generator=g))
            block.linear_conv_state[layer] = torch.randn(conv_dim, kw, generator=g).to(torch.bfloat16)

    def build(cls):
        g.manual_seed(3)
        s, a, b, fresh = (cls(torch.device("cpu"), 16) for _ in range(4))
        fill(s, (0, 1)); fill(a, (0,)); fill(b, (0, 1))
        return [[s, a], [s, b], [fresh]], [a, b, fresh]

    tabs = []
    for cls in (CacheBlock, shared_block.CacheBlock):
        chains, targets = build(cls)
        ar = SharedCacheGDN(num_heads=H, head_k_dim=dk, head_v_dim=dv, conv_dim=conv_dim, conv_kernel=kw,
                            device=torch.device("cpu"))
        ar.set_context(chains, targets)
        ar.prepare_decode(2, torch.bfloat16)
        host = ar._step["host"]
        # addresses differ between the two builds; which entries are set must not
        tabs.append((host[:4] != 0, host[ROW_CONV_READ] != 0))
        ar.finish_decode(True)
        for t in targets:
            assert set(t.linear_affine.keys()) == {0, 1}
    assert all(np.array_equal(x, y) for x, y in zip(*tabs))
