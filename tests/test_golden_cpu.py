"""CPU checks against the golden fixtures generated from the reference (tests/golden/make_golden.py):
the oracle's RoPE rotation is bit-equal to apply_rope_correction, and both the oracle planners and
the product planners emit the reference's integer tables exactly."""
import json
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from async_llm_b200 import CacheBlock, PrefillSpec, SharedCacheAttention, WorkerGroup
from async_llm_b200.session_plan import alloc_token_storage, plan_decode_writes
from oracle import view_oracle as vo

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def from_bits(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


@pytest.mark.parametrize("name,d", [("bf16_d128", 128), ("bf16_d256", 256), ("bf16_d64", 64)])
def test_oracle_rope_is_bit_equal_to_reference(name, d):
    z = np.load(os.path.join(GOLD, "rope_golden.npz"))
    max_pos, base = z[f"{name}_meta"]
    cache = vo.make_cos_sin_cache(d, int(max_pos), float(base))
    x = from_bits(z[f"{name}_x"])
    y = vo.rope_delta(x, torch.from_numpy(z[f"{name}_delta"]), cache)
    assert torch.equal(y.view(torch.int16), torch.from_numpy(z[f"{name}_y"]))


@pytest.mark.parametrize("name", ["mrope_d128_r64", "mrope_d256_r64", "mrope_d128_r128"])
def test_oracle_mrope_is_bit_equal_to_reference(name):
    z = np.load(os.path.join(GOLD, "rope_golden.npz"))
    rd, base, *section = z[f"{name}_meta"]
    rd, section = int(rd), [int(v) for v in section]
    inv = vo.mrope_inv_freq(rd, float(base))
    x = from_bits(z[f"{name}_x"])
    for pos_key, out_key in (("pos3", "y3"), ("pos1", "y1")):
        y = vo.rope_mrope(x, torch.from_numpy(z[f"{name}_{pos_key}"]), inv, section, rd)
        assert torch.equal(y.view(torch.int16), torch.from_numpy(z[f"{name}_{out_key}"]))


# the symbolic topologies of make_golden.py, rebuilt with this package's own classes
TOPOLOGIES = {
    "cross_readers": {
        "blocks": {"common": ([7, 2], "P+1", 1), "left": ([11], "P"), "right": ([], 0), "empty": ([], 0)},
        "views": [["common", "empty", "right", "left"], ["common", "left", "common"]],
        "writes": ["left", "right"],
    },
    "shared_prefix": {
        "blocks": {"s": ([3, 9, 4], "2*P+3"), "a": ([5], 1), "b": ([6, 8], "P+2"), "c": ([], 0),
                   "c2": ([10], "P-1")},
        "views": [["s", "a"], ["s", "b"], ["s", "c"], ["s"]],
        "writes": ["a", "b", "c", "c2"],
    },
    "thinker_writer": {
        "blocks": {"p": ([1, 2], "2*P"), "t": ([3], 2), "w": ([4], "P")},
        "views": [["p", "w", "t"], ["p", "t", "w"]],
        "writes": ["t", "w"],
    },
}


def build(topo, P):
    blocks = {}
    for name, item in topo["blocks"].items():
        length = int(eval(str(item[1]), {"P": P}))
        n_pages = -(-length // P) if length else 0
        pages = list(item[0])
        pages = pages[:n_pages] if n_pages <= len(pages) else pages + [40 + i for i in range(n_pages - len(pages))]
        b = CacheBlock(torch.device("cpu"), P)
        b.page_starts = [p * P for p in pages]
        b.num_tokens = length
        if len(item) > 2:
            b.mrope_span_override = item[2]
        blocks[name] = b
    group = WorkerGroup(cache_structure=[[blocks[n] for n in v] for v in topo["views"]],
                        write_to=[blocks[n] for n in topo["writes"]])
    return blocks, group


def cpu_attention(P):
    a = SharedCacheAttention(None, vo.make_cos_sin_cache(64, 4096, 1e4), 8, 2, 64, P, torch.bfloat16,
                             torch.device("cpu"))
    a._lanes = 16
    return a


def golden_cases(kind):
    with open(os.path.join(GOLD, "plan_golden.json")) as f:
        return json.load(f)[kind]


@pytest.mark.parametrize("case", golden_cases("decode"), ids=lambda c: f"{c['topology']}-P{c['page_size']}")
def test_decode_tables_match_reference(case):
    P = case["page_size"]
    blocks, group = build(TOPOLOGIES[case["topology"]], P)
    fresh = iter(range(60, 200))
    allocator = SimpleNamespace(alloc_pages=lambda n: torch.tensor([next(fresh) * P for _ in range(n)], dtype=torch.int32))
    pending, slots, positions = plan_decode_writes(group, allocator, P, torch.device("cpu"))
    assert [pending[id(b)] for b in group.write_to] == case["pending"]
    assert slots.tolist() == case["slots"] and slots.dtype == torch.int32
    assert positions == case["positions"]

    # the CPU oracle's planner
    plan = vo.plan_decode(group, pending, slots.tolist(), P)
    assert plan["sub_worker"] == case["sub_worker"]
    assert plan["sub_loc"] == case["sub_loc"]
    assert plan["pad_slot"] == case["pad_slot"]
    assert plan["max_segments"] == case["max_segments"]

    # the product planner
    meta = cpu_attention(P).prepare(group, pending, slots)
    assert meta.sub_worker.tolist() == case["sub_worker"]
    assert meta.sub_loc.tolist() == case["sub_loc"]
    assert meta.pad_slot.tolist() == case["pad_slot"]
    assert (meta.max_segments, meta.n_main, meta.n_aux) == (case["max_segments"], case["n_main"], case["n_aux"])
    main = case["main"] or {"indices": [], "indptr": [0], "seq_lens": [], "last_page_len": []}
    assert meta.tables.main_indices == main["indices"]
    assert meta.tables.main_indptr == main["indptr"]
    assert meta.tables.main_seq_lens == main["seq_lens"]
    assert meta.tables.main_last_page_len == main["last_page_len"]
    assert meta.tables.aux_slots == (case["aux"]["indices"] if case["aux"] else [])
    # prepare() must not publish anything into the blocks
    blocks2, _ = build(TOPOLOGIES[case["topology"]], P)
    for name in blocks:
        assert blocks[name].page_starts == blocks2[name].page_starts
        assert blocks[name].num_tokens == blocks2[name].num_tokens


@pytest.mark.parametrize("case", golden_cases("prefill"), ids=lambda c: f"case{c['case']}-P{c['page_size']}")
def test_prefill_tables_match_reference(case):
    P = case["page_size"]
    pool, specs = {}, []
    for req in case["requests"]:
        ctx = []
        for L, pages in zip(req["ctx_lens"], req["ctx_pages"]):
            if L not in pool:
                b = CacheBlock(torch.device("cpu"), P)
                b.page_starts = [p * P for p in pages]
                b.num_tokens = L
                pool[L] = b
            ctx.append(pool[L])
        specs.append(PrefillSpec(ctx, torch.tensor(req["self_pages"], dtype=torch.int32) * P,
                                 req["num_new"], req["prefix"]))
    for tables in (vo.plan_prefill(specs, P), None):
        if tables is None:
            meta = cpu_attention(P).prepare_prefill_batch(specs)
            got = {"sub_worker": meta.sub_worker.tolist(), "sub_loc": meta.sub_loc.tolist(),
                   "pad_slot": meta.pad_slot.tolist(), "max_segments": meta.max_segments,
                   "n_ctx_rows": meta.n_ctx_rows, "last_indices": meta.last_indices.tolist(),
                   "num_rows": meta.num_workers}
            ex = meta.tables.extra
            ctx_g, self_g = case["ctx"], case["self"]
            if ctx_g is not None:
                assert ex["ctx_qo_indptr"] == ctx_g["qo_indptr"]
                assert ex["ctx_kv_indptr"] == ctx_g["paged_kv_indptr"]
                assert ex["ctx_kv_indices"] == ctx_g["paged_kv_indices"]
                assert ex["ctx_seq_lens"] == ctx_g["seq_lens"]
                assert ex["ctx_last_page_len"] == ctx_g["paged_kv_last_page_len"]
            assert ex["self_qo_indptr"] == self_g["qo_indptr"]
            assert ex["self_kv_indptr"] == self_g["paged_kv_indptr"]
            assert ex["self_kv_indices"] == self_g["paged_kv_indices"]
            assert ex["self_seq_lens"] == self_g["seq_lens"]
            assert ex["self_last_page_len"] == self_g["paged_kv_last_page_len"]
        else:
            got = tables
        for key in ("sub_worker", "sub_loc", "pad_slot", "max_segments", "n_ctx_rows", "last_indices", "num_rows"):
            assert got[key] == case[key], key


def test_alloc_token_storage_fills_tail_first():
    P = 4
    handed = []

    class Alloc:
        page_size = P

        def alloc_pages(self, n):
            handed.append(n)
            return torch.tensor([40 + 4 * i for i in range(n)], dtype=torch.int32)

        def pages_to_tokens(self, starts):
            return (starts[:, None] + torch.arange(P, dtype=starts.dtype)[None, :]).flatten()

    b = CacheBlock(torch.device("cpu"), P)
    b.page_starts, b.num_tokens = [8], 2
    starts, slots = alloc_token_storage(Alloc(), P, torch.device("cpu"), 7, b)
    assert handed == [2] and starts.tolist() == [40, 44]
    assert slots.tolist() == [10, 11, 40, 41, 42, 43, 44]
    starts, slots = alloc_token_storage(Alloc(), P, torch.device("cpu"), 3, None)
    assert slots.tolist() == [40, 41, 42]
