"""Seeded ordinary (view-less) batches for the attention-backend tests: a pool, a page table of
token slots and request records shaped like the host framework's (``table_idx``, ``cached_len``,
``device_len``, ``extend_len`` -- minisgl/core.py Req)."""
from types import SimpleNamespace

import torch


def make_plain_case(lens, *, hq=8, hkv=2, d=128, page_size=16, seed=3, max_len=512, min_slots=0):
    """``lens``: list of (cached_len, extend_len).  Returns a namespace with the pool contents (CPU),
    the page table, the requests, the new rows' q/k/v, ``out_loc`` and ``positions``."""
    g = torch.Generator().manual_seed(seed)
    n_req = len(lens)
    total = sum(c + e for c, e in lens)
    num_slots = -(-max(total + 64, min_slots) // page_size) * page_size   # min_slots: one pool geometry for several cases
    perm = torch.randperm(num_slots, generator=g)
    table = torch.zeros(n_req + 2, max_len, dtype=torch.int32)
    k_pool = torch.zeros(num_slots // page_size, page_size, hkv, d, dtype=torch.bfloat16)
    v_pool = torch.zeros_like(k_pool)
    kf, vf = k_pool.view(-1, hkv, d), v_pool.view(-1, hkv, d)
    reqs, out_loc, positions, cur = [], [], [], 0
    for r, (cached, extend) in enumerate(lens):
        slots = perm[cur: cur + cached + extend]
        cur += cached + extend
        table[r + 1, : cached + extend] = slots.to(torch.int32)
        kf[slots[:cached]] = (torch.randn(cached, hkv, d, generator=g) * 0.5).to(torch.bfloat16)
        vf[slots[:cached]] = (torch.randn(cached, hkv, d, generator=g) * 0.5).to(torch.bfloat16)
        reqs.append(SimpleNamespace(table_idx=r + 1, cached_len=cached, device_len=cached + extend, extend_len=extend))
        out_loc += slots[cached:].tolist()
        positions += list(range(cached, cached + extend))
    rows = len(out_loc)
    q = torch.randn(rows, hq * d, generator=g).to(torch.bfloat16)
    k = (torch.randn(rows, hkv * d, generator=g) * 0.5).to(torch.bfloat16)
    v = (torch.randn(rows, hkv * d, generator=g) * 0.5).to(torch.bfloat16)
    return SimpleNamespace(hq=hq, hkv=hkv, d=d, page_size=page_size, k_pool=k_pool, v_pool=v_pool, table=table,
                           reqs=reqs, q=q, k=k, v=v, out_loc=torch.tensor(out_loc, dtype=torch.int32),
                           positions=torch.tensor(positions, dtype=torch.int32),
                           config=SimpleNamespace(num_qo_heads=hq, num_kv_heads=hkv, head_dim=d))


def make_batch(case, phase, device):
    n = len(case.reqs)
    return SimpleNamespace(reqs=case.reqs, padded_reqs=case.reqs, phase=phase, is_decode=phase == "decode",
                           is_prefill=phase == "prefill", size=n, padded_size=n,
                           out_loc=case.out_loc.to(device), positions=case.positions.to(device),
                           attn_metadata=None)


def oracle_rows(case):
    """Pool after the store and the oracle's output rows."""
    from oracle import view_oracle as vo

    k_pool, v_pool = case.k_pool.clone(), case.v_pool.clone()
    kf, vf = k_pool.view(-1, case.hkv * case.d), v_pool.view(-1, case.hkv * case.d)
    kf[case.out_loc.long()] = case.k
    vf[case.out_loc.long()] = case.v
    slot_rows = [case.table[r.table_idx, : r.device_len].tolist() for r in case.reqs]
    out = vo.plain_attention(case.q, k_pool, v_pool, slot_rows, [r.extend_len for r in case.reqs], case.hq)
    return out, k_pool, v_pool
