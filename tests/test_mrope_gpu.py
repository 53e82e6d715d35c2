"""Interleaved 3-axis mRoPE on the GPU: ``_rope`` of an attention op built with ``mrope_section``
against the fixture generated from the reference's ``_rope_mrope`` (bit-exact), and a decode step
whose new keys carry 3-axis positions against the CPU oracle (pool bit-exact, outputs within the
attention tolerance)."""
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from async_llm_b200 import MHAKVCache, SharedCacheAttention
import benchcases as wl
from helpers import assert_close_bf16
from oracle import view_oracle as vo

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def from_bits(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


@pytest.mark.parametrize("name", ["mrope_d128_r64", "mrope_d256_r64", "mrope_d128_r128"])
def test_rope_with_mrope_section_is_bit_equal_to_reference(cuda_device, name):
    z = np.load(os.path.join(GOLD, "rope_golden.npz"))
    rd, base, *section = z[f"{name}_meta"]
    rd, section = int(rd), tuple(int(v) for v in section)
    x = from_bits(z[f"{name}_x"])
    d = x.shape[-1]
    a = SharedCacheAttention(None, torch.zeros(4096, rd), 8, 2, d, 16, torch.bfloat16, cuda_device,
                             rotary_dim=rd, mrope_section=section, rope_base=float(base))
    for pos_key, out_key in (("pos3", "y3"), ("pos1", "y1")):
        pos = torch.from_numpy(z[f"{name}_{pos_key}"])
        y = a._rope(x.to(cuda_device), pos.to(cuda_device))
        assert torch.equal(y.cpu().view(torch.int16), torch.from_numpy(z[f"{name}_{out_key}"])), pos_key


def test_decode_step_with_three_axis_key_positions(cuda_device):
    # config-1 topology; the new token of every request is an "image" token whose (t, h, w)
    # positions differ, so its key is rotated per axis on its way into the pool
    case = wl.config1_decode(page_size=16)
    rd, section, base = 64, (11, 11, 10), 1e6
    D, Hkv, Hq = case.head_dim, case.num_kv_heads, case.num_q_heads
    table = vo.mrope_cos_sin_cache(rd, case.max_pos, base)
    pool = MHAKVCache(Hkv, 1, D, case.num_pages, case.page_size, torch.bfloat16, cuda_device)
    pool.k_cache(0).copy_(case.k_pool)
    pool.v_cache(0).copy_(case.v_pool)
    attn = SharedCacheAttention(pool, torch.zeros(case.max_pos, rd), Hq, Hkv, D, case.page_size, torch.bfloat16,
                                cuda_device, rotary_dim=rd, mrope_section=section, rope_base=base)
    assert torch.equal(attn._cos_sin.cpu(), table)
    pending, slots, positions = case.plan_writes()
    W = len(case.views)
    g = torch.Generator().manual_seed(5)
    pos3 = positions.long()[None, :] + torch.randint(0, 40, (3, W), generator=g)
    meta = attn.prepare(case.group, pending, slots)
    batch = SimpleNamespace(attn_metadata=meta, positions=positions.to(cuda_device), out_loc=slots.to(cuda_device),
                            mrope_positions=pos3.to(cuda_device))
    out = attn.forward(case.q.to(cuda_device), case.k_new.to(cuda_device), case.v_new.to(cuda_device), 0, batch)
    torch.cuda.synchronize()
    attn.check_status()

    k_ref, v_ref = case.k_pool.clone(), case.v_pool.clone()
    k_rot = vo.rope_mrope(case.k_new.view(W, Hkv, D), pos3, vo.mrope_inv_freq(rd, base), section, rd)
    k_ref.view(-1, Hkv, D)[slots.long()] = k_rot
    v_ref.view(-1, Hkv, D)[slots.long()] = case.v_new.view(W, Hkv, D)
    assert torch.equal(pool.k_cache(0).cpu(), k_ref), "keys rotated per axis land in the pool bit-exactly"
    assert torch.equal(pool.v_cache(0).cpu(), v_ref)
    want = vo.view_decode(case.q, k_ref, v_ref, case.group, pending, slots.tolist(), table, Hq, rotary_dim=rd)
    assert_close_bf16(out, want, "decode with 3-axis key positions")


def test_prefill_with_three_axis_query_positions(cuda_device):
    # two requests; the first one's new tokens are an image patch grid (per-axis positions), the
    # second one's are text.  Keys enter the pool rotated per axis, queries are rotated per axis
    # inside the dense-tile kernel; the causal mask stays on token indices.
    from benchcases import make_prefill_case
    rd, section, base = 64, (11, 11, 10), 1e6
    case = make_prefill_case(lengths={"sys": 200, "doc": 333, "a": 5, "b": 0},
                             requests=[{"context": ["sys", "doc"], "write": "a", "num_new": 70},
                                       {"context": ["sys"], "write": "b", "num_new": 33}],
                             num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, rope_base=base, seed=77)
    D, Hkv, Hq, P = case.head_dim, case.num_kv_heads, case.num_q_heads, case.page_size
    N = case.q.shape[0]
    table = vo.mrope_cos_sin_cache(rd, 4096, base)
    inv = vo.mrope_inv_freq(rd, base)
    g = torch.Generator().manual_seed(6)
    S0 = case.requests[0]["num_new"]
    grid = torch.stack((torch.zeros(S0, dtype=torch.long), torch.arange(S0) // 10, torch.arange(S0) % 10))
    specs = case.specs()
    specs[0].mrope_rel = grid + torch.randint(0, 3, (1, S0), generator=g)
    # block-relative 3-axis key positions of the new tokens: prefix span + per-axis rel
    key_pos3 = torch.cat([(sp.mrope_rel if sp.mrope_rel is not None
                           else torch.arange(sp.num_new).view(1, -1).expand(3, -1)) + sp.self_prefix_len
                          for sp in specs], dim=1)

    pool = MHAKVCache(Hkv, 1, D, case.num_pages, P, torch.bfloat16, cuda_device)
    pool.k_cache(0).copy_(case.k_pool)
    pool.v_cache(0).copy_(case.v_pool)
    attn = SharedCacheAttention(pool, torch.zeros(4096, rd), Hq, Hkv, D, P, torch.bfloat16, cuda_device,
                                rotary_dim=rd, mrope_section=section, rope_base=base)
    meta = attn.prepare_prefill_batch(specs)
    assert tuple(meta.sub_loc.shape) == (3, len(meta.sub_worker_list))
    batch = SimpleNamespace(attn_metadata=meta, positions=case.positions.to(cuda_device),
                            out_loc=case.out_loc.to(cuda_device), mrope_positions=key_pos3.to(cuda_device))
    out = attn.forward(case.q.to(cuda_device), case.k_new.to(cuda_device), case.v_new.to(cuda_device), 0, batch)
    torch.cuda.synchronize()
    attn.check_status()

    k_ref, v_ref = case.k_pool.clone(), case.v_pool.clone()
    k_ref.view(-1, Hkv, D)[case.out_loc.long()] = vo.rope_mrope(case.k_new.view(N, Hkv, D), key_pos3, inv, section, rd)
    v_ref.view(-1, Hkv, D)[case.out_loc.long()] = case.v_new.view(N, Hkv, D)
    assert torch.equal(pool.k_cache(0).cpu(), k_ref)
    want = vo.view_prefill(case.q, k_ref, v_ref, specs, table, Hq, rotary_dim=rd, mrope=(inv, section))
    assert_close_bf16(out, want, "prefill with 3-axis query positions")
    # the per-axis positions matter: with text positions the image rows move by several times the
    # mean-abs tolerance (1e-3), the text request not at all
    plain = vo.view_prefill(case.q, k_ref, v_ref, case.specs(), table, Hq, rotary_dim=rd, mrope=(inv, section))
    assert (plain[:S0] - want[:S0]).abs().mean() > 3e-3
    assert (out[:S0].float().cpu() - plain[:S0]).abs().mean() > 3e-3
    assert torch.equal(plain[S0:], want[S0:])


def test_three_axis_query_positions_under_fixed_prefill_buffers(cuda_device):
    # the same batch planned into fixed-capacity prefill tables (more rows, requests and pages than it
    # uses): the per-axis positions sit in the tables' [3, rows] region, a text-only batch planned into
    # the same tables afterwards gets its token indices on all axes
    from async_llm_b200 import SharedPrefillAttentionBuffers
    from benchcases import make_prefill_case
    rd, section, base = 64, (11, 11, 10), 1e6
    case = make_prefill_case(lengths={"sys": 200, "doc": 333, "a": 5, "b": 0},
                             requests=[{"context": ["sys", "doc"], "write": "a", "num_new": 70},
                                       {"context": ["sys"], "write": "b", "num_new": 33}],
                             num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, rope_base=base, seed=77)
    D, Hkv, Hq, P = case.head_dim, case.num_kv_heads, case.num_q_heads, case.page_size
    N, CAP = case.q.shape[0], 128
    table = vo.mrope_cos_sin_cache(rd, 4096, base)
    inv = vo.mrope_inv_freq(rd, base)
    S0 = case.requests[0]["num_new"]
    grid = torch.stack((torch.zeros(S0, dtype=torch.long), torch.arange(S0) // 10, torch.arange(S0) % 10))
    pool = MHAKVCache(Hkv, 1, D, case.num_pages, P, torch.bfloat16, cuda_device)
    attn = SharedCacheAttention(pool, torch.zeros(4096, rd), Hq, Hkv, D, P, torch.bfloat16, cuda_device,
                                rotary_dim=rd, mrope_section=section, rope_base=base)
    bufs = SharedPrefillAttentionBuffers(attn, workers=3, depth=3, rows=CAP, max_pages=case.num_pages)
    assert bufs.with_axes
    pad = lambda t, fill=0: torch.cat((t, torch.full((CAP - N, *t.shape[1:]), fill, dtype=t.dtype))).to(cuda_device)
    q, k, v = pad(case.q), pad(case.k_new), pad(case.v_new)
    for with_image in (True, False, True):
        specs = case.specs()
        if with_image:
            specs[0].mrope_rel = grid
        key_pos3 = torch.cat([(sp.mrope_rel if sp.mrope_rel is not None
                               else torch.arange(sp.num_new).view(1, -1).expand(3, -1)) + sp.self_prefix_len
                              for sp in specs], dim=1)
        pool.k_cache(0).copy_(case.k_pool)
        pool.v_cache(0).copy_(case.v_pool)
        meta = attn.prepare_prefill_batch(specs, graph_buffers=bufs)
        pos3 = torch.zeros(3, CAP, dtype=torch.long)
        pos3[:, :N] = key_pos3
        batch = SimpleNamespace(attn_metadata=meta, positions=pad(case.positions), out_loc=pad(case.out_loc, -1),
                                mrope_positions=pos3.to(cuda_device))
        out = attn.forward(q, k, v, 0, batch)
        torch.cuda.synchronize()
        attn.check_status()
        k_ref, v_ref = case.k_pool.clone(), case.v_pool.clone()
        k_ref.view(-1, Hkv, D)[case.out_loc.long()] = vo.rope_mrope(case.k_new.view(N, Hkv, D), key_pos3, inv, section, rd)
        v_ref.view(-1, Hkv, D)[case.out_loc.long()] = case.v_new.view(N, Hkv, D)
        assert torch.equal(pool.k_cache(0).cpu(), k_ref)
        want = vo.view_prefill(case.q, k_ref, v_ref, specs, table, Hq, rotary_dim=rd, mrope=(inv, section))
        assert_close_bf16(out[:N], want, f"fixed prefill buffers, image rows: {with_image}")
