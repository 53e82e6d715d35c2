"""The native decode planner (``va_plan_decode``) against its numpy restatement: every table,
word for word, over random sub-request lists, including frozen (graph) lane counts, degenerate
inputs and the capacity protocol."""
import ctypes as C

import numpy as np
import pytest

from async_llm_b200 import _lib
import plan_numpy


def native_plan(subs, pages, W, H, n_sms, width, per_tile, min_readers, min_keys, tiles_per_cta,
                stream_rate, dense_rate, fixed_lanes=0, fixed_dense=0, cap=None):
    p = _lib.VaPlanParams()
    p.num_workers, p.num_kv_heads, p.readers_per_tile = W, H, per_tile
    p.num_sms, p.lane_width = n_sms, width
    p.group_min_readers, p.group_min_keys, p.dense_tiles_per_cta = min_readers, min_keys, tiles_per_cta
    p.min_item_keys, p.cut_slack_keys = plan_numpy.MIN_ITEM_KEYS, plan_numpy.CUT_SLACK_KEYS
    p.fixed_stream_lanes, p.fixed_dense_sms = fixed_lanes, fixed_dense
    p.stream_rate, p.dense_rate = stream_rate, dense_rate
    arrs = [np.ascontiguousarray(a, np.int32) for a in subs]
    pages = np.ascontiguousarray(pages, np.int32)
    lay = _lib.VaPlanLayout()
    n = arrs[0].size
    fn = _lib.lib().va_plan_decode
    call = lambda blob, words: fn(C.byref(p), n, *[a.ctypes.data for a in arrs], pages.ctypes.data, pages.size,
                                  blob.ctypes.data if blob is not None else None, words, C.byref(lay))
    if cap is None:
        rc = call(None, 0)
        assert rc == _lib.VA_ERR_CAPACITY and lay.total_words >= 4
        cap = int(lay.total_words)
    blob = np.full(cap + 8, -77, np.int32)
    rc = call(blob, cap)
    return rc, lay, blob


def random_subs(rng, W, n_blocks, max_len, P):
    """Worker-major sub-requests over a pool of blocks, plus a few implicit-self ones."""
    lens = rng.integers(1, max_len, n_blocks)
    lens[rng.random(n_blocks) < 0.3] += 600
    n_pages = -(-lens // P)
    run_off = np.concatenate(([0], np.cumsum(n_pages)))
    sub = {k: [] for k in ("w", "loc", "len", "poff", "tok0", "key")}
    for w in range(W):
        for b in rng.permutation(n_blocks)[: rng.integers(0, min(n_blocks, 6) + 1)]:
            sub["w"].append(w); sub["loc"].append(int(rng.integers(-50, 5000))); sub["len"].append(int(lens[b]))
            sub["poff"].append(int(run_off[b])); sub["tok0"].append(0); sub["key"].append(int(run_off[b]))
    n_aux = int(rng.integers(0, 4))
    for i in range(n_aux):
        sub["w"].append(int(rng.integers(0, W))); sub["loc"].append(int(rng.integers(0, 99))); sub["len"].append(1)
        sub["poff"].append(int(run_off[-1]) + i); sub["tok0"].append(int(rng.integers(0, P))); sub["key"].append(-1)
    pages = rng.integers(0, 100000, int(run_off[-1]) + n_aux)
    return [np.asarray(sub[k], np.int64) for k in ("w", "loc", "len", "poff", "tok0", "key")], pages


def compare(subs, pages, W, H, kw, fixed=(0, 0)):
    want = plan_numpy.plan_decode(*subs, W, H, kw["n_sms"], kw["width"], kw["per_tile"], kw["min_readers"],
                                  kw["min_keys"], kw["tiles_per_cta"], kw["stream_rate"], kw["dense_rate"],
                                  fixed_stream_lanes=fixed[0], fixed_dense_sms=fixed[1])
    rc, lay, blob = native_plan(subs, pages, W, H, kw["n_sms"], kw["width"], kw["per_tile"], kw["min_readers"],
                                kw["min_keys"], kw["tiles_per_cta"], kw["stream_rate"], kw["dense_rate"],
                                fixed_lanes=fixed[0], fixed_dense=fixed[1])
    assert rc == 0
    sec = lambda off, n: blob[off: off + n]
    assert (lay.num_lanes, lay.num_partials, lay.dense_sms) == (want["num_lanes"], want["num_partials"], want["dense_sms"])
    assert (lay.quota, lay.total_keys) == (want["quota"], want["total_keys"])
    assert np.array_equal(sec(lay.off_pages, lay.num_pages), pages.astype(np.int32))
    assert lay.num_items == want["items"].shape[0]
    assert np.array_equal(sec(lay.off_items, lay.num_items * 8).reshape(-1, 8), want["items"])
    assert np.array_equal(sec(lay.off_lane_off, lay.num_lanes + 1), want["lane_off"])
    assert lay.num_groups == W * H
    assert np.array_equal(sec(lay.off_row_part_off, W * H + 1), want["row_part_off"])
    assert (lay.num_tiles, lay.num_entries, lay.num_segments) == (
        want["tiles"].shape[0], want["entries"].shape[0], want["segments"].shape[0])
    assert np.array_equal(sec(lay.off_tiles, lay.num_tiles * 8).reshape(-1, 8), want["tiles"])
    assert np.array_equal(sec(lay.off_entries, lay.num_entries * 4).reshape(-1, 4), want["entries"])
    assert np.array_equal(sec(lay.off_segments, lay.num_segments * 8).reshape(-1, 8), want["segments"])
    for off in (lay.off_pages, lay.off_items, lay.off_lane_off, lay.off_row_part_off, lay.off_tiles,
                lay.off_entries, lay.off_segments):
        assert off % 4 == 0
    assert (blob[int(lay.total_words):] == -77).all(), "nothing is written past total_words"
    return lay


@pytest.mark.parametrize("seed", range(12))
def test_native_tables_equal_numpy_restatement(seed):
    rng = np.random.default_rng(seed)
    W = int(rng.integers(1, 40))
    H = int(rng.choice([1, 2, 8]))
    P = int(rng.choice([1, 16, 64]))
    subs, pages = random_subs(rng, W, int(rng.integers(1, 30)), int(rng.choice([40, 900, 5000])), P)
    kw = dict(n_sms=int(rng.choice([3, 37, 148])), width=int(rng.choice([1, 4, 6])),
              per_tile=int(rng.choice([4, 16, 64])), min_readers=int(rng.choice([0, 2, 4])),
              min_keys=int(rng.choice([1, 256])), tiles_per_cta=int(rng.choice([1, 2])),
              stream_rate=31.0, dense_rate=float(rng.choice([10.0, 16.0, 30.0])))
    compare(subs, pages, W, H, kw)
    # the same step under a captured graph's frozen split
    compare(subs, pages, W, H, kw, fixed=(kw["width"] * 5, 0))
    compare(subs, pages, W, H, kw, fixed=(kw["width"] * 5, 2))


def test_native_planner_degenerate_inputs():
    kw = dict(n_sms=8, width=4, per_tile=16, min_readers=4, min_keys=256, tiles_per_cta=1,
              stream_rate=31.0, dense_rate=16.0)
    empty = [np.zeros(0, np.int64)] * 6
    lay = compare(empty, np.zeros(0, np.int64), 3, 2, kw)
    assert lay.num_items == 0 and lay.num_partials == 0 and lay.num_lanes == 4
    # every sub-request reads the same long block: nothing is left for the streaming lanes
    n = 9
    subs = [np.arange(n), np.full(n, 7), np.full(n, 4096), np.zeros(n, np.int64), np.zeros(n, np.int64),
            np.zeros(n, np.int64)]
    lay = compare([np.asarray(a, np.int64) for a in subs], np.arange(256), n, 2, kw)
    assert lay.num_items == 0 and lay.num_tiles > 0 and 0 < lay.dense_sms <= 8


def test_native_planner_capacity_and_bad_arguments():
    rng = np.random.default_rng(3)
    subs, pages = random_subs(rng, 5, 6, 900, 16)
    args = (5, 2, 8, 4, 16, 4, 256, 1, 31.0, 16.0)
    rc, lay, blob = native_plan(subs, pages, *args, cap=8)
    assert rc == _lib.VA_ERR_CAPACITY and lay.total_words > 8
    assert (blob == -77).all(), "a blob that is too small is left untouched"
    bad = [a.copy() for a in subs]
    bad[0][0] = 5                                     # worker index outside [0, W)
    rc, _, _ = native_plan(bad, pages, *args, cap=1 << 16)
    assert rc == -1
    rc, _, _ = native_plan(subs, pages, 5, 0, 8, 4, 16, 4, 256, 1, 31.0, 16.0, cap=1 << 16)
    assert rc == -1


def test_view_entry_point_checks_its_arguments():
    # va_plan_views on hand-built views: a good call, then malformed inputs (no GPU involved)
    p = _lib.VaPlanParams()
    p.num_workers, p.num_kv_heads, p.readers_per_tile, p.num_sms, p.lane_width = 2, 2, 16, 8, 4
    p.group_min_readers, p.group_min_keys, p.dense_tiles_per_cta = 4, 256, 1
    p.min_item_keys, p.cut_slack_keys = plan_numpy.MIN_ITEM_KEYS, plan_numpy.CUT_SLACK_KEYS
    p.stream_rate, p.dense_rate = 31.0, 16.0
    i32 = lambda *v: np.asarray(v, np.int32)
    view_start, view_block = i32(0, 2, 3), i32(0, 1, 0)          # worker 0: [b0, b1], worker 1: [b0]
    block_len, block_span, block_pages = i32(20, 0), i32(20, 0), i32(2, 0)   # b1 is empty: skipped
    pending, pages = i32(-1, -1), i32(5, 9)
    aux_w, aux_loc, aux_slot = i32(1), i32(7), np.asarray([83], np.int64)     # worker 1 writes outside its view
    step = _lib.VaViewStep()
    step.num_workers, step.num_blocks, step.num_aux, step.page_size = 2, 2, 1, 16
    for name, arr in (("view_start", view_start), ("view_block", view_block), ("block_len", block_len),
                      ("block_span", block_span), ("block_pages", block_pages), ("block_pending_page", pending),
                      ("pages", pages), ("aux_worker", aux_w), ("aux_loc", aux_loc), ("aux_slot", aux_slot)):
        setattr(step, name, arr.ctypes.data)
    lay, info = _lib.VaPlanLayout(), _lib.VaViewSubs()
    blob, subs = np.zeros(4096, np.int32), np.zeros((5, 4), np.int32)
    call = lambda stride=4: _lib.lib().va_plan_views(C.byref(p), C.byref(step), blob.ctypes.data, blob.size,
                                                     C.byref(lay), subs.ctypes.data, stride, C.byref(info))
    assert call() == 0
    assert (info.num_main, info.num_aux, info.max_segments) == (2, 1, 2)
    assert subs[0, :3].tolist() == [0, 1, 1] and subs[1, :3].tolist() == [19, 19, 7]     # worker, loc
    assert subs[2, :3].tolist() == [0, 0, 1] and subs[4, :3].tolist() == [0, 0, -1]      # segment, block
    assert blob[lay.off_pages: lay.off_pages + lay.num_pages].tolist() == [5, 9, 83 // 16]
    assert call(stride=2) == _lib.VA_ERR_CAPACITY          # sub_out rows too short
    view_block[1] = 7
    assert call() == -1                                    # block index outside the table
    view_block[1] = 1
    view_start[0] = 1
    assert call() == -1                                    # offsets must start at 0
    view_start[0] = 0
    p.num_workers = 3
    assert call() == -1                                    # params and step disagree on the worker count


def test_native_prefill_tile_planner_matches_the_numpy_restatement():
    import ctypes as C

    rng = np.random.default_rng(11)
    lib = _lib.lib()
    for case in range(40):
        R = int(rng.integers(1, 9))
        per_tile = int(rng.choice([4, 8, 32, 64]))
        H = int(rng.choice([1, 2, 8]))
        n_ctas_cap = int(rng.choice([1, 3, 16, 148]))
        segments, reqs = [], []
        off = 0
        for r in range(R):
            S = int(rng.integers(1, 300))
            T = int(rng.integers(0, 50))
            seg_begin = len(segments)
            for _ in range(int(rng.integers(0, 4))):
                segments.append([int(rng.integers(0, 99)), 0, int(rng.integers(1, 5000)), int(rng.integers(0, 9000)), -1, 0, 0, 0])
            segments.append([int(rng.integers(0, 99)), 0, T + S, T, T, 0, 0, 0])
            reqs.append((seg_begin, len(segments) - seg_begin, off, S))
            off += S
        want_entries, want_tiles = plan_numpy.prefill_tiles(segments, reqs, per_tile, H, n_ctas_cap)
        seg_arr = np.asarray(segments, np.int32).reshape(-1, 8)
        req_arr = np.asarray(reqs, np.int32).reshape(-1, 4)
        cap = sum(-(-S // per_tile) for _, _, _, S in reqs) * H
        entries = np.full((off, 4), -7, np.int32)
        tiles = np.full((cap, 8), -7, np.int32)
        n = C.c_int32(0)
        rc = lib.va_plan_prefill_tiles(seg_arr.ctypes.data, seg_arr.shape[0], req_arr.ctypes.data, R, per_tile, H,
                                       n_ctas_cap, entries.ctypes.data, off, tiles.ctypes.data, cap, C.byref(n))
        assert rc == 0 and n.value == want_tiles.shape[0] == cap, case
        assert np.array_equal(entries, want_entries), case
        assert np.array_equal(tiles, want_tiles), case
        # too small a table is refused and says how many rows it needs
        if cap > 1:
            rc = lib.va_plan_prefill_tiles(seg_arr.ctypes.data, seg_arr.shape[0], req_arr.ctypes.data, R, per_tile, H,
                                           n_ctas_cap, entries.ctypes.data, off, tiles.ctypes.data, cap - 1, C.byref(n))
            assert rc == _lib.VA_ERR_CAPACITY and n.value == cap


def test_native_gdn_tables_match_the_numpy_restatement():
    rng = np.random.default_rng(23)
    lib = _lib.lib()
    for case in range(60):
        B = int(rng.integers(1, 12))
        L = int(rng.integers(1, 5))
        W = int(rng.integers(1, 9))
        depth = int(rng.integers(1, 5))
        block_addr = rng.integers(1, 1 << 40, size=(B + 1, L, 2)).astype(np.int64)
        block_addr[rng.random((B + 1, L)) < 0.3] = 0          # blocks without a summary in a layer
        block_addr[0] = 0
        block_conv = rng.integers(1, 1 << 40, size=(B + 1, L)).astype(np.int64)
        block_conv[rng.random((B + 1, L)) < 0.5] = 0
        block_conv[0] = 0
        chain_idx = np.zeros((W, depth), np.int32)
        for w in range(W):
            n = int(rng.integers(0, depth + 1))
            chain_idx[w, :n] = rng.integers(1, B + 1, size=n)
        target_idx = rng.integers(1, B + 1, size=W).astype(np.int32)
        with_outputs = case % 3 != 0
        outs = [None, None, None]
        if with_outputs:
            outs = [(rng.integers(1, 1 << 40, size=W).astype(np.int64), int(rng.integers(1, 1 << 20))) for _ in range(3)]
        want = plan_numpy.gdn_tables(block_addr, block_conv if with_outputs else None, chain_idx.astype(np.int64),
                                     target_idx.astype(np.int64), *outs, L)
        tab = np.full((8, L, W, depth), -5, np.int64)
        ptr = lambda a: a.ctypes.data if a is not None else None
        base = [o[0] if o is not None else None for o in outs]
        stride = [o[1] if o is not None else 0 for o in outs]
        rc = lib.va_gdn_plan_tables(ptr(block_addr), ptr(block_conv) if with_outputs else None, ptr(chain_idx),
                                    ptr(target_idx), ptr(base[0]), stride[0], ptr(base[1]), stride[1], ptr(base[2]),
                                    stride[2], B, L, W, depth, ptr(tab))
        assert rc == 0, case
        assert np.array_equal(tab, want), case
    # a block number outside the table is refused
    bad = chain_idx.copy()
    bad[0, 0] = B + 1
    rc = lib.va_gdn_plan_tables(ptr(block_addr), None, ptr(bad), ptr(target_idx), None, 0, None, 0, None, 0,
                                B, L, W, depth, ptr(tab))
    assert rc == -1   # VA_ERR_BAD_ARG
