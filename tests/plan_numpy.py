"""numpy restatement of the native decode planner (``va_plan_decode``): the same scheduling rules
written with array operations, kept here as the checker the native tables are compared against
word for word."""
from typing import Dict

import numpy as np

VA_ITEM_WORDS = 8
MIN_ITEM_KEYS = 128
CUT_SLACK_KEYS = 48


def build_decode_work(
    sub_worker: np.ndarray, sub_loc: np.ndarray, sub_len: np.ndarray, sub_page_off: np.ndarray,
    sub_tok0: np.ndarray, num_workers: int, num_kv_heads: int, num_lanes: int,
) -> Dict[str, np.ndarray]:
    """Cut the step's (sub-request, kv head) key ranges into lane-balanced items.

    Units are ordered (worker, kv head, sub-request); the concatenation of their keys is cut at
    unit boundaries and at multiples of the per-lane quota, so every lane streams the same number
    of keys and the partials of one (worker, kv head) are consecutive item indices.
    """
    n_sub = int(sub_worker.shape[0])
    W, H, G = num_workers, num_kv_heads, num_lanes
    if n_sub == 0:
        return {"items": np.zeros((0, VA_ITEM_WORDS), np.int32),
                "lane_off": np.zeros(G + 1, np.int32), "group": np.zeros(0, np.int64),
                "quota": np.array([0]), "total_keys": np.array([0])}
    order = np.argsort(sub_worker, kind="stable")
    cnt = np.bincount(sub_worker, minlength=W).astype(np.int64)
    first = np.concatenate(([0], np.cumsum(cnt)))[:-1]
    per_worker_units = cnt * H
    n_units = int(per_worker_units.sum())
    unit_worker = np.repeat(np.arange(W, dtype=np.int64), per_worker_units)
    block_start = np.concatenate(([0], np.cumsum(per_worker_units)))[:-1]
    j = np.arange(n_units, dtype=np.int64) - block_start[unit_worker]
    cw = cnt[unit_worker]
    unit_head = j // np.maximum(cw, 1)
    unit_sub = order[first[unit_worker] + j % np.maximum(cw, 1)] if n_units else np.zeros(0, np.int64)
    ulen = sub_len[unit_sub].astype(np.int64)
    uend = np.cumsum(ulen)
    ustart = uend - ulen
    total = int(uend[-1]) if n_units else 0

    # lane cuts that even out the lanes' cost = sum over items of ceil(keys / 16) + 1 stages: the
    # smallest budget T for which a greedy walk needs at most G lanes
    piece_min = max(16, CUT_SLACK_KEYS)

    def walk(T):
        cuts, lanes, pos, u = [], 0, 0, 0
        while pos < total:
            lanes += 1
            budget, empty = T, True
            while pos < total:
                while uend[u] <= pos:
                    u += 1
                rem = int(uend[u]) - pos
                avail = budget - 1
                need = -(-rem // 16)
                if need <= avail:
                    pos = int(uend[u])
                    budget -= need + 1
                    empty = False
                    continue
                take = max(avail, 0) * 16
                if empty:
                    take = max(take, min(piece_min, rem))
                    if rem - take < piece_min:
                        take = rem
                else:
                    if rem - take < piece_min:
                        take = (rem - piece_min) // 16 * 16
                    if take < piece_min:
                        take = 0
                pos += take
                break
            if pos < total:
                cuts.append(pos)
        return lanes, cuts

    lanes_cap = max(G, 1)
    T = max(-(-(-(-total // 16) + n_units) // lanes_cap), -(-MIN_ITEM_KEYS // 16) + 1)
    while walk(T)[0] > lanes_cap:
        T += 1
    quota = T * 16
    lane_cuts = np.asarray(walk(T)[1], np.int64)
    cuts = np.unique(np.concatenate((ustart, lane_cuts, np.array([total], np.int64))))
    begin, end = cuts[:-1], cuts[1:]
    n_items = int(begin.shape[0])
    unit = np.searchsorted(ustart, begin, side="right") - 1
    # zero-length units (none are emitted by the planner) would alias; guard anyway
    sub = unit_sub[unit]
    items = np.zeros((n_items, VA_ITEM_WORDS), dtype=np.int32)
    items[:, 0] = sub_page_off[sub]
    items[:, 1] = sub_tok0[sub] + (begin - ustart[unit])
    items[:, 2] = end - begin
    items[:, 3] = sub_worker[sub]
    items[:, 4] = sub_loc[sub]
    items[:, 5] = np.arange(n_items)
    items[:, 6] = unit_head[unit]
    # lane i owns the items that begin in [lane_cuts[i-1], lane_cuts[i])
    lane = np.searchsorted(lane_cuts, begin, side="right")
    lane_off = np.searchsorted(lane, np.arange(G + 1), side="left").astype(np.int32)
    group = unit_worker[unit] * H + unit_head[unit]   # non-decreasing: (worker, kv head) of each item
    return {"items": items, "lane_off": lane_off, "group": group,
            "quota": np.array([quota]), "total_keys": np.array([total])}


def plan_decode(sub_w, sub_loc, sub_len, sub_poff, sub_tok0, sub_key, W, H, n_sms, width, per_tile,
                group_min_readers, group_min_keys, tiles_per_cta, stream_rate, dense_rate,
                fixed_stream_lanes=0, fixed_dense_sms=0) -> Dict[str, np.ndarray]:
    """Tables of one decode step from its sub-requests (int64 arrays)."""
    grouped = np.zeros(sub_w.shape[0], bool)
    allow_groups = fixed_stream_lanes <= 0 or fixed_dense_sms > 0
    if allow_groups and group_min_readers > 0 and sub_w.size:
        paged = sub_key >= 0
        keys, inv, counts = np.unique(sub_key[paged], return_inverse=True, return_counts=True)
        grouped[np.nonzero(paged)[0]] = (counts[inv] >= group_min_readers) & (sub_len[paged] >= group_min_keys)
    dense_sms = 0
    dense_units = []
    if grouped.any():
        for key in np.unique(sub_key[grouped]):
            dense_units.append((int(key), np.nonzero(grouped & (sub_key == key))[0]))
        stream_cost = float(sub_len[~grouped].sum()) * H / stream_rate
        dense_cost = sum(float(sub_len[idx[0]]) * H * -(-len(idx) // per_tile) for _, idx in dense_units)
        dense_cost /= dense_rate
        share = dense_cost / max(dense_cost + stream_cost, 1e-9)
        dense_sms = int(round(n_sms * share))
        dense_sms = min(max(dense_sms, 1), n_sms - 1) if stream_cost > 0 else n_sms
        n_units = sum(-(-len(idx) // per_tile) for _, idx in dense_units) * H
        if n_units <= dense_sms:
            dense_sms = max(1, round(dense_sms / n_units)) * n_units
            dense_sms = min(dense_sms, (n_sms - 1) // n_units * n_units) or n_units
    stream_sms = n_sms - dense_sms if (~grouped).any() else 0
    G = max(stream_sms, 1) * width
    if fixed_stream_lanes > 0:
        G = fixed_stream_lanes
        if grouped.any():
            dense_sms = fixed_dense_sms

    keep = ~grouped
    work = build_decode_work(sub_w[keep], sub_loc[keep], sub_len[keep], sub_poff[keep], sub_tok0[keep], W, H, G)
    items, lane_off, item_group = work["items"], work["lane_off"], work["group"]
    n_items = items.shape[0]

    tile_parts, entry_parts, seg_parts, group_parts = [], [], [], []
    n_ent = n_seg = n_qkeys = 0
    if dense_units:
        n_rows_units = sum(-(-len(idx) // per_tile) for _, idx in dense_units) * H
        chunks_wanted = max(1, (dense_sms * tiles_per_cta) // n_rows_units)
        heads = np.arange(H, dtype=np.int64)
        for key, idx in dense_units:
            L = int(sub_len[idx[0]])
            ck = max(128, -(-(-(-L // chunks_wanted)) // 64) * 64)
            k0 = np.arange(0, L, ck, dtype=np.int64)
            n_ch = k0.size
            seg = np.zeros((n_ch, 8), np.int64)
            seg[:, 0] = sub_poff[idx[0]]
            seg[:, 1] = sub_tok0[idx[0]] + k0
            seg[:, 2] = np.minimum(ck, L - k0)
            seg[:, 4] = -1
            seg_parts.append(seg)
            for r0 in range(0, len(idx), per_tile):
                readers = idx[r0: r0 + per_tile]
                m = readers.size
                n_t = n_ch * H
                t = np.zeros((n_t, 8), np.int64)
                t[:, 0] = n_ent + np.arange(n_t) * m
                t[:, 1] = m
                t[:, 2] = n_seg + np.repeat(np.arange(n_ch), H)
                t[:, 3] = 1
                t[:, 4] = np.tile(heads, n_ch)
                t[:, 5] = 1
                t[:, 6] = 1 + n_qkeys + t[:, 4]
                t[:, 7] = np.repeat(np.arange(n_ch), H)
                n_qkeys += H
                tile_parts.append(t)
                e = np.zeros((n_t, m, 4), np.int64)
                e[:, :, 0] = sub_w[readers][None, :]
                e[:, :, 1] = sub_loc[readers][None, :]
                entry_parts.append(e.reshape(-1, 4))
                group_parts.append((sub_w[readers][None, :] * H + t[:, 4][:, None]).reshape(-1))
                n_ent += n_t * m
            n_seg += n_ch
    dense_group = np.concatenate(group_parts) if group_parts else np.zeros(0, np.int64)
    tiles = np.zeros((0, 8), np.int32)
    entries = np.zeros((0, 4), np.int32)
    segments = np.zeros((0, 8), np.int32)
    if tile_parts:
        tiles_all = np.concatenate(tile_parts)
        tiles_all = tiles_all[np.lexsort((tiles_all[:, 6], tiles_all[:, 7]))]
        tiles_all[:, 7] = 0
        tiles = tiles_all.astype(np.int32)
        segments = np.concatenate(seg_parts).astype(np.int32)

    n_groups = W * H
    cnt_s = np.bincount(item_group, minlength=n_groups) if n_items else np.zeros(n_groups, np.int64)
    cnt_d = np.bincount(dense_group, minlength=n_groups) if dense_group.size else np.zeros(n_groups, np.int64)
    base = np.concatenate(([0], np.cumsum(cnt_s + cnt_d)))
    if n_items:
        first = np.searchsorted(item_group, item_group, side="left")
        items[:, 5] = base[item_group] + (np.arange(n_items) - first)
    if dense_group.size:
        order = np.argsort(dense_group, kind="stable")
        sorted_g = dense_group[order]
        rank = np.arange(order.size) - np.searchsorted(sorted_g, sorted_g, side="left")
        entries = np.concatenate(entry_parts).astype(np.int32)
        entries[order, 2] = base[sorted_g] + cnt_s[sorted_g] + rank
    return {"items": items, "lane_off": lane_off, "row_part_off": base.astype(np.int32), "tiles": tiles,
            "entries": entries, "segments": segments, "num_partials": int(base[-1]),
            "dense_sms": dense_sms if tiles.shape[0] else 0, "num_lanes": G,
            "quota": int(work["quota"][0]), "total_keys": int(work["total_keys"][0])}


def prefill_tiles(seg_arr, req_segments, per_tile, H, n_ctas_cap):
    """numpy restatement of ``va_plan_prefill_tiles``: ``(entries [n_rows, 4], tiles [n, 8])``.

    ``req_segments`` rows are (seg_begin, seg_count, row offset, S); a tile is ``per_tile`` consecutive
    new tokens of one (request, kv head); heaviest first (keys walked x rows, stable), every other round
    of ``min(n_ctas_cap, tiles)`` rows reversed."""
    seg_arr = np.asarray(seg_arr, np.int64).reshape(-1, 8)
    n_rows = max((off + S for _, _, off, S in req_segments), default=0)
    entries = np.zeros((n_rows, 4), np.int32)
    cols = []
    for seg_begin, seg_count, off, S in req_segments:
        entries[off: off + S, 0] = np.arange(off, off + S)
        entries[off: off + S, 1] = np.arange(S)
        segs = seg_arr[seg_begin: seg_begin + seg_count]
        open_keys = int(segs[segs[:, 4] < 0, 2].sum())
        causal = segs[segs[:, 4] >= 0]
        e0 = np.arange(0, S, per_tile, dtype=np.int64)
        cnt = np.minimum(per_tile, S - e0)
        keys = open_keys + np.minimum(causal[:, 2][None, :], causal[:, 4][None, :] + (e0 + cnt)[:, None]).sum(1)
        n = e0.size
        cols.append(np.stack((keys * cnt, off + e0, cnt, np.full(n, seg_begin), np.full(n, seg_count)), axis=1))
    rows_t = np.concatenate(cols)
    per_head = np.repeat(rows_t, H, axis=0)
    heads = np.tile(np.arange(H, dtype=np.int64), rows_t.shape[0])
    order = np.argsort(-per_head[:, 0], kind="stable")
    n_tiles = order.size
    n_ctas = max(1, min(n_ctas_cap, n_tiles))
    if n_ctas > 1:
        pos = np.arange(n_tiles)
        rnd, k = pos // n_ctas, pos % n_ctas
        width = np.minimum(n_ctas, n_tiles - rnd * n_ctas)
        order = order[np.where(rnd % 2 == 1, rnd * n_ctas + (width - 1 - k), pos)]
    tiles = np.zeros((n_tiles, 8), np.int32)
    tiles[:, 0:4] = per_head[order, 1:5]
    tiles[:, 4] = heads[order]
    return entries, tiles


def gdn_tables(block_addr, block_conv, chain_idx, target_idx, write_a, write_b, conv_write, layers):
    """Address tables of a GDN forward by array indexing: ``[8, L, W, depth]`` int64 (rows: chain
    A_hat, chain B_hat, read a, read b, conv read, write a, write b, conv write; rows 2..7 in
    ``[..., 0]``).  ``write_*`` are ``(base [W], stride)`` pairs or None.  The conv window read by a
    worker is the one of the last block of its chain that has one
    (minisgl/shared_cache/gdn.py:182-207)."""
    W, depth = chain_idx.shape
    tab = np.zeros((8, layers, W, depth), np.int64)
    tab[0] = block_addr[chain_idx, :, 0].transpose(2, 0, 1)
    tab[1] = block_addr[chain_idx, :, 1].transpose(2, 0, 1)
    tab[2, :, :, 0] = block_addr[target_idx, :, 0].T
    tab[3, :, :, 0] = block_addr[target_idx, :, 1].T
    if block_conv is not None:
        caddr = block_conv[chain_idx]                                    # [W, depth, L]
        has = caddr != 0
        last = depth - 1 - np.argmax(has[:, ::-1, :], axis=1)            # [W, L]
        picked = np.take_along_axis(caddr, last[:, None, :], axis=1)[:, 0, :]
        tab[4, :, :, 0] = np.where(has.any(axis=1), picked, 0).T
    steps = np.arange(layers, dtype=np.int64)
    for row, out in ((5, write_a), (6, write_b), (7, conv_write)):
        if out is not None:
            base, stride = out
            tab[row, :, :, 0] = base[None, :] + steps[:, None] * stride
    return tab
