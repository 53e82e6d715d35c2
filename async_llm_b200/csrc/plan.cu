// Host planner of one decode step: turns the step's sub-requests (worker, block) into the device
// work list of the streaming kernel (lane-balanced items) and the dense tiles of blocks read by
// many workers.  Pure host code; nothing here touches the GPU.
//
// The semantics of the sub-requests (post-append lengths, pending pages, implicit self segment)
// are those of SharedCacheAttention.prepare (shared_cache/attention.py:282-448) and are decided by
// the caller; this file only schedules them.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <vector>

#include "../../include/view_attn_b200.h"

namespace {

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int64_t align4(int64_t n) { return (n + 3) / 4 * 4; }

struct DenseUnit {
  int32_t key;
  std::vector<int32_t> readers;  // sub-request indices, ascending
};

struct Scratch {
  std::vector<uint8_t> grouped;
  std::vector<int32_t> sorted_keys, key_count;
  std::vector<DenseUnit> units;
  std::vector<int32_t> keep;                 // streamed sub-requests, input order
  std::vector<int32_t> by_worker;            // `keep` stably sorted by worker
  std::vector<int32_t> worker_first, worker_cnt;
  std::vector<int32_t> unit_sub, unit_head, unit_worker;
  std::vector<int64_t> ustart, uend, lane_cuts, cuts;
  std::vector<int32_t> items, lane_off, item_group;
  std::vector<int32_t> tiles, entries, segments, entry_group;
  std::vector<int32_t> tile_order;
  std::vector<int64_t> cnt_s, cnt_d, base, ctr;
};

}  // namespace

extern "C" int va_plan_decode(const VaPlanParams* params, int32_t num_subs, const int32_t* sub_worker,
                              const int32_t* sub_loc, const int32_t* sub_len, const int32_t* sub_page_off,
                              const int32_t* sub_tok0, const int32_t* sub_key, const int32_t* pages,
                              int32_t num_pages, int32_t* blob, int64_t blob_words, VaPlanLayout* layout) {
  if (params == nullptr || layout == nullptr || num_subs < 0 || num_pages < 0) return VA_ERR_BAD_ARG;
  if (num_subs > 0 && (!sub_worker || !sub_loc || !sub_len || !sub_page_off || !sub_tok0 || !sub_key))
    return VA_ERR_BAD_ARG;
  if (num_pages > 0 && pages == nullptr) return VA_ERR_BAD_ARG;
  const VaPlanParams& p = *params;
  const int W = p.num_workers, H = p.num_kv_heads;
  if (W <= 0 || H <= 0 || p.readers_per_tile <= 0 || p.num_sms <= 0 || p.lane_width <= 0) return VA_ERR_BAD_ARG;
  for (int i = 0; i < num_subs; ++i)
    if (sub_worker[i] < 0 || sub_worker[i] >= W || sub_len[i] < 0) return VA_ERR_BAD_ARG;

  static thread_local Scratch tls_scratch;  // vectors keep their capacity between steps
  Scratch& s = tls_scratch;
  const int n_sms = p.num_sms;
  const int per_tile = p.readers_per_tile;

  // ---- which sub-requests go to dense tiles: blocks read by several workers this step
  s.grouped.assign(num_subs, 0);
  s.units.clear();
  const bool allow_groups = p.fixed_stream_lanes <= 0 || p.fixed_dense_sms > 0;
  bool any_grouped = false;
  if (allow_groups && p.group_min_readers > 0 && num_subs > 0) {
    s.sorted_keys.clear();
    for (int i = 0; i < num_subs; ++i)
      if (sub_key[i] >= 0) s.sorted_keys.push_back(sub_key[i]);
    std::sort(s.sorted_keys.begin(), s.sorted_keys.end());
    for (int i = 0; i < num_subs; ++i) {
      if (sub_key[i] < 0) continue;
      auto range = std::equal_range(s.sorted_keys.begin(), s.sorted_keys.end(), sub_key[i]);
      const int64_t readers = range.second - range.first;
      if (readers >= p.group_min_readers && sub_len[i] >= p.group_min_keys) {
        s.grouped[i] = 1;
        any_grouped = true;
      }
    }
    if (any_grouped) {
      // one unit per distinct block, in ascending key order; its readers in input order
      s.by_worker.clear();
      for (int i = 0; i < num_subs; ++i)
        if (s.grouped[i]) s.by_worker.push_back(i);
      std::stable_sort(s.by_worker.begin(), s.by_worker.end(),
                       [&](int32_t a, int32_t b) { return sub_key[a] < sub_key[b]; });
      for (int32_t i : s.by_worker) {
        if (s.units.empty() || s.units.back().key != sub_key[i]) {
          s.units.emplace_back();
          s.units.back().key = sub_key[i];
        }
        s.units.back().readers.push_back(i);
      }
    }
  }

  // ---- split of the SMs between the two kernels by modelled cost
  s.keep.clear();
  int64_t stream_keys = 0;
  for (int i = 0; i < num_subs; ++i)
    if (!s.grouped[i]) {
      s.keep.push_back(i);
      stream_keys += sub_len[i];
    }
  int dense_sms = 0;
  int64_t n_rows_units = 0;  // (reader group, kv head) tile rows
  if (any_grouped) {
    const double stream_cost = static_cast<double>(stream_keys) * H / p.stream_rate;
    double dense_cost = 0.0;
    for (const DenseUnit& u : s.units) {
      const int64_t rows = ceil_div(static_cast<int64_t>(u.readers.size()), per_tile);
      dense_cost += static_cast<double>(sub_len[u.readers[0]]) * H * rows;
      n_rows_units += rows * H;
    }
    dense_cost /= p.dense_rate;
    const double share = dense_cost / std::max(dense_cost + stream_cost, 1e-9);
    dense_sms = static_cast<int>(std::nearbyint(n_sms * share));  // ties to even
    dense_sms = stream_cost > 0 ? std::min(std::max(dense_sms, 1), n_sms - 1) : n_sms;
    // whole rounds: the tile count (units x chunks) is a multiple of the CTA count
    if (n_rows_units <= dense_sms) {
      const int64_t n = n_rows_units;
      int64_t d = std::max<int64_t>(1, static_cast<int64_t>(std::nearbyint(static_cast<double>(dense_sms) / n))) * n;
      d = std::min<int64_t>(d, (n_sms - 1) / n * n);
      dense_sms = static_cast<int>(d != 0 ? d : n);
    }
  }
  const int stream_sms = s.keep.empty() ? 0 : n_sms - dense_sms;
  int G = std::max(stream_sms, 1) * p.lane_width;
  if (p.fixed_stream_lanes > 0) {
    G = p.fixed_stream_lanes;
    if (any_grouped) dense_sms = p.fixed_dense_sms;
  }

  // ---- streaming items: units ordered (worker, kv head, sub-request), cut at unit boundaries and
  // at multiples of the per-lane quota
  const int n_keep = static_cast<int>(s.keep.size());
  s.items.clear();
  s.item_group.clear();
  s.lane_off.assign(G + 1, 0);
  int64_t quota = 0, total = 0;
  if (n_keep > 0) {
    s.by_worker = s.keep;
    std::stable_sort(s.by_worker.begin(), s.by_worker.end(),
                     [&](int32_t a, int32_t b) { return sub_worker[a] < sub_worker[b]; });
    s.worker_cnt.assign(W, 0);
    for (int32_t i : s.keep) s.worker_cnt[sub_worker[i]]++;
    s.worker_first.assign(W, 0);
    for (int w = 1; w < W; ++w) s.worker_first[w] = s.worker_first[w - 1] + s.worker_cnt[w - 1];
    const int64_t n_units = static_cast<int64_t>(n_keep) * H;
    s.unit_sub.clear();
    s.unit_head.clear();
    s.unit_worker.clear();
    s.ustart.clear();
    s.uend.clear();
    s.unit_sub.reserve(n_units);
    for (int w = 0; w < W; ++w)
      for (int h = 0; h < H; ++h)
        for (int j = 0; j < s.worker_cnt[w]; ++j) {
          const int32_t sub = s.by_worker[s.worker_first[w] + j];
          s.unit_sub.push_back(sub);
          s.unit_head.push_back(h);
          s.unit_worker.push_back(w);
          s.ustart.push_back(total);
          total += sub_len[sub];
          s.uend.push_back(total);
        }
    // Lane cuts that even out the lanes' TIME, not their keys.  A lane streams its keys in stages of
    // 16 and pays about one stage more per item (query staging, the partial's write-out), so its cost
    // is sum over its items of ceil(keys / 16) + 1.  With equal key quotas a lane that contains a unit
    // boundary ran 1-3 stages longer than one that does not (cuts close to a boundary snap onto it):
    // on the shared-prefix decode configuration the last lane ended 3.5 us after the median lane, now
    // 2 us (the step gained 0.7 us: the memory system, not a lane's own pace, sets most of the time).  Here the smallest budget T
    // (in stages) is found for which a greedy walk needs at most G lanes; an item is never shorter
    // than cut_slack_keys unless it is a whole unit.
    const int64_t piece_min = std::max<int64_t>(16, p.cut_slack_keys);
    auto walk = [&](int64_t T, std::vector<int64_t>* cuts) -> int64_t {
      int64_t lanes = 0, pos = 0, u = 0;
      while (pos < total) {
        ++lanes;
        int64_t budget = T;
        bool empty = true;
        while (pos < total) {
          while (s.uend[u] <= pos) ++u;
          const int64_t rem = s.uend[u] - pos;
          const int64_t avail = budget - 1;                 // stages left for keys once the item is paid for
          const int64_t need = ceil_div(rem, 16);
          if (need <= avail) {                              // the rest of the unit fits
            pos = s.uend[u];
            budget -= need + 1;
            empty = false;
            continue;
          }
          int64_t take = std::max<int64_t>(avail, 0) * 16;  // keys of this unit the lane can still afford
          if (empty) {
            take = std::max(take, std::min(piece_min, rem));        // an empty lane always advances
            if (rem - take < piece_min) take = rem;
          } else {
            if (rem - take < piece_min) take = (rem - piece_min) / 16 * 16;   // leave no sliver behind
            if (take < piece_min) take = 0;                                  // and start none
          }
          pos += take;
          break;
        }
        if (cuts != nullptr && pos < total) cuts->push_back(pos);
      }
      return lanes;
    };
    const int64_t lanes_cap = std::max(G, 1);
    int64_t T = std::max<int64_t>(ceil_div(ceil_div(total, 16) + n_units, lanes_cap), ceil_div(p.min_item_keys, 16) + 1);
    while (walk(T, nullptr) > lanes_cap) ++T;
    quota = T * 16;
    s.lane_cuts.clear();
    walk(T, &s.lane_cuts);
    s.cuts.resize(s.ustart.size() + s.lane_cuts.size());
    std::merge(s.ustart.begin(), s.ustart.end(), s.lane_cuts.begin(), s.lane_cuts.end(), s.cuts.begin());
    s.cuts.push_back(total);
    s.cuts.erase(std::unique(s.cuts.begin(), s.cuts.end()), s.cuts.end());
    const int n_items = static_cast<int>(s.cuts.size()) - 1;
    s.items.assign(static_cast<size_t>(n_items) * VA_ITEM_WORDS, 0);
    s.item_group.resize(n_items);
    const int64_t n_lane_cuts = static_cast<int64_t>(s.lane_cuts.size());
    int64_t unit = 0, lane = 0;
    for (int it = 0; it < n_items; ++it) {
      const int64_t begin = s.cuts[it], end = s.cuts[it + 1];
      while (unit + 1 < n_units && s.ustart[unit + 1] <= begin) ++unit;   // last unit starting at or before
      const int32_t sub = s.unit_sub[unit];
      int32_t* item = &s.items[static_cast<size_t>(it) * VA_ITEM_WORDS];
      item[0] = sub_page_off[sub];
      item[1] = static_cast<int32_t>(sub_tok0[sub] + (begin - s.ustart[unit]));
      item[2] = static_cast<int32_t>(end - begin);
      item[3] = sub_worker[sub];
      item[4] = sub_loc[sub];
      item[5] = it;
      item[6] = s.unit_head[unit];
      s.item_group[it] = s.unit_worker[unit] * H + s.unit_head[unit];
      // lane i owns the items that begin in [lane_cuts[i-1], lane_cuts[i])
      while (lane < n_lane_cuts && s.lane_cuts[lane] <= begin) ++lane;
      if (lane + 1 <= G) s.lane_off[lane + 1]++;
    }
    // lane_off[g] = number of items whose lane is < g
    for (int g = 1; g <= G; ++g) s.lane_off[g] += s.lane_off[g - 1];
  }
  const int n_items = static_cast<int>(s.item_group.size());

  // ---- dense tiles (partial mode): readers in groups of per_tile, keys in equal chunks
  s.tiles.clear();
  s.entries.clear();
  s.segments.clear();
  s.entry_group.clear();
  if (!s.units.empty()) {
    const int64_t chunks_wanted =
        std::max<int64_t>(1, (static_cast<int64_t>(dense_sms) * p.dense_tiles_per_cta) / n_rows_units);
    int32_t n_ent = 0, n_seg = 0, n_qkeys = 0;
    for (const DenseUnit& u : s.units) {
      const int32_t first = u.readers[0];
      const int64_t L = sub_len[first];
      const int64_t ck = std::max<int64_t>(128, ceil_div(ceil_div(L, chunks_wanted), 64) * 64);
      const int32_t n_ch = static_cast<int32_t>(ceil_div(L, ck));
      for (int32_t c = 0; c < n_ch; ++c) {
        const int64_t k0 = c * ck;
        const int32_t seg[8] = {sub_page_off[first], static_cast<int32_t>(sub_tok0[first] + k0),
                                static_cast<int32_t>(std::min(ck, L - k0)), 0, -1, 0, 0, 0};
        s.segments.insert(s.segments.end(), seg, seg + 8);
      }
      const int n_readers = static_cast<int>(u.readers.size());
      for (int r0 = 0; r0 < n_readers; r0 += per_tile) {
        const int32_t m = std::min(per_tile, n_readers - r0);
        for (int32_t c = 0; c < n_ch; ++c)
          for (int32_t h = 0; h < H; ++h) {
            // same readers, same kv head, same block: the chunks share their rotated queries
            // (word 7 carries the chunk index as a sort key and is cleared below)
            const int32_t t[8] = {n_ent, m, n_seg + c, 1, h, 1, 1 + n_qkeys + h, c};
            s.tiles.insert(s.tiles.end(), t, t + 8);
            for (int32_t j = 0; j < m; ++j) {
              const int32_t reader = u.readers[r0 + j];
              const int32_t e[4] = {sub_worker[reader], sub_loc[reader], 0, 0};
              s.entries.insert(s.entries.end(), e, e + 4);
              s.entry_group.push_back(sub_worker[reader] * H + h);
            }
            n_ent += m;
          }
        n_qkeys += H;
      }
      n_seg += n_ch;
    }
    // chunk-major tile order: with the CTA count a multiple of the number of (reader group, kv head)
    // units, CTA c's tiles c, c + num_ctas, ... all belong to one unit, so its queries are staged once
    const int n_tiles = static_cast<int>(s.tiles.size() / 8);
    s.tile_order.resize(n_tiles);
    std::iota(s.tile_order.begin(), s.tile_order.end(), 0);
    std::stable_sort(s.tile_order.begin(), s.tile_order.end(), [&](int32_t a, int32_t b) {
      const int32_t* ta = &s.tiles[static_cast<size_t>(a) * 8];
      const int32_t* tb = &s.tiles[static_cast<size_t>(b) * 8];
      return ta[7] != tb[7] ? ta[7] < tb[7] : ta[6] < tb[6];
    });
  }
  const int n_tiles = static_cast<int>(s.tiles.size() / 8);
  const int n_entries = static_cast<int>(s.entries.size() / 4);
  const int n_segments = static_cast<int>(s.segments.size() / 8);

  // ---- partial slots: contiguous per (worker, kv head): streamed items first, then tile entries
  const int n_groups = W * H;
  s.cnt_s.assign(n_groups, 0);
  s.cnt_d.assign(n_groups, 0);
  for (int32_t g : s.item_group) s.cnt_s[g]++;
  for (int32_t g : s.entry_group) s.cnt_d[g]++;
  s.base.assign(n_groups + 1, 0);
  for (int g = 0; g < n_groups; ++g) s.base[g + 1] = s.base[g] + s.cnt_s[g] + s.cnt_d[g];
  s.ctr.assign(n_groups, 0);
  for (int it = 0; it < n_items; ++it) {
    const int32_t g = s.item_group[it];
    s.items[static_cast<size_t>(it) * VA_ITEM_WORDS + 5] = static_cast<int32_t>(s.base[g] + s.ctr[g]++);
  }
  for (int e = 0; e < n_entries; ++e) {
    const int32_t g = s.entry_group[e];
    s.entries[static_cast<size_t>(e) * 4 + 2] = static_cast<int32_t>(s.base[g] + s.ctr[g]++);
  }

  // ---- layout
  VaPlanLayout& L = *layout;
  std::memset(&L, 0, sizeof(L));
  int64_t off = 0;
  auto section = [&](int64_t words) {
    const int64_t at = off;
    off += align4(words);
    return static_cast<int32_t>(at);
  };
  L.off_pages = section(num_pages);
  L.num_pages = num_pages;
  L.off_items = section(static_cast<int64_t>(n_items) * VA_ITEM_WORDS);
  L.num_items = n_items;
  L.off_lane_off = section(G + 1);
  L.num_lanes = G;
  L.off_row_part_off = section(n_groups + 1);
  L.num_groups = n_groups;
  L.off_tiles = section(static_cast<int64_t>(n_tiles) * 8);
  L.num_tiles = n_tiles;
  L.off_entries = section(static_cast<int64_t>(n_entries) * 4);
  L.num_entries = n_entries;
  L.off_segments = section(static_cast<int64_t>(n_segments) * 8);
  L.num_segments = n_segments;
  L.total_words = std::max<int64_t>(off, 4);
  L.num_partials = static_cast<int32_t>(s.base[n_groups]);
  L.dense_sms = n_tiles > 0 ? dense_sms : 0;
  L.quota = quota;
  L.total_keys = total;
  if (blob == nullptr || blob_words < L.total_words) return VA_ERR_CAPACITY;

  if (num_pages > 0) std::memcpy(blob + L.off_pages, pages, sizeof(int32_t) * num_pages);
  if (n_items > 0) std::memcpy(blob + L.off_items, s.items.data(), sizeof(int32_t) * s.items.size());
  std::memcpy(blob + L.off_lane_off, s.lane_off.data(), sizeof(int32_t) * (G + 1));
  for (int g = 0; g <= n_groups; ++g) blob[L.off_row_part_off + g] = static_cast<int32_t>(s.base[g]);
  for (int t = 0; t < n_tiles; ++t) {
    int32_t* dst = blob + L.off_tiles + static_cast<int64_t>(t) * 8;
    std::memcpy(dst, &s.tiles[static_cast<size_t>(s.tile_order[t]) * 8], sizeof(int32_t) * 8);
    dst[7] = 0;
  }
  if (n_entries > 0) std::memcpy(blob + L.off_entries, s.entries.data(), sizeof(int32_t) * s.entries.size());
  if (n_segments > 0) std::memcpy(blob + L.off_segments, s.segments.data(), sizeof(int32_t) * s.segments.size());
  return VA_OK;
}

// The same step given as views: expands (worker, block of its view) into sub-requests with the
// reference's rules (shared_cache/attention.py:282-368) and schedules them with va_plan_decode.
extern "C" int va_plan_views(const VaPlanParams* params, const VaViewStep* step, int32_t* blob,
                             int64_t blob_words, VaPlanLayout* layout, int32_t* sub_out, int64_t sub_stride,
                             VaViewSubs* subs_info) {
  if (params == nullptr || step == nullptr || layout == nullptr || subs_info == nullptr) return VA_ERR_BAD_ARG;
  const VaViewStep& v = *step;
  const int W = v.num_workers, nb = v.num_blocks, n_aux = v.num_aux;
  if (W <= 0 || W != params->num_workers || nb < 0 || n_aux < 0 || v.page_size <= 0 || v.view_start == nullptr)
    return VA_ERR_BAD_ARG;
  const int n_view = v.view_start[W];
  if (n_view < 0 || v.view_start[0] != 0) return VA_ERR_BAD_ARG;
  if (nb > 0 && (!v.block_len || !v.block_span || !v.block_pages)) return VA_ERR_BAD_ARG;
  if (n_view > 0 && (!v.view_block || nb == 0)) return VA_ERR_BAD_ARG;
  if (n_aux > 0 && (!v.aux_worker || !v.aux_loc || !v.aux_slot)) return VA_ERR_BAD_ARG;
  const int64_t cap_subs = static_cast<int64_t>(n_view) + n_aux;
  if (sub_out != nullptr && sub_stride < cap_subs) return VA_ERR_CAPACITY;

  struct ViewScratch {
    std::vector<int32_t> w, loc, slot, len, blk, poff, tok0, key, n_seg, pages, page_off;
  };
  static thread_local ViewScratch tls_views;
  ViewScratch& s = tls_views;
  // page runs of the blocks, a page allocated for this step's token appended to its block's run
  s.page_off.assign(nb + 1, 0);
  s.pages.clear();
  {
    int64_t src = 0;
    for (int b = 0; b < nb; ++b) {
      const int32_t n = v.block_pages[b];
      if (n < 0 || (n > 0 && v.pages == nullptr)) return VA_ERR_BAD_ARG;
      s.pages.insert(s.pages.end(), v.pages + src, v.pages + src + n);
      src += n;
      if (v.block_pending_page != nullptr && v.block_pending_page[b] >= 0) s.pages.push_back(v.block_pending_page[b]);
      s.page_off[b + 1] = static_cast<int32_t>(s.pages.size());
    }
  }
  const int n_paged_pages = static_cast<int>(s.pages.size());
  for (auto* vec : {&s.w, &s.loc, &s.slot, &s.len, &s.blk, &s.poff, &s.tok0, &s.key}) {
    vec->clear();
    vec->reserve(cap_subs);
  }
  s.n_seg.assign(W, 0);
  for (int w = 0; w < W; ++w) {
    const int b0 = v.view_start[w], b1 = v.view_start[w + 1];
    if (b0 > b1 || b1 > n_view) return VA_ERR_BAD_ARG;
    int64_t span_left = 0;
    for (int i = b0; i < b1; ++i) {
      if (v.view_block[i] < 0 || v.view_block[i] >= nb) return VA_ERR_BAD_ARG;
      span_left += v.block_span[v.view_block[i]];
    }
    int seg = 0;
    for (int i = b0; i < b1; ++i) {
      const int32_t b = v.view_block[i];
      if (v.block_len[b] > 0) {   // empty blocks are skipped
        s.w.push_back(w);
        s.loc.push_back(static_cast<int32_t>(span_left - 1));
        s.slot.push_back(seg++);
        s.len.push_back(v.block_len[b]);
        s.blk.push_back(b);
        s.poff.push_back(s.page_off[b]);
        s.tok0.push_back(0);
        s.key.push_back(s.page_off[b]);   // the page-run offset names the block
      }
      span_left -= v.block_span[b];
    }
    s.n_seg[w] = seg;
  }
  const int n_main = static_cast<int>(s.w.size());
  // a worker whose write block is outside its view: one key at its new slot
  s.pages.resize(static_cast<size_t>(n_paged_pages) + n_aux);
  for (int j = 0; j < n_aux; ++j) {
    const int32_t w = v.aux_worker[j];
    if (w < 0 || w >= W || v.aux_slot[j] < 0) return VA_ERR_BAD_ARG;
    s.w.push_back(w);
    s.loc.push_back(v.aux_loc[j]);
    s.slot.push_back(s.n_seg[w]++);
    s.len.push_back(1);
    s.blk.push_back(-1);
    s.poff.push_back(n_paged_pages + j);
    s.tok0.push_back(static_cast<int32_t>(v.aux_slot[j] % v.page_size));
    s.key.push_back(-1);
    s.pages[static_cast<size_t>(n_paged_pages) + j] = static_cast<int32_t>(v.aux_slot[j] / v.page_size);
  }
  const int n_sub = static_cast<int>(s.w.size());
  subs_info->num_main = n_main;
  subs_info->num_aux = n_aux;
  subs_info->max_segments = *std::max_element(s.n_seg.begin(), s.n_seg.end());
  if (sub_out != nullptr && n_sub > 0) {
    const std::vector<int32_t>* rows[5] = {&s.w, &s.loc, &s.slot, &s.len, &s.blk};
    for (int r = 0; r < 5; ++r) std::memcpy(sub_out + r * sub_stride, rows[r]->data(), sizeof(int32_t) * n_sub);
  }
  return va_plan_decode(params, n_sub, s.w.data(), s.loc.data(), s.len.data(), s.poff.data(), s.tok0.data(),
                        s.key.data(), s.pages.data(), static_cast<int32_t>(s.pages.size()), blob, blob_words,
                        layout);
}

// ------------------------------------------------------------------------------------------------
// Tile table of a batched view-conditioned prefill (host code, no CUDA call).
//
// Request r owns output rows [row_offset, row_offset + num_new) and the segment rows
// [seg_begin, seg_begin + seg_count) of `segments` (8 words each: page run, token begin, keys,
// query rotation base, causal base or -1, ...).  Its new tokens are cut into tiles of `per_tile`
// consecutive tokens; every (request, token tile, kv head) is one row of `tiles` (8 words:
// entry_begin, entry_count, seg_begin, seg_count, kv head, 0, 0, 0).  Rows are ordered heaviest
// first (cost = keys the tile walks x its rows; a causal segment is walked up to the last key the
// tile's last row sees; ties keep request / token / head order) and every other round of `num_ctas`
// rows is reversed, so that the CTA that takes rows c, c + num_ctas, ... does not collect the
// heaviest tile of every round.  `entries` gets (row, relative position, 0, 0) per new token.
extern "C" int va_plan_prefill_tiles(const int32_t* segments, int32_t num_segments, const int32_t* requests,
                                     int32_t num_requests, int32_t per_tile, int32_t num_kv_heads,
                                     int32_t max_ctas, int32_t* entries, int32_t num_rows, int32_t* tiles,
                                     int32_t tile_capacity, int32_t* num_tiles_out) {
  if (num_tiles_out == nullptr || segments == nullptr || requests == nullptr || entries == nullptr ||
      tiles == nullptr || num_requests < 0 || num_segments < 0 || per_tile <= 0 || num_kv_heads <= 0 ||
      max_ctas <= 0 || num_rows < 0 || tile_capacity < 0)
    return VA_ERR_BAD_ARG;
  struct Row {
    int64_t cost;
    int32_t entry_begin, entry_count, seg_begin, seg_count, head;
  };
  std::vector<Row> rows;
  for (int r = 0; r < num_requests; ++r) {
    const int32_t* rq = requests + static_cast<int64_t>(r) * 4;
    const int seg_begin = rq[0], seg_count = rq[1], off = rq[2], S = rq[3];
    if (seg_begin < 0 || seg_count < 0 || seg_begin + seg_count > num_segments || off < 0 || S <= 0 ||
        off + S > num_rows)
      return VA_ERR_BAD_ARG;
    for (int i = 0; i < S; ++i) {
      int32_t* e = entries + static_cast<int64_t>(off + i) * 4;
      e[0] = off + i;
      e[1] = i;
      e[2] = 0;
      e[3] = 0;
    }
    int64_t open_keys = 0;
    for (int s = 0; s < seg_count; ++s) {
      const int32_t* sg = segments + static_cast<int64_t>(seg_begin + s) * 8;
      if (sg[4] < 0) open_keys += sg[2];
    }
    for (int e0 = 0; e0 < S; e0 += per_tile) {
      const int cnt = std::min(per_tile, S - e0);
      int64_t keys = open_keys;
      for (int s = 0; s < seg_count; ++s) {
        const int32_t* sg = segments + static_cast<int64_t>(seg_begin + s) * 8;
        if (sg[4] >= 0) keys += std::min<int64_t>(sg[2], static_cast<int64_t>(sg[4]) + e0 + cnt);
      }
      for (int h = 0; h < num_kv_heads; ++h)
        rows.push_back(Row{keys * cnt, off + e0, cnt, seg_begin, seg_count, h});
    }
  }
  const int64_t n = static_cast<int64_t>(rows.size());
  *num_tiles_out = static_cast<int32_t>(n);
  if (n > tile_capacity) return VA_ERR_CAPACITY;
  std::stable_sort(rows.begin(), rows.end(), [](const Row& a, const Row& b) { return a.cost > b.cost; });
  const int64_t n_ctas = std::max<int64_t>(1, std::min<int64_t>(max_ctas, n));
  for (int64_t pos = 0; pos < n; ++pos) {
    int64_t src = pos;
    if (n_ctas > 1) {
      const int64_t rnd = pos / n_ctas, k = pos % n_ctas;
      const int64_t width = std::min<int64_t>(n_ctas, n - rnd * n_ctas);   // the last round may be short
      if (rnd & 1) src = rnd * n_ctas + (width - 1 - k);
    }
    const Row& t = rows[src];
    int32_t* out = tiles + pos * 8;
    out[0] = t.entry_begin;
    out[1] = t.entry_count;
    out[2] = t.seg_begin;
    out[3] = t.seg_count;
    out[4] = t.head;
    out[5] = out[6] = out[7] = 0;
  }
  return VA_OK;
}

// ------------------------------------------------------------------------------------------------
// Address tables of a GDN forward (host code, no CUDA call): see va_gdn_plan_tables in the header.
// tab[row][layer][worker][position]; rows 2..7 use position 0 only.
extern "C" int va_gdn_plan_tables(const int64_t* block_addr, const int64_t* block_conv, const int32_t* chain_idx,
                                  const int32_t* target_idx, const int64_t* write_a_base, int64_t write_a_stride,
                                  const int64_t* write_b_base, int64_t write_b_stride,
                                  const int64_t* conv_write_base, int64_t conv_write_stride, int32_t num_blocks,
                                  int32_t layers, int32_t workers, int32_t depth, int64_t* tab) {
  if (num_blocks < 0 || layers <= 0 || workers < 0 || depth <= 0 || tab == nullptr) return VA_ERR_BAD_ARG;
  if (workers > 0 && (block_addr == nullptr || chain_idx == nullptr || target_idx == nullptr)) return VA_ERR_BAD_ARG;
  const int64_t L = layers, W = workers, Dp = depth;
  const int64_t plane = L * W * Dp;
  std::memset(tab, 0, sizeof(int64_t) * 8 * plane);
  for (int64_t w = 0; w < W; ++w) {
    const int32_t* chain = chain_idx + w * Dp;
    for (int64_t j = 0; j < Dp; ++j)
      if (chain[j] < 0 || chain[j] > num_blocks) return VA_ERR_BAD_ARG;
    const int32_t target = target_idx[w];
    if (target < 0 || target > num_blocks) return VA_ERR_BAD_ARG;
    for (int64_t l = 0; l < L; ++l) {
      int64_t* at = tab + (l * W + w) * Dp;   // [row 0][l][w][0]
      int64_t conv = 0;
      for (int64_t j = 0; j < Dp; ++j) {
        const int64_t* pair = block_addr + (static_cast<int64_t>(chain[j]) * L + l) * 2;
        at[j] = pair[0];
        at[plane + j] = pair[1];
        if (block_conv != nullptr) {
          const int64_t c = block_conv[static_cast<int64_t>(chain[j]) * L + l];
          if (c != 0) conv = c;   // the last block of the chain that has a window
        }
      }
      const int64_t* tp = block_addr + (static_cast<int64_t>(target) * L + l) * 2;
      at[2 * plane] = tp[0];
      at[3 * plane] = tp[1];
      at[4 * plane] = conv;
      if (write_a_base != nullptr) at[5 * plane] = write_a_base[w] + l * write_a_stride;
      if (write_b_base != nullptr) at[6 * plane] = write_b_base[w] + l * write_b_stride;
      if (conv_write_base != nullptr) at[7 * plane] = conv_write_base[w] + l * conv_write_stride;
    }
  }
  return VA_OK;
}
