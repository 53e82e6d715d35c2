// Dense-tile view attention on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
// Same contract as the mma.sync dense kernel (tiles / entries / segments, final rows or split-K
// partials), different engine.  One CTA owns a tile of up to 256 (head_dim 128) or 128
// (head_dim 256) query rows and issues, from one elected lane of a converged warp,
//     S = Qrot . K^T        tcgen05.mma  M=128, N=BN keys, K=head_dim   A, B from shared memory
//     O += P . V            tcgen05.mma  M=128, N=head_dim, K=BN keys   A (= P) from TMEM, B from smem
// with both accumulators in TMEM.  P never touches shared memory: the softmax warps read their S
// row from TMEM and write bf16 P back over the upper half of the S columns, and the PV product
// takes it from there.  The tensor pipe executes one thread's products in issue order, so the next
// S product of a region is simply issued after the PV product that read P from it.
//
// TMEM (512 columns): two S regions of BN fp32 columns at 0 and BN, outputs from column 256.
//   two streams (head_dim 128, tile of more than 128 rows): stream i owns S region i and O_i; issue
//       order S0(j+1) after PV0(j), S1(j+1) after PV1(j): while one stream's softmax warps work the
//       tensor core runs the other stream, and every K/V tile is fetched once for 256 rows;
//   one stream: key tile j uses S region j & 1, S(j+1) is issued BEFORE PV(j) and overlaps the
//       softmax of tile j.
// Shared memory: rotated queries (64 KB), a ring of five 32 KB slots holding K(0) V(0) K(1) V(1)...
// (128 keys at head_dim 128, 64 keys at head_dim 256), barriers.
//
// Warp roles (4 softmax warps per stream, 1 MMA warp, 1 loader warp per ring slot):
//   softmax    thread i of a stream owns TMEM lane i = query row i: pass 1 over its S row for the
//              maximum, LAZY rescale of O (only when the running max grew by > 2^8), pass 2
//              P = exp2(x - m) -> bf16 pairs -> TMEM; final normalisation / partial write.
//   MMA        walks the schedule converged (waits included); the elected lane issues the products
//              and the commits that signal mbarriers.
//   loaders    rotate-and-stage the tile's queries per segment (RoPE delta entry.rel +
//              segment.loc_base); fetch K/V tiles through the page table into 128-byte-swizzled
//              tiles: whole pages as TMA boxes (cp.async.bulk.tensor, one box per page and
//              128-byte panel, completion counted on the slot's mbarrier), ragged pages and
//              zero rows with 16-byte cp.async along rows; the same tile layout is the K-major
//              B operand of S and the MN-major B operand of PV.
//              A ring slot has exactly one producer warp: an mbarrier parity wait may only target
//              the current or the preceding phase.
// Every mbarrier wait is bounded; on expiry the CTA records VA_DEV_WAIT_EXPIRED, all
// roles leave their loops, TMEM is freed and the kernel returns.
#include <cuda.h>

#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "tc05.cuh"
#ifndef VA_TC_WAIT_NS
#define VA_TC_WAIT_NS 1000
#endif

namespace {

using namespace va;

struct TcParams {
  const __nv_bfloat16* k_pool;
  const __nv_bfloat16* v_pool;
  int64_t num_pages;
  int32_t page_size;
  int32_t num_q_heads;
  int32_t num_kv_heads;
  int32_t rotary_dim;
  int32_t max_pos;
  const float* cos_sin;
  float scale_log2;
  const int32_t* page_indices;
  const int32_t* tiles;
  const int32_t* entries;
  const int32_t* segments;
  int32_t num_page_indices;
  int32_t num_tiles;
  int32_t num_entries;
  int32_t num_segments;
  int32_t num_partials;
  int32_t num_rows;
  const __nv_bfloat16* q;
  int64_t q_row_stride;
  __nv_bfloat16* out;
  int64_t out_row_stride;
  float* partial_o;
  float* partial_ml;
  int32_t* status;
  const int32_t* q_pos3;   // [3, num_rows] per-axis rotation positions of the query rows, or null
  int32_t mrope_lim_h, mrope_lim_w;
  // Tensor maps of the K and V pools seen as [num_slots, num_kv_heads * head_dim] bf16 matrices, box
  // = one page of rows x 64 elements, SWIZZLE_128B: one box is one page of one 128-byte panel of a
  // tile.  use_tma = 0: no maps (page size or alignment does not fit), every row is gathered.
  int32_t use_tma;
  alignas(64) CUtensorMap tmap_k;
  alignas(64) CUtensorMap tmap_v;
};

constexpr int kRows = 128;           // query rows per stream (TMEM lanes)
constexpr int kTcPolls = 1 << 18;    // bound of every mbarrier wait
constexpr float kRescaleLog2 = 8.f;  // O is rescaled only when the running max grew by more

template <int D>
struct TcCfg {
  static constexpr int kStreams = D == 128 ? 2 : 1;
  static constexpr int kBN = D == 128 ? 128 : 64;       // keys per tile (a K or V tile is 32 KB)
  static constexpr int kChunks = D / 8;                 // 16-byte chunks per K/V/Q row
  static constexpr int kQBytes = kRows * D * 2;         // per stream
  static constexpr int kTileBytes = kBN * D * 2;        // K or V tile
  static constexpr int kSlots = 5;                      // ring: K(0) V(0) K(1) V(1) ...
  static constexpr int kOffQ = 0;
  static constexpr int kOffRing = kStreams * kQBytes;
  static constexpr int kOffBar = kOffRing + kSlots * kTileBytes;
  static constexpr int kTotalBytes = kOffBar + 256;
  static constexpr int kTmemCols = 512;
  static constexpr int kColS = 0;                       // S region r: columns [r * kBN, (r + 1) * kBN)
  static constexpr int kColO = 256;                     // O of stream i: kColO + i * D
  static constexpr int kSoftmaxWarps = 4 * kStreams;
  static constexpr int kMmaWarp = kSoftmaxWarps;
  static constexpr int kLoaderWarp0 = kSoftmaxWarps + 1;
  static constexpr int kLoaderWarps = kSlots;           // loader warp w fills ring slot w
  // Register reallocation (head_dim 128): a softmax thread keeps its whole 128-value S row in
  // registers, which needs more than the 128 a 512-thread CTA gets at launch; the other warps
  // give registers up (setmaxnreg works on whole warpgroups, so the CTA is padded to 16 warps).
  static constexpr bool kRegRealloc = D == 128;
  static constexpr int kRegsSoftmax = 152;
  static constexpr int kRegsOther = 104;
  static constexpr int kWarps = kRegRealloc ? ((kSoftmaxWarps + 1 + kLoaderWarps + 3) / 4) * 4
                                            : kSoftmaxWarps + 1 + kLoaderWarps;
  static constexpr int kThreads = kWarps * 32;
  static_assert(!kRegRealloc || kSoftmaxWarps * 32 * kRegsSoftmax + (kWarps - kSoftmaxWarps) * 32 * kRegsOther <= 65536,
                "register file");
  static constexpr int kTileRows = kStreams * kRows;    // query rows per CTA tile
  static_assert(2 * kBN <= kColO && kColO + kStreams * D <= kTmemCols, "TMEM column budget");
};

// One box of a tiled tensor map, global -> shared, completion counted in bytes on an mbarrier.
// x (elements of the innermost dimension) times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar,
                                            uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3}], [%4], %5;\n" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}

// barrier slots (8 bytes each) in the barrier area
enum Bar : int {
  kBarQFull = 0, kBarQEmpty = 1, kBarFull = 2, kBarEmpty = 7, kBarSFull = 12, kBarPFull = 14,
  kBarPVDone = 16, kBarOFree = 18, kBarCount = 19
};

// kAxes: the queries carry per-axis (interleaved mRoPE) positions, p.q_pos3; a separate
// instantiation, so that the common path pays nothing for it.
// kTma: whole pages of K/V arrive as TMA boxes (the host has encoded tensor maps of the pools);
// otherwise every row is gathered with cp.async (pages of fewer than 8 rows).
template <int D, bool kAxes, bool kTma>
__global__ void __launch_bounds__(TcCfg<D>::kThreads, 1) view_dense_tc_kernel(const __grid_constant__ TcParams p) {
  using Cfg = TcCfg<D>;
  constexpr int BN = Cfg::kBN;
  constexpr int CH = Cfg::kChunks;
  constexpr int NSLOT = Cfg::kSlots;
  extern __shared__ __align__(1024) unsigned char smem[];
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + Cfg::kOffBar;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kOffBar + kBarCount * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::kOffBar + kBarCount * 8 + 8);
  auto bar = [&](int slot) { return bar_base + slot * 8; };

  if (tid == 0) {
    mbar_init(bar(kBarQFull), Cfg::kLoaderWarps);  // one arrival per loader warp
    mbar_init(bar(kBarQEmpty), 1);
    for (int s = 0; s < NSLOT; ++s) {
      mbar_init(bar(kBarFull + s), 1);     // lane 0 of the loader warp that owns the slot
      mbar_init(bar(kBarEmpty + s), 1);    // commit of the last product that read the slot
    }
    for (int r = 0; r < 2; ++r) {
      mbar_init(bar(kBarSFull + r), 1);
      mbar_init(bar(kBarPFull + r), 4);    // one arrival per softmax warp of the stream
      mbar_init(bar(kBarPVDone + r), 1);
    }
    mbar_init(bar(kBarOFree), Cfg::kSoftmaxWarps);  // every softmax warp, once per CTA tile with keys
    mbar_fence_init();
    *abort_flag = 0;
  }
  if (warp == Cfg::kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(Cfg::kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int gqa = p.num_q_heads / p.num_kv_heads;
  const int P = p.page_size;
  const int64_t slot_stride = static_cast<int64_t>(p.num_kv_heads) * D;

  // Running use counters.  Every role walks the same sequence of tiles, segments and key tiles,
  // so these advance identically in all of them:
  //   ku      K/V ring units filled / consumed so far (unit 2j = K of key tile j, 2j+1 = V)
  //   qn      segments staged so far
  //   ru[r]   S tiles S region r has held so far (parity of its SFull / PFull / PVDone barriers)
  //   tn      CTA tiles with at least one key tile so far (parity of the OFree barrier)
  //   prev_qkey  query key of the tile whose queries are staged (0: none that may be reused)
  uint32_t ku = 0, qn = 0, tn = 0;
  int prev_qkey = 0;
  uint32_t ru[2] = {0u, 0u};
  bool dead = false;
  bool q_release_pending = false;  // MMA warp: the staged queries' QEmpty commit is still owed
  uint32_t last_fill = 0xffffffffu;  // loader warp: ring unit it filled last (none yet)
  // Bounded wait.  A role that gives up raises the CTA-wide abort flag, which every other wait
  // polls, so one expiry takes all roles out of their loops.
  auto wait = [&](int slot, uint32_t parity) -> bool {
    if (dead) return false;
    const uint32_t b = bar(slot);
    for (int i = 0; i < kTcPolls; ++i) {
#if VA_TC_WAIT_NS > 0
      const bool done = mbar_try_wait_hint(b, parity & 1u, VA_TC_WAIT_NS);
#else
      const bool done = mbar_try_wait(b, parity & 1u);
#endif
      if (done) return true;
      if ((i & 63) == 63 && *abort_flag != 0) break;
    }
    dead = true;
    if (*abort_flag == 0) report(p.status, VA_DEV_WAIT_EXPIRED);
    *abort_flag = 1;
    return false;
  };
  // the softmax and MMA warps run warp-collective instructions after their waits: a wait's
  // outcome is made uniform over the warp so that an expiry cannot split a warp around one
  auto wait_warp = [&](int slot, uint32_t parity) -> bool {
    const bool ok = __all_sync(0xffffffffu, wait(slot, parity));
    if (!ok) dead = true;
    return ok;
  };

  // The tile walk is instantiated once per role (0 loader, 1 MMA, 2 softmax) and called from a
  // branch of its own, so that the register reallocation below dominates all of a role's code.
  auto run_tiles = [&](auto role_tag) {
  constexpr int kRole = decltype(role_tag)::value;
  for (int tile_id = blockIdx.x; tile_id < p.num_tiles && !dead; tile_id += gridDim.x) {
    const int32_t* tile = p.tiles + static_cast<int64_t>(tile_id) * 8;
    const int entry_begin = tile[0];
    const int entry_count = tile[1];
    const int seg_begin = tile[2];
    const int seg_count = tile[3];
    const int kvh = tile[4];
    const int mode = tile[5];
    const int q_key = tile[6];       // non-zero: tiles with equal keys have identical rotated queries
    if (entry_count == 0) continue;  // padding tile of a fixed-capacity plan
    if (entry_begin < 0 || entry_count <= 0 || entry_begin + entry_count > p.num_entries ||
        entry_count * gqa > Cfg::kTileRows || seg_begin < 0 || seg_count < 0 ||
        seg_begin + seg_count > p.num_segments || kvh < 0 || kvh >= p.num_kv_heads) {
      if (tid == 0) report(p.status, VA_DEV_BAD_ROW);
      continue;
    }
    const int n_streams = entry_count * gqa > kRows ? 2 : 1;  // streams with at least one row
    const bool two = n_streams == 2;
    // largest `rel` of the tile (entries of a causal tile are consecutive tokens)
    const int rel_max = p.entries[static_cast<int64_t>(entry_begin + entry_count - 1) * 4 + 1];
    auto seg_field = [&](int s, int f) { return p.segments[static_cast<int64_t>(seg_begin + s) * 8 + f]; };
    // keys of segment s this tile has to look at (causal segments stop at the last visible key)
    auto seg_keys = [&](int s) {
      const int n = seg_field(s, 2);
      const int cb = seg_field(s, 4);
      return cb < 0 ? n : min(n, cb + rel_max + 1);
    };
    int total_kt = 0, total_seg = 0;
    for (int s = 0; s < seg_count; ++s) {
      const int n = max(seg_keys(s), 0);
      total_kt += (n + BN - 1) / BN;
      total_seg += n > 0 ? 1 : 0;
    }
    // S region of key tile j of stream i, and how many tiles that region has held before it
    // the previous tile of this CTA staged exactly these queries: they are still in shared memory
    const bool reuse_q = total_kt > 0 && q_key != 0 && q_key == prev_qkey && seg_count == 1;
    auto region_of = [&](int i, int j) { return two ? i : (j & 1); };
    auto use_of = [&](int i, int j) -> uint32_t { return two ? ru[i] + j : ru[j & 1] + (j >> 1); };

    if constexpr (kRole == 0) {
      // =========================================================== loaders
      const int lw = warp - Cfg::kLoaderWarp0;          // loader warp = ring slot it fills
      // the tile's K/V is read again by the CTAs of the other reader groups: keep it in L2
      const uint64_t kv_policy = l2_policy_evict_last();
      const int lt = tid - Cfg::kLoaderWarp0 * 32;      // index among the loader threads
      int j = 0;                                        // key tile of this CTA tile
      uint32_t q_idx = qn;
      for (int s = 0; s < seg_count && !dead; ++s) {
        const int n_keys = seg_keys(s);
        if (n_keys <= 0) continue;
        // ---- queries of this segment, rotated by rel + loc_base
        if (!reuse_q) {
        if (!wait(kBarQEmpty, (q_idx & 1u) ^ 1u)) break;
        {
          const int loc_base = seg_field(s, 3);
          const int half = p.rotary_dim >> 1;
          const int pair_chunks = half >> 3;
          // work item = (entry, pair of chunks c and c + half) for every head of the GQA group:
          // adjacent lanes take adjacent chunks (coalesced reads), the cos/sin values are loaded
          // once per item and the heads' query chunks are fetched four heads at a time.  Rows
          // beyond the tile's entries are not staged: their S rows are fully masked.
          const int pass_chunks = CH - 2 * pair_chunks;   // chunks beyond the rotary part
          const int per_ent = pair_chunks + pass_chunks;
          const int n_items = entry_count * per_ent;
          for (int item = lt; item < n_items; item += Cfg::kLoaderWarps * 32) {
            const int e = item / per_ent;
            const int c = item - e * per_ent;
            const int32_t* ent = p.entries + static_cast<int64_t>(entry_begin + e) * 4;
            const int q_row = ent[0];
            const bool live = q_row >= 0 && q_row < p.num_rows;
            if (!live) report(p.status, VA_DEV_BAD_ROW);
            const __nv_bfloat16* src = p.q + static_cast<int64_t>(live ? q_row : 0) * p.q_row_stride +
                                       static_cast<int64_t>(kvh * gqa) * D;
            const bool rot = c < pair_chunks;
            const int c_lo = rot ? c : 2 * pair_chunks + (c - pair_chunks);   // first chunk of the item
            float cosv[8], sinv[8];
            if (rot && kAxes) {
              // interleaved mRoPE: frequency f takes its position from the axis it belongs to
              const int row_i = live ? q_row : 0;
              const int pos3[3] = {p.q_pos3[row_i] + loc_base,
                                   p.q_pos3[static_cast<int64_t>(p.num_rows) + row_i] + loc_base,
                                   p.q_pos3[2 * static_cast<int64_t>(p.num_rows) + row_i] + loc_base};
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int f = c * 8 + i;
                const int r3 = f % 3;
                const int axis = (r3 == 1 && f < p.mrope_lim_h) ? 1 : ((r3 == 2 && f < p.mrope_lim_w) ? 2 : 0);
                bool neg = false;
                const float* cs = rope_row(p.cos_sin, p.rotary_dim, p.max_pos, pos3[axis], &neg);
                cosv[i] = cs[f];
                sinv[i] = neg ? -cs[half + f] : cs[half + f];
              }
            } else if (rot && !kAxes) {
              bool neg = false;
              const float* cs = rope_row(p.cos_sin, p.rotary_dim, p.max_pos, ent[1] + loc_base, &neg);
              const float4 ca = *reinterpret_cast<const float4*>(cs + c * 8);
              const float4 cb = *reinterpret_cast<const float4*>(cs + c * 8 + 4);
              const float4 sa = *reinterpret_cast<const float4*>(cs + half + c * 8);
              const float4 sb = *reinterpret_cast<const float4*>(cs + half + c * 8 + 4);
              const float sg = neg ? -1.f : 1.f;
              cosv[0] = ca.x; cosv[1] = ca.y; cosv[2] = ca.z; cosv[3] = ca.w;
              cosv[4] = cb.x; cosv[5] = cb.y; cosv[6] = cb.z; cosv[7] = cb.w;
              sinv[0] = sg * sa.x; sinv[1] = sg * sa.y; sinv[2] = sg * sa.z; sinv[3] = sg * sa.w;
              sinv[4] = sg * sb.x; sinv[5] = sg * sb.y; sinv[6] = sg * sb.z; sinv[7] = sg * sb.w;
            }
            constexpr int HB = D == 256 ? 8 : 4;   // heads fetched together (register budget)
            for (int hd0 = 0; hd0 < gqa; hd0 += HB) {
              uint4 lo4[HB], hi4[HB];
#pragma unroll
              for (int u = 0; u < HB; ++u) {
                lo4[u] = make_uint4(0u, 0u, 0u, 0u);
                hi4[u] = make_uint4(0u, 0u, 0u, 0u);
                if (live && hd0 + u < gqa) {
                  const __nv_bfloat16* s = src + static_cast<int64_t>(hd0 + u) * D;
                  lo4[u] = *reinterpret_cast<const uint4*>(s + c_lo * 8);
                  if (rot) hi4[u] = *reinterpret_cast<const uint4*>(s + half + c * 8);
                }
              }
#pragma unroll
              for (int u = 0; u < HB; ++u) {
                if (hd0 + u >= gqa) break;
                const int row = e * gqa + hd0 + u;
                unsigned char* qdst = smem + Cfg::kOffQ + (row / kRows) * Cfg::kQBytes;
                const int lrow = row % kRows;
                if (rot) {
                  uint4 olo, ohi;
                  const __nv_bfloat16* lo = reinterpret_cast<const __nv_bfloat16*>(&lo4[u]);
                  const __nv_bfloat16* hi = reinterpret_cast<const __nv_bfloat16*>(&hi4[u]);
                  __nv_bfloat16* ol = reinterpret_cast<__nv_bfloat16*>(&olo);
                  __nv_bfloat16* oh = reinterpret_cast<__nv_bfloat16*>(&ohi);
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    const float a = __bfloat162float(lo[i]);
                    const float b = __bfloat162float(hi[i]);
                    ol[i] = __float2bfloat16_rn(__fsub_rn(__fmul_rn(cosv[i], a), __fmul_rn(sinv[i], b)));
                    oh[i] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(cosv[i], b), __fmul_rn(sinv[i], a)));
                  }
                  *reinterpret_cast<uint4*>(qdst + sw_off(lrow, c, kRows)) = olo;
                  *reinterpret_cast<uint4*>(qdst + sw_off(lrow, c + pair_chunks, kRows)) = ohi;
                } else {
                  *reinterpret_cast<uint4*>(qdst + sw_off(lrow, c_lo, kRows)) = lo4[u];
                }
              }
            }
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(kBarQFull));
          ++q_idx;
        }
        }
        // ---- K and V tiles of this segment: this warp fills the ring units that map to its slot.
        // Pages that lie wholly inside the segment arrive as TMA boxes (one per page and 128-byte
        // panel, issued by the lane that looked the page up); the ragged last page, the rows past the
        // segment's end (zero-filled) and segments that do not start on a page boundary are
        // gathered row by row with cp.async.
        const int page_off = seg_field(s, 0);
        const int tok_begin = seg_field(s, 1);
        const int n_tiles = (n_keys + BN - 1) / BN;
        const bool seg_tma = kTma && tok_begin % P == 0;
        for (int t = 0; t < n_tiles && !dead; ++t, ++j) {
#pragma unroll 1
          for (int is_v = 0; is_v < 2 && !dead; ++is_v) {
            const uint32_t u = ku + 2u * static_cast<uint32_t>(j) + static_cast<uint32_t>(is_v);
            if (static_cast<int>(u % NSLOT) != lw) continue;
            const uint32_t dst = smem_base + Cfg::kOffRing + lw * Cfg::kTileBytes;
            const __nv_bfloat16* pool = is_v ? p.v_pool : p.k_pool;
            const int tma_pages = seg_tma ? min(BN, n_keys - t * BN) / P : 0;   // at most BN / 8 <= 16
            const int tma_rows = tma_pages * P;
            int my_page = -1;   // page of box `lane`
            if (lane < tma_pages) {
              const int pidx = page_off + (tok_begin + t * BN) / P + lane;
              if (pidx >= 0 && pidx < p.num_page_indices) {
                const int page = __ldg(p.page_indices + pidx);
                if (page >= 0 && page < p.num_pages) my_page = page;
              }
              if (my_page < 0) report(p.status, VA_DEV_BAD_PAGE);
            }
            // gathered tile: physical slot of keys lane, lane+32, ... (-1 past the segment's end),
            // one page-table read per key, shared with the other lanes by shuffle
            int my_slot[BN / 32];
            if constexpr (!kTma) {
#pragma unroll
              for (int i = 0; i < BN / 32; ++i) {
                const int kk = t * BN + i * 32 + lane;
                int slot = -1;
                if (kk < n_keys) {
                  const int tok = tok_begin + kk;
                  const int pg = tok / P;
                  const int pidx = page_off + pg;
                  if (pidx >= 0 && pidx < p.num_page_indices) {
                    const int page = __ldg(p.page_indices + pidx);
                    if (page >= 0 && page < p.num_pages) slot = page * P + (tok - pg * P);
                  }
                  if (slot < 0) report(p.status, VA_DEV_BAD_PAGE);
                }
                my_slot[i] = slot;
              }
            }
            // the page-table reads above are in flight while the slot is still being consumed
            if (!wait(kBarEmpty + lw, ((u / NSLOT) & 1u) ^ 1u)) break;
            // lanes run along a key's row (512 contiguous bytes per warp-wide copy: one row at
            // head_dim 256, two at 128)
            constexpr int kRowsPerCopy = 512 / (D * 2);
            constexpr int kLanesPerRow = 32 / kRowsPerCopy;
            const int chunk = lane % kLanesPerRow;
            const int sub = lane / kLanesPerRow;
            if constexpr (!kTma) {
#pragma unroll
              for (int it = 0; it < BN / kRowsPerCopy; ++it) {
                const int key = it * kRowsPerCopy + sub;
                const int slot = __shfl_sync(0xffffffffu, my_slot[(it * kRowsPerCopy) >> 5], key & 31);
                const int64_t row_off = static_cast<int64_t>(slot < 0 ? 0 : slot) * slot_stride +
                                        static_cast<int64_t>(kvh) * D;
                cp_async16_hint(dst + sw_off(key, chunk, BN), pool + row_off + chunk * 8, slot < 0 ? 0 : 16, kv_policy);
              }
            } else {
              const bool mine = lane < tma_pages && my_page >= 0;
              const uint32_t boxes = __popc(__ballot_sync(0xffffffffu, mine));
              if (lane == 0) mbar_expect_tx(bar(kBarFull + lw), boxes * static_cast<uint32_t>(P * D * 2));
              __syncwarp();
              if (mine) {
                const CUtensorMap* map = is_v ? &p.tmap_v : &p.tmap_k;
#pragma unroll
                for (int pn = 0; pn < D / 64; ++pn)
                  tma_load_2d(dst + pn * (BN * 128) + lane * (P * 128), map, kvh * D + pn * 64, my_page * P,
                              bar(kBarFull + lw), kv_policy);
              }
              // rows after the boxes: the segment's ragged last page, then zero rows
#pragma unroll 1
              for (int key = tma_rows + sub; key < BN; key += kRowsPerCopy) {
                const int kk = t * BN + key;
                int slot = -1;
                if (kk < n_keys) {
                  const int tok = tok_begin + kk;
                  const int pg = tok / P;
                  const int pidx = page_off + pg;
                  if (pidx >= 0 && pidx < p.num_page_indices) {
                    const int page = __ldg(p.page_indices + pidx);
                    if (page >= 0 && page < p.num_pages) slot = page * P + (tok - pg * P);
                  }
                  if (slot < 0) report(p.status, VA_DEV_BAD_PAGE);
                }
                const int64_t row_off = static_cast<int64_t>(slot < 0 ? 0 : slot) * slot_stride +
                                        static_cast<int64_t>(kvh) * D;
                cp_async16_hint(dst + sw_off(key, chunk, BN), pool + row_off + chunk * 8, slot < 0 ? 0 : 16, kv_policy);
              }
            }
            if (tma_rows < BN) {
              cp_async_commit();
              cp_async_wait<0>();  // this lane's part of the tile has landed
              fence_proxy_async();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kBarFull + lw));
            last_fill = u;
          }
        }
      }
      cp_async_wait<0>();
    } else if constexpr (kRole == 1) {
      // =========================================================== MMA issuer
      // the whole warp walks the schedule (waits included); one elected lane issues
      {
        const uint32_t elected = elect_one();
        const uint32_t idesc_s = instr_desc(BN, false);
        const uint32_t idesc_pv = instr_desc(D, true);
        // base descriptors (every buffer stays below the 256 KB the 14-bit address field covers,
        // so adding to the field never carries out of it)
        const uint64_t q_desc0 = smem_desc(smem_base + Cfg::kOffQ, 16, 1024);
        const uint64_t k_desc0 = smem_desc(smem_base + Cfg::kOffRing, 16, 1024);         // K-major view of slot 0
        const uint64_t v_desc0 = smem_desc(smem_base + Cfg::kOffRing, BN * 128, 1024);   // MN-major view of slot 0
        // segment walk of the S products (advanced by stream 0, read by the last stream)
        int seg_cur = 0, t_in_seg = 0, n_tiles_cur = 0;
        while (seg_cur < seg_count && seg_keys(seg_cur) <= 0) ++seg_cur;
        if (seg_cur < seg_count) n_tiles_cur = (seg_keys(seg_cur) + BN - 1) / BN;
        uint32_t q_idx = qn;
        bool cur_last = false;  // key tile being issued is the last of its segment
        bool cur_more = false;  // ... and another segment of this tile follows it
        bool ok = true;
        // The query buffer is released (QEmpty) once per staging: right after the last S product
        // of a segment when another segment follows, otherwise at the start of the next tile
        // that stages new queries (a tile that reuses them must find them untouched).
        if (total_kt > 0 && !reuse_q && q_release_pending) {
          umma_commit(elected, bar(kBarQEmpty));
          q_release_pending = false;
        }
        // S product of stream i for key tile j: Q_i . K(j)^T into its S region
        auto issue_s = [&](int i, int j) -> bool {
          const uint32_t u = ku + 2u * static_cast<uint32_t>(j);
          const int slot = static_cast<int>(u % NSLOT);
          if (i == 0) {
            if (t_in_seg == 0 && !reuse_q) {  // new segment: its queries must be staged
              if (!wait_warp(kBarQFull, q_idx & 1u)) return false;
              ++q_idx;
            }
            if (!wait_warp(kBarFull + slot, (u / NSLOT) & 1u)) return false;
            cur_last = t_in_seg + 1 >= n_tiles_cur;
            if (cur_last) {
              t_in_seg = 0;
              ++seg_cur;
              while (seg_cur < seg_count && seg_keys(seg_cur) <= 0) ++seg_cur;
              if (seg_cur < seg_count) n_tiles_cur = (seg_keys(seg_cur) + BN - 1) / BN;
              cur_more = seg_cur < seg_count;
            } else {
              ++t_in_seg;
            }
          }
          tc_fence_after();
          const uint64_t qd = q_desc0 + static_cast<uint64_t>(i * (Cfg::kQBytes >> 4));
          const uint64_t kd = k_desc0 + static_cast<uint64_t>(slot * (Cfg::kTileBytes >> 4));
          const int r = region_of(i, j);
          const uint32_t d_tmem = tmem_base + Cfg::kColS + r * BN;
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {  // panel ks / 4, 32 bytes per step inside it
            umma(elected, d_tmem, qd + static_cast<uint64_t>((ks >> 2) * (kRows * 8) + (ks & 3) * 2),
                 kd + static_cast<uint64_t>((ks >> 2) * (BN * 8) + (ks & 3) * 2), idesc_s, ks > 0);
          }
          umma_commit(elected, bar(kBarSFull + r));
          if (i == n_streams - 1) {
            umma_commit(elected, bar(kBarEmpty + slot));          // K(j) has been read by every stream
            if (cur_last) {  // and the segment's queries too
              if (cur_more) umma_commit(elected, bar(kBarQEmpty));
              else q_release_pending = true;
            }
          }
          return true;
        };
        // PV product of stream i for key tile j: O_i += P . V(j), P read from the S region
        auto issue_pv = [&](int i, int j) -> bool {
          const uint32_t u = ku + 2u * static_cast<uint32_t>(j) + 1u;
          const int slot = static_cast<int>(u % NSLOT);
          const int r = region_of(i, j);
          if (!wait_warp(kBarPFull + r, use_of(i, j) & 1u)) return false;
          if (i == 0 && !wait_warp(kBarFull + slot, (u / NSLOT) & 1u)) return false;
          tc_fence_after();
          const uint64_t vd = v_desc0 + static_cast<uint64_t>(slot * (Cfg::kTileBytes >> 4));
          const uint32_t a_tmem = tmem_base + Cfg::kColS + r * BN + BN / 2;   // P: upper half of the region
          const uint32_t d_tmem = tmem_base + Cfg::kColO + i * D;
#pragma unroll
          for (int ks = 0; ks < BN / 16; ++ks) {
            umma_ts(elected, d_tmem, a_tmem + ks * 8, vd + static_cast<uint64_t>(ks * 128), idesc_pv,
                    j > 0 || ks > 0);
          }
          umma_commit(elected, bar(kBarPVDone + r));
          if (i == n_streams - 1) umma_commit(elected, bar(kBarEmpty + slot));  // V(j) has been read
          return true;
        };
        // The first S products of a tile only need the S regions, which the previous tile's last PV
        // products have released; its first PV product overwrites O and waits until the softmax
        // warps have read the previous tile's output out of TMEM.
        auto o_free = [&]() -> bool { return tn == 0 || wait_warp(kBarOFree, (tn - 1) & 1u); };
        if (total_kt > 0) {
          if (two) {
            // S0(0) S1(0) | PV0(j) S0(j+1) PV1(j) S1(j+1) ...
            ok = issue_s(0, 0) && issue_s(1, 0) && o_free();
            for (int j = 0; j < total_kt && ok; ++j) {
              ok = issue_pv(0, j);
              if (ok && j + 1 < total_kt) ok = issue_s(0, j + 1);
              if (ok) ok = issue_pv(1, j);
              if (ok && j + 1 < total_kt) ok = issue_s(1, j + 1);
            }
          } else {
            // S(0) | S(j+1) PV(j) ...   (S regions alternate, so S(j+1) overlaps the softmax of j)
            ok = issue_s(0, 0);
            for (int j = 0; j < total_kt && ok; ++j) {
              if (j + 1 < total_kt) ok = issue_s(0, j + 1);
              if (ok && j == 0) ok = o_free();
              if (ok) ok = issue_pv(0, j);
            }
          }
        }
      }
      dead = __any_sync(0xffffffffu, dead);
    } else {
      // =========================================================== softmax (thread = query row)
      const int i_s = warp >> 2;                   // stream of this warp
      if (i_s < n_streams) {
        const int row = i_s * kRows + (tid & 127);  // row of the CTA tile
        const int e = row / gqa;
        const int hd = row - e * gqa;
        const bool live = e < entry_count;
        int rel = 0;
        if (live) rel = p.entries[static_cast<int64_t>(entry_begin + e) * 4 + 1];
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        const uint32_t o_addr = lane_addr + Cfg::kColO + i_s * D;
        float m_used = -INFINITY;  // offset the exponentials of this row are taken against
        float l_run = 0.f;
        int j = 0;  // key tiles of this CTA tile done so far
        for (int s = 0; s < seg_count && !dead; ++s) {
          const int n_keys = seg_keys(s);
          if (n_keys <= 0) continue;
          const int cb = seg_field(s, 4);
          const int klim = live ? (cb < 0 ? seg_field(s, 2) : min(seg_field(s, 2), cb + rel + 1)) : 0;
          const int n_tiles = (n_keys + BN - 1) / BN;
          for (int t = 0; t < n_tiles && !dead; ++t, ++j) {
            const int r = region_of(i_s, j);
            const uint32_t use = use_of(i_s, j);
            if (!wait_warp(kBarSFull + r, use & 1u)) break;
            tc_fence_after();
            const uint32_t s_addr = lane_addr + Cfg::kColS + r * BN;
            const int k0 = t * BN;
            const int vis = klim - k0;  // keys of this tile visible to the row: columns [0, vis)
            // ---- maximum of the visible raw dot products, half a row at a time; the second
            // half stays in registers for the exponentials
            constexpr int NH = BN / 64;   // 32-column loads per half row
            uint32_t raw[NH][32];
            float mx = -INFINITY;
            auto load_half = [&](int h) {
#pragma unroll
              for (int c = 0; c < NH; ++c) tmem_ld32_issue(s_addr + (h * NH + c) * 32, raw[c]);
              tmem_ld_wait();
              if (vis < (h + 1) * (BN / 2)) {  // tile edge or causal diagonal: mask the hidden keys
#pragma unroll
                for (int c = 0; c < NH; ++c) {
#pragma unroll
                  for (int i = 0; i < 32; ++i)
                    raw[c][i] = ((h * NH + c) * 32 + i) < vis ? raw[c][i] : 0xff800000u;  // -inf
                }
              }
            };
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              load_half(h);
#pragma unroll
              for (int c = 0; c < NH; ++c) {
#pragma unroll
                for (int i = 0; i < 32; i += 2)
                  mx = max3(mx, __uint_as_float(raw[c][i]), __uint_as_float(raw[c][i + 1]));
              }
            }
            mx *= p.scale_log2;  // the scale is positive: max of scaled = scaled max
            // ---- lazy rescale: move the offset only when the maximum grew a lot
            const bool grow = mx > m_used + kRescaleLog2 || (m_used == -INFINITY && mx > -INFINITY);
            float factor = 1.f;
            if (grow) {
              factor = m_used == -INFINITY ? 0.f : fast_exp2(m_used - mx);
              m_used = mx;
            }
            if (__any_sync(0xffffffffu, grow) && j > 0) {
              // O may only be rescaled after the PV product of the previous key tile has finished
              // (products complete in issue order, so every earlier one has finished too)
              if (!wait_warp(kBarPVDone + region_of(i_s, j - 1), use_of(i_s, j - 1) & 1u)) break;
              tc_fence_after();
#pragma unroll
              for (int c0 = 0; c0 < D; c0 += 32) {
                float v[32];
                tmem_ld32(o_addr + c0, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] *= factor;
                tmem_st32(o_addr + c0, v);
              }
            }
            l_run *= factor;
            // ---- P = exp2(x - m_used) as bf16 pairs in the upper half of the S region (key k in
            // column BN/2 + k/2).  The second half row is still in registers and goes first: its P
            // columns lie over S columns that are no longer needed; then the first half row is
            // read again (its S columns are untouched) and fills the P columns below.
            // Scale-and-offset and the row sum run as packed two-float instructions.
            const float neg_off = m_used == -INFINITY ? 0.f : -m_used;
            const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2);
            const uint64_t off2 = pack_f32x2(neg_off, neg_off);
            uint64_t rs2 = pack_f32x2(0.f, 0.f);
            const uint32_t p_addr = s_addr + BN / 2;
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              const int h = 1 - hh;
              if (h == 0) load_half(0);
#pragma unroll
              for (int c = 0; c < NH; ++c) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                  const uint64_t x2 = fma_f32x2(pack_b32x2(raw[c][i], raw[c][i + 1]), scale2, off2);
                  float a, b;
                  unpack_f32x2(x2, a, b);
                  const float e0 = fast_exp2(a);
                  const float e1 = fast_exp2(b);
                  rs2 = add_f32x2(rs2, pack_f32x2(e0, e1));
                  pk[i >> 1] = pack_bf16(e0, e1);
                }
                tmem_st16_issue(p_addr + (h * NH + c) * 16, pk);
              }
            }
            float rs;
            {
              float a, b;
              unpack_f32x2(rs2, a, b);
              rs = a + b;
            }
            l_run += rs;
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kBarPFull + r));
          }
        }
        // ---- epilogue: wait for the last PV product, then final rows or split-K partials
        if (!dead && total_kt > 0) {
          if (wait_warp(kBarPVDone + region_of(i_s, total_kt - 1), use_of(i_s, total_kt - 1) & 1u)) {
            tc_fence_after();
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            // destination of this row (null = nothing to write); the TMEM loads below are
            // warp-collective, so every lane runs them whether or not it has a row to store
            __nv_bfloat16* dst_final = nullptr;
            float* dst_part = nullptr;
            if (live) {
              const int32_t* ent = p.entries + static_cast<int64_t>(entry_begin + e) * 4;
              if (mode == 0) {
                const int q_row = ent[0];
                if (q_row >= 0 && q_row < p.num_rows)
                  dst_final = p.out + static_cast<int64_t>(q_row) * p.out_row_stride +
                              static_cast<int64_t>(kvh * gqa + hd) * D;
              } else {
                const int part = ent[2];
                if (part >= 0 && part < p.num_partials) {
                  dst_part = p.partial_o + (static_cast<int64_t>(part) * gqa + hd) * D;
                  float* ml = p.partial_ml + (static_cast<int64_t>(part) * gqa + hd) * 2;
                  ml[0] = m_used;
                  ml[1] = l_run;
                } else {
                  report(p.status, VA_DEV_BAD_ROW);
                }
              }
            }
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
              float v[32];
              tmem_ld32(o_addr + c0, v);
              if (dst_final != nullptr) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                  uint4 pk;
                  pk.x = pack_bf16(v[i] * inv, v[i + 1] * inv);
                  pk.y = pack_bf16(v[i + 2] * inv, v[i + 3] * inv);
                  pk.z = pack_bf16(v[i + 4] * inv, v[i + 5] * inv);
                  pk.w = pack_bf16(v[i + 6] * inv, v[i + 7] * inv);
                  *reinterpret_cast<uint4*>(dst_final + c0 + i) = pk;
                }
              }
              if (dst_part != nullptr) {
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                  *reinterpret_cast<float4*>(dst_part + c0 + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
              }
            }
            tc_fence_before();
          }
        } else if (!dead && live && mode == 0) {
          // a tile without any visible key: zero rows
          const int32_t* ent = p.entries + static_cast<int64_t>(entry_begin + e) * 4;
          const int q_row = ent[0];
          if (q_row >= 0 && q_row < p.num_rows) {
            __nv_bfloat16* dst = p.out + static_cast<int64_t>(q_row) * p.out_row_stride +
                                 static_cast<int64_t>(kvh * gqa + hd) * D;
            for (int i = 0; i < D; i += 8) *reinterpret_cast<uint4*>(dst + i) = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      }
      if (total_kt > 0) {  // this warp no longer reads the tile's S and O
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(kBarOFree));
      }
    }
    // every role advances the shared counters the same way
    ku += 2u * static_cast<uint32_t>(total_kt);
    qn += reuse_q ? 0 : total_seg;
    if (total_kt > 0) prev_qkey = seg_count == 1 ? q_key : 0;
    if (two) {
      ru[0] += total_kt;
      ru[1] += total_kt;
    } else {
      ru[0] += (total_kt + 1) >> 1;
      ru[1] += total_kt >> 1;
    }
    tn += total_kt > 0 ? 1u : 0u;
    // No CTA-wide meeting between tiles: the loaders run ahead into the next tile (its queries are
    // staged as soon as the last S product of this tile has read the query buffer), and the MMA
    // warp is held back only by the OFree barrier above.
    if (*abort_flag != 0) dead = true;
  }
  };
  if (warp < Cfg::kSoftmaxWarps) {
    if constexpr (Cfg::kRegRealloc) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(Cfg::kRegsSoftmax));
    run_tiles(std::integral_constant<int, 2>{});
  } else {
    if constexpr (Cfg::kRegRealloc) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(Cfg::kRegsOther));
    if (warp == Cfg::kMmaWarp) {
      run_tiles(std::integral_constant<int, 1>{});
    } else if (warp < Cfg::kLoaderWarp0 + Cfg::kLoaderWarps) {
      run_tiles(std::integral_constant<int, 0>{});
      // no box may still be on its way into shared memory when the CTA exits (only possible after
      // an abort: otherwise the MMA warp has consumed every filled slot)
      if (last_fill != 0xffffffffu)
        mbar_wait_bounded(bar(kBarFull + (warp - Cfg::kLoaderWarp0)), (last_fill / NSLOT) & 1u, kTcPolls);
    }  // padding warps of the last warpgroup have no work
  }

  tc_fence_before();
  __syncthreads();
  if (warp == Cfg::kMmaWarp) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(Cfg::kTmemCols));
  }
}

template <int D>
int launch_tc(const TcParams& p, int num_ctas, cudaStream_t stream) {
  using Cfg = TcCfg<D>;
  auto kernel = p.use_tma != 0
                    ? (p.q_pos3 != nullptr ? view_dense_tc_kernel<D, true, true> : view_dense_tc_kernel<D, false, true>)
                    : (p.q_pos3 != nullptr ? view_dense_tc_kernel<D, true, false> : view_dense_tc_kernel<D, false, false>);
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kTotalBytes);
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  kernel<<<num_ctas, Cfg::kThreads, Cfg::kTotalBytes, stream>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return VA_OK;
}

// cuTensorMapEncodeTiled, looked up through the runtime (no link against the driver library)
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
  static const EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}
// VA_DENSE_TMA=0 in the environment keeps every K/V row on the cp.async gather (for comparisons)
bool tma_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("VA_DENSE_TMA");
    return !(e != nullptr && e[0] == '0');
  }();
  return on && encode_tiled_fn() != nullptr;
}
// pool [num_slots, row_elems] bf16, box = page_size rows x 64 elements, 128-byte swizzle
bool encode_pool_map(CUtensorMap* map, const void* base, int64_t row_elems, int64_t num_slots, int page_size) {
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_elems), static_cast<cuuint64_t>(num_slots)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_elems) * 2};
  const cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(page_size)};
  const cuuint32_t elem_strides[2] = {1u, 1u};
  const CUresult r = encode_tiled_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                                       strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace

// Called by va_view_dense (view_dense.cu) when the plan asks for the tcgen05 engine.
int va_dense_tc_launch(const VaPool* pool, const VaDensePlan* plan, const void* q, int64_t q_row_stride,
                       void* out, int64_t out_row_stride, float* partial_o, float* partial_ml,
                       int32_t* status, cudaStream_t stream) {
  TcParams p;
  p.k_pool = static_cast<const __nv_bfloat16*>(pool->k);
  p.v_pool = static_cast<const __nv_bfloat16*>(pool->v);
  p.num_pages = pool->num_slots / pool->page_size;
  p.page_size = pool->page_size;
  p.num_q_heads = pool->num_q_heads;
  p.num_kv_heads = pool->num_kv_heads;
  p.rotary_dim = pool->rotary_dim;
  p.max_pos = pool->max_pos;
  p.cos_sin = pool->cos_sin;
  p.scale_log2 = pool->sm_scale * va::kLog2e;
  p.page_indices = plan->page_indices;
  p.tiles = plan->tiles;
  p.entries = plan->entries;
  p.segments = plan->segments;
  p.num_page_indices = plan->num_page_indices;
  p.num_tiles = plan->num_tiles;
  p.num_entries = plan->num_entries;
  p.num_segments = plan->num_segments;
  p.num_partials = plan->num_partials;
  p.num_rows = plan->num_rows;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_row_stride = q_row_stride;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_row_stride = out_row_stride;
  p.partial_o = partial_o;
  p.partial_ml = partial_ml;
  p.status = status;
  p.q_pos3 = plan->q_pos3;
  p.mrope_lim_h = plan->mrope_lim_h;
  p.mrope_lim_w = plan->mrope_lim_w;
  p.use_tma = 0;
  {
    // TMA boxes need pages of a multiple of 8 rows (a box must start on a swizzle atom of the
    // tile) that divide the key tile, and 16-byte aligned pools and row strides.
    const int bn = pool->head_dim == 128 ? TcCfg<128>::kBN : TcCfg<256>::kBN;
    const int64_t row_elems = static_cast<int64_t>(pool->num_kv_heads) * pool->head_dim;
    const bool fits = tma_enabled() && (pool->head_dim == 128 || pool->head_dim == 256) && pool->page_size >= 8 &&
                      pool->page_size % 8 == 0 && bn % pool->page_size == 0 && pool->num_slots > 0 &&
                      (reinterpret_cast<uintptr_t>(pool->k) & 15u) == 0 && (reinterpret_cast<uintptr_t>(pool->v) & 15u) == 0;
    if (fits && encode_pool_map(&p.tmap_k, pool->k, row_elems, pool->num_slots, pool->page_size) &&
        encode_pool_map(&p.tmap_v, pool->v, row_elems, pool->num_slots, pool->page_size))
      p.use_tma = 1;
  }
  int sms = va_sm_count();
  if (sms <= 0) return VA_ERR_LAUNCH;
  int ctas = plan->num_ctas > 0 ? plan->num_ctas : sms;
  if (ctas > plan->num_tiles) ctas = plan->num_tiles;
  if (pool->head_dim == 128) return launch_tc<128>(p, ctas, stream);
  if (pool->head_dim == 256) return launch_tc<256>(p, ctas, stream);
  return VA_ERR_UNSUPPORTED;
}
