// View decode for sm_100a: split-K flash decode over the page tables of a cache view.
//
// Replaces the decode branch of SharedCacheAttention.forward
// (shared_cache/attention.py:651-703): the per-(worker, segment) query copies and their RoPE
// delta rotation, the per-segment paged decode, the pad-scatter and the LSE merge.
//
// Work decomposition.  The host planner cuts the step into ITEMS -- a contiguous key range of one
// segment, read by one query row for one kv head -- and deals them out to LANES so that every
// lane streams the same number of keys.  A lane is one warp with its own shared-memory ring:
// warps never synchronise with each other, so one warp's prologue (query load + rotation) and
// epilogue (partial write) overlap the other warps' streaming.  Each item produces one partial
// (unnormalised O, running max, running sum); a second small kernel merges a row's partials.
//
// Tensor-core mapping (mma.sync m16n8k16, bf16 -> fp32).  The GQA group of one kv head (<= 8
// query heads) is the N=8 side, the keys are the M=16 side:
//     S^T[key, qh]  = K[key, :]   . Qrot[qh, :]^T        A = K tile (ldmatrix), B = Q (registers)
//     O^T[dim, qh] += V^T[dim,key] . P^T[key, qh]        A = V tile (ldmatrix.trans), B = P^T
// so no MMA lane is spent on padding rows and the O^T accumulator is D/16*4 registers.
// P^T is produced from the S^T accumulator fragment with two movmatrix transposes.
//
// Memory path.  K/V rows (head_dim bf16 = 256 or 512 B, contiguous per token and head) are
// fetched with 16-byte cp.async into rows padded by 16 B (conflict-free ldmatrix), 16 keys per
// stage, NST stages per warp.  Keys past the end of an item are zero-filled, so a stale pool
// value can never reach the accumulator.
#include "common.cuh"

namespace {

using namespace va;

struct DecodeParams {
  const __nv_bfloat16* k_pool;
  const __nv_bfloat16* v_pool;
  int64_t num_pages;
  int32_t page_size;
  int32_t num_q_heads;
  int32_t num_kv_heads;
  int32_t rotary_dim;
  int32_t max_pos;
  const float* cos_sin;
  float scale_log2;  // sm_scale * log2(e)
  const int32_t* page_indices;
  const int32_t* items;
  const int32_t* lane_off;
  const int32_t* row_part_off;
  int32_t num_items;
  int32_t num_lanes;
  int32_t num_rows;
  int32_t num_partials;
  int32_t num_page_indices;
  int32_t phase_mask;
  const __nv_bfloat16* q;
  int64_t q_row_stride;
  __nv_bfloat16* out;
  int64_t out_row_stride;
  float* partial_o;
  float* partial_ml;
  int32_t* status;
};

template <int D>
struct StreamCfg;
template <>
struct StreamCfg<256> {
  static constexpr int kWarps = 4;
  static constexpr int kStages = 3;
};
template <>
struct StreamCfg<128> {
  static constexpr int kWarps = 6;
  static constexpr int kStages = 4;
};

constexpr int kKeysPerStage = 16;
constexpr int kWaitPolls = 1 << 20;  // bound of every mbarrier wait (each poll may suspend a while)

template <int D>
struct StreamSmem {
  static constexpr int kRowBytes = D * 2 + 16;                       // padded bf16 row
  static constexpr int kBarBytes = 64;                               // per-warp mbarriers
  static constexpr int kQBytes = 8 * kRowBytes;                      // 8 query heads
  static constexpr int kTileBytes = kKeysPerStage * kRowBytes;       // K or V of one stage
  static constexpr int kStageBytes = 2 * kTileBytes;                 // K then V
  static constexpr int kWarpBytes = kBarBytes + kQBytes + StreamCfg<D>::kStages * kStageBytes;
  static constexpr int kTotalBytes = kWarpBytes * StreamCfg<D>::kWarps;
};

// Load one GQA group's queries (gqa <= 8 heads of D bf16), rotate them by `delta` and store
// them as bf16 rows of stride D+8 in shared memory; heads >= gqa are zero.  One warp; every lane
// keeps several independent 16-byte loads in flight.
template <int D>
__device__ __forceinline__ void stage_queries(__nv_bfloat16* qs, const __nv_bfloat16* qsrc, int gqa,
                                              int rotary_dim, const float* cos_sin, int max_pos,
                                              int delta, int lane) {
  constexpr int kRow = D + 8;
  bool neg;
  const float* cs = rope_row(cos_sin, rotary_dim, max_pos, delta, &neg);
  const int half = rotary_dim >> 1;
  for (int i = lane; i < (8 - gqa) * (D / 8); i += 32) {
    const int r = gqa + i / (D / 8);
    const int c = i % (D / 8);
    *reinterpret_cast<uint4*>(qs + r * kRow + c * 8) = make_uint4(0u, 0u, 0u, 0u);
  }
  if (rotary_dim == D) {
    // Full rotary width (the usual case): lane = (row r0, chunk c); a lane's rows r0, r0 + step,
    // ... share the chunk, so cos/sin are loaded once and every query load of the lane is issued
    // before the first is used -- one memory latency for the whole group.
    constexpr int kPairChunks = D / 16;          // 16-byte chunks in one half: 16 or 8 (<= 32)
    constexpr int kStep = 32 / kPairChunks;      // rows covered by one pass of the warp
    constexpr int kPasses = 8 / kStep;           // passes that cover 8 heads
    const int c = lane % kPairChunks;
    const int r0 = lane / kPairChunks;
    const float4 ca = *reinterpret_cast<const float4*>(cs + c * 8);
    const float4 cb = *reinterpret_cast<const float4*>(cs + c * 8 + 4);
    const float4 sa = *reinterpret_cast<const float4*>(cs + half + c * 8);
    const float4 sb = *reinterpret_cast<const float4*>(cs + half + c * 8 + 4);
    uint4 lo4[kPasses], hi4[kPasses];
#pragma unroll
    for (int k = 0; k < kPasses; ++k) {
      const int r = r0 + k * kStep;
      if (r < gqa) {
        lo4[k] = *reinterpret_cast<const uint4*>(qsrc + r * D + c * 8);
        hi4[k] = *reinterpret_cast<const uint4*>(qsrc + r * D + half + c * 8);
      }
    }
    const float sg = neg ? -1.f : 1.f;
    const float cosv[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
    const float sinv[8] = {sg * sa.x, sg * sa.y, sg * sa.z, sg * sa.w, sg * sb.x, sg * sb.y, sg * sb.z, sg * sb.w};
#pragma unroll
    for (int k = 0; k < kPasses; ++k) {
      const int r = r0 + k * kStep;
      if (r < gqa) {
        const __nv_bfloat16* lo = reinterpret_cast<const __nv_bfloat16*>(&lo4[k]);
        const __nv_bfloat16* hi = reinterpret_cast<const __nv_bfloat16*>(&hi4[k]);
        uint4 olo, ohi;
        __nv_bfloat16* ol = reinterpret_cast<__nv_bfloat16*>(&olo);
        __nv_bfloat16* oh = reinterpret_cast<__nv_bfloat16*>(&ohi);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float a = __bfloat162float(lo[e]);
          const float b = __bfloat162float(hi[e]);
          ol[e] = __float2bfloat16_rn(__fsub_rn(__fmul_rn(cosv[e], a), __fmul_rn(sinv[e], b)));
          oh[e] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(cosv[e], b), __fmul_rn(sinv[e], a)));
        }
        *reinterpret_cast<uint4*>(qs + r * kRow + c * 8) = olo;
        *reinterpret_cast<uint4*>(qs + r * kRow + half + c * 8) = ohi;
      }
    }
  } else if ((half & 7) == 0) {
    const int pair_chunks = half >> 3;               // 16-byte chunks in one half
    const int pass_chunks = (D - rotary_dim) >> 3;   // unrotated tail chunks
    const int per_row = pair_chunks + pass_chunks;
    for (int u = lane; u < gqa * per_row; u += 32) {
      const int r = u / per_row;
      const int c = u - r * per_row;
      const __nv_bfloat16* src = qsrc + r * D;
      __nv_bfloat16* dst = qs + r * kRow;
      if (c < pair_chunks) {
        const uint4 lo4 = *reinterpret_cast<const uint4*>(src + c * 8);
        const uint4 hi4 = *reinterpret_cast<const uint4*>(src + half + c * 8);
        const float4 ca = *reinterpret_cast<const float4*>(cs + c * 8);
        const float4 cb = *reinterpret_cast<const float4*>(cs + c * 8 + 4);
        const float4 sa = *reinterpret_cast<const float4*>(cs + half + c * 8);
        const float4 sb = *reinterpret_cast<const float4*>(cs + half + c * 8 + 4);
        const float cosv[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
        const float sinv[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};
        const __nv_bfloat16* lo = reinterpret_cast<const __nv_bfloat16*>(&lo4);
        const __nv_bfloat16* hi = reinterpret_cast<const __nv_bfloat16*>(&hi4);
        uint4 olo, ohi;
        __nv_bfloat16* ol = reinterpret_cast<__nv_bfloat16*>(&olo);
        __nv_bfloat16* oh = reinterpret_cast<__nv_bfloat16*>(&ohi);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float a = __bfloat162float(lo[e]);
          const float b = __bfloat162float(hi[e]);
          const float sn = neg ? -sinv[e] : sinv[e];
          ol[e] = __float2bfloat16_rn(__fsub_rn(__fmul_rn(cosv[e], a), __fmul_rn(sn, b)));
          oh[e] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(cosv[e], b), __fmul_rn(sn, a)));
        }
        *reinterpret_cast<uint4*>(dst + c * 8) = olo;
        *reinterpret_cast<uint4*>(dst + half + c * 8) = ohi;
      } else {
        const int d = rotary_dim + (c - pair_chunks) * 8;
        *reinterpret_cast<uint4*>(dst + d) = *reinterpret_cast<const uint4*>(src + d);
      }
    }
  } else {
    for (int idx = lane; idx < gqa * D; idx += 32) {
      const int r = idx / D;
      const int d = idx - r * D;
      qs[r * kRow + d] = __float2bfloat16_rn(rope_element(qsrc + r * D, d, rotary_dim, cs, neg));
    }
  }
}

// kBulk selects how the producers copy: one 512/256-byte bulk copy per row (TMA engine) or 16-byte
// cp.async through the load/store unit.  The bulk path is a little faster when every SM streams,
// but its per-SM throughput saturates near 55 GB/s; when part of the GPU is busy with dense tiles
// the remaining SMs pull more through the load/store path (measured 51 vs 68 us on 108 SMs).
template <int D, bool kBulk>
__global__ void __launch_bounds__(StreamCfg<D>::kWarps * 64, 1)
    view_decode_stream_kernel(const __grid_constant__ DecodeParams p) {
  using Cfg = StreamCfg<D>;
  using Sm = StreamSmem<D>;
  constexpr int NST = Cfg::kStages;
  constexpr int KSTEPS = D / 16;          // k-steps of the QK product = m-tiles of the PV product
  constexpr uint32_t kRowCopy = D * 2;    // bytes of one K or V row

  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Warps [0, kWarps) are the lanes' consumers (tensor-core math), warps [kWarps, 2 kWarps) their
  // producers: producer w + kWarps walks the same item list as consumer w one ring ahead and does
  // nothing but page-table lookups and bulk copies, so a copy engine that pushes back never
  // stalls the math and the next item's first stages are in flight while the consumer still
  // writes the previous item's partial and stages its queries.
  const bool producer = warp >= Cfg::kWarps;
  const int wl = producer ? warp - Cfg::kWarps : warp;   // lane of this CTA
  unsigned char* wbase = smem_raw + wl * Sm::kWarpBytes;
  const uint32_t full_u32 = smem_u32(wbase);             // NST "stage landed" barriers
  const uint32_t empty_u32 = full_u32 + NST * 8;         // NST "stage consumed" barriers
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(wbase + Sm::kBarBytes);
  unsigned char* ring = wbase + Sm::kBarBytes + Sm::kQBytes;
  const uint32_t ring_u32 = smem_u32(ring);
  static_assert(2 * NST * 8 <= Sm::kBarBytes, "barrier area");
  if (!producer && lane == 0) {
#pragma unroll
    for (int i = 0; i < NST; ++i) {
      mbar_init(full_u32 + i * 8, kBulk ? 1 : 32);   // expect_tx arrival, or one arrival per producer lane
      mbar_init(empty_u32 + i * 8, 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  // the merge pass may be made resident now; it waits for this grid to complete
  pdl_launch_dependents();

  const int lane_id = blockIdx.x * Cfg::kWarps + wl;
  if (lane_id >= p.num_lanes) return;
  const int it_begin = p.lane_off[lane_id];
  const int it_end = p.lane_off[lane_id + 1];
  const int gqa = p.num_q_heads / p.num_kv_heads;
  const int P = p.page_size;
  const int64_t slot_stride = static_cast<int64_t>(p.num_kv_heads) * D;  // elements per slot
  uint32_t gs = 0;  // stages of this lane so far: ring slot gs % NST, use gs / NST of that slot

  // an item both roles skip (the consumer reports it)
  auto item_ok = [&](int it, const int32_t* item) {
    return !(it < 0 || it >= p.num_items || item[3] < 0 || item[3] >= p.num_rows || item[5] < 0 ||
             item[5] >= p.num_partials || item[6] < 0 || item[6] >= p.num_kv_heads || item[2] <= 0 ||
             item[0] < 0 || item[1] < 0);
  };

  if (producer) {
    // =================================================================== producer
    // (when this grid was launched as a programmatic dependent of the kernel that stores the step's
    // new keys, its prologue ran beside that kernel; the pools may only be read from here on)
    pdl_wait();
    // streamed keys and values are read once: they should not push a shared block that the dense
    // tiles re-read out of L2
    const uint64_t stream_policy = l2_policy_evict_first();
    for (int it = it_begin; it < it_end; ++it) {
      const int32_t* item = p.items + static_cast<int64_t>(it) * VA_ITEM_WORDS;
      if (!item_ok(it, item)) continue;
      const int page_off = item[0];
      const int tok_begin = item[1];
      const int n_keys = item[2];
      const int kvh = item[6];
      const int n_stages = (n_keys + kKeysPerStage - 1) / kKeysPerStage;
      // page number of key `lane` of a stage (lanes 0..15): -1 past the end of the item, -2 for a
      // table index outside the plan; loaded one stage before it is needed
      auto fetch_page = [&](int stage) -> int {
        const int kk = stage * kKeysPerStage + lane;
        int page = -1;
        if (lane < kKeysPerStage && kk < n_keys) {
          const int pidx = page_off + (tok_begin + kk) / P;
          page = pidx < p.num_page_indices ? __ldg(p.page_indices + pidx) : -2;
        }
        return page;
      };
      int page_cur = fetch_page(0);
      for (int s = 0; s < n_stages; ++s, ++gs) {
        const int page_next = fetch_page(s + 1);
        const int b = gs % NST;
        if (!mbar_wait_bounded(empty_u32 + b * 8, ((gs / NST) & 1u) ^ 1u, kWaitPolls)) {
          // the consumer stopped freeing stages: give the copies already issued a bounded time
          report(p.status, VA_DEV_WAIT_EXPIRED);
          for (uint32_t k = 1; k <= NST && k <= gs; ++k) {
            const uint32_t g2 = gs - k;
            mbar_wait_bounded(full_u32 + (g2 % NST) * 8, (g2 / NST) & 1u, kWaitPolls);
          }
          return;
        }
        int my_slot = -1;
        if (page_cur != -1) {
          if (page_cur < 0 || page_cur >= p.num_pages) {
            report(p.status, VA_DEV_BAD_PAGE);
          } else {
            my_slot = page_cur * P + (tok_begin + s * kKeysPerStage + lane) % P;
          }
        }
        const uint32_t bar = full_u32 + b * 8;
        const uint32_t kdst = ring_u32 + b * Sm::kStageBytes + lane * Sm::kRowBytes;
        const unsigned valid = __ballot_sync(0xffffffffu, my_slot >= 0) & 0xffffu;
        if constexpr (kBulk) {
          if (lane < kKeysPerStage && my_slot < 0) {
            // rows past the end of the item are zeroed, so stale shared memory never reaches the
            // tensor cores; ordered before the consumer's wait by the arrive below
#pragma unroll 4
            for (uint32_t i = 0; i < kRowCopy; i += 16) {
              asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};\n" ::"r"(kdst + i), "r"(0) : "memory");
              asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};\n" ::"r"(kdst + Sm::kTileBytes + i), "r"(0)
                           : "memory");
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive_expect_tx(bar, __popc(valid) * 2 * kRowCopy);
          __syncwarp();
          if (lane < kKeysPerStage && my_slot >= 0) {
            const int64_t off = static_cast<int64_t>(my_slot) * slot_stride + static_cast<int64_t>(kvh) * D;
            bulk_g2s_hint(kdst, p.k_pool + off, kRowCopy, bar, stream_policy);
            bulk_g2s_hint(kdst + Sm::kTileBytes, p.v_pool + off, kRowCopy, bar, stream_policy);
          }
        } else {
          // the warp copies row after row, 512 bytes per instruction; a row past the end of the
          // item is zero-filled (source size 0); each lane's arrival fires when its copies land
          const uint32_t tile0 = ring_u32 + b * Sm::kStageBytes;
#pragma unroll 4
          for (int r = 0; r < kKeysPerStage; ++r) {
            const int sl = __shfl_sync(0xffffffffu, my_slot, r);
            const int64_t off = static_cast<int64_t>(sl < 0 ? 0 : sl) * slot_stride + static_cast<int64_t>(kvh) * D;
            const int nbytes = sl < 0 ? 0 : 16;
#pragma unroll
            for (int c = lane; c < D / 8; c += 32) {
              cp_async16_hint(tile0 + r * Sm::kRowBytes + c * 16, p.k_pool + off + c * 8, nbytes, stream_policy);
              cp_async16_hint(tile0 + Sm::kTileBytes + r * Sm::kRowBytes + c * 16, p.v_pool + off + c * 8, nbytes,
                              stream_policy);
            }
          }
          asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
        }
        page_cur = page_next;
      }
    }
    return;
  }

  // ===================================================================== consumer
  const int g = lane >> 2;  // fragment row group
  const int t = lane & 3;   // fragment column pair
  // ldmatrix lane addressing inside a tile of 16 padded rows.
  //   K (A operand, rows = keys):      matrix m = lane>>3 : key = (lane&7) + (m&1)*8, dim += (m>>1)*8
  //   V (A operand, transposed load):  matrix m = lane>>3 : key = (lane&7) + (m>>1)*8, dim += (m&1)*8
  const int lmat = lane >> 3;
  const uint32_t k_lane_off = ((lane & 7) + (lmat & 1) * 8) * Sm::kRowBytes + (lmat >> 1) * 16;
  const uint32_t v_lane_off =
      Sm::kTileBytes + ((lane & 7) + (lmat >> 1) * 8) * Sm::kRowBytes + (lmat & 1) * 16;

  for (int it = it_begin; it < it_end; ++it) {
    const int32_t* item = p.items + static_cast<int64_t>(it) * VA_ITEM_WORDS;
    if (!item_ok(it, item)) {
      report(p.status, VA_DEV_BAD_ROW);
      continue;
    }
    const int n_keys = item[2];
    const int qrow = item[3];
    const int delta = item[4];
    const int part = item[5];
    const int kvh = item[6];
    const int n_stages = (n_keys + kKeysPerStage - 1) / kKeysPerStage;

    // ---- stage the rotated queries of this kv head's GQA group: qs[8][D] (rows >= gqa are 0)
    stage_queries<D>(qs, p.q + static_cast<int64_t>(qrow) * p.q_row_stride +
                             static_cast<int64_t>(kvh) * gqa * D,
                     gqa, p.rotary_dim, p.cos_sin, p.max_pos, delta, lane);
    __syncwarp();
    // B fragments of Qrot^T: b0 = Q[g][16*ks + 2t..], b1 = Q[g][16*ks + 8 + 2t..]
    uint32_t qf[KSTEPS][2];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      const uint32_t* row = reinterpret_cast<const uint32_t*>(qs + g * (Sm::kRowBytes / 2));
      qf[ks][0] = row[ks * 8 + t];
      qf[ks][1] = row[ks * 8 + 4 + t];
    }
    __syncwarp();  // qs may be overwritten by the next item's staging only after these reads

    float acc[KSTEPS][4];
#pragma unroll
    for (int i = 0; i < KSTEPS; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};  // per-thread partial sums (reduced over g at the end)

    for (int s = 0; s < n_stages; ++s, ++gs) {
      const int b = gs % NST;
      if (!mbar_wait_bounded(full_u32 + b * 8, (gs / NST) & 1u, kWaitPolls)) {
        // A bounded wait ran out.  Copies the producer issued may still land in this lane's ring:
        // give every barrier a bounded time, then stop working.
        report(p.status, VA_DEV_WAIT_EXPIRED);
        for (uint32_t k = 1; k < NST; ++k)
          mbar_wait_bounded(full_u32 + ((gs + k) % NST) * 8, ((gs + k) / NST) & 1u, kWaitPolls);
        return;
      }
      __syncwarp();
      const uint32_t sbase = ring_u32 + b * Sm::kStageBytes;

      // ---- S^T (16 keys x 8 heads) = K . Qrot^T, four accumulators to shorten the dependency chain
      float sacc[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        uint32_t a[4];
        ldmatrix_x4(a, sbase + k_lane_off + ks * 32);
        mma_bf16_16816(sacc[ks & 3], a, qf[ks]);
      }
      // fragment: [0]=(key g, head 2t) [1]=(key g, head 2t+1) [2]=(key g+8, 2t) [3]=(key g+8, 2t+1)
      const int kbase = s * kKeysPerStage;
      const bool v_lo = kbase + g < n_keys;
      const bool v_hi = kbase + g + 8 < n_keys;
      float x[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = (sacc[0][i] + sacc[1][i]) + (sacc[2][i] + sacc[3][i]);
      x[0] = v_lo ? x[0] * p.scale_log2 : -INFINITY;
      x[1] = v_lo ? x[1] * p.scale_log2 : -INFINITY;
      x[2] = v_hi ? x[2] * p.scale_log2 : -INFINITY;
      x[3] = v_hi ? x[3] * p.scale_log2 : -INFINITY;
      float mx[2] = {fmaxf(x[0], x[2]), fmaxf(x[1], x[3])};
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], off));
        mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], off));
      }
      // key `kbase` is always valid, so the new maxima are finite
      const float mn0 = fmaxf(m_run[0], mx[0]);
      const float mn1 = fmaxf(m_run[1], mx[1]);
      const bool grew = (mn0 != m_run[0]) || (mn1 != m_run[1]);
      float pr[4];
      pr[0] = fast_exp2(x[0] - mn0);
      pr[1] = fast_exp2(x[1] - mn1);
      pr[2] = fast_exp2(x[2] - mn0);
      pr[3] = fast_exp2(x[3] - mn1);
      if (__any_sync(0xffffffffu, grew)) {
        const float c0 = fast_exp2(m_run[0] - mn0);
        const float c1 = fast_exp2(m_run[1] - mn1);
        l_run[0] *= c0;
        l_run[1] *= c1;
#pragma unroll
        for (int i = 0; i < KSTEPS; ++i) {
          acc[i][0] *= c0;
          acc[i][1] *= c1;
          acc[i][2] *= c0;
          acc[i][3] *= c1;
        }
        m_run[0] = mn0;
        m_run[1] = mn1;
      }
      l_run[0] += pr[0] + pr[2];
      l_run[1] += pr[1] + pr[3];
      uint32_t pb[2];
      pb[0] = movmatrix_trans(pack_bf16(pr[0], pr[1]));  // keys 0..7  -> k = 2t..2t+1
      pb[1] = movmatrix_trans(pack_bf16(pr[2], pr[3]));  // keys 8..15 -> k = 8+2t..
      // ---- O^T (D x 8 heads) += V^T . P^T
#pragma unroll
      for (int mt = 0; mt < KSTEPS; ++mt) {
        uint32_t a[4];
        ldmatrix_x4_trans(a, sbase + v_lane_off + mt * 32);
        mma_bf16_16816(acc[mt], a, pb);
      }
      __syncwarp();  // every lane has read this stage

      if (s == n_stages - 1) {
        // ---- last stage: write the partial.  Reduce the sums over the 8 key groups, stage O^T as
        // [head][dim] in this stage's buffer (still owned by the consumer), copy it out.
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
          l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], off);
          l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], off);
        }
        float* stage_f = reinterpret_cast<float*>(ring + b * Sm::kStageBytes);  // 8 x D fp32 <= one K tile
#pragma unroll
        for (int mt = 0; mt < KSTEPS; ++mt) {
          stage_f[(2 * t) * D + mt * 16 + g] = acc[mt][0];
          stage_f[(2 * t + 1) * D + mt * 16 + g] = acc[mt][1];
          stage_f[(2 * t) * D + mt * 16 + g + 8] = acc[mt][2];
          stage_f[(2 * t + 1) * D + mt * 16 + g + 8] = acc[mt][3];
        }
        __syncwarp();
        {
          const int64_t head0 = static_cast<int64_t>(part) * gqa;  // partials hold one GQA group
          float4* dst = reinterpret_cast<float4*>(p.partial_o + head0 * D);
          const float4* src = reinterpret_cast<const float4*>(stage_f);
          for (int i = lane; i < gqa * D / 4; i += 32) dst[i] = src[i];
          if (g == 0) {
            float* ml = p.partial_ml + head0 * 2;
            if (2 * t < gqa) {
              ml[(2 * t) * 2 + 0] = m_run[0];
              ml[(2 * t) * 2 + 1] = l_run[0];
            }
            if (2 * t + 1 < gqa) {
              ml[(2 * t + 1) * 2 + 0] = m_run[1];
              ml[(2 * t + 1) * 2 + 1] = l_run[1];
            }
          }
        }
        // the staging buffer was written through the generic proxy and is refilled by bulk copies
        fence_proxy_async();
        __syncwarp();
      }
      if (lane == 0) mbar_arrive(empty_u32 + b * 8);   // the producer may refill this stage
    }
  }
}

// One warp per (query row, query head); the partials of (row, kv head) are contiguous:
//     out = sum_i O_i 2^(m_i - M) / sum_i l_i 2^(m_i - M),   M = max_i m_i.
// The (m, l) pairs are read first, one partial per lane, so that the weights are known before
// any O row is touched and the O rows can be fetched several at a time.
template <int D>
__global__ void __launch_bounds__(128) view_decode_merge_kernel(const __grid_constant__ DecodeParams p) {
  pdl_wait();   // launched early: the partials are complete once the streaming grid has finished
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int total = p.num_rows * p.num_q_heads;
  if (warp_global >= total) return;
  const int row = warp_global / p.num_q_heads;
  const int head = warp_global - row * p.num_q_heads;
  const int gqa = p.num_q_heads / p.num_kv_heads;
  const int kvh = head / gqa;
  const int local = head - kvh * gqa;
  const int group = row * p.num_kv_heads + kvh;
  int s_begin = p.row_part_off[group];
  int s_end = p.row_part_off[group + 1];
  if (s_begin < 0 || s_end > p.num_partials || s_end < s_begin) {
    report(p.status, VA_DEV_BAD_ROW);
    s_end = s_begin = 0;
  }
  constexpr int VEC = D / 32;  // floats per lane
  float o[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) o[i] = 0.f;
  float m = -INFINITY, l = 0.f;   // running offset and sum of the chunks merged so far
  for (int c0 = s_begin; c0 < s_end; c0 += 32) {
    const int n = min(32, s_end - c0);
    // ---- (m, l) of partial c0 + lane, the chunk's maximum, every partial's weight
    float mi = -INFINITY, li = 0.f;
    if (lane < n) {
      const float2 ml = *reinterpret_cast<const float2*>(
          p.partial_ml + (static_cast<int64_t>(c0 + lane) * gqa + local) * 2);
      mi = ml.x;
      li = ml.y;
    }
    float mc = mi;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mc = fmaxf(mc, __shfl_xor_sync(0xffffffffu, mc, off));
    const float mn = fmaxf(m, mc);
    const float c_old = mn == -INFINITY ? 1.f : fast_exp2(m - mn);
    const float wi = (lane < n && mn != -INFINITY) ? fast_exp2(mi - mn) : 0.f;
    float lw = li * wi;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) lw += __shfl_xor_sync(0xffffffffu, lw, off);
    l = l * c_old + lw;
    m = mn;
#pragma unroll
    for (int i = 0; i < VEC; ++i) o[i] *= c_old;
    // ---- weighted sum of the O rows, four partials in flight
    const float* base = p.partial_o + (static_cast<int64_t>(c0) * gqa + local) * D + lane * VEC;
    const int64_t pstride = static_cast<int64_t>(gqa) * D;
    for (int i0 = 0; i0 < n; i0 += 4) {
      float4 v[4][VEC / 4];
      float w[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        w[u] = __shfl_sync(0xffffffffu, wi, min(i0 + u, 31));
        if (i0 + u < n) {
#pragma unroll
          for (int q = 0; q < VEC / 4; ++q)
            v[u][q] = *reinterpret_cast<const float4*>(base + (i0 + u) * pstride + q * 4);
        } else {
          w[u] = 0.f;
#pragma unroll
          for (int q = 0; q < VEC / 4; ++q) v[u][q] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
#pragma unroll
        for (int q = 0; q < VEC / 4; ++q) {
          o[q * 4 + 0] += v[u][q].x * w[u];
          o[q * 4 + 1] += v[u][q].y * w[u];
          o[q * 4 + 2] += v[u][q].z * w[u];
          o[q * 4 + 3] += v[u][q].w * w[u];
        }
      }
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  __nv_bfloat16* dst = p.out + static_cast<int64_t>(row) * p.out_row_stride + static_cast<int64_t>(head) * D + lane * VEC;
#pragma unroll
  for (int i = 0; i < VEC; i += 2) {
    *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(o[i] * inv, o[i + 1] * inv);
  }
}

template <int D>
int launch_decode(const DecodeParams& p, int sm_count, cudaStream_t stream) {
  using Cfg = StreamCfg<D>;
  using Sm = StreamSmem<D>;
  const int blocks = (p.num_lanes + Cfg::kWarps - 1) / Cfg::kWarps;
  // bulk copies when (nearly) every SM streams, the load/store path when the kernel shares the
  // GPU with dense tiles
  if (sm_count <= 0) sm_count = va_sm_count();
  const bool bulk = blocks * 10 >= sm_count * 9;
  {
    // per device and cheap; repeated so that every device a process uses gets the opt-in
    cudaError_t e = bulk ? cudaFuncSetAttribute(view_decode_stream_kernel<D, true>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, Sm::kTotalBytes)
                         : cudaFuncSetAttribute(view_decode_stream_kernel<D, false>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, Sm::kTotalBytes);
    if (e != cudaSuccess) return va_host::note_cuda_error(e);
  }
  if ((p.phase_mask & VA_PHASE_SKIP_STREAM) == 0 && p.num_items > 0) {
    // A plain launch, unless the dense tiles were forked before the store kernel
    // (VA_PHASE_GROUPS_FORKED): they then hold their SMs already and this grid may become resident
    // under the store kernel.  (Letting it start early while the dense tiles still waited for the
    // store changed where its CTAs land relative to theirs and cost 4 us per step.)
    cudaError_t e;
    if ((p.phase_mask & VA_PHASE_GROUPS_FORKED) != 0) {
      e = bulk ? va_host::launch_dependent(view_decode_stream_kernel<D, true>, dim3(blocks), dim3(Cfg::kWarps * 64),
                                           Sm::kTotalBytes, stream, p)
               : va_host::launch_dependent(view_decode_stream_kernel<D, false>, dim3(blocks), dim3(Cfg::kWarps * 64),
                                           Sm::kTotalBytes, stream, p);
    } else {
      if (bulk) view_decode_stream_kernel<D, true><<<blocks, Cfg::kWarps * 64, Sm::kTotalBytes, stream>>>(p);
      else view_decode_stream_kernel<D, false><<<blocks, Cfg::kWarps * 64, Sm::kTotalBytes, stream>>>(p);
      e = cudaGetLastError();
    }
    if (e != cudaSuccess) return va_host::note_cuda_error(e);
  }
  if ((p.phase_mask & VA_PHASE_SKIP_MERGE) == 0) {
    const int merge_warps = p.num_rows * p.num_q_heads;
    const int merge_blocks = (merge_warps + 3) / 4;
    cudaError_t e = va_host::launch_dependent(view_decode_merge_kernel<D>, dim3(merge_blocks), dim3(128), 0,
                                              stream, p);
    if (e != cudaSuccess) return va_host::note_cuda_error(e);
  }
  return VA_OK;
}

}  // namespace

extern "C" int va_view_dense(const VaPool* pool, const VaDensePlan* plan, const void* q,
                             int64_t q_row_stride, void* out, int64_t out_row_stride,
                             float* partial_o, float* partial_ml, int32_t* status,
                             va_stream_t stream);

namespace {
// Side stream and fork/join events for the dense tiles of a decode step, one set per device.
struct SideStream {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr;
  cudaEvent_t join = nullptr;
};
SideStream g_side[64];

int side_stream(SideStream** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  if (dev < 0 || dev >= 64) return VA_ERR_UNSUPPORTED;
  SideStream& s = g_side[dev];
  if (s.stream == nullptr) {
    e = cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) return va_host::note_cuda_error(e);
    e = cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming);
    if (e != cudaSuccess) return va_host::note_cuda_error(e);
    e = cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming);
    if (e != cudaSuccess) return va_host::note_cuda_error(e);
  }
  *out = &s;
  return VA_OK;
}
}  // namespace

extern "C" int va_decode_lane_width(int32_t head_dim) {
  if (head_dim == 256) return StreamCfg<256>::kWarps;
  if (head_dim == 128) return StreamCfg<128>::kWarps;
  return VA_ERR_UNSUPPORTED;
}

extern "C" int va_decode_lanes(int32_t head_dim) {
  const int sms = va_sm_count();
  if (sms <= 0) return VA_ERR_LAUNCH;
  if (head_dim == 256) return sms * StreamCfg<256>::kWarps;
  if (head_dim == 128) return sms * StreamCfg<128>::kWarps;
  return VA_ERR_UNSUPPORTED;
}

namespace {
// Argument checks of a decode step, shared by both entry points; nothing is launched on failure.
int check_decode_args(const VaPool* pool, const VaDecodePlan* plan, const void* q, int64_t q_row_stride,
                      const void* out, int64_t out_row_stride, const float* partial_o,
                      const float* partial_ml) {
  int rc = va_host::check_pool(pool);
  if (rc != VA_OK) return rc;
  if (plan == nullptr || q == nullptr || out == nullptr) return VA_ERR_BAD_ARG;
  if (plan->num_rows < 0 || plan->num_items < 0 || plan->num_partials < 0) return VA_ERR_BAD_ARG;
  if (plan->num_rows == 0) return VA_OK;
  if (plan->lane_off == nullptr || plan->row_part_off == nullptr) return VA_ERR_BAD_ARG;
  if (plan->num_items > 0 && (plan->items == nullptr || plan->page_indices == nullptr)) return VA_ERR_BAD_ARG;
  if (plan->num_partials > 0 && (partial_o == nullptr || partial_ml == nullptr)) return VA_ERR_BAD_ARG;
  const int gqa = pool->num_q_heads / pool->num_kv_heads;
  if (gqa < 1 || gqa > 8 || gqa * pool->num_kv_heads != pool->num_q_heads) return VA_ERR_UNSUPPORTED;
  {
    const int width = va_decode_lane_width(pool->head_dim);
    if (width <= 0) return VA_ERR_UNSUPPORTED;
    if (plan->num_lanes <= 0 || plan->num_lanes % width != 0 ||
        plan->num_lanes > va_decode_lanes(pool->head_dim))
      return VA_ERR_BAD_ARG;
  }
  // the dense tiles of `groups` write into the same scratch: they may not name a slot beyond it
  if (plan->groups != nullptr && plan->groups->num_tiles > 0 &&
      plan->groups->num_partials > plan->num_partials)
    return VA_ERR_CAPACITY;
  if ((reinterpret_cast<uintptr_t>(pool->k) | reinterpret_cast<uintptr_t>(pool->v) |
       reinterpret_cast<uintptr_t>(partial_o) | reinterpret_cast<uintptr_t>(q) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return VA_ERR_BAD_ARG;
  if ((q_row_stride & 7) || (out_row_stride & 1)) return VA_ERR_BAD_ARG;
  return VA_OK;
}
}  // namespace

extern "C" int va_view_decode(const VaPool* pool, const VaDecodePlan* plan, const void* q,
                              int64_t q_row_stride, void* out, int64_t out_row_stride,
                              float* partial_o, float* partial_ml, int32_t* status,
                              va_stream_t stream) {
  int rc = check_decode_args(pool, plan, q, q_row_stride, out, out_row_stride, partial_o, partial_ml);
  if (rc != VA_OK) return rc;
  if (plan->num_rows == 0) return VA_OK;

  DecodeParams p;
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
  p.items = plan->items;
  p.lane_off = plan->lane_off;
  p.row_part_off = plan->row_part_off;
  p.num_items = plan->num_items;
  p.num_lanes = plan->num_lanes;
  p.num_rows = plan->num_rows;
  p.num_partials = plan->num_partials;
  p.num_page_indices = plan->num_page_indices;
  p.phase_mask = plan->phase_mask;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_row_stride = q_row_stride;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_row_stride = out_row_stride;
  p.partial_o = partial_o;
  p.partial_ml = partial_ml;
  p.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // dense tiles of shared blocks: fork onto the side stream, join before the merge pass
  SideStream* side = nullptr;
  const bool with_groups = plan->groups != nullptr && plan->groups->num_tiles > 0 &&
                           (plan->phase_mask & VA_PHASE_SKIP_GROUPS) == 0;
  const bool forked = with_groups && (plan->phase_mask & VA_PHASE_GROUPS_FORKED) != 0;
  if (forked) {
    // va_view_decode_fork_groups launched the tiles earlier on this stream: only the join is left
    rc = side_stream(&side);
    if (rc != VA_OK) return rc;
  } else if (with_groups) {
    rc = side_stream(&side);
    if (rc != VA_OK) return rc;
    cudaError_t e = cudaEventRecord(side->fork, s);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(side->stream, side->fork, 0);
    if (e != cudaSuccess) return va_host::note_cuda_error(e);
    rc = va_view_dense(pool, plan->groups, q, q_row_stride, out, out_row_stride, partial_o, partial_ml,
                       status, side->stream);
    if (rc != VA_OK) return rc;
    e = cudaEventRecord(side->join, side->stream);
    if (e != cudaSuccess) return va_host::note_cuda_error(e);
  }
  const int merge_mask = p.phase_mask;
  p.phase_mask |= VA_PHASE_SKIP_MERGE;
  if (!forked) p.phase_mask &= ~VA_PHASE_GROUPS_FORKED;
  if (pool->head_dim == 256) rc = launch_decode<256>(p, 0, s);
  else if (pool->head_dim == 128) rc = launch_decode<128>(p, 0, s);
  else rc = VA_ERR_UNSUPPORTED;
  if (rc != VA_OK) return rc;
  if (with_groups) {
    cudaError_t e = cudaStreamWaitEvent(s, side->join, 0);
    if (e != cudaSuccess) return va_host::note_cuda_error(e);
  }
  if ((merge_mask & VA_PHASE_SKIP_MERGE) == 0) {
    p.phase_mask = VA_PHASE_SKIP_STREAM;
    if (pool->head_dim == 256) rc = launch_decode<256>(p, 0, s);
    else rc = launch_decode<128>(p, 0, s);
  }
  return rc;
}

// The dense tiles of a step, launched ahead of the rest: forked from `stream` where it stands (before
// the kernel that stores the step's new keys), joined by the va_view_decode call that follows on the
// same stream with VA_PHASE_GROUPS_FORKED set.
extern "C" int va_view_decode_fork_groups(const VaPool* pool, const VaDecodePlan* plan, const void* q,
                                          int64_t q_row_stride, float* partial_o, float* partial_ml,
                                          int32_t* status, va_stream_t stream) {
  if (pool == nullptr || plan == nullptr || plan->groups == nullptr || q == nullptr || partial_o == nullptr ||
      partial_ml == nullptr)
    return VA_ERR_BAD_ARG;
  if (plan->groups->num_tiles <= 0) return VA_OK;
  if (plan->groups->num_partials > plan->num_partials) return VA_ERR_CAPACITY;
  SideStream* side = nullptr;
  int rc = side_stream(&side);
  if (rc != VA_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaEventRecord(side->fork, s);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(side->stream, side->fork, 0);
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  // (mode-1 tiles write partials only: no output rows are needed here)
  rc = va_view_dense(pool, plan->groups, q, q_row_stride, nullptr, 0, partial_o, partial_ml, status, side->stream);
  if (rc != VA_OK) return rc;
  e = cudaEventRecord(side->join, side->stream);
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return VA_OK;
}

// ------------------------------------------------------------------------------------------------
// va_view_decode_static: the decode step for callers that cannot allocate device memory.
//
// va_view_decode wants its split-K scratch from the caller.  A serving process that has handed
// every free byte of HBM to its KV pool at start-up (the engine sizes the pool from the free
// memory it finds), or a host that binds this C ABI without a device allocator of its own, has
// nowhere to take that scratch from once it is running.  This variant keeps the scratch inside
// the library image instead: a fixed array in device memory that exists on every GPU that loads
// the library, from load until the process exits.
//
// What the caller has to know:
//   * Capacity.  The array holds kStaticMaxFloats floats of partial outputs and
//     kStaticMaxHeads (running max, running sum) pairs; a plan needs
//     num_partials * G * head_dim floats and num_partials * G pairs (G = query heads per kv head).
//     A larger plan is refused with VA_ERR_CAPACITY before anything is launched.
//   * First call per device.  The device address of the array is looked up on the first call made
//     while that device is current (cudaGetSymbolAddress).  Make that first call outside any
//     stream capture.
//   * One array per GPU.  All calls on a GPU use the same array, so two calls whose kernels may
//     overlap on the GPU (different streams, no dependency between them) race on it.  Calls issued
//     to one stream, one after the other, are fine.
//   * Old contents.  The array keeps whatever the previous call left.  Nothing has to be cleared:
//     every partial slot a plan names is written by exactly one work item before the merge pass
//     reads it, and slots the plan does not name are never read.
//   * Shared blocks planned as dense tiles run on the caller's stream, before the streaming pass,
//     rather than on the side stream va_view_decode uses: creating that stream would be an
//     allocation.  The results are the same.
namespace {
constexpr size_t kStaticMaxFloats = static_cast<size_t>(2048) * 8 * 256;  // 16 MiB of fp32 partial outputs
constexpr size_t kStaticMaxHeads = static_cast<size_t>(2048) * 8;         // (max, sum) pairs
static __device__ __align__(256) float g_static_partials[kStaticMaxFloats + 2 * kStaticMaxHeads];

struct StaticScratch {
  float* base = nullptr;
  bool ready = false;
};
StaticScratch g_static_by_device[64];

// Device address of the static array on the current device (looked up once per device).
int static_scratch(float** partial_o, float** partial_ml) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  if (dev < 0 || dev >= 64) return VA_ERR_UNSUPPORTED;
  StaticScratch& s = g_static_by_device[dev];
  if (!s.ready) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_partials);
    if (e != cudaSuccess) return va_host::note_cuda_error(e);
    if (ptr == nullptr) return VA_ERR_LAUNCH;
    s.base = static_cast<float*>(ptr);
    s.ready = true;
  }
  *partial_o = s.base;
  *partial_ml = s.base + kStaticMaxFloats;
  return VA_OK;
}
}  // namespace

extern "C" int va_view_decode_static(const VaPool* pool, const VaDecodePlan* plan, const void* q,
                                     int64_t q_row_stride, void* out, int64_t out_row_stride,
                                     int32_t* status, va_stream_t stream) {
  int rc = va_host::check_pool(pool);
  if (rc != VA_OK) return rc;
  if (plan == nullptr) return VA_ERR_BAD_ARG;
  if (plan->num_partials < 0) return VA_ERR_BAD_ARG;
  const size_t gqa = static_cast<size_t>(pool->num_q_heads / pool->num_kv_heads);
  // the larger of the two partial counts the step names: the dense tiles bound their writes by their own
  size_t partials = static_cast<size_t>(plan->num_partials);
  if (plan->groups != nullptr && plan->groups->num_tiles > 0) {
    if (plan->groups->num_partials < 0) return VA_ERR_BAD_ARG;
    partials = partials > static_cast<size_t>(plan->groups->num_partials)
                   ? partials : static_cast<size_t>(plan->groups->num_partials);
  }
  const size_t need_heads = partials * gqa;
  if (need_heads > kStaticMaxHeads || need_heads * static_cast<size_t>(pool->head_dim) > kStaticMaxFloats)
    return VA_ERR_CAPACITY;  // the plan does not fit the static scratch array
  float* partial_o = nullptr;
  float* partial_ml = nullptr;
  rc = static_scratch(&partial_o, &partial_ml);
  if (rc != VA_OK) return rc;
  // every check of the regular entry point, before the dense tiles are launched
  rc = check_decode_args(pool, plan, q, q_row_stride, out, out_row_stride, partial_o, partial_ml);
  if (rc != VA_OK) return rc;
  if (plan->num_rows == 0) return VA_OK;
  if (plan->groups != nullptr && plan->groups->num_tiles > 0 &&
      (plan->phase_mask & VA_PHASE_SKIP_GROUPS) == 0) {
    rc = va_view_dense(pool, plan->groups, q, q_row_stride, out, out_row_stride, partial_o, partial_ml,
                       status, stream);
    if (rc != VA_OK) return rc;
  }
  VaDecodePlan local = *plan;
  local.groups = nullptr;  // already done above, on the caller's stream
  return va_view_decode(pool, &local, q, q_row_stride, out, out_row_stride, partial_o, partial_ml, status,
                        stream);
}
