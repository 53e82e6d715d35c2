// Gated DeltaNet over an ordered block list for sm_100a: fused decode step, initial-state
// compose, and the token scan of a prefill.  head_k_dim = head_v_dim = 128.
//
// A block stores an affine summary (A_hat [H,dk,dk], B_hat [H,dv,dk]; fp32, or bf16 storage with
// fp32 arithmetic and one rounding per stored summary) of its tokens:
// S_out^T = S_in^T A_hat + B_hat (shared_cache/gdn_affine.py:1-24).  A worker's initial state is
// the fold of its chain, X0 = ((B_0) A_1 + B_1) A_2 + ... (shared_cache/gdn.py:127-180).
//
// va_gdn_step (decode).  The reference composes X0 with one GEMM per chain level, transposes it,
// runs a one-token recurrence whose stepped state it throws away, and then folds the token into
// the write block's summary with a separate scan kernel (models/qwen3_5_delta.py:443-490,
// kernel/gdn_compose.py, kernel/gdn_prefill.py:53-131).  For one token only two products with X0
// are needed, X0 k and X0 q, and a fold applied to a vector is a chain of matrix-VECTOR products:
//     (X A_j + B_j) u = X (A_j u) + B_j u
// so the step is a pure streaming kernel: every row of the write block's A_hat / B_hat is read
// once, dotted with k and q, updated (rank-1) and written once; the other chain blocks are read
// row-wise from L2.  No GEMM, no state materialised, HBM traffic = read + write of the write
// block's summary.
#include "common.cuh"
#include "tc05.cuh"

namespace {

using namespace va;

constexpr int kD = 128;  // head_k_dim = head_v_dim

struct StepParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const float* g;
  const float* beta;
  __nv_bfloat16* out;
  const int64_t* chain_a;
  const int64_t* chain_b;
  const int64_t* read_a;
  const int64_t* read_b;
  const int64_t* write_a;
  const int64_t* write_b;
  int32_t num_workers;
  int32_t depth;
  int32_t num_k_heads;
  int32_t num_v_heads;
  float l2_eps;
  float q_scale;
  int32_t* status;
  int64_t q_row_stride, k_row_stride, v_row_stride;   // elements between workers' rows
};

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
  return x;
}

// Row-group mapping of the step kernel: eight lanes share a summary row (lane l of the eight owns
// columns i * 32 + 4 l .. + 3, i = 0..3: every 16-byte piece a lane loads sits in a 128-byte run of
// its row), so a warp works on four consecutive rows at once and a dot product needs three shuffle
// steps for four rows instead of five per row.  (With one row per warp the two 5-step reductions
// per row -- 20 shuffles, a quarter-rate instruction -- cost more than the row's memory time: bf16
// rows, half the bytes, ran no faster than fp32 rows.)
// Row groups a warp has in flight: 2 x 2 KB of fp32 rows, 4 x 1 KB of bf16 rows.
template <bool kBf16>
constexpr int kGroupsInFlight = kBf16 ? 4 : 2;

__device__ __forceinline__ float dot4(float4 a, float4 b, float acc) {
  acc = fmaf(a.x, b.x, acc);
  acc = fmaf(a.y, b.y, acc);
  acc = fmaf(a.z, b.z, acc);
  return fmaf(a.w, b.w, acc);
}
// sum over the eight lanes that share a row
__device__ __forceinline__ float row_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  return x;
}

// grid (Hv, W), 256 threads.  Vectors live in shared memory as fp32.
template <bool kBf16>
__global__ void __launch_bounds__(256, 3) gdn_step_kernel(const __grid_constant__ StepParams p) {
  using IO = SumIO<kBf16>;
  constexpr int GF = kGroupsInFlight<kBf16>;
  constexpr int kPassRows = 8 * GF * 4;      // rows the CTA's eight warps cover per pass
  __shared__ __align__(16) float kn[kD];   // l2-normalised key
  __shared__ __align__(16) float qn[kD];   // l2-normalised, scaled query
  __shared__ __align__(16) float vv[kD];
  __shared__ __align__(16) float uk[2][kD];  // key / query vectors pushed back through the chain
  __shared__ __align__(16) float uq[2][kD];
  __shared__ float yk[kD];                 // X0 k, X0 q accumulated over chain blocks
  __shared__ float yq[kD];
  __shared__ float red[2][8];
  const int h = blockIdx.x;
  const int w = blockIdx.y;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int r4 = lane >> 3;   // row of the warp's group
  const int l8 = lane & 7;    // position among the row's eight lanes
  const int hk = h / (p.num_v_heads / p.num_k_heads);

  // ---- load and normalise the token's vectors
  float kx = 0.f, qx = 0.f;
  if (tid < kD) {
    kx = __bfloat162float(p.k[static_cast<int64_t>(w) * p.k_row_stride + hk * kD + tid]);
    qx = __bfloat162float(p.q[static_cast<int64_t>(w) * p.q_row_stride + hk * kD + tid]);
    vv[tid] = __bfloat162float(p.v[static_cast<int64_t>(w) * p.v_row_stride + h * kD + tid]);
    yk[tid] = 0.f;
    yq[tid] = 0.f;
  }
  {
    const float sk = warp_sum(kx * kx);
    const float sq = warp_sum(qx * qx);
    if (lane == 0) {
      red[0][warp] = sk;
      red[1][warp] = sq;
    }
  }
  __syncthreads();
  {
    const float sk = red[0][0] + red[0][1] + red[0][2] + red[0][3];
    const float sq = red[1][0] + red[1][1] + red[1][2] + red[1][3];
    if (tid < kD) {
      kn[tid] = kx * rsqrtf(sk + p.l2_eps);
      qn[tid] = qx * rsqrtf(sq + p.l2_eps) * p.q_scale;
    }
  }
  __syncthreads();
  const float gate = p.g[static_cast<int64_t>(w) * p.num_v_heads + h];
  const float bt = p.beta[static_cast<int64_t>(w) * p.num_v_heads + h];
  const float alpha = __expf(gate);
  const float ab = alpha * bt;  // same association as alpha_b * beta_b in update_affine_summary
  // this lane's columns of the key (registers); the query's are read from shared memory when needed
  float4 kc[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) kc[i] = *reinterpret_cast<const float4*>(kn + i * 32 + l8 * 4);

  // ---- phase 1: the write block's summary: dot every row with k and q, rank-1 update, write the
  //      fresh row.  rows 0..127 are A_hat, 128..255 are B_hat (a group of four rows lies in one).
  const void* ra = reinterpret_cast<const void*>(p.read_a[w]);
  const void* rb = reinterpret_cast<const void*>(p.read_b[w]);
  void* wa = reinterpret_cast<void*>(p.write_a[w]);
  void* wb = reinterpret_cast<void*>(p.write_b[w]);
  const int64_t head_off = static_cast<int64_t>(h) * kD * kD;
  // A warp fetches all the groups of a pass before it reduces the first: with little in flight per
  // warp the SM had too few bytes outstanding to cover the HBM latency.
  for (int r0 = warp * (GF * 4); r0 < 2 * kD; r0 += kPassRows) {
    typename IO::Raw xr[GF][4];
#pragma unroll
    for (int u = 0; u < GF; ++u) {
      const int r = r0 + u * 4 + r4;
      const bool is_b = r >= kD;
      const int row = is_b ? r - kD : r;
      const void* src = is_b ? rb : ra;
      // read once (and rewritten below): streaming loads and stores keep the chain blocks, which
      // every worker re-reads, in L2
      if (src != nullptr) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          xr[u][i] = IO::ld_stream(src, head_off + static_cast<int64_t>(row) * kD + i * 32 + l8 * 4);
      }
    }
#pragma unroll
    for (int u = 0; u < GF; ++u) {
      const int r = r0 + u * 4 + r4;
      const bool is_b = r >= kD;
      const int row = is_b ? r - kD : r;
      float4 x[4];
      if ((is_b ? rb : ra) != nullptr) {
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = IO::widen(xr[u][i]);
      } else {
        // no summary yet: A_hat = I, B_hat = 0
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c0 = is_b ? -8 : i * 32 + l8 * 4;   // first column of the piece (none matches for B_hat)
          x[i] = make_float4(row == c0 ? 1.f : 0.f, row == c0 + 1 ? 1.f : 0.f, row == c0 + 2 ? 1.f : 0.f,
                             row == c0 + 3 ? 1.f : 0.f);
        }
      }
      float dk_ = 0.f, dq_ = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        dk_ = dot4(x[i], kc[i], dk_);
        dq_ = dot4(x[i], *reinterpret_cast<const float4*>(qn + i * 32 + l8 * 4), dq_);
      }
      dk_ = row_sum(dk_);
      dq_ = row_sum(dq_);
      // A' = alpha A - (alpha beta (A k)) k^T ;  B' = alpha B - (alpha beta (B k)) k^T + (beta v) k^T
      const float t1 = ab * dk_;
      const float t2 = is_b ? bt * vv[row] : 0.f;
      void* dst = is_b ? wb : wa;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float4 y;
        y.x = __fsub_rn(__fmul_rn(alpha, x[i].x), __fmul_rn(t1, kc[i].x));
        y.y = __fsub_rn(__fmul_rn(alpha, x[i].y), __fmul_rn(t1, kc[i].y));
        y.z = __fsub_rn(__fmul_rn(alpha, x[i].z), __fmul_rn(t1, kc[i].z));
        y.w = __fsub_rn(__fmul_rn(alpha, x[i].w), __fmul_rn(t1, kc[i].w));
        if (is_b) {
          y.x = __fadd_rn(y.x, __fmul_rn(t2, kc[i].x));
          y.y = __fadd_rn(y.y, __fmul_rn(t2, kc[i].y));
          y.z = __fadd_rn(y.z, __fmul_rn(t2, kc[i].z));
          y.w = __fadd_rn(y.w, __fmul_rn(t2, kc[i].w));
        }
        if (dst != nullptr) IO::st_stream(dst, head_off + static_cast<int64_t>(row) * kD + i * 32 + l8 * 4, y);
      }
      if (l8 == 0) {
        if (is_b) {
          // contribution of the write block if it closes the chain (used in phase 2)
          uk[1][row] = dk_;  // scratch: B_w k
          uq[1][row] = dq_;  // scratch: B_w q
        } else {
          uk[0][row] = dk_;  // A_w k
          uq[0][row] = dq_;  // A_w q
        }
      }
    }
  }
  __syncthreads();

  // ---- phase 2: walk the chain from its last block to its first.
  //      y += B_j u ;  u <- A_j u  (only while an earlier block remains)
  int last = -1;
  for (int j = p.depth - 1; j >= 0; --j) {
    if (p.chain_b[static_cast<int64_t>(w) * p.depth + j] != 0) {
      last = j;
      break;
    }
  }
  int cur = 0;  // which of uk[cur]/uq[cur] holds the current vectors
  bool fresh = true;  // current vectors are still the token's own k / q
  for (int j = last; j >= 0; --j) {
    const void* bj = reinterpret_cast<const void*>(p.chain_b[static_cast<int64_t>(w) * p.depth + j]);
    const void* aj = reinterpret_cast<const void*>(p.chain_a[static_cast<int64_t>(w) * p.depth + j]);
    if (bj == nullptr) continue;
    bool earlier = false;
    for (int i = j - 1; i >= 0; --i) earlier = earlier || p.chain_b[static_cast<int64_t>(w) * p.depth + i] != 0;
    if (fresh && bj == rb && aj == ra && rb != nullptr) {
      // the chain ends with the write block: phase 1 already produced B_w k, B_w q, A_w k, A_w q
      if (tid < kD) {
        yk[tid] += uk[1][tid];
        yq[tid] += uq[1][tid];
      }
      __syncthreads();
      cur = 0;  // uk[0]/uq[0] = A_w k / A_w q
      fresh = false;
      continue;
    }
    // current vectors: this lane's columns, as registers
    const float* vk = fresh ? kn : uk[cur];
    const float* vq = fresh ? qn : uq[cur];
    float4 ck[4], cq[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      ck[i] = *reinterpret_cast<const float4*>(vk + i * 32 + l8 * 4);
      cq[i] = *reinterpret_cast<const float4*>(vq + i * 32 + l8 * 4);
    }
    const int nxt = fresh ? 0 : cur ^ 1;
    __syncthreads();  // everyone has read uk[cur] before uk[nxt] (== scratch) is overwritten
    const int n_rows = earlier ? 2 * kD : kD;
    for (int r0 = warp * (GF * 4); r0 < n_rows; r0 += kPassRows) {   // as in phase 1
      typename IO::Raw xr[GF][4];
#pragma unroll
      for (int u = 0; u < GF; ++u) {
        const int r = r0 + u * 4 + r4;
        const bool is_a = r >= kD;
        const int row = is_a ? r - kD : r;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          xr[u][i] = IO::ld(is_a ? aj : bj, head_off + static_cast<int64_t>(row) * kD + i * 32 + l8 * 4);
      }
#pragma unroll
      for (int u = 0; u < GF; ++u) {
        const int r = r0 + u * 4 + r4;
        const bool is_a = r >= kD;
        const int row = is_a ? r - kD : r;
        float dk_ = 0.f, dq_ = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 x = IO::widen(xr[u][i]);
          dk_ = dot4(x, ck[i], dk_);
          dq_ = dot4(x, cq[i], dq_);
        }
        dk_ = row_sum(dk_);
        dq_ = row_sum(dq_);
        if (l8 == 0) {
          if (is_a) {
            uk[nxt][row] = dk_;
            uq[nxt][row] = dq_;
          } else {
            yk[row] += dk_;
            yq[row] += dq_;
          }
        }
      }
    }
    __syncthreads();
    cur = nxt;
    fresh = false;
  }

  // ---- phase 3: one recurrent token on X0 without forming it.
  //      kv = alpha X0 k ; delta = (v - kv) beta ; o = alpha X0 q + delta (k.q)
  {
    const float4 k4 = *reinterpret_cast<const float4*>(kn + lane * 4);
    const float4 q4 = *reinterpret_cast<const float4*>(qn + lane * 4);
    const float kq = warp_sum(k4.x * q4.x + k4.y * q4.y + k4.z * q4.z + k4.w * q4.w);
    if (tid < kD) {
      const float kv = alpha * yk[tid];
      const float delta = (vv[tid] - kv) * bt;
      const float o = alpha * yq[tid] + delta * kq;
      p.out[(static_cast<int64_t>(w) * p.num_v_heads + h) * kD + tid] = __float2bfloat16_rn(o);
    }
  }
}

// ------------------------------------------------------------------------------------ compose
struct ComposeParams {
  const int64_t* chain_a;
  const int64_t* chain_b;
  float* state;  // [W, H, dk, dv]
  int32_t num_workers;
  int32_t depth;
  int32_t num_heads;
};

// grid (H, W), 256 threads; X (dv x dk), its successor and the level's A_j in shared memory
// (3 x 64 KB).  Thread (ty, tx) owns rows 8ty.. and the columns 4tx..4tx+3 and 64+4tx..64+4tx+3
// of X A_j + B_j (two runs, so that a warp's 16-byte reads of a row of A_j are contiguous: no bank
// conflict) and sums over i in ascending order.  (With A_j's rows read from global memory inside the loop a level took
// 146 us for 256 (worker, head) pairs, a tenth of the fp32 rate: every step waited for its row.)
template <bool kBf16>
__global__ void __launch_bounds__(256) gdn_compose_kernel(const __grid_constant__ ComposeParams p) {
  using IO = SumIO<kBf16>;
  extern __shared__ __align__(16) float xs[];  // 3 * 128 * 128
  const int h = blockIdx.x;
  const int w = blockIdx.y;
  const int tid = threadIdx.x;
  const int ty = tid >> 4;
  const int tx = tid & 15;
  const int64_t head_off = static_cast<int64_t>(h) * kD * kD;
  float* cur = xs;
  float* nxt = xs + kD * kD;
  float* as = xs + 2 * kD * kD;
  bool have = false;
  for (int j = 0; j < p.depth; ++j) {
    const void* aj = reinterpret_cast<const void*>(p.chain_a[static_cast<int64_t>(w) * p.depth + j]);
    const void* bj = reinterpret_cast<const void*>(p.chain_b[static_cast<int64_t>(w) * p.depth + j]);
    if (bj == nullptr || aj == nullptr) continue;
    if (!have) {
      // the fold starts at the first block with a summary: X = B_j
      for (int i = tid * 4; i < kD * kD; i += 256 * 4)
        *reinterpret_cast<float4*>(cur + i) = IO::widen(IO::ld(bj, head_off + i));
      have = true;
      __syncthreads();
      continue;
    }
    // A_j (widened) to shared memory, 16 pieces of four values per thread in flight
#pragma unroll 4
    for (int i = tid * 4; i < kD * kD; i += 256 * 4)
      *reinterpret_cast<float4*>(as + i) = IO::widen(IO::ld(aj, head_off + i));
    __syncthreads();
    float acc[8][8];
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[r][c] = 0.f;
#pragma unroll 1
    for (int i0 = 0; i0 < kD; i0 += 4) {
      float4 xv[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) xv[r] = *reinterpret_cast<const float4*>(cur + (ty * 8 + r) * kD + i0);
#pragma unroll
      for (int ii = 0; ii < 4; ++ii) {
        const float4 a0 = *reinterpret_cast<const float4*>(as + (i0 + ii) * kD + tx * 4);
        const float4 a1 = *reinterpret_cast<const float4*>(as + (i0 + ii) * kD + kD / 2 + tx * 4);
        const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const float x = ii == 0 ? xv[r].x : ii == 1 ? xv[r].y : ii == 2 ? xv[r].z : xv[r].w;
#pragma unroll
          for (int c = 0; c < 8; ++c) acc[r][c] = fmaf(x, av[c], acc[r][c]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int64_t brow = head_off + static_cast<int64_t>(ty * 8 + r) * kD + tx * 4;
      const float4 b0 = IO::widen(IO::ld(bj, brow));
      const float4 b1 = IO::widen(IO::ld(bj, brow + kD / 2));
      float* dst = nxt + (ty * 8 + r) * kD + tx * 4;
      *reinterpret_cast<float4*>(dst) =
          make_float4(acc[r][0] + b0.x, acc[r][1] + b0.y, acc[r][2] + b0.z, acc[r][3] + b0.w);
      *reinterpret_cast<float4*>(dst + kD / 2) =
          make_float4(acc[r][4] + b1.x, acc[r][5] + b1.y, acc[r][6] + b1.z, acc[r][7] + b1.w);
    }
    __syncthreads();
    float* tmp = cur;
    cur = nxt;
    nxt = tmp;
  }
  // state[w][h][i][c] = X[c][i]  (model convention [dk, dv]); zeros when the chain has no summary
  float* dst = p.state + (static_cast<int64_t>(w) * p.num_heads + h) * kD * kD;
  for (int idx = tid; idx < kD * kD; idx += 256) {
    const int i = idx / kD;
    const int c = idx - i * kD;
    dst[idx] = have ? cur[c * kD + i] : 0.f;
  }
}

// ------------------------------------------------------------------------------------ prefill scan
struct ScanParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const float* g;
  const float* beta;
  __nv_bfloat16* out;
  const int32_t* seg_off;    // [R+1] token offsets of the requests
  const float* state0;       // [R, H, dk, dv] or null
  const int64_t* init_a;     // [R] previous summary of the write block (0 = identity)
  const int64_t* init_b;     // [R] (0 = zero)
  const int64_t* write_a;    // [R] output summaries (0 = not wanted)
  const int64_t* write_b;
  float* final_state;        // [R, H, dk, dv] or null
  int32_t num_requests;
  int32_t num_k_heads;
  int32_t num_v_heads;
  float l2_eps;
  float q_scale;
  // chunk pre-pass outputs (device scratch of the caller), all indexed [v head][token]
  __nv_bfloat16* s_k;    // [Hv][N][128] l2-normalised keys
  __nv_bfloat16* s_q;    // [Hv][N][128] l2-normalised, scaled queries
  __nv_bfloat16* s_w;    // [Hv][N][128] -W
  __nv_bfloat16* s_u;    // [Hv][N][128] U
  __nv_bfloat16* s_p;    // [Hv][N][64]  row of tril(Q K^T decay) of the token's chunk
  float* s_eg;           // [Hv][N] e^gc
  float* s_ed;           // [Hv][N] e^(gc_last - gc)
  int64_t num_tokens;
  int32_t summary_bf16;  // init_a/init_b/write_a/write_b name bf16 tensors (fp32 otherwise)
  int32_t* status;       // device word for VA_DEV_* findings, or null
};

constexpr int kScanTokens = 16;  // tokens staged per pass

// grid (3, Hv, R), 128 threads: thread c owns column c of one part of the joint state
//   part 0: S[:, c]                      value v[t][c], emits o[t][c]
//   part 1: A_hat[c, :] (= column c of A_hat^T)   value 0
//   part 2: B_hat[c, :] (= column c of B_hat^T)   value v[t][c]
// All three obey  col <- alpha col + k (value - alpha k.col) beta  (models/qwen3_5_delta.py:149-160,
// shared_cache/gdn_prefill.py:67-85 for the joint [S | A | B] formulation).
__global__ void __launch_bounds__(128) gdn_scan_kernel(const __grid_constant__ ScanParams p) {
  __shared__ __align__(16) float ks[kScanTokens][kD];
  __shared__ __align__(16) float qs[kScanTokens][kD];
  __shared__ float vs[kScanTokens][kD];
  __shared__ float al[kScanTokens], be[kScanTokens], kq[kScanTokens];
  const int part = blockIdx.x;
  const int h = blockIdx.y;
  const int r = blockIdx.z;
  const int c = threadIdx.x;
  const int warp = c >> 5;
  const int lane = c & 31;
  const int hk = h / (p.num_v_heads / p.num_k_heads);
  const int t_begin = p.seg_off[r];
  const int t_end = p.seg_off[r + 1];
  const int64_t head_off = static_cast<int64_t>(h) * kD * kD;

  float col[kD];
  if (part == 0) {
    if (p.state0 != nullptr) {
      const float* s0 = p.state0 + (static_cast<int64_t>(r) * p.num_v_heads + h) * kD * kD;
#pragma unroll
      for (int i = 0; i < kD; ++i) col[i] = s0[i * kD + c];
    } else {
#pragma unroll
      for (int i = 0; i < kD; ++i) col[i] = 0.f;
    }
  } else {
    const void* init = reinterpret_cast<const void*>(part == 1 ? p.init_a[r] : p.init_b[r]);
    if (init != nullptr) {
      const int64_t row = head_off + static_cast<int64_t>(c) * kD;
#pragma unroll
      for (int i = 0; i < kD / 4; ++i) {
        const float4 x = sum_ld4(init, row + 4 * i, p.summary_bf16 != 0);
        col[4 * i] = x.x;
        col[4 * i + 1] = x.y;
        col[4 * i + 2] = x.z;
        col[4 * i + 3] = x.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < kD; ++i) col[i] = (part == 1 && i == c) ? 1.f : 0.f;
    }
  }

  for (int t0 = t_begin; t0 < t_end; t0 += kScanTokens) {
    const int n = min(kScanTokens, t_end - t0);
    __syncthreads();
    // ---- stage: warp w normalises tokens w, w+4, ...
    for (int tt = warp; tt < n; tt += 4) {
      const int64_t tok = t0 + tt;
      const int64_t qk_off = (tok * p.num_k_heads + hk) * kD + lane * 4;
      const uint2 kraw = *reinterpret_cast<const uint2*>(p.k + qk_off);
      const uint2 qraw = *reinterpret_cast<const uint2*>(p.q + qk_off);
      const __nv_bfloat162* kp = reinterpret_cast<const __nv_bfloat162*>(&kraw);
      const __nv_bfloat162* qp = reinterpret_cast<const __nv_bfloat162*>(&qraw);
      const float2 k01 = __bfloat1622float2(kp[0]), k23 = __bfloat1622float2(kp[1]);
      const float2 q01 = __bfloat1622float2(qp[0]), q23 = __bfloat1622float2(qp[1]);
      const float sk = warp_sum(k01.x * k01.x + k01.y * k01.y + k23.x * k23.x + k23.y * k23.y);
      const float sq = warp_sum(q01.x * q01.x + q01.y * q01.y + q23.x * q23.x + q23.y * q23.y);
      const float rk = rsqrtf(sk + p.l2_eps);
      const float rq = rsqrtf(sq + p.l2_eps) * p.q_scale;
      const float4 kn = make_float4(k01.x * rk, k01.y * rk, k23.x * rk, k23.y * rk);
      const float4 qn = make_float4(q01.x * rq, q01.y * rq, q23.x * rq, q23.y * rq);
      *reinterpret_cast<float4*>(&ks[tt][lane * 4]) = kn;
      *reinterpret_cast<float4*>(&qs[tt][lane * 4]) = qn;
      const float d = warp_sum(kn.x * qn.x + kn.y * qn.y + kn.z * qn.z + kn.w * qn.w);
      const uint2 vraw = *reinterpret_cast<const uint2*>(p.v + (tok * p.num_v_heads + h) * kD + lane * 4);
      const __nv_bfloat162* vp = reinterpret_cast<const __nv_bfloat162*>(&vraw);
      const float2 v01 = __bfloat1622float2(vp[0]), v23 = __bfloat1622float2(vp[1]);
      vs[tt][lane * 4 + 0] = v01.x;
      vs[tt][lane * 4 + 1] = v01.y;
      vs[tt][lane * 4 + 2] = v23.x;
      vs[tt][lane * 4 + 3] = v23.y;
      if (lane == 0) {
        al[tt] = __expf(p.g[tok * p.num_v_heads + h]);
        be[tt] = p.beta[tok * p.num_v_heads + h];
        kq[tt] = d;
      }
    }
    __syncthreads();
    // ---- scan the staged tokens
    for (int tt = 0; tt < n; ++tt) {
      const float alpha = al[tt];
      const float bt = be[tt];
      float dk_ = 0.f, dq_ = 0.f;
      const float4* k4 = reinterpret_cast<const float4*>(ks[tt]);
      const float4* q4 = reinterpret_cast<const float4*>(qs[tt]);
      if (part == 0) {
#pragma unroll
        for (int i = 0; i < kD / 4; ++i) {
          const float4 kk = k4[i];
          const float4 qq = q4[i];
          dk_ = fmaf(kk.x, col[4 * i], dk_);
          dk_ = fmaf(kk.y, col[4 * i + 1], dk_);
          dk_ = fmaf(kk.z, col[4 * i + 2], dk_);
          dk_ = fmaf(kk.w, col[4 * i + 3], dk_);
          dq_ = fmaf(qq.x, col[4 * i], dq_);
          dq_ = fmaf(qq.y, col[4 * i + 1], dq_);
          dq_ = fmaf(qq.z, col[4 * i + 2], dq_);
          dq_ = fmaf(qq.w, col[4 * i + 3], dq_);
        }
      } else {
#pragma unroll
        for (int i = 0; i < kD / 4; ++i) {
          const float4 kk = k4[i];
          dk_ = fmaf(kk.x, col[4 * i], dk_);
          dk_ = fmaf(kk.y, col[4 * i + 1], dk_);
          dk_ = fmaf(kk.z, col[4 * i + 2], dk_);
          dk_ = fmaf(kk.w, col[4 * i + 3], dk_);
        }
      }
      const float value = part == 1 ? 0.f : vs[tt][c];
      const float delta = (value - alpha * dk_) * bt;
#pragma unroll
      for (int i = 0; i < kD / 4; ++i) {
        const float4 kk = k4[i];
        col[4 * i] = fmaf(kk.x, delta, alpha * col[4 * i]);
        col[4 * i + 1] = fmaf(kk.y, delta, alpha * col[4 * i + 1]);
        col[4 * i + 2] = fmaf(kk.z, delta, alpha * col[4 * i + 2]);
        col[4 * i + 3] = fmaf(kk.w, delta, alpha * col[4 * i + 3]);
      }
      if (part == 0) {
        const float o = alpha * dq_ + delta * kq[tt];
        p.out[((static_cast<int64_t>(t0) + tt) * p.num_v_heads + h) * kD + c] = __float2bfloat16_rn(o);
      }
    }
  }

  // ---- hand the state off
  if (part == 0) {
    if (p.final_state != nullptr) {
      float* dst = p.final_state + (static_cast<int64_t>(r) * p.num_v_heads + h) * kD * kD;
#pragma unroll
      for (int i = 0; i < kD; ++i) dst[i * kD + c] = col[i];
    }
  } else {
    void* dst = reinterpret_cast<void*>(part == 1 ? p.write_a[r] : p.write_b[r]);
    if (dst != nullptr) {
      const int64_t row = head_off + static_cast<int64_t>(c) * kD;
#pragma unroll
      for (int i = 0; i < kD / 4; ++i)
        sum_st4(dst, row + 4 * i, make_float4(col[4 * i], col[4 * i + 1], col[4 * i + 2], col[4 * i + 3]),
                p.summary_bf16 != 0);
    }
  }
}

// ---------------------------------------------------------------------------- chunked prefill
// The same three delta-rule states as gdn_scan_kernel ([S | A_hat^T | B_hat^T]), advanced a CHUNK
// of 64 tokens at a time on the tensor cores: the UT transform of _chunk_gated_delta_rule
// (models/qwen3_5_delta.py:85-114).  With gc = cumsum(g) inside the chunk and
// decay_ij = exp(gc_i - gc_j) (j <= i):
//     L      = -strict_tril(beta_i (k_i.k_j) decay_ij)
//     T      = (I - L)^-1                       (unit lower triangular, fp32, 16 x 16 blocks)
//     U      = T diag(beta) V                   W = T diag(beta e^gc) K
//     Vnew   = U - W X                          (X: the part's [dk x 128] state, fp32)
//     O      = diag(e^gc) (Q X) + tril((Q K^T) decay) Vnew           (part 0 only)
//     X     <- e^gc_last X + K^T diag(e^(gc_last - gc)) Vnew
// Products run as mma.sync m16n8k16 with bf16 operands and fp32 accumulation.
// Part 1 (A_hat^T) has value 0 and identity start, part 2 (B_hat^T) value v and zero start.
constexpr int kC = 64;            // tokens per chunk
constexpr int kLdD = kD + 8;      // row stride (elements) of [*][128] bf16 tiles: 272 B, conflict-free ldmatrix
constexpr int kLdC = kC + 8;      // row stride of [64][64] bf16 tiles
constexpr int kLdF = kC + 1;      // row stride of [64][64] fp32 tiles

// A fragment (16 x 16) of a row-major [m][k] tile
__device__ __forceinline__ void frag_a(uint32_t (&a)[4], uint32_t base, int ld, int m0, int k0, int lane) {
  ldmatrix_x4(a, base + ((m0 + (lane & 15)) * ld + k0 + (lane >> 4) * 8) * 2);
}
// A fragment of M^T where M is a row-major [k][m] tile
__device__ __forceinline__ void frag_a_t(uint32_t (&a)[4], uint32_t base, int ld, int m0, int k0, int lane) {
  ldmatrix_x4_trans(a, base + ((k0 + (lane >> 4) * 8 + (lane & 7)) * ld + m0 + ((lane >> 3) & 1) * 8) * 2);
}
// B fragments of two adjacent n-tiles (n0, n0+8) from an [n][k] tile ("n-major": B = tile^T)
__device__ __forceinline__ void frag_b_nk(uint32_t (&b)[4], uint32_t base, int ld, int n0, int k0, int lane) {
  ldmatrix_x4(b, base + ((n0 + (lane >> 4) * 8 + (lane & 7)) * ld + k0 + ((lane >> 3) & 1) * 8) * 2);
}
// B fragments of two adjacent n-tiles from a row-major [k][n] tile
__device__ __forceinline__ void frag_b_kn(uint32_t (&b)[4], uint32_t base, int ld, int k0, int n0, int lane) {
  ldmatrix_x4_trans(b, base + ((k0 + ((lane >> 3) & 1) * 8 + (lane & 7)) * ld + n0 + (lane >> 4) * 8) * 2);
}

// ------------------------------------------------------------ chunked prefill in two passes
// The state-independent half of a chunk (normalisation, K K^T, Q K^T, the triangular inverse, W, U)
// is the same for the three parts and has no dependence between chunks: gdn_chunk_pre_kernel does
// it once per (chunk, head, request), all chunks in parallel, and leaves K, Q, -W, U, P, e^gc and
// e^(gc_last-gc) in the caller's scratch.  gdn_chunk_state_kernel then walks a part's chunks in
// order with only the state-dependent products (Vnew = U - W X, O, the state update); the state X
// stays in the accumulator registers of its sixteen warps for the whole block (a 16 x 64 tile each)
// and is rounded to bf16 into shared memory once per chunk as the B operand of W X and Q X.
struct PreSmem {
  // 56 KB, so that four CTAs (16 warps) share an SM.  Regions are reused as the phases go:
  //   Q tile  -> L (fp32)          once Q K^T has been taken (a CTA-wide barrier in between)
  //   L + scratch of the inverse -> T diag(beta) and T diag(beta e^gc) (bf16) once T is complete
  //   T (fp32) -> the V tile, fetched once T has been converted (V is only needed for U, at the end)
  static constexpr int kTile = kC * kLdD * 2;                  // one [C][128] bf16 tile
  static constexpr int kKs = 0;
  static constexpr int kT = kKs + kTile;
  static constexpr int kVs = kT;
  static constexpr int kQs = kT + kTile;
  static constexpr int kL = kQs;
  static constexpr int kScr = kQs + kTile;                     // 4 x 16 x 16 fp32 of the block inverse
  static constexpr int kTb = kQs;
  static constexpr int kTw = kTb + kC * kLdC * 2;
  static constexpr int kVec = kScr + 4 * 16 * 16 * 4;
  static constexpr int kTotal = kVec + 4 * kC * 4;
  static_assert(kC * kLdF * 4 <= kTile, "L fits in the Q tile, T in the V tile");
  static_assert(kTw + kC * kLdC * 2 <= kVec, "T diag(beta) tiles fit in L + scratch");
  static_assert(4 * (kTotal + 1024) <= 228 * 1024, "four CTAs per SM");
};

// grid (chunk, Hv, R), 128 threads
__global__ void __launch_bounds__(128, 4) gdn_chunk_pre_kernel(const __grid_constant__ ScanParams p) {
  extern __shared__ __align__(128) unsigned char csm[];
  using Sm = PreSmem;
  const uint32_t sb = smem_u32(csm);
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(csm + Sm::kKs);
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(csm + Sm::kQs);
  __nv_bfloat16* Tb = reinterpret_cast<__nv_bfloat16*>(csm + Sm::kTb);
  __nv_bfloat16* Tw = reinterpret_cast<__nv_bfloat16*>(csm + Sm::kTw);
  float* Lm = reinterpret_cast<float*>(csm + Sm::kL);
  float* Tm = reinterpret_cast<float*>(csm + Sm::kT);
  float* be = reinterpret_cast<float*>(csm + Sm::kVec);
  float* gc = be + kC;
  float* eg = gc + kC;
  float* ed = eg + kC;
  const int h = blockIdx.y;
  const int r = blockIdx.z;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int g = lane >> 2;
  const int t = lane & 3;
  const int hk = h / (p.num_v_heads / p.num_k_heads);
  const int t_end = p.seg_off[r + 1];
  const int t0 = p.seg_off[r] + static_cast<int>(blockIdx.x) * kC;
  if (t0 >= t_end) return;
  const int64_t hN = static_cast<int64_t>(h) * p.num_tokens;

  // ---- stage: the raw K and Q rows of the chunk go straight to their shared-memory tiles as
  //      16-byte asynchronous copies (2048 of them, 16 per thread, all in flight at once); rows past
  //      the end are zero-filled.  (Register loads did not do: with most of the SM's 256 KB taken
  //      as shared memory by the resident CTAs the L1 keeps few lines for misses in flight,
  //      and a warp's 48 row loads took 10 us.)  The rows are then normalised in place.
  {
    constexpr int kRowChunks = kD / 8;              // 16-byte chunks of a row
    constexpr int kTileChunks = kC * kRowChunks;
#pragma unroll
    for (int j = 0; j < 2 * kTileChunks / 128; ++j) {
      const int idx = tid + 128 * j;
      const int which = idx / kTileChunks;          // 0 = K, 1 = Q (uniform per j)
      const int rem = idx - which * kTileChunks;
      const int i = rem / kRowChunks;
      const int ch = rem - i * kRowChunks;
      const int64_t tok = static_cast<int64_t>(t0) + i;
      const bool live = tok < t_end;
      const int64_t row = live ? tok : static_cast<int64_t>(t0);
      const __nv_bfloat16* src = (which == 0 ? p.k : p.q) + (row * p.num_k_heads + hk) * kD;
      cp_async16(sb + (which == 0 ? Sm::kKs : Sm::kQs) + (i * kLdD + ch * 8) * 2, src + ch * 8, live ? 16 : 0);
    }
    cp_async_commit();
    if (warp == 0) {
      // while the rows are in flight: inclusive scan of g over the 64 tokens, two per lane
      const int64_t tok = static_cast<int64_t>(t0) + 2 * lane;
      const float a = tok < t_end ? p.g[tok * p.num_v_heads + h] : 0.f;
      const float b = tok + 1 < t_end ? p.g[(tok + 1) * p.num_v_heads + h] : 0.f;
      float s = a + b;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const float o = __shfl_up_sync(0xffffffffu, s, off);
        if (lane >= off) s += o;
      }
      const float hi = s, lo = s - b;
      const float tail = __shfl_sync(0xffffffffu, s, 31);
      const float e_lo = __expf(lo), e_hi = __expf(hi);
      const float d_lo = __expf(tail - lo), d_hi = __expf(tail - hi);
      gc[2 * lane] = lo;
      gc[2 * lane + 1] = hi;
      eg[2 * lane] = e_lo;
      eg[2 * lane + 1] = e_hi;
      ed[2 * lane] = d_lo;
      ed[2 * lane + 1] = d_hi;
      if (tok < t_end) {
        p.s_eg[hN + tok] = e_lo;
        p.s_ed[hN + tok] = d_lo;
      }
      if (tok + 1 < t_end) {
        p.s_eg[hN + tok + 1] = e_hi;
        p.s_ed[hN + tok + 1] = d_hi;
      }
    } else if (warp <= 2) {
      const int i = tid - 32;
      const int64_t tok = static_cast<int64_t>(t0) + i;
      be[i] = tok < t_end ? p.beta[tok * p.num_v_heads + h] : 0.f;
    }
    cp_async_wait<0>();
    __syncthreads();
    // eight lanes per token (lane l owns the 16-byte pieces l and l + 8 of the row), four tokens per
    // warp at once, the CTA's 64 tokens in four passes: three shuffle steps per reduction
    const int r4 = lane >> 3, l8 = lane & 7;
#pragma unroll
    for (int ps = 0; ps < kC / 16; ++ps) {
      const int i = ps * 16 + warp * 4 + r4;
      const int64_t tok = static_cast<int64_t>(t0) + i;
      const bool live = tok < t_end;   // rows past the end are zeros and stay zeros
      {
        uint4 kr[2], qr[2];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          kr[c] = *reinterpret_cast<const uint4*>(Ks + i * kLdD + (l8 + 8 * c) * 8);
          qr[c] = *reinterpret_cast<const uint4*>(Qs + i * kLdD + (l8 + 8 * c) * 8);
        }
        float kf[16], qf[16];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const __nv_bfloat162* kp = reinterpret_cast<const __nv_bfloat162*>(&kr[c]);
          const __nv_bfloat162* qp = reinterpret_cast<const __nv_bfloat162*>(&qr[c]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 a = __bfloat1622float2(kp[e]), b = __bfloat1622float2(qp[e]);
            kf[8 * c + 2 * e] = a.x;
            kf[8 * c + 2 * e + 1] = a.y;
            qf[8 * c + 2 * e] = b.x;
            qf[8 * c + 2 * e + 1] = b.y;
          }
        }
        float sk = 0.f, sq = 0.f;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          sk = fmaf(kf[e], kf[e], sk);
          sq = fmaf(qf[e], qf[e], sq);
        }
        sk = row_sum(sk);
        sq = row_sum(sq);
        const float rk = rsqrtf(sk + p.l2_eps);
        const float rq = rsqrtf(sq + p.l2_eps) * p.q_scale;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint4 kn4, qn4;
          kn4.x = pack_bf16(kf[8 * c] * rk, kf[8 * c + 1] * rk);
          kn4.y = pack_bf16(kf[8 * c + 2] * rk, kf[8 * c + 3] * rk);
          kn4.z = pack_bf16(kf[8 * c + 4] * rk, kf[8 * c + 5] * rk);
          kn4.w = pack_bf16(kf[8 * c + 6] * rk, kf[8 * c + 7] * rk);
          qn4.x = pack_bf16(qf[8 * c] * rq, qf[8 * c + 1] * rq);
          qn4.y = pack_bf16(qf[8 * c + 2] * rq, qf[8 * c + 3] * rq);
          qn4.z = pack_bf16(qf[8 * c + 4] * rq, qf[8 * c + 5] * rq);
          qn4.w = pack_bf16(qf[8 * c + 6] * rq, qf[8 * c + 7] * rq);
          if (live) {
            *reinterpret_cast<uint4*>(p.s_k + (hN + tok) * kD + (l8 + 8 * c) * 8) = kn4;
            *reinterpret_cast<uint4*>(p.s_q + (hN + tok) * kD + (l8 + 8 * c) * 8) = qn4;
            *reinterpret_cast<uint4*>(Ks + i * kLdD + (l8 + 8 * c) * 8) = kn4;
            *reinterpret_cast<uint4*>(Qs + i * kLdD + (l8 + 8 * c) * 8) = qn4;
          }
        }
      }
    }
  }
  __syncthreads();

  // ---- K K^T and Q K^T for this warp's 16 rows; L (fp32) and the causal score tile P (bf16, out)
  {
    float kk[8][4], qk[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) kk[nt][e] = qk[nt][e] = 0.f;
    }
#pragma unroll
    for (int ks = 0; ks < kD / 16; ++ks) {
      uint32_t ak[4], aq[4];
      frag_a(ak, sb + Sm::kKs, kLdD, 16 * warp, 16 * ks, lane);
      frag_a(aq, sb + Sm::kQs, kLdD, 16 * warp, 16 * ks, lane);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        if (np > warp) continue;   // columns past this warp's rows are masked out (j > i): left at zero
        uint32_t b[4];
        frag_b_nk(b, sb + Sm::kKs, kLdD, 16 * np, 16 * ks, lane);
        const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
        mma_bf16_16816(kk[2 * np], ak, b0);
        mma_bf16_16816(kk[2 * np + 1], ak, b1);
        mma_bf16_16816(qk[2 * np], aq, b0);
        mma_bf16_16816(qk[2 * np + 1], aq, b1);
      }
    }
    __syncthreads();   // every warp has taken its Q rows: L is written over the Q tile
    const int i0 = 16 * warp + g;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      if (nt < 2 * (warp + 1)) {   // blocks of L above the diagonal are never read; P is zero there
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = i0 + (e >> 1) * 8;
          const int j = 8 * nt + 2 * t + (e & 1);
          const float dec = j <= i ? __expf(gc[i] - gc[j]) : 0.f;
          Lm[i * kLdF + j] = j < i ? -be[i] * kk[nt][e] * dec : 0.f;
          qk[nt][e] *= dec;
        }
      }
      if (t0 + i0 < t_end)
        *reinterpret_cast<uint32_t*>(p.s_p + (hN + t0 + i0) * kC + 8 * nt + 2 * t) = pack_bf16(qk[nt][0], qk[nt][1]);
      if (t0 + i0 + 8 < t_end)
        *reinterpret_cast<uint32_t*>(p.s_p + (hN + t0 + i0 + 8) * kC + 8 * nt + 2 * t) = pack_bf16(qk[nt][2], qk[nt][3]);
    }
  }
  // ---- T = (I - L)^-1 (unit lower triangular), in 16 x 16 blocks:
  //   diagonal block I:  T_II = (I - L_II)^-1 by forward substitution; warp I, lane j keeps column j
  //                      in registers (T[i][j] = L[i][j] + sum_{j<m<i} L[i][m] T[m][j])
  //   block (I, J), I>J: T_IJ = T_II (sum_{M=J}^{I-1} L_IM T_MJ), by block distance I - J = 1, 2, 3
  //   (blocks above the diagonal are never written or read: they are zeros by construction)
  __syncthreads();   // L is complete
  if (lane < 16) {
    const int b0 = 16 * warp;
    float tj[16];
#pragma unroll
    for (int m = 0; m < 16; ++m) tj[m] = m == lane ? 1.f : 0.f;
#pragma unroll
    for (int i = 1; i < 16; ++i) {
      float s = 0.f;
#pragma unroll
      for (int m = 0; m < 16; ++m) {
        if (m < i) {
          const float l = Lm[(b0 + i) * kLdF + b0 + m];
          if (m == lane) s += l;
          if (m > lane) s = fmaf(l, tj[m], s);
        }
      }
      if (lane < i) tj[i] = s;
    }
#pragma unroll
    for (int m = 0; m < 16; ++m) Tm[(b0 + m) * kLdF + b0 + lane] = tj[m];
  }
  __syncthreads();
  {
    // per-warp 16 x 16 staging tile; row r keeps its columns rotated by r (conflict-light stores)
    float* scratch = reinterpret_cast<float*>(csm + Sm::kScr) + warp * 16 * 16;
    const int rr = lane >> 1, c0 = (lane & 1) * 8;
    for (int d = 1; d < 4; ++d) {
      if (warp < 4 - d) {
        const int J = warp, I = warp + d;
        float s[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) s[e] = 0.f;
        for (int M = J; M < I; ++M) {
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            const float l = Lm[(16 * I + rr) * kLdF + 16 * M + k];
#pragma unroll
            for (int e = 0; e < 8; ++e) s[e] = fmaf(l, Tm[(16 * M + k) * kLdF + 16 * J + c0 + e], s[e]);
          }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) scratch[rr * 16 + ((c0 + e + rr) & 15)] = s[e];
        __syncwarp();
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = 0.f;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          const float a = Tm[(16 * I + rr) * kLdF + 16 * I + k];
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = fmaf(a, scratch[k * 16 + ((c0 + e + k) & 15)], o[e]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) Tm[(16 * I + rr) * kLdF + 16 * J + c0 + e] = o[e];
      }
      __syncthreads();
    }
  }
  // T diag(beta) and T diag(beta e^gc) as bf16, two columns per thread and step
#pragma unroll 4
  for (int idx = tid; idx < kC * kC / 2; idx += 128) {
    const int i = idx / (kC / 2), j = 2 * (idx - i * (kC / 2));
    if ((j >> 4) > (i >> 4)) continue;   // blocks above the diagonal are zero and never multiplied
    const float t0v = Tm[i * kLdF + j];
    const float t1v = Tm[i * kLdF + j + 1];
    const float b0v = t0v * be[j], b1v = t1v * be[j + 1];
    *reinterpret_cast<uint32_t*>(Tb + i * kLdC + j) = pack_bf16(b0v, b1v);
    *reinterpret_cast<uint32_t*>(Tw + i * kLdC + j) = pack_bf16(b0v * eg[j], b1v * eg[j + 1]);
  }
  __syncthreads();
  // ---- T (fp32) is dead: the V rows go to its place while W is formed
  {
    constexpr int kRowChunks = kD / 8;
#pragma unroll
    for (int j = 0; j < kC * kRowChunks / 128; ++j) {
      const int idx = tid + 128 * j;
      const int i = idx / kRowChunks;
      const int ch = idx - i * kRowChunks;
      const int64_t tok = static_cast<int64_t>(t0) + i;
      const bool live = tok < t_end;
      const int64_t row = live ? tok : static_cast<int64_t>(t0);
      cp_async16(sb + Sm::kVs + (i * kLdD + ch * 8) * 2, p.v + (row * p.num_v_heads + h) * kD + ch * 8, live ? 16 : 0);
    }
    cp_async_commit();
  }
  // ---- W = Tw K (stored negated), then U = Tb V, for this warp's 16 token rows
  const int64_t tok0 = static_cast<int64_t>(t0) + 16 * warp + g;
#pragma unroll 1
  for (int pass = 0; pass < 2; ++pass) {
    if (pass == 1) {
      cp_async_wait<0>();
      __syncthreads();
    }
    const uint32_t a_tile = sb + (pass == 0 ? Sm::kTw : Sm::kTb);
    const uint32_t b_tile = sb + (pass == 0 ? Sm::kKs : Sm::kVs);
    float acc[16][4];
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
    }
#pragma unroll
    for (int ks = 0; ks < kC / 16; ++ks) {
      if (ks > warp) continue;   // T is lower triangular: no contribution from later tokens
      uint32_t a[4];
      frag_a(a, a_tile, kLdC, 16 * warp, 16 * ks, lane);
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        uint32_t b[4];
        frag_b_kn(b, b_tile, kLdD, 16 * ks, 16 * np, lane);
        const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
        mma_bf16_16816(acc[2 * np], a, b0);
        mma_bf16_16816(acc[2 * np + 1], a, b1);
      }
    }
    __nv_bfloat16* dst = pass == 0 ? p.s_w : p.s_u;
    const float sign = pass == 0 ? -1.f : 1.f;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      if (tok0 < t_end)
        *reinterpret_cast<uint32_t*>(dst + (hN + tok0) * kD + 8 * nt + 2 * t) = pack_bf16(sign * acc[nt][0], sign * acc[nt][1]);
      if (tok0 + 8 < t_end)
        *reinterpret_cast<uint32_t*>(dst + (hN + tok0 + 8) * kD + 8 * nt + 2 * t) = pack_bf16(sign * acc[nt][2], sign * acc[nt][3]);
    }
  }
}

struct StateSmem {
  // K, -W and U of a chunk are fetched one chunk ahead into two alternating buffers; Q and P (part 0)
  // are fetched at the start of their chunk and are not needed before its second product
  static constexpr int kTile = kC * kLdD * 2;                     // one [C][128] bf16 tile
  static constexpr int kKs = 0;                                   // K    [2][C][dk]
  static constexpr int kWs = kKs + 2 * kTile;                     // -W   [2][C][dk]
  static constexpr int kUs = kWs + 2 * kTile;                     // U    [2][C][128]
  static constexpr int kQs = kUs + 2 * kTile;                     // Q    [C][dk]     (part 0)
  static constexpr int kVn = kQs + kTile;                         // Vnew [C][128]    (part 0)
  static constexpr int kVd = kVn + kTile;                         // diag(e^(gc_last-gc)) Vnew
  static constexpr int kXs = kVd + kTile;                         // X    [dk][128] bf16
  static constexpr int kPs = kXs + kD * kLdD * 2;                 // P    [C][C]      (part 0)
  static constexpr int kVec = kPs + kC * kLdC * 2;                // [2][e^gc, e^(gc_last-gc)]
  static constexpr int kTotal = kVec + 2 * 2 * kC * 4;
  static_assert(kTotal <= 227 * 1024, "shared memory of the chunk state kernel");
};

// grid (3, Hv, R), 512 threads: one part of the joint state, chunks in order.  Sixteen warps, four
// per scheduler: the chunk's products are chains of ldmatrix -> mma.sync -> shared-memory hand-offs,
// and with one warp per scheduler (an earlier version: four warps owning 32 state rows each) every
// dependent instruction stalled the SM -- the tensor pipe was busy 34 % of the time.
//   state tile of warp w: rows 16 (w & 7) .., columns 64 (w >> 3) ..   (X update, 8 n-tiles)
//   token tile of warp w: rows 16 (w & 3) .., columns 32 (w >> 2) ..   (Vnew and O, 4 n-tiles)
constexpr int kStateThreads = 512;
__global__ void __launch_bounds__(kStateThreads, 1) gdn_chunk_state_kernel(const __grid_constant__ ScanParams p) {
  extern __shared__ __align__(128) unsigned char csm[];
  using Sm = StateSmem;
  const uint32_t sb = smem_u32(csm);
  __nv_bfloat16* Vn = reinterpret_cast<__nv_bfloat16*>(csm + Sm::kVn);
  __nv_bfloat16* Vd = reinterpret_cast<__nv_bfloat16*>(csm + Sm::kVd);
  __nv_bfloat16* Xs = reinterpret_cast<__nv_bfloat16*>(csm + Sm::kXs);
  float* vec = reinterpret_cast<float*>(csm + Sm::kVec);
  const int part = blockIdx.x;
  const int h = blockIdx.y;
  const int r = blockIdx.z;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int g = lane >> 2;
  const int t = lane & 3;
  const int srow = 16 * (warp & 7), scol = 64 * (warp >> 3);   // state tile
  const int trow = 16 * (warp & 3), tcol = 32 * (warp >> 2);   // token tile
  const int t_begin = p.seg_off[r];
  const int t_end = p.seg_off[r + 1];
  const int64_t head_off = static_cast<int64_t>(h) * kD * kD;
  const int64_t hN = static_cast<int64_t>(h) * p.num_tokens;

  float acc[8][4];
  {
    const void* src = nullptr;   // part 0: fp32 state; parts 1, 2: a summary in its storage type
    int64_t src_off = 0;
    bool transposed = false;
    const bool sum_bf16 = part != 0 && p.summary_bf16 != 0;
    if (part == 0) {
      if (p.state0 != nullptr) {
        src = p.state0;
        src_off = (static_cast<int64_t>(r) * p.num_v_heads + h) * kD * kD;
      }
    } else {
      src = reinterpret_cast<const void*>(part == 1 ? p.init_a[r] : p.init_b[r]);
      src_off = head_off;
      transposed = true;
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = srow + g + (e >> 1) * 8;
        const int col = scol + 8 * nt + 2 * t + (e & 1);
        float x = (part == 1 && row == col) ? 1.f : 0.f;
        if (src != nullptr) x = sum_ld1(src, src_off + (transposed ? col * kD + row : row * kD + col), sum_bf16);
        acc[nt][e] = x;
      }
    }
  }

  // one row of a [C][128] bf16 tile = 256 bytes = 16 copies of 16 bytes; 64 rows x 16 = 1024 per tile
  auto load_tile = [&](uint32_t dst, const __nv_bfloat16* src, int t0, int row_elems, int ld) {
    const int per_row = row_elems / 8;
    for (int idx = tid; idx < kC * per_row; idx += kStateThreads) {
      const int i = idx / per_row, c = idx - i * per_row;
      const bool live = t0 + i < t_end;
      cp_async16(dst + (i * ld + c * 8) * 2, src + (hN + (live ? t0 + i : t0)) * row_elems + c * 8, live ? 16 : 0);
    }
  };
  // K, -W, U and the decay vectors of the chunk at t0 into buffer `buf`
  auto prefetch = [&](int t0, int buf) {
    if (t0 < t_end) {
      load_tile(sb + Sm::kKs + buf * Sm::kTile, p.s_k, t0, kD, kLdD);
      load_tile(sb + Sm::kWs + buf * Sm::kTile, p.s_w, t0, kD, kLdD);
      if (part != 1) load_tile(sb + Sm::kUs + buf * Sm::kTile, p.s_u, t0, kD, kLdD);
      if (tid < kC) {
        const bool live = t0 + tid < t_end;
        vec[buf * 2 * kC + tid] = live ? p.s_eg[hN + t0 + tid] : 0.f;
        vec[buf * 2 * kC + kC + tid] = live ? p.s_ed[hN + t0 + tid] : 0.f;
      }
    }
    cp_async_commit();   // (an empty group past the last chunk keeps the group count uniform)
  };
  prefetch(t_begin, 0);
  int buf = 0;
  for (int t0 = t_begin; t0 < t_end; t0 += kC, buf ^= 1) {
    __syncthreads();   // the previous chunk's tiles (and the other buffer) are no longer read
    if (part == 0) {
      load_tile(sb + Sm::kQs, p.s_q, t0, kD, kLdD);
      load_tile(sb + Sm::kPs, p.s_p, t0, kC, kLdC);
    }
    cp_async_commit();
    prefetch(t0 + kC, buf ^ 1);
    const uint32_t Kb = sb + Sm::kKs + buf * Sm::kTile;
    const uint32_t Wb = sb + Sm::kWs + buf * Sm::kTile;
    const __nv_bfloat16* Us = reinterpret_cast<const __nv_bfloat16*>(csm + Sm::kUs + buf * Sm::kTile);
    const float* eg = vec + buf * 2 * kC;
    const float* ed = eg + kC;
    // ---- X as a bf16 B operand (every warp writes its state tile) while the copies are in flight
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int row = srow + g;
      const int col = scol + 8 * nt + 2 * t;
      *reinterpret_cast<uint32_t*>(Xs + row * kLdD + col) = pack_bf16(acc[nt][0], acc[nt][1]);
      *reinterpret_cast<uint32_t*>(Xs + (row + 8) * kLdD + col) = pack_bf16(acc[nt][2], acc[nt][3]);
    }
    cp_async_wait<2>();   // this chunk's K, -W, U (fetched during the previous chunk) have landed
    __syncthreads();

    // ---- Vnew = U - W X for this warp's token tile (16 tokens x 32 columns)
    float vn[4][4];
    {
      const int i = trow + g;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        if (part != 1) {
          const int col = tcol + 8 * nt + 2 * t;
          const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(Us + i * kLdD + col));
          const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(Us + (i + 8) * kLdD + col));
          vn[nt][0] = lo.x;
          vn[nt][1] = lo.y;
          vn[nt][2] = hi.x;
          vn[nt][3] = hi.y;
        } else {
          vn[nt][0] = vn[nt][1] = vn[nt][2] = vn[nt][3] = 0.f;
        }
      }
    }
#pragma unroll
    for (int ks = 0; ks < kD / 16; ++ks) {
      uint32_t a[4];
      frag_a(a, Wb, kLdD, trow, 16 * ks, lane);
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        uint32_t b[4];
        frag_b_kn(b, sb + Sm::kXs, kLdD, 16 * ks, tcol + 16 * np, lane);
        const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
        mma_bf16_16816(vn[2 * np], a, b0);
        mma_bf16_16816(vn[2 * np + 1], a, b1);
      }
    }
    {
      const int i = trow + g;
      const float d0 = ed[i], d1 = ed[i + 8];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int col = tcol + 8 * nt + 2 * t;
        if (part == 0) {
          *reinterpret_cast<uint32_t*>(Vn + i * kLdD + col) = pack_bf16(vn[nt][0], vn[nt][1]);
          *reinterpret_cast<uint32_t*>(Vn + (i + 8) * kLdD + col) = pack_bf16(vn[nt][2], vn[nt][3]);
        }
        *reinterpret_cast<uint32_t*>(Vd + i * kLdD + col) = pack_bf16(vn[nt][0] * d0, vn[nt][1] * d0);
        *reinterpret_cast<uint32_t*>(Vd + (i + 8) * kLdD + col) = pack_bf16(vn[nt][2] * d1, vn[nt][3] * d1);
      }
    }
    cp_async_wait<1>();   // this chunk's Q and P have landed (the next chunk's tiles may still be in flight)
    __syncthreads();

    // ---- O = diag(e^gc) (Q X) + P Vnew for this warp's token tile (part 0 only)
    if (part == 0) {
      float o[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) o[nt][e] = 0.f;
      }
#pragma unroll
      for (int ks = 0; ks < kD / 16; ++ks) {
        uint32_t a[4];
        frag_a(a, sb + Sm::kQs, kLdD, trow, 16 * ks, lane);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t b[4];
          frag_b_kn(b, sb + Sm::kXs, kLdD, 16 * ks, tcol + 16 * np, lane);
          const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
          mma_bf16_16816(o[2 * np], a, b0);
          mma_bf16_16816(o[2 * np + 1], a, b1);
        }
      }
      const int i = trow + g;
      const float e0 = eg[i], e1 = eg[i + 8];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        o[nt][0] *= e0;
        o[nt][1] *= e0;
        o[nt][2] *= e1;
        o[nt][3] *= e1;
      }
#pragma unroll
      for (int ks = 0; ks < kC / 16; ++ks) {
        uint32_t a[4];
        frag_a(a, sb + Sm::kPs, kLdC, trow, 16 * ks, lane);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t b[4];
          frag_b_kn(b, sb + Sm::kVn, kLdD, 16 * ks, tcol + 16 * np, lane);
          const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
          mma_bf16_16816(o[2 * np], a, b0);
          mma_bf16_16816(o[2 * np + 1], a, b1);
        }
      }
      const int64_t tok0 = static_cast<int64_t>(t0) + i;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int col = tcol + 8 * nt + 2 * t;
        if (tok0 < t_end)
          *reinterpret_cast<uint32_t*>(p.out + (tok0 * p.num_v_heads + h) * kD + col) = pack_bf16(o[nt][0], o[nt][1]);
        if (tok0 + 8 < t_end)
          *reinterpret_cast<uint32_t*>(p.out + ((tok0 + 8) * p.num_v_heads + h) * kD + col) =
              pack_bf16(o[nt][2], o[nt][3]);
      }
    }

    // ---- X <- e^gc_last X + K^T (diag(e^(gc_last - gc)) Vnew) for this warp's state tile
    {
      const int n_live = min(kC, t_end - t0);
      const float tail = eg[n_live - 1];   // tokens past the end do not decay the state
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[nt][e] *= tail;
      }
#pragma unroll
      for (int ks = 0; ks < kC / 16; ++ks) {
        uint32_t a0[4];
        frag_a_t(a0, Kb, kLdD, srow, 16 * ks, lane);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t b[4];
          frag_b_kn(b, sb + Sm::kVd, kLdD, 16 * ks, scol + 16 * np, lane);
          const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
          mma_bf16_16816(acc[2 * np], a0, b0);
          mma_bf16_16816(acc[2 * np + 1], a0, b1);
        }
      }
    }
  }

  // ---- hand the state off
  {
    void* dst = nullptr;
    int64_t dst_off = 0;
    bool transposed = false;
    const bool sum_bf16 = part != 0 && p.summary_bf16 != 0;
    if (part == 0) {
      if (p.final_state != nullptr) {
        dst = p.final_state;
        dst_off = (static_cast<int64_t>(r) * p.num_v_heads + h) * kD * kD;
      }
    } else {
      dst = reinterpret_cast<void*>(part == 1 ? p.write_a[r] : p.write_b[r]);
      dst_off = head_off;
      transposed = true;
    }
    if (dst != nullptr) {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int row = srow + g + (e >> 1) * 8;
          const int col = scol + 8 * nt + 2 * t + (e & 1);
          sum_st1(dst, dst_off + (transposed ? col * kD + row : row * kD + col), acc[nt][e], sum_bf16);
        }
      }
    }
  }
}

#include "gdn_chunk_tc.cuh"

int check_gdn_dims(int num_k_heads, int num_v_heads, int dk, int dv) {
  if (dk != kD || dv != kD) return VA_ERR_UNSUPPORTED;
  if (num_k_heads <= 0 || num_v_heads <= 0 || num_v_heads % num_k_heads != 0) return VA_ERR_BAD_ARG;
  return VA_OK;
}

}  // namespace

extern "C" int va_gdn_step(const VaGdnStep* a, va_stream_t stream) {
  if (a == nullptr) return VA_ERR_BAD_ARG;
  int rc = check_gdn_dims(a->num_k_heads, a->num_v_heads, a->head_k_dim, a->head_v_dim);
  if (rc != VA_OK) return rc;
  if (a->num_workers < 0 || a->depth < 0) return VA_ERR_BAD_ARG;
  if (a->num_workers == 0) return VA_OK;
  if (a->q == nullptr || a->k == nullptr || a->v == nullptr || a->g == nullptr || a->beta == nullptr ||
      a->out == nullptr || a->read_a == nullptr || a->read_b == nullptr || a->write_a == nullptr ||
      a->write_b == nullptr || (a->depth > 0 && (a->chain_a == nullptr || a->chain_b == nullptr)))
    return VA_ERR_BAD_ARG;
  StepParams p;
  p.q = static_cast<const __nv_bfloat16*>(a->q);
  p.k = static_cast<const __nv_bfloat16*>(a->k);
  p.v = static_cast<const __nv_bfloat16*>(a->v);
  p.g = a->g;
  p.beta = a->beta;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.chain_a = a->chain_a;
  p.chain_b = a->chain_b;
  p.read_a = a->read_a;
  p.read_b = a->read_b;
  p.write_a = a->write_a;
  p.write_b = a->write_b;
  p.num_workers = a->num_workers;
  p.depth = a->depth;
  p.num_k_heads = a->num_k_heads;
  p.num_v_heads = a->num_v_heads;
  p.l2_eps = a->l2_eps;
  p.q_scale = a->q_scale;
  p.status = a->status;
  // rows of q / k / v may lie inside wider rows (the conv output [q | k | v] of a layer): strides
  // in elements, 0 = dense
  p.q_row_stride = a->q_row_stride > 0 ? a->q_row_stride : static_cast<int64_t>(a->num_k_heads) * kD;
  p.k_row_stride = a->k_row_stride > 0 ? a->k_row_stride : static_cast<int64_t>(a->num_k_heads) * kD;
  p.v_row_stride = a->v_row_stride > 0 ? a->v_row_stride : static_cast<int64_t>(a->num_v_heads) * kD;
  if (p.q_row_stride < static_cast<int64_t>(a->num_k_heads) * kD || p.k_row_stride < static_cast<int64_t>(a->num_k_heads) * kD ||
      p.v_row_stride < static_cast<int64_t>(a->num_v_heads) * kD)
    return VA_ERR_BAD_ARG;
  if (a->summary_dtype != VA_SUMMARY_F32 && a->summary_dtype != VA_SUMMARY_BF16) return VA_ERR_BAD_ARG;
  dim3 grid(a->num_v_heads, a->num_workers);
  if (a->summary_dtype == VA_SUMMARY_BF16)
    gdn_step_kernel<true><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  else
    gdn_step_kernel<false><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return VA_OK;
}

extern "C" int va_gdn_compose(const int64_t* chain_a, const int64_t* chain_b, float* state,
                              int32_t num_workers, int32_t depth, int32_t num_heads, int32_t head_k_dim,
                              int32_t head_v_dim, int32_t summary_dtype, va_stream_t stream) {
  int rc = check_gdn_dims(num_heads, num_heads, head_k_dim, head_v_dim);
  if (rc != VA_OK) return rc;
  if (summary_dtype != VA_SUMMARY_F32 && summary_dtype != VA_SUMMARY_BF16) return VA_ERR_BAD_ARG;
  if (num_workers < 0 || depth < 0) return VA_ERR_BAD_ARG;
  if (num_workers == 0) return VA_OK;
  if (state == nullptr || (depth > 0 && (chain_a == nullptr || chain_b == nullptr))) return VA_ERR_BAD_ARG;
  ComposeParams p;
  p.chain_a = chain_a;
  p.chain_b = chain_b;
  p.state = state;
  p.num_workers = num_workers;
  p.depth = depth;
  p.num_heads = num_heads;
  const int smem = 3 * kD * kD * static_cast<int>(sizeof(float));
  auto kernel = summary_dtype == VA_SUMMARY_BF16 ? gdn_compose_kernel<true> : gdn_compose_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  dim3 grid(num_heads, num_workers);
  kernel<<<grid, 256, smem, static_cast<cudaStream_t>(stream)>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return VA_OK;
}

extern "C" int64_t va_gdn_prefill_scratch_bytes(int64_t num_tokens, int32_t num_v_heads) {
  if (num_tokens <= 0 || num_v_heads <= 0) return 0;
  const int64_t hn = num_tokens * num_v_heads;
  return hn * (4 * kD * 2 + kC * 2 + 2 * 4);   // K, Q, -W, U rows, P row, e^gc, e^(gc_last-gc)
}

extern "C" int va_gdn_prefill(const VaGdnPrefill* a, va_stream_t stream) {
  if (a == nullptr) return VA_ERR_BAD_ARG;
  int rc = check_gdn_dims(a->num_k_heads, a->num_v_heads, a->head_k_dim, a->head_v_dim);
  if (rc != VA_OK) return rc;
  if (a->num_requests < 0) return VA_ERR_BAD_ARG;
  if (a->num_requests == 0) return VA_OK;
  if (a->q == nullptr || a->k == nullptr || a->v == nullptr || a->g == nullptr || a->beta == nullptr ||
      a->out == nullptr || a->seg_off == nullptr || a->init_a == nullptr || a->init_b == nullptr ||
      a->write_a == nullptr || a->write_b == nullptr)
    return VA_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k) |
       reinterpret_cast<uintptr_t>(a->v)) & 7)
    return VA_ERR_BAD_ARG;
  ScanParams p;
  p.q = static_cast<const __nv_bfloat16*>(a->q);
  p.k = static_cast<const __nv_bfloat16*>(a->k);
  p.v = static_cast<const __nv_bfloat16*>(a->v);
  p.g = a->g;
  p.beta = a->beta;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.seg_off = a->seg_off;
  p.state0 = a->state0;
  p.init_a = a->init_a;
  p.init_b = a->init_b;
  p.write_a = a->write_a;
  p.write_b = a->write_b;
  p.final_state = a->final_state;
  p.num_requests = a->num_requests;
  p.num_k_heads = a->num_k_heads;
  p.num_v_heads = a->num_v_heads;
  p.l2_eps = a->l2_eps;
  p.q_scale = a->q_scale;
  p.s_k = p.s_q = p.s_w = p.s_u = p.s_p = nullptr;
  p.s_eg = p.s_ed = nullptr;
  p.num_tokens = 0;
  if (a->summary_dtype != VA_SUMMARY_F32 && a->summary_dtype != VA_SUMMARY_BF16) return VA_ERR_BAD_ARG;
  p.summary_bf16 = a->summary_dtype == VA_SUMMARY_BF16;
  p.status = a->status;
  dim3 grid(3, a->num_v_heads, a->num_requests);
  cudaError_t e;
  const bool chunked = a->engine == VA_GDN_ENGINE_CHUNK || a->engine == VA_GDN_ENGINE_CHUNK_TC;
  if (chunked && a->scratch != nullptr) {
    // two passes: the state-independent half of every chunk in parallel, then the states in order
    if (a->num_tokens <= 0 || a->scratch_bytes < va_gdn_prefill_scratch_bytes(a->num_tokens, a->num_v_heads) ||
        (reinterpret_cast<uintptr_t>(a->scratch) & 15))
      return VA_ERR_BAD_ARG;
    // the rows of q / k / v are fetched as 16-byte pieces
    if ((reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k) | reinterpret_cast<uintptr_t>(a->v)) & 15)
      return VA_ERR_BAD_ARG;
    const int64_t hn = static_cast<int64_t>(a->num_v_heads) * a->num_tokens;
    __nv_bfloat16* base = static_cast<__nv_bfloat16*>(a->scratch);
    p.s_k = base;
    p.s_q = base + hn * kD;
    p.s_w = base + 2 * hn * kD;
    p.s_u = base + 3 * hn * kD;
    p.s_p = base + 4 * hn * kD;
    p.s_eg = reinterpret_cast<float*>(base + 4 * hn * kD + hn * kC);
    p.s_ed = p.s_eg + hn;
    p.num_tokens = a->num_tokens;
    const int64_t longest = a->max_segment_tokens > 0 ? a->max_segment_tokens : a->num_tokens;
    dim3 pre_grid(static_cast<unsigned>((longest + kC - 1) / kC), a->num_v_heads, a->num_requests);
    e = cudaFuncSetAttribute(gdn_chunk_pre_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PreSmem::kTotal);
    if (e != cudaSuccess) return va_host::note_cuda_error(e);
    e = cudaFuncSetAttribute(gdn_chunk_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, StateSmem::kTotal);
    if (e != cudaSuccess) return va_host::note_cuda_error(e);
    e = cudaFuncSetAttribute(gdn_chunk_state_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TcStateSmem::kTotal);
    if (e != cudaSuccess) return va_host::note_cuda_error(e);
    gdn_chunk_pre_kernel<<<pre_grid, 128, PreSmem::kTotal, static_cast<cudaStream_t>(stream)>>>(p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return va_host::note_cuda_error(e);
    if (a->engine == VA_GDN_ENGINE_CHUNK_TC)
      gdn_chunk_state_tc_kernel<<<grid, kTcStateThreads, TcStateSmem::kTotal, static_cast<cudaStream_t>(stream)>>>(p);
    else
      gdn_chunk_state_kernel<<<grid, kStateThreads, StateSmem::kTotal, static_cast<cudaStream_t>(stream)>>>(p);
  } else if (chunked) {
    return VA_ERR_BAD_ARG;   // the chunk engine needs its scratch
  } else if (a->engine == VA_GDN_ENGINE_SCAN) {
    gdn_scan_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(p);
  } else {
    return VA_ERR_BAD_ARG;
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return VA_OK;
}
