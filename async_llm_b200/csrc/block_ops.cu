// Block merge / append on the device: the KV part and the recurrent-state part.
//
// va_block_copy replaces SharedCacheSession._copy_slots followed by _shift_keys_
// (shared_cache/session.py:489-528): the reference loops over the layers in Python and runs, per
// layer, index_select + index_copy_ for K and for V, then index_select + _rope (fp32) + index_copy_
// for the keys of the right-hand block.  Here one launch covers every layer: a CTA per (group of tokens,
// layer) reads the K and V rows of the source slot once, rotates the key by the left block's span
// when the token belongs to the right-hand block, and writes the destination slot once.
//
// va_gdn_compose_pairs replaces the per-layer compose_gdn_affines calls of _finish_block_merge
// (shared_cache/session.py:441-462, shared_cache/gdn_affine.py:104-127): A = A1 A2,
// B = B1 A2 + B2 for every (layer, head) in one launch.
#include "common.cuh"

namespace {

using namespace va;

struct CopyParams {
  __nv_bfloat16* k_pool;   // layer 0
  __nv_bfloat16* v_pool;
  int64_t layer_stride;    // elements between consecutive layers of either pool
  int64_t num_slots;
  int32_t row_elems;       // kv heads * head_dim
  int32_t head_dim;
  int32_t rotary_dim;
  int32_t max_pos;
  const float* cos_sin;
  const int32_t* src_slots;
  const int32_t* dst_slots;
  int32_t n;
  int32_t shift_begin;     // tokens [shift_begin, n) get their key rotated by `shift`
  int32_t shift;
  int32_t* status;
};

constexpr int kCopyTokens = 8;    // tokens of one CTA
constexpr int kCopyThreads = 256;
constexpr int kCopyUnroll = 4;    // 16-byte pieces a thread has in flight (8 measured slower)

// Eight consecutive elements [d, d + 8) of one head's key, rotated.  Same arithmetic as
// rope_element, on whole 16-byte pieces: needs rotary_dim % 16 == 0 so that a piece never straddles
// the two halves of the rotation.
__device__ __forceinline__ uint4 rotate_piece(const __nv_bfloat16* head, int d, int rotary_dim,
                                              const float* cs, bool neg) {
  const uint4 own = *reinterpret_cast<const uint4*>(head + d);
  if (d >= rotary_dim) return own;
  const int half = rotary_dim >> 1;
  const bool lo = d < half;
  const int f = lo ? d : d - half;   // frequency index of element d
  const uint4 oth = *reinterpret_cast<const uint4*>(head + (lo ? d + half : d - half));
  const float4 c0 = *reinterpret_cast<const float4*>(cs + f), c1 = *reinterpret_cast<const float4*>(cs + f + 4);
  const float4 s0 = *reinterpret_cast<const float4*>(cs + half + f);
  const float4 s1 = *reinterpret_cast<const float4*>(cs + half + f + 4);
  const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
  const __nv_bfloat16* xo = reinterpret_cast<const __nv_bfloat16*>(&own);
  const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(&oth);
  float r[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float a = __fmul_rn(c[j], __bfloat162float(xo[j]));
    const float b = __fmul_rn(neg ? -sn[j] : sn[j], __bfloat162float(xp[j]));
    r[j] = lo ? __fsub_rn(a, b) : __fadd_rn(a, b);
  }
  return make_uint4(pack_bf16(r[0], r[1]), pack_bf16(r[2], r[3]), pack_bf16(r[4], r[5]), pack_bf16(r[6], r[7]));
}

// grid = (group of kCopyTokens tokens, layer).  The CTA's work is the list of 16-byte pieces of
// its tokens' K rows and V rows; every thread keeps kCopyUnroll independent pieces in flight.
// (6 CTAs per SM: the rotation's load -> convert -> multiply chains need the extra warps to hide
// their latency; measured 5.2 TB/s against 4.0 with the 4 CTAs that 56 registers allow)
__global__ void __launch_bounds__(kCopyThreads, 6) block_copy_kernel(const __grid_constant__ CopyParams p) {
  __shared__ int s_src[kCopyTokens], s_dst[kCopyTokens];
  const int tok0 = blockIdx.x * kCopyTokens;
  const int layer = blockIdx.y;
  if (threadIdx.x < kCopyTokens) {
    const int t = tok0 + threadIdx.x;
    int src = -1, dst = -1;
    if (t < p.n) {
      src = p.src_slots[t];
      dst = p.dst_slots[t];
      if (src < 0 || src >= p.num_slots || dst < 0 || dst >= p.num_slots) {
        report(p.status, VA_DEV_BAD_PAGE);
        src = dst = -1;   // the token is skipped
      }
    }
    s_src[threadIdx.x] = src;
    s_dst[threadIdx.x] = dst;
  }
  __syncthreads();
  const int64_t base = static_cast<int64_t>(layer) * p.layer_stride;
  const int per_row = p.row_elems >> 3;    // pieces of one row
  const int per_tok = per_row * 2;         // K row, then V row
  const int total = kCopyTokens * per_tok;
  const bool vec_rotate = (p.rotary_dim & 15) == 0;
  bool neg = false;
  const float* cs = p.shift != 0 ? rope_row(p.cos_sin, p.rotary_dim, p.max_pos, p.shift, &neg) : nullptr;
  for (int first = threadIdx.x; first < total; first += kCopyThreads * kCopyUnroll) {
    uint4 val[kCopyUnroll];
    __nv_bfloat16* out[kCopyUnroll];
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) {
      out[u] = nullptr;
      const int idx = first + u * kCopyThreads;
      if (idx >= total) continue;
      const int ti = idx / per_tok;
      const int c = idx - ti * per_tok;
      const int src = s_src[ti];
      if (src < 0) continue;
      const bool is_v = c >= per_row;
      const int e = (is_v ? c - per_row : c) << 3;
      const __nv_bfloat16* pool = is_v ? p.v_pool : p.k_pool;
      const __nv_bfloat16* row = pool + base + static_cast<int64_t>(src) * p.row_elems;
      out[u] = const_cast<__nv_bfloat16*>(pool) + base + static_cast<int64_t>(s_dst[ti]) * p.row_elems + e;
      if (!is_v && cs != nullptr && tok0 + ti >= p.shift_begin) {
        // the stored bf16 key is widened, rotated in fp32 and rounded once, as the reference does
        const int h = e / p.head_dim;
        const int d = e - h * p.head_dim;
        const __nv_bfloat16* head = row + h * p.head_dim;
        if (vec_rotate) {
          val[u] = rotate_piece(head, d, p.rotary_dim, cs, neg);
        } else {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            w[j] = pack_bf16(rope_element(head, d + 2 * j, p.rotary_dim, cs, neg),
                             rope_element(head, d + 2 * j + 1, p.rotary_dim, cs, neg));
          val[u] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      } else {
        val[u] = __ldcs(reinterpret_cast<const uint4*>(row + e));   // read once
      }
    }
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u)
      if (out[u] != nullptr) __stcs(reinterpret_cast<uint4*>(out[u]), val[u]);
  }
}

// ---- pair composition ---------------------------------------------------------------------------
struct PairParams {
  const int64_t* a_first;
  const int64_t* b_first;
  const int64_t* a_second;
  const int64_t* b_second;
  const int64_t* out_a;
  const int64_t* out_b;
  int32_t num_pairs;
  int32_t heads;
  int32_t summary_bf16;   // the tensors are bf16 (fp32 otherwise); sums in fp32, one rounding per output
};

constexpr int kDim = 128;   // head_k_dim = head_v_dim
constexpr int kTile = 64;   // output tile of one CTA
constexpr int kChunk = 16;  // k-extent staged per step

// grid = (tile 0..3, head, pair * 2 + which); which 0: A = A1 A2, which 1: B = B1 A2 + B2.
// 256 threads, each a 4x4 piece of the 64x64 output tile, fp32 FMA.
__global__ void __launch_bounds__(256) gdn_compose_pairs_kernel(const __grid_constant__ PairParams p) {
  __shared__ float xs[kChunk][kTile + 1];   // left operand, transposed: xs[k][row]
  __shared__ float ys[kChunk][kTile];       // right operand: ys[k][col]
  const int tile = blockIdx.x;
  const int head = blockIdx.y;
  const int pair = blockIdx.z >> 1;
  const int which = blockIdx.z & 1;
  const int row0 = (tile >> 1) * kTile, col0 = (tile & 1) * kTile;
  const int64_t head_off = static_cast<int64_t>(head) * kDim * kDim;
  const bool bf16 = p.summary_bf16 != 0;
  const void* x = reinterpret_cast<const void*>(which ? p.b_first[pair] : p.a_first[pair]);
  const void* y = reinterpret_cast<const void*>(p.a_second[pair]);
  const void* add = which ? reinterpret_cast<const void*>(p.b_second[pair]) : nullptr;
  void* out = reinterpret_cast<void*>(which ? p.out_b[pair] : p.out_a[pair]);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < kDim; k0 += kChunk) {
    // 64 x 16 of x and 16 x 64 of y: 1024 floats each, 4 per thread
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = threadIdx.x + i * 256;
      const int xr = idx >> 4, xk = idx & 15;
      xs[xk][xr] = sum_ld1(x, head_off + static_cast<int64_t>(row0 + xr) * kDim + k0 + xk, bf16);
      const int yk = idx >> 6, yc = idx & 63;
      ys[yk][yc] = sum_ld1(y, head_off + static_cast<int64_t>(k0 + yk) * kDim + col0 + yc, bf16);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kChunk; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ys[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t o = head_off + static_cast<int64_t>(row0 + ty * 4 + i) * kDim + col0 + tx * 4;
    float4 r = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    if (add != nullptr) {
      const float4 b2 = sum_ld4(add, o, bf16);
      r.x += b2.x;
      r.y += b2.y;
      r.z += b2.z;
      r.w += b2.w;
    }
    sum_st4(out, o, r, bf16);
  }
}

}  // namespace

extern "C" int va_block_copy(const VaPool* pool, int32_t num_layers, int64_t layer_stride,
                             const int32_t* src_slots, const int32_t* dst_slots, int32_t n,
                             int32_t shift_begin, int32_t shift, int32_t* status, va_stream_t stream) {
  int rc = va_host::check_pool(pool);
  if (rc != VA_OK) return rc;
  if (n < 0 || num_layers <= 0 || num_layers > 65535 || shift_begin < 0) return VA_ERR_BAD_ARG;
  if (n == 0) return VA_OK;
  if (src_slots == nullptr || dst_slots == nullptr) return VA_ERR_BAD_ARG;
  const int64_t row_elems = static_cast<int64_t>(pool->num_kv_heads) * pool->head_dim;
  if ((pool->head_dim & 7) || (layer_stride & 7) || layer_stride < pool->num_slots * row_elems)
    return VA_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(pool->k) | reinterpret_cast<uintptr_t>(pool->v)) & 15) return VA_ERR_BAD_ARG;
  CopyParams p;
  p.k_pool = static_cast<__nv_bfloat16*>(pool->k);
  p.v_pool = static_cast<__nv_bfloat16*>(pool->v);
  p.layer_stride = layer_stride;
  p.num_slots = pool->num_slots;
  p.row_elems = static_cast<int32_t>(row_elems);
  p.head_dim = pool->head_dim;
  p.rotary_dim = pool->rotary_dim;
  p.max_pos = pool->max_pos;
  p.cos_sin = pool->cos_sin;
  p.src_slots = src_slots;
  p.dst_slots = dst_slots;
  p.n = n;
  p.shift_begin = shift_begin;
  p.shift = shift;
  p.status = status;
  block_copy_kernel<<<dim3((n + kCopyTokens - 1) / kCopyTokens, num_layers), kCopyThreads, 0,
                      static_cast<cudaStream_t>(stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return VA_OK;
}

extern "C" int va_gdn_compose_pairs(const int64_t* a_first, const int64_t* b_first, const int64_t* a_second,
                                    const int64_t* b_second, const int64_t* out_a, const int64_t* out_b,
                                    int32_t num_pairs, int32_t num_v_heads, int32_t head_k_dim,
                                    int32_t head_v_dim, int32_t summary_dtype, va_stream_t stream) {
  if (num_pairs < 0 || num_v_heads <= 0 || num_v_heads > 65535) return VA_ERR_BAD_ARG;
  if (summary_dtype != VA_SUMMARY_F32 && summary_dtype != VA_SUMMARY_BF16) return VA_ERR_BAD_ARG;
  if (head_k_dim != kDim || head_v_dim != kDim) return VA_ERR_UNSUPPORTED;
  if (num_pairs == 0) return VA_OK;
  if (num_pairs > 32767) return VA_ERR_CAPACITY;
  if (!a_first || !b_first || !a_second || !b_second || !out_a || !out_b) return VA_ERR_BAD_ARG;
  PairParams p{a_first, b_first, a_second, b_second, out_a, out_b, num_pairs, num_v_heads,
               summary_dtype == VA_SUMMARY_BF16 ? 1 : 0};
  gdn_compose_pairs_kernel<<<dim3(4, num_v_heads, num_pairs * 2), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return VA_OK;
}
