// Rotate-and-store of freshly projected keys/values, and the stand-alone RoPE delta rotation.
//
// va_store_kv replaces the three steps the reference runs per attention layer before the
// attention itself (shared_cache/attention.py:645-649): rotate K at its block-relative position
// (`_rope`, eager torch), make V contiguous, scatter both rows into the paged pool
// (kernel/csrc/jit/store.cu:25-57, one warp per token, negative slot = skip).  Here one launch
// reads the unrotated K/V rows once and writes the pool rows once.
#include "common.cuh"

namespace {

using namespace va;

struct StoreParams {
  __nv_bfloat16* k_pool;
  __nv_bfloat16* v_pool;
  int64_t num_slots;
  int32_t heads;
  int32_t head_dim;
  int32_t rotary_dim;
  int32_t max_pos;
  const float* cos_sin;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  int64_t k_row_stride;
  int64_t v_row_stride;
  const int32_t* positions;
  const int32_t* out_loc;
  int32_t n;
  int32_t* status;
};

// grid.x = token, threads stride over the row's heads*head_dim elements (pairs of bf16).
__global__ void __launch_bounds__(256) store_kv_kernel(const __grid_constant__ StoreParams p) {
  // a kernel launched behind this one as a programmatic dependent (the streaming pass of a decode
  // step) may become resident now; it waits for this grid to complete before it reads the pools
  pdl_launch_dependents();
  const int tok = blockIdx.x;
  if (tok >= p.n) return;
  const int slot = p.out_loc[tok];
  if (slot < 0) return;  // inactive (padding) row
  if (slot >= p.num_slots) {
    if (threadIdx.x == 0) report(p.status, VA_DEV_BAD_PAGE);
    return;
  }
  const int row_elems = p.heads * p.head_dim;
  const __nv_bfloat16* ksrc = p.k + static_cast<int64_t>(tok) * p.k_row_stride;
  const __nv_bfloat16* vsrc = p.v + static_cast<int64_t>(tok) * p.v_row_stride;
  __nv_bfloat16* kdst = p.k_pool + static_cast<int64_t>(slot) * row_elems;
  __nv_bfloat16* vdst = p.v_pool + static_cast<int64_t>(slot) * row_elems;
  bool neg = false;
  const float* cs = nullptr;
  if (p.positions != nullptr) cs = rope_row(p.cos_sin, p.rotary_dim, p.max_pos, p.positions[tok], &neg);
  for (int e = threadIdx.x * 2; e < row_elems; e += blockDim.x * 2) {
    const int h = e / p.head_dim;
    const int d = e - h * p.head_dim;
    __nv_bfloat162 kk;
    if (cs != nullptr) {
      const __nv_bfloat16* head = ksrc + h * p.head_dim;
      kk = __floats2bfloat162_rn(rope_element(head, d, p.rotary_dim, cs, neg),
                                 rope_element(head, d + 1, p.rotary_dim, cs, neg));
    } else {
      kk = *reinterpret_cast<const __nv_bfloat162*>(ksrc + e);
    }
    *reinterpret_cast<__nv_bfloat162*>(kdst + e) = kk;
    *reinterpret_cast<__nv_bfloat162*>(vdst + e) = *reinterpret_cast<const __nv_bfloat162*>(vsrc + e);
  }
}

// grid.x = row; rotates x[n, heads, head_dim] by delta[n].  Each thread owns whole rotation pairs
// (d, d + rotary_dim/2): it reads both elements before writing either, so out may alias x.
__global__ void __launch_bounds__(256) rope_rotate_kernel(const __nv_bfloat16* x, __nv_bfloat16* out,
                                                          const int32_t* delta, int n, int heads,
                                                          int head_dim, int rotary_dim,
                                                          const float* cos_sin, int max_pos) {
  const int row = blockIdx.x;
  if (row >= n) return;
  bool neg;
  const float* cs = rope_row(cos_sin, rotary_dim, max_pos, delta[row], &neg);
  const int half = rotary_dim >> 1;
  const int pairs = head_dim >> 1;
  const __nv_bfloat16* src = x + static_cast<int64_t>(row) * heads * head_dim;
  __nv_bfloat16* dst = out + static_cast<int64_t>(row) * heads * head_dim;
  for (int idx = threadIdx.x; idx < heads * pairs; idx += blockDim.x) {
    const int h = idx / pairs;
    const int j = idx - h * pairs;
    const __nv_bfloat16* head = src + h * head_dim;
    __nv_bfloat16* ohead = dst + h * head_dim;
    if (j < half) {
      const float lo = rope_element(head, j, rotary_dim, cs, neg);
      const float hi = rope_element(head, j + half, rotary_dim, cs, neg);
      ohead[j] = __float2bfloat16_rn(lo);
      ohead[j + half] = __float2bfloat16_rn(hi);
    } else {
      const int d = rotary_dim + 2 * (j - half);
      const __nv_bfloat16 a = head[d], b = head[d + 1];
      ohead[d] = a;
      ohead[d + 1] = b;
    }
  }
}

// ---- interleaved 3-axis mRoPE ---------------------------------------------------------------------
// Restates SharedCacheAttention._rope_mrope (shared_cache/attention.py:257-280) for bf16 rows:
// frequency f of the rotary half takes its position from axis 1 (height) when f % 3 == 1 and
// f < 3 * section[1], from axis 2 (width) when f % 3 == 2 and f < 3 * section[2], else from axis 0
// (time); cos and sin are rounded to bf16 and the two products and their sum are each rounded to
// bf16, as the reference's bf16 tensor arithmetic does.  The table row of position p holds
// cos / sin of p * inv_freq in fp32, which is what the reference computes on the fly.
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ void mrope_pair(const __nv_bfloat16* head, __nv_bfloat16* ohead, int f, int half,
                                           int rotary_dim, const float* cos_sin, int max_pos, int p_t,
                                           int p_h, int p_w, int lim_h, int lim_w) {
  const int r = f % 3;
  const int pos = (r == 1 && f < lim_h) ? p_h : ((r == 2 && f < lim_w) ? p_w : p_t);
  int a = pos < 0 ? -pos : pos;
  a = a > max_pos - 1 ? max_pos - 1 : a;
  const float* row = cos_sin + static_cast<int64_t>(a) * rotary_dim;
  const float c = bf16_round(row[f]);
  float sn = bf16_round(row[half + f]);
  sn = pos < 0 ? -sn : sn;
  const float x1 = __bfloat162float(head[f]), x2 = __bfloat162float(head[f + half]);
  ohead[f] = __float2bfloat16_rn(__fadd_rn(bf16_round(__fmul_rn(x1, c)), bf16_round(__fmul_rn(-x2, sn))));
  ohead[f + half] = __float2bfloat16_rn(__fadd_rn(bf16_round(__fmul_rn(x2, c)), bf16_round(__fmul_rn(x1, sn))));
}

struct MropeParams {
  const __nv_bfloat16* x;      // [n, heads*head_dim] rows, row stride x_stride
  int64_t x_stride;
  __nv_bfloat16* out;          // rotate: [n, heads*head_dim]; store: the K pool
  const __nv_bfloat16* v;      // store only
  int64_t v_stride;
  __nv_bfloat16* v_pool;       // store only
  const int32_t* out_loc;      // store only: slot per row (negative = skip); NULL = row index
  int64_t num_slots;
  const int32_t* pos;          // [axes, n]
  int32_t axes;                // 1 or 3
  int32_t n, heads, head_dim, rotary_dim, max_pos, lim_h, lim_w;
  const float* cos_sin;
  int32_t* status;
};

// grid.x = row.  Each thread owns whole rotation pairs (f, f + rotary_dim/2) and reads both elements
// before it writes either, so `out` may alias `x` in the rotate form.
__global__ void __launch_bounds__(256) mrope_kernel(const __grid_constant__ MropeParams p) {
  const int row = blockIdx.x;
  if (row >= p.n) return;
  int64_t dst_row = row;
  if (p.out_loc != nullptr) {
    const int slot = p.out_loc[row];
    if (slot < 0) return;
    if (slot >= p.num_slots) {
      if (threadIdx.x == 0) report(p.status, VA_DEV_BAD_PAGE);
      return;
    }
    dst_row = slot;
  }
  const int p_t = p.pos[row];
  const int p_h = p.axes == 3 ? p.pos[p.n + row] : p_t;
  const int p_w = p.axes == 3 ? p.pos[2 * p.n + row] : p_t;
  const int half = p.rotary_dim >> 1;
  const int pairs = p.head_dim >> 1;
  const int row_elems = p.heads * p.head_dim;
  const __nv_bfloat16* src = p.x + static_cast<int64_t>(row) * p.x_stride;
  __nv_bfloat16* dst = p.out + dst_row * row_elems;
  for (int idx = threadIdx.x; idx < p.heads * pairs; idx += blockDim.x) {
    const int h = idx / pairs;
    const int j = idx - h * pairs;
    const __nv_bfloat16* head = src + h * p.head_dim;
    __nv_bfloat16* ohead = dst + h * p.head_dim;
    if (j < half) {
      mrope_pair(head, ohead, j, half, p.rotary_dim, p.cos_sin, p.max_pos, p_t, p_h, p_w, p.lim_h, p.lim_w);
    } else {
      const int d = p.rotary_dim + 2 * (j - half);
      const __nv_bfloat16 a = head[d], b = head[d + 1];
      ohead[d] = a;
      ohead[d + 1] = b;
    }
  }
  if (p.v != nullptr) {
    const __nv_bfloat16* vsrc = p.v + static_cast<int64_t>(row) * p.v_stride;
    __nv_bfloat16* vdst = p.v_pool + dst_row * row_elems;
    for (int e = threadIdx.x * 2; e < row_elems; e += blockDim.x * 2)
      *reinterpret_cast<__nv_bfloat162*>(vdst + e) = *reinterpret_cast<const __nv_bfloat162*>(vsrc + e);
  }
}

}  // namespace

extern "C" int va_store_kv(const VaPool* pool, const void* k, int64_t k_row_stride, const void* v,
                           int64_t v_row_stride, const int32_t* positions, const int32_t* out_loc,
                           int32_t n, int32_t* status, va_stream_t stream) {
  int rc = va_host::check_pool(pool);
  if (rc != VA_OK) return rc;
  if (n < 0) return VA_ERR_BAD_ARG;
  if (n == 0) return VA_OK;
  if (k == nullptr || v == nullptr || out_loc == nullptr) return VA_ERR_BAD_ARG;
  if ((k_row_stride & 1) || (v_row_stride & 1)) return VA_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 3) return VA_ERR_BAD_ARG;
  StoreParams p;
  p.k_pool = static_cast<__nv_bfloat16*>(pool->k);
  p.v_pool = static_cast<__nv_bfloat16*>(pool->v);
  p.num_slots = pool->num_slots;
  p.heads = pool->num_kv_heads;
  p.head_dim = pool->head_dim;
  p.rotary_dim = pool->rotary_dim;
  p.max_pos = pool->max_pos;
  p.cos_sin = pool->cos_sin;
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.k_row_stride = k_row_stride;
  p.v_row_stride = v_row_stride;
  p.positions = positions;
  p.out_loc = out_loc;
  p.n = n;
  p.status = status;
  store_kv_kernel<<<n, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return VA_OK;
}

extern "C" int va_rope_rotate(const void* x, void* out, const int32_t* delta, int32_t n,
                              int32_t heads, int32_t head_dim, int32_t rotary_dim,
                              const float* cos_sin, int32_t max_pos, va_stream_t stream) {
  if (n < 0 || heads <= 0 || head_dim <= 0 || rotary_dim <= 0 || rotary_dim > head_dim ||
      (rotary_dim & 1) || max_pos <= 0)
    return VA_ERR_BAD_ARG;
  if (n == 0) return VA_OK;
  if (x == nullptr || out == nullptr || delta == nullptr || cos_sin == nullptr) return VA_ERR_BAD_ARG;
  if (head_dim & 1) return VA_ERR_BAD_ARG;
  rope_rotate_kernel<<<n, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), delta, n, heads,
      head_dim, rotary_dim, cos_sin, max_pos);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return VA_OK;
}

extern "C" int va_mrope_rotate(const void* x, void* out, const int32_t* pos, int32_t pos_axes, int32_t n,
                               int32_t heads, int32_t head_dim, int32_t rotary_dim, const float* cos_sin,
                               int32_t max_pos, int32_t lim_h, int32_t lim_w, va_stream_t stream) {
  if (n < 0 || heads <= 0 || head_dim <= 0 || (head_dim & 1) || rotary_dim <= 0 || rotary_dim > head_dim ||
      (rotary_dim & 1) || max_pos <= 0 || (pos_axes != 1 && pos_axes != 3) || lim_h < 0 || lim_w < 0)
    return VA_ERR_BAD_ARG;
  if (n == 0) return VA_OK;
  if (x == nullptr || out == nullptr || pos == nullptr || cos_sin == nullptr) return VA_ERR_BAD_ARG;
  MropeParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.x_stride = static_cast<int64_t>(heads) * head_dim;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.pos = pos;
  p.axes = pos_axes;
  p.n = n;
  p.heads = heads;
  p.head_dim = head_dim;
  p.rotary_dim = rotary_dim;
  p.max_pos = max_pos;
  p.lim_h = lim_h;
  p.lim_w = lim_w;
  p.cos_sin = cos_sin;
  mrope_kernel<<<n, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return VA_OK;
}

extern "C" int va_store_kv_mrope(const VaPool* pool, const void* k, int64_t k_row_stride, const void* v,
                                 int64_t v_row_stride, const int32_t* pos, int32_t pos_axes,
                                 const int32_t* out_loc, int32_t n, int32_t lim_h, int32_t lim_w,
                                 int32_t* status, va_stream_t stream) {
  int rc = va_host::check_pool(pool);
  if (rc != VA_OK) return rc;
  if (n < 0 || (pos_axes != 1 && pos_axes != 3) || lim_h < 0 || lim_w < 0) return VA_ERR_BAD_ARG;
  if (n == 0) return VA_OK;
  if (k == nullptr || v == nullptr || out_loc == nullptr || pos == nullptr) return VA_ERR_BAD_ARG;
  if ((k_row_stride & 1) || (v_row_stride & 1)) return VA_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 3) return VA_ERR_BAD_ARG;
  MropeParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(k);
  p.x_stride = k_row_stride;
  p.out = static_cast<__nv_bfloat16*>(pool->k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.v_stride = v_row_stride;
  p.v_pool = static_cast<__nv_bfloat16*>(pool->v);
  p.out_loc = out_loc;
  p.num_slots = pool->num_slots;
  p.pos = pos;
  p.axes = pos_axes;
  p.n = n;
  p.heads = pool->num_kv_heads;
  p.head_dim = pool->head_dim;
  p.rotary_dim = pool->rotary_dim;
  p.max_pos = pool->max_pos;
  p.lim_h = lim_h;
  p.lim_w = lim_w;
  p.cos_sin = pool->cos_sin;
  p.status = status;
  mrope_kernel<<<n, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return VA_OK;
}
