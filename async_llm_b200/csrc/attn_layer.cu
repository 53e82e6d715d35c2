// Elementwise steps of the gated full-attention layer either side of the view attention (sm_100a):
// per-head RMSNorm of the queries and keys straight out of the fused qkv projection, and the sigmoid
// output gate.  Each is one launch over rows that the projection GEMM has just written (L2 resident).
#include "common.cuh"

namespace {

using namespace va;

struct QkNormParams {
  const __nv_bfloat16* qkv;   // [n, (2*Hq + 2*Hkv) * D] rows: per query head [q | gate], then k heads, then v heads
  int64_t qkv_row_stride;
  const float* q_weight;      // [D]
  const float* k_weight;      // [D]
  __nv_bfloat16* q_out;       // [n, Hq * D]
  __nv_bfloat16* k_out;       // [n, Hkv * D]
  int32_t n, num_q_heads, num_kv_heads;
  float eps;
  float weight_offset;        // 1 for the (1 + weight) form, else 0
};

// One warp per (row, head) over the Hq query heads and the Hkv key heads of a row:
//     y = x * rsqrt(mean(x^2) + eps) * (offset + w), fp32 inside, one rounding to bf16.
template <int D>
__global__ void __launch_bounds__(256) attn_qk_norm_kernel(const __grid_constant__ QkNormParams p) {
  constexpr int VEC = D / 32;   // elements per lane: 4 or 8
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int heads = p.num_q_heads + p.num_kv_heads;
  if (warp_global >= static_cast<int64_t>(p.n) * heads) return;
  const int row = static_cast<int>(warp_global / heads);
  const int h = static_cast<int>(warp_global - static_cast<int64_t>(row) * heads);
  const bool is_q = h < p.num_q_heads;
  const __nv_bfloat16* src = p.qkv + static_cast<int64_t>(row) * p.qkv_row_stride +
                             (is_q ? static_cast<int64_t>(h) * 2 * D
                                   : static_cast<int64_t>(p.num_q_heads) * 2 * D + static_cast<int64_t>(h - p.num_q_heads) * D);
  const float* w = is_q ? p.q_weight : p.k_weight;
  __nv_bfloat16* dst = is_q ? p.q_out + (static_cast<int64_t>(row) * p.num_q_heads + h) * D
                            : p.k_out + (static_cast<int64_t>(row) * p.num_kv_heads + (h - p.num_q_heads)) * D;
  float x[VEC];
  if constexpr (VEC == 8) {
    const uint4 raw = *reinterpret_cast<const uint4*>(src + lane * 8);
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = __bfloat162float(e[i]);
  } else {
    const uint2 raw = *reinterpret_cast<const uint2*>(src + lane * 4);
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = __bfloat162float(e[i]);
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) ss += x[i] * x[i];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  const float r = rsqrtf(ss / static_cast<float>(D) + p.eps);
  __nv_bfloat16 y[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) y[i] = __float2bfloat16_rn(x[i] * r * (p.weight_offset + w[lane * VEC + i]));
  if constexpr (VEC == 8) *reinterpret_cast<uint4*>(dst + lane * 8) = *reinterpret_cast<const uint4*>(y);
  else *reinterpret_cast<uint2*>(dst + lane * 4) = *reinterpret_cast<const uint2*>(y);
}

struct GateParams {
  const __nv_bfloat16* o;     // [n, Hq * D] attention output
  const __nv_bfloat16* qkv;   // the projection rows: the gate of head h sits at h * 2D + D
  int64_t qkv_row_stride;
  __nv_bfloat16* out;         // [n, Hq * D]
  int64_t total8;             // n * Hq * D / 8
  int32_t num_q_heads, head_dim;
};

// out = bf16(float(o) * sigmoid(float(gate))), eight elements per thread
__global__ void __launch_bounds__(256) attn_output_gate_kernel(const __grid_constant__ GateParams p) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= p.total8) return;
  const int per_head = p.head_dim >> 3;
  const int per_row = p.num_q_heads * per_head;
  const int64_t row = i / per_row;
  const int rem = static_cast<int>(i - row * per_row);
  const int h = rem / per_head;
  const int c = rem - h * per_head;
  const uint4 ov = *reinterpret_cast<const uint4*>(p.o + i * 8);
  const uint4 gv = *reinterpret_cast<const uint4*>(p.qkv + row * p.qkv_row_stride +
                                                   static_cast<int64_t>(h) * 2 * p.head_dim + p.head_dim + c * 8);
  const __nv_bfloat16* oe = reinterpret_cast<const __nv_bfloat16*>(&ov);
  const __nv_bfloat16* ge = reinterpret_cast<const __nv_bfloat16*>(&gv);
  __nv_bfloat16 y[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float g = __bfloat162float(ge[k]);
    y[k] = __float2bfloat16_rn(__bfloat162float(oe[k]) * (1.0f / (1.0f + expf(-g))));
  }
  *reinterpret_cast<uint4*>(p.out + i * 8) = *reinterpret_cast<const uint4*>(y);
}

}  // namespace

extern "C" int va_attn_qk_norm(const VaAttnQkNorm* a, va_stream_t stream) {
  if (a == nullptr || a->n < 0 || a->num_q_heads <= 0 || a->num_kv_heads <= 0) return VA_ERR_BAD_ARG;
  if (a->head_dim != 128 && a->head_dim != 256) return VA_ERR_UNSUPPORTED;
  if (a->n == 0) return VA_OK;
  if (!a->qkv || !a->q_weight || !a->k_weight || !a->q_out || !a->k_out) return VA_ERR_BAD_ARG;
  const int64_t width = static_cast<int64_t>(2 * a->num_q_heads + 2 * a->num_kv_heads) * a->head_dim;
  if (a->qkv_row_stride < width || (a->qkv_row_stride & 7)) return VA_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(a->qkv) | reinterpret_cast<uintptr_t>(a->q_out) |
       reinterpret_cast<uintptr_t>(a->k_out)) & 15)
    return VA_ERR_BAD_ARG;
  QkNormParams p;
  p.qkv = static_cast<const __nv_bfloat16*>(a->qkv);
  p.qkv_row_stride = a->qkv_row_stride;
  p.q_weight = a->q_weight;
  p.k_weight = a->k_weight;
  p.q_out = static_cast<__nv_bfloat16*>(a->q_out);
  p.k_out = static_cast<__nv_bfloat16*>(a->k_out);
  p.n = a->n;
  p.num_q_heads = a->num_q_heads;
  p.num_kv_heads = a->num_kv_heads;
  p.eps = a->eps;
  p.weight_offset = a->weight_plus_one ? 1.0f : 0.0f;
  const int64_t warps = static_cast<int64_t>(a->n) * (a->num_q_heads + a->num_kv_heads);
  const int64_t blocks = (warps + 7) / 8;
  if (blocks > 0x7fffffffLL) return VA_ERR_CAPACITY;
  if (a->head_dim == 256)
    attn_qk_norm_kernel<256><<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  else
    attn_qk_norm_kernel<128><<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return VA_OK;
}

extern "C" int va_attn_output_gate(const void* o, const void* qkv, int64_t qkv_row_stride, void* out, int32_t n,
                                   int32_t num_q_heads, int32_t head_dim, va_stream_t stream) {
  if (n < 0 || num_q_heads <= 0 || head_dim <= 0 || (head_dim & 7)) return VA_ERR_BAD_ARG;
  if (n == 0) return VA_OK;
  if (!o || !qkv || !out) return VA_ERR_BAD_ARG;
  if (qkv_row_stride < static_cast<int64_t>(2) * num_q_heads * head_dim || (qkv_row_stride & 7)) return VA_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(out)) & 15)
    return VA_ERR_BAD_ARG;
  GateParams p;
  p.o = static_cast<const __nv_bfloat16*>(o);
  p.qkv = static_cast<const __nv_bfloat16*>(qkv);
  p.qkv_row_stride = qkv_row_stride;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.total8 = static_cast<int64_t>(n) * num_q_heads * head_dim / 8;
  p.num_q_heads = num_q_heads;
  p.head_dim = head_dim;
  const int64_t blocks = (p.total8 + 255) / 256;
  if (blocks > 0x7fffffffLL) return VA_ERR_CAPACITY;
  attn_output_gate_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return VA_OK;
}
