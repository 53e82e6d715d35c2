// Elementwise glue of a decoder layer around the attention / GDN steps (sm_100a): the fused residual
// add + RMSNorm between sub-layers and the SwiGLU gate of the MLP.  The reference calls FlashInfer's
// `fused_add_rmsnorm` / `gemma_fused_add_rmsnorm` (layers/norm.py:25-43) and `silu_and_mul`
// (layers/activation.py:9-12) here; a decode step runs each of them once per sub-layer on rows the
// GEMM before has just written (L2 resident), so each is one short launch.
#include "common.cuh"

namespace {

using namespace va;

// One CTA per row.  residual <- residual + delta (fp32 sum, stored as bf16); out <- the fp32 sum
// * rsqrt(mean(sum^2) + eps) * (offset + weight), one rounding.  delta == nullptr: no add (plain norm).
__global__ void __launch_bounds__(512) add_rmsnorm_kernel(__nv_bfloat16* residual, const __nv_bfloat16* delta,
                                                          const __nv_bfloat16* weight, __nv_bfloat16* out, int dim,
                                                          float eps, float weight_offset) {
  __shared__ float red[16];
  const int64_t row = blockIdx.x;
  __nv_bfloat16* r = residual + row * dim;
  const __nv_bfloat16* d = delta != nullptr ? delta + row * dim : nullptr;
  constexpr int kMaxPer = 4;            // 8-element pieces per thread: dim <= 512 * 8 * 4
  float x[kMaxPer][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxPer; ++i) {
    const int c = (i * 512 + threadIdx.x) * 8;
    if (c < dim) {
      const uint4 rv = *reinterpret_cast<const uint4*>(r + c);
      const __nv_bfloat16* re = reinterpret_cast<const __nv_bfloat16*>(&rv);
      if (d != nullptr) {
        const uint4 dv = *reinterpret_cast<const uint4*>(d + c);
        const __nv_bfloat16* de = reinterpret_cast<const __nv_bfloat16*>(&dv);
        uint4 sv;
        __nv_bfloat16* se = reinterpret_cast<__nv_bfloat16*>(&sv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          x[i][j] = __bfloat162float(re[j]) + __bfloat162float(de[j]);
          se[j] = __float2bfloat16_rn(x[i][j]);
        }
        *reinterpret_cast<uint4*>(r + c) = sv;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) x[i][j] = __bfloat162float(re[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += x[i][j] * x[i][j];
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < 16; ++w) total += red[w];
  const float inv = rsqrtf(total / static_cast<float>(dim) + eps);
  __nv_bfloat16* o = out + row * dim;
#pragma unroll
  for (int i = 0; i < kMaxPer; ++i) {
    const int c = (i * 512 + threadIdx.x) * 8;
    if (c < dim) {
      const uint4 wv = *reinterpret_cast<const uint4*>(weight + c);
      const __nv_bfloat16* we = reinterpret_cast<const __nv_bfloat16*>(&wv);
      uint4 ov;
      __nv_bfloat16* oe = reinterpret_cast<__nv_bfloat16*>(&ov);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        oe[j] = __float2bfloat16_rn(x[i][j] * inv * (weight_offset + __bfloat162float(we[j])));
      *reinterpret_cast<uint4*>(o + c) = ov;
    }
  }
}

// out[r, c] = bf16(silu(gate[r, c]) * up[r, c]) with gate = the first `inter` columns of a row of
// `gate_up`, up = the next `inter`; fp32 inside, one rounding.
__global__ void __launch_bounds__(256) silu_mul_kernel(const __nv_bfloat16* gate_up, int64_t row_stride,
                                                       __nv_bfloat16* out, int n, int inter) {
  const int per_row = inter >> 3;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(n) * per_row) return;
  const int row = static_cast<int>(idx / per_row);
  const int c = static_cast<int>(idx - static_cast<int64_t>(row) * per_row) * 8;
  const __nv_bfloat16* g = gate_up + static_cast<int64_t>(row) * row_stride + c;
  const uint4 gv = *reinterpret_cast<const uint4*>(g);
  const uint4 uv = *reinterpret_cast<const uint4*>(g + inter);
  const __nv_bfloat16* ge = reinterpret_cast<const __nv_bfloat16*>(&gv);
  const __nv_bfloat16* ue = reinterpret_cast<const __nv_bfloat16*>(&uv);
  uint4 ov;
  __nv_bfloat16* oe = reinterpret_cast<__nv_bfloat16*>(&ov);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float x = __bfloat162float(ge[j]);
    oe[j] = __float2bfloat16_rn(x / (1.0f + __expf(-x)) * __bfloat162float(ue[j]));
  }
  *reinterpret_cast<uint4*>(out + static_cast<int64_t>(row) * inter + c) = ov;
}

}  // namespace

extern "C" int va_add_rmsnorm(void* residual, const void* delta, const void* weight, void* out, int32_t n,
                              int32_t dim, float eps, int32_t weight_plus_one, va_stream_t stream) {
  if (n < 0 || dim <= 0 || (dim & 7) || dim > 512 * 8 * 4) return VA_ERR_BAD_ARG;
  if (n == 0) return VA_OK;
  if (!residual || !weight || !out) return VA_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(weight) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return VA_ERR_BAD_ARG;
  add_rmsnorm_kernel<<<n, 512, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(delta),
      static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(out), dim, eps, weight_plus_one ? 1.f : 0.f);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return VA_OK;
}

extern "C" int va_silu_mul(const void* gate_up, int64_t row_stride, void* out, int32_t n, int32_t inter,
                           va_stream_t stream) {
  if (n < 0 || inter <= 0 || (inter & 7) || row_stride < 2 * static_cast<int64_t>(inter) || (row_stride & 7))
    return VA_ERR_BAD_ARG;
  if (n == 0) return VA_OK;
  if (!gate_up || !out) return VA_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) & 15) return VA_ERR_BAD_ARG;
  const int64_t work = static_cast<int64_t>(n) * (inter >> 3);
  const int64_t blocks = (work + 255) / 256;
  if (blocks > 0x7fffffffLL) return VA_ERR_CAPACITY;
  silu_mul_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gate_up), row_stride, static_cast<__nv_bfloat16*>(out), n, inter);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return VA_OK;
}
