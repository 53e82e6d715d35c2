// Shared device helpers for the sm_100a cache-view kernels: PTX wrappers (cp.async, ldmatrix,
// mma.sync, movmatrix), bf16 packing, the RoPE delta rotation and the status word.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/view_attn_b200.h"

namespace va {

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte async copy global -> shared; src_bytes = 0 zero-fills the destination.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src),
               "r"(src_bytes)
               : "memory");
}
// L2 eviction policies for data that is read once (streamed K/V) or re-read by other CTAs
// (a shared block's K/V under dense tiles)
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;\n" : "=l"(p));
  return p;
}
__device__ __forceinline__ void cp_async16_hint(uint32_t dst, const void* src, int src_bytes, uint64_t policy) {
  asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;\n" ::"r"(dst), "l"(src),
               "r"(src_bytes), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// ---- mbarrier + bulk (TMA) copies -------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
// generic-proxy accesses to shared memory before this point are ordered before later async-proxy
// (bulk copy) accesses
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// try_wait that lets the hardware park the thread for up to `ns` nanoseconds before it reports
// "not yet" (fewer polls = fewer issue slots taken from the warps that have work)
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when the phase did not complete within `max_tries` polls.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, int max_tries) {
  for (int i = 0; i < max_tries; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}
// global -> shared bulk copy of `bytes` (multiple of 16, both addresses 16-byte aligned); completion
// is signalled on the mbarrier as transaction bytes.
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar,
                                              uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;\n" ::
          "r"(dst),
      "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// ---- GDN block summaries: stored as fp32 or bf16, arithmetic always fp32 ------------------------
// (the reference's optional bf16 state storage, shared_cache/gdn.py:40-45: values are widened when
// read and rounded once when a new summary is stored, shared_cache/gdn.py:249-269,
// shared_cache/gdn_affine.py:113-122)
__device__ __forceinline__ float4 widen_bf16x4(uint2 r) {
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ uint2 round_bf16x4(float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y);
  const __nv_bfloat162 hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 r;
  r.x = *reinterpret_cast<const uint32_t*>(&lo);
  r.y = *reinterpret_cast<const uint32_t*>(&hi);
  return r;
}
// element i (sum_ld1 / sum_st1) or elements i..i+3, i a multiple of 4 (sum_ld4 / sum_st4)
__device__ __forceinline__ float sum_ld1(const void* base, int64_t i, bool bf16) {
  return bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(base)[i]) : static_cast<const float*>(base)[i];
}
__device__ __forceinline__ void sum_st1(void* base, int64_t i, float v, bool bf16) {
  if (bf16) static_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16_rn(v);
  else static_cast<float*>(base)[i] = v;
}
__device__ __forceinline__ float4 sum_ld4(const void* base, int64_t i, bool bf16) {
  if (bf16) return widen_bf16x4(*reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(base) + i));
  return *reinterpret_cast<const float4*>(static_cast<const float*>(base) + i);
}
__device__ __forceinline__ void sum_st4(void* base, int64_t i, float4 v, bool bf16) {
  if (bf16) *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(base) + i) = round_bf16x4(v);
  else *reinterpret_cast<float4*>(static_cast<float*>(base) + i) = v;
}
// the same with the storage type fixed at compile time; Raw is what a row piece occupies in
// registers while it is in flight
template <bool kBf16>
struct SumIO;
template <>
struct SumIO<false> {
  using Raw = float4;
  static __device__ __forceinline__ Raw ld(const void* base, int64_t i) {
    return *reinterpret_cast<const float4*>(static_cast<const float*>(base) + i);
  }
  static __device__ __forceinline__ Raw ld_stream(const void* base, int64_t i) {
    return __ldcs(reinterpret_cast<const float4*>(static_cast<const float*>(base) + i));
  }
  static __device__ __forceinline__ float4 widen(Raw r) { return r; }
  static __device__ __forceinline__ void st_stream(void* base, int64_t i, float4 v) {
    __stcs(reinterpret_cast<float4*>(static_cast<float*>(base) + i), v);
  }
};
template <>
struct SumIO<true> {
  using Raw = uint2;
  static __device__ __forceinline__ Raw ld(const void* base, int64_t i) {
    return *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(base) + i);
  }
  static __device__ __forceinline__ Raw ld_stream(const void* base, int64_t i) {
    return __ldcs(reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(base) + i));
  }
  static __device__ __forceinline__ float4 widen(Raw r) { return widen_bf16x4(r); }
  static __device__ __forceinline__ void st_stream(void* base, int64_t i, float4 v) {
    __stcs(reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(base) + i), round_bf16x4(v));
  }
};

// ---- programmatic dependent launch -------------------------------------------------------------
// A kernel launched with the programmatic-serialization attribute may start while the kernel before
// it in the stream is still running, once every CTA of that kernel has called
// pdl_launch_dependents() (or exited).  pdl_wait() returns when the earlier kernel has completed and
// its writes are visible; a thread must call it before it reads anything that kernel wrote.  Both
// are no-ops in a launch without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n"
               : "=r"(r[0]), "=r"(r[1])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n"
               : "=r"(r[0]), "=r"(r[1])
               : "r"(addr));
}

// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4],
                                               const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Transpose an 8x8 b16 matrix held one 32-bit register per lane.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
  return d;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void report(int32_t* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

// One element of the neox-style RoPE rotation by a signed integer offset, restating
// apply_rope_correction (shared_cache/rope_correction.py:36-54): cos/sin are read at
// min(|delta|, max_pos-1), sin is negated for a negative delta, the two products and the
// add/sub are separate fp32 roundings (no fused multiply-add), dims >= rotary_dim pass through.
//   x      pointer to the head's head_dim bf16 values;  d  the output element index
__device__ __forceinline__ float rope_element(const __nv_bfloat16* x, int d, int rotary_dim,
                                              const float* cs_row, bool negate) {
  const int half = rotary_dim >> 1;
  const float xd = __bfloat162float(x[d]);
  if (d >= rotary_dim) return xd;
  if (d < half) {
    const float c = cs_row[d];
    float s = cs_row[half + d];
    s = negate ? -s : s;
    const float other = __bfloat162float(x[d + half]);
    return __fsub_rn(__fmul_rn(c, xd), __fmul_rn(s, other));
  }
  const float c = cs_row[d - half];
  float s = cs_row[d];
  s = negate ? -s : s;
  const float other = __bfloat162float(x[d - half]);
  return __fadd_rn(__fmul_rn(c, xd), __fmul_rn(s, other));
}

__device__ __forceinline__ const float* rope_row(const float* cos_sin, int rotary_dim, int max_pos,
                                                 int delta, bool* negate) {
  *negate = delta < 0;
  int a = delta < 0 ? -delta : delta;
  a = a > max_pos - 1 ? max_pos - 1 : a;
  return cos_sin + static_cast<int64_t>(a) * rotary_dim;
}

}  // namespace va

// Host-side error plumbing shared by the entry points (defined in capi.cu).
namespace va_host {
int note_cuda_error(cudaError_t e);
int check_pool(const VaPool* pool);

// Launch `kernel(params)` so that it may begin before the previous kernel of `stream` has finished
// (see pdl_wait above).
template <typename Params>
inline cudaError_t launch_dependent(void (*kernel)(Params), dim3 grid, dim3 block, size_t smem_bytes,
                                    cudaStream_t stream, const Params& params) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, params);
}
}  // namespace va_host
