// The elementwise steps either side of the GDN recurrent core in a decode step, fused.
//
// va_gdn_decode_pre replaces, in Qwen3_5GatedDeltaNet._forward_ar_decode
// (models/qwen3_5_delta.py:453-461), the torch.cat of the conv window, the slice that becomes the
// new conv state, _decode_conv_silu (models/qwen3_5_delta.py:232-245: fp32 products, fp32 running
// sum, fp32 SiLU, one cast) and _gates (models/qwen3_5_delta.py:296-299: beta = sigmoid(b) in the
// activation dtype, g = -exp(A_log) * softplus(a + dt_bias) in fp32): about twenty small launches
// per layer become one.
//
// va_gdn_gated_rmsnorm replaces _GatedRMSNorm.forward (models/qwen3_5_delta.py:248-263): fp32
// x * rsqrt(mean(x^2) + eps) * weight * silu(gate), one cast.
#include "common.cuh"

namespace {

using namespace va;

constexpr int kMaxConvKernel = 8;

struct PreParams {
  const __nv_bfloat16* qkv;
  int64_t qkv_row_stride;
  const __nv_bfloat16* prior_conv;   // [W, conv_dim, k] or null (zeros)
  const __nv_bfloat16* conv_weight;  // [conv_dim, k]
  const __nv_bfloat16* a;            // [W, Hv] rows a_row_stride elements apart
  const __nv_bfloat16* b;            // [W, Hv] rows b_row_stride elements apart
  int64_t a_row_stride, b_row_stride;
  const float* a_log;                // [Hv]
  const float* dt_bias;              // [Hv]
  __nv_bfloat16* qkv_out;            // [W, conv_dim]
  __nv_bfloat16* conv_out;           // [W, conv_dim, k]
  __nv_bfloat16* beta_out;           // [W, Hv]
  float* g_out;                      // [W, Hv]
  float* beta_f32_out;               // [W, Hv] the bf16 beta widened, or null
  const int64_t* prior_conv_ptrs;    // [W] addresses of [conv_dim, k] states (0 = zeros), or null
  const int64_t* conv_out_ptrs;      // [W] addresses of the [conv_dim, k] states to write, or null
  int32_t num_workers, conv_dim, conv_kernel, num_v_heads;
};

__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + expf(-x)); }

// grid = (worker, channel slice): the CTAs of a worker stride over its conv channels together (one
// CTA per worker left 32 serial passes over strided windows: 51 us for 32 workers x 8192 channels); the
// first slice also computes the gates of the worker's heads.
__global__ void __launch_bounds__(256) gdn_decode_pre_kernel(const __grid_constant__ PreParams p) {
  const int w = blockIdx.x;
  const int K = p.conv_kernel;
  const __nv_bfloat16* x_row = p.qkv + static_cast<int64_t>(w) * p.qkv_row_stride;
  // this worker's previous and next conv state: rows of the dense arrays, or separate tensors
  // named by address (the most recent window along the worker's chain / its write block's slab)
  const int64_t w_off = static_cast<int64_t>(w) * p.conv_dim * K;
  const __nv_bfloat16* prior_w =
      p.prior_conv_ptrs != nullptr ? reinterpret_cast<const __nv_bfloat16*>(p.prior_conv_ptrs[w])
                                   : (p.prior_conv != nullptr ? p.prior_conv + w_off : nullptr);
  __nv_bfloat16* out_w = p.conv_out_ptrs != nullptr ? reinterpret_cast<__nv_bfloat16*>(p.conv_out_ptrs[w])
                                                    : p.conv_out + w_off;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < p.conv_dim; c += gridDim.y * blockDim.x) {
    const int64_t ch = static_cast<int64_t>(w) * p.conv_dim + c;
    // window = the last K entries of [prior (K entries) | new input]
    __nv_bfloat16 win[kMaxConvKernel];
#pragma unroll
    for (int t = 0; t < kMaxConvKernel; ++t) {
      if (t < K - 1) win[t] = prior_w != nullptr ? prior_w[c * K + t + 1] : __float2bfloat16_rn(0.0f);
    }
    win[K - 1] = x_row[c];
    float total = 0.0f;
#pragma unroll
    for (int t = 0; t < kMaxConvKernel; ++t) {
      if (t < K) {
        const float prod = __fmul_rn(__bfloat162float(win[t]), __bfloat162float(p.conv_weight[c * K + t]));
        total = __fadd_rn(total, prod);
        if (out_w != nullptr) out_w[c * K + t] = win[t];   // null: a padding row of a fixed-capacity batch
      }
    }
    p.qkv_out[ch] = __float2bfloat16_rn(silu_f32(total));
  }
  if (blockIdx.y != 0) return;
  for (int h = threadIdx.x; h < p.num_v_heads; h += blockDim.x) {
    const int64_t i = static_cast<int64_t>(w) * p.num_v_heads + h;
    const float bv = __bfloat162float(p.b[static_cast<int64_t>(w) * p.b_row_stride + h]);
    const __nv_bfloat16 beta = __float2bfloat16_rn(1.0f / (1.0f + expf(-bv)));
    p.beta_out[i] = beta;
    if (p.beta_f32_out != nullptr) p.beta_f32_out[i] = __bfloat162float(beta);
    const float z = __fadd_rn(__bfloat162float(p.a[static_cast<int64_t>(w) * p.a_row_stride + h]), p.dt_bias[h]);
    const float sp = z > 20.0f ? z : log1pf(expf(z));   // softplus, threshold 20
    p.g_out[i] = __fmul_rn(-expf(p.a_log[h]), sp);
  }
}

// One warp per row of `dim` elements (dim a multiple of 32, at most 1024).  The gate rows of one
// token (rows_per_token of them, `dim` apart) may lie inside a wider projection row: tokens are
// gate_token_stride elements apart.
__global__ void __launch_bounds__(256) gdn_gated_rmsnorm_kernel(const __nv_bfloat16* x, const __nv_bfloat16* gate,
                                                                const float* weight, __nv_bfloat16* out,
                                                                int64_t rows, int dim, float eps, int rows_per_token,
                                                                int64_t gate_token_stride) {
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + row * dim;
  const int64_t tok = row / rows_per_token;
  const __nv_bfloat16* gr = gate + tok * gate_token_stride + (row - tok * rows_per_token) * dim;
  const int per = dim >> 5;
  float v[32];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    if (i < per) {
      v[i] = __bfloat162float(xr[lane + 32 * i]);
      ss += v[i] * v[i];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float inv = rsqrtf(ss / static_cast<float>(dim) + eps);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    if (i < per) {
      const int d = lane + 32 * i;
      const float y = __fmul_rn(weight[d], __fmul_rn(v[i], inv));
      out[row * dim + d] = __float2bfloat16_rn(__fmul_rn(y, silu_f32(__bfloat162float(gr[d]))));
    }
  }
}

struct PrefillConvParams {
  const __nv_bfloat16* qkv;          // [T, conv_dim] rows
  int64_t qkv_row_stride;
  const __nv_bfloat16* prior_conv;   // [R, conv_dim, k] or null (zeros)
  const __nv_bfloat16* conv_weight;  // [conv_dim, k]
  const int32_t* seg_off;            // [R + 1] token offsets of the requests
  __nv_bfloat16* qkv_out;            // [T, conv_dim]
  __nv_bfloat16* conv_out;           // [R, conv_dim, k]
  const int64_t* prior_conv_ptrs;    // [R] addresses of [conv_dim, k] states (0 = zeros), or null
  const int64_t* conv_out_ptrs;      // [R] addresses of the states to write (0 = skip), or null
  int32_t num_requests, num_tokens, conv_dim, conv_kernel;
};

// grid.x = token.  out[t][c] = SiLU(sum_tap bf16(in[t - (k-1) + tap][c] * w[c][tap])), inputs before
// the request's first token come from its prior conv state (zeros without one): the products are
// rounded to bf16, the sum and the SiLU are fp32 (_prefill_conv_silu, models/qwen3_5_delta.py:215-229).
// The block of a request's last token also writes the request's new conv state, the last k entries
// of [prior | inputs] (models/qwen3_5_delta.py:409-418).
__global__ void __launch_bounds__(256) gdn_prefill_conv_kernel(const __grid_constant__ PrefillConvParams p) {
  __shared__ int s_req, s_begin, s_end;
  const int t = blockIdx.x;
  if (threadIdx.x == 0) {
    int r = 0;
    while (r + 1 < p.num_requests && p.seg_off[r + 1] <= t) ++r;
    s_req = r;
    s_begin = p.seg_off[r];
    s_end = p.seg_off[r + 1];
  }
  __syncthreads();
  const int r = s_req, begin = s_begin, end = s_end;
  if (t < begin || t >= end) return;   // a token outside every segment (malformed offsets) is left alone
  const int K = p.conv_kernel;
  const int i = t - begin;             // index within the request
  const int64_t r_off = static_cast<int64_t>(r) * p.conv_dim * K;
  const __nv_bfloat16* prior_r =
      p.prior_conv_ptrs != nullptr ? reinterpret_cast<const __nv_bfloat16*>(p.prior_conv_ptrs[r])
                                   : (p.prior_conv != nullptr ? p.prior_conv + r_off : nullptr);
  __nv_bfloat16* out_r = p.conv_out_ptrs != nullptr ? reinterpret_cast<__nv_bfloat16*>(p.conv_out_ptrs[r])
                                                    : p.conv_out + r_off;
  auto input = [&](int idx, int c) -> __nv_bfloat16 {   // idx relative to the request's first token
    if (idx >= 0) return p.qkv[static_cast<int64_t>(begin + idx) * p.qkv_row_stride + c];
    if (prior_r == nullptr) return __float2bfloat16_rn(0.0f);
    return prior_r[static_cast<int64_t>(c) * K + (K + idx)];
  };
  for (int c = threadIdx.x; c < p.conv_dim; c += blockDim.x) {
    float total = 0.0f;
#pragma unroll
    for (int tap = 0; tap < kMaxConvKernel; ++tap) {
      if (tap < K) {
        const float x = __bfloat162float(input(i - (K - 1) + tap, c));
        const float w = __bfloat162float(p.conv_weight[c * K + tap]);
        total = __fadd_rn(total, __bfloat162float(__float2bfloat16_rn(__fmul_rn(x, w))));
      }
    }
    p.qkv_out[static_cast<int64_t>(t) * p.conv_dim + c] = __float2bfloat16_rn(silu_f32(total));
    if (t == end - 1 && out_r != nullptr) {
      const int L = end - begin;
      for (int j = 0; j < K; ++j) out_r[static_cast<int64_t>(c) * K + j] = input(L - K + j, c);
    }
  }
}

}  // namespace

extern "C" int va_gdn_decode_pre(const VaGdnDecodePre* a, va_stream_t stream) {
  if (a == nullptr || a->num_workers < 0 || a->conv_dim <= 0 || a->num_v_heads <= 0) return VA_ERR_BAD_ARG;
  if (a->conv_kernel < 1 || a->conv_kernel > kMaxConvKernel) return VA_ERR_UNSUPPORTED;
  if (a->num_workers == 0) return VA_OK;
  if (!a->qkv || !a->conv_weight || !a->a || !a->b || !a->a_log || !a->dt_bias || !a->qkv_out ||
      (!a->conv_out && !a->conv_out_ptrs) || !a->beta_out || !a->g_out)
    return VA_ERR_BAD_ARG;
  if (a->qkv_row_stride < a->conv_dim) return VA_ERR_BAD_ARG;
  PreParams p;
  p.qkv = static_cast<const __nv_bfloat16*>(a->qkv);
  p.qkv_row_stride = a->qkv_row_stride;
  p.prior_conv = static_cast<const __nv_bfloat16*>(a->prior_conv);
  p.conv_weight = static_cast<const __nv_bfloat16*>(a->conv_weight);
  p.a = static_cast<const __nv_bfloat16*>(a->a);
  p.b = static_cast<const __nv_bfloat16*>(a->b);
  p.a_row_stride = a->a_row_stride > 0 ? a->a_row_stride : a->num_v_heads;
  p.b_row_stride = a->b_row_stride > 0 ? a->b_row_stride : a->num_v_heads;
  if (p.a_row_stride < a->num_v_heads || p.b_row_stride < a->num_v_heads) return VA_ERR_BAD_ARG;
  p.a_log = a->a_log;
  p.dt_bias = a->dt_bias;
  p.qkv_out = static_cast<__nv_bfloat16*>(a->qkv_out);
  p.conv_out = static_cast<__nv_bfloat16*>(a->conv_out);
  p.beta_out = static_cast<__nv_bfloat16*>(a->beta_out);
  p.g_out = a->g_out;
  p.beta_f32_out = a->beta_f32_out;
  p.prior_conv_ptrs = a->prior_conv_ptrs;
  p.conv_out_ptrs = a->conv_out_ptrs;
  p.num_workers = a->num_workers;
  p.conv_dim = a->conv_dim;
  p.conv_kernel = a->conv_kernel;
  p.num_v_heads = a->num_v_heads;
  // enough channel slices to fill the GPU at small batch, at most one pass per thread
  int slices = (a->conv_dim + 255) / 256;
  const int want = (4 * 148 + a->num_workers - 1) / a->num_workers;
  if (slices > want) slices = want;
  if (slices < 1) slices = 1;
  gdn_decode_pre_kernel<<<dim3(a->num_workers, slices), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return VA_OK;
}

extern "C" int va_gdn_gated_rmsnorm(const void* x, const void* gate, const float* weight, void* out,
                                    int64_t rows, int32_t dim, float eps, int32_t rows_per_token,
                                    int64_t gate_token_stride, va_stream_t stream) {
  if (rows < 0 || dim <= 0 || (dim & 31) || dim > 1024) return VA_ERR_BAD_ARG;
  if (rows == 0) return VA_OK;
  if (!x || !gate || !weight || !out) return VA_ERR_BAD_ARG;
  if (rows_per_token <= 0) {   // dense gate rows
    rows_per_token = 1;
    gate_token_stride = dim;
  }
  if (gate_token_stride < static_cast<int64_t>(rows_per_token) * dim || rows % rows_per_token != 0) return VA_ERR_BAD_ARG;
  const int64_t blocks = (rows + 7) / 8;
  if (blocks > 0x7fffffffLL) return VA_ERR_CAPACITY;
  gdn_gated_rmsnorm_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gate), weight,
      static_cast<__nv_bfloat16*>(out), rows, dim, eps, rows_per_token, gate_token_stride);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return VA_OK;
}

extern "C" int va_gdn_prefill_conv(const VaGdnPrefillConv* a, va_stream_t stream) {
  if (a == nullptr || a->num_requests < 0 || a->num_tokens < 0 || a->conv_dim <= 0) return VA_ERR_BAD_ARG;
  if (a->conv_kernel < 1 || a->conv_kernel > kMaxConvKernel) return VA_ERR_UNSUPPORTED;
  if (a->num_tokens == 0 || a->num_requests == 0) return VA_OK;
  if (!a->qkv || !a->conv_weight || !a->seg_off || !a->qkv_out || (!a->conv_out && !a->conv_out_ptrs))
    return VA_ERR_BAD_ARG;
  if (a->qkv_row_stride < a->conv_dim) return VA_ERR_BAD_ARG;
  PrefillConvParams p;
  p.prior_conv_ptrs = a->prior_conv_ptrs;
  p.conv_out_ptrs = a->conv_out_ptrs;
  p.qkv = static_cast<const __nv_bfloat16*>(a->qkv);
  p.qkv_row_stride = a->qkv_row_stride;
  p.prior_conv = static_cast<const __nv_bfloat16*>(a->prior_conv);
  p.conv_weight = static_cast<const __nv_bfloat16*>(a->conv_weight);
  p.seg_off = a->seg_off;
  p.qkv_out = static_cast<__nv_bfloat16*>(a->qkv_out);
  p.conv_out = static_cast<__nv_bfloat16*>(a->conv_out);
  p.num_requests = a->num_requests;
  p.num_tokens = a->num_tokens;
  p.conv_dim = a->conv_dim;
  p.conv_kernel = a->conv_kernel;
  gdn_prefill_conv_kernel<<<a->num_tokens, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return VA_OK;
}
