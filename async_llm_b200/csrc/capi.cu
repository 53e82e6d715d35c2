// Library facts and host-side error plumbing of the C ABI.
#include <string.h>

#include "common.cuh"

namespace {
thread_local char g_last_error[256] = "";
}

namespace va_host {

int note_cuda_error(cudaError_t e) {
  const char* msg = cudaGetErrorString(e);
  strncpy(g_last_error, msg != nullptr ? msg : "unknown CUDA error", sizeof(g_last_error) - 1);
  g_last_error[sizeof(g_last_error) - 1] = '\0';
  return VA_ERR_LAUNCH;
}

int check_pool(const VaPool* pool) {
  if (pool == nullptr || pool->k == nullptr || pool->v == nullptr) return VA_ERR_BAD_ARG;
  if (pool->page_size <= 0 || pool->num_slots <= 0 || pool->num_slots % pool->page_size != 0 ||
      pool->num_slots > 0x7fffffffLL)
    return VA_ERR_BAD_ARG;
  if (pool->num_q_heads <= 0 || pool->num_kv_heads <= 0 ||
      pool->num_q_heads % pool->num_kv_heads != 0)
    return VA_ERR_BAD_ARG;
  if (pool->head_dim != 128 && pool->head_dim != 256) return VA_ERR_UNSUPPORTED;
  if (pool->rotary_dim <= 0 || pool->rotary_dim > pool->head_dim || (pool->rotary_dim & 1))
    return VA_ERR_BAD_ARG;
  if (pool->cos_sin == nullptr || pool->max_pos <= 0) return VA_ERR_BAD_ARG;
  return VA_OK;
}

}  // namespace va_host

extern "C" int va_abi_version(void) { return 5; }

extern "C" const char* va_last_cuda_error(void) { return g_last_error; }

extern "C" int va_sm_count(void) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  int sms = 0;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return va_host::note_cuda_error(e);
  return sms;
}
