// SwiGLU gate: out[t, i] = silu(gu[t, i]) * gu[t, I + i], silu(g) = g / (1 + exp(-g)),
// computed in float32 and rounded once.  gu is the [T, 2I] output of the packed
// gate/up projection.
#include "common.cuh"
using namespace arle;

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total) {
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter;
    const int i = (int)(idx - t * inter);
    const float g = to_f32(gu[t * 2 * (size_t)inter + i]);
    const float u = to_f32(gu[t * 2 * (size_t)inter + inter + i]);
    out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
  }
}

ARLE_API int arle_silu_mul(const void* gu, void* out, int dtype, int num_tokens, int inter, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (inter <= 0) return ARLE_E_BADARG;
  const size_t total = (size_t)num_tokens * inter;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (dtype == 0)
    silu_mul_kernel<float><<<(int)blocks, threads, 0, s>>>((const float*)gu, (float*)out, inter, total);
  else if (dtype == 1)
    silu_mul_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, s>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, total);
  else
    return ARLE_E_BADARG;
  return launch_status();
}
