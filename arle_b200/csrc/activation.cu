// SwiGLU gate: out[t, i] = silu(gu[t, 2i]) * gu[t, 2i + 1], silu(g) = g / (1 + exp(-g)),
// computed in float32 and rounded once.  gu is the [T, 2I] output of the packed
// gate/up projection, whose rows 2i and 2i + 1 are gate_i and up_i.
#include "common.cuh"
using namespace arle;

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter;
    const int i = (int)(idx - t * inter);
    const float g = to_f32(gu[t * 2 * (size_t)inter + 2 * i]);
    const float u = to_f32(gu[t * 2 * (size_t)inter + 2 * i + 1]);
    out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
  }
}

// Eight elements per thread and step for bfloat16 rows whose width is a multiple of 8.
__global__ void silu_mul_bf16_vec_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int inter,
                                         size_t total8) {
  pdl_launch_dependents();
  pdl_wait();
  const int i8 = inter >> 3;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / i8;
    const int c = (int)(idx - t * i8);
    const uint4 a4 = *reinterpret_cast<const uint4*>(gu + t * 2 * (size_t)inter + 16 * c);       // pairs 0..3
    const uint4 b4 = *reinterpret_cast<const uint4*>(gu + t * 2 * (size_t)inter + 16 * c + 8);   // pairs 4..7
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a4);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const __nv_bfloat162 p0 = k < 2 ? a2[2 * k] : b2[2 * k - 4], p1 = k < 2 ? a2[2 * k + 1] : b2[2 * k - 3];
      const float ga = __low2float(p0), gb = __low2float(p1);
      // fast exponential and division (a few ulp of float32, far below the bfloat16 rounding that follows):
      // with the exact ones the kernel was bound by arithmetic, not by memory
      o2[k] = __floats2bfloat162_rn(__fdividef(ga, 1.0f + __expf(-ga)) * __high2float(p0),
                                    __fdividef(gb, 1.0f + __expf(-gb)) * __high2float(p1));
    }
    *reinterpret_cast<uint4*>(out + t * (size_t)inter + 8 * c) = o4;
  }
}

ARLE_API int arle_silu_mul(const void* gu, void* out, int dtype, int num_tokens, int inter, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (inter <= 0) return ARLE_E_BADARG;
  const size_t total = (size_t)num_tokens * inter;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (dtype == 1 && inter % 8 == 0 && ((uintptr_t)gu & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    const size_t total8 = total / 8;
    size_t b8 = (total8 + threads - 1) / threads;
    if (b8 > 148 * 32) b8 = 148 * 32;
    launch_kernel(silu_mul_bf16_vec_kernel, dim3((int)b8), dim3(threads), 0, s, 1, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, total8);
    return launch_status();
  }
  if (dtype == 0)
    launch_kernel(silu_mul_kernel<float>, dim3((int)blocks), dim3(threads), 0, s, 1, (const float*)gu, (float*)out, inter, total);
  else if (dtype == 1)
    launch_kernel(silu_mul_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, s, 1, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, total);
  else
    return ARLE_E_BADARG;
  return launch_status();
}
