// RMSNorm over the 32-bit residual stream, fused with the residual sum.
//
// For output row i (source row r = rows ? rows[i] : i):
//     x      = resid[r, :] (+ delta[r, :] when delta is given)      in float32
//     resid[r, :] = x                      (when write_resid)
//     out[i, :]   = x * rsqrt(mean(x^2) + eps) * weight
// The sum of squares, the inverse and the product are float32; the only rounding
// to the activation type is the final store.  One block per row, the row staged
// in shared memory, so the reduction order depends on the row length alone and
// a row's result does not depend on what else is in the batch.
#include "common.cuh"
using namespace arle;

template <typename TA>
__global__ void rmsnorm_kernel(float* __restrict__ resid, const TA* __restrict__ delta,
                               const int* __restrict__ rows, const float* __restrict__ weight,
                               TA* __restrict__ out, int hidden, float eps, int write_resid) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float xs[];
  __shared__ float red[33];
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* xr = resid + (size_t)r * hidden;
  const TA* dr = delta ? delta + (size_t)r * hidden : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float x = xr[c];
    if (dr) x += to_f32(dr[c]);
    xs[c] = x;
    if (write_resid) xr[c] = x;
    ss += x * x;
  }
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  TA* o = out + (size_t)i * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x)
    o[c] = from_f32<TA>(xs[c] * inv * weight[c]);
}

// Four elements per thread and step through 16-byte (float) / 8-byte (bfloat16)
// accesses, the row kept in registers: the same arithmetic in the same order per
// element, a fraction of the memory instructions.  Needs hidden % 4 == 0,
// hidden <= 4 * kVecMax * blockDim.x, and 16-byte aligned rows.
constexpr int kVecMax = 4;

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename TA>
__global__ void rmsnorm_vec_kernel(float* __restrict__ resid, const TA* __restrict__ delta,
                                   const int* __restrict__ rows, const float* __restrict__ weight,
                                   TA* __restrict__ out, int hidden, float eps, int write_resid) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* xr = resid + (size_t)r * hidden;
  const TA* dr = delta ? delta + (size_t)r * hidden : nullptr;
  const int n4 = hidden >> 2;
  float4 x[kVecMax];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < kVecMax; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < n4) {
      float4 v = load4(xr + 4 * c);
      if (dr) {
        const float4 d = load4(dr + 4 * c);
        v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        if (write_resid) store4(xr + 4 * c, v);
      }
      x[k] = v;
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  }
  float4 wv[kVecMax];                         // fetched before the reduction so that it is not waited for after it
#pragma unroll
  for (int k = 0; k < kVecMax; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < n4) wv[k] = load4(weight + 4 * c);
  }
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  TA* o = out + (size_t)i * hidden;
#pragma unroll
  for (int k = 0; k < kVecMax; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < n4) {
      const float4 w = wv[k];
      store4(o + 4 * c, make_float4(x[k].x * inv * w.x, x[k].y * inv * w.y, x[k].z * inv * w.z, x[k].w * inv * w.w));
    }
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename TA>
static int launch(float* resid, const void* delta, const int* rows, const float* weight, void* out,
                  int n_out, int hidden, float eps, int write_resid, cudaStream_t s) {
  if (hidden % 4 == 0 && hidden <= 4 * kVecMax * 1024 && aligned16(resid) && aligned16(weight) && aligned16(out) &&
      aligned16(delta)) {
    const int n4 = hidden / 4;
    int threads = (n4 + kVecMax - 1) / kVecMax;
    threads = threads <= 64 ? 64 : (threads <= 128 ? 128 : (threads <= 256 ? 256 : (threads <= 512 ? 512 : 1024)));
    launch_kernel(rmsnorm_vec_kernel<TA>, dim3(n_out), dim3(threads), 0, s, 1, resid, (const TA*)delta, rows, weight, (TA*)out, hidden, eps,
                                                     write_resid);
    return launch_status();
  }
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return ARLE_E_UNSUPPORTED;
  if (smem > 32 * 1024) {  // static shared memory counts against the 48 KB default too
    cudaError_t e = cudaFuncSetAttribute(rmsnorm_kernel<TA>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  launch_kernel(rmsnorm_kernel<TA>, dim3(n_out), dim3(threads), smem, s, 1, resid, (const TA*)delta, rows, weight, (TA*)out, hidden,
                                                  eps, write_resid);
  return launch_status();
}

// act_dtype: type of delta and out.  The gain vector is float32 (norm gains are
// widened once at load; they are a few KB).
ARLE_API int arle_rmsnorm(float* resid, const void* delta, const int* rows, const float* weight,
                          void* out, int act_dtype, int n_out, int hidden, float eps, int write_resid,
                          cudaStream_t s) {
  if (n_out <= 0) return 0;
  if (hidden <= 0) return ARLE_E_BADARG;
  if (act_dtype == 0) return launch<float>(resid, delta, rows, weight, out, n_out, hidden, eps, write_resid, s);
  if (act_dtype == 1) return launch<__nv_bfloat16>(resid, delta, rows, weight, out, n_out, hidden, eps, write_resid, s);
  return ARLE_E_BADARG;
}

// resid[r, :] += delta[r, :] for all rows: the residual sum alone, for a branch
// output that no norm follows directly.
template <typename TA>
__global__ void residual_add_kernel(float* __restrict__ resid, const TA* __restrict__ delta, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    resid[i] += to_f32(delta[i]);
}

ARLE_API int arle_residual_add(float* resid, const void* delta, int act_dtype, int rows, int hidden, cudaStream_t s) {
  if (rows <= 0) return 0;
  const size_t total = (size_t)rows * hidden;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (act_dtype == 0)
    launch_kernel(residual_add_kernel<float>, dim3((int)blocks), dim3(256), 0, s, 1, resid, (const float*)delta, total);
  else if (act_dtype == 1)
    launch_kernel(residual_add_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, s, 1, resid, (const __nv_bfloat16*)delta, total);
  else
    return ARLE_E_BADARG;
  return launch_status();
}
