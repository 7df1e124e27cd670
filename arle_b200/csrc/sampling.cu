// Next-token choice from float32 logits, one block per row.
//
// A row with temperature <= 0 or top_k == 1 is greedy: the index of the largest
// logit, ties to the lowest index.  Otherwise
//     p = softmax(logits / temperature)                    (float32, max-subtracted)
//     min_p:  drop p_i < min_p * max(p)                    (0 = off)
//     top_k:  keep the k most probable                     (<= 0 = off)
//     top_p:  keep the most probable tokens whose mass first reaches top_p (>= 1 = off)
// each followed by a renormalisation, then the first index, in index order, whose
// cumulative probability exceeds u (u in [0, 1) comes from the host's generator).
// The top_k and top_p cut-offs are found by 32 bisection steps on a probability
// threshold, which converges to the exact set when no two probabilities tie at
// the threshold.  The probabilities live in a caller-provided scratch row
// [rows, vocab] of float32.
#include "common.cuh"
using namespace arle;

constexpr int kSampleThreads = 256;

__device__ __forceinline__ void block_argmax(const float* __restrict__ x, int n, float* sval, int* sidx,
                                             int* out) {
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = x[i];
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
  sval[threadIdx.x] = best;
  sidx[threadIdx.x] = bi;
  __syncthreads();
  for (int s = blockDim.x >> 1; s > 0; s >>= 1) {
    if (threadIdx.x < s) {
      const float v = sval[threadIdx.x + s];
      const int i = sidx[threadIdx.x + s];
      if (v > sval[threadIdx.x] || (v == sval[threadIdx.x] && i < sidx[threadIdx.x])) {
        sval[threadIdx.x] = v;
        sidx[threadIdx.x] = i;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) *out = sidx[0] == 0x7fffffff ? 0 : sidx[0];
}

// Zero what lies below thr, renormalise the rest; returns nothing, probabilities sum to 1 after.
__device__ __forceinline__ void cut_below(float* p, int n, float thr, float* red) {
  float kept = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = p[i];
    if (v < thr) p[i] = 0.f; else kept += v;
  }
  kept = block_sum(kept, red);
  const float inv = 1.0f / kept;
  for (int i = threadIdx.x; i < n; i += blockDim.x) p[i] *= inv;
  __syncthreads();
}

__global__ void __launch_bounds__(kSampleThreads) sample_kernel(
    const float* __restrict__ logits, int ld, int vocab, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
    const float* __restrict__ uniform, float* __restrict__ scratch, int* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  __shared__ float sval[kSampleThreads];
  __shared__ int sidx[kSampleThreads];
  __shared__ int chosen_chunk;
  const int row = blockIdx.x;
  const float* x = logits + (size_t)row * ld;
  const float temp = temperature ? temperature[row] : 0.f;
  const int k = top_k ? top_k[row] : -1;
  if (!(temp > 0.f) || k == 1) {
    block_argmax(x, vocab, sval, sidx, out + row);
    return;
  }
  float* p = scratch + (size_t)row * vocab;
  const float inv_t = 1.0f / temp;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, x[i] * inv_t);
  mx = block_max(mx, red);
  float sum = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float e = expf(x[i] * inv_t - mx);
    p[i] = e;
    sum += e;
  }
  sum = block_sum(sum, red);
  const float inv_sum = 1.0f / sum;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) p[i] *= inv_sum;
  __syncthreads();
  float pmax = inv_sum;  // exp(0) / sum

  const float mp = min_p ? min_p[row] : 0.f;
  if (mp > 0.f) {
    cut_below(p, vocab, mp * pmax, red);
    float m2 = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) m2 = fmaxf(m2, p[i]);
    pmax = block_max(m2, red);
  }
  if (k > 0 && k < vocab) {
    // smallest threshold that keeps at most k entries
    float lo = 0.f, hi = pmax;
    for (int it = 0; it < 32; ++it) {
      const float mid = 0.5f * (lo + hi);
      float c = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) c += p[i] >= mid ? 1.f : 0.f;
      c = block_sum(c, red);
      if (c > (float)k) lo = mid; else hi = mid;
    }
    cut_below(p, vocab, hi, red);
    float m2 = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) m2 = fmaxf(m2, p[i]);
    pmax = block_max(m2, red);
  }
  const float tp = top_p ? top_p[row] : 1.f;
  if (tp < 1.f) {
    // largest threshold whose kept mass still reaches top_p
    float lo = 0.f, hi = pmax;
    for (int it = 0; it < 32; ++it) {
      const float mid = 0.5f * (lo + hi);
      float mass = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = p[i];
        if (v >= mid) mass += v;
      }
      mass = block_sum(mass, red);
      if (mass >= tp) lo = mid; else hi = mid;
    }
    cut_below(p, vocab, lo, red);
  }
  // inverse CDF in index order: contiguous chunk per thread, then a scan of one chunk
  const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
  const int b = threadIdx.x * chunk, e = min(vocab, b + chunk);
  float part = 0.f;
  for (int i = b; i < e; ++i) part += p[i];
  sval[threadIdx.x] = part;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int i = 0; i < (int)blockDim.x; ++i) total += sval[i];
    const float target = uniform[row] * total;
    float c = 0.f;
    int pick = -1;
    for (int i = 0; i < (int)blockDim.x; ++i) {
      if (target < c + sval[i]) { pick = i; break; }
      c += sval[i];
    }
    chosen_chunk = pick;
    red[0] = c;       // mass before the chosen chunk
    red[1] = target;
  }
  __syncthreads();
  const int cc = chosen_chunk;
  if (cc < 0) {
    // rounding left u beyond the total mass: the last index with non-zero probability
    int last = -1;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) if (p[i] > 0.f) last = max(last, i);
    sidx[threadIdx.x] = last;
    __syncthreads();
    for (int s = blockDim.x >> 1; s > 0; s >>= 1) {
      if (threadIdx.x < s) sidx[threadIdx.x] = max(sidx[threadIdx.x], sidx[threadIdx.x + s]);
      __syncthreads();
    }
    if (threadIdx.x == 0) out[row] = max(sidx[0], 0);
    return;
  }
  if (threadIdx.x == cc) {
    float c = red[0];
    const float target = red[1];
    int pick = -1, last = b;
    for (int i = b; i < e; ++i) {
      if (p[i] > 0.f) last = i;
      c += p[i];
      if (target < c) { pick = i; break; }
    }
    out[row] = pick >= 0 ? pick : last;
  }
}

// Greedy rows only, large vocabularies: the row is cut into kArgmaxParts parts that
// are searched by separate blocks, then one small block per row picks the best
// part (ties: the lowest index, as everywhere).
constexpr int kArgmaxParts = 32;

__global__ void __launch_bounds__(kSampleThreads) argmax_part_kernel(const float* __restrict__ logits, int ld, int vocab,
                                                                     float* __restrict__ part_val, int* __restrict__ part_idx) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sval[kSampleThreads];
  __shared__ int sidx[kSampleThreads];
  const int row = blockIdx.y, part = blockIdx.x;
  const int per = (vocab + kArgmaxParts - 1) / kArgmaxParts;
  const int b = part * per, e = min(vocab, b + per);
  const float* x = logits + (size_t)row * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  auto take = [&](float v, int i) {
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  };
  // 16-byte loads over the aligned middle of the part, four of them under way per thread; the ragged ends one by one
  const int a0 = min(e, (int)((b + ((4 - ((reinterpret_cast<uintptr_t>(x + b) >> 2) & 3)) & 3))));
  const int n4 = (e - a0) >> 2;
  for (int i = b + threadIdx.x; i < a0; i += blockDim.x) take(x[i], i);
  const float4* x4 = reinterpret_cast<const float4*>(x + a0);
  int q = threadIdx.x;
  for (; q + 3 * (int)blockDim.x < n4; q += 4 * blockDim.x) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = x4[q + u * blockDim.x];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = a0 + 4 * (q + u * blockDim.x);
      take(v[u].x, i), take(v[u].y, i + 1), take(v[u].z, i + 2), take(v[u].w, i + 3);
    }
  }
  for (; q < n4; q += blockDim.x) {
    const float4 v = x4[q];
    const int i = a0 + 4 * q;
    take(v.x, i), take(v.y, i + 1), take(v.z, i + 2), take(v.w, i + 3);
  }
  for (int i = a0 + 4 * n4 + threadIdx.x; i < e; i += blockDim.x) take(x[i], i);
  // the warps' bests by shuffles, then one warp over the warps
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  if (lane == 0) sval[warp] = best, sidx[warp] = bi;
  __syncthreads();
  if (warp == 0) {
    best = lane < nwarps ? sval[lane] : -INFINITY;
    bi = lane < nwarps ? sidx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) {
      part_val[row * kArgmaxParts + part] = best;
      part_idx[row * kArgmaxParts + part] = bi;
    }
  }
}

__global__ void argmax_pick_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx, int* __restrict__ out,
                                   const int* __restrict__ scatter, int* __restrict__ last_token) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, lane = threadIdx.x;       // one warp, kArgmaxParts == 32
  float v = part_val[row * kArgmaxParts + lane];
  int i = part_idx[row * kArgmaxParts + lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
  if (lane == 0) {
    const int tok = i == 0x7fffffff ? 0 : i;
    out[row] = tok;
    if (scatter) last_token[scatter[row]] = tok;
  }
}

// All rows greedy.  scratch: float32 [rows * 64] (values in the first half, indices in the second).
// scatter / last_token (may both be null): last_token[scatter[row]] = the row's token, for the
// placeholder ids of the embedding kernel.
ARLE_API int arle_argmax(const float* logits, int ld, int rows, int vocab, float* scratch, int* out, const int* scatter,
                         int* last_token, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || ld < vocab || !scratch) return ARLE_E_BADARG;
  if (rows > 65535) return ARLE_E_UNSUPPORTED;
  float* pv = scratch;
  int* pi = reinterpret_cast<int*>(scratch + (size_t)rows * kArgmaxParts);
  launch_kernel(argmax_part_kernel, dim3(dim3(kArgmaxParts, rows)), dim3(kSampleThreads), 0, s, 1, logits, ld, vocab, pv, pi);
  int rc = launch_status();
  if (rc) return rc;
  launch_kernel(argmax_pick_kernel, dim3(rows), dim3(32), 0, s, 1, pv, pi, out, scatter, last_token);
  return launch_status();
}

__global__ void scatter_tokens_kernel(const int* __restrict__ tokens, const int* __restrict__ scatter,
                                      int* __restrict__ last_token, int rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < rows) last_token[scatter[r]] = tokens[r];
}

ARLE_API int arle_scatter_tokens(const int* tokens, const int* scatter, int* last_token, int rows, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (!tokens || !scatter || !last_token) return ARLE_E_BADARG;
  launch_kernel(scatter_tokens_kernel, dim3((rows + 127) / 128), dim3(128), 0, s, 1, tokens, scatter, last_token, rows);
  return launch_status();
}

ARLE_API int arle_sample(const float* logits, int ld, int rows, int vocab, const float* temperature,
                         const int* top_k, const float* top_p, const float* min_p, const float* uniform,
                         float* scratch, int* out, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || ld < vocab) return ARLE_E_BADARG;
  if (temperature && (!uniform || !scratch)) return ARLE_E_BADARG;
  launch_kernel(sample_kernel, dim3(rows), dim3(kSampleThreads), 0, s, 1, logits, ld, vocab, temperature, top_k, top_p, min_p, uniform,
                                                scratch, out);
  return launch_status();
}

// ---------------------------------------------------------------------------
// arle_sample_static: the same sampling kernel for callers that cannot allocate
// device memory.  See no_alloc.h for the contract.  The probabilities go into a
// fixed array that is part of this library's device image instead of a buffer
// from the caller.
// ---------------------------------------------------------------------------
#include "no_alloc.h"

static __device__ __align__(256) float g_sample_scratch[ARLE_SAMPLE_STATIC_MAX_FLOATS];

// In host code g_sample_scratch names a host-side shadow of the device array, not
// a device address, so the address the kernel gets is asked from the runtime:
// once per device, with that device current, and kept here.
constexpr int kMaxDevices = 64;
static float* g_scratch_addr[kMaxDevices];

static int scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return ARLE_E_BADARG;
  float* p = __atomic_load_n(&g_scratch_addr[dev], __ATOMIC_ACQUIRE);
  if (!p) {
    void* sym = nullptr;
    e = cudaGetSymbolAddress(&sym, g_sample_scratch);
    if (e != cudaSuccess) return (int)e;
    if (!sym) return ARLE_E_BADARG;
    p = (float*)sym;
    __atomic_store_n(&g_scratch_addr[dev], p, __ATOMIC_RELEASE);   // every thread would store the same value
  }
  *out = p;
  return 0;
}

ARLE_API long long arle_sample_static_max_floats(void) { return (long long)ARLE_SAMPLE_STATIC_MAX_FLOATS; }

ARLE_API const char* arle_no_alloc_error_string(int code) {
  switch (code) {
    case 0: return "success";
    case ARLE_E_TOO_LARGE: return "arle_sample_static: rows * vocab exceeds ARLE_SAMPLE_STATIC_MAX_FLOATS, the size of the built-in scratch array";
    case ARLE_E_BADARG: return "arle_sample_static: bad argument (null pointer, vocab <= 0, ld < vocab, or device ordinal out of range)";
    case ARLE_E_UNSUPPORTED: return "arle_sample_static: sizes not supported";
    default: return code > 0 ? "arle_sample_static: CUDA runtime error (the code is a cudaError_t)" : "arle_sample_static: unknown error";
  }
}

ARLE_API int arle_sample_static(const float* logits, int ld, int rows, int vocab, const float* temperature,
                                const int* top_k, const float* top_p, const float* min_p, const float* uniform,
                                int* out, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (!logits || !out || vocab <= 0 || ld < vocab) return ARLE_E_BADARG;
  if (temperature && !uniform) return ARLE_E_BADARG;
  // with no temperatures every row is greedy and the array is not touched: any size goes
  if (temperature && (long long)rows * (long long)vocab > (long long)ARLE_SAMPLE_STATIC_MAX_FLOATS) return ARLE_E_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  // Nothing in the scratch has to start at zero: the kernel writes every
  // probability of a row before it reads any, so the last call's leftovers are
  // overwritten, not cleared.
  launch_kernel(sample_kernel, dim3(rows), dim3(kSampleThreads), 0, s, 1, logits, ld, vocab, temperature, top_k, top_p, min_p, uniform,
                                                scratch, out);
  return launch_status();
}
