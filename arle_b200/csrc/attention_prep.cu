// Per-head q/k RMSNorm + rotary position encoding + paged KV store, one pass.
//
// Input is the packed projection output qkv[t, :] = [q heads | k heads | v heads]
// (row stride given).  One warp handles one (token, head):
//   q head: x <- rmsnorm_over_head(x; q_weight, eps) (if q_weight), rotate, store in place
//   k head: the same with k_weight, then store into k_cache at the token's slot
//   v head: copy into v_cache at the token's slot (no norm, no rotation)
// Norm statistics, the product x * inv * w and the rotation stay in float32; the
// angle of pair i at position p is p * inv_freq[i], evaluated with sincosf in
// float32.  Rotation pairs element i with i + rotary_dim/2 ("half split") inside
// the first rotary_dim elements of the head; the rest passes through.
// Cache layout: [page][kv_head][slot_in_page][head_dim]; slot_mapping[t] is
// page * page_size + slot_in_page, negative = do not store.
#include "common.cuh"
using namespace arle;

constexpr int kPrepWarps = 4;
constexpr int kMaxHeadDim = 256;

template <typename T>
__global__ void attention_prep_kernel(T* __restrict__ qkv, int row_stride,
                                      const int* __restrict__ positions,
                                      const int* __restrict__ slot_mapping,
                                      const float* __restrict__ q_weight,
                                      const float* __restrict__ k_weight, float eps,
                                      const float* __restrict__ inv_freq, int rotary_dim,
                                      T* __restrict__ k_cache, T* __restrict__ v_cache, int nq, int nkv,
                                      int hd, int page_size, int num_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float bufs[kPrepWarps][kMaxHeadDim];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = nq + 2 * nkv;
  const long long unit = (long long)blockIdx.x * kPrepWarps + w;
  if (unit >= (long long)num_tokens * heads) return;
  const int t = (int)(unit / heads), h = (int)(unit % heads);
  T* src = qkv + (size_t)t * row_stride + (size_t)h * hd;
  const int kind = h < nq ? 0 : (h < nq + nkv ? 1 : 2);
  const int kvh = kind == 1 ? h - nq : h - nq - nkv;

  size_t cache_base = 0;
  bool store = false;
  if (kind != 0) {
    const int slot = slot_mapping[t];
    if (slot >= 0) {
      const int page = slot / page_size, off = slot - page * page_size;
      cache_base = (((size_t)page * nkv + kvh) * page_size + off) * hd;
      store = true;
    }
  }
  if (kind == 2) {
    if (store)
      for (int e = lane; e < hd; e += 32) v_cache[cache_base + e] = src[e];
    return;
  }
  float* buf = bufs[w];
  const float* wt = kind == 0 ? q_weight : k_weight;
  float ss = 0.f;
  for (int e = lane; e < hd; e += 32) {
    const float x = to_f32(src[e]);
    buf[e] = x;
    ss += x * x;
  }
  if (wt) {
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
    for (int e = lane; e < hd; e += 32) buf[e] = buf[e] * inv * wt[e];
  }
  __syncwarp();
  const float pos = (float)positions[t];
  const int half = rotary_dim >> 1;
  for (int e = lane; e < hd; e += 32) {
    float o;
    if (e < rotary_dim) {
      const int i = e < half ? e : e - half;
      float sn, cs;
      sincosf(pos * inv_freq[i], &sn, &cs);
      o = e < half ? buf[e] * cs - buf[e + half] * sn : buf[e - half] * sn + buf[e] * cs;
    } else {
      o = buf[e];
    }
    if (kind == 0)
      src[e] = from_f32<T>(o);
    else if (store)
      k_cache[cache_base + e] = from_f32<T>(o);
  }
}

// Head sizes 64 and 128 with whole-head rotation, bfloat16: every lane keeps
// hd/32 consecutive elements in registers (one 4- or 8-byte access), the norm's
// sum is a warp reduction and the rotation partner (element i +- hd/2) lives in
// lane ^ 16, so no shared memory is touched.  Same arithmetic as the general
// kernel.
template <int HD>
__global__ void attention_prep_bf16_kernel(__nv_bfloat16* __restrict__ qkv, int row_stride,
                                           const int* __restrict__ positions, const int* __restrict__ slot_mapping,
                                           const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                                           float eps, const float* __restrict__ inv_freq,
                                           __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                           int nq, int nkv, int page_size, int num_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int VE = HD / 32;                   // elements per lane: 2 or 4
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = nq + 2 * nkv;
  const long long unit = (long long)blockIdx.x * kPrepWarps + w;
  if (unit >= (long long)num_tokens * heads) return;
  const int t = (int)(unit / heads), h = (int)(unit % heads);
  __nv_bfloat16* src = qkv + (size_t)t * row_stride + (size_t)h * HD + lane * VE;
  const int kind = h < nq ? 0 : (h < nq + nkv ? 1 : 2);
  const int kvh = kind == 1 ? h - nq : h - nq - nkv;
  size_t cache_at = 0;
  bool store = false;
  if (kind != 0) {
    const int slot = slot_mapping[t];
    if (slot >= 0) {
      const int page = slot / page_size, off = slot - page * page_size;
      cache_at = (((size_t)page * nkv + kvh) * page_size + off) * HD + lane * VE;
      store = true;
    }
  }
  uint32_t raw[VE / 2];
  if (VE == 4) {
    const uint2 u = *reinterpret_cast<const uint2*>(src);
    raw[0] = u.x;
    raw[VE / 2 - 1] = u.y;
  } else {
    raw[0] = *reinterpret_cast<const uint32_t*>(src);
  }
  if (kind == 2) {
    if (store) {
      if (VE == 4) *reinterpret_cast<uint2*>(v_cache + cache_at) = make_uint2(raw[0], raw[VE / 2 - 1]);
      else *reinterpret_cast<uint32_t*>(v_cache + cache_at) = raw[0];
    }
    return;
  }
  float x[VE];
#pragma unroll
  for (int i = 0; i < VE / 2; ++i) {
    const __nv_bfloat162 p = *reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
    x[2 * i] = __low2float(p);
    x[2 * i + 1] = __high2float(p);
  }
  const float* wt = kind == 0 ? q_weight : k_weight;
  if (wt) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VE; ++i) ss += x[i] * x[i];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
    for (int i = 0; i < VE; ++i) x[i] = x[i] * inv * wt[lane * VE + i];
  }
  const float pos = (float)positions[t];
  float o[VE];
#pragma unroll
  for (int i = 0; i < VE; ++i) {
    const float other = __shfl_xor_sync(0xffffffffu, x[i], 16);
    const int fi = (lane & 15) * VE + i;        // index of the pair
    float sn, cs;
    sincosf(pos * inv_freq[fi], &sn, &cs);
    o[i] = lane < 16 ? x[i] * cs - other * sn : other * sn + x[i] * cs;
  }
  uint32_t packed[VE / 2];
#pragma unroll
  for (int i = 0; i < VE / 2; ++i) {
    __nv_bfloat162 p = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
    packed[i] = *reinterpret_cast<uint32_t*>(&p);
  }
  __nv_bfloat16* dst = kind == 0 ? src : (store ? k_cache + cache_at : nullptr);
  if (dst) {
    if (VE == 4) *reinterpret_cast<uint2*>(dst) = make_uint2(packed[0], packed[VE / 2 - 1]);
    else *reinterpret_cast<uint32_t*>(dst) = packed[0];
  }
}

// The same for many tokens (prompt portions).  One block per token: the cosines and sines
// of the token's position are computed once (they are the same for every head) and the
// block's warps then take the heads in turn.  Every lane keeps hd/32
// consecutive elements in registers (one 4- or 8-byte access), the norm's sum is a warp
// reduction and the rotation partner (element i +- hd/2) lives in lane ^ 16, so the heads
// themselves never touch shared memory.  Same arithmetic as the general kernel.
constexpr int kPrepVecWarps = 8;

template <int HD>
__global__ void __launch_bounds__(kPrepVecWarps * 32) attention_prep_bf16_token_kernel(
    __nv_bfloat16* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
    const int* __restrict__ slot_mapping, const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
    const float* __restrict__ inv_freq, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int nq,
    int nkv, int page_size, int num_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int VE = HD / 32;                   // elements per lane: 2 or 4
  __shared__ float cs_s[HD / 2], sn_s[HD / 2];
  const int t = blockIdx.x;
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x < HD / 2) {
    float sn, cs;
    sincosf((float)positions[t] * inv_freq[threadIdx.x], &sn, &cs);
    cs_s[threadIdx.x] = cs;
    sn_s[threadIdx.x] = sn;
  }
  __syncthreads();
  const int heads = nq + 2 * nkv;
  const int slot = nkv > 0 ? slot_mapping[t] : -1;
  const int page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? slot - page * page_size : 0;
  float cs[VE], sn[VE];
#pragma unroll
  for (int i = 0; i < VE; ++i) {
    cs[i] = cs_s[(lane & 15) * VE + i];
    sn[i] = sn_s[(lane & 15) * VE + i];
  }
  for (int h = w; h < heads; h += kPrepVecWarps) {
    __nv_bfloat16* src = qkv + (size_t)t * row_stride + (size_t)h * HD + lane * VE;
    const int kind = h < nq ? 0 : (h < nq + nkv ? 1 : 2);
    const int kvh = kind == 1 ? h - nq : h - nq - nkv;
    const bool store = kind != 0 && slot >= 0;
    const size_t cache_at = store ? (((size_t)page * nkv + kvh) * page_size + off) * HD + lane * VE : 0;
    uint32_t raw[VE / 2];
    if (VE == 4) {
      const uint2 u = *reinterpret_cast<const uint2*>(src);
      raw[0] = u.x;
      raw[VE / 2 - 1] = u.y;
    } else {
      raw[0] = *reinterpret_cast<const uint32_t*>(src);
    }
    if (kind == 2) {
      if (store) {
        if (VE == 4) *reinterpret_cast<uint2*>(v_cache + cache_at) = make_uint2(raw[0], raw[VE / 2 - 1]);
        else *reinterpret_cast<uint32_t*>(v_cache + cache_at) = raw[0];
      }
      continue;
    }
    float x[VE];
#pragma unroll
    for (int i = 0; i < VE / 2; ++i) {
      const __nv_bfloat162 p = *reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
      x[2 * i] = __low2float(p);
      x[2 * i + 1] = __high2float(p);
    }
    const float* wt = kind == 0 ? q_weight : k_weight;
    if (wt) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < VE; ++i) ss += x[i] * x[i];
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
      for (int i = 0; i < VE; ++i) x[i] = x[i] * inv * wt[lane * VE + i];
    }
    float o[VE];
#pragma unroll
    for (int i = 0; i < VE; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, x[i], 16);
      o[i] = lane < 16 ? x[i] * cs[i] - other * sn[i] : other * sn[i] + x[i] * cs[i];
    }
    uint32_t packed[VE / 2];
#pragma unroll
    for (int i = 0; i < VE / 2; ++i) {
      __nv_bfloat162 p = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
      packed[i] = *reinterpret_cast<uint32_t*>(&p);
    }
    __nv_bfloat16* dst = kind == 0 ? src : (store ? k_cache + cache_at : nullptr);
    if (dst) {
      if (VE == 4) *reinterpret_cast<uint2*>(dst) = make_uint2(packed[0], packed[VE / 2 - 1]);
      else *reinterpret_cast<uint32_t*>(dst) = packed[0];
    }
  }
}

ARLE_API int arle_attention_prep(void* qkv, int dtype, int row_stride, const int* positions,
                                 const int* slot_mapping, const float* q_weight, const float* k_weight,
                                 float eps, const float* inv_freq, int rotary_dim, void* k_cache,
                                 void* v_cache, int nq, int nkv, int hd, int page_size, int num_tokens,
                                 cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (hd <= 0 || hd > kMaxHeadDim || nq < 0 || nkv < 0 || nq + nkv == 0) return ARLE_E_UNSUPPORTED;
  if (rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1)) return ARLE_E_BADARG;
  if (rotary_dim > 0 && !inv_freq) return ARLE_E_BADARG;
  if (nkv > 0 && (!k_cache || !v_cache || !slot_mapping || page_size <= 0)) return ARLE_E_BADARG;
  const long long units = (long long)num_tokens * (nq + 2 * nkv);
  const long long blocks = (units + kPrepWarps - 1) / kPrepWarps;
  if (blocks > 0x7fffffffLL) return ARLE_E_UNSUPPORTED;
  if (dtype == 1 && (hd == 64 || hd == 128) && rotary_dim == hd && row_stride % 4 == 0 && ((uintptr_t)qkv & 7) == 0 &&
      ((uintptr_t)k_cache & 7) == 0 && ((uintptr_t)v_cache & 7) == 0) {
    if (num_tokens >= 32) {                      // enough tokens to fill the GPU with one block each
      if (hd == 128)
        launch_kernel(attention_prep_bf16_token_kernel<128>, dim3(num_tokens), dim3(kPrepVecWarps * 32), 0, s, 1,
                      (__nv_bfloat16*)qkv, row_stride, positions, slot_mapping, q_weight, k_weight, eps, inv_freq,
                      (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nq, nkv, page_size, num_tokens);
      else
        launch_kernel(attention_prep_bf16_token_kernel<64>, dim3(num_tokens), dim3(kPrepVecWarps * 32), 0, s, 1,
                      (__nv_bfloat16*)qkv, row_stride, positions, slot_mapping, q_weight, k_weight, eps, inv_freq,
                      (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nq, nkv, page_size, num_tokens);
      return launch_status();
    }
    if (hd == 128)
      launch_kernel(attention_prep_bf16_kernel<128>, dim3((int)blocks), dim3(kPrepWarps * 32), 0, s, 1, 
          (__nv_bfloat16*)qkv, row_stride, positions, slot_mapping, q_weight, k_weight, eps, inv_freq,
          (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nq, nkv, page_size, num_tokens);
    else
      launch_kernel(attention_prep_bf16_kernel<64>, dim3((int)blocks), dim3(kPrepWarps * 32), 0, s, 1, 
          (__nv_bfloat16*)qkv, row_stride, positions, slot_mapping, q_weight, k_weight, eps, inv_freq,
          (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nq, nkv, page_size, num_tokens);
    return launch_status();
  }
  if (dtype == 0)
    launch_kernel(attention_prep_kernel<float>, dim3((int)blocks), dim3(kPrepWarps * 32), 0, s, 1, 
        (float*)qkv, row_stride, positions, slot_mapping, q_weight, k_weight, eps, inv_freq, rotary_dim,
        (float*)k_cache, (float*)v_cache, nq, nkv, hd, page_size, num_tokens);
  else if (dtype == 1)
    launch_kernel(attention_prep_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(kPrepWarps * 32), 0, s, 1, 
        (__nv_bfloat16*)qkv, row_stride, positions, slot_mapping, q_weight, k_weight, eps, inv_freq,
        rotary_dim, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nq, nkv, hd, page_size, num_tokens);
  else
    return ARLE_E_BADARG;
  return launch_status();
}
