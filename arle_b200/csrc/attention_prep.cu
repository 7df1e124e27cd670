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
// of the token's position are taken from the step's table (or computed once per block: they
// are the same for every head) and the block's warps then take the heads in turn.  A lane
// holds four consecutive elements of the head's first half and their rotation partners in
// the second half (two 8-byte accesses), so the rotation needs no exchange between lanes;
// hd / 8 lanes make a head and a warp takes 32 / (hd / 8) heads at a time; the norm's sum is
// a reduction over those lanes.  All of a warp's loads are asked for before the first is
// used.  Same arithmetic as the general kernel.
constexpr int kPrepVecWarps = 8;
constexpr int kPrepMaxPasses = 3;               // heads a warp takes, in passes, with its loads batched (more: in further rounds)

template <int HD>
__global__ void __launch_bounds__(kPrepVecWarps * 32, 4) attention_prep_bf16_token_kernel(
    __nv_bfloat16* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
    const int* __restrict__ slot_mapping, const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
    const float* __restrict__ inv_freq, const float2* __restrict__ angles, __nv_bfloat16* __restrict__ k_cache,
    __nv_bfloat16* __restrict__ v_cache, int nq, int nkv, int page_size, int num_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int LPH = HD / 8;                   // lanes per head: 16 or 8
  constexpr int HPW = 32 / LPH;                 // heads per warp and pass: 2 or 4
  constexpr int HALF = HD / 2;
  __shared__ float cs_s[HALF], sn_s[HALF];
  const int t = blockIdx.x;
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (!angles && threadIdx.x < HALF) {
    float sn, cs;
    sincosf((float)positions[t] * inv_freq[threadIdx.x], &sn, &cs);
    cs_s[threadIdx.x] = cs;
    sn_s[threadIdx.x] = sn;
  }
  const int heads = nq + 2 * nkv;
  const int sub = lane / LPH, l = lane % LPH;   // head of the pass, lane within the head
  const int e0 = l * 4;                         // this lane's elements: e0 .. e0 + 3 and HALF + e0 .. HALF + e0 + 3
  const int slot = nkv > 0 ? slot_mapping[t] : -1;
  const int page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? slot - page * page_size : 0;
  __nv_bfloat16* row = qkv + (size_t)t * row_stride + e0;
  const int stride_h = kPrepVecWarps * HPW;     // heads the block takes per pass
  uint2 lo[kPrepMaxPasses], hi[kPrepMaxPasses];
  auto fetch = [&](int h0) {
#pragma unroll
    for (int p = 0; p < kPrepMaxPasses; ++p) {
      const int h = h0 + p * stride_h;
      lo[p] = h < heads ? *reinterpret_cast<const uint2*>(row + (size_t)h * HD) : make_uint2(0, 0);
      hi[p] = h < heads ? *reinterpret_cast<const uint2*>(row + (size_t)h * HD + HALF) : make_uint2(0, 0);
    }
  };
  fetch(w * HPW + sub);                         // under way while the cosines and sines are fetched or computed
  float cs[4], sn[4];
  if (angles) {
    // the step's table (the same for every layer): (cos, sin) of this token's hd / 2 angles
    const float4* a4 = reinterpret_cast<const float4*>(angles + (size_t)t * HALF + e0);
    const float4 v0 = a4[0], v1 = a4[1];
    cs[0] = v0.x, sn[0] = v0.y, cs[1] = v0.z, sn[1] = v0.w;
    cs[2] = v1.x, sn[2] = v1.y, cs[3] = v1.z, sn[3] = v1.w;
  } else {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) cs[i] = cs_s[e0 + i], sn[i] = sn_s[e0 + i];
  }
  // the loop's condition is the same for all lanes of a warp: lanes without a head take part in the shuffles
  for (int hb = w * HPW; hb < heads; hb += stride_h * kPrepMaxPasses) {
    const int h0 = hb + sub;
    if (hb != w * HPW) fetch(h0);
#pragma unroll
    for (int p = 0; p < kPrepMaxPasses; ++p) {
      const int h = h0 + p * stride_h;
      const bool live = h < heads;
      const bool is_q = h < nq, is_v = h >= nq + nkv;
      const bool store = live && !is_q && slot >= 0;
      const size_t cache_at = store ? (((size_t)page * nkv + (is_v ? h - nq - nkv : h - nq)) * page_size + off) * HD + e0 : 0;
      if (is_v && store) {
        *reinterpret_cast<uint2*>(v_cache + cache_at) = lo[p];
        *reinterpret_cast<uint2*>(v_cache + cache_at + HALF) = hi[p];
      }
      if (__all_sync(0xffffffffu, is_v || !live)) continue;      // nothing to norm or rotate in this pass
      float a[4], b[4];                          // first half, second half
      {
        const __nv_bfloat162 a0 = *reinterpret_cast<const __nv_bfloat162*>(&lo[p].x), a1 = *reinterpret_cast<const __nv_bfloat162*>(&lo[p].y);
        const __nv_bfloat162 b0 = *reinterpret_cast<const __nv_bfloat162*>(&hi[p].x), b1 = *reinterpret_cast<const __nv_bfloat162*>(&hi[p].y);
        a[0] = __low2float(a0), a[1] = __high2float(a0), a[2] = __low2float(a1), a[3] = __high2float(a1);
        b[0] = __low2float(b0), b[1] = __high2float(b0), b[2] = __low2float(b1), b[3] = __high2float(b1);
      }
      const float* wt = is_q ? q_weight : k_weight;
      // The sum of squares in the order of the other preparation kernels (a warp per head, hd / 32 consecutive
      // elements per lane, butterfly over lane distances 16, 8, 4, 2, 1), so that a key prepared here has the
      // bits of one prepared there.  This lane holds the elements of 4 / VE of that warp's lanes in each half:
      // t[s] is what its lane l * S + s holds after the first step (which adds the two halves).  All lanes
      // take part, whether their head has a norm or not: the two heads of a pass may differ in that.
      constexpr int VE = HD / 32, S = 4 / VE;
      float t[S];
#pragma unroll
      for (int st = 0; st < S; ++st) {
        float pa = 0.f, pb = 0.f;
#pragma unroll
        for (int i = 0; i < VE; ++i) pa += a[st * VE + i] * a[st * VE + i], pb += b[st * VE + i] * b[st * VE + i];
        t[st] = pa + pb;
      }
#pragma unroll
      for (int d = 8; d > 0; d >>= 1) {
        if (d >= S) {
#pragma unroll
          for (int st = 0; st < S; ++st) t[st] += __shfl_xor_sync(0xffffffffu, t[st], d / S);
        } else {
          float u[S];
#pragma unroll
          for (int st = 0; st < S; ++st) u[st] = t[st] + t[st ^ d];
#pragma unroll
          for (int st = 0; st < S; ++st) t[st] = u[st];
        }
      }
      const float ss = t[0];
      if (wt) {
        const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
        const float4 ga = *reinterpret_cast<const float4*>(wt + e0), gb = *reinterpret_cast<const float4*>(wt + HALF + e0);
        a[0] = a[0] * inv * ga.x, a[1] = a[1] * inv * ga.y, a[2] = a[2] * inv * ga.z, a[3] = a[3] * inv * ga.w;
        b[0] = b[0] * inv * gb.x, b[1] = b[1] * inv * gb.y, b[2] = b[2] * inv * gb.z, b[3] = b[3] * inv * gb.w;
      }
      float oa[4], ob[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        oa[i] = a[i] * cs[i] - b[i] * sn[i];
        ob[i] = a[i] * sn[i] + b[i] * cs[i];
      }
      if (live && !is_v) {
        __nv_bfloat16* dst = is_q ? row + (size_t)h * HD : (store ? k_cache + cache_at : nullptr);
        if (dst) {
          __nv_bfloat162 p0 = __floats2bfloat162_rn(oa[0], oa[1]), p1 = __floats2bfloat162_rn(oa[2], oa[3]);
          __nv_bfloat162 q0 = __floats2bfloat162_rn(ob[0], ob[1]), q1 = __floats2bfloat162_rn(ob[2], ob[3]);
          *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1));
          *reinterpret_cast<uint2*>(dst + HALF) = make_uint2(*reinterpret_cast<uint32_t*>(&q0), *reinterpret_cast<uint32_t*>(&q1));
        }
      }
    }
  }
}

// out[t][i] = (cos, sin)(positions[t] * inv_freq[i]): what every layer of a step would evaluate again.
__global__ void rotary_angles_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                     float2* __restrict__ out, int half, long long total) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int t = (int)(i / half), f = (int)(i - (long long)t * half);
  float sn, cs;
  sincosf((float)positions[t] * inv_freq[f], &sn, &cs);
  out[i] = make_float2(cs, sn);
}

// angles: float32 [num_tokens, half, 2], (cos, sin) of position * inv_freq in float32, as the preparation kernels
// evaluate them.
ARLE_API int arle_rotary_angles(const int* positions, const float* inv_freq, float* angles, int num_tokens, int half,
                                cudaStream_t s) {
  if (num_tokens <= 0 || half <= 0) return 0;
  const long long total = (long long)num_tokens * half;
  launch_kernel(rotary_angles_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, 1, positions, inv_freq,
                reinterpret_cast<float2*>(angles), half, total);
  return launch_status();
}

// angles (may be null): the table of arle_rotary_angles for these positions and inv_freq; kernels that can use it
// then skip the evaluation of the angles (16-byte aligned).
ARLE_API int arle_attention_prep(void* qkv, int dtype, int row_stride, const int* positions,
                                 const int* slot_mapping, const float* q_weight, const float* k_weight,
                                 float eps, const float* inv_freq, const float* angles, int rotary_dim, void* k_cache,
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
    const bool wide = row_stride % 8 == 0 && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)k_cache & 15) == 0 &&
                      ((uintptr_t)v_cache & 15) == 0 && (!q_weight || ((uintptr_t)q_weight & 15) == 0) &&
                      (!k_weight || ((uintptr_t)k_weight & 15) == 0);      // 16-byte accesses
    if (num_tokens >= 32 && wide) {              // enough tokens to fill the GPU with one block each
      const float2* tab = ((uintptr_t)angles & 15) == 0 ? reinterpret_cast<const float2*>(angles) : nullptr;
      if (hd == 128)
        launch_kernel(attention_prep_bf16_token_kernel<128>, dim3(num_tokens), dim3(kPrepVecWarps * 32), 0, s, 1,
                      (__nv_bfloat16*)qkv, row_stride, positions, slot_mapping, q_weight, k_weight, eps, inv_freq, tab,
                      (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nq, nkv, page_size, num_tokens);
      else
        launch_kernel(attention_prep_bf16_token_kernel<64>, dim3(num_tokens), dim3(kPrepVecWarps * 32), 0, s, 1,
                      (__nv_bfloat16*)qkv, row_stride, positions, slot_mapping, q_weight, k_weight, eps, inv_freq, tab,
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
