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
  if (dtype == 0)
    attention_prep_kernel<float><<<(int)blocks, kPrepWarps * 32, 0, s>>>(
        (float*)qkv, row_stride, positions, slot_mapping, q_weight, k_weight, eps, inv_freq, rotary_dim,
        (float*)k_cache, (float*)v_cache, nq, nkv, hd, page_size, num_tokens);
  else if (dtype == 1)
    attention_prep_kernel<__nv_bfloat16><<<(int)blocks, kPrepWarps * 32, 0, s>>>(
        (__nv_bfloat16*)qkv, row_stride, positions, slot_mapping, q_weight, k_weight, eps, inv_freq,
        rotary_dim, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nq, nkv, hd, page_size, num_tokens);
  else
    return ARLE_E_BADARG;
  return launch_status();
}
