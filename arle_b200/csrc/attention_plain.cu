// General paged causal attention: any head size up to 256, any page size, any
// number of heads and groups, float32 or bfloat16 storage, float32 arithmetic
// throughout (scores, softmax, P.V; P is not rounded before P.V).  It serves the
// 32-bit path of the engine and is the yardstick of the tensor-core kernels.
//
// One block per (token, query head).  The query at absolute position p of request
// row r sees keys j in [max(0, p - window + 1), p] (window <= 0: from 0), found
// through the row's block table.  Warp w takes key tiles w, w+4, ... of 32 keys
// counted from the first visible key, keeps an online softmax (m, l, acc), and
// the four partial results are merged at the end.  The order of all sums depends
// on (first key, p) only, so a token's result is the same however the prompt was
// cut into steps and whatever else is in the batch.
#include "common.cuh"
using namespace arle;

constexpr int kAttnWarps = 4;
constexpr int kAttnMaxD = 8;  // head_dim <= 256

template <typename T>
__global__ void paged_attention_plain_kernel(const T* __restrict__ q, int q_row_stride, T* __restrict__ out,
                                             const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                                             const int* __restrict__ positions,
                                             const int* __restrict__ row_of_token,
                                             const int* __restrict__ block_table, int bt_stride, int nq,
                                             int nkv, int hd, int page_size, float scale, int window) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float qs[256];
  __shared__ float acc_s[kAttnWarps][256];
  __shared__ float m_s[kAttnWarps], l_s[kAttnWarps];
  const int t = blockIdx.x, h = blockIdx.y;
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = h / (nq / nkv);
  const int pos = positions[t];
  const int* bt = block_table + (size_t)row_of_token[t] * bt_stride;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

  const T* qp = q + (size_t)t * q_row_stride + (size_t)h * hd;
  for (int e = threadIdx.x; e < hd; e += blockDim.x) qs[e] = to_f32(qp[e]) * scale;
  __syncthreads();

  float m = -INFINITY, l = 0.f;
  float acc[kAttnMaxD];
#pragma unroll
  for (int i = 0; i < kAttnMaxD; ++i) acc[i] = 0.f;

  const size_t page_stride = (size_t)nkv * page_size * hd;
  for (int j0 = lo + w * 32; j0 <= pos; j0 += kAttnWarps * 32) {
    const int j = j0 + lane;
    float sc = -INFINITY;
    if (j <= pos) {
      const int page = bt[j / page_size];
      const T* kp = k_cache + (size_t)page * page_stride + ((size_t)kvh * page_size + j % page_size) * hd;
      float d = 0.f;
      for (int e = 0; e < hd; ++e) d = fmaf(qs[e], to_f32(kp[e]), d);
      sc = d;
    }
    const float mt = warp_max(sc);
    const float m_new = fmaxf(m, mt);
    const float p = j <= pos ? expf(sc - m_new) : 0.f;
    const float corr = expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < kAttnMaxD; ++i) acc[i] *= corr;
    m = m_new;
    const int nvalid = min(32, pos - j0 + 1);
    for (int jj = 0; jj < nvalid; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int jk = j0 + jj;
      const int page = bt[jk / page_size];
      const T* vp = v_cache + (size_t)page * page_stride + ((size_t)kvh * page_size + jk % page_size) * hd;
#pragma unroll
      for (int i = 0; i < kAttnMaxD; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] = fmaf(pj, to_f32(vp[d]), acc[i]);
      }
    }
  }
  if (lane == 0) {
    m_s[w] = m;
    l_s[w] = l;
  }
#pragma unroll
  for (int i = 0; i < kAttnMaxD; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) acc_s[w][d] = acc[i];
  }
  __syncthreads();
  float mm = m_s[0];
  for (int i = 1; i < kAttnWarps; ++i) mm = fmaxf(mm, m_s[i]);
  float f[kAttnWarps], ll = 0.f;
  for (int i = 0; i < kAttnWarps; ++i) {
    f[i] = expf(m_s[i] - mm);  // a warp without keys has m = -inf, so f = 0
    ll += l_s[i] * f[i];
  }
  T* op = out + ((size_t)t * nq + h) * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float o = 0.f;
    for (int i = 0; i < kAttnWarps; ++i) o += acc_s[i][d] * f[i];
    op[d] = from_f32<T>(o / ll);
  }
}

ARLE_API int arle_paged_attention_plain(const void* q, int q_row_stride, void* out, const void* k_cache,
                                        const void* v_cache, int dtype, const int* positions,
                                        const int* row_of_token, const int* block_table, int bt_stride,
                                        int nq, int nkv, int hd, int page_size, float scale, int window,
                                        int num_tokens, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (hd <= 0 || hd > 256 || nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0) return ARLE_E_UNSUPPORTED;
  if (nq > 65535) return ARLE_E_UNSUPPORTED;
  dim3 grid(num_tokens, nq);
  if (dtype == 0)
    launch_kernel(paged_attention_plain_kernel<float>, dim3(grid), dim3(kAttnWarps * 32), 0, s, 1, 
        (const float*)q, q_row_stride, (float*)out, (const float*)k_cache, (const float*)v_cache, positions,
        row_of_token, block_table, bt_stride, nq, nkv, hd, page_size, scale, window);
  else if (dtype == 1)
    launch_kernel(paged_attention_plain_kernel<__nv_bfloat16>, dim3(grid), dim3(kAttnWarps * 32), 0, s, 1, 
        (const __nv_bfloat16*)q, q_row_stride, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_cache,
        (const __nv_bfloat16*)v_cache, positions, row_of_token, block_table, bt_stride, nq, nkv, hd,
        page_size, scale, window);
  else
    return ARLE_E_BADARG;
  return launch_status();
}
