// Split-KV paged attention for decoded tokens (one query per request), bfloat16,
// head sizes 64 and 128, up to 16 query heads per kv head.
//
// Decoding reads every key and value of a request once and does little arithmetic
// per byte, so the kernel is built to stream the cache at HBM speed:
//   grid = (request rows, kv heads, splits).  A CTA owns one kv head of one
//   request and one contiguous chunk of its keys, and serves all G query heads
//   of that kv head at once, so each key/value byte is read once per step.
//   Keys and values come in tiles of 64 through cp.async into double-buffered,
//   padded shared memory (each row found through the block table, any page size);
//   warp w takes keys 16w..16w+15 of the tile.  Q.K^T and P.V run on the tensor
//   cores (mma.sync m16n8k16, the G query heads padded to the 16 rows of the A
//   operand); scores, the online softmax and the accumulators are float32, P is
//   rounded to bfloat16 for P.V as in cklxx/arle's decode kernel
//   (crates/cuda-kernels/tools/tilelang/batch_decode_paged_hd128.py:134-231).
//   The four warps' partial results are merged in shared memory; with more than
//   one split the CTA writes an unnormalised partial (o, m, l), and the split that
//   finishes last (a counter per request and kv head) combines them in the same
//   launch (FlashDecoding; the reference's split-KV variant uses a second kernel,
//   :239-463).
// Rows whose step entry has more than one token are skipped (the prefill kernel
// takes them).  The key range of a row is [max(0, kv_len - window), kv_len).
#include "common.cuh"
#include "mma_utils.cuh"
using namespace arle;

namespace {

constexpr int kThreads = 128;
constexpr int kTile = 64;   // keys per tile

template <int HD>
__global__ void __launch_bounds__(kThreads) paged_decode_kernel(
    const __nv_bfloat16* __restrict__ q, int q_row_stride, __nv_bfloat16* __restrict__ out,
    const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
    const int* __restrict__ q_indptr, const int* __restrict__ kv_lens, const int* __restrict__ block_table,
    int bt_stride, float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters, int nq, int nkv,
    int page_size, int ps_shift, float scale_log2, int window, int splits) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int ROW = HD + 8;                 // padded row, in elements: 16 B more keeps ldmatrix conflict-free
  constexpr int CHUNKS = HD / 8;              // 16-byte chunks per row
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);          // [2][kTile][ROW]
  __nv_bfloat16* vs = ks + 2 * kTile * ROW;                                // [2][kTile][ROW]
  __nv_bfloat16* qs = vs + 2 * kTile * ROW;                                // [16][ROW]
  __shared__ int pgbuf[4][kTile + 1];          // page ids of four tiles in turn, fetched two tiles ahead of the data

  const int r = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int G = nq / nkv;
  const int t = q_indptr[r];
  if (q_indptr[r + 1] - t != 1) return;
  const int kv_len = kv_lens[r];
  const int lo = (window > 0 && kv_len > window) ? kv_len - window : 0;
  const int span = kv_len - lo;
  const int chunk = ((span + splits - 1) / splits + kTile - 1) / kTile * kTile;
  const int beg = lo + split * chunk;
  const int end = min(beg + chunk, kv_len);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;

  const bool empty = beg >= end;               // nothing for this split: it publishes an empty partial
  if (empty) {
    if (tid < G) {
      float* ml = part_ml + (((size_t)r * nq + kvh * G + tid) * splits + split) * 2;
      ml[0] = -INFINITY;
      ml[1] = 0.f;
    }
  } else {
  const int* bt = block_table + (size_t)r * bt_stride;
  const size_t head_stride = (size_t)page_size * HD;
  const size_t page_stride = (size_t)nkv * head_stride;
  const __nv_bfloat16* kbase = k_cache + (size_t)kvh * head_stride;
  const __nv_bfloat16* vbase = v_cache + (size_t)kvh * head_stride;

  // Page ids of a tile go to shared memory two tiles before its keys are fetched, so that
  // fetching a tile does not first wait for a block-table read.
  auto fetch_ids = [&](int tile, bool async) {
    const int k0 = beg + tile * kTile;
    if (k0 >= end) return;
    const int first = k0 / page_size, last = (min(end, k0 + kTile) - 1) / page_size;
    if (tid <= last - first) {
      if (async) cp_async4(smem_u32(&pgbuf[tile & 3][tid]), bt + first + tid, 4);
      else pgbuf[tile & 3][tid] = bt[first + tid];
    }
  };
  auto load_tile = [&](int tile, int stage) {
    const int k0 = beg + tile * kTile;
    const int first = ps_shift >= 0 ? (k0 >> ps_shift) : k0 / page_size;
    const int* pg = pgbuf[tile & 3];
    __nv_bfloat16* kd = ks + stage * kTile * ROW;
    __nv_bfloat16* vd = vs + stage * kTile * ROW;
#pragma unroll
    for (int i = 0; i < kTile * CHUNKS / kThreads; ++i) {
      const int c = tid + i * kThreads;
      const int key = c / CHUNKS, part = c % CHUNKS;
      const int kj = k0 + key;
      const bool ok = kj < end;
      size_t off = 0;
      if (ok) {
        const int pidx = ps_shift >= 0 ? (kj >> ps_shift) : kj / page_size;     // pages are mostly a power of two
        off = (size_t)pg[pidx - first] * page_stride + (size_t)(kj - pidx * page_size) * HD + part * 8;
      }
      cp_async16(smem_u32(kd + key * ROW + part * 8), kbase + off, ok ? 16 : 0);
      cp_async16(smem_u32(vd + key * ROW + part * 8), vbase + off, ok ? 16 : 0);
    }
  };

  const int ntiles = (end - beg + kTile - 1) / kTile;
  fetch_ids(0, false);
  fetch_ids(1, false);
  fetch_ids(2, false);
  __syncthreads();
  load_tile(0, 0);
  cp_commit();

  // the G query heads of this kv head into rows 0..G-1 of a 16-row tile, the rest zero
  for (int i = tid; i < 16 * CHUNKS; i += kThreads) {
    const int row = i / CHUNKS, part = i % CHUNKS;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < G) v = *reinterpret_cast<const uint4*>(q + (size_t)t * q_row_stride + (size_t)(kvh * G + row) * HD + part * 8);
    *reinterpret_cast<uint4*>(qs + row * ROW + part * 8) = v;
  }
  __syncthreads();
  uint32_t qa[HD / 16][4];
#pragma unroll
  for (int s = 0; s < HD / 16; ++s) {
    qa[s][0] = *reinterpret_cast<const uint32_t*>(qs + g * ROW + s * 16 + 2 * tq);
    qa[s][1] = *reinterpret_cast<const uint32_t*>(qs + (g + 8) * ROW + s * 16 + 2 * tq);
    qa[s][2] = *reinterpret_cast<const uint32_t*>(qs + g * ROW + s * 16 + 8 + 2 * tq);
    qa[s][3] = *reinterpret_cast<const uint32_t*>(qs + (g + 8) * ROW + s * 16 + 8 + 2 * tq);
  }

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows g and g+8

  for (int tile = 0; tile < ntiles; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < ntiles) {
      load_tile(tile + 1, stage ^ 1);
      fetch_ids(tile + 3, true);
      cp_commit();
      cp_wait<1>();
    } else {
      cp_wait<0>();
    }
    __syncthreads();
    const int kbeg = beg + tile * kTile + warp * 16;       // this warp's 16 keys
    if (kbeg < end) {
      const __nv_bfloat16* kt = ks + stage * kTile * ROW + warp * 16 * ROW;
      const __nv_bfloat16* vt = vs + stage * kTile * ROW + warp * 16 * ROW;
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(smem_u32(kt + ((lane >> 4) * 8 + (lane & 7)) * ROW + kk * 16 + ((lane >> 3) & 1) * 8), b0, b1, b2, b3);
        mma_bf16(s[0], qa[kk], b0, b1);
        mma_bf16(s[1], qa[kk], b2, b3);
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const int kj = kbeg + 8 * n + 2 * tq;
        s[n][0] = kj < end ? s[n][0] * scale_log2 : -INFINITY;
        s[n][1] = kj + 1 < end ? s[n][1] * scale_log2 : -INFINITY;
        s[n][2] = kj < end ? s[n][2] * scale_log2 : -INFINITY;
        s[n][3] = kj + 1 < end ? s[n][3] * scale_log2 : -INFINITY;
        mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
        mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);   // finite: key kbeg is valid
      const float c0 = exp2f(m0 - mn0), c1 = exp2f(m1 - mn1);
      m0 = mn0;
      m1 = mn1;
      uint32_t pa[4];
      float p[2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        p[n][0] = exp2f(s[n][0] - mn0);
        p[n][1] = exp2f(s[n][1] - mn0);
        p[n][2] = exp2f(s[n][2] - mn1);
        p[n][3] = exp2f(s[n][3] - mn1);
      }
      l0 = l0 * c0 + p[0][0] + p[0][1] + p[1][0] + p[1][1];
      l1 = l1 * c1 + p[0][2] + p[0][3] + p[1][2] + p[1][3];
      pa[0] = pack_bf16(p[0][0], p[0][1]);
      pa[1] = pack_bf16(p[0][2], p[0][3]);
      pa[2] = pack_bf16(p[1][0], p[1][1]);
      pa[3] = pack_bf16(p[1][2], p[1][3]);
#pragma unroll
      for (int dn = 0; dn < HD / 16; ++dn) {
        o[2 * dn][0] *= c0; o[2 * dn][1] *= c0; o[2 * dn][2] *= c1; o[2 * dn][3] *= c1;
        o[2 * dn + 1][0] *= c0; o[2 * dn + 1][1] *= c0; o[2 * dn + 1][2] *= c1; o[2 * dn + 1][3] *= c1;
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(smem_u32(vt + (((lane >> 3) & 1) * 8 + (lane & 7)) * ROW + dn * 16 + (lane >> 4) * 8), b0, b1, b2, b3);
        mma_bf16(o[2 * dn], pa, b0, b1);
        mma_bf16(o[2 * dn + 1], pa, b2, b3);
      }
    }
    __syncthreads();
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

  // merge the four warps (shared memory of the tiles is free now)
  float* mo = reinterpret_cast<float*>(smem_raw);       // [4][16][HD]
  float* mm = mo + 4 * 16 * HD;                         // [4][16] m, then [4][16] l
  float* mlv = mm + 64;
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) {
    *reinterpret_cast<float2*>(mo + ((warp * 16 + g) * HD) + i * 8 + 2 * tq) = make_float2(o[i][0], o[i][1]);
    *reinterpret_cast<float2*>(mo + ((warp * 16 + g + 8) * HD) + i * 8 + 2 * tq) = make_float2(o[i][2], o[i][3]);
  }
  if (tq == 0) {
    mm[warp * 16 + g] = m0;
    mm[warp * 16 + g + 8] = m1;
    mlv[warp * 16 + g] = l0;
    mlv[warp * 16 + g + 8] = l1;
  }
  __syncthreads();
  for (int i = tid; i < G * HD; i += kThreads) {
    const int row = i / HD, d = i % HD;
    float M = mm[row];
#pragma unroll
    for (int w = 1; w < 4; ++w) M = fmaxf(M, mm[w * 16 + row]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(mm[w * 16 + row] - M);      // a warp without keys has m = -inf: factor 0
      L += mlv[w * 16 + row] * f;
      O += mo[(w * 16 + row) * HD + d] * f;
    }
    const int head = kvh * G + row;
    if (splits == 1) {
      out[((size_t)t * nq + head) * HD + d] = __float2bfloat16_rn(O / L);
    } else {
      const size_t pidx = ((size_t)r * nq + head) * splits + split;
      part_o[pidx * HD + d] = O;
      if (d == 0) {
        part_ml[pidx * 2] = M;
        part_ml[pidx * 2 + 1] = L;
      }
    }
  }
  }  // !empty
  if (splits == 1) return;

  // The split that arrives last combines all of them:
  //   out = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M),  M = max_s m_s.
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int prev = atomicAdd(&counters[r * nkv + kvh], 1);
    is_last = prev == splits - 1;
    if (is_last) counters[r * nkv + kvh] = 0;            // ready for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  float* fac = reinterpret_cast<float*>(smem_raw);        // [G][splits] factors, then [G] 1 / L
  float* invl = fac + 16 * 64;
  for (int i = tid; i < G * splits; i += kThreads) {
    const int row = i / splits, sp = i % splits;
    fac[row * 64 + sp] = __ldcg(part_ml + (((size_t)r * nq + kvh * G + row) * splits + sp) * 2);
  }
  __syncthreads();
  if (tid < G) {
    float M = -INFINITY;
    for (int sp = 0; sp < splits; ++sp) M = fmaxf(M, fac[tid * 64 + sp]);
    float L = 0.f;
    for (int sp = 0; sp < splits; ++sp) {
      const float l = __ldcg(part_ml + (((size_t)r * nq + kvh * G + tid) * splits + sp) * 2 + 1);
      const float f = l > 0.f ? exp2f(fac[tid * 64 + sp] - M) : 0.f;
      fac[tid * 64 + sp] = f;
      L += l * f;
    }
    invl[tid] = 1.0f / L;
  }
  __syncthreads();
  for (int i = tid; i < G * HD; i += kThreads) {
    const int row = i / HD, d = i % HD;
    const float* po = part_o + ((size_t)r * nq + kvh * G + row) * splits * HD + d;
    float O = 0.f;
#pragma unroll 4
    for (int sp = 0; sp < splits; ++sp) {
      const float f = fac[row * 64 + sp];
      if (f > 0.f) O += __ldcg(po + (size_t)sp * HD) * f;
    }
    out[((size_t)t * nq + kvh * G + row) * HD + d] = __float2bfloat16_rn(O * invl[row]);
  }
}

template <int HD>
int launch_decode(const void* q, int q_row_stride, void* out, const void* k_cache, const void* v_cache,
                  const int* q_indptr, const int* kv_lens, const int* block_table, int bt_stride, float* part_o,
                  float* part_ml, int* counters, int nq, int nkv, int page_size, float scale, int window, int rows,
                  int splits, cudaStream_t s) {
  constexpr int ROW = HD + 8;
  int ps_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (ps_shift = 0; (1 << ps_shift) < page_size; ++ps_shift) {}
  const size_t tiles = (size_t)(4 * kTile + 16) * ROW * sizeof(__nv_bfloat16);
  const size_t merge = (size_t)(4 * 16 * HD + 128) * sizeof(float);
  const size_t smem = tiles > merge ? tiles : merge;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(paged_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(rows, nkv, splits);
  launch_kernel(paged_decode_kernel<HD>, dim3(grid), dim3(kThreads), smem, s, 1, 
      (const __nv_bfloat16*)q, q_row_stride, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_cache,
      (const __nv_bfloat16*)v_cache, q_indptr, kv_lens, block_table, bt_stride, part_o, part_ml, counters, nq, nkv,
      page_size, ps_shift, scale * 1.4426950408889634f, window, splits);
  return launch_status();
}

}  // namespace

// Scratch when splits > 1: part_o float32 [rows * nq * splits * hd], part_ml float32 [rows * nq * splits * 2],
// and counters int32 [rows * nkv] that must be zero before the first launch (the kernel leaves them zero).
ARLE_API int arle_paged_attention_decode(const void* q, int q_row_stride, void* out, const void* k_cache,
                                         const void* v_cache, const int* q_indptr, const int* kv_lens,
                                         const int* block_table, int bt_stride, float* part_o, float* part_ml,
                                         int* counters, int nq, int nkv, int hd, int page_size, float scale, int window,
                                         int rows, int splits, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || nq / nkv > 16 || page_size <= 0) return ARLE_E_UNSUPPORTED;
  if (splits < 1 || splits > 64 || nkv > 65535) return ARLE_E_UNSUPPORTED;
  if (splits > 1 && (!part_o || !part_ml || !counters)) return ARLE_E_BADARG;
  if ((q_row_stride % 8) != 0) return ARLE_E_UNSUPPORTED;     // 16-byte loads of q rows
  if (hd == 128)
    return launch_decode<128>(q, q_row_stride, out, k_cache, v_cache, q_indptr, kv_lens, block_table, bt_stride, part_o,
                              part_ml, counters, nq, nkv, page_size, scale, window, rows, splits, s);
  if (hd == 64)
    return launch_decode<64>(q, q_row_stride, out, k_cache, v_cache, q_indptr, kv_lens, block_table, bt_stride, part_o,
                             part_ml, counters, nq, nkv, page_size, scale, window, rows, splits, s);
  return ARLE_E_UNSUPPORTED;
}
