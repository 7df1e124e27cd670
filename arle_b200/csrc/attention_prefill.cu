// Paged causal attention for prompt portions (several queries per request),
// bfloat16, head sizes 64 and 128: a flash-attention forward pass on the tensor
// cores over the block table.
//
//   grid = (query blocks of 64, query heads, request rows); 4 warps, each owning
//   16 consecutive queries.  Keys and values arrive in tiles of 64 through
//   cp.async into double-buffered padded shared memory, each row located through
//   the block table (any page size); tile boundaries sit at multiples of 64 of the
//   absolute key position.  S = Q.K^T and O += P.V are mma.sync m16n8k16 with
//   float32 accumulators; the mask (key <= query position, and > position - window
//   when a window is set), the online softmax and the rescaling are float32; P is
//   rounded to bfloat16 for P.V, as in cklxx/arle's prefill kernel
//   (crates/cuda-kernels/tools/tilelang/batch_prefill_paged_hd128.py:170-232).
// A query i of a row with q_len queries and kv_len keys after the step stands at
// position kv_len - q_len + i.  Rows with a single query are skipped when
// skip_single is set (the decode kernel takes them).
#include "common.cuh"
#include "mma_utils.cuh"
using namespace arle;

namespace {

constexpr int kThreads = 128;
constexpr int kBlockM = 64;
constexpr int kTile = 64;

template <int HD>
__global__ void __launch_bounds__(kThreads, 3) paged_prefill_kernel(
    const __nv_bfloat16* __restrict__ q, int q_row_stride, __nv_bfloat16* __restrict__ out,
    const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
    const int* __restrict__ q_indptr, const int* __restrict__ kv_lens, const int* __restrict__ block_table,
    int bt_stride, int nq, int nkv, int page_size, int ps_shift, float scale_log2, int window, int skip_single) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int ROW = HD + 8;
  constexpr int CHUNKS = HD / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [2][kTile][ROW]
  __nv_bfloat16* vs = ks + 2 * kTile * ROW;                         // [2][kTile][ROW]
  __nv_bfloat16* qs = ks + kTile * ROW;        // the queries pass through stage 1 of K before its first tile arrives
  __shared__ int pgbuf[4][kTile + 1];          // page ids of four tiles in turn, fetched two tiles ahead of the data

  const int r = blockIdx.z, h = blockIdx.y;
  const int t0 = q_indptr[r];
  const int qlen = q_indptr[r + 1] - t0;
  const int mbeg = blockIdx.x * kBlockM;
  if (mbeg >= qlen || (skip_single && qlen == 1)) return;
  const int kv_len = kv_lens[r];
  const int pos0 = kv_len - qlen;                       // position of the row's first query
  const int rows_here = min(kBlockM, qlen - mbeg);
  const int p_first = pos0 + mbeg, p_last = pos0 + mbeg + rows_here - 1;
  const int lo = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
  const int kb = lo / kTile * kTile;
  const int ntiles = (p_last - kb) / kTile + 1;
  const int kvh = h / (nq / nkv);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;

  const int* bt = block_table + (size_t)r * bt_stride;
  const size_t head_stride = (size_t)page_size * HD;
  const size_t page_stride = (size_t)nkv * head_stride;
  const __nv_bfloat16* kbase = k_cache + (size_t)kvh * head_stride;
  const __nv_bfloat16* vbase = v_cache + (size_t)kvh * head_stride;

  auto fetch_ids = [&](int tile, bool async) {
    const int k0 = max(lo, kb + tile * kTile);
    const int k1 = min(p_last, kb + tile * kTile + kTile - 1);
    if (k0 > k1) return;
    const int first = k0 / page_size, last = k1 / page_size;
    if (tid <= last - first) {
      if (async) cp_async4(smem_u32(&pgbuf[tile & 3][tid]), bt + first + tid, 4);
      else pgbuf[tile & 3][tid] = bt[first + tid];
    }
  };
  auto load_tile = [&](int tile, int stage) {
    const int k0 = kb + tile * kTile;
    const int first = ps_shift >= 0 ? (max(lo, k0) >> ps_shift) : max(lo, k0) / page_size;
    const int* pg = pgbuf[tile & 3];
    __nv_bfloat16* kd = ks + stage * kTile * ROW;
    __nv_bfloat16* vd = vs + stage * kTile * ROW;
#pragma unroll
    for (int i = 0; i < kTile * CHUNKS / kThreads; ++i) {
      const int c = tid + i * kThreads;
      const int key = c / CHUNKS, part = c % CHUNKS;
      const int kj = k0 + key;
      const bool ok = kj >= lo && kj <= p_last;
      size_t off = 0;
      if (ok) {
        const int pidx = ps_shift >= 0 ? (kj >> ps_shift) : kj / page_size;     // pages are mostly a power of two
        off = (size_t)pg[pidx - first] * page_stride + (size_t)(kj - pidx * page_size) * HD + part * 8;
      }
      cp_async16(smem_u32(kd + key * ROW + part * 8), kbase + off, ok ? 16 : 0);
      cp_async16(smem_u32(vd + key * ROW + part * 8), vbase + off, ok ? 16 : 0);
    }
  };
  fetch_ids(0, false);
  fetch_ids(1, false);
  fetch_ids(2, false);
  __syncthreads();
  load_tile(0, 0);
  cp_commit();

  for (int i = tid; i < kBlockM * CHUNKS; i += kThreads) {
    const int row = i / CHUNKS, part = i % CHUNKS;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < rows_here)
      v = *reinterpret_cast<const uint4*>(q + (size_t)(t0 + mbeg + row) * q_row_stride + (size_t)h * HD + part * 8);
    *reinterpret_cast<uint4*>(qs + row * ROW + part * 8) = v;
  }
  __syncthreads();
  uint32_t qa[HD / 16][4];
  {
    const __nv_bfloat16* qw = qs + warp * 16 * ROW;
#pragma unroll
    for (int s = 0; s < HD / 16; ++s) {
      qa[s][0] = *reinterpret_cast<const uint32_t*>(qw + g * ROW + s * 16 + 2 * tq);
      qa[s][1] = *reinterpret_cast<const uint32_t*>(qw + (g + 8) * ROW + s * 16 + 2 * tq);
      qa[s][2] = *reinterpret_cast<const uint32_t*>(qw + g * ROW + s * 16 + 8 + 2 * tq);
      qa[s][3] = *reinterpret_cast<const uint32_t*>(qw + (g + 8) * ROW + s * 16 + 8 + 2 * tq);
    }
  }
  __syncthreads();                             // every warp holds its query fragments: stage 1 may be overwritten
  // positions of this thread's two query rows; rows past the portion's end copy the last one
  const int prow0 = min(pos0 + mbeg + warp * 16 + g, p_last);
  const int prow1 = min(pos0 + mbeg + warp * 16 + g + 8, p_last);
  const int plo0 = window > 0 ? prow0 - window + 1 : 0;
  const int plo1 = window > 0 ? prow1 - window + 1 : 0;
  const int warp_last = min(pos0 + mbeg + warp * 16 + 15, p_last);   // last key any row of this warp may see
  const int warp_first = window > 0 ? max(0, min(pos0 + mbeg + warp * 16, p_last) - window + 1) : 0;

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  for (int tile = 0; tile < ntiles; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < ntiles) {
      load_tile(tile + 1, stage ^ 1);
      if (tile + 3 < ntiles) fetch_ids(tile + 3, true);
      cp_commit();
      cp_wait<1>();
    } else {
      cp_wait<0>();
    }
    __syncthreads();
    const int k0 = kb + tile * kTile;
    if (warp * 16 < rows_here && k0 <= warp_last && k0 + kTile > warp_first) {
      const __nv_bfloat16* kt = ks + stage * kTile * ROW;
      const __nv_bfloat16* vt = vs + stage * kTile * ROW;
      float s[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
        for (int nb = 0; nb < 4; ++nb) {        // 16 keys per ldmatrix.x4
          uint32_t b0, b1, b2, b3;
          ldsm_x4(smem_u32(kt + (nb * 16 + (lane >> 4) * 8 + (lane & 7)) * ROW + kk * 16 + ((lane >> 3) & 1) * 8), b0, b1, b2, b3);
          mma_bf16(s[2 * nb], qa[kk], b0, b1);
          mma_bf16(s[2 * nb + 1], qa[kk], b2, b3);
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const int kj = k0 + 8 * n + 2 * tq;
        s[n][0] = (kj <= prow0 && kj >= plo0) ? s[n][0] * scale_log2 : -INFINITY;
        s[n][1] = (kj + 1 <= prow0 && kj + 1 >= plo0) ? s[n][1] * scale_log2 : -INFINITY;
        s[n][2] = (kj <= prow1 && kj >= plo1) ? s[n][2] * scale_log2 : -INFINITY;
        s[n][3] = (kj + 1 <= prow1 && kj + 1 >= plo1) ? s[n][3] * scale_log2 : -INFINITY;
        mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
        mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      // a row that has seen no key yet keeps m = -inf; use 0 in the exponents so that nothing is NaN
      const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
      const float c0 = exp2f(m0 - mu0), c1 = exp2f(m1 - mu1);
      m0 = mn0;
      m1 = mn1;
      float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        s[n][0] = exp2f(s[n][0] - mu0);
        s[n][1] = exp2f(s[n][1] - mu0);
        s[n][2] = exp2f(s[n][2] - mu1);
        s[n][3] = exp2f(s[n][3] - mu1);
        ps0 += s[n][0] + s[n][1];
        ps1 += s[n][2] + s[n][3];
      }
      l0 = l0 * c0 + ps0;
      l1 = l1 * c1 + ps1;
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1;
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {          // 16 keys per step of P.V
        uint32_t pa[4];
        pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dn = 0; dn < HD / 16; ++dn) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(smem_u32(vt + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * ROW + dn * 16 + (lane >> 4) * 8), b0, b1, b2, b3);
          mma_bf16(o[2 * dn], pa, b0, b1);
          mma_bf16(o[2 * dn + 1], pa, b2, b3);
        }
      }
    }
    __syncthreads();
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;
  const int row0 = mbeg + warp * 16 + g, row1 = row0 + 8;
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) {
    if (row0 < qlen) {
      __nv_bfloat162 v = __floats2bfloat162_rn(o[i][0] * inv0, o[i][1] * inv0);
      *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)(t0 + row0) * nq + h) * HD + i * 8 + 2 * tq) = v;
    }
    if (row1 < qlen) {
      __nv_bfloat162 v = __floats2bfloat162_rn(o[i][2] * inv1, o[i][3] * inv1);
      *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)(t0 + row1) * nq + h) * HD + i * 8 + 2 * tq) = v;
    }
  }
}

template <int HD>
int launch_prefill(const void* q, int q_row_stride, void* out, const void* k_cache, const void* v_cache,
                   const int* q_indptr, const int* kv_lens, const int* block_table, int bt_stride, int nq, int nkv,
                   int page_size, float scale, int window, int rows, int max_q_len, int skip_single, cudaStream_t s) {
  constexpr int ROW = HD + 8;
  int ps_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (ps_shift = 0; (1 << ps_shift) < page_size; ++ps_shift) {}
  const size_t smem = (size_t)(4 * kTile) * ROW * sizeof(__nv_bfloat16);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(paged_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((max_q_len + kBlockM - 1) / kBlockM, nq, rows);
  launch_kernel(paged_prefill_kernel<HD>, dim3(grid), dim3(kThreads), smem, s, 1, 
      (const __nv_bfloat16*)q, q_row_stride, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_cache,
      (const __nv_bfloat16*)v_cache, q_indptr, kv_lens, block_table, bt_stride, nq, nkv, page_size, ps_shift,
      scale * 1.4426950408889634f, window, skip_single);
  return launch_status();
}

}  // namespace

ARLE_API int arle_paged_attention_prefill(const void* q, int q_row_stride, void* out, const void* k_cache,
                                          const void* v_cache, const int* q_indptr, const int* kv_lens,
                                          const int* block_table, int bt_stride, int nq, int nkv, int hd, int page_size,
                                          float scale, int window, int rows, int max_q_len, int skip_single,
                                          cudaStream_t s) {
  if (rows <= 0 || max_q_len <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || nq > 65535 || rows > 65535) return ARLE_E_UNSUPPORTED;
  if ((q_row_stride % 8) != 0) return ARLE_E_UNSUPPORTED;
  if (hd == 128)
    return launch_prefill<128>(q, q_row_stride, out, k_cache, v_cache, q_indptr, kv_lens, block_table, bt_stride, nq,
                               nkv, page_size, scale, window, rows, max_q_len, skip_single, s);
  if (hd == 64)
    return launch_prefill<64>(q, q_row_stride, out, k_cache, v_cache, q_indptr, kv_lens, block_table, bt_stride, nq,
                              nkv, page_size, scale, window, rows, max_q_len, skip_single, s);
  return ARLE_E_UNSUPPORTED;
}
