// Paged causal attention for prompt portions on the fifth-generation tensor cores
// (tcgen05), head size 128, bfloat16, page sizes that are multiples of 16.
//
// One CTA serves 128 consecutive queries of one request and one query head and walks
// the visible keys in tiles of 128 (boundaries at multiples of 128 of the absolute key
// position).  Everything big lives where the tensor cores want it:
//   shared memory : Q (128 x 128) and three stages each of K and V (128 keys x 128), in the
//                   128-byte swizzled layout that TMA writes and tcgen05.mma reads;
//   tensor memory : two buffers for the scores S (128 lanes x 128 columns, float32), the
//                   output accumulator O (128 x 128, float32) and two buffers for P
//                   (128 lanes x 64 columns, two bfloat16 per column): all 512 columns.
// Roles by warp:
//   warps 4 and 6    : loaders (keys; values).  TMA tile loads (cp.async.bulk.tensor.2d): Q
//                      once from the packed projection output, then per tile the keys or the
//                      values page by page (16 keys x 64 elements per box, one box per lane)
//                      at the rows the block table names.
//   warp 5, one lane : MMA issuer.  S(j) = Q . K(j)^T (eight tcgen05.mma of K 16, both operands
//                      K-major) into S buffer j mod 2, one tile ahead of the softmax;
//                      O += P(j) . V(j) (eight tcgen05.mma with P as the A operand read from
//                      tensor memory, and V used as it lies in the cache: an MN-major B
//                      operand).  tcgen05.commit signals the mbarriers.
//   warps 0-3        : softmax and epilogue; thread i owns query row i (TMEM lane i), so row
//                      maxima and sums need no shuffles.  A thread reads its row of S into
//                      registers, masks (key <= query position, and > position - window)
//                      and finds the row maximum; O and the running sum are rescaled only
//                      when the maximum grew by more than 2^8 since the last rescale (the
//                      exponentials stay within float32 and bfloat16 range); then it
//                      exponentiates, adds up and writes P as bfloat16 into tensor memory
//                      (tcgen05.st, two buffers), as cklxx/arle's prefill kernel rounds P
//                      (crates/cuda-kernels/tools/tilelang/batch_prefill_paged_hd128.py:223-225).
//                      After the last tile the rows are divided by their sums and stored.
// Scores, maxima, sums and the accumulator are float32.  Every mbarrier wait is bounded;
// when one runs out the kernel raises the error flag, stops, frees its TMEM and returns.
#include "common.cuh"
#include "tcgen05_utils.cuh"
using namespace arle;

namespace {

constexpr int HD = 128;
constexpr int BQ = 128;                      // queries per CTA
constexpr int BKV = 128;                     // keys per tile
constexpr int kThreads = 224;
constexpr uint32_t SUB = 128 * 128;          // bytes of a [128 rows x 64 elements] swizzled sub-tile
constexpr uint32_t TILE = 2 * SUB;           // 128 x 128 bfloat16
constexpr int kStages = 3;                   // stages of keys and of values
constexpr float kRescaleStep = 8.0f;         // log2 units the maximum may grow before O is rescaled

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
// tcgen05.mma with the A operand in tensor memory: lane = row of A, each 32-bit column holds two
// consecutive bfloat16 elements of K (16 elements of K = 8 columns).
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
               ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ float ex2_fast(float x) {          // 2^x on the special-function unit; -inf gives 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}

// Descriptor of an MN-major, 128-byte swizzled operand: rows of 64 contiguous elements
// along N (128 bytes), one row per K index; groups of 8 rows 1024 bytes apart (stride
// offset), the next 64 elements of N `lbo` bytes further (leading offset).
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t addr, uint32_t lbo) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

__global__ void __launch_bounds__(kThreads, 1) paged_prefill_tc_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, const int* __restrict__ q_indptr,
    const int* __restrict__ kv_lens, const int* __restrict__ block_table, int bt_stride, int bt_width, int nq, int nkv,
    int page_size, float scale_log2, int window, int skip_single, int* __restrict__ err) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.z, h = blockIdx.y;
  const int t0 = q_indptr[r];
  const int qlen = q_indptr[r + 1] - t0;
  // the blocks with the most keys (the last queries) are scheduled first
  const int mbeg = (int)(gridDim.x - 1 - blockIdx.x) * BQ;
  if (mbeg >= qlen || (skip_single && qlen == 1)) return;
  const int kv_len = kv_lens[r];
  const int pos0 = kv_len - qlen;
  const int rows_here = min(BQ, qlen - mbeg);
  const int p_first = pos0 + mbeg, p_last = pos0 + mbeg + rows_here - 1;
  const int lo = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
  const int kb = lo / BKV * BKV;
  const int ntiles = (p_last - kb) / BKV + 1;
  const int kvh = h / (nq / nkv);

  extern __shared__ unsigned char smem_dyn[];
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = base;                      // TILE
  unsigned char* k_s = base + TILE;                       // kStages x TILE
  unsigned char* v_s = base + (1 + kStages) * TILE;       // kStages x TILE
  __shared__ __align__(8) uint64_t q_full, k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages], s_full[2], s_empty[2], p_full[2],
      pv_done[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(smem_addr(&q_full), 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(smem_addr(&k_full[i]), 1);
      mbar_init(smem_addr(&k_empty[i]), 1);
      mbar_init(smem_addr(&v_full[i]), 1);
      mbar_init(smem_addr(&v_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_addr(&s_full[i]), 1);
      mbar_init(smem_addr(&s_empty[i]), 4);
    }
    mbar_init(smem_addr(&p_full[0]), 4);
    mbar_init(smem_addr(&p_full[1]), 4);
    mbar_init(smem_addr(&pv_done[0]), 1);
    mbar_init(smem_addr(&pv_done[1]), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  // Value rows that no load ever fills (beyond the last key) meet P = 0; they must hold
  // numbers, not whatever bits shared memory had.
  for (uint32_t i = threadIdx.x; i < kStages * TILE / 16; i += kThreads) reinterpret_cast<uint4*>(v_s)[i] = make_uint4(0, 0, 0, 0);
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  if (warp == 5) {
    tmem_alloc(smem_addr(&tmem_base_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const uint32_t tmem_o = tmem_base + 256;
  const uint32_t tmem_p = tmem_base + 384;                    // two buffers of 64 columns: P as packed bfloat16 pairs
  const volatile int* aborted = &abort_flag;

  if (warp == 4 || warp == 6) {
    // Warp 4 loads the keys, warp 6 the values, each at its own pace: a tile is 16 boxes per
    // operand (8 pages x 2 halves of the head), one per lane, so that their issue overlaps;
    // lane 0 waits for the stage and arms its barrier.  A key stage frees as soon as S of two
    // tiles ago is computed, a value stage only after P.V of two tiles ago.
    const bool keys = warp == 4;
    if (keys && lane == 0) {
      mbar_expect_tx(smem_addr(&q_full), TILE);
      tma_load_2d(smem_addr(q_s), &map_q, h * HD, t0 + mbeg, smem_addr(&q_full));
      tma_load_2d(smem_addr(q_s + SUB), &map_q, h * HD + 64, t0 + mbeg, smem_addr(&q_full));
    }
    const int* bt = block_table + (size_t)r * bt_stride;
    const int c = (lane >> 1) & 7, half = lane & 1;      // page of the tile, half of the head (lanes 0..15)
    const CUtensorMap* map = keys ? &map_k : &map_v;
    unsigned char* tile_s = keys ? k_s : v_s;
    // Page ids come 32 at a time, one per lane, with the next 32 already in flight, so that no
    // tile waits for a read of the block table; a lane picks its page with a shuffle.
    int p0 = kb / page_size;
    int cur = __ldg(bt + min(p0 + lane, bt_width - 1));
    int nxt = __ldg(bt + min(p0 + 32 + lane, bt_width - 1));
    for (int j = 0; j < ntiles; ++j) {
      const int st = j % kStages;
      const uint32_t par = (uint32_t)((j / kStages) & 1);
      const int key0 = kb + j * BKV + c * 16;
      while ((kb + j * BKV) / page_size - p0 >= 32) {
        cur = nxt;
        p0 += 32;
        nxt = __ldg(bt + min(p0 + 32 + lane, bt_width - 1));
      }
      const int pi = key0 / page_size;
      const int rel = pi - p0;                                // 0 .. 63: a tile spans at most 8 pages
      const int from_cur = __shfl_sync(0xffffffffu, cur, rel & 31), from_nxt = __shfl_sync(0xffffffffu, nxt, rel & 31);
      int row = -1;
      if (lane < 16 && key0 <= p_last && key0 + 15 >= lo) {
        const int page = rel < 32 ? from_cur : from_nxt;
        row = (page * nkv + kvh) * page_size + (key0 - pi * page_size);
      }
      const int n = __popc(__ballot_sync(0xffffffffu, row >= 0)) >> 1;      // pages of this tile
      uint64_t* full = keys ? &k_full[st] : &v_full[st];
      int go = 1;
      if (lane == 0) {
        if (!mbar_wait_bounded(smem_addr(keys ? &k_empty[st] : &v_empty[st]), par ^ 1, aborted)) {
          abort_flag = 1;
          go = 0;
        } else {
          mbar_expect_tx(smem_addr(full), (uint32_t)n * 4096u);
        }
      }
      go = __shfl_sync(0xffffffffu, go, 0);
      if (!go || *aborted) break;
      if (row >= 0) tma_load_2d(smem_addr(tile_s + st * TILE + half * SUB + c * 2048), map, half * 64, row, smem_addr(full));
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_bf16(BQ, BKV);                  // A and B K-major
      constexpr uint32_t idesc_pv = idesc_bf16(BQ, HD) | (1u << 16);    // B (values) MN-major
      bool ok = mbar_wait_bounded(smem_addr(&q_full), 0, aborted);
      auto issue_s = [&](int j) {
        const int st = j & 1, kst = j % kStages;
        const uint32_t par = (uint32_t)((j >> 1) & 1);
        if (!mbar_wait_bounded(smem_addr(&k_full[kst]), (uint32_t)((j / kStages) & 1), aborted)) return false;
        if (!mbar_wait_bounded(smem_addr(&s_empty[st]), par ^ 1, aborted)) return false;
        tc_fence_after();
#pragma unroll
        for (int dh = 0; dh < 2; ++dh) {
          const uint64_t ad = smem_desc_sw128(smem_addr(q_s + dh * SUB));
          const uint64_t bd = smem_desc_sw128(smem_addr(k_s + kst * TILE + dh * SUB));
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_bf16(tmem_base + (uint32_t)(st * BKV), ad + 2 * k, bd + 2 * k, idesc_s, (dh | k) != 0 ? 1u : 0u);
        }
        umma_commit(smem_addr(&k_empty[kst]));
        umma_commit(smem_addr(&s_full[st]));
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < ntiles && ok; ++j) {
        if (j + 1 < ntiles) ok = issue_s(j + 1);
        if (!ok) break;
        const int st = j & 1, vst = j % kStages;
        if (!mbar_wait_bounded(smem_addr(&p_full[st]), (uint32_t)((j >> 1) & 1), aborted)) { ok = false; break; }
        if (!mbar_wait_bounded(smem_addr(&v_full[vst]), (uint32_t)((j / kStages) & 1), aborted)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t bd = smem_desc_mn_sw128(smem_addr(v_s + vst * TILE + kk * 2048), SUB);
          umma_bf16_a_tmem(tmem_o, tmem_p + (uint32_t)(st * 64 + kk * 8), bd, idesc_pv, (j | kk) != 0 ? 1u : 0u);
        }
        umma_commit(smem_addr(&v_empty[vst]));
        umma_commit(smem_addr(&pv_done[st]));
      }
      if (!ok) abort_flag = 1;
    }
  } else {
    const int row = warp * 32 + lane;                         // query row of the tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    const int p_row = min(p_first + row, p_last);
    const int lo_row = window > 0 ? p_row - window + 1 : 0;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < ntiles; ++j) {
      const int buf = j & 1;
      const int k0 = kb + j * BKV;
      const bool full_tile = k0 + BKV - 1 <= p_first && (window <= 0 || k0 >= p_last - window + 1);
      bool ready = mbar_wait_bounded(smem_addr(&s_full[buf]), (uint32_t)((j >> 1) & 1), aborted);
      if (__any_sync(0xffffffffu, !ready)) { ok = false; break; }
      tc_fence_after();
      // The whole row of scores comes into registers at once (four loads in flight, one
      // wait), which frees the S buffer for the tile after next right away.
      uint32_t sv[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(tmem_base + lane_addr + (uint32_t)(buf * BKV + c * 32), sv[c]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&s_empty[buf]));
      // the row maximum (raw scores; the scale is positive, so it is applied to the maximum
      // alone).  Four running maxima keep the chain of dependent instructions short: a
      // softmax warp has its scheduler to itself.
      float mx;
      {
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (full_tile) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(sv[c][i]));
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int kj = k0 + c * 32 + i;
              if (!(kj <= p_row && kj >= lo_row)) sv[c][i] = 0xff800000u;      // -inf: masked for good
              m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(sv[c][i]));
            }
        }
        mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * scale_log2;
      }
      const float m_new = fmaxf(m_used, mx);
      const bool grow = m_new > m_used + kRescaleStep;        // also true when the row sees its first key
      const float f = (grow && m_used != -INFINITY) ? exp2f(m_used - m_new) : 1.0f;
      if (grow) m_used = m_new;
      const float m_eff = m_used == -INFINITY ? 0.f : m_used;
      l *= f;
      // O may be touched, and P buffer j mod 2 overwritten, only after the products that
      // still use them: P.V of tile j-2 read this P buffer; a rescale of O needs P.V of
      // tile j-1 complete (which implies tile j-2).  Tile t signals pv_done[t mod 2]; its
      // completions there are numbered t / 2, so a waiter is never two phases behind.
      const bool rescale = j > 0 && __any_sync(0xffffffffu, f != 1.0f);
      if (rescale) {
        ready = mbar_wait_bounded(smem_addr(&pv_done[(j - 1) & 1]), (uint32_t)(((j - 1) >> 1) & 1), aborted);
        if (__any_sync(0xffffffffu, !ready)) { ok = false; break; }
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld32(tmem_o + lane_addr + (uint32_t)(c * 32), v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
          tmem_st32(tmem_o + lane_addr + (uint32_t)(c * 32), v);
        }
        tmem_st_wait();
      } else if (j > 1) {
        ready = mbar_wait_bounded(smem_addr(&pv_done[j & 1]), (uint32_t)(((j - 2) >> 1) & 1), aborted);
        if (__any_sync(0xffffffffu, !ready)) { ok = false; break; }
      }
      // exponentials (one fused multiply-add and one ex2 each; a masked score is -inf and
      // gives 0), their sum in four partial sums, and P as bfloat16 in the swizzled
      // K-major layout
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        uint32_t packed[32];                                  // 64 keys of this row as bfloat16 pairs
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float e0 = ex2_fast(fmaf(__uint_as_float(sv[2 * h2 + c][i]), scale_log2, -m_eff));
            const float e1 = ex2_fast(fmaf(__uint_as_float(sv[2 * h2 + c][i + 1]), scale_log2, -m_eff));
            l4[(i >> 1) & 3] += e0 + e1;
            packed[c * 16 + (i >> 1)] = pack_bf16x2(e0, e1);
          }
        tmem_st32(tmem_p + lane_addr + (uint32_t)(buf * 64 + h2 * 32), packed);
      }
      tmem_st_wait();
      l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&p_full[buf]));
    }
    if (ok) {
      const bool ready = mbar_wait_bounded(smem_addr(&pv_done[(ntiles - 1) & 1]), (uint32_t)(((ntiles - 1) >> 1) & 1), aborted);
      if (__any_sync(0xffffffffu, !ready)) ok = false;
    }
    if (ok) {
      tc_fence_after();
      const float inv = 1.0f / l;
      __nv_bfloat16* orow = out + ((size_t)(t0 + mbeg + row) * nq + h) * HD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_o + lane_addr + (uint32_t)(c * 32), v);
        tmem_ld_wait();
        if (row < rows_here) {
          uint32_t p[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(v[2 * i]) * inv, __uint_as_float(v[2 * i + 1]) * inv);
            p[i] = *reinterpret_cast<uint32_t*>(&b);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i)
            reinterpret_cast<uint4*>(orow + c * 32)[i] = make_uint4(p[4 * i], p[4 * i + 1], p[4 * i + 2], p[4 * i + 3]);
        }
      }
    } else if (lane == 0) {
      abort_flag = 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && abort_flag && err) atomicExch(err, 3);
}

}  // namespace

// q: the packed projection output [T, q_row_stride] whose first nq * 128 columns are the queries.
// k_cache / v_cache: [pages, nkv, page_size, 128].  Needs page_size % 16 == 0, head size 128,
// q_row_stride % 8 == 0, 16-byte aligned q, and out rows of nq * 128 elements.
ARLE_API int arle_paged_attention_prefill_tc(const void* q, int q_row_stride, int num_tokens, void* out, const void* k_cache,
                                             const void* v_cache, long long cache_pages, const int* q_indptr,
                                             const int* kv_lens, const int* block_table, int bt_stride, int bt_width, int nq, int nkv,
                                             int hd, int page_size, float scale, int window, int rows, int max_q_len,
                                             int skip_single, int* err, cudaStream_t s) {
  if (rows <= 0 || max_q_len <= 0) return 0;
  if (bt_width < 1) return ARLE_E_BADARG;
  if (hd != HD || page_size % 16 != 0 || nq <= 0 || nkv <= 0 || nq % nkv != 0 || nq > 65535 || rows > 65535)
    return ARLE_E_UNSUPPORTED;
  if (q_row_stride % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
    return ARLE_E_UNSUPPORTED;
  CUtensorMap mq, mk, mv;
  int rc = tensor_map_2d_bf16(q, num_tokens, nq * HD, q_row_stride, BQ, &mq);
  if (rc) return rc;
  const long long cache_rows = cache_pages * nkv * page_size;
  rc = tensor_map_2d_bf16(k_cache, cache_rows, HD, HD, 16, &mk);
  if (rc) return rc;
  rc = tensor_map_2d_bf16(v_cache, cache_rows, HD, HD, 16, &mv);
  if (rc) return rc;
  const size_t smem = (1 + 2 * kStages) * (size_t)TILE + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(paged_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((max_q_len + BQ - 1) / BQ, nq, rows);
  cudaError_t e = launch_kernel(paged_prefill_tc_kernel, grid, dim3(kThreads), smem, s, 1, mq, mk, mv, (__nv_bfloat16*)out,
                                q_indptr, kv_lens, block_table, bt_stride, bt_width, nq, nkv, page_size,
                                scale * 1.4426950408889634f, window, skip_single, err);
  if (e != cudaSuccess) return (int)e;
  return launch_status();
}
