// bfloat16 matrix product on the fifth-generation tensor cores, two SMs to a tile:
//     out[M, N] = x[M, K] . W[N, K]^T      (float32 accumulation, bfloat16 or float32 out)
// or, gated, out[M, N / 2] = silu(x . W[2i]) * (x . W[2i + 1]) for a weight whose rows 2i and 2i + 1 are
// gate_i and up_i (the first half of a gated feed-forward without the round trip of the product through
// memory and without the kernel that applies the gate).
//
// Why two SMs: a 128 x 256 tile fed from one SM's shared memory needs 48 KB per 64 elements of K, and at
// the tensor cores' pace that is more than an SM can take in from L2 (the one-SM kernel, gemm_tcgen05.cu,
// stops at 0.85 of cuBLAS for that reason).  Here a pair of CTAs (a cluster of two) owns a 256 x 256 tile:
// each CTA loads its 128 rows of x and its 128 of the tile's 256 weight rows (32 KB per 64 elements of K for
// the same arithmetic per SM), and one tcgen05.mma with cta_group::2, issued by the pair's first CTA, reads
// both CTAs' shared memory and writes both CTAs' tensor memory: rows 0-127 of the tile accumulate in the
// first CTA's TMEM, rows 128-255 in the second's.
//
// Per CTA, by warp:
//   warp 4, one lane : producer.  Waits for a free stage (its own `empty` barrier) and issues two TMA loads
//                      into its own shared memory whose bytes are counted on the FIRST CTA's `full` barrier
//                      of the stage (cp.async.bulk.tensor with cta_group::2 and that barrier's cluster
//                      address); the first CTA's producer arms that barrier with the bytes of both CTAs.
//   warp 5, one lane : in the first CTA only, the MMA issuer: waits for a full stage, issues four
//                      tcgen05.mma (256 x 256 x 16 over the pair), and hands the stage back to both
//                      producers with one tcgen05.commit that arrives on the `empty` barrier of both CTAs
//                      (multicast over the cluster); after a tile's last block a commit on both CTAs'
//                      `acc_full`.  Warp 5 of both CTAs allocates and frees the TMEM columns (cta_group::2).
//   warps 0-3        : epilogue of the CTA's own 128 rows: tcgen05.ld 32 columns at a time, convert (or apply
//                      the gate to neighbouring columns), store; then arrive on the first CTA's `acc_empty`.
// The accumulators are double-buffered (2 x 256 of the 512 TMEM columns): the tensor cores fill one while the
// epilogue drains the other.  Edges: TMA zero-fills rows beyond M or N and columns beyond K; stores are
// guarded.  Every wait is bounded; a CTA whose wait runs out raises the error flag, stops issuing and runs to
// its end (its partner's waits then run out in turn), and both meet at the cluster barrier before they free
// their tensor memory.  No TMA load here is a multicast; the only cluster-wide operation besides the MMA is
// the commit.
//
// cklxx/arle calls cuBLASLt for these products (crates/cuda-kernels/csrc/gemm/gemv.cu:298-482).
#include "common.cuh"
#include "tcgen05_utils.cuh"
using namespace arle;

namespace {

constexpr int BM = 128;                      // rows of x per CTA (256 per pair)
constexpr int BNH = 128;                     // weight rows per CTA (256 per pair)
constexpr int BN = 256;
constexpr int BK = 64;                       // 64 bfloat16 = 128 bytes = one swizzle span
constexpr int kEpilogueWarps = 4;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// The cluster address of the same shared-memory location in the CTA of the given rank.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
      ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives, when the MMAs issued so far are done, on the barrier at this address in both CTAs of the pair.
__device__ __forceinline__ void umma_commit_both(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}

template <int STAGES, bool GATED, typename OutT>
__global__ void __launch_bounds__(kThreads, 1) gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                        const __grid_constant__ CUtensorMap map_w,
                                                                        OutT* __restrict__ out, int ldo, int M, int N,
                                                                        int K, int* __restrict__ err) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BNH * BK * 2, STAGE = A_BYTES + B_BYTES;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES];      // first CTA's: both CTAs' copies of the stage have landed
  __shared__ __align__(8) uint64_t empty_bar[STAGES];     // each CTA's: the MMAs have read the stage
  __shared__ __align__(8) uint64_t acc_full[2];           // each CTA's: accumulator buffer complete
  __shared__ __align__(8) uint64_t acc_empty[2];          // first CTA's: both CTAs' epilogues have drained the buffer
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair = (int)(blockIdx.x >> 1), npairs = (int)(gridDim.x >> 1);
  const int tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int kblocks = (K + BK - 1) / BK;
  // Order of the tiles: bands of kBand rows of tiles; inside a band the row index runs fastest, then the
  // column.  The pairs that run together then share a few weight tiles and at most kBand tiles' rows of x, which
  // stay in L2 however many rows x has (with the row index fastest over all of x, a long x is swept from HBM
  // once per couple of weight tiles).
  constexpr int kBand = 8;
  auto tile_at = [&](int t, int& tm, int& tn) {
    const int band = t / (kBand * tiles_n);
    const int rows_here = min(kBand, tiles_m - band * kBand);
    const int in_band = t - band * kBand * tiles_n;
    tm = band * kBand + in_band % rows_here;
    tn = in_band / rows_here;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_addr(&full_bar[s]), 1);
      mbar_init(smem_addr(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_addr(&acc_full[b]), 1);
      mbar_init(smem_addr(&acc_empty[b]), 2 * kEpilogueWarps);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 5) {
    tmem_alloc_pair(smem_addr(&tmem_base_slot), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                      // the partner's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const volatile int* aborted = &abort_flag;

  if (warp == 4) {
    if (lane == 0) {
      int issued = 0;
      for (int t = pair; t < num_tiles && !*aborted; t += npairs) {
        int tm, tn;
        tile_at(t, tm, tn);
        const int m0 = tm * 2 * BM + (int)rank * BM;
        const int n0 = tn * BN + (int)rank * BNH;
        for (int kb = 0; kb < kblocks; ++kb, ++issued) {
          const int s = issued % STAGES;
          if (!mbar_wait_bounded(smem_addr(&empty_bar[s]), ((issued / STAGES) & 1) ^ 1, aborted)) {
            abort_flag = 1;
            break;
          }
          const uint32_t bar_local = smem_addr(&full_bar[s]);
          if (leader) mbar_expect_tx(bar_local, 2 * STAGE);                 // the bytes of both CTAs
          const uint32_t bar = map_to_rank(bar_local, 0);
          tma_load_2d_pair(smem_addr(tiles + (size_t)s * STAGE), &map_x, kb * BK, m0, bar);
          tma_load_2d_pair(smem_addr(tiles + (size_t)s * STAGE + A_BYTES), &map_w, kb * BK, n0, bar);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = idesc_bf16(2 * BM, BN);
      int consumed = 0, iter = 0;
      for (int t = pair; t < num_tiles && !*aborted; t += npairs, ++iter) {
        const int buf = iter & 1;
        if (!mbar_wait_bounded(smem_addr(&acc_empty[buf]), ((iter >> 1) & 1) ^ 1, aborted)) {
          abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < kblocks; ++kb, ++consumed) {
          const int s = consumed % STAGES;
          if (!mbar_wait_bounded(smem_addr(&full_bar[s]), (consumed / STAGES) & 1, aborted)) {
            abort_flag = 1;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_addr(tiles + (size_t)s * STAGE);
          const uint64_t adesc = smem_desc_sw128(a_addr), bdesc = smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_bf16_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit_both(smem_addr(&empty_bar[s]));
        }
        umma_commit_both(smem_addr(&acc_full[buf]));
      }
    }
  } else {
    // epilogue of this CTA's 128 rows: warp i reads TMEM lanes 32 i .. 32 i + 31
    int iter = 0;
    const uint32_t acc_empty_leader[2] = {map_to_rank(smem_addr(&acc_empty[0]), 0), map_to_rank(smem_addr(&acc_empty[1]), 0)};
    for (int t = pair; t < num_tiles; t += npairs, ++iter) {
      const int buf = iter & 1;
      int tm, tn;
      tile_at(t, tm, tn);
      const int m0 = tm * 2 * BM + (int)rank * BM, n0 = tn * BN;
      const bool ready = mbar_wait_bounded(smem_addr(&acc_full[buf]), (iter >> 1) & 1, aborted);
      if (!ready) abort_flag = 1;
      if (__any_sync(0xffffffffu, !ready || *aborted)) break;
      tc_fence_after();
      const int row = m0 + warp * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(buf * BN + c * 32), r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (row >= M || col >= N) continue;
        if (GATED) {
          // columns 2i and 2i + 1 are gate_i and up_i: sixteen outputs per thread and step
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * ldo + (col >> 1);
          float v[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float g = __uint_as_float(r[2 * i]), u = __uint_as_float(r[2 * i + 1]);
            v[i] = g / (1.0f + __expf(-g)) * u;
          }
          if (col + 32 <= N && (((uintptr_t)dst) & 15) == 0) {
            uint32_t p[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
              p[i] = *reinterpret_cast<uint32_t*>(&b);
            }
            reinterpret_cast<uint4*>(dst)[0] = make_uint4(p[0], p[1], p[2], p[3]);
            reinterpret_cast<uint4*>(dst)[1] = make_uint4(p[4], p[5], p[6], p[7]);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (col + 2 * i + 1 < N) dst[i] = __float2bfloat16_rn(v[i]);
          }
        } else {
          OutT* dst = out + (size_t)row * ldo + col;
          if (sizeof(OutT) == 2) {
            if (col + 32 <= N && (((uintptr_t)dst) & 15) == 0) {
              uint32_t p[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                p[i] = *reinterpret_cast<uint32_t*>(&v);
              }
#pragma unroll
              for (int i = 0; i < 4; ++i)
                reinterpret_cast<uint4*>(dst)[i] = make_uint4(p[4 * i], p[4 * i + 1], p[4 * i + 2], p[4 * i + 3]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col + i < N) reinterpret_cast<__nv_bfloat16*>(dst)[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
            }
          } else {
            if (col + 32 <= N && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                reinterpret_cast<uint4*>(dst)[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col + i < N) reinterpret_cast<float*>(dst)[i] = __uint_as_float(r[i]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader[buf]);
    }
  }
  // A producer whose wait ran out may still have copies under way into its shared memory: wait for them
  // (bounded) before the CTA ends.  They are counted on the first CTA's barriers, so only it can look.
  if (warp == 4 && lane == 0 && leader && *aborted)
    for (int s = 0; s < STAGES; ++s) mbar_wait_plain(smem_addr(&full_bar[s]), 0), mbar_wait_plain(smem_addr(&full_bar[s]), 1);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                      // neither CTA frees tensor memory the other's MMAs may still write
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && abort_flag && err) atomicExch(err, 3);
}

template <int STAGES, bool GATED, typename OutT>
int launch(const void* x, int ldx, const void* W, int ldw, void* out, int ldo, int M, int N, int K, int* err, cudaStream_t s) {
  CUtensorMap mx, mw;
  int rc = tensor_map_2d_bf16(x, M, K, ldx, BM, &mx);
  if (rc) return rc;
  rc = tensor_map_2d_bf16(W, N, K, ldw, BNH, &mw);
  if (rc) return rc;
  const size_t smem = (size_t)STAGES * (BM * BK * 2 + BNH * BK * 2) + 1024;
  auto kern = gemm_tcgen05_pair_kernel<STAGES, GATED, OutT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long num_tiles = (long long)((N + BN - 1) / BN) * ((M + 2 * BM - 1) / (2 * BM));
  long long pairs = sms / 2;
  if (num_tiles < pairs) pairs = num_tiles;
  cudaError_t e = launch_kernel(kern, dim3((unsigned)(2 * pairs)), dim3(kThreads), smem, s, 2, mx, mw, (OutT*)out, ldo, M, N, K, err);
  if (e != cudaSuccess) return (int)e;
  return launch_status();
}

}  // namespace

// out_dtype: 0 float32, 1 bfloat16.  gated != 0: W holds (gate_i, up_i) in rows 2i and 2i + 1 and out is bfloat16
// [M, N / 2] (N even).  Needs K, ldx, ldw multiples of 8 and 16-byte aligned x and W.  err: set to 3 if a bounded
// wait ran out.
ARLE_API int arle_gemm_tcgen05_pair(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M,
                                    int N, int K, int gated, int* err, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return ARLE_E_UNSUPPORTED;
  if (((uintptr_t)x & 15) || ((uintptr_t)W & 15)) return ARLE_E_UNSUPPORTED;
  if (gated) {
    if (N % 2 != 0 || out_dtype != 1) return ARLE_E_BADARG;
    return launch<6, true, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, M, N, K, err, s);
  }
  if (out_dtype == 1) return launch<6, false, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, M, N, K, err, s);
  if (out_dtype == 0) return launch<6, false, float>(x, ldx, W, ldw, out, ldo, M, N, K, err, s);
  return ARLE_E_BADARG;
}
