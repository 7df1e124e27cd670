// bfloat16 matrix product on the fifth-generation tensor cores of sm_100a:
//     out[M, N] = x[M, K] . W[N, K]^T      (float32 accumulation, bfloat16 or float32 out)
// for the many-row case (prompt portions, large decode batches).
//
// A persistent grid (one CTA per SM) walks the 128 x BN output tiles (BN = 256 or 128),
// M index fastest, so that CTAs running together share weight tiles through L2.  The
// accumulator lives in tensor memory (TMEM) and is double-buffered: while the epilogue
// warps drain one tile, the tensor cores already fill the next.  Roles by warp:
//   warp 4, one lane : producer.  For every 64-wide block of K it waits for a free
//                      stage, arms the stage's mbarrier with the byte count and issues
//                      two TMA tile loads (cp.async.bulk.tensor.2d): 128 rows of x and
//                      BN rows of W, 128-byte swizzled, into the stage.
//   warp 5, one lane : MMA issuer.  Waits for a full stage and issues four
//                      tcgen05.mma (M 128, N BN, K 16 each) whose operands are shared
//                      memory descriptors of the stage and whose accumulator is a
//                      128-lane x BN-column block of tensor memory (TMEM);
//                      tcgen05.commit hands the stage back to the producer when the
//                      MMAs have read it, and signals the epilogue after a tile's last block.
//                      Warp 5 also allocates and frees the TMEM columns (2 x BN).
//   warps 0-3        : epilogue.  Warp i owns TMEM lanes 32i..32i+31 = tile rows;
//                      tcgen05.ld brings 32 columns at a time into registers, which are
//                      converted and stored, each thread writing a contiguous piece of
//                      its row.
// Edges: TMA zero-fills rows beyond M or N and columns beyond K; stores are guarded.
// Every mbarrier wait is bounded; when one runs out the kernel raises the error flag,
// stops issuing, waits (bounded) for the copies it has in flight, frees its TMEM and
// returns.
//
// cklxx/arle calls cuBLASLt here (crates/cuda-kernels/csrc/gemm/gemv.cu:298-482).
#include "common.cuh"
#include "tcgen05_utils.cuh"
using namespace arle;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;                       // 64 bfloat16 = 128 bytes = one swizzle span
constexpr int kEpilogueWarps = 4;
constexpr int kThreads = 192;

template <int BN, int STAGES, typename OutT>
__global__ void __launch_bounds__(kThreads, 1) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                   const __grid_constant__ CUtensorMap map_w,
                                                                   OutT* __restrict__ out, int ldo, int M, int N, int K,
                                                                   int* __restrict__ err) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  constexpr uint32_t kTmemCols = 2 * BN <= 256 ? 256 : 512;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES];      // producer -> MMA: stage holds its two tiles
  __shared__ __align__(8) uint64_t empty_bar[STAGES];     // MMA -> producer: stage has been read
  __shared__ __align__(8) uint64_t acc_full[2];           // MMA -> epilogue: accumulator buffer complete
  __shared__ __align__(8) uint64_t acc_empty[2];          // epilogue -> MMA: accumulator buffer drained
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int kblocks = (K + BK - 1) / BK;
  // Tiles are numbered with the M index fastest, and CTA c takes tiles c, c + grid, ...:
  // the CTAs running at the same time share a few weight tiles, which then come from L2.

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_addr(&full_bar[s]), 1);
      mbar_init(smem_addr(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_addr(&acc_full[b]), 1);
      mbar_init(smem_addr(&acc_empty[b]), kEpilogueWarps);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 5) {
    tmem_alloc(smem_addr(&tmem_base_slot), kTmemCols);     // two accumulator buffers (a power of two of columns)
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const volatile int* aborted = &abort_flag;

  if (warp == 4) {
    if (lane == 0) {
      int issued = 0;                                       // k blocks issued over all tiles
      for (int t = blockIdx.x; t < num_tiles && !*aborted; t += gridDim.x) {
        const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++issued) {
          const int s = issued % STAGES;
          if (!mbar_wait_bounded(smem_addr(&empty_bar[s]), ((issued / STAGES) & 1) ^ 1, aborted)) {
            abort_flag = 1;
            break;
          }
          const uint32_t bar = smem_addr(&full_bar[s]);
          mbar_expect_tx(bar, A_BYTES + B_BYTES);
          tma_load_2d(smem_addr(tiles + (size_t)s * (A_BYTES + B_BYTES)), &map_x, kb * BK, m0, bar);
          tma_load_2d(smem_addr(tiles + (size_t)s * (A_BYTES + B_BYTES) + A_BYTES), &map_w, kb * BK, n0, bar);
        }
      }
      if (*aborted) {
        // wait (bounded) for the copies still under way before the CTA gives its shared memory back
        for (int i = max(0, issued - STAGES); i < issued; ++i)
          mbar_wait_plain(smem_addr(&full_bar[i % STAGES]), (i / STAGES) & 1);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_bf16(BM, BN);
      int consumed = 0, iter = 0;
      for (int t = blockIdx.x; t < num_tiles && !*aborted; t += gridDim.x, ++iter) {
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
          const uint32_t a_addr = smem_addr(tiles + (size_t)s * (A_BYTES + B_BYTES));
          const uint64_t adesc = smem_desc_sw128(a_addr), bdesc = smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)      // 16 elements of K = 32 bytes = 2 descriptor address units
            umma_bf16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(smem_addr(&empty_bar[s]));
        }
        umma_commit(smem_addr(&acc_full[buf]));  // arrives when all MMAs issued so far are done
      }
    }
  } else {
    // epilogue: warp i reads TMEM lanes 32 i .. 32 i + 31 of the finished accumulator buffer
    int iter = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++iter) {
      const int buf = iter & 1;
      const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * BN;
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
        if (row < M && col < N) {
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
      if (lane == 0) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(&acc_empty[buf])) : "memory");
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && abort_flag && err) atomicExch(err, 2);
}

// ------------------------------------------------------------------ host side
template <int BN, int STAGES, typename OutT>
int launch(const void* x, int ldx, const void* W, int ldw, void* out, int ldo, int M, int N, int K, int* err,
           cudaStream_t s) {
  CUtensorMap mx, mw;
  int rc = tensor_map_2d_bf16(x, M, K, ldx, BM, &mx);
  if (rc) return rc;
  rc = tensor_map_2d_bf16(W, N, K, ldw, BN, &mw);
  if (rc) return rc;
  const size_t smem = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + 1024;
  auto kern = gemm_tcgen05_kernel<BN, STAGES, OutT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long num_tiles = (long long)((N + BN - 1) / BN) * ((M + BM - 1) / BM);
  const int grid = (int)(num_tiles < sms ? num_tiles : sms);      // persistent: one CTA per SM
  launch_kernel(kern, dim3(grid), dim3(kThreads), smem, s, 1, mx, mw, (OutT*)out, ldo, M, N, K, err);
  return launch_status();
}

}  // namespace

// out_dtype: 0 float32, 1 bfloat16.  Needs K, ldx, ldw multiples of 8 and 16-byte aligned x and W.
ARLE_API int arle_gemm_tcgen05(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M,
                               int N, int K, int* err, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return ARLE_E_UNSUPPORTED;
  if (((uintptr_t)x & 15) || ((uintptr_t)W & 15)) return ARLE_E_UNSUPPORTED;
  if (M > 65535 * BM) return ARLE_E_UNSUPPORTED;
  // Tile width 256, or 128 for narrow outputs.  (Narrower tiles that fill the last wave of
  // CTAs better were tried and lost more in per-tile efficiency than they gained.)
  const int best = N >= 256 ? 256 : 128;
#define ARLE_TC_CASE(BN_, ST_)                                                                                        \
  if (best == BN_)                                                                                                    \
    return out_dtype == 1 ? launch<BN_, ST_, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, M, N, K, err, s)                \
                          : launch<BN_, ST_, float>(x, ldx, W, ldw, out, ldo, M, N, K, err, s);
  if (out_dtype != 0 && out_dtype != 1) return ARLE_E_BADARG;
  ARLE_TC_CASE(256, 4)
  ARLE_TC_CASE(128, 6)
#undef ARLE_TC_CASE
  return ARLE_E_BADARG;
}
