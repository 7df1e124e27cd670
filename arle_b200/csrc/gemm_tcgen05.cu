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
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
using namespace arle;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;                       // 64 bfloat16 = 128 bytes = one swizzle span
constexpr int kEpilogueWarps = 4;
constexpr int kThreads = 192;
constexpr uint32_t kSpinLimit = 1u << 24;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, const volatile int* abort_flag) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023) == 1023 && *abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ bool mbar_wait_plain(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major, 128-byte swizzled tile whose rows are
// 128 bytes apart: start address, stride between 8-row groups 1024 bytes, descriptor
// version 1 (sm_100), layout 2 (SWIZZLE_128B).  The leading-dimension offset is not
// used by this layout.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// Instruction descriptor, kind::f16: D float32, A and B bfloat16, both K-major, N and M.
__host__ __device__ constexpr uint32_t idesc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

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
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  int rows, k, ld, box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && k == o.k && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    h ^= std::hash<long long>()(((long long)k.rows << 32) ^ k.k) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
    h ^= std::hash<long long>()(((long long)k.ld << 32) ^ k.box_rows) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
    return h;
  }
};

// Tensor map of a row-major [rows, k] bfloat16 matrix (row stride ld elements): boxes of
// box_rows x 64 elements, 128-byte swizzle, zero fill out of bounds.  Cached per matrix.
int tensor_map_for(const void* ptr, int rows, int k, int ld, int box_rows, CUtensorMap* out) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const MapKey key{ptr, rows, k, ld, box_rows};
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return 0;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return ARLE_E_UNSUPPORTED;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return ARLE_E_BADARG;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return 0;
}

template <int BN, int STAGES, typename OutT>
int launch(const void* x, int ldx, const void* W, int ldw, void* out, int ldo, int M, int N, int K, int* err,
           cudaStream_t s) {
  CUtensorMap mx, mw;
  int rc = tensor_map_for(x, M, K, ldx, BM, &mx);
  if (rc) return rc;
  rc = tensor_map_for(W, N, K, ldw, BN, &mw);
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
