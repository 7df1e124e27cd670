// Weight-streaming matrix product for decoding: out[M, N] = x[M, K] . W[N, K]^T with
// few rows (M <= 16, one per decoded token), bfloat16 operands, float32 sums.
//
// With so few rows the product is one read of W at HBM speed, and everything here
// serves that read:
//  * one CTA per SM (a persistent grid); the N weight rows are divided evenly among
//    the CTAs to the row, not to a tile, so no SM gets a larger share;
//  * weights travel global -> shared memory by the bulk async-copy engine
//    (cp.async.bulk, one copy per weight-row segment, completion counted in bytes
//    on an mbarrier), so the bytes in flight sit in shared memory rather than in
//    registers: every warp keeps a ring of stages (16 weight rows x 256 or 128
//    elements of K) filled ahead of its arithmetic;
//  * x stays in shared memory for the whole launch;
//  * the tensor cores do the arithmetic with W as the 16-row A operand and x^T as
//    the B operand (mma.sync m16n8k16), float32 accumulators;
//  * a K too long for x to fit in shared memory is split over a thread-block
//    cluster: each CTA of the cluster owns one K range (its slice of x and of every
//    weight row) and rank 0 adds the partial sums through distributed shared
//    memory, in rank order, so the result does not depend on timing;
//  * the warps of a CTA take stages round-robin and their partial sums are added
//    in warp order.
// Every wait on an mbarrier is bounded: after kSpinLimit polls the kernel raises
// the error flag and carries on to its end instead of hanging.
//
// cklxx/arle calls cuBLASLt for these products (crates/cuda-kernels/csrc/gemm/gemv.cu:298-482)
// and keeps a hand-written GEMV for one row (:45-...); this kernel replaces both for M <= 16.
#include <cooperative_groups.h>

#include "common.cuh"
#include "mma_utils.cuh"
using namespace arle;
namespace cg = cooperative_groups;

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kXPad = 8;                     // elements of padding per x row (16 bytes): rows fall on different banks
constexpr int kRowPad = 16;                  // bytes of padding per weight-row segment of a stage
constexpr int kPartTiles = 16;                // tiles whose partial sums a CTA of a cluster keeps for one reduction at the end
constexpr uint32_t kSpinLimit = 1u << 22;    // polls of an mbarrier before giving up (a few hundred ms)

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
// Returns false when the limit ran out (the caller raises the error flag).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// NT: 8-row groups of x (1: M <= 8, 2: M <= 16).  KB: K elements per stage.  SLOTS: stages per warp.
// KS: K elements owned by one CTA (K / cluster size, a multiple of 32).
template <int NT, int KB, int SLOTS, typename OutT>
__global__ void __launch_bounds__(kThreads, 1) skinny_gemm_kernel(
    const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ W, int ldw, OutT* __restrict__ out,
    int ldo, int M, int N, int K, int KS, int csize, int early, int gated, int* __restrict__ err) {
  constexpr int PITCH = KB * 2 + kRowPad;                 // bytes per weight-row segment in a stage
  constexpr int STAGE = 16 * PITCH;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int xrow = KS + kXPad;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                           // [NT*8][xrow]
  size_t off = ((size_t)NT * 8 * xrow * 2 + 127) / 128 * 128;
  unsigned char* stages = smem_raw + off;                                                    // [kWarps][SLOTS][STAGE]
  off += (size_t)kWarps * SLOTS * STAGE;
  float* red = reinterpret_cast<float*>(smem_raw + off);                                     // [2][kWarps][16][NT*8]
  off += (size_t)2 * kWarps * 16 * NT * 8 * sizeof(float);
  float* part = reinterpret_cast<float*>(smem_raw + off);                                    // [kPartTiles][16][NT*8] (clusters)
  off += (size_t)kPartTiles * 16 * NT * 8 * sizeof(float);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + off);                              // [kWarps][SLOTS], then x's
  uint64_t* xbar = bars + kWarps * SLOTS;

  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int rank = csize > 1 ? (int)(blockIdx.x % csize) : 0;
  const int group = blockIdx.x / csize, ngroups = gridDim.x / csize;
  // gated: weight rows come in (gate, up) pairs that stay in one CTA and one tile
  const int unit = gated ? 2 : 1;
  const int r0 = (int)((long long)(N / unit) * group / ngroups) * unit;
  const int r1 = (int)((long long)(N / unit) * (group + 1) / ngroups) * unit;
  const int ks0 = rank * KS;
  const int ks1 = min(K, ks0 + KS);
  const int klen = max(0, ks1 - ks0);
  const int tiles = (r1 - r0 + 15) / 16;
  const int spt = (klen + KB - 1) / KB;                   // stages per 16-row tile
  const int total = tiles * spt;
  const bool batched = csize > 1 && tiles <= kPartTiles;    // few tiles: one cluster reduction at the end

  if (lane == 0) {
    for (int s = 0; s < SLOTS; ++s) mbar_init(smem_u32(&bars[warp * SLOTS + s]), 1);
    if (warp == 0) mbar_init(smem_u32(xbar), 1);
  }
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  __syncwarp();
  // this CTA's slice of x: one bulk copy per row (rows beyond M are zeroed by hand)
  auto fetch_x = [&]() {
    if (warp == 0 && klen > 0) {
      if (lane == 0) mbar_expect_tx(smem_u32(xbar), (uint32_t)(min(M, NT * 8) * klen * 2));
      __syncwarp();
      if (lane < M && lane < NT * 8)
        bulk_copy_g2s(smem_u32(xs + (size_t)lane * xrow), x + (size_t)lane * ldx + ks0, (uint32_t)(klen * 2), smem_u32(xbar));
    }
  };
  // x is the output of the kernel before this one.  Launched early (programmatic launch),
  // the kernel fills its weight ring first (no kernel writes weights), then waits for that
  // kernel, then fetches x; launched in stream order, x goes first because it is needed first.
  if (!early) {
    pdl_wait();
    fetch_x();
  }

  // stage number s of this CTA = (tile s / spt, K block s % spt); warp w owns s = w, w + kWarps, ...
  auto issue = [&](int s, int slot) {
    const int tile = s / spt, kb = s - tile * spt;
    const int k0 = ks0 + kb * KB;
    const int len = min(KB, ks1 - k0);
    const int rt = r0 + tile * 16;
    const int nvalid = min(16, r1 - rt);
    const uint32_t bar = smem_u32(&bars[warp * SLOTS + slot]);
    if (lane == 0) mbar_expect_tx(bar, (uint32_t)(nvalid * len * 2));
    __syncwarp();
    if (lane < nvalid)
      bulk_copy_g2s(smem_u32(stages + (size_t)(warp * SLOTS + slot) * STAGE + lane * PITCH),
                    W + (size_t)(rt + lane) * ldw + k0, (uint32_t)(len * 2), bar);
  };
  int issued = 0;                                           // stages of this warp issued so far
  for (; issued < SLOTS; ++issued) {
    const int s = warp + issued * kWarps;
    if (s < total) issue(s, issued);
  }

  if (early) {
    pdl_wait();
    fetch_x();
  }
  bool timed_out = false;
  {
    const int per_row = klen / 8;
    for (int i = tid; i < (NT * 8 - M) * per_row; i += kThreads) {
      const int m = M + i / per_row, c = i % per_row;
      *reinterpret_cast<uint4*>(xs + (size_t)m * xrow + c * 8) = make_uint4(0, 0, 0, 0);
    }
  }
  __syncthreads();                                          // zero rows written, x barrier initialised for all
  if (klen > 0 && !mbar_wait_bounded(smem_u32(xbar), 0)) timed_out = true;

  int done = 0;                                             // stages of this warp consumed so far
  for (int tile = 0; tile < tiles; ++tile) {
    // two accumulator sets, used by alternate K steps, halve the chain of dependent MMAs
    float acc[NT][4], acc2[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
      acc2[n][0] = acc2[n][1] = acc2[n][2] = acc2[n][3] = 0.f;
    }
    for (;;) {
      const int s = warp + done * kWarps;
      if (s >= total || s / spt != tile) break;
      const int slot = done % SLOTS;
      const uint32_t bar = smem_u32(&bars[warp * SLOTS + slot]);
      if (!mbar_wait_bounded(bar, (uint32_t)((done / SLOTS) & 1))) timed_out = true;
      const int kb = s - tile * spt;
      const int kloc = kb * KB;                             // offset inside this CTA's K range
      const int len = min(KB, klen - kloc);
      const uint32_t st = smem_u32(stages + (size_t)(warp * SLOTS + slot) * STAGE);
      const uint32_t a_addr = st + (lane & 15) * PITCH + (lane >> 4) * 16;
      const __nv_bfloat16* xb = xs + (size_t)g * xrow + kloc + 2 * tq;
#pragma unroll 2
      for (int kk = 0; kk < len; kk += 32) {          // len is a multiple of 32
        uint32_t a[4], a2[4];
        ldsm_x4(a_addr + kk * 2, a[0], a[1], a[2], a[3]);
        ldsm_x4(a_addr + kk * 2 + 32, a2[0], a2[1], a2[2], a2[3]);
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          const uint32_t b0 = *reinterpret_cast<const uint32_t*>(xb + (size_t)n * 8 * xrow + kk);
          const uint32_t b1 = *reinterpret_cast<const uint32_t*>(xb + (size_t)n * 8 * xrow + kk + 8);
          const uint32_t b2 = *reinterpret_cast<const uint32_t*>(xb + (size_t)n * 8 * xrow + kk + 16);
          const uint32_t b3 = *reinterpret_cast<const uint32_t*>(xb + (size_t)n * 8 * xrow + kk + 24);
          mma_bf16(acc[n], a, b0, b1);
          mma_bf16(acc2[n], a2, b2, b3);
        }
      }
      __syncwarp();
      ++done;
      const int nxt = warp + issued * kWarps;               // refill the slot just drained
      if (nxt < total) {
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        issue(nxt, slot);
      }
      ++issued;
    }
    // c0,c1: (weight row g, x rows 2t, 2t+1); c2,c3: (weight row g+8, same x rows)
    float* rw = red + ((size_t)(tile & 1) * kWarps + warp) * 16 * NT * 8;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      rw[g * NT * 8 + n * 8 + 2 * tq] = acc[n][0] + acc2[n][0];
      rw[g * NT * 8 + n * 8 + 2 * tq + 1] = acc[n][1] + acc2[n][1];
      rw[(g + 8) * NT * 8 + n * 8 + 2 * tq] = acc[n][2] + acc2[n][2];
      rw[(g + 8) * NT * 8 + n * 8 + 2 * tq + 1] = acc[n][3] + acc2[n][3];
    }
    __syncthreads();
    const int rt = r0 + tile * 16;
    if (tid < 16 * NT * 8) {
      const int row = tid & 15, m = tid >> 4;
      const float* rb = red + (size_t)(tile & 1) * kWarps * 16 * NT * 8 + row * NT * 8 + m;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) s += rb[(size_t)w * 16 * NT * 8];
      if (gated) {
        // rows 2i and 2i+1 of W are gate_i and up_i: out[m, i] = silu(gate) * up, in float32
        const float up = __shfl_down_sync(0xffffffffu, s, 1);
        if (!(row & 1) && m < M && rt + row < r1)
          store_out<OutT>(out + (size_t)m * ldo + ((rt + row) >> 1), s / (1.0f + expf(-s)) * up);
      } else if (csize == 1) {
        if (m < M && rt + row < r1) store_out<OutT>(out + (size_t)m * ldo + rt + row, s);
      } else {
        part[(batched ? tile : (tile & 1)) * 16 * NT * 8 + tid] = s;
      }
    }
    if (csize > 1 && !batched) {
      // too many tiles to keep: rank 0 adds the ranks' sums tile by tile
      cg::cluster_group cluster = cg::this_cluster();
      cluster.sync();
      if (rank == 0 && tid < 16 * NT * 8) {
        const int row = tid & 15, m = tid >> 4;
        float s = 0.f;
        for (int rk = 0; rk < csize; ++rk) {
          const float* remote = cluster.map_shared_rank(part, rk);
          s += remote[(tile & 1) * 16 * NT * 8 + tid];
        }
        if (m < M && rt + row < r1) store_out<OutT>(out + (size_t)m * ldo + rt + row, s);
      }
    }
  }
  if (csize > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (batched && rank == 0 && tid < 16 * NT * 8) {
      // one reduction for all tiles: rank 0 adds the ranks' sums, in rank order
      const int row = tid & 15, m = tid >> 4;
      for (int tile = 0; tile < tiles; ++tile) {
        float s = 0.f;
        for (int rk = 0; rk < csize; ++rk) {
          const float* remote = cluster.map_shared_rank(part, rk);
          s += remote[tile * 16 * NT * 8 + tid];
        }
        const int rt = r0 + tile * 16;
        if (m < M && rt + row < r1) store_out<OutT>(out + (size_t)m * ldo + rt + row, s);
      }
    }
    if (batched) cluster.sync();                            // no CTA leaves while its partial sums may still be read
  }
  if (timed_out && err) atomicExch(err, 1);
}

template <int NT, int KB, int SLOTS>
size_t smem_bytes(int KS) {
  size_t n = ((size_t)NT * 8 * (KS + kXPad) * 2 + 127) / 128 * 128;
  n += (size_t)kWarps * SLOTS * 16 * (KB * 2 + kRowPad);
  n += (size_t)2 * kWarps * 16 * NT * 8 * sizeof(float);
  n += (size_t)kPartTiles * 16 * NT * 8 * sizeof(float);
  n += (size_t)(kWarps * SLOTS + 1) * sizeof(uint64_t);
  return n;
}

template <int NT, int KB, int SLOTS, typename OutT>
int plan_and_launch(const void* x, int ldx, const void* W, int ldw, void* out, int ldo, int M, int N, int K, int gated,
                    int* err, cudaStream_t s) {
  int dev = 0, sms = 0, max_smem = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  // the smallest cluster whose CTAs can each hold their slice of x
  int csize = 1;
  int KS = K;
  while (smem_bytes<NT, KB, SLOTS>(KS) > (size_t)max_smem) {
    ++csize;
    if (csize > 8) return ARLE_E_UNSUPPORTED;
    KS = ((K + csize - 1) / csize + 31) / 32 * 32;
  }
  if (gated && csize > 1) return ARLE_E_UNSUPPORTED;       // the gate needs whole sums in one CTA
  auto kern = skinny_gemm_kernel<NT, KB, SLOTS, OutT>;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<NT, KB, SLOTS>(KS));
  if (e != cudaSuccess) return (int)e;
  // A persistent grid must be resident at once: as many clusters as the GPU can hold together.
  // Clusters do not span GPCs, so one size may leave more SMs idle than the next: of the
  // smallest size that fits and the one above it, take the one that fills more SMs.
  int groups = sms;
  if (csize > 1) {
    static int resident[10] = {};                       // clusters of each size that run together (this instantiation)
    int best = csize, best_sms = 0;
    for (int c = csize; c <= csize + 1 && c <= 8; ++c) {
      if (resident[c] == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(sms / c * c);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = smem_bytes<NT, KB, SLOTS>(((K + c - 1) / c + 31) / 32 * 32);
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = c;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int max_clusters = 0;
        e = cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg);
        if (e != cudaSuccess) return (int)e;
        resident[c] = max_clusters > 0 ? max_clusters : 1;
      }
      const int filled = (resident[c] < sms / c ? resident[c] : sms / c) * c;
      if (filled > best_sms + 2) best = c, best_sms = filled;   // a larger cluster must win by more than 2 SMs
    }
    csize = best;
    KS = ((K + csize - 1) / csize + 31) / 32 * 32;
    groups = resident[csize] < sms / csize ? resident[csize] : sms / csize;
  }
  const size_t smem = smem_bytes<NT, KB, SLOTS>(KS);
  const int tiles = (N + 15) / 16;
  if (groups > tiles) groups = tiles;
  if (groups < 1) groups = 1;
  const bool early = (pdl_enabled() & 3) != 0;
  e = launch_kernel_as(early, kern, dim3(groups * csize), dim3(kThreads), smem, s, csize, (const __nv_bfloat16*)x, ldx,
                       (const __nv_bfloat16*)W, ldw, (OutT*)out, ldo, M, N, K, KS, csize, early ? 1 : 0, gated, err);
  if (e != cudaSuccess) return (int)e;
  return launch_status();
}

int skinny_entry(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M, int N, int K,
                 int gated, int* err, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K <= 0 || K % 32 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return ARLE_E_UNSUPPORTED;
  if (((uintptr_t)x & 15) || ((uintptr_t)W & 15)) return ARLE_E_UNSUPPORTED;
  if (gated && N % 2 != 0) return ARLE_E_BADARG;
  if (M <= 8) {
    if (out_dtype == 0) return plan_and_launch<1, 256, 2, float>(x, ldx, W, ldw, out, ldo, M, N, K, gated, err, s);
    if (out_dtype == 1) return plan_and_launch<1, 256, 2, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, M, N, K, gated, err, s);
  } else {
    if (out_dtype == 0) return plan_and_launch<2, 256, 2, float>(x, ldx, W, ldw, out, ldo, M, N, K, gated, err, s);
    if (out_dtype == 1) return plan_and_launch<2, 256, 2, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, M, N, K, gated, err, s);
  }
  return ARLE_E_BADARG;
}

}  // namespace

// out_dtype: 0 float32, 1 bfloat16.  Needs M <= 16, K a multiple of 32, ldx and ldw multiples of 8,
// 16-byte aligned x and W.  err (may be null): set to 1 if a bounded wait ran out.
ARLE_API int arle_gemm_skinny(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M, int N,
                              int K, int* err, cudaStream_t s) {
  return skinny_entry(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, 0, err, s);
}

// The gated feed-forward's first half in one launch: W [N, K] holds (gate_i, up_i) in rows 2i and
// 2i + 1, and out[M, N / 2] = silu(x . gate_i) * (x . up_i), the gate computed on the float32 sums.
// Same needs as arle_gemm_skinny, and a K short enough for x to stay in one CTA's shared memory.
ARLE_API int arle_gemm_skinny_gated(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M,
                                    int N, int K, int* err, cudaStream_t s) {
  return skinny_entry(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, 1, err, s);
}
