// Weight-streaming matrix product for decoding: out[M, N] = x[M, K] . W[N, K]^T with
// few rows (M <= 16, one per decoded token), bfloat16 operands, float32 sums.
//
// With so few rows the product is one read of W at HBM speed, and everything here
// serves that read:
//  * one CTA per SM (a persistent grid); the N weight rows are divided evenly among
//    the CTAs to the row, not to a tile, so no SM gets a larger share;
//  * weights travel global -> shared memory by the bulk async-copy engine
//    (cp.async.bulk, completion counted in bytes on an mbarrier), so the bytes in
//    flight sit in shared memory rather than in registers.  Four producer warps keep
//    a ring of stages filled ahead of the arithmetic; a stage is 16 weight rows x
//    1,024 elements of K, one copy of 2 KB per row: issuing a copy costs a warp some
//    150 cycles whatever its size, so rows of 512 bytes could not keep up with HBM
//    (1.75 TB/s measured with 512-byte copies, 3.2 with 1 KB, 6.0 with 2 KB);
//  * eight consumer warps share a stage, its blocks of 32 elements of K going round
//    them;
//  * x stays in shared memory for the whole launch;
//  * the tensor cores do the arithmetic with W as the 16-row A operand and x^T as
//    the B operand (mma.sync m16n8k16), float32 accumulators;
//  * a K too long for x to fit in shared memory is split over a thread-block
//    cluster: each CTA of the cluster owns one K range (its slice of x and of every
//    weight row) and rank 0 adds the partial sums through distributed shared
//    memory, in rank order, so the result does not depend on timing;
//  * the consumer warps' partial sums are added in warp order.
// Two optional fusions take the RMSNorm kernels out of a decode step (a norm between two
// of these products is then no launch at all):
//  * "sink": instead of storing its sums, the product adds them to the float32 residual,
//    r = resid + sum, and stores resid = r and xs = bfloat16(r * gamma), the next norm's
//    input without its per-row factor; every CTA also leaves the sum of r^2 over its
//    columns in a slot of its own of a small table (no atomics, so the order of the
//    additions is fixed);
//  * "row scale": the product reads such a table, forms 1 / sqrt(sum r^2 / width + eps)
//    per row of x, and multiplies its sums by it, which is the same as having normalised
//    x before (the factor is one number per row, the product is linear in x).
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

constexpr int kConsumerWarps = 8;
constexpr int kProducerWarps = 4;
constexpr int kRowsPerProducer = 16 / kProducerWarps;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + kProducerWarps * 32;
constexpr int kXPad = 8;                     // elements of padding per x row (16 bytes): rows fall on different banks
constexpr int kRowPad = 16;                  // bytes of padding per weight-row segment of a stage
constexpr int kPartTiles = 16;                // tiles whose partial sums a CTA of a cluster keeps between two reductions
constexpr uint32_t kSpinLimit = 1u << 22;    // polls of an mbarrier before giving up (a few hundred ms)
constexpr int kSsSlots = 192;                // slots of a sum-of-squares table (one per CTA or cluster of the product that fills it)
constexpr int kSsRows = 16;                  // rows of x a slot covers

// The optional fusions (see the top of the file).  All pointers null: a plain product.
struct Fusion {
  const float* in_ss;          // [kSsRows][kSsSlots]: sums of squares of the rows of x, a row's slots to be added up (a row is
                               // contiguous: every CTA reads the whole table, and reads scattered over it queue up at a few
                               // L2 sectors, 10 us for a 200 MB product); null: x is used as it is
  float inv_width, eps;        // factor of row m: rsqrt(sum_m * inv_width + eps)
  float* resid;                // [M, ldr] float32, read and written; null: the sums go to out
  int ldr;
  const float* gamma;          // [N]
  __nv_bfloat16* xs;           // [M, ldxs]
  int ldxs;
  float* out_ss;               // [kSsRows][kSsSlots]: this launch fills every slot (zeros beyond its own CTAs)
};

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
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(kConsumers) : "memory"); }
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// NT: 8-row groups of x (1: M <= 8, 2: M <= 16).  KS: K elements owned by one CTA (K / cluster
// size, a multiple of 32).  KC: K elements per stage (a multiple of 32).  S: stages.
template <int NT, typename OutT>
__global__ void __launch_bounds__(kThreads, 1) skinny_gemm_kernel(
    const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ W, int ldw, OutT* __restrict__ out,
    int ldo, int M, int N, int K, int KS, int KC, int S, int csize, int early, int gated, Fusion fu, int* __restrict__ err) {
  const int pitch = KC * 2 + kRowPad;                     // bytes per weight row of a stage
  const int stage_bytes = 16 * pitch;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int xrow = KS + kXPad;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                           // [NT*8][xrow]
  size_t off = ((size_t)NT * 8 * xrow * 2 + 127) / 128 * 128;
  unsigned char* stages = smem_raw + off;                                                    // [S][16][pitch]
  off += (size_t)S * stage_bytes;
  float* red = reinterpret_cast<float*>(smem_raw + off);                                     // [2][warps][16][NT*8]
  off += (size_t)2 * kConsumerWarps * 16 * NT * 8 * sizeof(float);
  float* part = reinterpret_cast<float*>(smem_raw + off);                                    // [kPartTiles][16][NT*8] (clusters)
  off += csize > 1 ? (size_t)kPartTiles * 16 * NT * 8 * sizeof(float) : 0;      // only clusters keep partial sums
  float* ss_in = reinterpret_cast<float*>(smem_raw + off);                                   // [NT*8][kSsSlots]: the table's rows, staged
  off += (size_t)NT * 8 * kSsSlots * sizeof(float);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + off);                              // [S], then empty [S], then x's
  uint64_t* empty = full + S;
  uint64_t* xbar = empty + S;
  __shared__ float row_scale[NT * 8];

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
  const int spt = (klen + KC - 1) / KC;                   // stages per 16-row tile
  const int total = tiles * spt;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&full[s]), kProducerWarps);      // each producer warp arrives once, with its bytes
      mbar_init(smem_u32(&empty[s]), kConsumerWarps);
    }
    mbar_init(smem_u32(xbar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  __syncthreads();
  bool timed_out = false;

  if (warp >= kConsumerWarps) {
    // ------------------------------------------------------------------ producers
    // Warp p brings its four rows of every stage, one bulk copy per row (KC elements, 2 KB,
    // contiguous in memory), as far ahead as the ring is deep.  (Issuing a copy costs a warp
    // some 150 cycles whatever its size: hence long copies, issued from several warps.)
    const int pw = warp - kConsumerWarps;
    const int row = pw * kRowsPerProducer + lane;           // lanes 0 .. kRowsPerProducer - 1
    // this CTA's slice of x: one bulk copy per row (rows beyond M are zeroed by the consumers)
    auto fetch_x = [&]() {
      if (pw == 0 && (klen > 0 || fu.in_ss)) {
        // with x comes the table of sums of squares, one copy of all the rows this kernel reads.  Both are
        // asked for before any weight: a small load issued behind a ring-full of weight copies waits for all
        // their bytes to come in first (some 3 us).
        const uint32_t ss_bytes = fu.in_ss ? (uint32_t)(NT * 8 * kSsSlots * sizeof(float)) : 0u;
        if (lane == 0) {
          mbar_expect_tx(smem_u32(xbar), (uint32_t)(min(M, NT * 8) * klen * 2) + ss_bytes);   // klen may be 0
          if (ss_bytes) bulk_copy_g2s(smem_u32(ss_in), fu.in_ss, ss_bytes, smem_u32(xbar));
        }
        __syncwarp();
        if (lane < M && lane < NT * 8 && klen > 0)
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
    int slot = 0;
    uint32_t par = 0;
    for (int s = 0; s < total; ++s) {
      if (early && s == min(S, total)) {
        pdl_wait();
        fetch_x();
      }
      const int tile = s / spt, c = s - tile * spt;
      const int k0 = ks0 + c * KC;
      const int len = min(KC, ks1 - k0);
      const int rt = r0 + tile * 16;
      const int nvalid = min(16, r1 - rt);
      const int mine = max(0, min(kRowsPerProducer, nvalid - pw * kRowsPerProducer));     // rows of this warp
      if (lane == 0) {
        if (!timed_out && !mbar_wait_bounded(smem_u32(&empty[slot]), par ^ 1)) timed_out = true;   // gives up once, not at every stage
        mbar_expect_tx(smem_u32(&full[slot]), (uint32_t)(mine * len * 2));
      }
      __syncwarp();
      if (lane < mine)
        bulk_copy_g2s(smem_u32(stages + (size_t)slot * stage_bytes + (size_t)row * pitch), W + (size_t)(rt + row) * ldw + k0,
                      (uint32_t)(len * 2), smem_u32(&full[slot]));
      if (++slot == S) slot = 0, par ^= 1;
      // The cluster's barriers are for all its threads.  The consumers meet twice after every kPartTiles
      // tiles (and after the last): the producers meet them there, after the copies of those tiles are
      // issued, and go on with the next tiles afterwards.  (Meeting them only at the very end would leave
      // the consumers waiting at the first barrier for producers that wait for free stages.)
      if (csize > 1 && c == spt - 1 && ((tile + 1) % kPartTiles == 0 || tile + 1 == tiles)) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        cluster.sync();
      }
    }
    if (early && total <= S) {                              // fewer stages than the ring holds: x not fetched in the loop
      pdl_wait();
      fetch_x();
    }
    timed_out = __any_sync(0xffffffffu, timed_out);
    if (csize > 1 && spt == 0) {                            // a rank without a K range still meets the others
      cg::cluster_group cluster = cg::this_cluster();
      for (int ch = 0; ch < (tiles + kPartTiles - 1) / kPartTiles; ++ch) {
        cluster.sync();
        cluster.sync();
      }
    }
    if (timed_out && lane == 0 && err) atomicExch(err, 1);
    return;
  }

  // -------------------------------------------------------------------- consumers
  // Row factors, from the staged table: warp m adds up row m's slots, each lane its share in ascending
  // order, then across the lanes; the order is fixed.
  if ((klen > 0 || fu.in_ss) && !mbar_wait_bounded(smem_u32(xbar), 0)) timed_out = true;
  if (fu.in_ss) {
    for (int m = warp; m < NT * 8; m += kConsumerWarps) {
      float t = 0.f;
      for (int sl = lane; sl < kSsSlots; sl += 32) t += ss_in[m * kSsSlots + sl];
      t = warp_sum(t);
      if (lane == 0) row_scale[m] = rsqrtf(t * fu.inv_width + fu.eps);
    }
  } else if (tid < NT * 8) {
    row_scale[tid] = 1.0f;
  }
  {
    const int per_row = klen / 8;
    for (int i = tid; i < (NT * 8 - M) * per_row; i += kConsumers) {
      const int m = M + i / per_row, c = i % per_row;
      *reinterpret_cast<uint4*>(xs + (size_t)m * xrow + c * 8) = make_uint4(0, 0, 0, 0);
    }
  }
  consumer_sync();                                          // zero rows written

  // What becomes of a finished sum (thread tid < 16 * NT * 8 owns weight row tid & 15 of a tile and row
  // tid >> 4 of x): stored, or (sink) added to the residual, which is stored together with its gamma-
  // scaled copy; then the squares of the 16 threads that share a row of x are added up and returned to
  // the one of them with the lowest lane.
  // The residual element and the gain are fetched ahead (``fetch_sink``) so that no load stands between a
  // tile's last MMA and the next tile.
  auto fetch_sink = [&](int m, int n, bool valid, float& r, float& gn) {
    r = gn = 0.f;
    if (fu.resid && valid) {
      r = __ldcg(fu.resid + (size_t)m * fu.ldr + n);
      gn = __ldg(fu.gamma + n);
    }
  };
  auto finish = [&](float v, int m, int n, bool valid, float r_old, float gn) -> float {
    if (!fu.resid) {
      if (valid) store_out<OutT>(out + (size_t)m * ldo + n, v);
      return 0.f;
    }
    float r = 0.f;
    if (valid) {
      r = r_old + v;
      fu.resid[(size_t)m * fu.ldr + n] = r;
      fu.xs[(size_t)m * fu.ldxs + n] = __float2bfloat16_rn(r * gn);
    }
    float q = r * r;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    return q;
  };
  float ss_acc = 0.f;
  int slot = 0;
  uint32_t par = 0;
  // Clusters: the finished sums of a chunk of kPartTiles tiles are added up across the ranks by all the
  // ranks, tile i of the chunk by rank i % csize.  kMine: the most tiles of a chunk one rank finishes.
  constexpr int kMine = kPartTiles / 2;
  float pre_r[kMine], pre_g[kMine];                         // residual elements and gains of this rank's tiles of a chunk
  for (int tile = 0; tile < tiles; ++tile) {
    float sink_r = 0.f, sink_g = 0.f;
    if (csize == 1 && tid < 16 * NT * 8)
      fetch_sink(tid >> 4, r0 + tile * 16 + (tid & 15), (tid >> 4) < M && r0 + tile * 16 + (tid & 15) < r1, sink_r, sink_g);
    if (csize > 1 && tile % kPartTiles == 0 && tid < 16 * NT * 8 && fu.resid) {
      // asked for at the start of the chunk, used at its end
#pragma unroll
      for (int j = 0; j < kMine; ++j) {
        const int t = tile + rank + j * csize;
        const int n = r0 + t * 16 + (tid & 15);
        fetch_sink(tid >> 4, n, rank + j * csize < kPartTiles && t < tiles && (tid >> 4) < M && n < r1, pre_r[j], pre_g[j]);
      }
    }
    // two accumulator sets, used by alternate K steps, halve the chain of dependent MMAs
    float acc[NT][4], acc2[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
      acc2[n][0] = acc2[n][1] = acc2[n][2] = acc2[n][3] = 0.f;
    }
    for (int c = 0; c < spt; ++c) {
      if (!timed_out && !mbar_wait_bounded(smem_u32(&full[slot]), par)) timed_out = true;
      const int kloc = c * KC;                              // offset inside this CTA's K range
      const int len = min(KC, klen - kloc);
      const uint32_t st = smem_u32(stages + (size_t)slot * stage_bytes);
      const uint32_t a_addr = st + (lane & 15) * pitch + (lane >> 4) * 16;
      const __nv_bfloat16* xb = xs + (size_t)g * xrow + kloc + 2 * tq;
      // the stage's blocks of 32 elements of K go round the warps
#pragma unroll 2
      for (int kk = warp * 32; kk < len; kk += kConsumerWarps * 32) {
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
      if (lane == 0) mbar_arrive(smem_u32(&empty[slot]));
      if (++slot == S) slot = 0, par ^= 1;
    }
    // c0,c1: (weight row g, x rows 2t, 2t+1); c2,c3: (weight row g+8, same x rows)
    float* rw = red + ((size_t)(tile & 1) * kConsumerWarps + warp) * 16 * NT * 8;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      rw[g * NT * 8 + n * 8 + 2 * tq] = acc[n][0] + acc2[n][0];
      rw[g * NT * 8 + n * 8 + 2 * tq + 1] = acc[n][1] + acc2[n][1];
      rw[(g + 8) * NT * 8 + n * 8 + 2 * tq] = acc[n][2] + acc2[n][2];
      rw[(g + 8) * NT * 8 + n * 8 + 2 * tq + 1] = acc[n][3] + acc2[n][3];
    }
    consumer_sync();
    const int rt = r0 + tile * 16;
    if (tid < 16 * NT * 8) {
      const int row = tid & 15, m = tid >> 4;
      const float* rb = red + (size_t)(tile & 1) * kConsumerWarps * 16 * NT * 8 + row * NT * 8 + m;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) s += rb[(size_t)w * 16 * NT * 8];
      if (gated) {
        // rows 2i and 2i+1 of W are gate_i and up_i: out[m, i] = silu(gate) * up, in float32
        s *= row_scale[m];
        const float up = __shfl_down_sync(0xffffffffu, s, 1);
        if (!(row & 1) && m < M && rt + row < r1)
          store_out<OutT>(out + (size_t)m * ldo + ((rt + row) >> 1), s / (1.0f + expf(-s)) * up);
      } else if (csize == 1) {
        ss_acc += finish(s * row_scale[m], m, rt + row, m < M && rt + row < r1, sink_r, sink_g);
      } else {
        part[(tile % kPartTiles) * 16 * NT * 8 + tid] = s;
      }
    }
    if (csize > 1 && ((tile + 1) % kPartTiles == 0 || tile + 1 == tiles)) {
      // one reduction for the last kPartTiles tiles (or fewer): rank 0 adds the ranks' sums, in rank order
      cg::cluster_group cluster = cg::this_cluster();
      const int t_first = tile / kPartTiles * kPartTiles;
      cluster.sync();
      if (tid < 16 * NT * 8) {
        // All of a rank's loads from the other ranks' shared memory go out before its first store (a store
        // in between would hold the next load back: they may alias for all the compiler knows), the ranks
        // in ascending order for every sum, so the result does not depend on timing.
        const int row = tid & 15, m = tid >> 4;
        float sum[kMine];
#pragma unroll
        for (int j = 0; j < kMine; ++j) sum[j] = 0.f;
        for (int rk = 0; rk < csize; ++rk) {
          const float* remote = cluster.map_shared_rank(part, rk);
#pragma unroll
          for (int j = 0; j < kMine; ++j) {
            const int i = rank + j * csize;                 // tile of the chunk
            if (i < kPartTiles && t_first + i <= tile) sum[j] += remote[i * 16 * NT * 8 + tid];
          }
        }
#pragma unroll
        for (int j = 0; j < kMine; ++j) {
          const int i = rank + j * csize;
          if (i < kPartTiles && t_first + i <= tile) {
            const int rt2 = r0 + (t_first + i) * 16;
            ss_acc += finish(sum[j] * row_scale[m], m, rt2 + row, m < M && rt2 + row < r1, fu.resid ? pre_r[j] : 0.f,
                             fu.resid ? pre_g[j] : 0.f);
          }
        }
      }
      cluster.sync();                                       // no CTA overwrites or leaves while its sums may still be read
    }
  }
  if (fu.out_ss) {
    // this CTA's slot; the first CTA also zeroes the slots no CTA owns
    const int mine = blockIdx.x, used = gridDim.x;
    if (tid < 16 * NT * 8 && (tid & 15) == 0) fu.out_ss[(tid >> 4) * kSsSlots + mine] = (tid >> 4) < M ? ss_acc : 0.f;
    if (NT == 1 && tid < 8) fu.out_ss[(8 + tid) * kSsSlots + mine] = 0.f;
    if (mine == 0)
      for (int i = tid; i < kSsRows * (kSsSlots - used); i += kConsumers)
        fu.out_ss[(i / (kSsSlots - used)) * kSsSlots + used + i % (kSsSlots - used)] = 0.f;
  }
  if (timed_out && err) atomicExch(err, 1);
}

template <int NT>
size_t smem_bytes(int KS, int KC, int S, int csize) {
  size_t n = ((size_t)NT * 8 * (KS + kXPad) * 2 + 127) / 128 * 128;
  n += (size_t)S * 16 * (KC * 2 + kRowPad);
  n += (size_t)2 * kConsumerWarps * 16 * NT * 8 * sizeof(float);
  n += csize > 1 ? (size_t)kPartTiles * 16 * NT * 8 * sizeof(float) : 0;
  n += (size_t)NT * 8 * kSsSlots * sizeof(float);
  n += (size_t)(2 * S + 1) * sizeof(uint64_t);
  return n;
}

// The ring: stages of KC elements of K for 16 weight rows.  Long copies are what the copy engine
// likes (a row of a stage is one copy of up to 2 KB), several stages keep enough bytes in flight.
struct Ring {
  int KC, S;
};
template <int NT>
bool pick_ring(int KS, int max_smem, int csize, Ring* ring) {
  const Ring tries[] = {{1024, 4}, {1024, 3}, {512, 4}, {256, 4}, {128, 4}, {64, 4}, {32, 4}};
  for (const Ring& t : tries) {
    Ring r = t;
    if (r.KC > KS) r.KC = (KS + 31) / 32 * 32;            // a short K is one stage per tile
    if (smem_bytes<NT>(KS, r.KC, r.S, csize) <= (size_t)max_smem) {
      *ring = r;
      return true;
    }
  }
  return false;
}

template <int NT, typename OutT>
int plan_and_launch(const void* x, int ldx, const void* W, int ldw, void* out, int ldo, int M, int N, int K, int gated,
                    const Fusion& fu, int* err, cudaStream_t s) {
  int dev = 0, sms = 0, max_smem = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  max_smem -= 256;                                         // the kernel's few static words count against the same limit
  // the smallest cluster whose CTAs can each hold their slice of x beside a full-size ring
  // (pairs of CTAs with three stages filled all SMs but measured no faster than triples with four)
  const Ring want = {1024, 4};
  int csize = 1;
  int KS = K;
  while (smem_bytes<NT>(KS, want.KC < KS ? want.KC : (KS + 31) / 32 * 32, want.S, csize) > (size_t)max_smem) {
    ++csize;
    if (csize > 8) return ARLE_E_UNSUPPORTED;
    KS = ((K + csize - 1) / csize + 31) / 32 * 32;
  }
  if (gated && csize > 1) return ARLE_E_UNSUPPORTED;       // the gate needs whole sums in one CTA
  auto kern = skinny_gemm_kernel<NT, OutT>;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
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
        cfg.dynamicSmemBytes = (size_t)max_smem - 1024;
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
  Ring ring;
  if (!pick_ring<NT>(KS, max_smem, csize, &ring)) return ARLE_E_UNSUPPORTED;
  const size_t smem = smem_bytes<NT>(KS, ring.KC, ring.S, csize);
  const int tiles = (N + 15) / 16;
  if (groups > tiles) groups = tiles;
  if (groups < 1) groups = 1;
  if (fu.out_ss && groups * csize > kSsSlots) return ARLE_E_UNSUPPORTED;
  const bool early = (pdl_enabled() & 3) != 0;
  e = launch_kernel_as(early, kern, dim3(groups * csize), dim3(kThreads), smem, s, csize, (const __nv_bfloat16*)x, ldx,
                       (const __nv_bfloat16*)W, ldw, (OutT*)out, ldo, M, N, K, KS, ring.KC, ring.S, csize, early ? 1 : 0,
                       gated, fu, err);
  if (e != cudaSuccess) return (int)e;
  return launch_status();
}

int skinny_entry(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M, int N, int K,
                 int gated, const Fusion& fu, int* err, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K <= 0 || K % 32 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return ARLE_E_UNSUPPORTED;
  if (((uintptr_t)x & 15) || ((uintptr_t)W & 15)) return ARLE_E_UNSUPPORTED;
  if (gated && N % 2 != 0) return ARLE_E_BADARG;
  if (fu.resid && (gated || !fu.gamma || !fu.xs || !fu.out_ss)) return ARLE_E_BADARG;
  if (!fu.resid && !out) return ARLE_E_BADARG;
  if (M <= 8) {
    if (out_dtype == 0) return plan_and_launch<1, float>(x, ldx, W, ldw, out, ldo, M, N, K, gated, fu, err, s);
    if (out_dtype == 1) return plan_and_launch<1, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, M, N, K, gated, fu, err, s);
  } else {
    if (out_dtype == 0) return plan_and_launch<2, float>(x, ldx, W, ldw, out, ldo, M, N, K, gated, fu, err, s);
    if (out_dtype == 1) return plan_and_launch<2, __nv_bfloat16>(x, ldx, W, ldw, out, ldo, M, N, K, gated, fu, err, s);
  }
  return ARLE_E_BADARG;
}

}  // namespace

// out_dtype: 0 float32, 1 bfloat16.  Needs M <= 16, K a multiple of 32, ldx and ldw multiples of 8,
// 16-byte aligned x and W.  err (may be null): set to 1 if a bounded wait ran out.
ARLE_API int arle_gemm_skinny(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M, int N,
                              int K, int* err, cudaStream_t s) {
  return skinny_entry(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, 0, Fusion{}, err, s);
}

// The gated feed-forward's first half in one launch: W [N, K] holds (gate_i, up_i) in rows 2i and
// 2i + 1, and out[M, N / 2] = silu(x . gate_i) * (x . up_i), the gate computed on the float32 sums.
// Same needs as arle_gemm_skinny, and a K short enough for x to stay in one CTA's shared memory.
ARLE_API int arle_gemm_skinny_gated(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M,
                                    int N, int K, int* err, cudaStream_t s) {
  return skinny_entry(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, 1, Fusion{}, err, s);
}

// The same two products with the fusions described at the top of the file.
//  in_ss (may be null): float32 [16][192], sums of squares of x's rows as left by an earlier launch
//    with a sink; the sums of this product are multiplied by rsqrt(sum(in_ss[m, :]) * inv_width + eps).
//  resid (may be null; not with gated): float32 [M, ldr].  When given, nothing goes to out (it may be
//    null): resid[m, n] += sum, xs[m, n] = bfloat16(resid[m, n] * gamma[n]), and out_ss [16][192] gets
//    the sums of squares of the new residual rows, every slot written.
ARLE_API int arle_gemm_skinny_fused(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M,
                                    int N, int K, int gated, const float* in_ss, float inv_width, float eps, float* resid,
                                    int ldr, const float* gamma, void* xs, int ldxs, float* out_ss, int* err,
                                    cudaStream_t s) {
  Fusion fu{in_ss, inv_width, eps, resid, ldr, gamma, (__nv_bfloat16*)xs, ldxs, out_ss};
  return skinny_entry(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, gated, fu, err, s);
}
