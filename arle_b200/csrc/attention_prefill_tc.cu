// Paged causal attention for prompt portions on the fifth-generation tensor cores
// (tcgen05), head size 128, bfloat16, page sizes that are multiples of 16.
//
// A block is 256 consecutive queries of one request and one query head, served by one CTA as two query
// tiles of 128 (A: the first 128 rows, B: the next) and walks the visible keys in tiles of
// 128 (boundaries at multiples of 128 of the absolute key position).  The two tiles share
// every key and value tile the CTA loads, and while the softmax of one runs the tensor core
// works for the other.  Everything big lives where the tensor cores want it:
//   shared memory : Q of both tiles (2 x 128 x 128) and two stages each of K and V (128 keys x
//                   128), in the 128-byte swizzled layout that TMA writes and tcgen05.mma reads;
//   tensor memory : the scores S of tile A and of tile B (128 lanes x 128 columns, float32
//                   each) and the output accumulators O of A and of B (128 x 128, float32):
//                   all 512 columns.  P of a tile is written, as bfloat16 pairs, over the first
//                   64 columns of its S once the row of S is in registers.
// Roles by warp (three warp groups; the first two take registers from the third with setmaxnreg):
//   warps 0-3, 4-7   : softmax and epilogue of tile A and of tile B; thread i owns query row i
//                      (TMEM lane i), so row maxima and sums need no shuffles.  A thread reads
//                      its row of S into registers, masks (key <= query position, and >
//                      position - window) and finds the row maximum; O and the running sum are
//                      rescaled only when the maximum grew by more than 2^8 since the last
//                      rescale (the exponentials stay within float32 and bfloat16 range); then
//                      it exponentiates, adds up and writes P into tensor memory (tcgen05.st),
//                      rounded to bfloat16 as cklxx/arle's prefill kernel rounds P
//                      (crates/cuda-kernels/tools/tilelang/batch_prefill_paged_hd128.py:223-225).
//                      After the last tile the rows are divided by their sums and stored.
//   warp 8, one lane : MMA issuer.  Per key tile j and query tile x: O_x += P_x(j) . V(j) (eight
//                      tcgen05.mma with P as the A operand read from tensor memory, and V used
//                      as it lies in the cache: an MN-major B operand), then S_x(j + 1) = Q_x .
//                      K(j + 1)^T (eight tcgen05.mma of K 16, both operands K-major) over the P
//                      just used: the tensor core runs one thread's instructions in order.
//                      tcgen05.commit signals the mbarriers; since a commit covers everything
//                      issued before it, "S_x(j + 1) is ready" also says that P_x(j) . V(j) is
//                      done, so the softmax may rescale O_x without a further wait.
//   warps 9 and 10   : loaders (keys and Q; values).  TMA tile loads (cp.async.bulk.tensor.2d):
//                      per tile the keys or the values page by page (16 keys x 64 elements per
//                      box, one box per lane) at the rows the block table names.
// CTAs stay resident (one per SM) and draw their blocks from a counter, heaviest first (the last
// queries of all heads before any earlier block).  The key loader's first lane draws the ticket, works
// out the block's shape and hands both to the other roles through a two-slot ring in shared memory; every
// role runs through the blocks at its own pace with barrier phases that count on across blocks.  So the
// loaders fetch the next block's first keys and values while the last tiles of this one are computed, its
// Q as soon as this block's last S product is done, and the tensor core has the next block's first scores
// ready when the softmax warps have normalised and stored this block's output (the next block's first
// product with the values waits until they have taken O out of tensor memory).
// Scores, maxima, sums and the accumulators are float32.  Every mbarrier wait is bounded; when one runs
// out the kernel raises the error flag, stops, draws the remaining tickets so that the counter ends at
// zero, frees its TMEM and returns.
#include "common.cuh"
#include "tcgen05_utils.cuh"
using namespace arle;

namespace {

constexpr int HD = 128;
constexpr int BQ = 128;                      // queries per query tile
constexpr int BQ2 = 2 * BQ;                  // queries per CTA: two query tiles
constexpr int BKV = 128;                     // keys per tile
constexpr int kThreads = 384;                // three warp groups: softmax of tile A, softmax of tile B, the rest
constexpr int kMmaWarp = 8, kKeyWarp = 9, kValueWarp = 10;
constexpr int kRegsSoftmax = 208, kRegsOther = 80;   // registers per thread after the warp groups have traded
constexpr uint32_t SUB = 128 * 128;          // bytes of a [128 rows x 64 elements] swizzled sub-tile
constexpr uint32_t TILE = 2 * SUB;           // 128 x 128 bfloat16
constexpr int kStages = 2;                   // stages of keys and of values
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

template <int N>
__device__ __forceinline__ void reg_more() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_less() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(N)); }

// The blocks of a running launch that were drawn after every CTA's first (which is the block of its own index).  Every
// CTA draws tickets until it draws one beyond the last block; the last ticket of all sets the counter back to zero.
// Launches take the counters in turn, so launches that run at the same time (on several streams) do not share one
// unless more than kTicketSlots of them are under way.
constexpr int kTicketSlots = 64;
__device__ unsigned int g_ticket[kTicketSlots];

// Ticket number gridDim.x + (draws before this one); the draw that must be the last of the launch resets the counter.
__device__ __forceinline__ unsigned int draw_ticket(int nblocks, int slot) {
  const unsigned int raw = atomicAdd(&g_ticket[slot], 1u);
  if (raw + 1 == (unsigned int)nblocks) atomicExch(&g_ticket[slot], 0u);      // nblocks - grid blocks and grid tickets beyond them
  return raw + gridDim.x;
}

// What a CTA's roles need to know of one block: 256 queries of one request and one query head.
struct Block {
  int r, h, kvh, t0, mbeg;
  int rows_x[2], pf_x[2], pl_x[2], jlo_x[2], jhi_x[2];
  int kb, ntiles, lo, p_last;
  // false: the block is beyond the request's queries (or the request is one that the decode kernel serves)
  __device__ bool init(int b, int nq, int nkv, int nyb, const int* q_indptr, const int* kv_lens, int window, int skip_single) {
    h = b % nq;
    const int y = (b / nq) % nyb;
    r = b / (nq * nyb);
    t0 = q_indptr[r];
    const int qlen = q_indptr[r + 1] - t0;
    // The blocks with the most keys (the last queries) come first, for all heads before any block with fewer:
    // a long block that starts late is what the others would wait for at the end.
    mbeg = (nyb - 1 - y) * BQ2;
    if (mbeg >= qlen || (skip_single && qlen == 1)) return false;
    const int kv_len = kv_lens[r];
    const int pos0 = kv_len - qlen;
    kvh = h / (nq / nkv);
    // The two query tiles: rows, positions of the first and last row, first key, tiles [jlo, jhi) of
    // the block's sequence of key tiles (which starts at kb, a multiple of 128).
    int lo_x[2];
    rows_x[0] = min(BQ, qlen - mbeg);
    rows_x[1] = max(0, min(BQ, qlen - mbeg - BQ));
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      pf_x[x] = pos0 + mbeg + x * BQ;
      pl_x[x] = pf_x[x] + max(rows_x[x], 1) - 1;
      lo_x[x] = (window > 0 && pf_x[x] - window + 1 > 0) ? pf_x[x] - window + 1 : 0;
    }
    kb = lo_x[0] / BKV * BKV;
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      jlo_x[x] = (lo_x[x] / BKV * BKV - kb) / BKV;
      jhi_x[x] = rows_x[x] > 0 ? (pl_x[x] - kb) / BKV + 1 : 0;
      if (rows_x[x] == 0) jlo_x[x] = 0;
    }
    ntiles = max(jhi_x[0], jhi_x[1]);
    lo = lo_x[0];                                      // first key any row of the block sees
    p_last = rows_x[1] > 0 ? pl_x[1] : pl_x[0];        // last key any row of the block sees
    return true;
  }
  __device__ bool in_range(int x, int j) const { return j >= jlo_x[x] && j < jhi_x[x]; }
};

constexpr int kWorkReaders = 11;             // who reads a drawn ticket: the two loader warps, the MMA thread, eight softmax warps

__global__ void __launch_bounds__(kThreads, 1) paged_prefill_tc_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, const int* __restrict__ q_indptr,
    const int* __restrict__ kv_lens, const int* __restrict__ block_table, int bt_stride, int bt_width, int nq, int nkv,
    int page_size, float scale_log2, int window, int skip_single, int nyb, int nblocks, int ticket_slot, int* __restrict__ err) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = base;                              // 2 x TILE
  unsigned char* k_s = base + 2 * TILE;                   // kStages x TILE
  unsigned char* v_s = base + (2 + kStages) * TILE;       // kStages x TILE
  __shared__ __align__(8) uint64_t q_full, q_empty, k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages], s_full[2],
      p_full[2], o_full[2], o_empty[2], work_full[2], work_empty[2];
  __shared__ int work_id[2];                             // the drawn block, -1: none left; -2: a block without queries
  __shared__ Block work_blk[2];                          // and its shape, worked out by the thread that drew it
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the CTA's first block is the one of its own index: its shape is worked out while the rest is set up
  bool first_has_queries = false;
  if (warp == kKeyWarp && lane == 0)
    first_has_queries = work_blk[0].init((int)blockIdx.x, nq, nkv, nyb, q_indptr, kv_lens, window, skip_single);
  if (threadIdx.x == 0) {
    mbar_init(smem_addr(&q_full), 1);
    mbar_init(smem_addr(&q_empty), 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(smem_addr(&k_full[i]), 1);
      mbar_init(smem_addr(&k_empty[i]), 1);
      mbar_init(smem_addr(&v_full[i]), 1);
      mbar_init(smem_addr(&v_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_addr(&s_full[i]), 1);
      mbar_init(smem_addr(&p_full[i]), 4);
      mbar_init(smem_addr(&o_full[i]), 1);
      mbar_init(smem_addr(&o_empty[i]), 4);
      mbar_init(smem_addr(&work_full[i]), 1);
      mbar_init(smem_addr(&work_empty[i]), kWorkReaders);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  // Value rows that no load ever fills (beyond the last key) meet P = 0; they must hold
  // numbers, not whatever bits shared memory had (later blocks find an earlier tile's values there).
  for (uint32_t i = threadIdx.x; i < kStages * TILE / 16; i += kThreads) reinterpret_cast<uint4*>(v_s)[i] = make_uint4(0, 0, 0, 0);
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  if (warp == kMmaWarp) {
    tmem_alloc(smem_addr(&tmem_base_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  // columns: S of tile A, S of tile B, O of tile A, O of tile B (128 each).  P of a tile is written over
  // the first 64 columns of its S (two bfloat16 a column) once the row of S is in registers.
  const volatile int* aborted = &abort_flag;

  // The i-th ticket that this CTA drew, as every role learns it: -1 when the blocks are used up (or a wait ran out),
  // -2 for a block without queries.  A reader copies the block's shape and then says that it has it, so that the slot
  // can take the ticket after the next.
  auto wait_ticket = [&](int i) -> int {
    if (!mbar_wait_bounded(smem_addr(&work_full[i & 1]), (uint32_t)((i >> 1) & 1), aborted)) return -1;
    return work_id[i & 1];
  };
  auto release_ticket = [&](int i) { mbar_arrive(smem_addr(&work_empty[i & 1])); };

  if (warp >= 8) {
    reg_less<kRegsOther>();
    if (warp == kKeyWarp || warp == kValueWarp) {
      // One warp loads the keys, one the values, each at its own pace: a tile is 16 boxes per
      // operand (8 pages x 2 halves of the head), one per lane, so that their issue overlaps;
      // lane 0 waits for the stage and arms its barrier.  The key warp's first lane also draws the tickets.
      const bool keys = warp == kKeyWarp;
      const int c = (lane >> 1) & 7, half = lane & 1;      // page of the tile, half of the head (lanes 0..15)
      const CUtensorMap* map = keys ? &map_k : &map_v;
      unsigned char* tile_s = keys ? k_s : v_s;
      int issued = 0;                                       // tiles whose loads were issued, over all blocks
      int q_loads = 0;                                      // blocks whose Q was asked for
      bool ended = false;                                   // the terminal ticket is drawn
      for (int it = 0;; ++it) {
        if (keys && lane == 0) {
          int b = -1;
          if (it == 0) {
            b = first_has_queries ? (int)blockIdx.x : -2;
          } else if (it < 2 || mbar_wait_bounded(smem_addr(&work_empty[it & 1]), (uint32_t)(((it >> 1) & 1) ^ 1), aborted)) {
            if (!*aborted) {
              const unsigned int tk = draw_ticket(nblocks, ticket_slot);
              if (tk < (unsigned int)nblocks) b = (int)tk; else ended = true;
              if (b >= 0 && !work_blk[it & 1].init(b, nq, nkv, nyb, q_indptr, kv_lens, window, skip_single)) b = -2;
            }
          } else {
            abort_flag = 1;
          }
          work_id[it & 1] = b;
          asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(&work_full[it & 1])) : "memory");
        }
        __syncwarp();
        const int b = __shfl_sync(0xffffffffu, lane == 0 ? wait_ticket(it) : 0, 0);
        __syncwarp();                                       // the first lane's wait orders the other lanes' reads of the slot
        Block blk;
        if (b >= 0) blk = work_blk[it & 1];
        __syncwarp();
        if (lane == 0 && b != -1) release_ticket(it);
        if (b == -1) break;
        if (b == -2) continue;
        if (keys && lane == 0) {
          // Q of this block, once the S products of the block before have read theirs
          bool free_q = q_loads == 0 || mbar_wait_bounded(smem_addr(&q_empty), (uint32_t)((q_loads - 1) & 1), aborted);
          if (!free_q) abort_flag = 1;
          if (free_q) {
            const int nload = blk.rows_x[1] > 0 ? 2 : 1;
            mbar_expect_tx(smem_addr(&q_full), (uint32_t)nload * TILE);
            for (int x = 0; x < nload; ++x) {
              tma_load_2d(smem_addr(q_s + x * TILE), &map_q, blk.h * HD, blk.t0 + blk.mbeg + x * BQ, smem_addr(&q_full));
              tma_load_2d(smem_addr(q_s + x * TILE + SUB), &map_q, blk.h * HD + 64, blk.t0 + blk.mbeg + x * BQ, smem_addr(&q_full));
            }
            ++q_loads;
          }
        }
        const int* bt = block_table + (size_t)blk.r * bt_stride;
        // Page ids come 32 at a time, one per lane, with the next 32 already in flight, so that no
        // tile waits for a read of the block table; a lane picks its page with a shuffle.
        int p0 = blk.kb / page_size;
        int cur = __ldg(bt + min(p0 + lane, bt_width - 1));
        int nxt = __ldg(bt + min(p0 + 32 + lane, bt_width - 1));
        bool stop = false;
        for (int j = 0; j < blk.ntiles; ++j) {
          const int st = issued % kStages;
          const uint32_t par = (uint32_t)((issued / kStages) & 1);
          const int key0 = blk.kb + j * BKV + c * 16;
          while ((blk.kb + j * BKV) / page_size - p0 >= 32) {
            cur = nxt;
            p0 += 32;
            nxt = __ldg(bt + min(p0 + 32 + lane, bt_width - 1));
          }
          const int pi = key0 / page_size;
          const int rel = pi - p0;                                // 0 .. 63: a tile spans at most 8 pages
          const int from_cur = __shfl_sync(0xffffffffu, cur, rel & 31), from_nxt = __shfl_sync(0xffffffffu, nxt, rel & 31);
          int row = -1;
          if (lane < 16 && key0 <= blk.p_last && key0 + 15 >= blk.lo) {
            const int page = rel < 32 ? from_cur : from_nxt;
            row = (page * nkv + blk.kvh) * page_size + (key0 - pi * page_size);
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
          if (!go || *aborted) {
            stop = true;
            break;
          }
          if (row >= 0) tma_load_2d(smem_addr(tile_s + st * TILE + half * SUB + c * 2048), map, half * 64, row, smem_addr(full));
          ++issued;
        }
        if (stop) break;
      }
      if (keys && lane == 0 && !ended) {
        // a wait ran out: the tickets are still drawn to the end, so that the counter is back at zero for the next launch
        for (int i = 0; i <= nblocks; ++i)
          if (draw_ticket(nblocks, ticket_slot) >= (unsigned int)nblocks) break;
      }
      // No copy may still be in flight when the CTA ends.  The issuing thread has waited for every tile
      // unless a wait ran out, so this is free otherwise.
      if (lane == 0) {
        if (keys && q_loads > 0) mbar_wait_plain(smem_addr(&q_full), (uint32_t)((q_loads - 1) & 1));
        for (int s2 = 0; s2 < kStages && s2 < issued; ++s2) {
          const int last = (issued - 1 - s2) / kStages * kStages + s2;       // last tile loaded into stage s2
          mbar_wait_plain(smem_addr(keys ? &k_full[s2] : &v_full[s2]), (uint32_t)((last / kStages) & 1));
        }
      }
    } else if (warp == kMmaWarp && lane == 0) {
      constexpr uint32_t idesc_s = idesc_bf16(BQ, BKV);                  // A and B K-major
      constexpr uint32_t idesc_pv = idesc_bf16(BQ, HD) | (1u << 16);    // B (values) MN-major
      bool ok = true;
      int g0 = 0;                                                        // key tiles of the blocks before
      int q_uses = 0;                                                    // blocks whose Q was used
      int done_p[2] = {0, 0};                                            // P tiles of each query tile consumed so far, over all blocks
      int o_blocks[2] = {0, 0};                                          // blocks in which each query tile had rows
      for (int it = 0; ok; ++it) {
        const int b = wait_ticket(it);
        Block blk;
        if (b >= 0) blk = work_blk[it & 1];
        release_ticket(it);
        if (b == -1) break;
        if (b == -2) continue;
        ok = mbar_wait_bounded(smem_addr(&q_full), (uint32_t)(q_uses & 1), aborted);
        ++q_uses;
        // S of query tile x for key tile j (the key stage must be full)
        auto issue_s = [&](int x, int j) {
          const int kst = (g0 + j) % kStages;
#pragma unroll
          for (int dh = 0; dh < 2; ++dh) {
            const uint64_t ad = smem_desc_sw128(smem_addr(q_s + x * TILE + dh * SUB));
            const uint64_t bd = smem_desc_sw128(smem_addr(k_s + kst * TILE + dh * SUB));
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_bf16(tmem_base + (uint32_t)(x * BKV), ad + 2 * k, bd + 2 * k, idesc_s, (dh | k) != 0 ? 1u : 0u);
          }
          umma_commit(smem_addr(&s_full[x]));
        };
        // key tile 0 for the query tiles that start there (S of a tile goes over the P of the tile before, the
        // last of the block before included: the tensor core runs them in the order issued)
        if (ok) {
          ok = mbar_wait_bounded(smem_addr(&k_full[g0 % kStages]), (uint32_t)((g0 / kStages) & 1), aborted);
          if (ok) {
            tc_fence_after();
            if (blk.in_range(0, 0)) issue_s(0, 0);
            if (blk.in_range(1, 0)) issue_s(1, 0);
            umma_commit(smem_addr(&k_empty[g0 % kStages]));
            if (blk.ntiles == 1) umma_commit(smem_addr(&q_empty));        // every S of the block is issued
          }
        }
        int first_pv[2] = {1, 1};
        for (int j = 0; j < blk.ntiles && ok; ++j) {
          const int vst = (g0 + j) % kStages, knext = (g0 + j + 1) % kStages;
          bool v_ready = false, k_ready = false;
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            if (blk.in_range(x, j)) {
              if (!mbar_wait_bounded(smem_addr(&p_full[x]), (uint32_t)(done_p[x] & 1), aborted)) { ok = false; break; }
              if (!v_ready) {
                if (!mbar_wait_bounded(smem_addr(&v_full[vst]), (uint32_t)(((g0 + j) / kStages) & 1), aborted)) { ok = false; break; }
                v_ready = true;
              }
              if (first_pv[x] && o_blocks[x] > 0) {
                // the block before has taken its O out of tensor memory
                if (!mbar_wait_bounded(smem_addr(&o_empty[x]), (uint32_t)((o_blocks[x] - 1) & 1), aborted)) { ok = false; break; }
              }
              tc_fence_after();
#pragma unroll
              for (int kk = 0; kk < 8; ++kk) {
                const uint64_t bd = smem_desc_mn_sw128(smem_addr(v_s + vst * TILE + kk * 2048), SUB);
                umma_bf16_a_tmem(tmem_base + (uint32_t)(256 + x * HD), tmem_base + (uint32_t)(x * BKV + kk * 8), bd, idesc_pv,
                                 (first_pv[x] && kk == 0) ? 0u : 1u);
              }
              first_pv[x] = 0;
              ++done_p[x];
              if (j + 1 == blk.jhi_x[x]) {
                umma_commit(smem_addr(&o_full[x]));
                ++o_blocks[x];
              }
            }
            // S of the next key tile goes over this P: the tensor core runs them in the order issued
            if (blk.in_range(x, j + 1)) {
              if (!k_ready) {
                if (!mbar_wait_bounded(smem_addr(&k_full[knext]), (uint32_t)(((g0 + j + 1) / kStages) & 1), aborted)) { ok = false; break; }
                k_ready = true;
                tc_fence_after();
              }
              issue_s(x, j + 1);
            }
          }
          if (!ok) break;
          umma_commit(smem_addr(&v_empty[vst]));                  // tile j's values are read by what was issued so far
          if (j + 1 < blk.ntiles) {
            umma_commit(smem_addr(&k_empty[knext]));
            if (j + 2 == blk.ntiles) umma_commit(smem_addr(&q_empty));    // every S of the block is issued
          }
        }
        g0 += blk.ntiles;
      }
      if (!ok) abort_flag = 1;
    }
  } else {
    reg_more<kRegsSoftmax>();
    const int x = warp >> 2;                                   // query tile of this warp group
    const int row = (warp & 3) * 32 + lane;                    // query row of the tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tmem_s = tmem_base + (uint32_t)(x * BKV), tmem_o = tmem_base + (uint32_t)(256 + x * HD);
    bool ok = true;
    int n_all = 0;                                             // S tiles of this query tile taken so far, over all blocks
    int o_all = 0;                                             // blocks in which this query tile had rows
    for (int it = 0; ok; ++it) {
      int b = lane == 0 ? wait_ticket(it) : 0;
      b = __shfl_sync(0xffffffffu, b, 0);
      __syncwarp();                                         // the first lane's wait orders the other lanes' reads of the slot
      Block blk;
      if (b >= 0) blk = work_blk[it & 1];
      __syncwarp();
      if (lane == 0) release_ticket(it);
      if (b == -1) break;
      if (b == -2) continue;
      const int p_first = blk.pf_x[x], pl = blk.pl_x[x];
      const int jlo = blk.jlo_x[x], jhi = blk.jhi_x[x], rows_here = blk.rows_x[x];
      const int kb = blk.kb;
      const int p_row = min(p_first + row, pl);
      const int lo_row = window > 0 ? p_row - window + 1 : 0;
      float m_used = -INFINITY, l = 0.f;
      int n = 0;
      for (int j = jlo; j < jhi; ++j, ++n, ++n_all) {
        const int k0 = kb + j * BKV;
        const bool full_tile = k0 + BKV - 1 <= p_first && (window <= 0 || k0 >= pl - window + 1);
        bool ready = mbar_wait_bounded(smem_addr(&s_full[x]), (uint32_t)(n_all & 1), aborted);
        if (__any_sync(0xffffffffu, !ready)) { ok = false; break; }
        tc_fence_after();
        // The whole row of scores comes into registers at once (four loads in flight, one wait).
        uint32_t sv[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(tmem_s + lane_addr + (uint32_t)(c * 32), sv[c]);
        tmem_ld_wait();
        // the row maximum (raw scores; the scale is positive, so it is applied to the maximum
        // alone).  Four running maxima keep the chain of dependent instructions short.
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
        // O may be rescaled here without a wait: S of this key tile was issued after P.V of the tile
        // before, and its completion (which s_full reports) covers everything issued before it.
        const bool rescale = n > 0 && __any_sync(0xffffffffu, f != 1.0f);
        if (rescale) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t v[32];
            tmem_ld32(tmem_o + lane_addr + (uint32_t)(c * 32), v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
            tmem_st32(tmem_o + lane_addr + (uint32_t)(c * 32), v);
          }
        }
        // exponentials (one fused multiply-add and one ex2 each; a masked score is -inf and
        // gives 0), their sum in four partial sums, and P as bfloat16 over the first half of S
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
          tmem_st32(tmem_s + lane_addr + (uint32_t)(h2 * 32), packed);
        }
        tmem_st_wait();
        l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_addr(&p_full[x]));
      }
      if (ok && n > 0) {
        const bool ready = mbar_wait_bounded(smem_addr(&o_full[x]), (uint32_t)(o_all & 1), aborted);
        if (__any_sync(0xffffffffu, !ready)) ok = false;
      }
      if (ok && n > 0) {
        ++o_all;
        tc_fence_after();
        const float inv = 1.0f / l;
        __nv_bfloat16* orow = out + ((size_t)(blk.t0 + blk.mbeg + x * BQ + row) * nq + blk.h) * HD;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld32(tmem_o + lane_addr + (uint32_t)(c * 32), v);
          tmem_ld_wait();
          if (c == 3) {
            // O is in registers: the next block's first product with the values may overwrite it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_addr(&o_empty[x]));
          }
          if (row < rows_here) {
            uint32_t p[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(v[2 * i]) * inv, __uint_as_float(v[2 * i + 1]) * inv);
              p[i] = *reinterpret_cast<uint32_t*>(&b2);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
              reinterpret_cast<uint4*>(orow + c * 32)[i] = make_uint4(p[4 * i], p[4 * i + 1], p[4 * i + 2], p[4 * i + 3]);
          }
        }
      }
    }
    if (!ok && lane == 0) abort_flag = 1;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
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
  if (hd != HD || page_size % 16 != 0 || nq <= 0 || nkv <= 0 || nq % nkv != 0 || rows > 65535 || (max_q_len + BQ2 - 1) / BQ2 > 65535)
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
  const size_t smem = (2 + 2 * kStages) * (size_t)TILE + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(paged_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  // CTAs stay resident and draw blocks (a query head, 256 queries of a request) from a counter, the heaviest first
  const int nyb = (max_q_len + BQ2 - 1) / BQ2;
  const long long nblocks = (long long)nq * nyb * rows;
  if (nblocks > 0x3fffffffLL) return ARLE_E_UNSUPPORTED;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int ctas = (int)(nblocks < sms ? nblocks : sms);
  static unsigned int launches = 0;
  const int ticket_slot = (int)(launches++ % kTicketSlots);
  cudaError_t e = launch_kernel(paged_prefill_tc_kernel, dim3(ctas), dim3(kThreads), smem, s, 1, mq, mk, mv, (__nv_bfloat16*)out,
                                q_indptr, kv_lens, block_table, bt_stride, bt_width, nq, nkv, page_size,
                                scale * 1.4426950408889634f, window, skip_single, nyb, (int)nblocks, ticket_slot, err);
  if (e != cudaSuccess) return (int)e;
  return launch_status();
}
