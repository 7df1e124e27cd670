// Streaming paged attention for decoded tokens (one query per request), bfloat16, head
// sizes 64 and 128, up to 16 query heads per kv head, page sizes that are multiples of 16.
//
// Decoding reads every key and value of the batch once; the kernel is built so that this
// stream never stops.  A grid of one CTA per SM stays resident.  The work is cut into units
// of one 64-key tile of one (request, kv head) pair, ordered by request, kv head and key
// position, and every CTA takes the same number of consecutive units whatever the lengths
// of the requests are; a CTA's range may end in the middle of one pair and go on into the
// next.  Roles by warp:
//   warps 8 and 9    : producers (keys; values).  Each walks the CTA's units and brings its
//                      operand of every tile in with TMA (cp.async.bulk.tensor.3d, boxes of 16
//                      keys of the whole head at the rows the block table names, 128-byte
//                      swizzle) into a ring of stages, as far ahead as the ring is deep; they
//                      never wait for arithmetic.  (Issuing a box costs a warp some 130
//                      cycles whatever its size, hence two warps and boxes as big as a page.)
//   warps 0-7        : two groups of four warps take tiles in turn.  A warp owns 16 keys of
//                      its group's tile: Q.K^T and P.V on the tensor cores (mma.sync
//                      m16n8k16, the query heads of the kv head padded to 16 rows), scores,
//                      online softmax and accumulators in float32, P rounded to bfloat16 for
//                      P.V as in cklxx/arle's decode kernel
//                      (crates/cuda-kernels/tools/tilelang/batch_decode_paged_hd128.py:134-231).
// When a pair's units end (or the CTA's range does) the eight warps merge their partial
// results in shared memory.  A pair that one CTA covered alone is written out; otherwise the
// CTA stores an unnormalised partial (o, m, l) and the CTA that arrives last at the pair's
// counter combines the pieces in the order of the keys (the reference's split-KV variant
// runs a second kernel for that, :239-463).  Nothing waits for another CTA.
// Fused preparation (optional, for steps that decode only): the kernel is given the raw projection
// output [q heads | k heads | v heads] of every token instead of prepared queries and does what the
// preparation kernel does for a decoded token itself: per-head RMSNorm and rotation of the pair's
// query heads (every CTA, for the pairs it holds a piece of: a few hundred numbers), and of the
// token's new key (the CTA that holds the pair's last tile), whose key and value it stores into the
// cache and writes over the stale slot of the tile in shared memory before the tile is used.  One
// launch and one pass over the projection output fewer per layer.
// The table of the rows, the shares of the CTAs and each CTA's first page ids depend on the step alone, not on the
// layer: arle_decode_stream_plan writes them out once per step (one block per CTA of the launches to come), and a launch
// that is given the plan reads it in one round trip to memory instead of working it out in three.
// Rows whose step entry has more than one token are skipped.  The key range of a row is
// [max(0, kv_len - window), kv_len).  Every mbarrier wait is bounded: when one runs out the
// kernel raises the error flag, stops waiting and runs to its end.
#include "common.cuh"
#include "mma_utils.cuh"
#include "tcgen05_utils.cuh"
using namespace arle;

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + 64;          // two producer warps: keys, values
constexpr int kTile = 64;                          // keys per unit
constexpr int kMaxStages = 8;
constexpr int kStaticSmem = 2 * kMaxStages * 8 + 32;   // bytes of __shared__ variables in the kernel: the barriers, six words

__device__ __forceinline__ void mbar_arrive_one(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(kConsumers) : "memory"); }

// Where a CTA's range of units meets the rows: which row, kv head and tile a unit is.
struct Rows {
  const int* prefix;     // [R + 1] units before each row
  const int* kvl;        // [R] keys of the row, -1 for a row that is not decoded here
  int R, nkv, window;
  __device__ __forceinline__ void tiles_of(int r, int& lo, int& kv_len, int& tlo, int& thi) const {
    kv_len = kvl[r];
    lo = (window > 0 && kv_len > window) ? kv_len - window : 0;
    tlo = lo / kTile;
    thi = (kv_len + kTile - 1) / kTile;
  }
  // the row r with prefix[r] <= u < prefix[r + 1]
  __device__ __forceinline__ int row_of(int u) const {
    int a = 0, b = R;                   // invariant: prefix[a] <= u < prefix[b]
    while (b - a > 1) {
      const int mid = (a + b) >> 1;
      if (prefix[mid] <= u) a = mid; else b = mid;
    }
    return a;
  }
};

// Fused preparation: q then points at the raw projection output of the step's tokens (row stride
// q_row_stride, a row holds nq query heads, nkv key heads, nkv value heads).
struct Prep {
  int on;                       // 0: q holds prepared queries, nothing else here is used
  const int* slot_mapping;      // [tokens] page * page_size + slot of the token's key and value
  const float* q_weight;        // [HD] or null: no norm
  const float* k_weight;
  float eps;
  const float* inv_freq;        // [HD / 2] or null: no rotation
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
};

// One head of HD elements, lane l holding elements l * HD / 32 ..: RMSNorm over the head (if w), then the
// half-split rotation by pos (if inv_freq); the same arithmetic, in the same order, as the preparation kernel.
template <int HD>
__device__ __forceinline__ void prep_head(const __nv_bfloat16* src, const float* w, float eps, const float* inv_freq,
                                          float pos, int lane, __nv_bfloat16* dst) {
  constexpr int VE = HD / 32;
  float x[VE];
#pragma unroll
  for (int i = 0; i < VE; ++i) x[i] = __bfloat162float(src[lane * VE + i]);
  if (w) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VE; ++i) ss += x[i] * x[i];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
    for (int i = 0; i < VE; ++i) x[i] = x[i] * inv * w[lane * VE + i];
  }
#pragma unroll
  for (int i = 0; i < VE; ++i) {
    float o = x[i];
    if (inv_freq) {
      const float other = __shfl_xor_sync(0xffffffffu, x[i], 16);
      float sn, cs;
      sincosf(pos * inv_freq[(lane & 15) * VE + i], &sn, &cs);
      o = lane < 16 ? x[i] * cs - other * sn : other * sn + x[i] * cs;
    }
    dst[lane * VE + i] = __float2bfloat16_rn(o);
  }
}

constexpr int kPlanHeader = 4;               // units, units per CTA, shared out by pair or not, unused

// The rows' table and the CTAs' shares, by all threads of a block (kThreads of them).  prefix [R + 1], kvl [R], tok [R]
// and the scalars are in shared memory; the scalars own_* are those of CTA `cta`.  Ends with a barrier.
__device__ __forceinline__ void stream_shares(const int* __restrict__ q_indptr, const int* __restrict__ kv_lens, int R, int nkv,
                                              int window, int C, int cta, int* prefix, int* kvl, int* tok, int* units_out,
                                              int* per_out, int* by_pair_out, int* own_row_out, int* own_first_out,
                                              int* own_k_out) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int r = tid; r < R; r += kThreads) {
    const int t = q_indptr[r], t_end = q_indptr[r + 1], len = kv_lens[r];     // three loads under way at once, not one after another
    const bool single = t_end - t == 1;
    const int kv_len = single ? len : -1;
    kvl[r] = kv_len;
    tok[r] = t;
    int units = 0;
    if (kv_len > 0) {
      const int lo = (window > 0 && kv_len > window) ? kv_len - window : 0;
      units = ((kv_len + kTile - 1) / kTile - lo / kTile) * nkv;
    }
    prefix[r + 1] = units;
  }
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    if (lane == 0) prefix[0] = 0;
    for (int base = 0; base < R; base += 32) {
      const int i = base + lane;
      int v = i < R ? prefix[i + 1] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
      }
      if (i < R) prefix[i + 1] = carry + v;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();

  const int U = prefix[R];
  const int per = max(1, (U + C - 1) / C);               // units per CTA
  if (tid == 0) *units_out = U, *per_out = per;
  // Two ways of sharing out the units.  Evenly, whatever the pairs are: CTA c takes units
  // [c * per, (c + 1) * per), and its range may end inside one pair and go on into the next; every such
  // piece costs a merge and a hand-over.  Or, when there are fewer pairs than CTAs (few rows), by pair:
  // the pairs of row r get k_r = T_r C / U CTAs each (T_r tiles, rounded down, at least one) and a CTA takes
  // one piece of one pair, ceil(T_r / k_r) tiles: one merge per CTA, and none handed over when k_r = 1.
  // By pair is taken when no CTA gets more than 5/4 of an even share.
  if (warp == 0) {
    int mine_row = -1, mine_first = 0, mine_k = 0, carry = 0, worst = 0;
    const bool may = U > 0 && (long long)R * nkv <= C;
    for (int base = 0; may && base < R; base += 32) {
      const int i = base + lane;
      const int T_i = i < R ? (prefix[i + 1] - prefix[i]) / nkv : 0;
      const int k_i = T_i > 0 ? max(1, (int)((long long)T_i * C / U)) : 0;
      worst = max(worst, k_i ? (T_i + k_i - 1) / k_i : 0);
      int v = k_i * nkv;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
      }
      const int first = carry + v - k_i * nkv;
      if (k_i && first <= cta && cta < first + k_i * nkv) mine_row = i, mine_first = first, mine_k = k_i;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) worst = max(worst, __shfl_xor_sync(0xffffffffu, worst, o));
    const bool take = may && carry <= C && 4 * worst <= 5 * per;
    if (lane == 0) *by_pair_out = take ? 1 : 0, *own_row_out = -1;
    __syncwarp();
    if (take && mine_row >= 0) *own_row_out = mine_row, *own_first_out = mine_first, *own_k_out = mine_k;
  }
  __syncthreads();
}

// The units [u0, u1) of CTA `cta` from the shares (u0 >= u1: none).
__device__ __forceinline__ void own_units(int cta, int by_pair, int own_row, int own_first, int own_k, const int* prefix, int nkv,
                                          int U, int per, int& u0, int& u1) {
  if (by_pair) {
    if (own_row < 0) {
      u0 = u1 = 0;
      return;
    }
    const int T = (prefix[own_row + 1] - prefix[own_row]) / nkv;
    const int rel = cta - own_first;
    const int kvh = rel / own_k, piece = rel - kvh * own_k;
    const int tp = (T + own_k - 1) / own_k;
    const int pair_begin = prefix[own_row] + kvh * T;
    u0 = pair_begin + piece * tp;
    u1 = min(pair_begin + T, u0 + tp);
  } else {
    u0 = cta * per;
    u1 = min(U, u0 + per);
  }
}

// The plan of a step: what every launch of decode_stream_kernel with these rows, kv heads, window, block table and grid
// works out before it can ask for its first keys, written out once (one block per CTA of those launches) so that the
// launches of the step's layers read it instead: one round trip to memory where they made three, one after another.
// plan: [units, units per CTA, by pair, 0], then (own_row, own_first, own_k) of every CTA, then the first 32 page ids of
// every CTA's first piece (what its producers would read from the block table first), then prefix [R + 1], kvl [R], tok [R].
__global__ void __launch_bounds__(kThreads) decode_stream_plan_kernel(const int* __restrict__ q_indptr, const int* __restrict__ kv_lens,
                                                                      const int* __restrict__ block_table, int bt_stride, int bt_width,
                                                                      int page_size, int R, int nkv, int window, int* __restrict__ plan) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int rows_s[];                         // prefix [R + 1], kvl [R], tok [R]
  __shared__ int units, per, by_pair, own_row, own_first, own_k;
  const int C = (int)gridDim.x, cta = (int)blockIdx.x;
  stream_shares(q_indptr, kv_lens, R, nkv, window, C, cta, rows_s, rows_s + R + 1, rows_s + 2 * R + 1, &units, &per, &by_pair, &own_row,
                &own_first, &own_k);
  const int tid = threadIdx.x;
  int* triples = plan + kPlanHeader;
  int* pages = triples + 3 * C;
  int* rows_out = pages + 32 * C;
  if (cta == 0) {
    for (int i = tid; i < 3 * R + 1; i += kThreads) rows_out[i] = rows_s[i];
    if (tid == 0) plan[0] = units, plan[1] = per, plan[2] = by_pair, plan[3] = 0;
  }
  if (tid == 0) triples[3 * cta] = own_row, triples[3 * cta + 1] = own_first, triples[3 * cta + 2] = own_k;
  if (tid < 32) {
    int u0, u1, page = 0;
    own_units(cta, by_pair, own_row, own_first, own_k, rows_s, nkv, units, per, u0, u1);
    if (u0 < u1) {
      const Rows rows{rows_s, rows_s + R + 1, R, nkv, window};
      const int r = rows.row_of(u0);
      int lo, kv_len, tlo, thi;
      rows.tiles_of(r, lo, kv_len, tlo, thi);
      const int tile0 = tlo + (u0 - rows_s[r]) % (thi - tlo);
      const int p0 = tile0 * kTile / page_size;
      page = block_table[(size_t)r * bt_stride + min(p0 + tid, bt_width - 1)];
    }
    pages[32 * cta + tid] = page;
  }
}

template <int HD>
__global__ void __launch_bounds__(kThreads, 1) decode_stream_kernel(
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
    const __nv_bfloat16* __restrict__ q, int q_row_stride, __nv_bfloat16* __restrict__ out,
    const int* __restrict__ q_indptr, const int* __restrict__ kv_lens, const int* __restrict__ block_table, int bt_stride,
    float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters, int R, int nq, int nkv,
    int bt_width, int page_size, int ps_shift, float scale_log2, int window, int stages, Prep prep, const int* __restrict__ plan,
    int* __restrict__ err) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr uint32_t OPERAND = kTile * HD * 2;            // bytes of the keys (or the values) of one stage
  constexpr uint32_t STAGE = 2 * OPERAND;
  constexpr uint32_t BOX = 16 * HD * 2;                   // bytes of one box: 16 keys, as HD / 64 blocks of [16 x 128 bytes]
  constexpr int NBOX = 4;                                 // boxes of an operand in a stage: 4 x 16 keys
  const int G = nq / nkv;
  const int C = (int)gridDim.x;

  extern __shared__ unsigned char smem_dyn[];
  unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  float* mo = reinterpret_cast<float*>(ring + (size_t)stages * STAGE);      // [8][G][HD] partial outputs of the warps
  float* mm = mo + kConsumerWarps * G * HD;                                 // [8][16] maxima
  float* mlv = mm + kConsumerWarps * 16;                                    // [8][16] sums
  int* prefix = reinterpret_cast<int*>(mlv + kConsumerWarps * 16);          // [R + 1]
  int* kvl = prefix + R + 1;                                                // [R]
  int* tok = kvl + R;                                                       // [R]
  __nv_bfloat16* heads = reinterpret_cast<__nv_bfloat16*>(mlv + kConsumerWarps * 16 + ((3 * R + 1 + 3) & ~3));   // [18][HD]: 16 query heads, new key, new value
  __shared__ __align__(8) uint64_t full[kMaxStages], empty[kMaxStages];
  __shared__ int abort_flag, is_last;
  __shared__ int own_row, own_first, own_k, by_pair;        // the CTA's place when pairs are shared out whole (below)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int i = 0; i < stages; ++i) {
      mbar_init(smem_addr(&full[i]), 2);                  // the two producer warps, each with its bytes
      mbar_init(smem_addr(&empty[i]), 4);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  // A warp reads a 16-key block of a stage only if the block has a key in range, and such a
  // block was loaded whole (slots of its page beyond the last key hold old, finite cache
  // contents that meet P = 0), so the ring needs no clearing.
  if (warp >= kConsumerWarps && lane == 0) {
    const CUtensorMap* m = warp > kConsumerWarps ? &map_v : &map_k;
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(m) : "memory");
  }
  __shared__ int plan_units, plan_per;
  int first_pages = 0;                                    // a producer lane's page id of the CTA's first piece (with a plan)
  if (plan) {
    // The step's plan (arle_decode_stream_plan): the rows' table and the shares worked out once for all layers
    const int* rows_plan = plan + kPlanHeader + (3 + 32) * C;
    for (int i = tid; i < 3 * R + 1; i += kThreads) prefix[i] = rows_plan[i];          // prefix, kvl, tok lie one after the other
    if (warp >= kConsumerWarps) first_pages = plan[kPlanHeader + 3 * C + 32 * blockIdx.x + lane];
    if (tid == 0) {
      plan_units = plan[0], plan_per = plan[1], by_pair = plan[2];
      own_row = plan[kPlanHeader + 3 * blockIdx.x], own_first = plan[kPlanHeader + 3 * blockIdx.x + 1];
      own_k = plan[kPlanHeader + 3 * blockIdx.x + 2];
    }
    __syncthreads();
  } else {
    stream_shares(q_indptr, kv_lens, R, nkv, window, C, (int)blockIdx.x, prefix, kvl, tok, &plan_units, &plan_per, &by_pair, &own_row,
                  &own_first, &own_k);
  }
  const int U = plan_units;
  const int per = plan_per;
  int u0, u1;
  own_units((int)blockIdx.x, by_pair, own_row, own_first, own_k, prefix, nkv, U, per, u0, u1);
  if (u0 >= u1) return;
  const Rows rows{prefix, kvl, R, nkv, window};
  const volatile int* aborted = &abort_flag;
  const uint32_t ring_addr = smem_addr(ring);

  if (warp >= kConsumerWarps) {
    // ------------------------------------------------------------------ producer
    const int op = warp - kConsumerWarps;                 // 0: this warp brings the keys, 1: the values
    const int c = lane & 3;                               // 16-key block of the tile
    const CUtensorMap* map = op ? &map_v : &map_k;
    const uint32_t dst_off = (uint32_t)op * OPERAND + (uint32_t)c * BOX;
    int st = 0, issued = 0;
    uint32_t par = 0;
    bool ok = true;
    for (int u = u0; u < u1 && ok;) {
      const int r = rows.row_of(u);
      int lo, kv_len, tlo, thi;
      rows.tiles_of(r, lo, kv_len, tlo, thi);
      const int T = thi - tlo;
      const int rem = u - prefix[r];
      const int kvh = rem / T;
      const int tile0 = tlo + rem % T;
      const int pe = min(prefix[r] + (kvh + 1) * T, u1);
      const int ntile = pe - u;
      const int* bt = block_table + (size_t)r * bt_stride;
      auto wanted = [&](int key0) { return lane < NBOX && key0 < kv_len && key0 + 16 > lo; };
      auto page_index = [&](int key) { return ps_shift >= 0 ? key >> ps_shift : key / page_size; };
      // Page ids come 32 at a time, one per lane, and a second 32 ahead of them, so that no
      // tile waits for a read of the block table; a lane picks its page with a shuffle.
      int p0 = page_index(tile0 * kTile);
      int cur = (plan && u == u0) ? first_pages : __ldg(bt + min(p0 + lane, bt_width - 1));
      int nxt = __ldg(bt + min(p0 + 32 + lane, bt_width - 1));
      int key0 = tile0 * kTile + c * 16;
      for (int i = 0; i < ntile; ++i) {
        while (page_index(key0 - c * 16) - p0 >= 32) {
          cur = nxt;
          p0 += 32;
          nxt = __ldg(bt + min(p0 + 32 + lane, bt_width - 1));
        }
        const bool active = wanted(key0);
        const int pi = page_index(key0);
        const int rel = pi - p0;                       // 0 .. 63
        const int from_cur = __shfl_sync(0xffffffffu, cur, rel & 31), from_nxt = __shfl_sync(0xffffffffu, nxt, rel & 31);
        const int page = rel < 32 ? from_cur : from_nxt;
        const int row = (page * nkv + kvh) * page_size + (key0 - pi * page_size);
        const int nb = __popc(__ballot_sync(0xffffffffu, active));
        int go = 1;
        if (lane == 0) {
          if (!mbar_wait_bounded(smem_addr(&empty[st]), par ^ 1, aborted)) {
            abort_flag = 1;
            go = 0;
          } else {
            mbar_expect_tx(smem_addr(&full[st]), (uint32_t)nb * BOX);
          }
        }
        go = __shfl_sync(0xffffffffu, go, 0);
        if (!go) {
          ok = false;
          break;
        }
        if (active) tma_load_3d(ring_addr + (uint32_t)st * STAGE + dst_off, map, 0, row, 0, smem_addr(&full[st]));
        ++issued;
        key0 += kTile;
        if (++st == stages) st = 0, par ^= 1;
      }
      u = pe;
    }
    // No copy may still be in flight when the CTA ends.  The consumers have waited for every tile
    // unless a wait ran out, so this is free otherwise.
    if (lane == 0) {
      for (int s = 0; s < stages && s < issued; ++s) {
        const int last = (issued - 1 - s) / stages * stages + s;       // last tile issued into stage s
        mbar_wait_plain(smem_addr(&full[s]), (uint32_t)((last / stages) & 1));
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    const int grp = warp >> 2, wk = warp & 3;
    const int g = lane >> 2, tq = lane & 3;
    const uint32_t sw = (uint32_t)(lane & 7);
    int st = 0, n = 0;
    uint32_t par = 0;
    for (int u = u0; u < u1;) {
      const int r = rows.row_of(u);
      int lo, kv_len, tlo, thi;
      rows.tiles_of(r, lo, kv_len, tlo, thi);
      const int T = thi - tlo;
      const int rem = u - prefix[r];
      const int kvh = rem / T;
      const int tile0 = tlo + rem % T;
      const int pair_begin = prefix[r] + kvh * T;
      const int pe = min(pair_begin + T, u1);
      const int ntile = pe - u;
      const int t = tok[r];

      // the G query heads of this kv head as the A operand: rows 0..G-1 of 16, the rest zero
      uint32_t qa[HD / 16][4];
      const bool has_last = prep.on && pair_begin + T <= u1;      // this piece holds the pair's last tile, hence the new key
      if (prep.on) {
        // heads 0..G-1: the pair's queries; G: the new key; G + 1: the new value (copied).  A warp a head.
        const __nv_bfloat16* row = q + (size_t)t * q_row_stride;
        const float pos = (float)(kv_len - 1);
        for (int hh = warp; hh < G + (has_last ? 2 : 0); hh += kConsumerWarps) {
          if (hh < G)
            prep_head<HD>(row + (size_t)(kvh * G + hh) * HD, prep.q_weight, prep.eps, prep.inv_freq, pos, lane, heads + hh * HD);
          else if (hh == G)
            prep_head<HD>(row + (size_t)(nq + kvh) * HD, prep.k_weight, prep.eps, prep.inv_freq, pos, lane, heads + 16 * HD);
          else
            prep_head<HD>(row + (size_t)(nq + nkv + kvh) * HD, nullptr, 0.f, nullptr, 0.f, lane, heads + 17 * HD);
        }
        consumer_sync();
      }
      {
        const uint32_t* q0 = prep.on ? reinterpret_cast<const uint32_t*>(heads + (size_t)g * HD) + tq
                                     : reinterpret_cast<const uint32_t*>(q + (size_t)t * q_row_stride + (size_t)(kvh * G + g) * HD) + tq;
        const uint32_t* q1 = q0 + 8 * HD / 2;
#pragma unroll
        for (int s = 0; s < HD / 16; ++s) {
          qa[s][0] = g < G ? q0[s * 8] : 0u;
          qa[s][1] = g + 8 < G ? q1[s * 8] : 0u;
          qa[s][2] = g < G ? q0[s * 8 + 4] : 0u;
          qa[s][3] = g + 8 < G ? q1[s * 8 + 4] : 0u;
        }
      }
      float o[HD / 8][4];
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
      float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows g and g+8

      for (int i = 0; i < ntile; ++i, ++n) {
        const int my_st = st;
        const uint32_t my_par = par;
        if (++st == stages) st = 0, par ^= 1;
        if ((n & 1) != grp) continue;
        if (!mbar_wait_bounded(smem_addr(&full[my_st]), my_par, aborted)) abort_flag = 1;
        const int kbeg = (tile0 + i) * kTile + wk * 16;        // this warp's 16 keys
        if (kbeg < kv_len && kbeg + 16 > lo) {
          const uint32_t kt = ring_addr + (uint32_t)my_st * STAGE + (uint32_t)wk * BOX;
          const uint32_t vt = kt + OPERAND;
          if (has_last && kbeg + 16 >= kv_len) {
            // The new token's key and value: over the stale slot of this warp's block (lanes 0-15 the key's
            // 16-byte pieces, lanes 16-31 the value's) and into the cache for the steps to come.
            const int rr = (kv_len - 1) - kbeg;                // row of the block
            const int j = lane & 15;
            if (j < HD / 8) {
              const uint4 val = *reinterpret_cast<const uint4*>(heads + (lane < 16 ? 16 : 17) * HD + j * 8);
              const uint32_t at = (lane < 16 ? kt : vt) + (uint32_t)(j >> 3) * (16 * 128) + (uint32_t)rr * 128 +
                                  (uint32_t)(((j & 7) ^ (rr & 7)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(at), "r"(val.x), "r"(val.y), "r"(val.z), "r"(val.w)
                           : "memory");
              const int slot = prep.slot_mapping[t];
              if (slot >= 0) {
                const int page = slot / page_size, off = slot - page * page_size;
                __nv_bfloat16* cache = lane < 16 ? prep.k_cache : prep.v_cache;
                *reinterpret_cast<uint4*>(cache + (((size_t)page * nkv + kvh) * page_size + off) * HD + j * 8) = val;
              }
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");    // before a later copy writes the stage again
            __syncwarp();
          }
          // two accumulator sets, one for the even and one for the odd 16-element steps of the
          // head: half as long a chain of dependent tensor-core instructions
          float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
          float s2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            const uint32_t j = (uint32_t)(kk * 2 + ((lane >> 3) & 1));
            uint32_t b0, b1, b2, b3;
            ldsm_x4(kt + (j >> 3) * (16 * 128) + (uint32_t)((lane >> 4) * 8 + (lane & 7)) * 128 + (((j & 7) ^ sw) << 4), b0, b1,
                    b2, b3);
            if (kk & 1) {
              mma_bf16(s2[0], qa[kk], b0, b1);
              mma_bf16(s2[1], qa[kk], b2, b3);
            } else {
              mma_bf16(s[0], qa[kk], b0, b1);
              mma_bf16(s[1], qa[kk], b2, b3);
            }
          }
#pragma unroll
          for (int nn = 0; nn < 2; ++nn)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nn][e] += s2[nn][e];
          float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
          for (int nn = 0; nn < 2; ++nn) {
            const int kj = kbeg + 8 * nn + 2 * tq;
            const bool in0 = kj < kv_len && kj >= lo, in1 = kj + 1 < kv_len && kj + 1 >= lo;
            s[nn][0] = in0 ? s[nn][0] * scale_log2 : -INFINITY;
            s[nn][1] = in1 ? s[nn][1] * scale_log2 : -INFINITY;
            s[nn][2] = in0 ? s[nn][2] * scale_log2 : -INFINITY;
            s[nn][3] = in1 ? s[nn][3] * scale_log2 : -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(s[nn][0], s[nn][1]));
            mx1 = fmaxf(mx1, fmaxf(s[nn][2], s[nn][3]));
          }
          mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
          mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
          mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
          mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
          const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);   // finite: the block has a key in range
          const float c0 = exp2f(m0 - mn0), c1 = exp2f(m1 - mn1);
          m0 = mn0;
          m1 = mn1;
          float p[2][4];
#pragma unroll
          for (int nn = 0; nn < 2; ++nn) {
            p[nn][0] = exp2f(s[nn][0] - mn0);
            p[nn][1] = exp2f(s[nn][1] - mn0);
            p[nn][2] = exp2f(s[nn][2] - mn1);
            p[nn][3] = exp2f(s[nn][3] - mn1);
          }
          l0 = l0 * c0 + p[0][0] + p[0][1] + p[1][0] + p[1][1];
          l1 = l1 * c1 + p[0][2] + p[0][3] + p[1][2] + p[1][3];
          uint32_t pa[4];
          pa[0] = pack_bf16(p[0][0], p[0][1]);
          pa[1] = pack_bf16(p[0][2], p[0][3]);
          pa[2] = pack_bf16(p[1][0], p[1][1]);
          pa[3] = pack_bf16(p[1][2], p[1][3]);
          // the accumulator is rescaled only when some row's maximum grew (a factor of exactly 1 otherwise)
          const bool rescale = __any_sync(0xffffffffu, c0 != 1.0f || c1 != 1.0f);
          if (rescale) {
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
              o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1;
            }
          }
#pragma unroll
          for (int dn = 0; dn < HD / 16; ++dn) {
            const uint32_t j = (uint32_t)(dn * 2 + (lane >> 4));
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(vt + (j >> 3) * (16 * 128) + (uint32_t)(((lane >> 3) & 1) * 8 + (lane & 7)) * 128 + (((j & 7) ^ sw) << 4),
                      b0, b1, b2, b3);
            mma_bf16(o[2 * dn], pa, b0, b1);
            mma_bf16(o[2 * dn + 1], pa, b2, b3);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive_one(smem_addr(&empty[my_st]));
      }

      // ---- merge the eight warps' partial results of this piece
      l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
      l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
      l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
      l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        if (g < G) *reinterpret_cast<float2*>(mo + (warp * G + g) * HD + i * 8 + 2 * tq) = make_float2(o[i][0], o[i][1]);
        if (g + 8 < G) *reinterpret_cast<float2*>(mo + (warp * G + g + 8) * HD + i * 8 + 2 * tq) = make_float2(o[i][2], o[i][3]);
      }
      if (tq == 0) {
        mm[warp * 16 + g] = m0;
        mm[warp * 16 + g + 8] = m1;
        mlv[warp * 16 + g] = l0;
        mlv[warp * 16 + g + 8] = l1;
      }
      consumer_sync();
      const int pidx = r * nkv + kvh;
      // pieces of a pair lie side by side in the scratch: from slot first_cta + pidx when the units are shared
      // out evenly (a CTA index alone would repeat where a CTA holds pieces of two pairs), from the pair's first
      // CTA when they are shared out by pair
      int first_cta, pieces, slot;
      if (by_pair) {
        const int tp = (T + own_k - 1) / own_k;
        first_cta = own_first + kvh * own_k;                  // the pair's first CTA; a piece's slot is its CTA
        pieces = (T + tp - 1) / tp;                           // pieces that have tiles
        slot = (int)blockIdx.x;
      } else {
        first_cta = pair_begin / per + pidx;
        pieces = (pair_begin + T - 1) / per - pair_begin / per + 1;
        slot = (int)blockIdx.x + pidx;
      }
      for (int i = tid; i < G * HD; i += kConsumers) {
        const int row = i / HD, d = i % HD;
        float M = mm[row];
#pragma unroll
        for (int w = 1; w < kConsumerWarps; ++w) M = fmaxf(M, mm[w * 16 + row]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) {
          const float f = exp2f(mm[w * 16 + row] - M);        // a warp without keys has m = -inf: factor 0
          L += mlv[w * 16 + row] * f;
          O += mo[(w * G + row) * HD + d] * f;
        }
        if (pieces == 1) {
          out[((size_t)t * nq + kvh * G + row) * HD + d] = __float2bfloat16_rn(O / L);
        } else {
          part_o[((size_t)slot * G + row) * HD + d] = O;
          if (d == 0) {
            part_ml[((size_t)slot * G + row) * 2] = M;
            part_ml[((size_t)slot * G + row) * 2 + 1] = L;
          }
        }
      }
      if (pieces > 1) {
        // The piece that arrives last combines all of them:
        //   out = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M),  M = max_s m_s,
        // accumulated piece by piece in the order of the keys.
        __threadfence();
        consumer_sync();
        if (tid == 0) {
          const int prev = atomicAdd(&counters[pidx], 1);
          is_last = prev == pieces - 1;
          if (is_last) counters[pidx] = 0;                    // ready for the next launch
        }
        consumer_sync();
        if (is_last) {
          __threadfence();
          const size_t base = (size_t)first_cta * G;
          for (int i = tid; i < G * HD / 2; i += kConsumers) {
            const int row = i / (HD / 2), d = (i % (HD / 2)) * 2;
            const float2* po = reinterpret_cast<const float2*>(part_o + (base + row) * HD + d);
            const float2* pml = reinterpret_cast<const float2*>(part_ml) + base + row;
            float M = -INFINITY, L = 0.f, O0 = 0.f, O1 = 0.f;
            for (int sp0 = 0; sp0 < pieces; sp0 += 8) {        // eight pieces' loads in flight together
              float2 ml[8], ov[8];
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const int sp = min(sp0 + k, pieces - 1);
                ml[k] = __ldcg(pml + (size_t)sp * G);
                ov[k] = __ldcg(po + (size_t)sp * G * HD / 2);
              }
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                if (sp0 + k < pieces && ml[k].y > 0.f) {
                  const float Mn = fmaxf(M, ml[k].x);
                  const float c = exp2f(M - Mn), f = exp2f(ml[k].x - Mn);
                  L = L * c + ml[k].y * f;
                  O0 = O0 * c + ov[k].x * f;
                  O1 = O1 * c + ov[k].y * f;
                  M = Mn;
                }
              }
            }
            const float inv = 1.0f / L;
            *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)t * nq + kvh * G + row) * HD + d) = __floats2bfloat162_rn(O0 * inv, O1 * inv);
          }
        }
      }
      consumer_sync();                                        // the scratch is free for the next piece
      u = pe;
    }
  }
  if (*aborted && lane == 0 && err) atomicExch(err, 4);
}

size_t fixed_smem(int G, int hd, int ctas, int R) {
  size_t n = (size_t)kConsumerWarps * G * hd * 4 + (size_t)kConsumerWarps * 16 * 2 * 4;
  n += (size_t)((3 * R + 1 + 3) & ~3) * 4;
  n += (size_t)18 * hd * 2;                                  // prepared query heads, new key, new value
  return (n + 15) / 16 * 16;
}

template <int HD>
int launch_stream(const CUtensorMap& mk, const CUtensorMap& mv, const void* q, int q_row_stride, void* out,
                  const int* q_indptr, const int* kv_lens, const int* block_table, int bt_stride, float* part_o,
                  float* part_ml, int* counters, int rows, int nq, int nkv, int bt_width, int page_size, float scale, int window,
                  int ctas, const Prep& prep, const int* plan, int* err, cudaStream_t s) {
  int ps_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (ps_shift = 0; (1 << ps_shift) < page_size; ++ps_shift) {}
  int dev = 0, max_smem = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  const size_t stage = (size_t)2 * kTile * HD * 2;
  const size_t fixed = fixed_smem(nq / nkv, HD, ctas, rows) + 1024 + kStaticSmem;      // alignment slack, static shared memory
  if (fixed + 2 * stage > (size_t)max_smem) return ARLE_E_UNSUPPORTED;
  // The ring's depth is even.  The two consumer groups take alternate tiles, so with an even depth a
  // stage always serves the same group, whose waits on it alternate in parity.  With an odd depth a
  // stage serves the groups in turn and each group waits on it with the same parity every time: a
  // group that comes back to a stage while the other group's load into it has not landed yet (copies
  // issued later may land earlier) would find the phase of its parity complete, read the stage as it
  // is and release it a phase early, and from there on copies overwrite stages in use and may still
  // be in flight when the CTA ends.
  int stages = (int)(((size_t)max_smem - fixed) / stage);
  if (stages > kMaxStages) stages = kMaxStages;
  stages &= ~1;
  const size_t smem = fixed - kStaticSmem + (size_t)stages * stage;
  e = cudaFuncSetAttribute(decode_stream_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem - kStaticSmem);
  if (e != cudaSuccess) return (int)e;
  e = launch_kernel(decode_stream_kernel<HD>, dim3(ctas), dim3(kThreads), smem, s, 1, mk, mv, (const __nv_bfloat16*)q,
                    q_row_stride, (__nv_bfloat16*)out, q_indptr, kv_lens, block_table, bt_stride, part_o, part_ml, counters,
                    rows, nq, nkv, bt_width, page_size, ps_shift, scale * 1.4426950408889634f, window, stages, prep, plan, err);
  if (e != cudaSuccess) return (int)e;
  return launch_status();
}

}  // namespace

ARLE_API int arle_paged_attention_decode_stream_prep(const void* q, int q_row_stride, void* out, const void* k_cache,
                                                     const void* v_cache, long long cache_pages, const int* q_indptr,
                                                     const int* kv_lens, const int* block_table, int bt_stride, int bt_width,
                                                     float* part_o, float* part_ml, int* counters, int nq, int nkv, int hd,
                                                     int page_size, float scale, int window, int rows, int ctas, int fused,
                                                     const int* slot_mapping, const float* q_weight, const float* k_weight,
                                                     float eps, const float* inv_freq, const int* plan, int* err, cudaStream_t s);

// k_cache / v_cache: [cache_pages, nkv, page_size, hd].  Scratch: part_o float32
// [(ctas + rows * nkv) * (nq / nkv) * hd], part_ml float32 [(ctas + rows * nkv) * (nq / nkv) * 2], counters
// int32 [rows * nkv] that must be zero before the first launch (the kernel leaves them zero).
// ctas: CTAs of the grid (the number of SMs).  bt_width: columns of the block table, which bound
// a row's keys.  err: set to 4 if a bounded wait ran out.
ARLE_API int arle_paged_attention_decode_stream(const void* q, int q_row_stride, void* out, const void* k_cache,
                                                const void* v_cache, long long cache_pages, const int* q_indptr,
                                                const int* kv_lens, const int* block_table, int bt_stride, int bt_width,
                                                float* part_o, float* part_ml, int* counters, int nq, int nkv, int hd,
                                                int page_size, float scale, int window, int rows, int ctas, int* err,
                                                cudaStream_t s) {
  return arle_paged_attention_decode_stream_prep(q, q_row_stride, out, k_cache, v_cache, cache_pages, q_indptr, kv_lens,
                                                 block_table, bt_stride, bt_width, part_o, part_ml, counters, nq, nkv, hd,
                                                 page_size, scale, window, rows, ctas, 0, nullptr, nullptr, nullptr, 0.f, nullptr,
                                                 nullptr, err, s);
}

// Ints of a step's plan for this many rows and CTAs.
ARLE_API int arle_decode_stream_plan_ints(int rows, int ctas) { return kPlanHeader + (3 + 32) * ctas + 3 * rows + 1; }

// Fills a step's plan (arle_decode_stream_plan_ints(rows, ctas) ints): launches of the streaming kernel with the same
// q_indptr, kv_lens, block table, page size, rows, nkv, window and ctas that are given it skip their own working out of
// the shares and their first read of the block table.
ARLE_API int arle_decode_stream_plan(const int* q_indptr, const int* kv_lens, const int* block_table, int bt_stride, int bt_width,
                                     int page_size, int rows, int nkv, int window, int ctas, int* plan, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (rows > 2048 || ctas < 1 || ctas > 1024 || nkv <= 0 || page_size <= 0 || bt_width < 1 || !plan || !block_table) return ARLE_E_BADARG;
  launch_kernel(decode_stream_plan_kernel, dim3(ctas), dim3(kThreads), (size_t)(3 * rows + 1) * sizeof(int), s, 1, q_indptr, kv_lens,
                block_table, bt_stride, bt_width, page_size, rows, nkv, window, plan);
  return launch_status();
}

// The same with the fused preparation (fused != 0): q is the raw projection output of the step's tokens
// ([q heads | k heads | v heads] per row, stride q_row_stride), every row a decoded token at position
// kv_len - 1; q_weight / k_weight (float32 [hd], may be null: no norm), inv_freq (float32 [hd / 2], may be null: no
// rotation; otherwise the whole head is rotated), slot_mapping int32 [tokens].  The new keys and values are
// stored into the cache by this launch.
ARLE_API int arle_paged_attention_decode_stream_prep(const void* q, int q_row_stride, void* out, const void* k_cache,
                                                     const void* v_cache, long long cache_pages, const int* q_indptr,
                                                     const int* kv_lens, const int* block_table, int bt_stride, int bt_width,
                                                     float* part_o, float* part_ml, int* counters, int nq, int nkv, int hd,
                                                     int page_size, float scale, int window, int rows, int ctas, int fused,
                                                     const int* slot_mapping, const float* q_weight, const float* k_weight,
                                                     float eps, const float* inv_freq, const int* plan, int* err, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (fused && (!slot_mapping || ((uintptr_t)q & 15) || (q_row_stride % 8) != 0)) return ARLE_E_BADARG;
  const Prep prep{fused ? 1 : 0, slot_mapping, q_weight, k_weight, eps, inv_freq, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache};
  if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || nq / nkv > 16 || page_size <= 0 || page_size % 16 != 0) return ARLE_E_UNSUPPORTED;
  if (ctas < 1 || ctas > 1024 || rows > 2048 || !part_o || !part_ml || !counters) return ARLE_E_BADARG;
  if ((q_row_stride % 2) != 0 || ((uintptr_t)q & 3) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15)) return ARLE_E_UNSUPPORTED;
  // units are counted in 32 bits
  const long long max_units = (long long)rows * nkv * (((long long)bt_width * page_size + kTile - 1) / kTile + 1);
  if (max_units >= (1ll << 30)) return ARLE_E_UNSUPPORTED;
  if (hd != 64 && hd != 128) return ARLE_E_UNSUPPORTED;
  CUtensorMap mk, mv;
  const long long cache_rows = cache_pages * nkv * page_size;
  int rc = tensor_map_rows_bf16(k_cache, cache_rows, hd, &mk);
  if (rc) return rc;
  rc = tensor_map_rows_bf16(v_cache, cache_rows, hd, &mv);
  if (rc) return rc;
  if (hd == 128)
    return launch_stream<128>(mk, mv, q, q_row_stride, out, q_indptr, kv_lens, block_table, bt_stride, part_o, part_ml, counters,
                              rows, nq, nkv, bt_width, page_size, scale, window, ctas, prep, plan, err, s);
  return launch_stream<64>(mk, mv, q, q_row_stride, out, q_indptr, kv_lens, block_table, bt_stride, part_o, part_ml, counters,
                           rows, nq, nkv, bt_width, page_size, scale, window, ctas, prep, plan, err, s);
}
