// tcgen05 / TMEM / TMA kernels (sm_100a) of the attention-with-scores family.
//
// Forward kernel: one CTA = 256 query rows (two tiles of 128) of one (batch, query
// head); key tiles of 128 shared by both query tiles.  Warp roles (12 warps):
//   warp 0       TMA producer: both Q tiles once, then K and V tiles through one 3-slot ring
//   warp 1       allocates TMEM; one lane issues the tcgen05 MMAs.  Per query tile t:
//                S_t = Q_t.K^T (fp32, TMEM) and O_t += P_t.V (fp32, TMEM; P_t is read
//                from TMEM, where it overwrites S_t).  The two query tiles alternate, so
//                the tensor pipe works on one while the other is in its softmax.
//   warps 2,3    idle (they only give their registers to the softmax warps)
//   warps 4..7   softmax of query tile 0; warps 8..11 softmax of query tile 1.
//                Thread r owns query row r (TMEM lane r): it reads the row's 128 scores
//                once, keeps them in registers for the running max and for exp2, rescales
//                O in TMEM only when the running max moved by more than 2^8, and writes P
//                back to TMEM as 16-bit pairs.
// Score-tile hooks (what attention_with_scores.py:141-162, attention_with_row_sum.py:146-156,
// attention_with_col_sum.py:170-191 add to the FlashAttention loop):
//   scores      fp32 tile staged per warp (32x32, swizzled) and written with TMA stores;
//               key tiles the causal loop never visits are filled from one constant tile
//   row sum     per-thread running sum
//   column sum  per-warp transpose-reduce with shuffles, 4 warps combined through smem,
//               one partial row per 128-row query tile (summed later in fixed order)
//   scratch     the cross region's scores (buffered cross-token variant) via TMA stores
//
// Every mbarrier wait is bounded (about 2 s); on give-up the CTA raises a flag in
// *status, lets in-flight copies drain, frees its TMEM and returns.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <mutex>
#include <queue>
#include <vector>
#include <type_traits>

#include "faws_internal.cuh"
#include "faws_tc_host.cuh"
#include "faws_tc_ptx.cuh"

namespace faws {
namespace {
using namespace ptx;

constexpr int BM = kTcBlockM;   // rows of one query tile
constexpr int BN = kTcBlockN;
constexpr int NTHREADS = 384;
constexpr int MAX_KV_SLOTS = 4;
constexpr int TMEM_COLS = 512;
// setmaxnreg budget: the CTA is launched with 168 registers per thread (384 threads, one
// CTA per SM); after re-allocation the total must not exceed that pool, otherwise the
// .inc never returns.  88 / 208: with fewer registers for the producer and MMA warps their loops
// spill (at 56 / 224 the score-materialising launch measured 5 % slower, the others 2-3 %); 104 / 200 and
// 120 / 192 measured the same as 88 / 208.
constexpr int REGS_LAUNCH = 168;
constexpr int REGS_AUX = 88;
constexpr int REGS_SOFTMAX = ((REGS_LAUNCH * NTHREADS - 128 * REGS_AUX) / 256) & ~7;
static_assert(128 * REGS_AUX + 256 * REGS_SOFTMAX <= REGS_LAUNCH * NTHREADS, "setmaxnreg would block");
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
#define FAWS_NEG_INF (__int_as_float(0xff800000))

struct TcMaps {
  CUtensorMap q, k, v, o;  // o: 32-row store boxes of the output
  CUtensorMap st;          // scores (or score-scratch) store map
};

// SPLIT = false: the CTA owns two query tiles (256 rows), one per softmax warpgroup.
// SPLIT = true : the CTA owns one query tile (128 rows) and the two warpgroups take alternate
//                key tiles of it (their partial O, m, l are merged at the end), which halves
//                the longest dependent chain; used when a launch has few CTAs.
template <int D, bool SPLIT>
struct Smem {
  static constexpr int kTile = 128 * D * 2;  // one Q / K / V tile
  static constexpr int kSub = 128 * 128;     // one 64-element-wide sub-tile: 128 rows x 128 B
  static constexpr int kQTiles = SPLIT ? 1 : 2;
  static constexpr int kSlots = SPLIT ? 4 : 3;
  static constexpr int kRows = kQTiles * 128;
  static constexpr int q_off = 0;                             // query tile(s)
  static constexpr int kv_off = q_off + kQTiles * kTile;      // K/V ring
  static constexpr int stage_off = kv_off + kSlots * kTile;   // 8 warps x 2 x 4 KB
  static constexpr int bar_off = stage_off + 8 * 2 * 4096;
  static constexpr int total = bar_off + 256;
  static constexpr int alloc = total + 1024;  // slack to align the base to 1024 B
};

struct Bars {
  uint64_t q_full;
  uint64_t q_empty;       // persistent CTAs: the item's last Q.K^T has completed, the next item's Q tiles may land
  uint64_t kv_full[MAX_KV_SLOTS], kv_empty[MAX_KV_SLOTS];
  uint64_t s_full[2];     // per query tile: S_t written by the tensor pipe
  uint64_t p_half[2];     // per query tile: the first 64 columns of P_t are in TMEM
  uint64_t p_ready[2];    // per query tile: P_t written by its 128 softmax threads
  uint64_t col_ready[2];  // per query tile: column-sum partial rows of its 4 warps are in smem
  uint64_t o_done;        // every MMA of the CTA has completed
  uint64_t merge_ready;   // SPLIT: warpgroup 1 has published its (m, l, row sum)
  uint32_t tmem_base;
  int abort_flag;
};

template <typename T> __device__ __forceinline__ float2 unpack2(uint32_t w);
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t w) {
  return __half22float2(*reinterpret_cast<__half2*>(&w));
}
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t w) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w));
}
template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <typename T> __device__ __forceinline__ uint32_t pack_bits(T lo, T hi) {
  return (uint32_t)(*reinterpret_cast<const uint16_t*>(&lo)) | ((uint32_t)(*reinterpret_cast<const uint16_t*>(&hi)) << 16);
}

// In-warp transpose-reduce: on entry lane L holds v[0..31] (its row, 32 columns); on exit
// v[0] of lane c is the sum over the 32 lanes of their v[c].  31 shuffles.
__device__ __forceinline__ void warp_column_sums(float (&v)[32], int lane) {
#pragma unroll
  for (int step = 16; step >= 1; step >>= 1) {
    const bool upper = (lane & step) != 0;
#pragma unroll
    for (int x = 0; x < step; ++x) {
      const float send = upper ? v[x] : v[x + step];
      const float keep = upper ? v[x + step] : v[x];
      v[x] = keep + __shfl_xor_sync(0xffffffffu, send, step);
    }
  }
}

// Score-tile hook compiled into a kernel instance (one per operator family).
enum Hook : int {
  kHookNone = 0, kHookScores = 1, kHookRowSum = 2, kHookColPart = 3, kHookScratch = 4,
  kHookScores16 = 5  // scores in the input dtype (what the reference kernel writes)
};

// Persistent launches: one CTA per SM walks a list of work items (an item is what one CTA of the
// plain launch does: a row block of one head), in the order of the plain launch's grid.  The
// lists are made on the host (longest item first onto the least loaded CTA) and travel as a
// kernel parameter, so that no device-side counter is shared between launches; launches with
// more items than the lists hold deal the items to the CTAs in rounds of alternating direction.
constexpr int kMaxListedItems = 2048;
constexpr int kMaxListCtas = 192;
struct WorkList {
  int n_items;  // 0: plain launch, every CTA does the item its block index names
  int listed;   // 1: CTA c does ids[start[c]] .. ids[start[c + 1] - 1]
  int gx, gy, gz;  // the grid of the plain launch; an item is a linear block index of it (x fastest)
  uint16_t start[kMaxListCtas + 1];
  uint16_t ids[kMaxListedItems];
};

template <typename T, int D, int HOOK, bool SPLIT, bool DROP = false>
__global__ void __launch_bounds__(NTHREADS, 1)
tc_fwd_kernel(const __grid_constant__ TcMaps maps, const FwdParams p, const __grid_constant__ WorkList wl,
              int* __restrict__ status) {
  using L = Smem<D, SPLIT>;
  constexpr int KV_SLOTS = L::kSlots;
  constexpr int CTA_ROWS = L::kRows;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  Bars* bars = reinterpret_cast<Bars*>(smem + L::bar_off);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Launch order.  Default: row blocks fastest, so the CTAs of a head run together and share its
  // K/V through L2.  lpt_order (causal, K/V small enough to stay in L2 anyway): row blocks
  // slowest, so the heaviest row blocks of every head are dispatched first (longest-processing-
  // time-first packing of the causal triangle onto the SMs).
  // fill_ctas (score hooks, causal): the row-block axis holds two CTAs per row block, a compute
  // CTA and a fill CTA that only writes the row block's never-visited key tiles.  All compute
  // CTAs come first in launch order (heaviest first), the fill CTAs after them (most-masked row
  // block first): measured against interleaving the two kinds, cfg2 runs 2 % faster.
  // The geometry of the work item in hand.  Plain launches have one item per CTA, named by the block
  // index; persistent CTAs (never SPLIT, split-KV or fill launches) set it again for every item.
  constexpr bool kStoreHook = HOOK == kHookScores || HOOK == kHookScores16 || HOOK == kHookScratch;
  const bool persist = !SPLIT && !kStoreHook && wl.n_items > 0;  // (the launcher keeps the other instances plain)
  bool is_fill;
  int cb_rel, h, b, ksplit, kt0, hk, bh, ho, cb_abs, nt, rr_start;
  int r_tile_of[2];  // first row of the item's query tile(s)
  int nt_q[2];       // end of the key-tile range each query tile visits (kt0 for a tile outside the row window)
  auto set_item = [&](int ix, int iy, int iz, int gx, int gz) {
    const int slot = p.lpt_order ? iz : ix;
    const int ncb = (p.lpt_order ? gz : gx) >> (p.fill_ctas ? 1 : 0);
    is_fill = p.fill_ctas && slot >= ncb;
    cb_rel = is_fill ? slot - ncb : ncb - 1 - slot;  // compute: heaviest (last) blocks first
    h = p.lpt_order ? ix : iy;
    // Split-KV launches (n_splits > 1) fold the key-range index into the batch axis of the grid.
    const int bz = p.lpt_order ? iy : iz;
    b = bz / p.n_splits;
    ksplit = bz - b * p.n_splits;
    kt0 = ksplit * p.tiles_per_split;  // the item visits key tiles [kt0, kt0 + tiles_per_split)
    hk = h / p.G;
    bh = b * p.Hq + h;
    ho = h * p.n_splits + ksplit;  // head index of the (partial) output the item writes
    r_tile_of[0] = p.m_begin + cb_rel * CTA_ROWS;
    r_tile_of[1] = r_tile_of[0] + (SPLIT ? 0 : BM);
    cb_abs = r_tile_of[0] / CTA_ROWS;  // start offset of the round-robin key-tile order
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int r0 = r_tile_of[t];
      int hi = 0;
      if (r0 < p.m_end) {
        hi = p.N;
        if (p.causal) hi = max(0, min(p.N, p.p_seq + min(r0 + BM, p.m_end)));
      }
      nt_q[t] = min(max((hi + BN - 1) / BN, kt0), kt0 + p.tiles_per_split);
    }
    nt = max(nt_q[0], nt_q[1]) - kt0;  // key tiles the item visits
    rr_start = p.causal ? nt - 1 : cb_abs % max(nt, 1);
  };
  // k-th item of this CTA, or -1 when it has no more
  auto item_at = [&](int k) -> int {
    if (wl.listed) {
      const int at = (int)wl.start[blockIdx.x] + k;
      return at < (int)wl.start[blockIdx.x + 1] ? (int)wl.ids[at] : -1;
    }
    const int G = (int)gridDim.x;
    const int idx = k * G + ((k & 1) ? G - 1 - (int)blockIdx.x : (int)blockIdx.x);
    return idx < wl.n_items ? idx : -1;
  };
  // moves on to the CTA's k-th item; false when there is none
  auto goto_item = [&](int k) -> bool {
    if (!persist) return false;  // (the first item of a plain launch is set below)
    const int item = item_at(k);
    if (item < 0) return false;
    const int ix = item % wl.gx, rest = item / wl.gx;
    set_item(ix, rest % wl.gy, rest / wl.gy, wl.gx, wl.gz);
    return true;
  };
  if (persist) {
    if (!goto_item(0)) return;  // (a CTA without work: nothing has been set up yet)
  } else set_item((int)blockIdx.x, (int)blockIdx.y, (int)blockIdx.z, (int)gridDim.x, (int)gridDim.z);

  if constexpr (HOOK == kHookScores || HOOK == kHookScores16) {
    if (is_fill) {
      // Fill CTA: no barriers, no TMEM.  Every warp owns a constant 32-row x 128-byte tile and
      // stores it over its share of the (32-row group, 128-byte column chunk) units.
      constexpr int kCols = HOOK == kHookScores ? 32 : 64;  // elements per 128-byte chunk
      unsigned char* tile = smem + warp * 4096;
      const float masked_f = __uint_as_float(p.masked_bits);
      uint32_t word = p.masked_bits;
      if (HOOK == kHookScores16) {
        const T mt = from_float<T>(masked_f);
        word = pack_bits<T>(mt, mt);
      }
      const uint4 fill = make_uint4(word, word, word, word);
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) *reinterpret_cast<uint4*>(tile + lane * 128 + (cc << 4)) = fill;
      fence_proxy_async_smem();
      griddep_wait();  // the previous kernel of the stream may still be reading or writing the scores
      griddep_launch_dependents();
      __syncwarp();
      if (lane == 0) {
        constexpr int kGroups = CTA_ROWS / 32;
        int unit = 0;  // (row group, column chunk) units are dealt round-robin to the 12 warps
        for (int rg = 0; rg < kGroups; ++rg) {
          const int t = SPLIT ? 0 : rg / 4;
          const int r0 = r_tile_of[t] + (rg & 3) * 32;
          if (r0 >= p.m_end) continue;
          for (int j0 = nt_q[t] * BN; j0 < p.N; j0 += kCols, ++unit) {
            if (unit % 12 == warp) tma_store_3d(&maps.st, tile, j0, r0 - p.m_begin, bh);
          }
        }
        tma_store_commit();
        tma_store_wait<0>();
      }
      return;
    }
  }

  // Round-robin: the key tiles in cyclic order from a start tile that differs from CTA to CTA
  // (attention_with_col_sum_sequential.py:116-122), walked downwards.  Causal CTAs start at their last key
  // tile, the one only the second query tile visits, so that this lone step overlaps the CTA's set-up
  // instead of stalling the two-tile pipeline in mid-loop (a start in mid-range measured 10 % slower on
  // cfg3, an upward walk 5 %); the causal round-robin walk is then the reverse order itself.
  auto tile_of = [&](int it) -> int {
    if (p.schedule == kReverse) return kt0 + nt - 1 - it;
    if (p.schedule == kRoundRobin) return kt0 + (rr_start - it + nt) % nt;
    return kt0 + it;
  };
  // K(0), V(0), K(1), V(1), ... go through the ring in this order
  // (idx counts within the item, ring_idx over all items of the CTA)
  auto issue_kv_load = [&](int idx, int ring_idx) {
    const int s = ring_idx % KV_SLOTS;
    const int n0 = tile_of(idx >> 1) * BN;
    mbar_arrive_expect_tx(&bars->kv_full[s], L::kTile);
    const CUtensorMap* map = (idx & 1) ? &maps.v : &maps.k;
    for (int c = 0; c < D / 64; ++c)
      tma_load_4d(smem + L::kv_off + s * L::kTile + c * L::kSub, map, &bars->kv_full[s], c * 64, n0, hk, b);
  };
  const int n_early = min(KV_SLOTS, 2 * nt);  // loads issued before the CTA-wide set-up barrier

  if (threadIdx.x == 64) {
    // Descriptor fetches off the critical path: the load maps while thread 0 initialises the
    // barriers, the store maps long before the epilogue (the CTA cannot exit before its stores).
    prefetch_tmap(&maps.q);
    prefetch_tmap(&maps.k);
    prefetch_tmap(&maps.v);
    prefetch_tmap(&maps.o);
    if constexpr (HOOK == kHookScores || HOOK == kHookScores16 || HOOK == kHookScratch) prefetch_tmap(&maps.st);
  }
  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    mbar_init(&bars->q_empty, HOOK == kHookColPart ? 3 : 1);  // the MMA warp (+ the two warps that sum the Q rows)
    for (int s = 0; s < KV_SLOTS; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->kv_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&bars->s_full[t], 1);
      mbar_init(&bars->p_half[t], 128);
      mbar_init(&bars->p_ready[t], 128);
      mbar_init(&bars->col_ready[t], 128);
    }
    mbar_init(&bars->o_done, 1);
    mbar_init(&bars->merge_ready, 128);
    bars->abort_flag = 0;
    mbar_fence_init();
    // This thread is also the TMA producer: start the first loads now so that their HBM
    // latency overlaps the TMEM allocation and the set-up barrier.  Everything before this
    // point (barriers, descriptor prefetch) touched no global data and may overlap the previous
    // kernel of the stream.
    griddep_wait();
    if (nt > 0) {
      mbar_arrive_expect_tx(&bars->q_full, L::kQTiles * L::kTile);
      for (int t = 0; t < L::kQTiles; ++t)
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(smem + L::q_off + t * L::kTile + c * L::kSub, &maps.q, &bars->q_full, c * 64,
                      r_tile_of[t] - p.m_begin, h, b);
      for (int idx = 0; idx < n_early; ++idx) issue_kv_load(idx, idx);
    }
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  griddep_wait();  // every thread, before its first global access
  // Only now (the kernels before this one are complete) may a dependent launch begin: the key-major
  // pass of the same call reads q and k while this grid drains, the next forward launch sets itself
  // up on SMs this grid no longer needs.
  griddep_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp < 4) {
    reg_dealloc<REGS_AUX>();
    if (warp == 0 && lane == 0) {
      // ---------------------------------------------------------- TMA producer (rest of the ring)
      // Persistent CTAs: the ring runs on across items, so the next item's first K and V tiles arrive
      // while the current item's last tiles are computed; its Q tiles follow as soon as the current
      // item's last Q.K^T has completed.
      int ring_base = 0;
      bool ok = true;
      for (int k = 0; ok; ++k) {
        if (k > 0) {
          if (!(ok = mbar_wait(&bars->q_empty, (k - 1) & 1, abort_flag))) break;
          if (nt > 0) {
            mbar_arrive_expect_tx(&bars->q_full, L::kQTiles * L::kTile);
            for (int t = 0; t < L::kQTiles; ++t)
              for (int c = 0; c < D / 64; ++c)
                tma_load_4d(smem + L::q_off + t * L::kTile + c * L::kSub, &maps.q, &bars->q_full, c * 64,
                            r_tile_of[t] - p.m_begin, h, b);
          }
        }
        for (int idx = (k == 0 ? n_early : 0); idx < 2 * nt; ++idx) {
          const int g = ring_base + idx;
          const int s = g % KV_SLOTS, u = g / KV_SLOTS;
          if (!(ok = mbar_wait(&bars->kv_empty[s], (u & 1) ^ 1, abort_flag))) break;
          issue_kv_load(idx, g);
        }
        ring_base += 2 * nt;
        if (!ok || !goto_item(k + 1)) break;
      }
    } else if (HOOK == kHookColPart && warp >= 2) {
      // ---------------------------------------------------------- per-tile sums of the query rows
      // The linear part of the raw column sums needs sum_i q_i of every fully contributing query
      // tile; the tiles are in shared memory anyway, so the two otherwise idle warps add them up.
      // A warp reads one 128-byte swizzled row segment per step (conflict-free).
      int q_cnt = 0;  // items of this CTA whose Q tiles were loaded (those with key tiles to visit)
      for (int k = 0;; ++k) {
      if (nt > 0) ++q_cnt;
      if (p.col_lin != 0 && p.qsum != nullptr && nt > 0) {
        if (mbar_wait(&bars->q_full, (q_cnt - 1) & 1, abort_flag)) {
          const int nqb_total = (p.M + 127) / 128;
          for (int unit = (warp - 2) * 32 + lane; unit < L::kQTiles * (D / 2); unit += 64) {
            const int t = unit / (D / 2), pair = unit % (D / 2);
            // (a tile that starts before the first contributing row is never a linear one: its sum is not read)
            if (r_tile_of[t] < p.col_row_lo) continue;
            const int c = pair >> 5, word = pair & 31;
            const unsigned char* base = smem + L::q_off + t * L::kTile + c * L::kSub + ((word & 3) << 2);
            float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll 8
            for (int r = 0; r < BM; r += 2) {
              const float2 x = unpack2<T>(*reinterpret_cast<const uint32_t*>(
                  base + r * 128 + (((word >> 2) ^ (r & 7)) << 4)));
              const float2 y = unpack2<T>(*reinterpret_cast<const uint32_t*>(
                  base + (r + 1) * 128 + (((word >> 2) ^ ((r + 1) & 7)) << 4)));
              a0 += x.x; a1 += x.y;
              b0 += y.x; b1 += y.y;
            }
            const int r0 = r_tile_of[t];
            if (r0 < p.M) {
              float* dst = p.qsum + (((int64_t)bh * nqb_total + r0 / BM) * 128 + c * 64 + word * 2);
              *reinterpret_cast<float2*>(dst) = make_float2(a0 + b0, a1 + b1);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->q_empty);  // this warp no longer reads the item's Q tiles
      // (its arrival for the next item must not be counted in this item's phase)
      if (!persist || !mbar_wait(&bars->q_empty, k & 1, abort_flag) || !goto_item(k + 1)) break;
      }
    } else if (warp == 1) {
      // ---------------------------------------------------------- MMA issuer
      // The whole warp runs this loop (converged control flow); inside each group one elected
      // lane issues the tcgen05 instructions.
      constexpr int kFmt = std::is_same<T, __half>::value ? 0 : 1;
      constexpr uint32_t idesc_qk = make_idesc_f16(128, BN, kFmt, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_f16(128, D, kFmt, 0, 1);
      // Operand descriptors are built once; inside the loops only compile-time offsets (in
      // 16-byte units) are added to their address field, so the issuing thread spends a few
      // instructions per MMA.
      const uint64_t q_desc0 = make_desc_sw128(smem_u32(smem + L::q_off), 16, 1024);
      const uint64_t k_desc0 = make_desc_sw128(smem_u32(smem + L::kv_off), 16, 1024);
      const uint64_t v_desc0 = make_desc_sw128(smem_u32(smem + L::kv_off), L::kSub, 1024);
      int ring_base = 0;  // ring entries of the CTA's earlier items
      auto kv_wait = [&](int idx) -> bool {
        const int g = ring_base + idx;
        if (!mbar_wait(&bars->kv_full[g % KV_SLOTS], (g / KV_SLOTS) & 1, abort_flag)) return false;
        tc_fence_after();
        return true;
      };
      auto ring_slot = [&](int idx) -> int { return (ring_base + idx) % KV_SLOTS; };
      // S_t = Q_t . K^T for the key tile in ring slot `slot`
      auto issue_qk = [&](int t, int slot) {
        const uint64_t qd = q_desc0 + (uint64_t)((SPLIT ? 0 : t) * (L::kTile >> 4));
        const uint64_t kd = k_desc0 + (uint64_t)(slot * (L::kTile >> 4));
        const uint32_t d_tmem = tmem_base + (uint32_t)(t * BN);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t off = (uint64_t)(((kk >> 2) * L::kSub + (kk & 3) * 32) >> 4);
            if (kk == 0) mma_ss(d_tmem, qd + off, kd + off, idesc_qk, 0u);
            else mma_ss_acc(d_tmem, qd + off, kd + off, idesc_qk);
          }
          mma_commit(&bars->s_full[t]);
        }
        __syncwarp();
      };
      // O_t (+)= P_t . V; P_t sits in the first 64 columns of S_t (two 16-bit values per column)
      // The softmax hands P over in two halves of 64 key columns, so the first four K-steps of
      // P.V run while the second half of the exponentials is still being computed.
      auto issue_pv_half = [&](int t, int slot, bool accumulate, int half) {
        const uint64_t vd = v_desc0 + (uint64_t)(slot * (L::kTile >> 4));
        const uint32_t d_tmem = tmem_base + 256 + (uint32_t)(t * BN);
        const uint32_t a_tmem = tmem_base + (uint32_t)(t * BN);
        if (elect_one()) {
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            const int kk = half * 4 + k4;
            const uint64_t off = (uint64_t)((kk * 16 * 128) >> 4);
            if (kk == 0) mma_ts(d_tmem, a_tmem, vd, idesc_pv, accumulate ? 1u : 0u);
            else mma_ts_acc(d_tmem, a_tmem + (uint32_t)(kk * 8), vd + off, idesc_pv);
          }
        }
        __syncwarp();
      };
      // waits for the two hand-offs of query tile / warpgroup t and issues both halves
      // (c: hand-offs of t so far over all items, the barrier phase; first: is it the item's first)
      auto pv_when_ready = [&](int t, int slot, int c, bool first) -> bool {
        if (!mbar_wait(&bars->p_half[t], c & 1, abort_flag)) return false;
        tc_fence_after();
        issue_pv_half(t, slot, !first, 0);
        if (!mbar_wait(&bars->p_ready[t], c & 1, abort_flag)) return false;
        tc_fence_after();
        issue_pv_half(t, slot, true, 1);
        return true;
      };
      auto issue_pv = [&](int t, int slot, bool accumulate) {
        const uint64_t vd = v_desc0 + (uint64_t)(slot * (L::kTile >> 4));
        const uint32_t d_tmem = tmem_base + 256 + (uint32_t)(t * BN);
        const uint32_t a_tmem = tmem_base + (uint32_t)(t * BN);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk) {
            const uint64_t off = (uint64_t)((kk * 16 * 128) >> 4);
            if (kk == 0) mma_ts(d_tmem, a_tmem, vd, idesc_pv, accumulate ? 1u : 0u);
            else mma_ts_acc(d_tmem, a_tmem + (uint32_t)(kk * 8), vd + off, idesc_pv);
          }
        }
        __syncwarp();
      };
      auto commit = [&](uint64_t* bar) {
        if (elect_one()) mma_commit(bar);
        __syncwarp();
      };
      int cnt[2] = {0, 0};  // key tiles each warpgroup has been given so far, over all items
      int q_cnt = 0;        // items whose Q tiles were loaded
      bool ok = true;
      for (int k = 0; ok; ++k) {
      if (nt > 0) {
      ok = mbar_wait(&bars->q_full, q_cnt & 1, abort_flag);
      ++q_cnt;
      const int cnt0[2] = {cnt[0], cnt[1]};
      if constexpr (SPLIT) {
        // Visiting index `it` belongs to warpgroup it & 1.  Before S of that warpgroup is
        // overwritten by Q.K^T of tile it, the P.V of its previous tile (it - 2) is issued.
        for (int it = 0; ok && it < nt + 2; ++it) {
          const int w = it & 1;
          if (it >= 2) {
            const int v_idx = 2 * (it - 2) + 1;
            if (!(ok = kv_wait(v_idx))) break;
            if (!(ok = pv_when_ready(w, v_idx % KV_SLOTS, cnt[w], cnt[w] == cnt0[w]))) break;
            ++cnt[w];
            commit(&bars->kv_empty[v_idx % KV_SLOTS]);
          }
          if (it < nt) {
            if (!(ok = kv_wait(2 * it))) break;
            issue_qk(w, (2 * it) % KV_SLOTS);
            commit(&bars->kv_empty[(2 * it) % KV_SLOTS]);
          }
        }
      } else {
      if (ok) ok = kv_wait(0);
      if (ok) {
        const int t0 = tile_of(0);
        if (t0 < nt_q[0]) issue_qk(0, ring_slot(0));
        if (t0 < nt_q[1]) issue_qk(1, ring_slot(0));
        commit(&bars->kv_empty[ring_slot(0)]);
      }
      for (int it = 0; ok && it < nt; ++it) {
        const int tk = tile_of(it);
        const bool more = it + 1 < nt;
        const int tk_next = more ? tile_of(it + 1) : 0;
        const int v_slot = ring_slot(2 * it + 1), k_slot = ring_slot(2 * it + 2);
        // every Q.K^T of the item has been issued: when they complete, the next item's Q tiles may land
        if (!more) commit(&bars->q_empty);
        if (!(ok = kv_wait(2 * it + 1))) break;
        if (tk < nt_q[0]) {
          if (!(ok = pv_when_ready(0, v_slot, cnt[0], cnt[0] == cnt0[0]))) break;
          ++cnt[0];
        }
        if (more) {
          if (!(ok = kv_wait(2 * it + 2))) break;
          if (tk_next < nt_q[0]) issue_qk(0, k_slot);
        }
        if (tk < nt_q[1]) {
          if (!(ok = pv_when_ready(1, v_slot, cnt[1], cnt[1] == cnt0[1]))) break;
          ++cnt[1];
        }
        commit(&bars->kv_empty[v_slot]);
        if (more) {
          if (tk_next < nt_q[1]) issue_qk(1, k_slot);
          commit(&bars->kv_empty[k_slot]);
        }
      }
      }  // !SPLIT
      if (ok) commit(&bars->o_done);
      ring_base += 2 * nt;
      } else {  // an item without key tiles: nothing was loaded, nothing to issue
        if (elect_one()) mbar_arrive(&bars->q_empty);
        __syncwarp();
      }
      if (!ok || !goto_item(k + 1)) break;
      }
    }
  } else {
    reg_alloc<REGS_SOFTMAX>();
    // ------------------------------------------------------------ softmax warps
    const int qt = (warp - 4) >> 2;  // warpgroup: its query tile (or, SPLIT, its half of the key tiles)
    const int lg = warp & 3;         // TMEM lane group this warp may touch
    const int row = lg * 32 + lane;
    const uint32_t t_lane = tmem_base + ((uint32_t)(lg * 32) << 16);
    const uint32_t t_s = t_lane + (uint32_t)(qt * BN);
    const uint32_t t_o = t_lane + 256 + (uint32_t)(qt * BN);
    const float scale = p.sm_scale;
    const float scale_log2 = p.sm_scale * kLog2e;
    unsigned char* stage = smem + L::stage_off + (warp - 4) * 8192;
    float* colbuf = reinterpret_cast<float*>(smem + L::stage_off + qt * 32768);  // [2][4][128], col hook only
    constexpr bool store_scores = HOOK == kHookScores;
    constexpr bool store_scores16 = HOOK == kHookScores16;
    constexpr bool store_scratch = HOOK == kHookScratch;
    const float masked_f = __uint_as_float(p.masked_bits);
    // per item
    int r_tile, i, my_nt, qb128;  // first row of the query tile, this thread's row, end of its key-tile range
    bool row_ok, part_on;
    uint32_t drop_row;  // Philox counter of (b, h, i, key 0) without the call's offset, 32-bit wrap-around
    float m_run, l_run, rs_raw;
    // over all items of the CTA
    bool alive = true;
    int hook_cnt = 0;  // column hook executions (selects its smem buffer and barrier phase)
    int s_cnt = 0;     // key tiles processed (phase of s_full)
    int o_cnt = 0;     // items with key tiles (phase of o_done)

    // One key tile.  The row's 128 scores are read from TMEM once and stay in registers: first
    // for the max and exp2 passes (the chain the tensor pipe waits on), then, after P has been
    // handed back, for the score-tile hook.  kMasked = false is the fully visible tile.
    auto tile_body = [&](auto masked_tag, int cnt, int n0) -> bool {
      constexpr bool kMasked = decltype(masked_tag)::value;
      uint32_t r[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(t_s + c * 32, reinterpret_cast<uint32_t(&)[32]>(r[c * 32]));
      tmem_wait_ld();
      int nvis = 128;  // visible columns form a prefix of the tile's row
      if (kMasked) {
        int lim = p.N;
        if (p.causal) lim = min(lim, i + p.p_seq + 1);
        nvis = max(0, min(128, lim - n0));
      }
#define FAWS_VIS(x) (!kMasked || (x) < nvis)

      // ---- row max (4 independent chains)
      float a0 = FAWS_NEG_INF, a1 = FAWS_NEG_INF, a2 = FAWS_NEG_INF, a3 = FAWS_NEG_INF;
#pragma unroll
#define FAWS_SV(x) (FAWS_VIS(x) ? __uint_as_float(r[x]) : FAWS_NEG_INF)
      for (int x = 0; x < 128; x += 8) {  // three-input max: 64 instructions for 128 values
        a0 = fmax3(a0, FAWS_SV(x), FAWS_SV(x + 1));
        a1 = fmax3(a1, FAWS_SV(x + 2), FAWS_SV(x + 3));
        a2 = fmax3(a2, FAWS_SV(x + 4), FAWS_SV(x + 5));
        a3 = fmax3(a3, FAWS_SV(x + 6), FAWS_SV(x + 7));
      }
#undef FAWS_SV
      const float mx = fmaxf(fmaxf(a0, a1), fmaxf(a2, a3)) * scale_log2;  // sm_scale > 0

      // ---- running max, lazy rescale of O.  s_full for this tile was committed after this
      // query tile's previous P.V MMA, so O_t is quiescent here.
      const float m_new = fmaxf(m_run, mx);
      const bool need = m_new > m_run + kRescaleThreshold;
      float alpha = 1.f;
      if (need) {
        alpha = fast_exp2(m_run - m_new);
        m_run = m_new;
        l_run *= alpha;
      }
      if (cnt > 0 && __any_sync(0xffffffffu, need)) {
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t ro[32];
          tmem_ld32(t_o + c * 32, ro);
          tmem_wait_ld();
#pragma unroll
          for (int x = 0; x < 32; ++x) ro[x] = __float_as_uint(__uint_as_float(ro[x]) * alpha);
          tmem_st32(t_o + c * 32, ro);
        }
      }

      // ---- P = exp2(s*scale*log2e - m), row sum of P, P -> TMEM over S as 16-bit pairs
      const float neg_m = (m_run == FAWS_NEG_INF) ? 0.f : -m_run;
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
      const uint64_t neg_m2 = pack_f32x2(neg_m, neg_m);
      const uint64_t scale2 = pack_f32x2(scale_log2, scale_log2);
      uint64_t lp0 = 0ull, lp1 = 0ull;
      // masked tiles: the most columns any row of this warp sees (a 32-column block beyond it is all
      // zeros in P for the whole warp and skips its 32 exponentials per row: 6 of the 16 blocks of a
      // diagonal tile)
      const int nvis_warp = kMasked ? __reduce_max_sync(0xffffffffu, nvis) : 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
        const bool block_hidden = kMasked && c * 32 >= nvis_warp;
        if (block_hidden) {
#pragma unroll
          for (int x = 0; x < 16; ++x) pk[x] = 0u;
        } else {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float e[8];
          // packed 2 x fp32 FMA / ADD: half the FMA-pipe instructions of the scalar form
#pragma unroll
          for (int y = 0; y < 8; y += 2) {
            const int x = c * 32 + g * 8 + y;
            float t0, t1;
            const uint64_t t2 = fma_f32x2(pack_f32x2(__uint_as_float(r[x]), __uint_as_float(r[x + 1])), scale2, neg_m2);
            unpack_f32x2(t2, t0, t1);
            t0 = fast_exp2(t0);
            t1 = fast_exp2(t1);
            e[y] = FAWS_VIS(x) ? t0 : 0.f;
            e[y + 1] = FAWS_VIS(x + 1) ? t1 : 0.f;
          }
          lp0 = add_f32x2(lp0, add_f32x2(pack_f32x2(e[0], e[1]), pack_f32x2(e[4], e[5])));
          lp1 = add_f32x2(lp1, add_f32x2(pack_f32x2(e[2], e[3]), pack_f32x2(e[6], e[7])));
          if constexpr (DROP) {
            // dropout acts on the weights that multiply V only; the row sums above are taken
            // before it (flash.py:459-466)
            const uint32_t base = drop_row + (uint32_t)(n0 + c * 32 + g * 8);
#pragma unroll
            for (int y = 0; y < 8; ++y)
              if (!dropout_keep(p.drop, base + (uint32_t)y)) e[y] = 0.f;
          }
          pk[g * 4 + 0] = pack2<T>(e[0], e[1]);
          pk[g * 4 + 1] = pack2<T>(e[2], e[3]);
          pk[g * 4 + 2] = pack2<T>(e[4], e[5]);
          pk[g * 4 + 3] = pack2<T>(e[6], e[7]);
        }
        }
        tmem_st16(t_s + c * 16, pk);
        if (c == 1) {  // first 64 key columns of P are complete: let their P.V K-steps start
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(&bars->p_half[qt]);
        }
      }
      tmem_wait_st();
      unpack_f32x2(lp0, l0, l1);
      unpack_f32x2(lp1, l2, l3);
      l_run += (l0 + l1) + (l2 + l3);
      tc_fence_before();
      mbar_arrive(&bars->p_ready[qt]);

      // ---- score-tile hooks: off the chain above, they overlap this tile's P.V MMA
      if constexpr (HOOK == kHookRowSum) {
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;  // (packed 2 x fp32 adds measured 3 % slower here)
#pragma unroll
        for (int x = 0; x < 128; x += 4) {
          s0 += FAWS_VIS(x) ? __uint_as_float(r[x]) : 0.f;
          s1 += FAWS_VIS(x + 1) ? __uint_as_float(r[x + 1]) : 0.f;
          s2 += FAWS_VIS(x + 2) ? __uint_as_float(r[x + 2]) : 0.f;
          s3 += FAWS_VIS(x + 3) ? __uint_as_float(r[x + 3]) : 0.f;
        }
        rs_raw += (s0 + s1) + (s2 + s3);
      }
      if constexpr (store_scores16) {
        // 16-bit scores: a 64-column half tile is one 32-row x 128-byte box; the two 4 KB staging
        // buffers alternate, lane 0 issues the stores.
        const T masked_t = from_float<T>(masked_f);
        const uint32_t masked2 = pack_bits<T>(masked_t, masked_t);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          unsigned char* sb = stage + half * 4096;
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
#pragma unroll
          for (int cc = 0; cc < 8; ++cc) {
            uint32_t w[4];
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) {
              const int x = half * 64 + cc * 8 + e2 * 2;
              w[e2] = pack2<T>(__uint_as_float(r[x]) * scale, __uint_as_float(r[x + 1]) * scale);
              if (kMasked) {
                const bool v0 = x < nvis, v1 = x + 1 < nvis;
                if (!v0 && !v1) w[e2] = masked2;
                else if (!v1) w[e2] = (w[e2] & 0xffffu) | (masked2 & 0xffff0000u);
              }
            }
            *reinterpret_cast<uint4*>(sb + lane * 128 + ((cc ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(&maps.st, sb, n0 + half * 64, r_tile + lg * 32 - p.m_begin, bh);
            tma_store_commit();
          }
        }
      }
      if constexpr (store_scores || store_scratch) {
        // Two rounds of two 32-column chunks: both 4 KB staging buffers are rewritten per round,
        // one proxy fence per round, lanes 0 and 1 each issue (and later wait for) one TMA store.
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const bool rows_in = store_scores || (r_tile + lg * 32 >= p.split);
          const bool round_on = rows_in && (store_scores || n0 + half * 64 < p.split);
          if (round_on) {
            if (lane < 2) tma_store_wait_read<0>();
            __syncwarp();
#pragma unroll
            for (int c2 = 0; c2 < 2; ++c2) {
              const int c = half * 2 + c2;
              unsigned char* sb = stage + c2 * 4096;
#pragma unroll
              for (int cc = 0; cc < 8; ++cc) {
                float4 val;
                val.x = __uint_as_float(r[c * 32 + cc * 4 + 0]) * scale;
                val.y = __uint_as_float(r[c * 32 + cc * 4 + 1]) * scale;
                val.z = __uint_as_float(r[c * 32 + cc * 4 + 2]) * scale;
                val.w = __uint_as_float(r[c * 32 + cc * 4 + 3]) * scale;
                if (kMasked && store_scores) {
                  if (!(c * 32 + cc * 4 + 0 < nvis)) val.x = masked_f;
                  if (!(c * 32 + cc * 4 + 1 < nvis)) val.y = masked_f;
                  if (!(c * 32 + cc * 4 + 2 < nvis)) val.z = masked_f;
                  if (!(c * 32 + cc * 4 + 3 < nvis)) val.w = masked_f;
                }
                *reinterpret_cast<float4*>(sb + lane * 128 + ((cc ^ (lane & 7)) << 4)) = val;
              }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane < 2) {
              const int jb = n0 + (half * 2 + lane) * 32;
              if (store_scores) {
                tma_store_3d(&maps.st, stage + lane * 4096, jb, r_tile + lg * 32 - p.m_begin, bh);
              } else if (jb < p.split) {
                tma_store_3d(&maps.st, stage + lane * 4096, jb, r_tile + lg * 32 - p.split, bh);
              }
              tma_store_commit();
            }
          }
        }
      }
      if constexpr (HOOK == kHookColPart) {
        // Tiles in which every entry is visible and every row contributes are left to the
        // reduce kernel (column sums are linear in q there); only edge / diagonal tiles are
        // reduced here.
        const bool lin = p.col_lin != 0 &&
                         col_tile_linear(qb128, n0 / BN, p.col_row_lo, p.m_end, p.N, p.causal, p.p_seq);
        // Nothing to do either where no partial is kept: query tiles before the first contributing row
        // (cross-token sums: rows below the split) and key tiles beyond the summed columns.
        if (!lin && part_on && n0 < p.ncols_pad) {
          const bool contrib = row_ok && i >= p.col_row_begin;
          const int cbuf = hook_cnt & 1;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            // a 32 x 32 block in which none of the warp's rows sees or contributes anything (above the
            // diagonal, outside the row range) sums to zero without the 31 shuffles
            if (!__any_sync(0xffffffffu, contrib && FAWS_VIS(c * 32))) {
              colbuf[(cbuf * 4 + lg) * 128 + c * 32 + lane] = 0.f;
              continue;
            }
            float cv[32];
#pragma unroll
            for (int x = 0; x < 32; ++x)
              cv[x] = (contrib && FAWS_VIS(c * 32 + x)) ? __uint_as_float(r[c * 32 + x]) * scale : 0.f;
            warp_column_sums(cv, lane);
            colbuf[(cbuf * 4 + lg) * 128 + c * 32 + lane] = cv[0];
          }
          mbar_arrive(&bars->col_ready[qt]);
          if (!mbar_wait(&bars->col_ready[qt], hook_cnt & 1, abort_flag)) return false;
          ++hook_cnt;
          if (part_on && n0 + row < p.ncols_pad) {
            const float* cb = colbuf + cbuf * 512;
            // fixed order: the warps that own rows 0-31, 32-63, 64-95, 96-127
            const float sum = ((cb[row] + cb[128 + row]) + cb[256 + row]) + cb[384 + row];
            p.col_partial[((int64_t)bh * p.n_qb_part + (qb128 - p.qb_first)) * (int64_t)p.ncols_pad + n0 + row] = sum;
          }
        }
      }
#undef FAWS_VIS
      return true;
    };

    for (int k = 0;; ++k) {
    r_tile = r_tile_of[qt];
    i = r_tile + row;
    my_nt = nt_q[qt];
    row_ok = i >= p.m_begin && i < p.m_end;
    qb128 = r_tile / BM;
    part_on = HOOK == kHookColPart && qb128 >= p.qb_first && r_tile < p.m_end;
    drop_row = ((uint32_t)bh * (uint32_t)p.M + (uint32_t)i) * (uint32_t)p.N;
    m_run = FAWS_NEG_INF;
    l_run = 0.f;
    rs_raw = 0.f;

    // Key tiles the causal loop never visits hold only the fill value.  They are written first,
    // from one constant 32 x 32 tile, so that HBM is busy while the first tiles are computed
    // (these stores carry 44 % of the bytes of a causal S = N problem).
    if constexpr (store_scores) if (!p.fill_ctas && r_tile < p.m_end && my_nt * BN < p.N) {
      const float4 fill = make_float4(masked_f, masked_f, masked_f, masked_f);
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) *reinterpret_cast<float4*>(stage + lane * 128 + (cc << 4)) = fill;
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int r0 = r_tile + lg * 32 - p.m_begin;
        for (int j0 = my_nt * BN; j0 < p.N; j0 += 32) {
          // SPLIT: the two warpgroups share the rows, so they take alternate key tiles
          if (!SPLIT || ((j0 / BN) & 1) == qt) tma_store_3d(&maps.st, stage, j0, r0, bh);
        }
        tma_store_commit();
      }
      __syncwarp();
    }

    if constexpr (store_scores16) if (!p.fill_ctas && r_tile < p.m_end && my_nt * BN < p.N) {
      const T masked_t = from_float<T>(masked_f);
      const uint32_t m2 = pack_bits<T>(masked_t, masked_t);
      const uint4 fill = make_uint4(m2, m2, m2, m2);
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) *reinterpret_cast<uint4*>(stage + lane * 128 + (cc << 4)) = fill;
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int r0 = r_tile + lg * 32 - p.m_begin;
        for (int j0 = my_nt * BN; j0 < p.N; j0 += 64) {
          if (!SPLIT || ((j0 / BN) & 1) == qt) tma_store_3d(&maps.st, stage, j0, r0, bh);
        }
        tma_store_commit();
      }
      __syncwarp();
    }

    {
      int cnt = 0;
      for (int it = 0; it < nt; ++it) {
        const int tk = tile_of(it);
        if (SPLIT ? ((it & 1) != qt) : (tk >= my_nt)) continue;
        const int n0 = tk * BN;
        if (!mbar_wait(&bars->s_full[qt], s_cnt & 1, abort_flag)) { alive = false; break; }
        ++s_cnt;
        tc_fence_after();
        const bool full_vis = (n0 + BN <= p.N) && (!p.causal || (n0 + BN - 1 <= r_tile + p.p_seq));
        const bool ok = full_vis ? tile_body(std::false_type{}, cnt, n0) : tile_body(std::true_type{}, cnt, n0);
        if (!ok) { alive = false; break; }
        ++cnt;
      }
    }
    const float rs = rs_raw * scale;

    // ---- epilogue: O / l -> out, log-normaliser, row sums, masked fill of unvisited tiles
    if (alive && my_nt > kt0) {
      if (!mbar_wait(&bars->o_done, o_cnt & 1, abort_flag)) alive = false;
      tc_fence_after();
    }
    if (nt > 0) ++o_cnt;
    // SPLIT: warpgroup 1 publishes its running state; warpgroup 0 merges the two partial results.
    float* merge = reinterpret_cast<float*>(smem + L::kv_off);  // ring is free after o_done
    bool write_out = alive && r_tile < p.m_end;
    float l_all = l_run, m_all = m_run, w0 = 1.f, w1 = 0.f;
    float rs_all = rs;
    bool have1 = false;
    if constexpr (SPLIT) {
      if (qt == 1) {
        merge[row] = m_run;
        merge[128 + row] = l_run;
        merge[256 + row] = rs;
        mbar_arrive(&bars->merge_ready);
        write_out = false;
      } else {
        if (!mbar_wait(&bars->merge_ready, 0, abort_flag)) { alive = false; write_out = false; }
        const float m1 = merge[row], l1 = merge[128 + row];
        rs_all = rs + merge[256 + row];
        have1 = nt > 1;  // warpgroup 1 processed at least one tile
        m_all = fmaxf(m_run, m1);
        w0 = (m_run == FAWS_NEG_INF) ? 0.f : fast_exp2(m_run - m_all);
        w1 = (m1 == FAWS_NEG_INF) ? 0.f : fast_exp2(m1 - m_all);
        l_all = l_run * w0 + l1 * w1;
      }
    }
    if (write_out) {
      float inv = l_all > 0.f ? 1.f / l_all : 0.f;
      if constexpr (DROP) inv *= p.drop.out_scale;
      if (my_nt > kt0) {
        // Each warp stages its 32 x D output block (128B-swizzled) and stores it with TMA: in its own
        // staging block where the hook leaves that free, so that a persistent CTA's next Q tiles can land
        // meanwhile; in the Q tiles' shared memory (every MMA of the CTA has completed) under the hooks
        // that stage score tiles.  The column hook keeps partial sums in the first 4 KB of some warps'
        // blocks: under it every warp stages 64 columns at a time in the upper 4 KB of its block
        // (rows written straight from registers, 16 bytes per lane and instruction, measured 1.7 us per item).
        constexpr bool kHalfStage = HOOK == kHookColPart;
        constexpr bool kOwnStage = HOOK == kHookNone || HOOK == kHookRowSum;
        unsigned char* ost = kHalfStage ? stage + 4096
                                        : (kOwnStage ? stage : smem + L::q_off + (warp - 4) * (32 * D * 2));
        if (!kHalfStage && k > 0) {  // the previous item's store has read the staging block
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
        }
        [[maybe_unused]] const float f0 = w0 * inv, f1 = w1 * inv;
        auto put_chunk = [&](int c, const uint32_t (&ro)[32]) {  // 32 columns of the row, already scaled
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w;
            w.x = pack2<T>(__uint_as_float(ro[g * 8 + 0]), __uint_as_float(ro[g * 8 + 1]));
            w.y = pack2<T>(__uint_as_float(ro[g * 8 + 2]), __uint_as_float(ro[g * 8 + 3]));
            w.z = pack2<T>(__uint_as_float(ro[g * 8 + 4]), __uint_as_float(ro[g * 8 + 5]));
            w.w = pack2<T>(__uint_as_float(ro[g * 8 + 6]), __uint_as_float(ro[g * 8 + 7]));
            const int cc = (c & 1) * 4 + g;  // 16-byte chunk inside the 64-column sub-tile
            *reinterpret_cast<uint4*>(ost + (kHalfStage ? 0 : (c >> 1) * 4096) + lane * 128 + ((cc ^ (lane & 7)) << 4)) = w;
          }
        };
        // (all D / 32 loads of the row in flight together measured 2-3 % slower: the registers they hold)
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t ro[32];
          tmem_ld32(t_o + c * 32, ro);
          if (kHalfStage && (c & 1) == 0 && (c > 0 || k > 0)) {  // the store before this one has read the half block
            if (lane == 0) tma_store_wait_read<0>();
            __syncwarp();
          }
          tmem_wait_ld();
          if constexpr (SPLIT) {
            if (have1) {
              uint32_t r1[32];
              tmem_ld32(t_o + BN + c * 32, r1);  // warpgroup 1's accumulator, same lanes
              tmem_wait_ld();
#pragma unroll
              for (int x = 0; x < 32; ++x)
                ro[x] = __float_as_uint(__uint_as_float(ro[x]) * f0 + __uint_as_float(r1[x]) * f1);
            } else {
#pragma unroll
              for (int x = 0; x < 32; ++x) ro[x] = __float_as_uint(__uint_as_float(ro[x]) * f0);
            }
          } else {
#pragma unroll
            for (int x = 0; x < 32; ++x) ro[x] = __float_as_uint(__uint_as_float(ro[x]) * inv);
          }
          put_chunk(c, ro);
          if (kHalfStage && (c & 1) == 1) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_4d(&maps.o, ost, (c >> 1) * 64, r_tile + lg * 32 - p.m_begin, ho, b);
              tma_store_commit();
            }
          }
        }
        if (!kHalfStage) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            for (int sub = 0; sub < D / 64; ++sub)
              tma_store_4d(&maps.o, ost + sub * 4096, sub * 64, r_tile + lg * 32 - p.m_begin, ho, b);
            tma_store_commit();
          }
        }
      } else if (row_ok) {
        // no key is visible to this query tile: its rows are zero
        T* orow = reinterpret_cast<T*>(p.o) + b * p.o_sb + ho * p.o_sh + (int64_t)i * p.o_ss;
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int g = 0; g < D / 8; ++g) *reinterpret_cast<uint4*>(orow + g * 8) = z;
      }
      if (row_ok) {
        if (p.L != nullptr)
          p.L[((int64_t)bh * p.n_splits + ksplit) * p.M + i] = l_all > 0.f ? (m_all + log2f(l_all)) * kLn2 : FAWS_NEG_INF;
        if constexpr (HOOK == kHookRowSum) p.row_sum[(int64_t)bh * p.M + i] = rs_all;
      }
    }
    if (!alive || !goto_item(k + 1)) break;
    }  // items of the CTA
    // Full completion, not only the reads: measured on the score-materialising launches, CTAs that leave
    // while their stores are still draining make the launch 4 % slower; no difference elsewhere.
    if (lane < 2) tma_store_wait<0>();
  }

  // ------------------------------------------------------------ common exit
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && status != nullptr) atomicExch(status, 1);
    // give copies that are still in flight time to land before the smem goes away
    for (int w = 0; w < 50; ++w) __nanosleep(20000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------- key-major pass
// Softmax column sums from a saved log-normaliser (the structure of total.py:50-142 and of the
// reference's second passes, attention_with_col_softmax_sum.py:195-270,
// attention_cross_token_softmax_sum.py:203-268, without atomics):
//   out[j] = sum over heads of the CTA and queries i of exp(s_ij - L_i).
// One CTA owns 128 keys of one (batch, kv head or query head) and walks the query tiles of its
// heads.  S^T = K.Q^T puts keys on TMEM lanes, so thread j accumulates column j in a register:
// no cross-thread reduction, fixed order, one store.
// One CTA owns CS_KT = 2 key tiles (256 keys) of one (batch, kv head or query head): every Q tile
// it streams feeds two MMAs, which halves the Q traffic from L2 (32 KB per 128^3 MMA otherwise).
// (Measured: 1-3 % faster, not more: halving the Q traffic, and, in a separate experiment, moving half of
// the exponentials from the MUFU pipe to a cubic on the FMA pipe, both left the pass where it was.)
// Four consumer warpgroups: warpgroup w owns S^T buffer w = key tile (w & 1) of the query tiles
// of parity (w >> 1); it walks its tiles in chunks of CS_CHUNK columns (that many live score
// registers); the two partial sums of a key tile are added in a fixed order at the end.
constexpr int CS_KT = 2;
constexpr int CS_WGS = 4;
constexpr int CS_QSLOTS = CS_WGS;
constexpr int CS_CHUNK = 64;  // score columns a consumer thread holds at a time
constexpr int CS_LSLOTS = 8;  // query tiles whose -L values are in shared memory (see the producer)
constexpr int CS_THREADS = 128 + CS_WGS * 128;
constexpr int CS_REGS_LAUNCH = (65536 / CS_THREADS) & ~7;  // what the launch bound lets ptxas allocate
constexpr int CS_REGS_AUX = 56;
constexpr int CS_REGS_CONSUMER = ((CS_REGS_LAUNCH * CS_THREADS - 128 * CS_REGS_AUX) / (CS_WGS * 128)) & ~7;
static_assert(128 * CS_REGS_AUX + CS_WGS * 128 * CS_REGS_CONSUMER <= CS_REGS_LAUNCH * CS_THREADS,
              "setmaxnreg would block");
static_assert(CS_WGS == 2 * CS_KT, "buffer w = key tile (w & 1) of query-tile parity (w >> 1)");

template <int D>
struct CsSmem {
  static constexpr int kTile = 128 * D * 2;
  static constexpr int kSub = 128 * 128;
  static constexpr int k_off = 0;                           // CS_KT key tiles
  static constexpr int q_off = k_off + CS_KT * kTile;
  static constexpr int l_off = q_off + CS_QSLOTS * kTile;  // [warpgroup][2][128] floats: -L_i*log2e per query
  static constexpr int comb_off = l_off + CS_WGS * 2 * 128 * 4;  // [key tile][128] floats
  static constexpr int bar_off = comb_off + CS_KT * 128 * 4;
  static constexpr int total = bar_off + 256;
  static constexpr int alloc = total + 1024;
};

struct CsBars {
  uint64_t k_full;
  uint64_t q_full[CS_QSLOTS], q_empty[CS_QSLOTS];
  uint64_t s_full[CS_WGS], s_free[CS_WGS];  // per S^T buffer
  uint64_t l_ready[CS_WGS];
  uint64_t l_full[CS_LSLOTS];  // -L*log2e of a query tile has landed (bulk copy from the padded array)
  uint32_t tmem_base;
  int abort_flag;
};

struct CsMaps {
  CUtensorMap q, k;
};

template <typename T, int D>
__global__ void __launch_bounds__(CS_THREADS, 1)
tc_colsoftmax_kernel(const __grid_constant__ CsMaps maps, const ColSoftmaxParams p, int heads_per_cta,
                     int* __restrict__ status) {
  using L = CsSmem<D>;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  CsBars* bars = reinterpret_cast<CsBars*>(smem + L::bar_off);
  volatile int* abort_flag = &bars->abort_flag;
  float* lbuf = reinterpret_cast<float*>(smem + L::l_off);
  float* comb = reinterpret_cast<float*>(smem + L::comb_off);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Causal: key tiles are the slowest grid dimension, so the key tiles that see the most queries
  // (the first ones) of all heads are dispatched first.  Otherwise key tiles are fastest.
  const int n0 = (p.causal ? blockIdx.z : blockIdx.x) * (CS_KT * BN);  // first key of the CTA's CS_KT key tiles
  const int ho = p.causal ? blockIdx.x : blockIdx.y;
  const int b = p.causal ? blockIdx.y : blockIdx.z;
  const int n_heads_out = p.causal ? gridDim.x : gridDim.y;
  const int h0 = ho * heads_per_cta;  // first query head of this CTA
  const int hk = h0 / p.G;

  // query tiles (absolute multiples of 128) the CTA's first key tile needs, per head (the second key tile
  // sees a suffix of them; what it does not see is masked)
  const int i_lo = max(p.i_begin, p.m_begin);
  int i_first = i_lo;
  if (p.causal) i_first = max(i_first, n0 - p.p_seq);
  const int qt0 = i_first / BM;
  const int ntq = max(0, (p.m_end + BM - 1) / BM - qt0);
  const int total = ntq * heads_per_cta;

  if (threadIdx.x == 0) {
    mbar_init(&bars->k_full, 1);
    for (int s = 0; s < CS_QSLOTS; ++s) {
      mbar_init(&bars->q_full[s], 1);
      mbar_init(&bars->q_empty[s], 1);
    }
    for (int w = 0; w < CS_WGS; ++w) {
      mbar_init(&bars->s_full[w], 1);
      mbar_init(&bars->s_free[w], 128);
      mbar_init(&bars->l_ready[w], 128);
    }
    for (int l = 0; l < CS_LSLOTS; ++l) mbar_init(&bars->l_full[l], 1);
    bars->abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&maps.q);
    prefetch_tmap(&maps.k);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  float acc = 0.f;
  if (warp < 4) {
    reg_dealloc<CS_REGS_AUX>();
    if (warp == 0 && lane == 0 && total > 0) {
      // ---------------------------------------------------------- TMA producer
      mbar_arrive_expect_tx(&bars->k_full, CS_KT * L::kTile);
      for (int kt = 0; kt < CS_KT; ++kt)
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(smem + L::k_off + kt * L::kTile + c * L::kSub, &maps.k, &bars->k_full, c * 64, n0 + kt * BN, hk, b);
      // -L_i*log2e of query tile u goes to slot u % 8 by one 512-byte bulk copy, issued after the Q load
      // of tile u.  That load waited for the MMA of tile u - 4, which was issued only after both
      // warpgroups of this parity had taken all of S^T of tile u - 6 out of TMEM, i.e. after they had
      // finished tile u - 8: its slot is free.  The first copy waits for the kernel that wrote the
      // array; the first Q loads (inputs of the whole call) are in flight by then.
      int l_next = 0;
      bool waited = false;
      for (int u = 0; u < total; ++u) {
        const int s = u % CS_QSLOTS, use = u / CS_QSLOTS;
        const int g = u / ntq, qt = qt0 + (u - g * ntq);
        if (!mbar_wait(&bars->q_empty[s], (use & 1) ^ 1, abort_flag)) break;
        mbar_arrive_expect_tx(&bars->q_full[s], L::kTile);
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(smem + L::q_off + s * L::kTile + c * L::kSub, &maps.q, &bars->q_full[s], c * 64, qt * BM,
                      h0 + g, b);
        if (p.negl_pad != nullptr && (u >= CS_QSLOTS - 1 || u == total - 1)) {
          if (!waited) {
            griddep_wait();
            waited = true;
          }
          for (; l_next <= u; ++l_next) {
            const int gl = l_next / ntq, ql = qt0 + (l_next - gl * ntq);
            const int sl = l_next % CS_LSLOTS;
            mbar_arrive_expect_tx(&bars->l_full[sl], BM * 4);
            bulk_load_1d(lbuf + sl * BM, p.negl_pad + ((int64_t)b * p.Hq + h0 + gl) * p.m_pad + ql * BM, BM * 4,
                         &bars->l_full[sl]);
          }
        }
      }
    } else if (warp == 1 && total > 0) {
      // ---------------------------------------------------------- MMA issuer: S^T = K . Q^T
      // (whole warp in the loop, one elected lane issues)
      constexpr int kFmt = std::is_same<T, __half>::value ? 0 : 1;
      constexpr uint32_t idesc = make_idesc_f16(128, BM, kFmt, 0, 0);
      const uint64_t k_desc = make_desc_sw128(smem_u32(smem + L::k_off), 16, 1024);
      const uint64_t q_desc0 = make_desc_sw128(smem_u32(smem + L::q_off), 16, 1024);
      bool ok = mbar_wait(&bars->k_full, 0, abort_flag);
      for (int u = 0; ok && u < total; ++u) {
        const int s = u % CS_QSLOTS, use = u / CS_QSLOTS;
        const int buf0 = (u & 1) * CS_KT, buse = u >> 1;  // S^T buffers of this query tile, and their use count
        if (!(ok = mbar_wait(&bars->q_full[s], use & 1, abort_flag))) break;
        for (int kt = 0; ok && kt < CS_KT; ++kt) ok = mbar_wait(&bars->s_free[buf0 + kt], (buse & 1) ^ 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint64_t qd = q_desc0 + (uint64_t)(s * (L::kTile >> 4));
        if (elect_one()) {
#pragma unroll
          for (int kt = 0; kt < CS_KT; ++kt) {
            const uint32_t d_tmem = tmem_base + (uint32_t)((buf0 + kt) * BM);
            const uint64_t kd = k_desc + (uint64_t)(kt * (L::kTile >> 4));
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint64_t off = (uint64_t)(((kk >> 2) * L::kSub + (kk & 3) * 32) >> 4);
              if (kk == 0) mma_ss(d_tmem, kd + off, qd + off, idesc, 0u);
              else mma_ss_acc(d_tmem, kd + off, qd + off, idesc);
            }
            if (kt == CS_KT - 1) mma_commit(&bars->q_empty[s]);
            mma_commit(&bars->s_full[buf0 + kt]);
          }
        }
        __syncwarp();
      }
    }
  } else {
    reg_alloc<CS_REGS_CONSUMER>();
    // ------------------------------------------------------------ consumers: thread = key
    // L comes from the forward pass this launch may overlap (programmatic dependent launch): the
    // consumers are the only threads that read it, and the only ones that write the result.
    griddep_wait();
    const int wg = (warp - 4) >> 2;
    const int lg = warp & 3;
    const int row = lg * 32 + lane;
    const int kt = wg & (CS_KT - 1), par = wg / CS_KT;  // this warpgroup's key tile and query-tile parity
    const int nk0 = n0 + kt * BN;                      // first key of that tile
    const int j = nk0 + row;
    const uint32_t t_buf = tmem_base + ((uint32_t)(lg * 32) << 16) + (uint32_t)(wg * BM);
    const float scale_log2 = p.sm_scale * kLog2e;

    // -L_i*log2e of query tile u (for this thread's column x = row), -inf where the query is
    // outside the summed range or has no visible key
    auto load_negl = [&](int u) -> float {
      const int g = u / ntq, qt = qt0 + (u - g * ntq);
      const int i = qt * BM + row;
      float v = FAWS_NEG_INF;
      if (i >= i_lo && i < p.m_end) {
        const float Li = p.L[((int64_t)b * p.Hq + h0 + g) * p.M + i];
        if (Li != FAWS_NEG_INF) v = -Li * kLog2e;
      }
      return v;
    };

    bool alive = true;
    int mine = 0;  // tiles this warpgroup has processed
    const bool padded = p.negl_pad != nullptr;  // the producer fetches -L*log2e; else the warpgroup loads L itself
    float negl_next = (!padded && par < total) ? load_negl(par) : FAWS_NEG_INF;
    for (int u = par; u < total; u += 2, ++mine) {
      float* lb;
      if (padded) {
        lb = lbuf + (u % CS_LSLOTS) * BM;
        if (!mbar_wait(&bars->l_full[u % CS_LSLOTS], (u / CS_LSLOTS) & 1, abort_flag)) { alive = false; break; }
      } else {
        // Two L buffers per warpgroup: the barrier below completes only when every thread of the
        // warpgroup has finished the previous tile, so the buffer of the tile before that is free.
        lb = lbuf + (wg * 2 + (mine & 1)) * 128;
        lb[row] = negl_next;
        mbar_arrive(&bars->l_ready[wg]);
        if (u + 2 < total) negl_next = load_negl(u + 2);
        if (!mbar_wait(&bars->l_ready[wg], mine & 1, abort_flag)) { alive = false; break; }
      }
      if (!mbar_wait(&bars->s_full[wg], mine & 1, abort_flag)) { alive = false; break; }
      tc_fence_after();
      const int g = u / ntq, qt = qt0 + (u - g * ntq);
      const int i0 = qt * BM;
      // causal: query column x is visible to key j iff i0 + x + p_seq >= j
      const int xlo = p.causal ? (j - p.p_seq - i0) : 0;
      const bool full = !p.causal || (nk0 + BN - 1 - p.p_seq - i0 <= 0);
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < BM; c0 += CS_CHUNK) {
        uint32_t r[CS_CHUNK];
#pragma unroll
        for (int c = 0; c < CS_CHUNK; c += 32)
          tmem_ld32(t_buf + c0 + c, reinterpret_cast<uint32_t(&)[32]>(r[c]));
        tmem_wait_ld();
        if (c0 + CS_CHUNK == BM) {  // the buffer can take the next S^T of this warpgroup
          tc_fence_before();
          mbar_arrive(&bars->s_free[wg]);
        }
        const float* lh = lb + c0;
        if (full) {
          const uint64_t scale2 = pack_f32x2(scale_log2, scale_log2);
          uint64_t ap0 = pack_f32x2(a0, a1), ap1 = pack_f32x2(a2, a3);
#pragma unroll
          for (int x = 0; x < CS_CHUNK; x += 4) {
            const float4 nl = *reinterpret_cast<const float4*>(lh + x);
            float t0, t1, t2, t3;
            unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(r[x]), __uint_as_float(r[x + 1])), scale2,
                                   pack_f32x2(nl.x, nl.y)), t0, t1);
            unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(r[x + 2]), __uint_as_float(r[x + 3])), scale2,
                                   pack_f32x2(nl.z, nl.w)), t2, t3);
            ap0 = add_f32x2(ap0, pack_f32x2(fast_exp2(t0), fast_exp2(t1)));
            ap1 = add_f32x2(ap1, pack_f32x2(fast_exp2(t2), fast_exp2(t3)));
          }
          unpack_f32x2(ap0, a0, a1);
          unpack_f32x2(ap1, a2, a3);
        } else {
          const int xh = xlo - c0;
          // query columns below the smallest bound in the warp are hidden from all of its keys: no exp2 there
          const int xh_warp = __reduce_min_sync(0xffffffffu, xh);
#pragma unroll
          for (int x = 0; x < CS_CHUNK; x += 4) {
            if (x + 3 < xh_warp) continue;
            const float4 nl = *reinterpret_cast<const float4*>(lh + x);
            a0 += (x >= xh) ? fast_exp2(fmaf(__uint_as_float(r[x]), scale_log2, nl.x)) : 0.f;
            a1 += (x + 1 >= xh) ? fast_exp2(fmaf(__uint_as_float(r[x + 1]), scale_log2, nl.y)) : 0.f;
            a2 += (x + 2 >= xh) ? fast_exp2(fmaf(__uint_as_float(r[x + 2]), scale_log2, nl.z)) : 0.f;
            a3 += (x + 3 >= xh) ? fast_exp2(fmaf(__uint_as_float(r[x + 3]), scale_log2, nl.w)) : 0.f;
          }
        }
      }
      acc += (a0 + a1) + (a2 + a3);
    }
    if (!alive) acc = 0.f;
    if (par > 0) comb[kt * 128 + row] = acc;  // the odd query tiles' share of key tile kt
  }

  // ------------------------------------------------------------ common exit
  tc_fence_before();
  __syncthreads();
  if (warp >= 4 && warp < 4 + 4 * CS_KT) {  // the even-parity warpgroup of each key tile writes it
    const int row = (warp & 3) * 32 + lane;
    const int kt = (warp - 4) >> 2;
    const int j = n0 + kt * BN + row;
    if (j < p.n_end) {  // even query tiles first, then the odd ones
      p.out[((int64_t)b * n_heads_out + ho) * p.n_end + j] = acc + comb[kt * 128 + row];
    }
  }
  if (*abort_flag) {
    if (threadIdx.x == 0 && status != nullptr) atomicExch(status, 1);
    for (int w = 0; w < 50; ++w) __nanosleep(20000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------- host side
// Per-device status word the kernels raise when a bounded wait gives up.
__device__ int g_tc_status = 0;

}  // namespace

int* tc_status_word() {
  static int* words[kMaxDevices] = {nullptr};
  static std::mutex mu;
  const int dev = current_device();
  if (dev < 0) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (words[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_tc_status) == cudaSuccess) words[dev] = static_cast<int*>(ptr);
  }
  return words[dev];
}

namespace {

// Work lists of a persistent launch.  An item costs its key tiles plus a fixed part; the items, heaviest
// first, go one by one to the CTA with the least work so far (what the hardware does with the CTAs of a
// plain launch, here decided ahead).  Made once per problem geometry and kept for the next call.
bool persistent_allowed();

struct WorkKey {
  int gx, gy, gz, lpt, causal, p_seq, m_begin, m_end, N, rows, ctas;
  bool operator==(const WorkKey& o) const { return std::memcmp(this, &o, sizeof(WorkKey)) == 0; }
};

const WorkList& plain_work_list() {
  static const WorkList wl{};  // n_items = 0
  return wl;
}

// false: the launch should stay a plain one
bool make_work_list(const FwdParams& p, dim3 grid, int cta_rows, int ctas, WorkList* out) {
  const int n_items = (int)(grid.x * grid.y * grid.z);
  if (ctas > kMaxListCtas || n_items <= ctas || n_items > 65535) return false;
  const bool listed = n_items <= kMaxListedItems;
  if (!listed && p.causal) return false;  // unequal items in no useful order: leave them to the hardware
  thread_local WorkKey last_key{};
  thread_local WorkList last{};
  const WorkKey key{(int)grid.x, (int)grid.y, (int)grid.z, p.lpt_order, p.causal, p.p_seq, p.m_begin, p.m_end, p.N,
                    cta_rows, ctas};
  if (last.n_items > 0 && key == last_key) {
    *out = last;
    return true;
  }
  WorkList& wl = last;
  wl = WorkList{};
  wl.n_items = n_items;
  wl.listed = listed ? 1 : 0;
  wl.gx = (int)grid.x;
  wl.gy = (int)grid.y;
  wl.gz = (int)grid.z;
  if (listed) {
    const int ncb = (int)(p.lpt_order ? grid.z : grid.x);
    std::vector<int> cost(ncb);
    for (int slot = 0; slot < ncb; ++slot) {
      const int r0 = p.m_begin + (ncb - 1 - slot) * cta_rows;
      int tiles = 0;
      for (int t = 0; t * BM < cta_rows; ++t) {
        const int r = r0 + t * BM;
        int hi = 0;
        if (r < p.m_end) hi = p.causal ? std::max(0, std::min(p.N, p.p_seq + std::min(r + BM, p.m_end))) : p.N;
        tiles = std::max(tiles, (hi + BN - 1) / BN);
      }
      cost[slot] = 19 * tiles + 30;  // measured on cfg3: 1.90 us per key tile + 3.0 us per item (unit 0.1 us)
    }
    auto cost_of = [&](int item) {
      const int ix = item % wl.gx, iz = item / (wl.gx * wl.gy);
      return cost[p.lpt_order ? iz : ix];
    };
    std::vector<int> order(n_items);
    for (int i = 0; i < n_items; ++i) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return cost_of(a) > cost_of(b); });
    // Heaviest item first onto the CTA with the least work so far (what the hardware does with the CTAs
    // of a plain grid), then exchanges of single items between any two CTAs that bring their loads closer
    // together, fuller CTAs first against the emptiest.  Exchanges keep the number of items per CTA, so
    // the result does not lean on the fixed cost per item, which differs between the hooks (3 us plain,
    // 6 us with the column hook, measured on cfg3; packing to a capacity instead put up to 30 small items
    // on one CTA and was 30 % slower under the column hook).  cfg3: 48..56 key tiles per CTA -> 50..52.
    std::vector<std::vector<uint16_t>> mine(ctas);
    std::vector<long long> load(ctas, 0);
    {
      using Load = std::pair<long long, int>;  // (work so far, CTA)
      std::priority_queue<Load, std::vector<Load>, std::greater<Load>> heap;
      for (int c = 0; c < ctas; ++c) heap.push({0, c});
      for (int item : order) {
        Load l = heap.top();
        heap.pop();
        mine[l.second].push_back((uint16_t)item);
        load[l.second] = l.first + cost_of(item);
        heap.push({load[l.second], l.second});
      }
    }
    for (int round = 0; round < 32; ++round) {
      bool improved = false;
      std::vector<int> by_load(ctas);
      for (int c = 0; c < ctas; ++c) by_load[c] = c;
      std::stable_sort(by_load.begin(), by_load.end(), [&](int x, int y) { return load[x] > load[y]; });
      for (int ai = 0; ai < ctas; ++ai) {
        const int A = by_load[ai];
        for (int bi = ctas - 1; bi >= 0; --bi) {
          const int B = by_load[bi];
          const long long gap = load[A] - load[B];
          if (gap <= 0) break;  // (the order is the one before this round's exchanges: good enough)
          long long best_gain = 0, best_d = 0;
          int bia = -1, bib = -1;
          for (size_t ia = 0; ia < mine[A].size(); ++ia)
            for (size_t ib = 0; ib < mine[B].size(); ++ib) {
              const long long d = cost_of(mine[A][ia]) - cost_of(mine[B][ib]);
              if (d <= 0 || d >= gap) continue;
              const long long after = gap - 2 * d;
              const long long gain = gap - (after < 0 ? -after : after);  // how much closer the two get
              if (gain > best_gain) { best_gain = gain; best_d = d; bia = (int)ia; bib = (int)ib; }
            }
          if (bia < 0) continue;
          std::swap(mine[A][bia], mine[B][bib]);
          load[A] -= best_d;
          load[B] += best_d;
          improved = true;
        }
      }
      if (!improved) break;
    }
    for (int c = 0; c < ctas; ++c)  // heaviest item first within a CTA
      std::stable_sort(mine[c].begin(), mine[c].end(), [&](uint16_t x, uint16_t y) { return cost_of(x) > cost_of(y); });
    int at = 0;
    for (int c = 0; c < ctas; ++c) {
      wl.start[c] = (uint16_t)at;
      for (uint16_t id : mine[c]) wl.ids[at++] = id;
    }
    for (int c = ctas; c <= kMaxListCtas; ++c) wl.start[c] = (uint16_t)at;
  }
  last_key = key;
  *out = wl;
  return true;
}

template <typename T, int D, int HOOK, bool SPLIT, bool DROP = false>
cudaError_t launch_fwd_s(const TcMaps& maps, const FwdParams& p, cudaStream_t s) {
  using L = Smem<D, SPLIT>;
  static PerDeviceOnce attr_once;
  if (cudaError_t e = set_max_smem_once(attr_once, tc_fwd_kernel<T, D, HOOK, SPLIT, DROP>, L::alloc); e != cudaSuccess)
    return e;
  const int ncb = (p.m_end - p.m_begin + L::kRows - 1) / L::kRows;
  FwdParams pp = p;
  // K and V of all heads together stay resident in the 126 MB L2 -> order CTAs for load balance
  const long long kv_bytes = 2LL * p.B * p.Hk * p.N * p.D * 2;
  pp.lpt_order = (p.causal && kv_bytes <= (48LL << 20) && 2 * ncb <= 65535) ? 1 : 0;
  // masked key tiles exist (causal, some row block ends before N): give them their own CTAs
  pp.fill_ctas = ((HOOK == kHookScores || HOOK == kHookScores16) && p.causal && p.p_seq + p.m_begin + 128 < p.N) ? 1 : 0;
  const int nslots = pp.fill_ctas ? 2 * ncb : ncb;
  // the causal round-robin walk (down from the CTA's last key tile) is the reverse order: take its cheaper index form
  if (pp.schedule == kRoundRobin && pp.causal) pp.schedule = kReverse;
  if (pp.n_splits < 1) pp.n_splits = 1;
  if (pp.n_splits == 1) pp.tiles_per_split = (p.N + BN - 1) / BN;
  dim3 grid = pp.lpt_order ? dim3(p.Hq, p.B * pp.n_splits, nslots) : dim3(nslots, p.Hq, p.B * pp.n_splits);
  // Tensor-bound launches with more items than SMs: one persistent CTA per SM walks a work list.
  WorkList wl_persist;
  const WorkList* wl = &plain_work_list();
  if constexpr (!SPLIT && (HOOK == kHookNone || HOOK == kHookRowSum || HOOK == kHookColPart)) {
    if (pp.n_splits == 1 && !pp.fill_ctas && persistent_allowed() &&
        make_work_list(pp, grid, L::kRows, sm_count(), &wl_persist)) {
      wl = &wl_persist;
      grid = dim3(sm_count(), 1, 1);
    }
  }
  // Programmatic stream serialization: this launch may begin (CTA placement, barrier and TMEM set-up)
  // while the previous kernel of the stream drains; the kernel waits before any global access.
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(NTHREADS, 1, 1);
  cfg.dynamicSmemBytes = L::alloc;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int* status_word = tc_status_word();
  const cudaError_t e = cudaLaunchKernelEx(&cfg, tc_fwd_kernel<T, D, HOOK, SPLIT, DROP>, maps, pp, *wl, status_word);
  count_launch();
  return e != cudaSuccess ? e : cudaGetLastError();
}

// FAWS_PERSISTENT=0 in the environment keeps every launch a plain one (tests, ablations).
bool persistent_allowed() {
  static const bool on = [] {
    const char* e = std::getenv("FAWS_PERSISTENT");
    return e == nullptr || e[0] != '0';
  }();
  return on;
}

// Few CTAs (less than two per SM with 256-row CTAs): the launch is bound by the longest chain of
// dependent key tiles, so use 128-row CTAs whose two warpgroups split the key tiles.
// FAWS_SPLIT_KV=0/1 in the environment overrides the choice (tests, ablations).
bool use_split_kv(const FwdParams& p) {
  static const int forced = [] {
    const char* e = std::getenv("FAWS_SPLIT_KV");
    return e == nullptr ? -1 : (e[0] == '1' ? 1 : 0);
  }();
  if (forced >= 0) return forced == 1;
  const int sms = sm_count();
  const long long ctas256 = (long long)((p.m_end - p.m_begin + 255) / 256) * p.Hq * p.B;
  return ctas256 < 2LL * sms;
}

template <typename T, int D, int HOOK>
cudaError_t launch_fwd_h(const TcMaps& maps, const FwdParams& p, cudaStream_t s) {
  // Score-materialising causal launches are bound by their stores, not by the chain of key
  // tiles: measured, the 256-row CTAs (half as many set-ups) are faster there.
  if constexpr (HOOK != kHookScores16 && HOOK != kHookScratch) {
    // dropout: 256-row CTAs only (the mask generation, not the chain of key tiles, bounds it)
    if (p.drop.p > 0.f) return launch_fwd_s<T, D, HOOK, false, true>(maps, p, s);
  }
  const bool store_bound = (HOOK == kHookScores || HOOK == kHookScores16) && p.causal;
  static const bool forced = std::getenv("FAWS_SPLIT_KV") != nullptr;
  const bool split = use_split_kv(p) && (forced || !store_bound);
  return split ? launch_fwd_s<T, D, HOOK, true>(maps, p, s) : launch_fwd_s<T, D, HOOK, false>(maps, p, s);
}

template <typename T, int D>
cudaError_t launch_fwd_t(const TcMaps& maps, const FwdParams& p, cudaStream_t s) {
  if (p.scores != nullptr)
    return p.scores_f32 ? launch_fwd_h<T, D, kHookScores>(maps, p, s) : launch_fwd_h<T, D, kHookScores16>(maps, p, s);
  if (p.row_sum != nullptr) return launch_fwd_h<T, D, kHookRowSum>(maps, p, s);
  if (p.col_partial != nullptr) return launch_fwd_h<T, D, kHookColPart>(maps, p, s);
  if (p.s_scratch != nullptr) return launch_fwd_h<T, D, kHookScratch>(maps, p, s);
  return launch_fwd_h<T, D, kHookNone>(maps, p, s);
}

}  // namespace

bool tc_fwd_supported(const FwdParams& p, int dtype) {
  (void)dtype;
  if (p.D != 64 && p.D != 128) return false;
  if (p.drop.p > 0.f && (p.s_scratch != nullptr || (p.scores != nullptr && !p.scores_f32)))
    return false;  // no dropout variant of the scratch and 16-bit-score hooks: CUDA-core kernels
  if (!(p.sm_scale > 0.f)) return false;  // the row max is taken on unscaled scores
  if (!device_is_sm100() || get_encode() == nullptr) return false;
  if (p.m_begin % BM != 0 || p.m_end <= p.m_begin) return false;
  if (!ok16(p.q, p.q_sb, p.q_sh, p.q_ss) || !ok16(p.k, p.k_sb, p.k_sh, p.k_ss) ||
      !ok16(p.v, p.v_sb, p.v_sh, p.v_ss) || !ok16(p.o, p.o_sb, p.o_sh, p.o_ss))
    return false;
  if (p.scores != nullptr) {  // TMA store rows must start on 16-byte boundaries
    if (p.N % (p.scores_f32 ? 4 : 8) != 0 || reinterpret_cast<uintptr_t>(p.scores) % 16 != 0) return false;
  }
  if (p.s_scratch != nullptr) {
    if (p.scores != nullptr) return false;
    if (p.split % 32 != 0 || reinterpret_cast<uintptr_t>(p.s_scratch) % 16 != 0) return false;
  }
  return true;
}

cudaError_t launch_tc_fwd(const FwdParams& p, int dtype, cudaStream_t s) {
  TcMaps maps;
  const int q_rows = p.m_end - p.m_begin;
  const char* qbase = static_cast<const char*>(p.q) + (int64_t)p.m_begin * p.q_ss * 2;
  if (!make_map_bhsd(&maps.q, qbase, p.D, q_rows, p.Hq, p.B, p.q_ss, p.q_sh, p.q_sb, 128) ||
      !make_map_bhsd(&maps.k, p.k, p.D, p.N, p.Hk, p.B, p.k_ss, p.k_sh, p.k_sb, 128) ||
      !make_map_bhsd(&maps.v, p.v, p.D, p.N, p.Hk, p.B, p.v_ss, p.v_sh, p.v_sb, 128))
    return cudaErrorInvalidValue;
  const char* obase = static_cast<const char*>(p.o) + (int64_t)p.m_begin * p.o_ss * 2;
  // split-KV: p.o is the (B, Hq * n_splits, M, D) buffer of partial results
  const int o_heads = p.Hq * (p.n_splits > 1 ? p.n_splits : 1);
  if (!make_map_bhsd(&maps.o, obase, p.D, q_rows, o_heads, p.B, p.o_ss, p.o_sh, p.o_sb, 32)) return cudaErrorInvalidValue;
  maps.st = maps.q;
  if (p.scores != nullptr) {
    const int esize = p.scores_f32 ? 4 : 2;
    char* base = static_cast<char*>(p.scores) + (int64_t)p.m_begin * p.N * esize;
    if (!make_map_store_f32(&maps.st, base, p.N, q_rows, p.N, (int64_t)p.M * p.N, p.B * p.Hq, esize))
      return cudaErrorInvalidValue;
  } else if (p.s_scratch != nullptr) {
    const int rows = p.m_end - p.split;  // rows of the cross region inside the window
    if (rows > 0 &&
        !make_map_store_f32(&maps.st, p.s_scratch, p.split, rows, p.split, (int64_t)(p.M - p.split) * p.split,
                            p.B * p.Hq))
      return cudaErrorInvalidValue;
  }
  if (dtype == FAWS_FP16)
    return p.D == 128 ? launch_fwd_t<__half, 128>(maps, p, s) : launch_fwd_t<__half, 64>(maps, p, s);
  return p.D == 128 ? launch_fwd_t<__nv_bfloat16, 128>(maps, p, s) : launch_fwd_t<__nv_bfloat16, 64>(maps, p, s);
}

namespace {
// Exercises the give-up path of mbar_wait: one thread waits (bounded, about a millisecond) on an
// mbarrier nobody arrives at, the wait runs out, the CTA raises the status word and returns.
__global__ void wait_give_up_kernel(int* __restrict__ status, long long limit_cycles) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait(&bar, 0, &abort_flag, limit_cycles);
  __syncthreads();
  if (abort_flag != 0 && threadIdx.x == 0 && status != nullptr) atomicExch(status, 1);
}
}  // namespace

cudaError_t launch_wait_give_up(cudaStream_t s) {
  int* status_word = tc_status_word();
  if (status_word == nullptr) return cudaErrorInvalidDevice;
  wait_give_up_kernel<<<1, 32, 0, s>>>(status_word, 2000000ll);
  count_launch();
  return cudaGetLastError();
}

int tc_read_status(int reset) {
  int* word = tc_status_word();
  if (word == nullptr) return -1;
  int v = 0;
  if (cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (reset && v != 0) cudaMemset(word, 0, sizeof(int));
  return v;
}

// Whether the kernel should walk the G heads of a kv head inside one CTA (output already group
// summed) or run one CTA per query head followed by a group-sum kernel.  The latter gives G times
// more CTAs, which matters for causal problems where the key tiles' work is very uneven.
bool tc_colsoftmax_group_in_kernel(const ColSoftmaxParams& p) {
  if (p.G == 1) return true;
  const int sms = sm_count();
  const long long ctas = (long long)((p.n_end + CS_KT * BN - 1) / (CS_KT * BN)) * p.Hk * p.B;
  return !(p.causal && ctas < 8LL * sms) && ctas >= 2LL * sms;
}

bool tc_colsoftmax_supported(const ColSoftmaxParams& p, int dtype) {
  (void)dtype;
  if (p.D != 64 && p.D != 128) return false;
  if (p.s_scratch != nullptr) return false;  // the buffered pass reads stored scores, no MMA
  if (p.drop.p > 0.f) return false;
  if (p.m_begin % BM != 0 || !(p.sm_scale > 0.f)) return false;
  if (!device_is_sm100() || get_encode() == nullptr) return false;
  if (!ok16(p.q, p.q_sb, p.q_sh, p.q_ss) || !ok16(p.k, p.k_sb, p.k_sh, p.k_ss)) return false;
  return p.n_end > 0;
}

namespace {
// -L_i*log2e into the tile-padded array the key-major kernel copies from; -inf for rows that do not
// contribute (outside [i_lo, m_end), padding, or without a visible key).
__global__ void negl_prep_kernel(const float* __restrict__ L, float* __restrict__ out, int M, int m_pad, int i_lo,
                                 int m_end, long long total) {
  griddep_wait();  // L comes from the forward pass before this launch
  griddep_launch_dependents();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long bh = idx / m_pad;
  const int i = (int)(idx - bh * m_pad);
  float v = FAWS_NEG_INF;
  if (i >= i_lo && i < m_end) {
    const float Li = L[bh * M + i];
    if (Li != FAWS_NEG_INF) v = -Li * kLog2e;
  }
  out[idx] = v;
}

cudaError_t launch_negl_prep(const ColSoftmaxParams& p, cudaStream_t s) {
  const long long total = (long long)p.B * p.Hq * p.m_pad;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)((total + 255) / 256), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.after_forward ? 1 : 0;
  const float* L = p.L;
  float* out = p.negl_pad;
  const int i_lo = p.i_begin > p.m_begin ? p.i_begin : p.m_begin;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, negl_prep_kernel, L, out, p.M, p.m_pad, i_lo, p.m_end, total);
  count_launch();
  return e != cudaSuccess ? e : cudaGetLastError();
}

template <typename T, int D>
cudaError_t launch_cs_t(const CsMaps& maps, const ColSoftmaxParams& p, int heads_per_cta, cudaStream_t s) {
  using L = CsSmem<D>;
  static PerDeviceOnce attr_once;
  if (cudaError_t e = set_max_smem_once(attr_once, tc_colsoftmax_kernel<T, D>, L::alloc); e != cudaSuccess) return e;
  const int nkt = (p.n_end + CS_KT * BN - 1) / (CS_KT * BN);  // CTAs along the keys: CS_KT key tiles each
  dim3 grid = p.causal ? dim3(p.Hq / heads_per_cta, p.B, nkt) : dim3(nkt, p.Hq / heads_per_cta, p.B);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(CS_THREADS, 1, 1);
  cfg.dynamicSmemBytes = L::alloc;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.after_forward ? 1 : 0;  // q and k must not come from the previous kernel
  int* status_word = tc_status_word();
  const cudaError_t e = cudaLaunchKernelEx(&cfg, tc_colsoftmax_kernel<T, D>, maps, p, heads_per_cta, status_word);
  count_launch();
  return e != cudaSuccess ? e : cudaGetLastError();
}
}  // namespace

// group_sum != 0: one CTA walks the G query heads of a kv head and p.out is (B,Hk,n_end);
// otherwise one CTA per query head and p.out is (B,Hq,n_end).
cudaError_t launch_tc_colsoftmax(const ColSoftmaxParams& p, int dtype, int group_sum, cudaStream_t s) {
  CsMaps maps;
  if (!make_map_bhsd(&maps.q, p.q, p.D, p.m_end, p.Hq, p.B, p.q_ss, p.q_sh, p.q_sb, 128) ||
      !make_map_bhsd(&maps.k, p.k, p.D, p.N, p.Hk, p.B, p.k_ss, p.k_sh, p.k_sb, 128))
    return cudaErrorInvalidValue;
  const int hpc = group_sum ? p.G : 1;
  if (p.negl_pad != nullptr) {
    if (cudaError_t e = launch_negl_prep(p, s); e != cudaSuccess) return e;
  }
  if (dtype == FAWS_FP16)
    return p.D == 128 ? launch_cs_t<__half, 128>(maps, p, hpc, s) : launch_cs_t<__half, 64>(maps, p, hpc, s);
  return p.D == 128 ? launch_cs_t<__nv_bfloat16, 128>(maps, p, hpc, s)
                    : launch_cs_t<__nv_bfloat16, 64>(maps, p, hpc, s);
}

}  // namespace faws
