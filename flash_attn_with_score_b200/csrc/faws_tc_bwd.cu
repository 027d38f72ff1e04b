// tcgen05 backward kernels of attention() (sm_100a): dQ, dK, dV from q, k, v, out, dout and the
// saved log-normaliser L.
//
// Same split as the reference (flash.py:172-261): a pre-pass (delta_i = sum_d out_id dout_id,
// flash.py:532-577), a key-major kernel for dK and dV (flash.py:581-754) and a query-major kernel
// for dQ (flash.py:758-918).  Both kernels are one template, tc_bwd_kernel<T, D, KEY_MAJOR>:
//
//   the CTA owns 128 rows of two *stationary* tiles X, Y and streams tile pairs (A_u, B_u):
//                       X   Y      A_u         B_u           accumulators
//     key-major         K   V      Q tile u    dout tile u   dV += P^T.dout,  dK += dS^T.Q
//     query-major       Q   dout   K tile u    V tile u      dQ += dS.K
//   per streamed pair:  S' = X.A^T and dP' = Y.B^T (fp32, TMEM; rows = the owned index), then
//   P' = exp(S'*scale - L), dS' = P' * (dP' - delta) in registers, written back to TMEM as 16-bit
//   operands over S' and dP', then the accumulating MMAs (A operand from TMEM).
//
// The 128 streamed rows are processed as two halves of 64 with their own TMEM columns, each by
// its own consumer warpgroup, so the tensor pipe works on one half while the other is in registers.
// (Measured alternatives, all slower on the same box: four parts of 32 with four consumer
// warpgroups, 1.5-1.7x; S' and dP' as full 128-column MMAs handed back in four chunks, 1.15-1.25x;
// separate barriers for S' and dP' plus a hand-off per 32-column chunk, 1.1-1.2x.)
// Warp roles (12 warps): warp 0 TMA producer (X, Y once, then a 2-stage ring of (A, B) pairs and,
// key-major, the L / delta vectors of the streamed query tile), warp 1 TMEM allocation and the
// MMA-issuing lane, warps 4-7 / 8-11 consumers of half 0 / 1 (thread = owned row = TMEM lane).
// Deterministic: every output element is written once, by one CTA, in a fixed order; with GQA the
// key-major kernel writes per-query-head dK / dV and a second kernel adds the G heads in order.
// Out-of-range rows need no predicates: TMA zero-fills the loads (a zero Q / dout / K / V row
// contributes nothing to any accumulator) and clips the stores.  Every mbarrier wait is bounded.
#include <cuda.h>

#include <type_traits>

#include "faws_internal.cuh"
#include "faws_tc_host.cuh"
#include "faws_tc_ptx.cuh"

namespace faws {
namespace {
using namespace ptx;

constexpr int BT = 128;        // tile edge (owned rows and streamed rows)
constexpr int HALF = 64;       // streamed rows per consumer warpgroup
constexpr int NTHREADS = 384;
constexpr int NSTAGE = 2;
constexpr int TMEM_COLS = 512;
constexpr int REGS_LAUNCH = 168;
constexpr int REGS_AUX = 88;
constexpr int REGS_CONSUMER = ((REGS_LAUNCH * NTHREADS - 128 * REGS_AUX) / 256) & ~7;
static_assert(128 * REGS_AUX + 256 * REGS_CONSUMER <= REGS_LAUNCH * NTHREADS, "setmaxnreg would block");
constexpr float kLog2e = 1.4426950408889634f;

// TMEM columns: S'_0, S'_1, dP'_0, dP'_1 (64 fp32 columns each), then the accumulators.
constexpr uint32_t COL_S = 0, COL_DP = 128, COL_ACC = 256;

template <int D>
struct BwSmem {
  static constexpr int kTile = 128 * D * 2;
  static constexpr int kSub = 128 * 128;  // one 64-element-wide sub-tile: 128 rows x 128 B
  static constexpr int x_off = 0;
  static constexpr int y_off = kTile;
  static constexpr int ring_off = 2 * kTile;                    // NSTAGE x (A tile, B tile)
  static constexpr int vec_off = ring_off + NSTAGE * 2 * kTile; // NSTAGE x (128 -L*log2e, 128 delta) floats
  static constexpr int bar_off = vec_off + NSTAGE * 1024;
  static constexpr int total = bar_off + 256;
  static constexpr int alloc = total + 1024;
};

struct BwBars {
  uint64_t x_full;
  uint64_t r_full[NSTAGE], r_empty[NSTAGE];
  uint64_t s_full[2];   // per half: S' and dP' written by the tensor pipe
  uint64_t p_ready[2];  // per half: P' and dS' written by its 128 consumer threads
  uint64_t acc_done;
  uint32_t tmem_base;
  int abort_flag;
};

struct BwMaps {
  CUtensorMap x, y, a, b;  // loads, 128-row boxes
  CUtensorMap o0, o1;      // stores, 32-row boxes: key-major dV, dK; query-major dQ (o1 unused)
};

struct BwTcParams {
  int Hq, G, M, N, p_seq, causal, Mpad;
  float sm_scale;
  const float* negl2;  // (B,Hq,Mpad): -L_i * log2(e), 0 for padded rows and rows without a visible key
  const float* delta;  // (B,Hq,Mpad): sum_d out_id * dout_id, 0 for padded rows
};

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <typename T, int D, bool KM>
__global__ void __launch_bounds__(NTHREADS, 1)
tc_bwd_kernel(const __grid_constant__ BwMaps maps, const BwTcParams p, int* __restrict__ status) {
  using L = BwSmem<D>;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  BwBars* bars = reinterpret_cast<BwBars*>(smem + L::bar_off);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Heaviest work first in launch order: key-major, the first key tiles see the most queries when
  // causal; query-major, the last query tiles see the most keys.
  const int own_tiles = (int)gridDim.z;
  const int own_tile = KM ? (int)blockIdx.z : (p.causal ? own_tiles - 1 - (int)blockIdx.z : (int)blockIdx.z);
  const int h = blockIdx.x, b = blockIdx.y;
  const int hk = h / p.G;
  const int own0 = own_tile * BT;  // first owned row: key n0 (key-major) or query i0 (query-major)

  // streamed tiles [u0, u0 + nu)
  int u0 = 0, nu;
  if (KM) {
    if (p.causal) u0 = max(0, own0 - p.p_seq) / BT;  // first query tile with a row that sees key own0
    nu = max(0, (p.M + BT - 1) / BT - u0);
  } else {
    int hi = p.N;
    if (p.causal) hi = max(0, min(p.N, p.p_seq + min(own0 + BT, p.M)));
    nu = (hi + BT - 1) / BT;
  }

  if (threadIdx.x == 0) {
    mbar_init(&bars->x_full, 1);
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(&bars->r_full[s], 1);
      mbar_init(&bars->r_empty[s], 1);
    }
    for (int e = 0; e < 2; ++e) {
      mbar_init(&bars->s_full[e], 1);
      mbar_init(&bars->p_ready[e], 128);
    }
    mbar_init(&bars->acc_done, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&maps.x);
    prefetch_tmap(&maps.y);
    prefetch_tmap(&maps.a);
    prefetch_tmap(&maps.b);
    prefetch_tmap(&maps.o0);
    if (KM) prefetch_tmap(&maps.o1);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  const int64_t vec_row = ((int64_t)b * p.Hq + h) * p.Mpad;  // this head's row of the padded L / delta arrays

  if (warp < 4) {
    reg_dealloc<REGS_AUX>();
    if (warp == 0 && lane == 0 && nu > 0) {
      // ---------------------------------------------------------- TMA producer
      const int x_head = KM ? hk : h;
      mbar_arrive_expect_tx(&bars->x_full, 2 * L::kTile);
      for (int c = 0; c < D / 64; ++c) {
        tma_load_4d(smem + L::x_off + c * L::kSub, &maps.x, &bars->x_full, c * 64, own0, x_head, b);
        tma_load_4d(smem + L::y_off + c * L::kSub, &maps.y, &bars->x_full, c * 64, own0, x_head, b);
      }
      const int a_head = KM ? h : hk;
      for (int u = 0; u < nu; ++u) {
        const int s = u % NSTAGE, use = u / NSTAGE;
        if (use > 0 && !mbar_wait(&bars->r_empty[s], (use - 1) & 1, abort_flag)) break;
        const int row0 = (u0 + u) * BT;
        mbar_arrive_expect_tx(&bars->r_full[s], 2 * L::kTile + (KM ? 1024 : 0));
        unsigned char* st = smem + L::ring_off + s * 2 * L::kTile;
        for (int c = 0; c < D / 64; ++c) {
          tma_load_4d(st + c * L::kSub, &maps.a, &bars->r_full[s], c * 64, row0, a_head, b);
          tma_load_4d(st + L::kTile + c * L::kSub, &maps.b, &bars->r_full[s], c * 64, row0, a_head, b);
        }
        if (KM) {
          bulk_load_1d(smem + L::vec_off + s * 1024, p.negl2 + vec_row + row0, 512, &bars->r_full[s]);
          bulk_load_1d(smem + L::vec_off + s * 1024 + 512, p.delta + vec_row + row0, 512, &bars->r_full[s]);
        }
      }
    } else if (warp == 1 && nu > 0) {
      // ---------------------------------------------------------- MMA issuer (whole warp loops, one lane issues)
      constexpr int kFmt = std::is_same<T, __half>::value ? 0 : 1;
      constexpr uint32_t idesc1 = make_idesc_f16(128, HALF, kFmt, 0, 0);  // S', dP': 128 x 64, K = D
      constexpr uint32_t idesc2 = make_idesc_f16(128, D, kFmt, 0, 1);     // accumulators: 128 x D, K = 64
      const uint64_t x_desc = make_desc_sw128(smem_u32(smem + L::x_off), 16, 1024);
      const uint64_t y_desc = make_desc_sw128(smem_u32(smem + L::y_off), 16, 1024);
      const uint64_t ak_desc0 = make_desc_sw128(smem_u32(smem + L::ring_off), 16, 1024);          // A, B as K-major
      const uint64_t am_desc0 = make_desc_sw128(smem_u32(smem + L::ring_off), L::kSub, 1024);     // A, B as MN-major
      // S'_e = X . A_e^T and dP'_e = Y . B_e^T for the 64 streamed rows of half e in ring stage s
      auto issue_mma1 = [&](int e, int s) {
        const uint64_t a_rows = ak_desc0 + (uint64_t)((s * 2 * L::kTile + e * HALF * 128) >> 4);
        const uint64_t b_rows = a_rows + (uint64_t)(L::kTile >> 4);
        const uint32_t d_s = tmem_base + COL_S + (uint32_t)(e * HALF);
        const uint32_t d_dp = tmem_base + COL_DP + (uint32_t)(e * HALF);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t off = (uint64_t)(((kk >> 2) * L::kSub + (kk & 3) * 32) >> 4);
            if (kk == 0) mma_ss(d_s, x_desc + off, a_rows + off, idesc1, 0u);
            else mma_ss_acc(d_s, x_desc + off, a_rows + off, idesc1);
          }
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t off = (uint64_t)(((kk >> 2) * L::kSub + (kk & 3) * 32) >> 4);
            if (kk == 0) mma_ss(d_dp, y_desc + off, b_rows + off, idesc1, 0u);
            else mma_ss_acc(d_dp, y_desc + off, b_rows + off, idesc1);
          }
          mma_commit(&bars->s_full[e]);
        }
        __syncwarp();
      };
      // accumulators (+)= the 16-bit operands of half e (in TMEM over S'_e / dP'_e) times the 64 streamed rows
      auto issue_mma2 = [&](int e, int s, bool first) {
        const uint64_t a_tile = am_desc0 + (uint64_t)((s * 2 * L::kTile) >> 4);
        const uint64_t b_tile = a_tile + (uint64_t)(L::kTile >> 4);
        const uint32_t t_p = tmem_base + COL_S + (uint32_t)(e * HALF);    // P'_e: 64 values = 32 columns
        const uint32_t t_ds = tmem_base + COL_DP + (uint32_t)(e * HALF);  // dS'_e
        const uint32_t acc0 = tmem_base + COL_ACC, acc1 = tmem_base + COL_ACC + (uint32_t)D;
        if (elect_one()) {
#pragma unroll
          for (int k4 = 0; k4 < HALF / 16; ++k4) {
            const uint64_t off = (uint64_t)(((e * 4 + k4) * 16 * 128) >> 4);  // 16 streamed rows per K-step
            const uint32_t accumulate = (first && k4 == 0) ? 0u : 1u;
            if (KM) {
              mma_ts(acc0, t_p + (uint32_t)(k4 * 8), b_tile + off, idesc2, accumulate);   // dV += P^T . dout
              mma_ts(acc1, t_ds + (uint32_t)(k4 * 8), a_tile + off, idesc2, accumulate);  // dK += dS^T . Q
            } else {
              mma_ts(acc0, t_ds + (uint32_t)(k4 * 8), a_tile + off, idesc2, accumulate);  // dQ += dS . K
            }
          }
        }
        __syncwarp();
      };
      auto commit = [&](uint64_t* bar) {
        if (elect_one()) mma_commit(bar);
        __syncwarp();
      };
      bool ok = mbar_wait(&bars->x_full, 0, abort_flag);
      if (ok) ok = mbar_wait(&bars->r_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_mma1(0, 0);
        issue_mma1(1, 0);
      }
      for (int u = 0; ok && u < nu; ++u) {
        const int s = u % NSTAGE;
        const bool more = u + 1 < nu;
        const int s1 = (u + 1) % NSTAGE;
        if (!(ok = mbar_wait(&bars->p_ready[0], u & 1, abort_flag))) break;
        tc_fence_after();
        issue_mma2(0, s, u == 0);
        if (more) {
          if (!(ok = mbar_wait(&bars->r_full[s1], ((u + 1) / NSTAGE) & 1, abort_flag))) break;
          tc_fence_after();
          issue_mma1(0, s1);  // S'_0 of the next pair while half 1 of this one is still in registers
        }
        if (!(ok = mbar_wait(&bars->p_ready[1], u & 1, abort_flag))) break;
        tc_fence_after();
        issue_mma2(1, s, false);
        commit(&bars->r_empty[s]);
        if (more) issue_mma1(1, s1);
      }
      if (ok) commit(&bars->acc_done);
    }
  } else {
    reg_alloc<REGS_CONSUMER>();
    // ------------------------------------------------------------ consumers: thread = owned row
    const int e = (warp - 4) >> 2;  // half of the streamed rows this warpgroup handles
    const int lg = warp & 3;
    const int row = lg * 32 + lane;
    const int own = own0 + row;  // key j (key-major) or query i (query-major)
    const uint32_t t_lane = tmem_base + ((uint32_t)(lg * 32) << 16);
    const uint32_t t_s = t_lane + COL_S + (uint32_t)(e * HALF);
    const uint32_t t_dp = t_lane + COL_DP + (uint32_t)(e * HALF);
    const float c2 = p.sm_scale * kLog2e;
    float my_nl = 0.f, my_dl = 0.f;  // query-major: this thread's query
    if (!KM) {
      my_nl = p.negl2[vec_row + own];  // own < Mpad always
      my_dl = p.delta[vec_row + own];
    }
    bool alive = true;
    for (int u = 0; u < nu; ++u) {
      if (!mbar_wait(&bars->s_full[e], u & 1, abort_flag)) { alive = false; break; }
      tc_fence_after();
      uint32_t sv[HALF], dv[HALF];
      tmem_ld32(t_s, reinterpret_cast<uint32_t(&)[32]>(sv[0]));
      tmem_ld32(t_s + 32, reinterpret_cast<uint32_t(&)[32]>(sv[32]));
      tmem_ld32(t_dp, reinterpret_cast<uint32_t(&)[32]>(dv[0]));
      tmem_ld32(t_dp + 32, reinterpret_cast<uint32_t(&)[32]>(dv[32]));
      tmem_wait_ld();
      const int str0 = (u0 + u) * BT + e * HALF;  // first streamed row of this half
      // causal: (query i, key j) is visible iff j <= i + p_seq.  Column x of the half is streamed row
      // str0 + x.  Key-major (own = j, streamed = i): visible iff x >= own - p_seq - str0.
      // Query-major (own = i, streamed = j): visible iff x <= own + p_seq - str0.
      int x_lo = 0, x_hi = HALF - 1;
      if (p.causal) {
        if (KM) x_lo = own - p.p_seq - str0;
        else x_hi = own + p.p_seq - str0;
      }
      const float* vl = reinterpret_cast<const float*>(smem + L::vec_off + (u % NSTAGE) * 1024) + e * HALF;
      const float* vd = vl + 128;
      uint32_t pk[HALF / 2], dk[HALF / 2];
#pragma unroll
      for (int x = 0; x < HALF; x += 4) {
        float nl[4], dl[4];
        if (KM) {
          const float4 a = *reinterpret_cast<const float4*>(vl + x);
          const float4 d4 = *reinterpret_cast<const float4*>(vd + x);
          nl[0] = a.x; nl[1] = a.y; nl[2] = a.z; nl[3] = a.w;
          dl[0] = d4.x; dl[1] = d4.y; dl[2] = d4.z; dl[3] = d4.w;
        } else {
#pragma unroll
          for (int y = 0; y < 4; ++y) { nl[y] = my_nl; dl[y] = my_dl; }
        }
        float pr[4], ds[4];
#pragma unroll
        for (int y = 0; y < 4; ++y) {
          const bool vis = (x + y >= x_lo) && (x + y <= x_hi);
          const float pe = fast_exp2(fmaf(__uint_as_float(sv[x + y]), c2, nl[y]));
          pr[y] = vis ? pe : 0.f;
          ds[y] = pr[y] * (__uint_as_float(dv[x + y]) - dl[y]);
        }
        pk[x / 2] = pack2<T>(pr[0], pr[1]);
        pk[x / 2 + 1] = pack2<T>(pr[2], pr[3]);
        dk[x / 2] = pack2<T>(ds[0], ds[1]);
        dk[x / 2 + 1] = pack2<T>(ds[2], ds[3]);
      }
      if (KM) tmem_st32(t_s, pk);  // P' is an operand only where dV is formed
      tmem_st32(t_dp, dk);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&bars->p_ready[e]);
    }

    // ---- epilogue: accumulators -> 16-bit -> swizzled smem -> TMA store (clips at the tensor's edge)
    if (alive && nu > 0) {
      if (!mbar_wait(&bars->acc_done, 0, abort_flag)) alive = false;
      tc_fence_after();
    }
    if (alive) {
      // Every MMA has completed, so the ring is free for staging: 32 rows x 64 columns (4 KB) per (warp, sub-tile).
      unsigned char* ost = smem + L::ring_off + (warp - 4) * (32 * D * 2);
      // key-major: warpgroup 0 stores dV (acc0), warpgroup 1 stores dK (acc1, times sm_scale);
      // query-major: dQ (acc0, times sm_scale), warpgroup w takes the 64-column sub-tiles w, w + 2, ...
      const uint32_t t_acc = t_lane + COL_ACC + (KM ? (uint32_t)(e * D) : 0u);
      const float oscale = (KM && e == 0) ? 1.f : p.sm_scale;
      const int sub_first = KM ? 0 : e, sub_step = KM ? 1 : 2;
      for (int sub = sub_first; sub < D / 64; sub += sub_step) {
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t ro[32];
          if (nu > 0) {
            tmem_ld32(t_acc + (uint32_t)(sub * 64 + c * 32), ro);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int x = 0; x < 32; ++x) ro[x] = 0u;  // no streamed tile at all: the gradient rows are zero
          }
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w;
            w.x = pack2<T>(__uint_as_float(ro[g * 8 + 0]) * oscale, __uint_as_float(ro[g * 8 + 1]) * oscale);
            w.y = pack2<T>(__uint_as_float(ro[g * 8 + 2]) * oscale, __uint_as_float(ro[g * 8 + 3]) * oscale);
            w.z = pack2<T>(__uint_as_float(ro[g * 8 + 4]) * oscale, __uint_as_float(ro[g * 8 + 5]) * oscale);
            w.w = pack2<T>(__uint_as_float(ro[g * 8 + 6]) * oscale, __uint_as_float(ro[g * 8 + 7]) * oscale);
            const int cc = c * 4 + g;  // 16-byte chunk inside the 64-column sub-tile
            *reinterpret_cast<uint4*>(ost + sub * 4096 + lane * 128 + ((cc ^ (lane & 7)) << 4)) = w;
          }
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const CUtensorMap* om = (KM && e == 1) ? &maps.o1 : &maps.o0;
        for (int sub = sub_first; sub < D / 64; sub += sub_step)
          tma_store_4d(om, ost + sub * 4096, sub * 64, own0 + lg * 32, h, b);
        tma_store_commit();
        tma_store_wait<0>();
      }
    }
  }

  // ------------------------------------------------------------ common exit
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && status != nullptr) atomicExch(status, 1);
    for (int w = 0; w < 50; ++w) __nanosleep(20000);  // let copies in flight land before the smem goes away
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Pre-pass: delta_i = sum_d out_id * dout_id and -L_i * log2(e), both into arrays padded to whole
// 128-row tiles (zeros in the padding), so that the kernels can fetch a tile's 128 values with one
// aligned bulk copy.  One warp per (padded) row.
template <typename T>
__global__ void bwd_prep_kernel(BwdParams p, float* negl2, float* delta, int Mpad) {
  const int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (int64_t)p.B * p.Hq * Mpad) return;
  const int i = (int)(w % Mpad);
  const int64_t bh = w / Mpad;
  const int h = (int)(bh % p.Hq), b = (int)(bh / p.Hq);
  float sum = 0.f, nl = 0.f;
  if (i < p.M) {
    const T* o = reinterpret_cast<const T*>(p.o) + b * p.o_sb + h * p.o_sh + (int64_t)i * p.o_ss;
    const T* g = reinterpret_cast<const T*>(p.dout) + b * p.do_sb + h * p.do_sh + (int64_t)i * p.do_ss;
    for (int d = lane * 2; d < p.D; d += 64) {
      float2 a, c;
      if constexpr (std::is_same<T, __half>::value) {
        a = __half22float2(*reinterpret_cast<const __half2*>(o + d));
        c = __half22float2(*reinterpret_cast<const __half2*>(g + d));
      } else {
        a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o + d));
        c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(g + d));
      }
      sum = fmaf(a.x, c.x, fmaf(a.y, c.y, sum));
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
    const float Li = p.L[bh * p.M + i];
    nl = (Li == __int_as_float(0xff800000)) ? 0.f : -Li * kLog2e;  // no visible key: every weight is masked anyway
  }
  if (lane == 0) {
    delta[w] = sum;
    negl2[w] = nl;
  }
}

// out[b,hk,j,:] = sum over the G query heads of the kv head, in head order, of part[b,hk*G+g,j,:]
template <typename T>
__global__ void bwd_group_sum_kernel(const T* __restrict__ part, T* out, int64_t o_sb, int64_t o_sh, int64_t o_ss,
                                     int B, int Hk, int G, int N, int D) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per 2 elements
  const int half_d = D / 2;
  if (idx >= (int64_t)B * Hk * N * half_d) return;
  const int d2 = (int)(idx % half_d);
  const int64_t r = idx / half_d;
  const int j = (int)(r % N);
  const int64_t bk = r / N;
  const int hk = (int)(bk % Hk), b = (int)(bk / Hk);
  float s0 = 0.f, s1 = 0.f;
  for (int g = 0; g < G; ++g) {
    const T* src = part + ((((int64_t)b * Hk + hk) * G + g) * N + j) * D + d2 * 2;
    float2 v;
    if constexpr (std::is_same<T, __half>::value) v = __half22float2(*reinterpret_cast<const __half2*>(src));
    else v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src));
    s0 += v.x;
    s1 += v.y;
  }
  const uint32_t w = pack2<T>(s0, s1);
  *reinterpret_cast<uint32_t*>(out + b * o_sb + hk * o_sh + (int64_t)j * o_ss + d2 * 2) = w;
}

int mpad_of(int M) { return (M + BT - 1) / BT * BT; }

template <typename T, int D>
cudaError_t launch_bwd_td(const BwdParams& p, cudaStream_t s) {
  using L = BwSmem<D>;
  static PerDeviceOnce once_km, once_qm;
  cudaError_t e;
  if ((e = set_max_smem_once(once_km, tc_bwd_kernel<T, D, true>, L::alloc)) != cudaSuccess) return e;
  if ((e = set_max_smem_once(once_qm, tc_bwd_kernel<T, D, false>, L::alloc)) != cudaSuccess) return e;
  const int Mpad = mpad_of(p.M);
  const size_t vec_bytes = ((size_t)p.B * p.Hq * Mpad * 4 + 255) & ~size_t(255);
  float* negl2 = p.delta;  // workspace: [-L*log2e | delta | per-head dK | per-head dV]
  float* delta = reinterpret_cast<float*>(reinterpret_cast<char*>(p.delta) + vec_bytes);
  char* part = reinterpret_cast<char*>(p.delta) + 2 * vec_bytes;
  const size_t part_bytes = ((size_t)p.B * p.Hq * p.N * p.D * 2 + 255) & ~size_t(255);
  {
    const int64_t warps = (int64_t)p.B * p.Hq * Mpad;
    bwd_prep_kernel<T><<<(unsigned)((warps * 32 + 255) / 256), 256, 0, s>>>(p, negl2, delta, Mpad);
    count_launch();
  }
  BwTcParams tp{p.Hq, p.G, p.M, p.N, p.p_seq, p.causal, Mpad, p.sm_scale, negl2, delta};
  int* status_word = tc_status_word();
  const bool per_head = p.G > 1;
  // key-major: dV, dK (per query head)
  {
    BwMaps m;
    void* dv_dst = per_head ? static_cast<void*>(part + part_bytes) : p.dv;
    void* dk_dst = per_head ? static_cast<void*>(part) : p.dk;
    const int64_t ph_ss = p.D, ph_sh = (int64_t)p.N * p.D, ph_sb = (int64_t)p.Hq * p.N * p.D;
    if (!make_map_bhsd(&m.x, p.k, D, p.N, p.Hk, p.B, p.k_ss, p.k_sh, p.k_sb, 128) ||
        !make_map_bhsd(&m.y, p.v, D, p.N, p.Hk, p.B, p.v_ss, p.v_sh, p.v_sb, 128) ||
        !make_map_bhsd(&m.a, p.q, D, p.M, p.Hq, p.B, p.q_ss, p.q_sh, p.q_sb, 128) ||
        !make_map_bhsd(&m.b, p.dout, D, p.M, p.Hq, p.B, p.do_ss, p.do_sh, p.do_sb, 128) ||
        !make_map_bhsd(&m.o0, dv_dst, D, p.N, p.Hq, p.B, per_head ? ph_ss : p.dv_ss, per_head ? ph_sh : p.dv_sh,
                       per_head ? ph_sb : p.dv_sb, 32) ||
        !make_map_bhsd(&m.o1, dk_dst, D, p.N, p.Hq, p.B, per_head ? ph_ss : p.dk_ss, per_head ? ph_sh : p.dk_sh,
                       per_head ? ph_sb : p.dk_sb, 32))
      return cudaErrorInvalidValue;
    dim3 grid(p.Hq, p.B, (p.N + BT - 1) / BT);
    tc_bwd_kernel<T, D, true><<<grid, NTHREADS, L::alloc, s>>>(m, tp, status_word);
    count_launch();
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    if (per_head) {
      const int64_t n = (int64_t)p.B * p.Hk * p.N * (p.D / 2);
      const unsigned blocks = (unsigned)((n + 255) / 256);
      bwd_group_sum_kernel<T><<<blocks, 256, 0, s>>>(reinterpret_cast<const T*>(part), reinterpret_cast<T*>(p.dk),
                                                     p.dk_sb, p.dk_sh, p.dk_ss, p.B, p.Hk, p.G, p.N, p.D);
      bwd_group_sum_kernel<T><<<blocks, 256, 0, s>>>(reinterpret_cast<const T*>(part + part_bytes),
                                                     reinterpret_cast<T*>(p.dv), p.dv_sb, p.dv_sh, p.dv_ss, p.B, p.Hk,
                                                     p.G, p.N, p.D);
      count_launch(2);
    }
  }
  // query-major: dQ
  {
    BwMaps m;
    if (!make_map_bhsd(&m.x, p.q, D, p.M, p.Hq, p.B, p.q_ss, p.q_sh, p.q_sb, 128) ||
        !make_map_bhsd(&m.y, p.dout, D, p.M, p.Hq, p.B, p.do_ss, p.do_sh, p.do_sb, 128) ||
        !make_map_bhsd(&m.a, p.k, D, p.N, p.Hk, p.B, p.k_ss, p.k_sh, p.k_sb, 128) ||
        !make_map_bhsd(&m.b, p.v, D, p.N, p.Hk, p.B, p.v_ss, p.v_sh, p.v_sb, 128) ||
        !make_map_bhsd(&m.o0, p.dq, D, p.M, p.Hq, p.B, p.dq_ss, p.dq_sh, p.dq_sb, 32))
      return cudaErrorInvalidValue;
    m.o1 = m.o0;
    dim3 grid(p.Hq, p.B, (p.M + BT - 1) / BT);
    tc_bwd_kernel<T, D, false><<<grid, NTHREADS, L::alloc, s>>>(m, tp, status_word);
    count_launch();
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
  }
  return cudaSuccess;
}

}  // namespace

size_t tc_bwd_workspace_bytes(int B, int Hq, int Hk, int M, int N, int D) {
  const size_t vec_bytes = ((size_t)B * Hq * mpad_of(M) * 4 + 255) & ~size_t(255);
  const size_t part_bytes = ((size_t)B * Hq * N * D * 2 + 255) & ~size_t(255);
  return 2 * vec_bytes + (Hq != Hk ? 2 * part_bytes : 0);
}

bool tc_bwd_supported(const BwdParams& p, int dtype) {
  (void)dtype;
  if (p.D != 64 && p.D != 128) return false;
  if (p.drop.p > 0.f) return false;  // the dropout mask is regenerated by the CUDA-core kernels only
  if (!(p.sm_scale > 0.f)) return false;
  if (!device_is_sm100() || get_encode() == nullptr) return false;
  if ((p.N + BT - 1) / BT > 65535 || (p.M + BT - 1) / BT > 65535 || p.B > 65535) return false;
  return ok16(p.q, p.q_sb, p.q_sh, p.q_ss) && ok16(p.k, p.k_sb, p.k_sh, p.k_ss) &&
         ok16(p.v, p.v_sb, p.v_sh, p.v_ss) && ok16(p.o, p.o_sb, p.o_sh, p.o_ss) &&
         ok16(p.dout, p.do_sb, p.do_sh, p.do_ss) && ok16(p.dq, p.dq_sb, p.dq_sh, p.dq_ss) &&
         ok16(p.dk, p.dk_sb, p.dk_sh, p.dk_ss) && ok16(p.dv, p.dv_sb, p.dv_sh, p.dv_ss);
}

cudaError_t launch_tc_bwd(const BwdParams& p, int dtype, cudaStream_t s) {
  if (dtype == FAWS_FP16) return p.D == 128 ? launch_bwd_td<__half, 128>(p, s) : launch_bwd_td<__half, 64>(p, s);
  return p.D == 128 ? launch_bwd_td<__nv_bfloat16, 128>(p, s) : launch_bwd_td<__nv_bfloat16, 64>(p, s);
}

}  // namespace faws
