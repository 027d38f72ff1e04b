// Score-only operator on tcgen05 (sm_100a): scores = q.k^T * sm_scale, nothing else
// (compute_attention_scores, attention_scores.py:154-223; kernel :56-151).
//
// One CTA = 128 query rows of one (batch, query head).  Warp roles (12 warps):
//   warp 0      TMA producer: the Q tile once, then the K tiles through a 3-slot ring
//   warp 1      allocates TMEM (two S buffers of 128 columns); one lane issues S = Q.K^T per key tile
//   warps 4-7   epilogue of the even key tiles, warps 8-11 of the odd ones: a thread owns one
//               query row, reads its 128 scores from TMEM in chunks of 32 columns, scales and
//               converts them, stages 32-row boxes in swizzled shared memory and writes them with
//               TMA stores (which clip at the tensor's edge, so ragged M and N need no predicates).
// HBM-bound: the (B,Hq,M,N) score write is the traffic; every wait on an mbarrier is bounded.
#include <cuda.h>

#include <type_traits>

#include "faws_internal.cuh"
#include "faws_tc_host.cuh"
#include "faws_tc_ptx.cuh"

namespace faws {
namespace {
using namespace ptx;

constexpr int BM = 128, BN = 128;
constexpr int NTHREADS = 384;
constexpr int K_SLOTS = 3;
constexpr int TMEM_COLS = 256;

template <int D>
struct ScSmem {
  static constexpr int kTile = 128 * D * 2;
  static constexpr int kSub = 128 * 128;
  static constexpr int q_off = 0;
  static constexpr int k_off = q_off + kTile;
  static constexpr int stage_off = k_off + K_SLOTS * kTile;  // 8 warps x 2 x 4 KB
  static constexpr int bar_off = stage_off + 8 * 2 * 4096;
  static constexpr int total = bar_off + 256;
  static constexpr int alloc = total + 1024;
};

struct ScBars {
  uint64_t q_full;
  uint64_t k_full[K_SLOTS], k_empty[K_SLOTS];
  uint64_t s_full[2], s_free[2];
  uint32_t tmem_base;
  int abort_flag;
};

struct ScMaps {
  CUtensorMap q, k, st;
};

struct ScParams {
  int M, N, Hq, G;
  float sm_scale;
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

template <typename T, int D, bool F32OUT>
__global__ void __launch_bounds__(NTHREADS, 1)
tc_qk_scores_kernel(const __grid_constant__ ScMaps maps, const ScParams p, int* __restrict__ status) {
  using L = ScSmem<D>;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  ScBars* bars = reinterpret_cast<ScBars*>(smem + L::bar_off);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BM, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / p.G;
  const int bh = b * p.Hq + h;
  const int nkt = (p.N + BN - 1) / BN;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < K_SLOTS; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
    }
    for (int e = 0; e < 2; ++e) {
      mbar_init(&bars->s_full[e], 1);
      mbar_init(&bars->s_free[e], 128);
    }
    bars->abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&maps.q);
    prefetch_tmap(&maps.k);
    prefetch_tmap(&maps.st);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------------------------------------------------- TMA producer
      mbar_arrive_expect_tx(&bars->q_full, L::kTile);
      for (int c = 0; c < D / 64; ++c)
        tma_load_4d(smem + L::q_off + c * L::kSub, &maps.q, &bars->q_full, c * 64, m0, h, b);
      for (int t = 0; t < nkt; ++t) {
        const int s = t % K_SLOTS, use = t / K_SLOTS;
        if (use > 0 && !mbar_wait(&bars->k_empty[s], (use - 1) & 1, abort_flag)) break;
        mbar_arrive_expect_tx(&bars->k_full[s], L::kTile);
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(smem + L::k_off + s * L::kTile + c * L::kSub, &maps.k, &bars->k_full[s], c * 64, t * BN, hk, b);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (whole warp loops, one lane issues)
    constexpr int kFmt = std::is_same<T, __half>::value ? 0 : 1;
    constexpr uint32_t idesc = make_idesc_f16(128, BN, kFmt, 0, 0);
    const uint64_t q_desc = make_desc_sw128(smem_u32(smem + L::q_off), 16, 1024);
    const uint64_t k_desc0 = make_desc_sw128(smem_u32(smem + L::k_off), 16, 1024);
    bool ok = mbar_wait(&bars->q_full, 0, abort_flag);
    for (int t = 0; ok && t < nkt; ++t) {
      const int s = t % K_SLOTS, e = t & 1, use = t >> 1;
      if (!(ok = mbar_wait(&bars->k_full[s], (t / K_SLOTS) & 1, abort_flag))) break;
      if (use > 0 && !(ok = mbar_wait(&bars->s_free[e], (use - 1) & 1, abort_flag))) break;
      tc_fence_after();
      const uint64_t kd = k_desc0 + (uint64_t)(s * (L::kTile >> 4));
      const uint32_t d_tmem = tmem_base + (uint32_t)(e * BN);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t off = (uint64_t)(((kk >> 2) * L::kSub + (kk & 3) * 32) >> 4);
          if (kk == 0) mma_ss(d_tmem, q_desc + off, kd + off, idesc, 0u);
          else mma_ss_acc(d_tmem, q_desc + off, kd + off, idesc);
        }
        mma_commit(&bars->k_empty[s]);
        mma_commit(&bars->s_full[e]);
      }
      __syncwarp();
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue: thread = query row
    const int e = (warp - 4) >> 2;
    const int lg = warp & 3;
    const uint32_t t_s = tmem_base + ((uint32_t)(lg * 32) << 16) + (uint32_t)(e * BN);
    unsigned char* stage = smem + L::stage_off + (warp - 4) * 8192;
    const float scale = p.sm_scale;
    int nstaged = 0;  // boxes staged so far by this warp (selects the 4 KB buffer)
    for (int t = e; t < nkt; t += 2) {
      if (!mbar_wait(&bars->s_full[e], (t >> 1) & 1, abort_flag)) break;
      tc_fence_after();
      const int n0 = t * BN;
      constexpr int kBoxCols = F32OUT ? 32 : 64;  // one box = 32 rows x 128 bytes
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += kBoxCols) {
        uint32_t r[kBoxCols];
#pragma unroll
        for (int c = 0; c < kBoxCols; c += 32) tmem_ld32(t_s + c0 + c, reinterpret_cast<uint32_t(&)[32]>(r[c]));
        tmem_wait_ld();
        if (c0 + kBoxCols == BN) {  // the S buffer can take this warpgroup's next key tile
          tc_fence_before();
          mbar_arrive(&bars->s_free[e]);
        }
        unsigned char* sb = stage + (nstaged & 1) * 4096;
        if (lane == 0) tma_store_wait_read<1>();  // the store that last read this buffer has fetched it
        __syncwarp();
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          uint4 w;
          if constexpr (F32OUT) {
            w.x = __float_as_uint(__uint_as_float(r[cc * 4 + 0]) * scale);
            w.y = __float_as_uint(__uint_as_float(r[cc * 4 + 1]) * scale);
            w.z = __float_as_uint(__uint_as_float(r[cc * 4 + 2]) * scale);
            w.w = __float_as_uint(__uint_as_float(r[cc * 4 + 3]) * scale);
          } else {
            w.x = pack2<T>(__uint_as_float(r[cc * 8 + 0]) * scale, __uint_as_float(r[cc * 8 + 1]) * scale);
            w.y = pack2<T>(__uint_as_float(r[cc * 8 + 2]) * scale, __uint_as_float(r[cc * 8 + 3]) * scale);
            w.z = pack2<T>(__uint_as_float(r[cc * 8 + 4]) * scale, __uint_as_float(r[cc * 8 + 5]) * scale);
            w.w = pack2<T>(__uint_as_float(r[cc * 8 + 6]) * scale, __uint_as_float(r[cc * 8 + 7]) * scale);
          }
          *reinterpret_cast<uint4*>(sb + lane * 128 + ((cc ^ (lane & 7)) << 4)) = w;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_3d(&maps.st, sb, n0 + c0, m0 + lg * 32, bh);
          tma_store_commit();
        }
        ++nstaged;
      }
    }
    if (lane == 0) tma_store_wait<0>();
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

template <typename T, int D, bool F32OUT>
cudaError_t launch_sc(const ScMaps& maps, const ScoresOnlyParams& p, cudaStream_t s) {
  using L = ScSmem<D>;
  static PerDeviceOnce attr_once;
  if (cudaError_t e = set_max_smem_once(attr_once, tc_qk_scores_kernel<T, D, F32OUT>, L::alloc); e != cudaSuccess)
    return e;
  ScParams sp{p.M, p.N, p.Hq, p.Hq / p.Hk, p.sm_scale};
  dim3 grid((p.M + BM - 1) / BM, p.Hq, p.B);
  tc_qk_scores_kernel<T, D, F32OUT><<<grid, NTHREADS, L::alloc, s>>>(maps, sp, tc_status_word());
  count_launch();
  return cudaGetLastError();
}

template <typename T, int D>
cudaError_t launch_sc_d(const ScMaps& maps, const ScoresOnlyParams& p, cudaStream_t s) {
  return p.scores_f32 ? launch_sc<T, D, true>(maps, p, s) : launch_sc<T, D, false>(maps, p, s);
}

}  // namespace

bool tc_scores_only_supported(const ScoresOnlyParams& p, int dtype) {
  (void)dtype;
  if (p.D != 64 && p.D != 128) return false;
  if (!device_is_sm100() || get_encode() == nullptr) return false;
  if (!ok16(p.q, p.q_sb, p.q_sh, p.q_ss) || !ok16(p.k, p.k_sb, p.k_sh, p.k_ss)) return false;
  // TMA store rows must start on 16-byte boundaries
  if (p.N % (p.scores_f32 ? 4 : 8) != 0 || reinterpret_cast<uintptr_t>(p.scores) % 16 != 0) return false;
  return true;
}

cudaError_t launch_tc_scores_only(const ScoresOnlyParams& p, int dtype, cudaStream_t s) {
  ScMaps maps;
  const int esize = p.scores_f32 ? 4 : 2;
  if (!make_map_bhsd(&maps.q, p.q, p.D, p.M, p.Hq, p.B, p.q_ss, p.q_sh, p.q_sb, 128) ||
      !make_map_bhsd(&maps.k, p.k, p.D, p.N, p.Hk, p.B, p.k_ss, p.k_sh, p.k_sb, 128) ||
      !make_map_store_f32(&maps.st, p.scores, p.N, p.M, p.N, (int64_t)p.M * p.N, p.B * p.Hq, esize))
    return cudaErrorInvalidValue;
  if (dtype == FAWS_FP16)
    return p.D == 128 ? launch_sc_d<__half, 128>(maps, p, s) : launch_sc_d<__half, 64>(maps, p, s);
  return p.D == 128 ? launch_sc_d<__nv_bfloat16, 128>(maps, p, s) : launch_sc_d<__nv_bfloat16, 64>(maps, p, s);
}

}  // namespace faws
