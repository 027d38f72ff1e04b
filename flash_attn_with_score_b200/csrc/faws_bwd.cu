// Backward pass of attention(), CUDA-core kernels.
//
// Same split as the reference's FlashAttention.backward (flash.py:172-261): a pre-pass computes
// delta_i = sum_d o_id * do_id (flash.py:532-577), a key-major kernel owns a tile of keys and
// produces dK and dV (flash.py:581-754), a query-major kernel owns a tile of queries and produces
// dQ (flash.py:758-918).  Both recompute P = exp(s - L_i) from the saved log-normaliser.  Nothing
// is accumulated with atomics: the key-major kernel walks the G query heads of its kv head itself
// and writes dK, dV in the (B,Hk,N,D) layout once (the reference writes per-query-head tensors and
// sums them on the host, flash.py:259-260).
//
// These kernels cover every accepted shape (head dim 16..128, ragged lengths, M != N, dropout);
// the tcgen05 kernels in faws_tc_bwd.cu take over when the problem fits them.
#include "faws_internal.cuh"

namespace faws {
namespace {

constexpr int BT = 64;   // tile edge (queries and keys)
constexpr int NT = 256;
constexpr int SLD = BT + 1;
constexpr float kLog2e = 1.4426950408889634f;
#define FAWS_NEG_INF (__int_as_float(0xff800000))

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// rows [r0, r0+64) of a (rows, D) matrix -> smem, zero at and beyond r_hi
template <typename T>
__device__ __forceinline__ void load_rows(T* dst, int lds, const T* src, int64_t stride_s, int r0, int r_hi, int D) {
  for (int idx = threadIdx.x; idx < BT * D; idx += NT) {
    const int r = idx / D, c = idx - r * D;
    const int row = r0 + r;
    dst[r * lds + c] = row < r_hi ? src[(int64_t)row * stride_s + c] : from_f<T>(0.f);
  }
}

// acc[r][c] = sum_d A[ty*4+r][d] * Bm[tx+16c][d]
template <typename T>
__device__ __forceinline__ void dot_rows(const T* A, const T* Bm, int lds, int D, int ty, int tx, float (&acc)[4][4]) {
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
  for (int d = 0; d < D; ++d) {
    float a[4], b[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) a[r] = to_f(A[(ty * 4 + r) * lds + d]);
#pragma unroll
    for (int c = 0; c < 4; ++c) b[c] = to_f(Bm[(tx + 16 * c) * lds + d]);
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[r][c] = fmaf(a[r], b[c], acc[r][c]);
  }
}

// delta[b,h,i] = sum_d out[b,h,i,d] * dout[b,h,i,d]; one warp per row
template <typename T>
__global__ void bwd_delta_kernel(BwdParams p) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int64_t rows = (int64_t)p.B * p.Hq * p.M;
  if (warp >= rows) return;
  const int i = warp % p.M;
  const int bh = warp / p.M;
  const int h = bh % p.Hq, b = bh / p.Hq;
  const T* o = reinterpret_cast<const T*>(p.o) + b * p.o_sb + h * p.o_sh + (int64_t)i * p.o_ss;
  const T* g = reinterpret_cast<const T*>(p.dout) + b * p.do_sb + h * p.do_sh + (int64_t)i * p.do_ss;
  float sum = 0.f;
  for (int d = lane; d < p.D; d += 32) sum = fmaf(to_f(o[d]), to_f(g[d]), sum);
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
  if (lane == 0) p.delta[warp] = sum;
}

// What both kernels recompute for one (query i, key j): the softmax weight, and the gradient of
// the scaled score.  With dropout (flash.py:698-726): the weight that multiplied V is
// keep * p / (1 - p_drop) and dP is masked and rescaled the same way.
struct PairGrad {
  float p_v;  // weight that multiplied v_j in the forward pass (dV += p_v * do_i)
  float ds;   // d loss / d (q_i . k_j)  (includes sm_scale)
};
__device__ __forceinline__ PairGrad pair_grad(const BwdParams& p, float s_raw, float dp, float Li, float delta_i,
                                              bool vis, uint32_t lin) {
  PairGrad g{0.f, 0.f};
  if (!vis || Li == FAWS_NEG_INF) return g;
  const float pr = exp2f((s_raw * p.sm_scale - Li) * kLog2e);
  float keep_scale = 1.f;
  if (p.drop.p > 0.f) keep_scale = dropout_keep(p.drop, lin) ? 1.f / (1.f - p.drop.p) : 0.f;
  g.p_v = pr * keep_scale;
  g.ds = pr * (dp * keep_scale - delta_i) * p.sm_scale;
  return g;
}

// Key-major: CTA = 64 keys of one (batch, kv head); walks the group's query heads and their query tiles.
template <typename T>
__global__ void __launch_bounds__(NT) generic_bwd_kv_kernel(BwdParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = p.D, lds = D + 2;
  T* Ks = reinterpret_cast<T*>(smem_raw);
  T* Vs = Ks + BT * lds;
  T* Qs = Vs + BT * lds;
  T* Gs = Qs + BT * lds;  // dout tile
  float* Ps = reinterpret_cast<float*>(Gs + BT * lds);
  float* dSs = Ps + BT * SLD;
  float* Ls = dSs + BT * SLD;
  float* Ds = Ls + BT;

  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int n0 = blockIdx.x * BT, hk = blockIdx.y, b = blockIdx.z;
  const T* kp = reinterpret_cast<const T*>(p.k) + b * p.k_sb + hk * p.k_sh;
  const T* vp = reinterpret_cast<const T*>(p.v) + b * p.v_sb + hk * p.v_sh;
  load_rows(Ks, lds, kp, p.k_ss, n0, p.N, D);
  load_rows(Vs, lds, vp, p.v_ss, n0, p.N, D);
  const int ncd = D >> 4;  // output columns per thread
  float dk[4][8], dv[4][8];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 8; ++c) dk[r][c] = dv[r][c] = 0.f;

  int i_start = 0;  // first query that sees key n0: j <= i + p_seq
  if (p.causal) i_start = max(0, n0 - p.p_seq);
  for (int g = 0; g < p.G; ++g) {
    const int h = hk * p.G + g;
    const int64_t bh = (int64_t)b * p.Hq + h;
    const T* qp = reinterpret_cast<const T*>(p.q) + b * p.q_sb + h * p.q_sh;
    const T* gp = reinterpret_cast<const T*>(p.dout) + b * p.do_sb + h * p.do_sh;
    for (int m0 = (i_start / BT) * BT; m0 < p.M; m0 += BT) {
      __syncthreads();
      load_rows(Qs, lds, qp, p.q_ss, m0, p.M, D);
      load_rows(Gs, lds, gp, p.do_ss, m0, p.M, D);
      if (tid < BT) {
        const int i = m0 + tid;
        Ls[tid] = i < p.M ? p.L[bh * p.M + i] : FAWS_NEG_INF;
        Ds[tid] = i < p.M ? p.delta[bh * p.M + i] : 0.f;
      }
      __syncthreads();
      float s[4][4], dp[4][4];
      dot_rows(Qs, Ks, lds, D, ty, tx, s);
      dot_rows(Gs, Vs, lds, D, ty, tx, dp);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int i = m0 + ty * 4 + r;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int j = n0 + tx + 16 * c;
          const bool vis = i < p.M && j < p.N && (!p.causal || j <= i + p.p_seq);
          const PairGrad pg = pair_grad(p, s[r][c], dp[r][c], Ls[ty * 4 + r], Ds[ty * 4 + r], vis,
                                        ((uint32_t)bh * (uint32_t)p.M + (uint32_t)i) * (uint32_t)p.N + (uint32_t)j);
          Ps[(ty * 4 + r) * SLD + tx + 16 * c] = to_f(from_f<T>(pg.p_v));  // P is rounded like the forward pass rounds it
          dSs[(ty * 4 + r) * SLD + tx + 16 * c] = pg.ds;
        }
      }
      __syncthreads();
      // dV[key][d] += sum_q P[q][key] * dO[q][d];  dK[key][d] += sum_q dS[q][key] * Q[q][d]
      for (int qi = 0; qi < BT; ++qi) {
        float pw[4], dw[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          pw[r] = Ps[qi * SLD + ty * 4 + r];
          dw[r] = dSs[qi * SLD + ty * 4 + r];
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          if (c < ncd) {
            const float gv = to_f(Gs[qi * lds + tx + 16 * c]);
            const float qv = to_f(Qs[qi * lds + tx + 16 * c]);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              dv[r][c] = fmaf(pw[r], gv, dv[r][c]);
              dk[r][c] = fmaf(dw[r], qv, dk[r][c]);
            }
          }
        }
      }
    }
  }
  T* dkp = reinterpret_cast<T*>(p.dk) + b * p.dk_sb + hk * p.dk_sh;
  T* dvp = reinterpret_cast<T*>(p.dv) + b * p.dv_sb + hk * p.dv_sh;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int j = n0 + ty * 4 + r;
    if (j < p.N) {
#pragma unroll
      for (int c = 0; c < 8; ++c)
        if (c < ncd) {
          dkp[(int64_t)j * p.dk_ss + tx + 16 * c] = from_f<T>(dk[r][c]);
          dvp[(int64_t)j * p.dv_ss + tx + 16 * c] = from_f<T>(dv[r][c]);
        }
    }
  }
}

// Query-major: CTA = 64 queries of one (batch, query head); walks the visible key tiles.
template <typename T>
__global__ void __launch_bounds__(NT) generic_bwd_q_kernel(BwdParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = p.D, lds = D + 2;
  T* Ks = reinterpret_cast<T*>(smem_raw);
  T* Vs = Ks + BT * lds;
  T* Qs = Vs + BT * lds;
  T* Gs = Qs + BT * lds;
  float* dSs = reinterpret_cast<float*>(Gs + BT * lds);
  float* Ls = dSs + BT * SLD;
  float* Ds = Ls + BT;

  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int m0 = blockIdx.x * BT, h = blockIdx.y, b = blockIdx.z, hk = h / p.G;
  const int64_t bh = (int64_t)b * p.Hq + h;
  const T* qp = reinterpret_cast<const T*>(p.q) + b * p.q_sb + h * p.q_sh;
  const T* gp = reinterpret_cast<const T*>(p.dout) + b * p.do_sb + h * p.do_sh;
  const T* kp = reinterpret_cast<const T*>(p.k) + b * p.k_sb + hk * p.k_sh;
  const T* vp = reinterpret_cast<const T*>(p.v) + b * p.v_sb + hk * p.v_sh;
  load_rows(Qs, lds, qp, p.q_ss, m0, p.M, D);
  load_rows(Gs, lds, gp, p.do_ss, m0, p.M, D);
  if (tid < BT) {
    const int i = m0 + tid;
    Ls[tid] = i < p.M ? p.L[bh * p.M + i] : FAWS_NEG_INF;
    Ds[tid] = i < p.M ? p.delta[bh * p.M + i] : 0.f;
  }
  const int ncd = D >> 4;
  float dq[4][8];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 8; ++c) dq[r][c] = 0.f;
  int hi = p.N;
  if (p.causal) hi = max(0, min(p.N, p.p_seq + min(m0 + BT, p.M)));
  for (int n0 = 0; n0 < hi; n0 += BT) {
    __syncthreads();
    load_rows(Ks, lds, kp, p.k_ss, n0, p.N, D);
    load_rows(Vs, lds, vp, p.v_ss, n0, p.N, D);
    __syncthreads();
    float s[4][4], dp[4][4];
    dot_rows(Qs, Ks, lds, D, ty, tx, s);
    dot_rows(Gs, Vs, lds, D, ty, tx, dp);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = m0 + ty * 4 + r;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int j = n0 + tx + 16 * c;
        const bool vis = i < p.M && j < p.N && (!p.causal || j <= i + p.p_seq);
        const PairGrad pg = pair_grad(p, s[r][c], dp[r][c], Ls[ty * 4 + r], Ds[ty * 4 + r], vis,
                                      ((uint32_t)bh * (uint32_t)p.M + (uint32_t)i) * (uint32_t)p.N + (uint32_t)j);
        dSs[(ty * 4 + r) * SLD + tx + 16 * c] = pg.ds;
      }
    }
    __syncthreads();
    // dQ[query][d] += sum_key dS[query][key] * K[key][d]
    for (int kk = 0; kk < BT; ++kk) {
      float dw[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) dw[r] = dSs[(ty * 4 + r) * SLD + kk];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (c < ncd) {
          const float kv = to_f(Ks[kk * lds + tx + 16 * c]);
#pragma unroll
          for (int r = 0; r < 4; ++r) dq[r][c] = fmaf(dw[r], kv, dq[r][c]);
        }
      }
    }
  }
  T* dqp = reinterpret_cast<T*>(p.dq) + b * p.dq_sb + h * p.dq_sh;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int i = m0 + ty * 4 + r;
    if (i < p.M) {
#pragma unroll
      for (int c = 0; c < 8; ++c)
        if (c < ncd) dqp[(int64_t)i * p.dq_ss + tx + 16 * c] = from_f<T>(dq[r][c]);
    }
  }
}

size_t kv_smem(int D) { return (size_t)(4 * BT * (D + 2)) * 2 + (size_t)(2 * BT * SLD + 2 * BT) * 4; }
size_t q_smem(int D) { return (size_t)(4 * BT * (D + 2)) * 2 + (size_t)(BT * SLD + 2 * BT) * 4; }

template <typename T>
cudaError_t launch_bwd_t(const BwdParams& p, cudaStream_t s) {
  cudaError_t e;
  if ((e = cudaFuncSetAttribute(generic_bwd_kv_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)kv_smem(p.D))) != cudaSuccess)
    return e;
  if ((e = cudaFuncSetAttribute(generic_bwd_q_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)q_smem(p.D))) != cudaSuccess)
    return e;
  generic_bwd_kv_kernel<T><<<dim3((p.N + BT - 1) / BT, p.Hk, p.B), NT, kv_smem(p.D), s>>>(p);
  generic_bwd_q_kernel<T><<<dim3((p.M + BT - 1) / BT, p.Hq, p.B), NT, q_smem(p.D), s>>>(p);
  count_launch(2);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_bwd_delta(const BwdParams& p, int dtype, cudaStream_t s) {
  const int64_t rows = (int64_t)p.B * p.Hq * p.M;
  const unsigned blocks = (unsigned)((rows * 32 + 255) / 256);
  if (dtype == FAWS_FP16) bwd_delta_kernel<__half><<<blocks, 256, 0, s>>>(p);
  else bwd_delta_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(p);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_generic_bwd(const BwdParams& p, int dtype, cudaStream_t s) {
  return dtype == FAWS_FP16 ? launch_bwd_t<__half>(p, s) : launch_bwd_t<__nv_bfloat16>(p, s);
}

}  // namespace faws
