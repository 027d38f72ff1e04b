// CUDA-core kernels of the attention-with-scores family.
//
// These cover every shape the operators accept (head dim 16/32/64/128, ragged
// lengths, M != N, unaligned views).  The tcgen05 kernels in faws_tc.cu take
// over whenever a problem fits them; these stay as the path for the rest and
// as the on-device cross-check in the tests.
//
// One CTA = 64 query rows of one (batch, query head); key tiles of 64 are
// streamed through shared memory.  The loop body is the FlashAttention-2
// forward step (flash.py:432-470) with the score-tile hooks of
// attention_with_scores.py:141-162 (store), attention_with_row_sum.py:146-156
// (row reduce) and attention_with_col_sum.py:170-191 (column reduce, written as
// a per-CTA partial instead of an atomic add).
#include "faws_internal.cuh"

namespace faws {
namespace {

constexpr int BM = kGenericBlockM;
constexpr int BN = kGenericBlockN;
constexpr int NT = 256;
constexpr int SLD = BN + 1;
constexpr float kLog2e = 1.4426950408889634f;
#define FAWS_NEG_INF (__int_as_float(0xff800000))

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// rows [r0, r0+64) of a (rows, D) matrix -> smem, zero outside [r_lo, r_hi)
template <typename T>
__device__ __forceinline__ void load_tile(T* dst, int lds, const T* src, int64_t stride_s, int r0,
                                          int r_lo, int r_hi, int D, int vec) {
  if (vec) {
    const int chunks = D >> 3;
    for (int idx = threadIdx.x; idx < 64 * chunks; idx += NT) {
      const int r = idx / chunks, c = idx - r * chunks;
      const int row = r0 + r;
      uint4 val = make_uint4(0u, 0u, 0u, 0u);
      if (row >= r_lo && row < r_hi)
        val = *reinterpret_cast<const uint4*>(src + (int64_t)row * stride_s + c * 8);
      *reinterpret_cast<uint4*>(dst + r * lds + c * 8) = val;
    }
  } else {
    for (int idx = threadIdx.x; idx < 64 * D; idx += NT) {
      const int r = idx / D, c = idx - r * D;
      const int row = r0 + r;
      T val = from_f<T>(0.f);
      if (row >= r_lo && row < r_hi) val = src[(int64_t)row * stride_s + c];
      dst[r * lds + c] = val;
    }
  }
}

// acc[r][c] = sum_d A[(ty*4+r)][d] * Bm[(tx+16c)][d]
template <typename T>
__device__ __forceinline__ void tile_dot(const T* A, const T* Bm, int lds, int D, int ty, int tx,
                                         float (&acc)[4][4]) {
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
  for (int d = 0; d < D; d += 2) {
    float ax[4], ay[4], bx[4], by[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      ax[r] = to_f(A[(ty * 4 + r) * lds + d]);
      ay[r] = to_f(A[(ty * 4 + r) * lds + d + 1]);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      bx[c] = to_f(Bm[(tx + 16 * c) * lds + d]);
      by[c] = to_f(Bm[(tx + 16 * c) * lds + d + 1]);
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[r][c] = fmaf(ax[r], bx[c], fmaf(ay[r], by[c], acc[r][c]));
  }
}

template <typename T>
__global__ void __launch_bounds__(NT) generic_fwd_kernel(FwdParams p, int vec) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = p.D, lds = D + 8;
  T* Qs = reinterpret_cast<T*>(smem_raw);
  T* Ks = Qs + BM * lds;
  T* Vs = Ks + BN * lds;
  float* Ss = reinterpret_cast<float*>(Vs + BN * lds);
  float* m_s = Ss + BM * SLD;
  float* l_s = m_s + BM;
  float* a_s = l_s + BM;

  const int tid = threadIdx.x;
  const int qb_abs = p.m_begin / BM + blockIdx.x;
  const int m0 = qb_abs * BM;
  const int h = blockIdx.y, b = blockIdx.z, hk = h / p.G;
  const int ty = tid >> 4, tx = tid & 15;

  const T* qp = reinterpret_cast<const T*>(p.q) + b * p.q_sb + h * p.q_sh;
  const T* kp = reinterpret_cast<const T*>(p.k) + b * p.k_sb + hk * p.k_sh;
  const T* vp = reinterpret_cast<const T*>(p.v) + b * p.v_sb + hk * p.v_sh;
  T* op = reinterpret_cast<T*>(p.o) + b * p.o_sb + h * p.o_sh;
  const int64_t bh = (int64_t)b * p.Hq + h;

  load_tile(Qs, lds, qp, p.q_ss, m0, p.m_begin, p.m_end, D, vec);
  if (tid < BM) {
    m_s[tid] = FAWS_NEG_INF;
    l_s[tid] = 0.f;
    a_s[tid] = 1.f;
  }
  float o[4][8];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 8; ++c) o[r][c] = 0.f;
  float rs_acc = 0.f;
  const int ncd = D >> 4;  // output columns per thread in the PV step

  int hi = p.N;
  if (p.causal) {
    const int last = min(m0 + BM, p.m_end);
    hi = max(0, min(p.N, p.p_seq + last));
  }
  const int nt = (hi + BN - 1) / BN;
  const float masked_f = __uint_as_float(p.masked_bits);
  const bool part_on = p.col_partial != nullptr && qb_abs >= p.qb_first &&
                       (m0 + BM) > p.col_row_begin;

  for (int it = 0; it < nt; ++it) {
    int t = it;
    if (p.schedule == kReverse) t = nt - 1 - it;
    else if (p.schedule == kRoundRobin) t = (qb_abs + it) % nt;
    const int n0 = t * BN;
    __syncthreads();
    load_tile(Ks, lds, kp, p.k_ss, n0, 0, p.N, D, vec);
    load_tile(Vs, lds, vp, p.v_ss, n0, 0, p.N, D, vec);
    __syncthreads();

    float acc[4][4];
    tile_dot(Qs, Ks, lds, D, ty, tx, acc);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = m0 + ty * 4 + r;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int j = n0 + tx + 16 * c;
        const float s = acc[r][c] * p.sm_scale;
        const bool inb = i >= p.m_begin && i < p.m_end && j < p.N;
        const bool vis = inb && (!p.causal || j <= i + p.p_seq);
        if (p.scores != nullptr && inb) {
          const int64_t off = (bh * p.M + i) * (int64_t)p.N + j;
          const float val = vis ? s : masked_f;
          if (p.scores_f32) reinterpret_cast<float*>(p.scores)[off] = val;
          else reinterpret_cast<T*>(p.scores)[off] = from_f<T>(val);
        }
        if (p.s_scratch != nullptr && inb && i >= p.split && j < p.split)
          p.s_scratch[(bh * (p.M - p.split) + (i - p.split)) * (int64_t)p.split + j] =
              vis ? s : FAWS_NEG_INF;
        Ss[(ty * 4 + r) * SLD + tx + 16 * c] = vis ? s : FAWS_NEG_INF;
      }
    }
    __syncthreads();

    if (p.col_partial != nullptr) {  // uniform branch
      if (part_on && tid < BN && n0 + tid < p.ncols_pad) {
        float sum = 0.f;
        for (int r = 0; r < BM; ++r) {
          const float val = Ss[r * SLD + tid];
          if (m0 + r >= p.col_row_begin && val != FAWS_NEG_INF) sum += val;
        }
        p.col_partial[(bh * p.n_qb_part + (qb_abs - p.qb_first)) * (int64_t)p.ncols_pad + n0 + tid] = sum;
      }
      __syncthreads();
    }

    {  // online softmax, 4 threads per row
      const int row = tid >> 2, qd = tid & 3;
      float mx = FAWS_NEG_INF;
#pragma unroll
      for (int c = 0; c < 16; ++c) mx = fmaxf(mx, Ss[row * SLD + qd + 4 * c]);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_old = m_s[row];
      const float l_old = l_s[row];
      const float m_new = fmaxf(m_old, mx);
      const float alpha = (m_new == FAWS_NEG_INF) ? 1.f : exp2f((m_old - m_new) * kLog2e);
      float psum = 0.f, rsum = 0.f;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const float s = Ss[row * SLD + qd + 4 * c];
        const bool hid = (s == FAWS_NEG_INF);
        const float pr = hid ? 0.f : exp2f((s - m_new) * kLog2e);
        rsum += hid ? 0.f : s;
        psum += pr;  // the normaliser is taken before dropout (flash.py:459-460)
        bool keep = true;
        if (p.drop.p > 0.f)
          keep = dropout_keep(p.drop, ((uint32_t)bh * (uint32_t)p.M + (uint32_t)(m0 + row)) * (uint32_t)p.N +
                                          (uint32_t)(n0 + qd + 4 * c));
        Ss[row * SLD + qd + 4 * c] = keep ? to_f(from_f<T>(pr)) : 0.f;
      }
      psum += __shfl_xor_sync(0xffffffffu, psum, 1);
      psum += __shfl_xor_sync(0xffffffffu, psum, 2);
      rs_acc += rsum;
      __syncwarp();
      if (qd == 0) {
        m_s[row] = m_new;
        l_s[row] = l_old * alpha + psum;
        a_s[row] = alpha;
      }
    }
    __syncthreads();

#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const float a = a_s[ty * 4 + r];
#pragma unroll
      for (int c = 0; c < 8; ++c) o[r][c] *= a;
    }
    for (int n = 0; n < BN; ++n) {
      float pv[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) pv[r] = Ss[(ty * 4 + r) * SLD + n];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (c < ncd) {
          const float vv = to_f(Vs[n * lds + tx + 16 * c]);
#pragma unroll
          for (int r = 0; r < 4; ++r) o[r][c] = fmaf(pv[r], vv, o[r][c]);
        }
      }
    }
  }
  __syncthreads();

#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int i = m0 + ty * 4 + r;
    if (i >= p.m_begin && i < p.m_end) {
      const float l = l_s[ty * 4 + r];
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const float oscale = p.drop.p > 0.f ? p.drop.out_scale : 1.f;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        if (c < ncd) op[(int64_t)i * p.o_ss + tx + 16 * c] = from_f<T>(o[r][c] * inv * oscale);
    }
  }
  if (p.L != nullptr && tid < BM) {
    const int i = m0 + tid;
    if (i >= p.m_begin && i < p.m_end) {
      const float l = l_s[tid];
      p.L[bh * p.M + i] = l > 0.f ? m_s[tid] + logf(l) : FAWS_NEG_INF;
    }
  }
  if (p.row_sum != nullptr) {
    rs_acc += __shfl_xor_sync(0xffffffffu, rs_acc, 1);
    rs_acc += __shfl_xor_sync(0xffffffffu, rs_acc, 2);
    const int i = m0 + (tid >> 2);
    if ((tid & 3) == 0 && i >= p.m_begin && i < p.m_end) p.row_sum[bh * p.M + i] = rs_acc;
  }
  if (p.scores != nullptr) {  // key tiles the causal loop never visits: all hidden
    const int c_begin = nt * BN;
    const int width = p.N - c_begin;
    if (width > 0) {
      for (int idx = tid; idx < BM * width; idx += NT) {
        const int r = idx / width, j = c_begin + (idx - r * width);
        const int i = m0 + r;
        if (i >= p.m_begin && i < p.m_end) {
          const int64_t off = (bh * p.M + i) * (int64_t)p.N + j;
          if (p.scores_f32) reinterpret_cast<float*>(p.scores)[off] = masked_f;
          else reinterpret_cast<T*>(p.scores)[off] = from_f<T>(masked_f);
        }
      }
    }
  }
}

// Score-only operator: one CTA writes a 64 x 64 tile of q.k^T * sm_scale (attention_scores.py:56-151).
template <typename T>
__global__ void __launch_bounds__(NT) generic_scores_only_kernel(ScoresOnlyParams p, int vec) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = p.D, lds = D + 8;
  T* Qs = reinterpret_cast<T*>(smem_raw);
  T* Ks = Qs + BM * lds;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int n_nt = (p.N + BN - 1) / BN;
  const int m0 = (blockIdx.x / n_nt) * BM, n0 = (blockIdx.x % n_nt) * BN;
  const int h = blockIdx.y, b = blockIdx.z, hk = h / (p.Hq / p.Hk);
  const T* qp = reinterpret_cast<const T*>(p.q) + b * p.q_sb + h * p.q_sh;
  const T* kp = reinterpret_cast<const T*>(p.k) + b * p.k_sb + hk * p.k_sh;
  load_tile(Qs, lds, qp, p.q_ss, m0, 0, p.M, D, vec);
  load_tile(Ks, lds, kp, p.k_ss, n0, 0, p.N, D, vec);
  __syncthreads();
  float acc[4][4];
  tile_dot(Qs, Ks, lds, D, ty, tx, acc);
  const int64_t bh = (int64_t)b * p.Hq + h;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int i = m0 + ty * 4 + r;
    if (i >= p.M) continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int j = n0 + tx + 16 * c;
      if (j >= p.N) continue;
      const int64_t off = (bh * p.M + i) * (int64_t)p.N + j;
      const float val = acc[r][c] * p.sm_scale;
      if (p.scores_f32) reinterpret_cast<float*>(p.scores)[off] = val;
      else reinterpret_cast<T*>(p.scores)[off] = from_f<T>(val);
    }
  }
}

// Key-major softmax column sums (the structure of total.py:50-142): a CTA owns
// 64 keys and walks the query tiles; thread c < 64 accumulates column c in a
// register in a fixed order, so there are no atomics and no partials.
template <typename T>
__global__ void __launch_bounds__(NT) generic_colsoftmax_kernel(ColSoftmaxParams p, int vec) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = p.D, lds = D + 8;
  T* Ks = reinterpret_cast<T*>(smem_raw);
  T* Qs = Ks + BN * lds;
  float* Ss = reinterpret_cast<float*>(Qs + BM * lds);
  float* Ls = Ss + BM * SLD;

  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * BN;
  const int h = blockIdx.y, b = blockIdx.z, hk = h / p.G;
  const int ty = tid >> 4, tx = tid & 15;
  const T* qp = reinterpret_cast<const T*>(p.q) + b * p.q_sb + h * p.q_sh;
  const T* kp = reinterpret_cast<const T*>(p.k) + b * p.k_sb + hk * p.k_sh;
  const int64_t bh = (int64_t)b * p.Hq + h;
  const bool from_scratch = p.s_scratch != nullptr;

  if (!from_scratch) load_tile(Ks, lds, kp, p.k_ss, n0, 0, min(p.N, p.n_end), D, vec);
  int i_lo = max(p.i_begin, p.m_begin);
  int i_start = i_lo;
  if (p.causal) i_start = max(i_start, n0 - p.p_seq);
  float colacc = 0.f;
  for (int m0 = (i_start / BM) * BM; m0 < p.m_end; m0 += BM) {
    __syncthreads();
    if (!from_scratch) load_tile(Qs, lds, qp, p.q_ss, m0, i_lo, p.m_end, D, vec);
    if (tid < BM) {
      const int i = m0 + tid;
      Ls[tid] = (i >= i_lo && i < p.m_end) ? p.L[bh * p.M + i] : FAWS_NEG_INF;
    }
    __syncthreads();
    float acc[4][4];
    if (!from_scratch) tile_dot(Qs, Ks, lds, D, ty, tx, acc);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = m0 + ty * 4 + r;
      const float Li = Ls[ty * 4 + r];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int j = n0 + tx + 16 * c;
        const bool vis = i >= i_lo && i < p.m_end && j < p.n_end && j < p.N &&
                         (!p.causal || j <= i + p.p_seq) && Li != FAWS_NEG_INF;
        float s = 0.f;
        if (vis) {
          s = from_scratch
                  ? p.s_scratch[(bh * (p.M - p.split) + (i - p.split)) * (int64_t)p.split + j]
                  : acc[r][c] * p.sm_scale;
        }
        bool keep = vis;
        if (vis && p.drop.p > 0.f)
          keep = dropout_keep(p.drop, ((uint32_t)bh * (uint32_t)p.M + (uint32_t)i) * (uint32_t)p.N + (uint32_t)j);
        Ss[(ty * 4 + r) * SLD + tx + 16 * c] = keep ? exp2f((s - Li) * kLog2e) : 0.f;
      }
    }
    __syncthreads();
    if (tid < BN) {
      for (int r = 0; r < BM; ++r) colacc += Ss[r * SLD + tid];
    }
  }
  if (tid < BN && n0 + tid < p.n_end) p.out[bh * p.n_end + n0 + tid] = colacc;
}

// Second pass of the buffered cross-token variant: the scaled scores of the cross region were
// stored by the forward pass as (B,Hq,M-split,split) fp32; this kernel streams them back
// (attention_cross_token_softmax_sum.py:581-627, without atomics).  HBM-bound, so it is built to keep
// many bytes in flight: a CTA owns 128 key columns of one output head; a thread owns 4 adjacent columns
// (one 16-byte load per row) and one of 8 row groups, and issues 8 independent row loads before it
// uses any (32 threads x 8 row groups x 8 rows x 16 B = 32 KB in flight per CTA).  The exponentials are
// accumulated per thread in registers and the 8 row groups are added in a fixed order at the end.
constexpr int kScRowGroups = 8;
constexpr int kScUnroll = 8;

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(32 * kScRowGroups) scratch_colsum_kernel(ColSoftmaxParams p, int heads_per_cta, int Hout) {
  __shared__ float4 red[kScRowGroups - 1][32];
  const int ct = threadIdx.x & 31, rg = threadIdx.x >> 5;
  const int j0 = blockIdx.x * 128 + ct * 4;  // first of this thread's 4 columns
  const int ho = blockIdx.y, b = blockIdx.z;
  const int i_lo = max(max(p.i_begin, p.m_begin), p.split);
  const int rows = p.M - p.split;
  const int n_lim = min(p.n_end, p.split);
  const bool vec_ok = (p.split % 4 == 0) && (j0 + 3 < n_lim);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int g = 0; g < heads_per_cta; ++g) {
    const int h = ho * heads_per_cta + g;
    const int64_t bh = (int64_t)b * p.Hq + h;
    const float* sbase = p.s_scratch + bh * (int64_t)rows * p.split;
    const float* Lbase = p.L + bh * p.M;
    // key j is visible to query i iff j <= i + p_seq: rows before i_first see none of this CTA's columns
    int i_first = i_lo;
    if (p.causal) i_first = max(i_first, (int)blockIdx.x * 128 - p.p_seq);  // signed: p_seq may exceed the tile start
    for (int i0 = i_first + rg * kScUnroll; i0 < p.m_end; i0 += kScRowGroups * kScUnroll) {
      float4 sv[kScUnroll];
      float Lv[kScUnroll];
#pragma unroll
      for (int r = 0; r < kScUnroll; ++r) {  // loads first: eight rows in flight per thread
        const int i = i0 + r;
        sv[r] = make_float4(0.f, 0.f, 0.f, 0.f);
        Lv[r] = FAWS_NEG_INF;
        if (i < p.m_end) {
          const float* rowp = sbase + (int64_t)(i - p.split) * p.split + j0;
          if (vec_ok) {
            sv[r] = __ldcs(reinterpret_cast<const float4*>(rowp));  // streamed once
          } else {
            if (j0 < n_lim) sv[r].x = rowp[0];
            if (j0 + 1 < n_lim) sv[r].y = rowp[1];
            if (j0 + 2 < n_lim) sv[r].z = rowp[2];
            if (j0 + 3 < n_lim) sv[r].w = rowp[3];
          }
          Lv[r] = Lbase[i];
        }
      }
#pragma unroll
      for (int r = 0; r < kScUnroll; ++r) {
        const int i = i0 + r;
        if (Lv[r] == FAWS_NEG_INF) continue;  // row outside the window, or a row without a visible key
        const float nl = -Lv[r] * kLog2e;
        const int jmax = p.causal ? i + p.p_seq : 0x7fffffff;  // last visible key of this row
        acc.x += (j0 <= jmax) ? ex2_approx(fmaf(sv[r].x, kLog2e, nl)) : 0.f;
        acc.y += (j0 + 1 <= jmax) ? ex2_approx(fmaf(sv[r].y, kLog2e, nl)) : 0.f;
        acc.z += (j0 + 2 <= jmax) ? ex2_approx(fmaf(sv[r].z, kLog2e, nl)) : 0.f;
        acc.w += (j0 + 3 <= jmax) ? ex2_approx(fmaf(sv[r].w, kLog2e, nl)) : 0.f;
      }
    }
  }
  if (rg > 0) red[rg - 1][ct] = acc;
  __syncthreads();
  if (rg == 0) {
#pragma unroll
    for (int w = 0; w < kScRowGroups - 1; ++w) {  // row groups 0, 1, 2, ... in this order
      const float4 o = red[w][ct];
      acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w;
    }
    float* dst = p.out + ((int64_t)b * Hout + ho) * p.n_end + j0;
    if (j0 < n_lim) dst[0] = acc.x;
    if (j0 + 1 < n_lim) dst[1] = acc.y;
    if (j0 + 2 < n_lim) dst[2] = acc.z;
    if (j0 + 3 < n_lim) dst[3] = acc.w;
  }
}

// out[b,ho,j] = sum over the group's heads (or the single head) and over the
// query blocks that visited column j, in a fixed order.
__global__ void reduce_partials_kernel(ReducePartialParams p) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= p.n_end) return;
  const int ho = blockIdx.y, b = blockIdx.z;
  const int h0 = p.per_q_head ? ho : ho * p.G;
  const int nh = p.per_q_head ? 1 : p.G;
  const int Hout = p.per_q_head ? p.Hq : p.Hk;
  const int tile_start = (j / p.block_n) * p.block_n;
  float sum = 0.f;
  for (int g = 0; g < nh; ++g) {
    const float* base = p.partial + ((int64_t)(b * p.Hq + h0 + g) * p.n_qb_part) * p.ncols_pad;
    for (int qb = 0; qb < p.n_qb_part; ++qb) {
      if (p.causal) {
        const int last = min((p.qb_first + qb + 1) * p.block_m, p.m_end);
        const int hi = min(p.N, p.p_seq + last);
        if (tile_start >= hi) continue;  // the forward kernel never visited this key tile
      }
      sum += base[(int64_t)qb * p.ncols_pad + j];
    }
  }
  p.out[((int64_t)b * Hout + ho) * p.n_end + j] = sum;
}

// Column sums with the linear part: a block owns one 128-wide key tile t of one output head.
// out[j] = sm_scale * sum_h k_j . V_h(t) + sum_h sum_{qb hooked} partial[h][qb][j], where
// V_h(t) = sum of qsum[h][qb] over the query tiles for which col_tile_linear(qb, t) holds.
// Eight thread groups of 128 work on eight heads of the group at a time (the per-head chains of
// dependent global loads are what the kernel waits for); their sums are combined in the fixed
// order group 0..7 at the end.
constexpr int kLinGroups = 8;

template <typename T>
__global__ void __launch_bounds__(128 * kLinGroups) reduce_colsum_lin_kernel(ReducePartialParams p) {
  constexpr int LDK = 130;                 // padded row (elements): conflict-free column walks
  __shared__ T Ks[128 * LDK];              // the key tile, loaded once and reused by every head
  __shared__ float V[kLinGroups][128];
  __shared__ float comb[kLinGroups - 1][2][128];
  const int t = blockIdx.x, tid = threadIdx.x & 127, tg = threadIdx.x >> 7;
  const int j = t * 128 + tid;
  const int ho = blockIdx.y, b = blockIdx.z;
  const int h0 = p.per_q_head ? ho : ho * p.G;
  const int nh = p.per_q_head ? 1 : p.G;
  const int Hout = p.per_q_head ? p.Hq : p.Hk;
  const int hk = h0 / p.G;
  const bool j_ok = j < p.n_end && j < p.N;
  {
    const T* kbase = reinterpret_cast<const T*>(p.k) + b * p.k_sb + hk * p.k_sh;
    const bool vec = (reinterpret_cast<uintptr_t>(kbase) % 16 == 0) && (p.k_ss % 8 == 0);
    const int chunks = p.D >> 3;  // 16-byte chunks per row
    if (vec) {
#pragma unroll 4
      for (int idx = threadIdx.x; idx < 128 * chunks; idx += 128 * kLinGroups) {
        const int row = idx / chunks, c = idx - row * chunks;
        const int jr = t * 128 + row;
        uint4 w = make_uint4(0u, 0u, 0u, 0u);
        if (jr < p.N) w = *reinterpret_cast<const uint4*>(kbase + (int64_t)jr * p.k_ss + 8 * c);
        uint32_t* dst = reinterpret_cast<uint32_t*>(&Ks[row * LDK + 8 * c]);
        dst[0] = w.x; dst[1] = w.y; dst[2] = w.z; dst[3] = w.w;
      }
    } else {
      for (int idx = threadIdx.x; idx < 128 * p.D; idx += 128 * kLinGroups) {
        const int row = idx / p.D, c = idx - row * p.D;
        const int jr = t * 128 + row;
        Ks[row * LDK + c] = jr < p.N ? kbase[(int64_t)jr * p.k_ss + c] : from_f<T>(0.f);
      }
    }
  }
  float lin_sum = 0.f, part_sum = 0.f;
  for (int g0 = 0; g0 < nh; g0 += kLinGroups) {  // uniform trip count: barriers inside
    const int g = g0 + tg;
    const bool g_ok = g < nh;
    const int h = h0 + (g_ok ? g : 0);
    float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
    if (g_ok && tid < p.D) {
      const float* qs = p.qsum + (((int64_t)b * p.Hq + h) * p.nqb_total) * 128 + tid;
      int qb = 0;
      for (; qb + 7 < p.nqb_total; qb += 8) {  // loads first, predicates after: eight in flight
        float x[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = qs[(int64_t)(qb + e) * 128];
#pragma unroll
        for (int e = 0; e < 8; e += 4) {
          v0 += col_tile_linear(qb + e, t, p.row_lo, p.m_end, p.N, p.causal, p.p_seq) ? x[e] : 0.f;
          v1 += col_tile_linear(qb + e + 1, t, p.row_lo, p.m_end, p.N, p.causal, p.p_seq) ? x[e + 1] : 0.f;
          v2 += col_tile_linear(qb + e + 2, t, p.row_lo, p.m_end, p.N, p.causal, p.p_seq) ? x[e + 2] : 0.f;
          v3 += col_tile_linear(qb + e + 3, t, p.row_lo, p.m_end, p.N, p.causal, p.p_seq) ? x[e + 3] : 0.f;
        }
      }
      for (; qb < p.nqb_total; ++qb)
        v0 += col_tile_linear(qb, t, p.row_lo, p.m_end, p.N, p.causal, p.p_seq) ? qs[(int64_t)qb * 128] : 0.f;
    }
    __syncthreads();  // K tile loaded (first pass); previous heads' V consumed
    V[tg][tid] = (v0 + v1) + (v2 + v3);
    __syncthreads();
    if (g_ok && j_ok) {
      float d0 = 0.f, d1 = 0.f;
      const T* kr = &Ks[tid * LDK];
      const float* Vg = V[tg];
#pragma unroll 8
      for (int d = 0; d < p.D; d += 2) {
        d0 = fmaf(to_f(kr[d]), Vg[d], d0);
        d1 = fmaf(to_f(kr[d + 1]), Vg[d + 1], d1);
      }
      lin_sum += d0 + d1;
      const float* base = p.partial + ((int64_t)(b * p.Hq + h) * p.n_qb_part) * p.ncols_pad + j;
      float p0 = 0.f, p1 = 0.f;
#pragma unroll 4
      for (int qb = 0; qb < p.n_qb_part; ++qb) {
        const int qa = p.qb_first + qb;
        bool use = !col_tile_linear(qa, t, p.row_lo, p.m_end, p.N, p.causal, p.p_seq);  // else in lin_sum
        if (p.causal) {
          const int last = min((qa + 1) * p.block_m, p.m_end);
          use = use && (t * 128 < min(p.N, p.p_seq + last));  // else the forward kernel never visited it
        }
        const float x = use ? base[(int64_t)qb * p.ncols_pad] : 0.f;
        if (qb & 1) p1 += x; else p0 += x;
      }
      part_sum += p0 + p1;
    }
  }
  if (tg > 0) {
    comb[tg - 1][0][tid] = lin_sum;
    comb[tg - 1][1][tid] = part_sum;
  }
  __syncthreads();
  if (tg == 0 && j < p.n_end) {
#pragma unroll
    for (int w = 0; w < kLinGroups - 1; ++w) {
      lin_sum += comb[w][0][tid];
      part_sum += comb[w][1][tid];
    }
    p.out[((int64_t)b * Hout + ho) * p.n_end + j] = j_ok ? (p.sm_scale * lin_sum + part_sum) : 0.f;
  }
}

__global__ void group_sum_kernel(const float* in, float* out, int Hk, int G, int len) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= len) return;
  const int hk = blockIdx.y, b = blockIdx.z;
  float sum = 0.f;
  for (int g = 0; g < G; ++g) sum += in[((int64_t)(b * Hk + hk) * G + g) * len + j];
  out[((int64_t)b * Hk + hk) * len + j] = sum;
}

__global__ void reduce_ranks_kernel(const float* parts, int n_ranks, int64_t count, float* out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  float sum = 0.f;
  for (int r = 0; r < n_ranks; ++r) sum += parts[(int64_t)r * count + i];
  out[i] = sum;
}

// Split-KV combine (the role of _fwd_combine_kv_splits, split_kv.py:163-227): every key range s left
// a normalised partial result o_s and its log-normaliser L_s; out = sum_s exp(L_s - L) o_s with
// L = log sum_s exp(L_s), added in the order s = 0, 1, ...  One warp per query row.
template <typename T>
__global__ void combine_splits_kernel(const T* __restrict__ o_part, const float* __restrict__ L_part, T* out,
                                      int64_t o_sb, int64_t o_sh, int64_t o_ss, float* L, int B, int Hq, int M, int D,
                                      int S) {
  const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= (int64_t)B * Hq * M) return;
  const int i = (int)(row % M);
  const int64_t bh = row / M;
  const int h = (int)(bh % Hq), b = (int)(bh / Hq);
  const float* Ls = L_part + bh * S * M + i;
  float mx = FAWS_NEG_INF;
  for (int s = 0; s < S; ++s) mx = fmaxf(mx, Ls[(int64_t)s * M]);
  float den = 0.f;
  for (int s = 0; s < S; ++s) {
    const float l = Ls[(int64_t)s * M];
    den += (l == FAWS_NEG_INF) ? 0.f : exp2f((l - mx) * kLog2e);
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
  T* orow = out + b * o_sb + h * o_sh + (int64_t)i * o_ss;
  for (int d = lane; d < D; d += 32) {
    float acc = 0.f;
    for (int s = 0; s < S; ++s) {
      const float l = Ls[(int64_t)s * M];
      if (l == FAWS_NEG_INF) continue;
      acc += exp2f((l - mx) * kLog2e) * to_f(o_part[((bh * S + s) * M + i) * (int64_t)D + d]);
    }
    orow[d] = from_f<T>(acc * inv);
  }
  if (L != nullptr && lane == 0) L[row] = den > 0.f ? mx + logf(den) : FAWS_NEG_INF;
}

size_t fwd_smem(int D) { return (size_t)(3 * 64 * (D + 8)) * 2 + (size_t)(BM * SLD + 3 * BM) * 4; }
size_t cs_smem(int D) { return (size_t)(2 * 64 * (D + 8)) * 2 + (size_t)(BM * SLD + BM) * 4; }

template <typename K>
cudaError_t set_smem(K kernel, size_t bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

bool aligned16(const void* ptr, int64_t a, int64_t b, int64_t c) {
  return (reinterpret_cast<uintptr_t>(ptr) % 16 == 0) && a % 8 == 0 && b % 8 == 0 && c % 8 == 0;
}

}  // namespace

cudaError_t launch_generic_fwd(const FwdParams& p, int dtype, cudaStream_t s) {
  const int vec = aligned16(p.q, p.q_sb, p.q_sh, p.q_ss) && aligned16(p.k, p.k_sb, p.k_sh, p.k_ss) &&
                  aligned16(p.v, p.v_sb, p.v_sh, p.v_ss);
  const int nqb = (p.m_end + BM - 1) / BM - p.m_begin / BM;
  if (nqb <= 0) return cudaSuccess;
  dim3 grid(nqb, p.Hq, p.B);
  const size_t smem = fwd_smem(p.D);
  cudaError_t e;
  if (dtype == FAWS_FP16) {
    if ((e = set_smem(generic_fwd_kernel<__half>, smem)) != cudaSuccess) return e;
    generic_fwd_kernel<__half><<<grid, NT, smem, s>>>(p, vec);
  } else {
    if ((e = set_smem(generic_fwd_kernel<__nv_bfloat16>, smem)) != cudaSuccess) return e;
    generic_fwd_kernel<__nv_bfloat16><<<grid, NT, smem, s>>>(p, vec);
  }
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_generic_scores_only(const ScoresOnlyParams& p, int dtype, cudaStream_t s) {
  const int vec = aligned16(p.q, p.q_sb, p.q_sh, p.q_ss) && aligned16(p.k, p.k_sb, p.k_sh, p.k_ss);
  const long long tiles = (long long)((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  if (tiles <= 0 || tiles > 0x7fffffffLL) return tiles <= 0 ? cudaSuccess : cudaErrorInvalidValue;
  dim3 grid((unsigned)tiles, p.Hq, p.B);
  const size_t smem = (size_t)(2 * 64 * (p.D + 8)) * 2;
  if (dtype == FAWS_FP16) generic_scores_only_kernel<__half><<<grid, NT, smem, s>>>(p, vec);
  else generic_scores_only_kernel<__nv_bfloat16><<<grid, NT, smem, s>>>(p, vec);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_generic_colsoftmax(const ColSoftmaxParams& p, int dtype, cudaStream_t s) {
  const int vec = aligned16(p.q, p.q_sb, p.q_sh, p.q_ss) && aligned16(p.k, p.k_sb, p.k_sh, p.k_ss);
  if (p.n_end <= 0) return cudaSuccess;
  dim3 grid((p.n_end + BN - 1) / BN, p.Hq, p.B);
  const size_t smem = cs_smem(p.D);
  cudaError_t e;
  if (dtype == FAWS_FP16) {
    if ((e = set_smem(generic_colsoftmax_kernel<__half>, smem)) != cudaSuccess) return e;
    generic_colsoftmax_kernel<__half><<<grid, NT, smem, s>>>(p, vec);
  } else {
    if ((e = set_smem(generic_colsoftmax_kernel<__nv_bfloat16>, smem)) != cudaSuccess) return e;
    generic_colsoftmax_kernel<__nv_bfloat16><<<grid, NT, smem, s>>>(p, vec);
  }
  count_launch();
  return cudaGetLastError();
}

// group_sum != 0: p.out is (B,Hk,n_end) and a CTA adds the G heads of its kv head; else (B,Hq,n_end).
cudaError_t launch_scratch_colsum(const ColSoftmaxParams& p, int group_sum, cudaStream_t s) {
  if (p.n_end <= 0) return cudaSuccess;
  const int hpc = group_sum ? p.G : 1;
  const int Hout = p.Hq / hpc;
  dim3 grid((p.n_end + 127) / 128, Hout, p.B);
  scratch_colsum_kernel<<<grid, 32 * kScRowGroups, 0, s>>>(p, hpc, Hout);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_reduce_partials(const ReducePartialParams& p, int dtype, cudaStream_t s) {
  if (p.n_end <= 0) return cudaSuccess;
  if (p.lin) {
    dim3 grid((p.n_end + 127) / 128, p.per_q_head ? p.Hq : p.Hk, p.B);
    if (dtype == FAWS_FP16) reduce_colsum_lin_kernel<__half><<<grid, 128 * kLinGroups, 0, s>>>(p);
    else reduce_colsum_lin_kernel<__nv_bfloat16><<<grid, 128 * kLinGroups, 0, s>>>(p);
  } else {
    dim3 grid((p.n_end + 255) / 256, p.per_q_head ? p.Hq : p.Hk, p.B);
    reduce_partials_kernel<<<grid, 256, 0, s>>>(p);
  }
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_group_sum(const float* in, float* out, int B, int Hk, int G, int len,
                             cudaStream_t s) {
  if (len <= 0) return cudaSuccess;
  dim3 grid((len + 255) / 256, Hk, B);
  group_sum_kernel<<<grid, 256, 0, s>>>(in, out, Hk, G, len);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_combine_splits(const void* o_part, const float* L_part, void* out, int64_t o_sb, int64_t o_sh,
                                  int64_t o_ss, float* L, int B, int Hq, int M, int D, int n_splits, int dtype,
                                  cudaStream_t s) {
  const int64_t rows = (int64_t)B * Hq * M;
  const unsigned blocks = (unsigned)((rows * 32 + 255) / 256);
  if (dtype == FAWS_FP16)
    combine_splits_kernel<__half><<<blocks, 256, 0, s>>>(static_cast<const __half*>(o_part), L_part,
                                                         static_cast<__half*>(out), o_sb, o_sh, o_ss, L, B, Hq, M, D,
                                                         n_splits);
  else
    combine_splits_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(o_part), L_part,
                                                                static_cast<__nv_bfloat16*>(out), o_sb, o_sh, o_ss, L,
                                                                B, Hq, M, D, n_splits);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_reduce_ranks(const float* parts, int n_ranks, int64_t count, float* out,
                                cudaStream_t s) {
  if (count <= 0) return cudaSuccess;
  reduce_ranks_kernel<<<(unsigned)((count + 255) / 256), 256, 0, s>>>(parts, n_ranks, count, out);
  count_launch();
  return cudaGetLastError();
}

}  // namespace faws
