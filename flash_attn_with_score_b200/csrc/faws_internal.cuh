// Shared between the ABI layer and the kernel translation units.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "faws.h"

namespace faws {

// Key-tile visiting orders (attention_with_col_sum.py:119-137 reverse,
// attention_with_col_sum_sequential.py:116-122 round-robin, flash.py:432 forward).
enum Schedule : int { kForward = 0, kReverse = 1, kRoundRobin = 2 };

// Everything a forward kernel needs.  Plain data, passed by value.
// Dropout on the weights that multiply V.  keep(b,h,i,j) = philox6(seed, offset + linear index) > p.
struct DropoutParams {
  float p;            // 0 = off
  float out_scale;    // multiplies out when p > 0
  uint32_t seed_lo, seed_hi;
  uint32_t offset;
};

#ifdef __CUDACC__
// First output of Philox-4x32 with six rounds for counter (c, 0, 0, 0) and key (seed_lo, seed_hi),
// mapped to [0, 1) the way triton's tl.rand does (sign-folded int32 times 2^-31 rounded to fp32):
// the generator the reference kernels draw dropout masks from (flash.py:465).
__device__ __forceinline__ float philox6_uniform(uint32_t c, uint32_t k0, uint32_t k1) {
  uint32_t c0 = c, c1 = 0u, c2 = 0u, c3 = 0u;
#pragma unroll
  for (int r = 0; r < 6; ++r) {
    const uint32_t hb = __umulhi(0xCD9E8D57u, c2), lb = 0xCD9E8D57u * c2;
    const uint32_t ha = __umulhi(0xD2511F53u, c0), la = 0xD2511F53u * c0;
    c0 = hb ^ c1 ^ k0;
    c2 = ha ^ c3 ^ k1;
    c1 = lb;
    c3 = la;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  int x = static_cast<int>(c0);
  x = x < 0 ? ~x : x;
  return __int2float_rn(x) * 4.6566127342e-10f;
}
__device__ __forceinline__ bool dropout_keep(const DropoutParams& d, uint32_t linear_index) {
  return philox6_uniform(d.offset + linear_index, d.seed_lo, d.seed_hi) > d.p;
}
#endif

struct FwdParams {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  int64_t q_sb, q_sh, q_ss;
  int64_t k_sb, k_sh, k_ss;
  int64_t v_sb, v_sh, v_ss;
  int64_t o_sb, o_sh, o_ss;
  float* L;  // (B,Hq,M) or null
  int B, Hq, Hk, G, M, N, D;
  int p_seq;             // N - M: key j visible to query i iff j <= i + p_seq
  int m_begin, m_end;    // query-row window
  int causal;
  float sm_scale;
  int schedule;
  // --- score-tile hooks (null pointer = hook off) ---
  void* scores;          // (B,Hq,M,N) contiguous
  int scores_f32;        // 1: fp32, 0: input dtype
  uint32_t masked_bits;  // fp32 bit pattern written at hidden entries
  float* row_sum;        // (B,Hq,M)
  float* col_partial;    // (B,Hq,n_qb_part,ncols_pad): per-query-block column sums
  int col_row_begin;     // only queries i >= this contribute (0, or split)
  int col_n_end;         // only keys j < this are summed (N, or split)
  int ncols_pad;         // col_n_end rounded up to the key-tile width
  int qb_first;          // first query block (of width block_m) that owns a partial row
  int n_qb_part;         // partial rows per (b,h)
  float* s_scratch;      // buffered variant: (B,Hq,M-split,split) scaled scores
  int split;
  int lpt_order;         // set by the tcgen05 launcher: heaviest causal row blocks of all heads first
  int fill_ctas;         // set by the tcgen05 launcher: masked score tiles are written by extra CTAs
  int n_splits;          // split-KV: key ranges per (batch, head); 0 or 1 = off.  o and L then address the
                         // partial buffers (B, Hq*n_splits, M, D) and (B, Hq, n_splits, M)
  int tiles_per_split;   // key tiles per range
  int col_lin;           // column hook skips tiles that col_tile_linear() accepts (see below)
  int col_row_lo;        // max(col_row_begin, m_begin): first query row that contributes
  float* qsum;           // col_lin: (B,Hq,ceil(M/128),128) per-tile sums of the query rows, written by the
  DropoutParams drop;
};

// Raw column sums are linear in q: for a 128 x 128 (query tile, key tile) pair in which every
// entry is visible and every row contributes, sum_i s_ij = sm_scale * k_j . (sum_i q_i).  Such
// pairs are not reduced inside the forward kernel; the reduce kernel adds them from per-tile sums
// of the query rows.  Both sides use this one predicate.
__host__ __device__ inline bool col_tile_linear(int qb, int t, int row_lo, int m_end, int N, int causal,
                                                int p_seq) {
  const int r0 = qb * 128;
  if (r0 < row_lo || r0 + 128 > m_end) return false;
  if (t * 128 + 128 > N) return false;
  if (causal && t * 128 + 127 > r0 + p_seq) return false;
  return true;
}

// Key-major softmax column-sum pass: out[b,h,j] = sum_{i>=i_begin, visible} exp(s_ij - L_i).
struct ColSoftmaxParams {
  const void* q;
  const void* k;
  int64_t q_sb, q_sh, q_ss;
  int64_t k_sb, k_sh, k_ss;
  const float* L;        // (B,Hq,M)
  float* out;            // (B,Hq,n_end) per query head
  int B, Hq, Hk, G, M, N, D;
  int p_seq, m_begin, m_end, causal;
  float sm_scale;
  int i_begin;           // queries i >= i_begin
  int n_end;             // keys j < n_end
  const float* s_scratch;  // if non-null read scaled scores (B,Hq,M-split,split) instead of q.k
  int split;
  DropoutParams drop;    // p > 0: dropped weights are left out of the sum (no rescale)
  int after_forward;     // launched right after this call's forward pass, which wrote L but not q, k:
                         // the tcgen05 kernel may start its loads and MMAs while that pass drains
  float* negl_pad;       // scratch (B,Hq,m_pad) or null: the tcgen05 launcher fills it with -L_i*log2e (-inf for
                         // rows that do not contribute) and the kernel fetches it tile by tile with bulk copies
  int m_pad;             // M rounded up to the query-tile height
};

struct ReducePartialParams {
  const float* partial;  // (B,Hq,n_qb_part,ncols_pad)
  float* out;            // (B,Hout,n_end)
  int B, Hq, Hk, G, per_q_head;
  int n_end, ncols_pad, n_qb_part, qb_first;
  int block_m, block_n;  // tile sizes the forward kernel used
  int causal, p_seq, N, m_end;
  // linear part (tcgen05 forward only; lin == 0 otherwise)
  int lin;               // 1: add k_j . (sum of the query rows of the linear tiles)
  const float* qsum;     // (B,Hq,nqb_total,128): per 128-row query tile, sum of its rows (fp32)
  int nqb_total, D, row_lo;
  const void* k;
  int64_t k_sb, k_sh, k_ss;
  float sm_scale;
};

// Backward pass of attention(): inputs q, k, v, out, dout, L; outputs dq (B,Hq,M,D), dk, dv (B,Hk,N,D).
struct BwdParams {
  const void* q;
  const void* k;
  const void* v;
  const void* o;
  const void* dout;
  void* dq;
  void* dk;
  void* dv;
  int64_t q_sb, q_sh, q_ss;
  int64_t k_sb, k_sh, k_ss;
  int64_t v_sb, v_sh, v_ss;
  int64_t o_sb, o_sh, o_ss;
  int64_t do_sb, do_sh, do_ss;
  int64_t dq_sb, dq_sh, dq_ss;
  int64_t dk_sb, dk_sh, dk_ss;
  int64_t dv_sb, dv_sh, dv_ss;
  const float* L;  // (B,Hq,M) log-normaliser saved by the forward pass
  float* delta;    // (B,Hq,M) scratch: sum_d out * dout per query row
  int B, Hq, Hk, G, M, N, D;
  int p_seq, causal;
  float sm_scale;
  DropoutParams drop;  // out_scale unused: the kept weights are rescaled by 1/(1-p) (flash.py:655,713,724)
};

// Score-only operator (compute_attention_scores, attention_scores.py:154-223): scores = q.k^T * sm_scale.
struct ScoresOnlyParams {
  const void* q;
  const void* k;
  int64_t q_sb, q_sh, q_ss;
  int64_t k_sb, k_sh, k_ss;
  void* scores;    // (B,Hq,M,N) contiguous
  int scores_f32;  // 1: fp32, 0: the dtype of q
  int B, Hq, Hk, M, N, D;
  float sm_scale;
};

// Launchers (each returns a cudaError_t from the launch).
cudaError_t launch_generic_scores_only(const ScoresOnlyParams& p, int dtype, cudaStream_t s);
bool tc_scores_only_supported(const ScoresOnlyParams& p, int dtype);
cudaError_t launch_tc_scores_only(const ScoresOnlyParams& p, int dtype, cudaStream_t s);
cudaError_t launch_bwd_delta(const BwdParams& p, int dtype, cudaStream_t s);
cudaError_t launch_generic_bwd(const BwdParams& p, int dtype, cudaStream_t s);
cudaError_t launch_generic_fwd(const FwdParams& p, int dtype, cudaStream_t s);
cudaError_t launch_generic_colsoftmax(const ColSoftmaxParams& p, int dtype, cudaStream_t s);
cudaError_t launch_scratch_colsum(const ColSoftmaxParams& p, int group_sum, cudaStream_t s);
cudaError_t launch_reduce_partials(const ReducePartialParams& p, int dtype, cudaStream_t s);
cudaError_t launch_group_sum(const float* in, float* out, int B, int Hk, int G, int len,
                             cudaStream_t s);
cudaError_t launch_reduce_ranks(const float* parts, int n_ranks, int64_t count, float* out,
                                cudaStream_t s);
// out (B,Hq,M,D) and L (B,Hq,M) or null from the split-KV partials o_part (B,Hq,S,M,D) in the dtype of q
// and L_part (B,Hq,S,M)
cudaError_t launch_combine_splits(const void* o_part, const float* L_part, void* out, int64_t o_sb, int64_t o_sh,
                                  int64_t o_ss, float* L, int B, int Hq, int M, int D, int n_splits, int dtype,
                                  cudaStream_t s);

// tcgen05 family.  tc_supported() is a pure host-side check.
bool tc_fwd_supported(const FwdParams& p, int dtype);
cudaError_t launch_tc_fwd(const FwdParams& p, int dtype, cudaStream_t s);
bool tc_colsoftmax_supported(const ColSoftmaxParams& p, int dtype);
bool tc_colsoftmax_group_in_kernel(const ColSoftmaxParams& p);
cudaError_t launch_tc_colsoftmax(const ColSoftmaxParams& p, int dtype, int group_sum, cudaStream_t s);

bool tc_bwd_supported(const BwdParams& p, int dtype);
cudaError_t launch_tc_bwd(const BwdParams& p, int dtype, cudaStream_t s);  // p.delta = the workspace base
size_t tc_bwd_workspace_bytes(int B, int Hq, int Hk, int M, int N, int D);

int tc_read_status(int reset);  // synchronising read of the device status word
cudaError_t launch_wait_give_up(cudaStream_t s);  // self-test: a bounded wait that runs out

constexpr int kGenericBlockM = 64;
constexpr int kGenericBlockN = 64;
constexpr int kTcBlockM = 128;
constexpr int kTcBlockN = 128;

void count_launch(int n = 1);

}  // namespace faws
