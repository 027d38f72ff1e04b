/*
 * faws.h -- C ABI of the B200 (sm_100a) attention-with-scores library.
 *
 * One entry point per operator exported by the reference package
 * (__init__.py:29-39).  Every function takes plain device pointers, sizes and
 * element strides; nothing here depends on PyTorch.  The library owns no
 * memory: the caller allocates inputs, outputs and the scratch workspace
 * (size from faws_workspace_bytes) and passes the CUDA stream to launch on.
 * All functions return 0 on success or a negative FAWS_E* code and never
 * throw.  They are asynchronous with respect to the host: only launches are
 * enqueued on `stream`.
 *
 * Tensor layout is the reference's: q (B,Hq,M,D); k, v (B,Hk,N,D); out
 * (B,Hq,M,D); last dimension contiguous, other strides free
 * (flash.py:23-26).  Hq must be a multiple of Hk (GQA; kv head = q head / G,
 * flash.py:364).  Causal masking is bottom-right aligned: key j is visible to
 * query i iff j <= i + (N - M) (flash.py:451).
 */
#ifndef FAWS_H_
#define FAWS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FAWS_VERSION 2

/* element types of q, k, v, out */
#define FAWS_FP16 0
#define FAWS_BF16 1
/* element type of the scores tensor */
#define FAWS_SCORES_F32 0   /* fp32 (default of this library)                  */
#define FAWS_SCORES_INPUT 1 /* same as q (what the reference kernel writes,    */
                            /* attention_with_scores.py:284)                   */

/* status codes */
#define FAWS_OK 0
#define FAWS_EINVAL (-1)      /* bad shape, NULL pointer, split out of range  */
#define FAWS_EUNSUPPORTED (-2) /* head dim / dtype / alignment not supported  */
#define FAWS_EWORKSPACE (-3)  /* workspace missing, too small or misaligned   */
#define FAWS_ECUDA (-4)       /* a CUDA runtime / driver call failed          */
#define FAWS_EBACKEND (-5)    /* forced backend cannot run this problem       */
#define FAWS_ETOOLARGE (-6)   /* problem exceeds the built-in scratch of the  */
                              /* _noalloc entry point                         */

/* kernel families ("backend" below) */
#define FAWS_BACKEND_AUTO 0    /* tcgen05 kernels when the problem fits them   */
#define FAWS_BACKEND_GENERIC 1 /* CUDA-core kernels: any D in {16,32,64,128},  */
                               /* any alignment                                */
#define FAWS_BACKEND_TCGEN05 2 /* TMA + tcgen05/TMEM kernels: D in {64,128},   */
                               /* 16-byte aligned rows                         */

/* operator ids for faws_workspace_bytes */
#define FAWS_OP_ATTENTION 0
#define FAWS_OP_SCORES 1
#define FAWS_OP_ROW_SUM 2
#define FAWS_OP_COL_SUM 3
#define FAWS_OP_COL_SUM_SEQUENTIAL 4
#define FAWS_OP_SOFTMAX_COL_SUM 5
#define FAWS_OP_CROSS_QK_SUM 6
#define FAWS_OP_CROSS_SOFTMAX_SUM 7
#define FAWS_OP_CROSS_SOFTMAX_SUM_BUFFERED 8
#define FAWS_OP_TOTAL_ATTENTION 9
#define FAWS_OP_ATTENTION_BACKWARD 10
#define FAWS_OP_ATTENTION_SPLIT_KV 11

/* A (B,H,S,D) view; strides in elements; the D axis has stride 1. */
typedef struct faws_tensor {
  void* ptr;
  int64_t stride_b;
  int64_t stride_h;
  int64_t stride_s;
} faws_tensor;

/*
 * The part every operator shares: the arguments of the reference's
 * attention(q, k, v, causal, sm_scale) (flash.py:264-266) plus its outputs.
 *
 * m_begin/m_end select the query rows [m_begin, m_end) this call processes
 * (0, M for the whole problem).  Pointers always address logical row 0; rows
 * outside the window are neither read (q) nor written (out, log_normalizer,
 * scores, row_sum), so a rank that holds only its slice may pass
 * `slice_ptr - m_begin * stride_s`.  Column-type sums then cover the window's
 * queries only (the query-split multi-GPU variant sums them over ranks with
 * faws_reduce_ranks).
 */
typedef struct faws_problem {
  int32_t B, Hq, Hk, M, N, D;
  int32_t dtype;          /* FAWS_FP16 | FAWS_BF16 */
  int32_t causal;         /* 0 | 1 */
  float sm_scale;         /* scores = q.k^T * sm_scale */
  int32_t m_begin, m_end; /* query-row window */
  faws_tensor q, k, v, out;
  float* log_normalizer;  /* (B,Hq,M) fp32 contiguous or NULL: logsumexp of   */
                          /* the scaled scores, -inf for empty rows           */
                          /* (flash.py:480-486)                               */
  int32_t backend;        /* FAWS_BACKEND_* */
  /* Dropout on the softmax weights that multiply V (flash.py:463-466).  0 = off.  An entry
   * (b,h,i,j) is kept iff u > dropout_p, u being the first output of Philox-4x32 with 6 rounds
   * (triton's tl.rand(seed, c, n_rounds=6)) for key = philox_seed and counter
   * c = philox_offset + ((b*Hq + h)*M + i)*N + j in 32-bit wrap-around arithmetic
   * (flash.py:376-380).  The softmax normaliser and every raw-score output ignore the mask. */
  float dropout_p;        /* in [0, 1) */
  float dropout_scale;    /* out is multiplied by this when dropout_p > 0: 1/(1-p) in          */
                          /* attention and attention_with_scores (flash.py:488-491,             */
                          /* attention_with_scores.py:201-203), 1 in the reference's other      */
                          /* operators, which mask without rescaling                            */
  int32_t reserved;
  uint64_t philox_seed;
  uint64_t philox_offset; /* < 2^31 (beyond that triton switches to its 64-bit generator:      */
                          /* FAWS_EUNSUPPORTED)                                                 */
} faws_problem;

/* Replaces attention() forward (flash.py:264-295, kernel flash.py:335-498). */
int faws_attention(const faws_problem* p, void* stream);

/*
 * Replaces attention_with_scores (attention_with_scores.py:214-333).
 * scores: (B,Hq,M,N) contiguous, fp32 or the input dtype.  Visible entries get
 * q.k^T * sm_scale, hidden entries (causal) the fp32 bit pattern `masked_bits`
 * (0xFF800000 = -inf, the reference oracle's fill,
 * reference_implementations.py:40; 0 = the reference kernel's fill,
 * attention_with_scores.py:141-152), converted when scores are 16-bit.
 * Every element of the window's rows is written; no pre-fill is needed.
 */
int faws_attention_with_scores(const faws_problem* p, void* scores, int32_t scores_dtype,
                               uint32_t masked_bits, void* stream);

/*
 * Split-KV ("flash-decoding") form of faws_attention for problems with few query rows, where one
 * CTA per (batch, head, 128 query rows) would leave most SMs idle: replaces the split path of
 * FlashAttention.forward (flash.py:68-70,97-134; kernels split_kv.py:14-227).  The keys are cut
 * into n_splits contiguous ranges of whole 128-key tiles, each range is attended to by its own
 * CTAs, which leave a normalised partial result in the dtype of q and its log-normaliser in the
 * workspace (the reference's multiple_o / multiple_l, flash.py:106-107), and a combine kernel
 * merges the ranges in a fixed order (deterministic).  faws_split_kv_plan returns the number of
 * ranges the library would choose for p (the rule of split_kv.py:234-262; 1 = do not split: enough
 * CTAs already, dropout, a query-row window, or a problem the tcgen05 kernels cannot take).
 * Workspace: faws_workspace_bytes(FAWS_OP_ATTENTION_SPLIT_KV, p, n_splits).  Dropout is refused
 * (FAWS_EUNSUPPORTED), as in the reference (flash.py:98).
 */
int32_t faws_split_kv_plan(const faws_problem* p);
int faws_attention_split_kv(const faws_problem* p, int32_t n_splits, void* workspace, size_t workspace_bytes,
                            void* stream);

/*
 * Replaces compute_attention_scores (attention_scores.py:154-223, kernel :56-151): the score
 * tensor alone, scores = q.k^T * sm_scale, (B,Hq,M,N) contiguous in the dtype of q (what the
 * reference writes, :203) or fp32.  No mask is applied whatever p->causal says: the reference
 * accepts `causal` and ignores it (:166,:171,:195).  p->v, p->out and the query-row window are
 * not used.
 */
int faws_compute_attention_scores(const faws_problem* p, void* scores, int32_t scores_dtype, void* stream);

/* Replaces attention_with_row_sum (attention_with_row_sum.py:204-326).
 * row_sum: (B,Hq,M) fp32, sum over visible keys of q.k^T * sm_scale. */
int faws_attention_with_row_sum(const faws_problem* p, float* row_sum, void* stream);

/*
 * Replaces attention_with_col_sum (attention_with_col_sum.py:297-419): key
 * tiles are visited last-to-first when causal, round-robin otherwise
 * (:119-137, :207-216).  col_sum: per_q_head == 0: (B,Hk,N) fp32 summed over
 * the G query heads of a kv head (the reference's layout, :72,:370);
 * per_q_head != 0: (B,Hq,N).  Deterministic: per-query-block partial sums go
 * to `workspace` and a second kernel adds them in a fixed order (the
 * reference uses fp32 atomics, :186-191).
 */
int faws_attention_with_col_sum(const faws_problem* p, float* col_sum, int32_t per_q_head,
                                void* workspace, size_t workspace_bytes, void* stream);

/*
 * faws_attention_with_col_sum for callers that cannot supply a workspace: a host whose own
 * pool allocator owns the device and forbids cudaMalloc in plugins, a serving loop that
 * cannot afford the device-wide synchronisation of cudaMalloc/cudaFree, a plugin interface
 * that hands over tensor pointers only.  Same arguments and results as
 * faws_attention_with_col_sum minus the workspace; the per-query-tile partial sums go to a
 * fixed FAWS_NOALLOC_SCRATCH_BYTES array inside the library (held on every GPU that loads
 * the library until the process exits).  It has no counterpart in the reference.
 *  - Returns FAWS_ETOOLARGE when faws_workspace_bytes(FAWS_OP_COL_SUM, p, 0) exceeds
 *    FAWS_NOALLOC_SCRATCH_BYTES.
 *  - Calls no cudaMalloc / cudaFree / allocating routine.  The first call on a device
 *    resolves the array's address once; make it before any stream capture.
 *  - The array that is used is the current device's: make the device that holds the tensors
 *    current before the call (the same rule as for every other entry point's launches).
 *  - All calls on a device share the array: calls whose kernels may overlap on the GPU
 *    race; order them on one stream or with events.  Nothing needs to be zeroed between
 *    calls (each call writes every partial it later reads).
 */
#define FAWS_NOALLOC_SCRATCH_BYTES (8u << 20)
int faws_attention_with_col_sum_noalloc(const faws_problem* p, float* col_sum, int32_t per_q_head,
                                        void* stream);

/* Replaces attention_with_col_sum_sequential
 * (attention_with_col_sum_sequential.py:214-341): round-robin key-tile order
 * in all cases (:116-122).  Same result as faws_attention_with_col_sum. */
int faws_attention_with_col_sum_sequential(const faws_problem* p, float* col_sum,
                                           int32_t per_q_head, void* workspace,
                                           size_t workspace_bytes, void* stream);

/*
 * Replaces attention_with_softmax_col_sum
 * (attention_with_col_softmax_sum.py:274-401): col_sum[j] = sum over queries
 * of softmax(scores)[i][j].  Pass 1 is plain attention writing out and the
 * log-normaliser; pass 2 is a key-major kernel that recomputes q.k^T and uses
 * P = exp(s - L_i) (the reference's second pass, :195-270, without atomics).
 */
int faws_attention_with_softmax_col_sum(const faws_problem* p, float* col_sum,
                                        int32_t per_q_head, void* workspace,
                                        size_t workspace_bytes, void* stream);

/*
 * Replaces attention_cross_token_qk_sum
 * (attention_cross_token_qk_sum.py:255-408).  sum_out: (B,Hk,split) or
 * (B,Hq,split) fp32; sum over queries i >= split of the visible scaled score
 * into keys j < split.  Requires 0 < split <= N (:307).
 */
int faws_attention_cross_token_qk_sum(const faws_problem* p, int32_t split, float* sum_out,
                                      int32_t per_q_head, void* workspace,
                                      size_t workspace_bytes, void* stream);

/* Replaces attention_cross_token_softmax_sum
 * (attention_cross_token_softmax_sum.py:735-863): softmax-weight version of
 * the above, second q.k^T over the cross region only. */
int faws_attention_cross_token_softmax_sum(const faws_problem* p, int32_t split, float* sum_out,
                                           int32_t per_q_head, void* workspace,
                                           size_t workspace_bytes, void* stream);

/*
 * Replaces attention_cross_token_softmax_sum_buffered
 * (attention_cross_token_softmax_sum.py:639-732).  Pass 1 stores the scaled
 * raw scores of the cross region only (queries >= split, keys < split; the
 * reference stores the whole (B,H,M,N) tensor, :705) in the workspace; pass 2
 * reads them back instead of recomputing q.k^T.
 */
int faws_attention_cross_token_softmax_sum_buffered(const faws_problem* p, int32_t split,
                                                    float* sum_out, int32_t per_q_head,
                                                    void* workspace, size_t workspace_bytes,
                                                    void* stream);

/*
 * Replaces total_attention (total.py:9-47, kernel total.py:50-142), the
 * per-query-head softmax column sum computed from a saved log-normaliser:
 * total[b,h,j] = sum_i exp(s_ij - L_i).  p->log_normalizer is an INPUT here;
 * v and out are ignored.  total: (B,Hq,N) fp32.
 */
int faws_total_attention(const faws_problem* p, float* total, void* stream);

/*
 * Replaces FlashAttention.backward (flash.py:172-261; kernels flash.py:532-577 delta pre-pass,
 * :581-754 dK/dV, :758-918 dQ).  Inputs: p->q, p->k, p->v, p->out (the forward result),
 * p->log_normalizer (the forward pass's L, required) and g->dout, the gradient of out.  Outputs:
 * g->dq (B,Hq,M,D); g->dk, g->dv (B,Hk,N,D), already summed over the G query heads of each kv head
 * (the reference sums per-query-head tensors on the host, flash.py:259-260).  All tensors in the
 * dtype of q.  Dropout: pass the forward call's dropout_p and philox pair; dropout_scale is not
 * used (kept weights are rescaled by 1/(1-p), flash.py:655,713,724).  The query-row window must
 * be the whole problem.  Deterministic: no atomics.  Workspace:
 * faws_workspace_bytes(FAWS_OP_ATTENTION_BACKWARD, p, 0).
 */
typedef struct faws_grads {
  faws_tensor dout, dq, dk, dv;
} faws_grads;
int faws_attention_backward(const faws_problem* p, const faws_grads* g, void* workspace,
                            size_t workspace_bytes, void* stream);

/* Bytes of scratch `op` needs for `p` (0 if none).  Alignment: 256 bytes. */
size_t faws_workspace_bytes(int32_t op, const faws_problem* p, int32_t split);

/*
 * Query-split multi-GPU variant: out[i] = parts[0][i] + parts[1][i] + ... in
 * rank order (deterministic).  parts: n_ranks contiguous vectors of `count`
 * floats each, rank-major, in this GPU's own memory (e.g. the landing buffer
 * of an all-gather).  No counterpart in the reference (it is single-GPU).
 */
int faws_reduce_ranks(const float* parts, int32_t n_ranks, int64_t count, float* out,
                      void* stream);

/*
 * The tcgen05 kernels bound every wait on an mbarrier (2 s).  A CTA that gives up
 * raises a per-device status word, frees its TMEM and returns; its outputs are then
 * invalid.  This call synchronises the device and returns that word (0 = no give-up,
 * 1 = some wait gave up, -1 = the word could not be read); `reset` != 0 clears it.
 * No counterpart in the reference.
 */
int faws_device_status(int32_t reset);

/*
 * Self-test of that give-up path: launches one tiny kernel whose only thread waits, with a limit
 * of about a millisecond, on an mbarrier nobody arrives at.  The wait runs out, the kernel raises
 * the status word and returns normally (nothing faults, nothing hangs); faws_device_status then
 * reads 1.  No counterpart in the reference.
 */
int faws_selftest_wait_give_up(void* stream);

/* Which kernel family the calling thread's last successful call used
 * (FAWS_BACKEND_GENERIC or FAWS_BACKEND_TCGEN05; 0 before any call) and how
 * many kernels this library has launched from this process. */
int faws_last_backend(void);
int64_t faws_launch_count(void);

const char* faws_strerror(int status);
int faws_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FAWS_H_ */
