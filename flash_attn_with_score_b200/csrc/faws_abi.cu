// extern "C" entry points declared in include/faws.h: argument validation,
// workspace carving, kernel-family selection and the launch sequences.
#include <atomic>
#include <cstdio>

#include "faws_internal.cuh"

namespace faws {

static std::atomic<int64_t> g_launches{0};
static thread_local int t_last_backend = 0;
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

namespace {

inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }
inline int cdiv(int a, int b) { return (a + b - 1) / b; }

int validate(const faws_problem* p) {
  if (p == nullptr) return FAWS_EINVAL;
  if (p->B <= 0 || p->Hq <= 0 || p->Hk <= 0 || p->M <= 0 || p->N <= 0) return FAWS_EINVAL;
  if (p->Hq % p->Hk != 0) return FAWS_EINVAL;
  if (p->D != 16 && p->D != 32 && p->D != 64 && p->D != 128) return FAWS_EUNSUPPORTED;
  if (p->dtype != FAWS_FP16 && p->dtype != FAWS_BF16) return FAWS_EUNSUPPORTED;
  if (p->m_begin < 0 || p->m_end > p->M || p->m_begin > p->m_end) return FAWS_EINVAL;
  if (!(p->dropout_p >= 0.f && p->dropout_p < 1.f)) return FAWS_EINVAL;
  if (p->dropout_p > 0.f && p->philox_offset >= (1ull << 31)) return FAWS_EUNSUPPORTED;
  if (p->q.ptr == nullptr || p->k.ptr == nullptr) return FAWS_EINVAL;
  if (p->backend < FAWS_BACKEND_AUTO || p->backend > FAWS_BACKEND_TCGEN05) return FAWS_EINVAL;
  return FAWS_OK;
}

DropoutParams make_drop(const faws_problem* p) {
  DropoutParams d{};
  if (p->dropout_p > 0.f) {
    d.p = p->dropout_p;
    d.out_scale = p->dropout_scale;
    d.seed_lo = static_cast<uint32_t>(p->philox_seed);
    d.seed_hi = static_cast<uint32_t>(p->philox_seed >> 32);
    d.offset = static_cast<uint32_t>(p->philox_offset);
  }
  return d;
}

FwdParams make_fwd(const faws_problem* p) {
  FwdParams f{};
  f.q = p->q.ptr; f.k = p->k.ptr; f.v = p->v.ptr; f.o = p->out.ptr;
  f.q_sb = p->q.stride_b; f.q_sh = p->q.stride_h; f.q_ss = p->q.stride_s;
  f.k_sb = p->k.stride_b; f.k_sh = p->k.stride_h; f.k_ss = p->k.stride_s;
  f.v_sb = p->v.stride_b; f.v_sh = p->v.stride_h; f.v_ss = p->v.stride_s;
  f.o_sb = p->out.stride_b; f.o_sh = p->out.stride_h; f.o_ss = p->out.stride_s;
  f.L = p->log_normalizer;
  f.B = p->B; f.Hq = p->Hq; f.Hk = p->Hk; f.G = p->Hq / p->Hk;
  f.M = p->M; f.N = p->N; f.D = p->D;
  f.p_seq = p->N - p->M;
  f.m_begin = p->m_begin; f.m_end = p->m_end;
  f.causal = p->causal ? 1 : 0;
  f.sm_scale = p->sm_scale;
  f.schedule = kForward;
  f.masked_bits = 0xff800000u;
  f.scores_f32 = 1;
  f.drop = make_drop(p);
  return f;
}

// Scratch must start on a 256-byte boundary (faws_workspace_bytes says so): the kernels read and write it with
// 16-byte vectors, TMA stores and bulk copies.
bool misaligned_ws(const void* ws) { return reinterpret_cast<uintptr_t>(ws) % 256 != 0; }

ColSoftmaxParams make_cs(const faws_problem* p, const float* L, float* out, int i_begin, int n_end) {
  ColSoftmaxParams c{};
  c.q = p->q.ptr; c.k = p->k.ptr;
  c.q_sb = p->q.stride_b; c.q_sh = p->q.stride_h; c.q_ss = p->q.stride_s;
  c.k_sb = p->k.stride_b; c.k_sh = p->k.stride_h; c.k_ss = p->k.stride_s;
  c.L = L; c.out = out;
  c.B = p->B; c.Hq = p->Hq; c.Hk = p->Hk; c.G = p->Hq / p->Hk;
  c.M = p->M; c.N = p->N; c.D = p->D;
  c.p_seq = p->N - p->M; c.m_begin = p->m_begin; c.m_end = p->m_end;
  c.causal = p->causal ? 1 : 0; c.sm_scale = p->sm_scale;
  c.i_begin = i_begin; c.n_end = n_end;
  return c;
}

// Runs the forward kernel on the family that fits; reports which one ran.
int run_fwd(const faws_problem* p, FwdParams& f, cudaStream_t s, int* block_m, int* block_n) {
  if (f.v == nullptr || f.o == nullptr) return FAWS_EINVAL;
  bool use_tc = false;
  if (p->backend != FAWS_BACKEND_GENERIC) use_tc = tc_fwd_supported(f, p->dtype);
  if (p->backend == FAWS_BACKEND_TCGEN05 && !use_tc) return FAWS_EBACKEND;
  if (!use_tc) f.col_lin = 0;
  *block_m = use_tc ? kTcBlockM : kGenericBlockM;
  *block_n = use_tc ? kTcBlockN : kGenericBlockN;
  if (f.col_partial != nullptr) {
    f.ncols_pad = cdiv(f.col_n_end, 128) * 128;
    f.qb_first = (f.col_row_begin > f.m_begin ? f.col_row_begin : f.m_begin) / *block_m;
    f.n_qb_part = cdiv(f.m_end, *block_m) - f.qb_first;
    if (f.n_qb_part < 0) f.n_qb_part = 0;
  }
  cudaError_t e = use_tc ? launch_tc_fwd(f, p->dtype, s) : launch_generic_fwd(f, p->dtype, s);
  if (e != cudaSuccess) {
    std::fprintf(stderr, "faws: forward launch failed: %s\n", cudaGetErrorString(e));
    return FAWS_ECUDA;
  }
  t_last_backend = use_tc ? FAWS_BACKEND_TCGEN05 : FAWS_BACKEND_GENERIC;
  return FAWS_OK;
}

// Key-major pass.  `final_out` receives (B,Hk,n_end) when group_sum != 0, else (B,Hq,n_end);
// `per_head_ws` is scratch for the per-head sums when the CUDA-core kernel has to be followed
// by a group sum.
int run_colsoftmax(const faws_problem* p, ColSoftmaxParams& c, float* final_out, float* per_head_ws,
                   int group_sum, cudaStream_t s) {
  bool use_tc = false;
  if (p->backend != FAWS_BACKEND_GENERIC) use_tc = tc_colsoftmax_supported(c, p->dtype);
  if (p->backend == FAWS_BACKEND_TCGEN05 && !use_tc && c.s_scratch == nullptr) return FAWS_EBACKEND;
  cudaError_t e;
  if (c.s_scratch != nullptr) {  // buffered variant: stream the stored scores back
    // one CTA per (128 keys, query head): G times more CTAs in flight than walking the group inside
    // the CTA, which this bandwidth-bound pass needs; the G heads are added afterwards
    const bool direct = !group_sum || c.G == 1;
    c.out = direct ? final_out : per_head_ws;
    e = launch_scratch_colsum(c, 0, s);
    if (e == cudaSuccess && !direct) e = launch_group_sum(per_head_ws, final_out, c.B, c.Hk, c.G, c.n_end, s);
  } else if (use_tc) {
    const bool in_kernel = !group_sum || tc_colsoftmax_group_in_kernel(c);
    c.out = in_kernel ? final_out : per_head_ws;
    e = launch_tc_colsoftmax(c, p->dtype, in_kernel ? group_sum : 0, s);
    if (e == cudaSuccess && !in_kernel) e = launch_group_sum(per_head_ws, final_out, c.B, c.Hk, c.G, c.n_end, s);
  } else {
    const bool direct = !group_sum || c.G == 1;
    c.out = direct ? final_out : per_head_ws;
    e = launch_generic_colsoftmax(c, p->dtype, s);
    if (e == cudaSuccess && !direct) e = launch_group_sum(per_head_ws, final_out, c.B, c.Hk, c.G, c.n_end, s);
  }
  if (e != cudaSuccess) {
    std::fprintf(stderr, "faws: column-softmax launch failed: %s\n", cudaGetErrorString(e));
    return FAWS_ECUDA;
  }
  return FAWS_OK;
}

// per-128-row-tile sums of the query rows, (B,Hq,ceil(M/128),128) floats
size_t qsum_floats(const faws_problem* p) { return (size_t)p->B * p->Hq * cdiv(p->M, 128) * 128; }

size_t partial_floats(const faws_problem* p, int row_begin, int n_end) {
  const int first = (row_begin > p->m_begin ? row_begin : p->m_begin) / kGenericBlockM;
  int nqb = cdiv(p->m_end, kGenericBlockM) - first;
  if (nqb < 0) nqb = 0;
  return (size_t)p->B * p->Hq * nqb * (size_t)(cdiv(n_end, 128) * 128);
}

// Raw column-type sums: forward pass with per-query-block partials + fixed-order reduce.
int raw_col_sums(const faws_problem* p, float* sum_out, int per_q_head, void* ws, size_t ws_bytes,
                 void* stream, int schedule, int row_begin, int n_end) {
  int st = validate(p);
  if (st != FAWS_OK) return st;
  if (sum_out == nullptr) return FAWS_EINVAL;
  const size_t part_bytes = align256(partial_floats(p, row_begin, n_end) * 4);
  const size_t need = part_bytes + align256(qsum_floats(p) * 4);
  if (ws == nullptr || ws_bytes < need || misaligned_ws(ws)) return FAWS_EWORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  FwdParams f = make_fwd(p);
  f.schedule = schedule;
  f.col_partial = static_cast<float*>(ws);
  f.col_row_begin = row_begin;
  f.col_n_end = n_end;
  f.col_lin = 1;  // cleared by run_fwd when the CUDA-core kernels run
  f.col_row_lo = row_begin > p->m_begin ? row_begin : p->m_begin;
  float* qsum = reinterpret_cast<float*>(static_cast<char*>(ws) + part_bytes);
  f.qsum = qsum;  // the tcgen05 forward kernel writes the per-tile query sums itself
  int bm = 0, bn = 0;
  st = run_fwd(p, f, s, &bm, &bn);
  if (st != FAWS_OK) return st;
  ReducePartialParams r{};
  r.partial = f.col_partial; r.out = sum_out;
  r.B = p->B; r.Hq = p->Hq; r.Hk = p->Hk; r.G = p->Hq / p->Hk; r.per_q_head = per_q_head ? 1 : 0;
  r.n_end = n_end; r.ncols_pad = f.ncols_pad; r.n_qb_part = f.n_qb_part; r.qb_first = f.qb_first;
  r.block_m = bm; r.block_n = bn;
  r.causal = f.causal; r.p_seq = f.p_seq; r.N = p->N; r.m_end = p->m_end;
  r.lin = f.col_lin; r.qsum = qsum; r.nqb_total = cdiv(p->M, 128); r.D = p->D; r.row_lo = f.col_row_lo;
  r.k = f.k; r.k_sb = f.k_sb; r.k_sh = f.k_sh; r.k_ss = f.k_ss; r.sm_scale = f.sm_scale;
  if (launch_reduce_partials(r, p->dtype, s) != cudaSuccess) return FAWS_ECUDA;
  return FAWS_OK;
}

struct SoftmaxWs {
  float* L;
  float* per_head;
  float* negl;  // (B,Hq,M rounded up to 128): -L*log2e for the key-major tcgen05 kernel
  float* scratch;
  size_t total;
};

SoftmaxWs carve_softmax_ws(const faws_problem* p, void* ws, int n_end, int split_for_scratch) {
  SoftmaxWs w{};
  size_t off = 0;
  char* base = static_cast<char*>(ws);
  const size_t lbytes = align256((size_t)p->B * p->Hq * p->M * 4);
  const size_t hbytes = align256((size_t)p->B * p->Hq * (size_t)n_end * 4);
  w.L = reinterpret_cast<float*>(base + off); off += lbytes;
  w.per_head = reinterpret_cast<float*>(base + off); off += hbytes;
  w.negl = reinterpret_cast<float*>(base + off); off += align256((size_t)p->B * p->Hq * (size_t)(cdiv(p->M, 128) * 128) * 4);
  if (split_for_scratch > 0 && p->M > split_for_scratch) {
    w.scratch = reinterpret_cast<float*>(base + off);
    off += align256((size_t)p->B * p->Hq * (size_t)(p->M - split_for_scratch) * split_for_scratch * 4);
  }
  w.total = off;
  return w;
}

// Softmax-normalised column-type sums: forward pass (out, L[, score scratch]) then the
// key-major pass and, unless per-q-head output was asked for, the group sum.
int softmax_col_sums(const faws_problem* p, float* sum_out, int per_q_head, void* ws, size_t ws_bytes,
                     void* stream, int i_begin, int n_end, int buffered_split, int schedule,
                     bool dropout_in_sum = false) {
  int st = validate(p);
  if (st != FAWS_OK) return st;
  if (sum_out == nullptr) return FAWS_EINVAL;
  SoftmaxWs w = carve_softmax_ws(p, nullptr, n_end, buffered_split);
  if (ws == nullptr || ws_bytes < w.total || misaligned_ws(ws)) return FAWS_EWORKSPACE;
  w = carve_softmax_ws(p, ws, n_end, buffered_split);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  FwdParams f = make_fwd(p);
  f.schedule = schedule;
  if (f.L == nullptr) f.L = w.L;
  if (w.scratch != nullptr) { f.s_scratch = w.scratch; f.split = buffered_split; }
  int bm = 0, bn = 0;
  st = run_fwd(p, f, s, &bm, &bn);
  if (st != FAWS_OK) return st;
  ColSoftmaxParams c = make_cs(p, f.L, sum_out, i_begin, n_end);
  if (w.scratch != nullptr) { c.s_scratch = w.scratch; c.split = buffered_split; }
  if (dropout_in_sum) c.drop = make_drop(p);
  c.after_forward = 1;
  c.negl_pad = w.negl;  // (16-byte aligned like every region of the scratch: bulk copies read it)
  c.m_pad = cdiv(p->M, 128) * 128;
  if (i_begin >= p->m_end) {
    // no query of the window lies beyond the split: the sums are zero
    if (cudaMemsetAsync(sum_out, 0, (size_t)p->B * (per_q_head ? p->Hq : p->Hk) * (size_t)n_end * 4, s) != cudaSuccess)
      return FAWS_ECUDA;
    return FAWS_OK;
  }
  return run_colsoftmax(p, c, sum_out, w.per_head, per_q_head ? 0 : 1, s);
}

// Decoding with grouped queries: when the G query heads of a kv head have so few rows that all of them
// fit one 128-row tile, they are run as ONE head of G*M rows, so K and V are streamed once per kv head
// instead of once per query head.  Pure re-indexing: row r = g*M + i of the packed head is row i of query
// head hk*G + g, which for contiguous heads (stride_h == M * stride_s) is a plain row stride; out and L
// index the same way.  Needs an unmasked problem (not causal, or a single query row, which sees every key).
bool pack_gqa(const faws_problem* p, faws_problem* packed) {
  const int G = p->Hq / p->Hk;
  if (G <= 1 || (long long)G * p->M > kTcBlockM) return false;
  if (p->causal && p->M != 1) return false;
  if (p->causal && p->N < p->M) return false;
  if (p->dropout_p > 0.f || p->m_begin != 0 || p->m_end != p->M) return false;
  if (p->out.ptr == nullptr) return false;
  if (p->q.stride_h != (int64_t)p->M * p->q.stride_s || p->out.stride_h != (int64_t)p->M * p->out.stride_s) return false;
  *packed = *p;
  packed->Hq = p->Hk;
  packed->M = G * p->M;
  packed->m_end = G * p->M;
  packed->causal = 0;
  packed->q.stride_h = p->q.stride_h * G;
  packed->out.stride_h = p->out.stride_h * G;
  return true;
}

// Number of key ranges for a problem that leaves most SMs idle: the plan of the reference's
// num_splits_herustic (split_kv.py:234-262; its tiles are 16 x 128, here 128 x 128), i.e. the
// smallest count whose wave efficiency is within 85 % of the best, among counts that leave no range
// empty.
int plan_splits(const faws_problem* p, int sms) {
  const long long ctas = (long long)p->B * p->Hq * cdiv(p->M, kTcBlockM);
  if (ctas * 10 >= 8LL * sms) return 1;
  const int nkt = cdiv(p->N, kTcBlockN);
  int max_splits = sms < nkt ? sms : nkt;
  if (max_splits > 128) max_splits = 128;
  if ((long long)p->B * max_splits > 65535) max_splits = 65535 / p->B;
  double best = 0.0;
  double eff[129];
  for (int s = 1; s <= max_splits; ++s) {
    const int per = cdiv(nkt, s);
    eff[s] = -1.0;
    if (s > 1 && per * s - nkt >= per) continue;  // the last range would be empty
    const double waves = (double)(ctas * s) / sms;
    const double whole = waves > (double)(long long)waves ? (double)((long long)waves + 1) : waves;
    eff[s] = waves / whole;
    if (eff[s] > best) best = eff[s];
  }
  for (int s = 1; s <= max_splits; ++s)
    if (eff[s] >= 0.85 * best) return s;
  return 1;
}

size_t split_kv_bytes(const faws_problem* p, int n_splits) {
  return align256((size_t)p->B * p->Hq * n_splits * p->M * 4) +
         align256((size_t)p->B * p->Hq * n_splits * p->M * p->D * 2);
}

}  // namespace
}  // namespace faws

using namespace faws;

extern "C" {

int faws_attention(const faws_problem* p, void* stream) {
  int st = validate(p);
  if (st != FAWS_OK) return st;
  faws_problem packed;
  if (p->backend != FAWS_BACKEND_GENERIC && pack_gqa(p, &packed)) {
    FwdParams fp = make_fwd(&packed);
    if (fp.v != nullptr && tc_fwd_supported(fp, packed.dtype)) p = &packed;
  }
  FwdParams f = make_fwd(p);
  int bm, bn;
  return run_fwd(p, f, static_cast<cudaStream_t>(stream), &bm, &bn);
}

int faws_attention_with_scores(const faws_problem* p, void* scores, int32_t scores_dtype,
                               uint32_t masked_bits, void* stream) {
  int st = validate(p);
  if (st != FAWS_OK) return st;
  if (scores == nullptr) return FAWS_EINVAL;
  if (scores_dtype != FAWS_SCORES_F32 && scores_dtype != FAWS_SCORES_INPUT) return FAWS_EINVAL;
  FwdParams f = make_fwd(p);
  f.scores = scores;
  f.scores_f32 = scores_dtype == FAWS_SCORES_F32 ? 1 : 0;
  f.masked_bits = masked_bits;
  int bm, bn;
  return run_fwd(p, f, static_cast<cudaStream_t>(stream), &bm, &bn);
}

int32_t faws_split_kv_plan(const faws_problem* p) {
  if (validate(p) != FAWS_OK) return 1;
  if (p->dropout_p > 0.f || p->m_begin != 0 || p->m_end != p->M || p->backend == FAWS_BACKEND_GENERIC) return 1;
  if (p->v.ptr == nullptr || p->out.ptr == nullptr) return 1;
  faws_problem packed;
  if (pack_gqa(p, &packed)) {
    FwdParams fp = make_fwd(&packed);
    if (tc_fwd_supported(fp, packed.dtype)) p = &packed;
  }
  FwdParams f = make_fwd(p);
  if (!tc_fwd_supported(f, p->dtype)) return 1;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return plan_splits(p, sms);
}

int faws_attention_split_kv(const faws_problem* p, int32_t n_splits, void* workspace, size_t workspace_bytes,
                            void* stream) {
  int st = validate(p);
  if (st != FAWS_OK) return st;
  const int nkt = cdiv(p->N, kTcBlockN);
  if (n_splits < 1 || n_splits > nkt || (long long)p->B * n_splits > 65535) return FAWS_EINVAL;
  if (p->dropout_p > 0.f) return FAWS_EUNSUPPORTED;  // the reference refuses dropout with split-KV too (flash.py:98)
  if (p->m_begin != 0 || p->m_end != p->M) return FAWS_EINVAL;
  if (n_splits == 1) return faws_attention(p, stream);
  if (workspace == nullptr || workspace_bytes < split_kv_bytes(p, n_splits) || misaligned_ws(workspace))
    return FAWS_EWORKSPACE;
  if (p->out.ptr == nullptr || p->v.ptr == nullptr) return FAWS_EINVAL;
  faws_problem packed;  // same bytes of workspace either way: B*Hq*M is unchanged by the packing
  if (p->backend != FAWS_BACKEND_GENERIC && pack_gqa(p, &packed)) {
    FwdParams fp = make_fwd(&packed);
    if (tc_fwd_supported(fp, packed.dtype)) p = &packed;
  }
  FwdParams f = make_fwd(p);
  if (p->backend == FAWS_BACKEND_GENERIC || !tc_fwd_supported(f, p->dtype)) return FAWS_EBACKEND;
  float* L_part = static_cast<float*>(workspace);
  char* o_part = static_cast<char*>(workspace) + align256((size_t)p->B * p->Hq * n_splits * p->M * 4);
  f.o = o_part;
  f.o_ss = p->D;
  f.o_sh = (int64_t)p->M * p->D;  // per (query head, key range)
  f.o_sb = (int64_t)p->Hq * n_splits * p->M * p->D;
  f.L = L_part;
  f.n_splits = n_splits;
  f.tiles_per_split = cdiv(nkt, n_splits);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (launch_tc_fwd(f, p->dtype, s) != cudaSuccess) return FAWS_ECUDA;
  if (launch_combine_splits(o_part, L_part, p->out.ptr, p->out.stride_b, p->out.stride_h, p->out.stride_s,
                            p->log_normalizer, p->B, p->Hq, p->M, p->D, n_splits, p->dtype, s) != cudaSuccess)
    return FAWS_ECUDA;
  t_last_backend = FAWS_BACKEND_TCGEN05;
  return FAWS_OK;
}

int faws_compute_attention_scores(const faws_problem* p, void* scores, int32_t scores_dtype, void* stream) {
  int st = validate(p);
  if (st != FAWS_OK) return st;
  if (scores == nullptr) return FAWS_EINVAL;
  if (scores_dtype != FAWS_SCORES_F32 && scores_dtype != FAWS_SCORES_INPUT) return FAWS_EINVAL;
  ScoresOnlyParams sp{};
  sp.q = p->q.ptr; sp.k = p->k.ptr;
  sp.q_sb = p->q.stride_b; sp.q_sh = p->q.stride_h; sp.q_ss = p->q.stride_s;
  sp.k_sb = p->k.stride_b; sp.k_sh = p->k.stride_h; sp.k_ss = p->k.stride_s;
  sp.scores = scores;
  sp.scores_f32 = scores_dtype == FAWS_SCORES_F32 ? 1 : 0;
  sp.B = p->B; sp.Hq = p->Hq; sp.Hk = p->Hk; sp.M = p->M; sp.N = p->N; sp.D = p->D;
  sp.sm_scale = p->sm_scale;
  bool use_tc = false;
  if (p->backend != FAWS_BACKEND_GENERIC) use_tc = tc_scores_only_supported(sp, p->dtype);
  if (p->backend == FAWS_BACKEND_TCGEN05 && !use_tc) return FAWS_EBACKEND;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const cudaError_t e = use_tc ? launch_tc_scores_only(sp, p->dtype, s) : launch_generic_scores_only(sp, p->dtype, s);
  if (e != cudaSuccess) {
    std::fprintf(stderr, "faws: score-only launch failed: %s\n", cudaGetErrorString(e));
    return FAWS_ECUDA;
  }
  t_last_backend = use_tc ? FAWS_BACKEND_TCGEN05 : FAWS_BACKEND_GENERIC;
  return FAWS_OK;
}

int faws_attention_with_row_sum(const faws_problem* p, float* row_sum, void* stream) {
  int st = validate(p);
  if (st != FAWS_OK) return st;
  if (row_sum == nullptr) return FAWS_EINVAL;
  FwdParams f = make_fwd(p);
  f.row_sum = row_sum;
  int bm, bn;
  return run_fwd(p, f, static_cast<cudaStream_t>(stream), &bm, &bn);
}

int faws_attention_with_col_sum(const faws_problem* p, float* col_sum, int32_t per_q_head,
                                void* workspace, size_t workspace_bytes, void* stream) {
  if (p == nullptr) return FAWS_EINVAL;
  return raw_col_sums(p, col_sum, per_q_head, workspace, workspace_bytes, stream,
                      p->causal ? kReverse : kRoundRobin, 0, p->N);
}

int faws_attention_with_col_sum_sequential(const faws_problem* p, float* col_sum, int32_t per_q_head,
                                           void* workspace, size_t workspace_bytes, void* stream) {
  if (p == nullptr) return FAWS_EINVAL;
  return raw_col_sums(p, col_sum, per_q_head, workspace, workspace_bytes, stream, kRoundRobin, 0, p->N);
}

int faws_attention_with_softmax_col_sum(const faws_problem* p, float* col_sum, int32_t per_q_head,
                                        void* workspace, size_t workspace_bytes, void* stream) {
  if (p == nullptr) return FAWS_EINVAL;
  // the one operator whose sum sees the dropout mask (attention_with_col_softmax_sum.py:238-244)
  return softmax_col_sums(p, col_sum, per_q_head, workspace, workspace_bytes, stream, 0, p->N, 0,
                          kRoundRobin, /*dropout_in_sum=*/true);
}

int faws_attention_cross_token_qk_sum(const faws_problem* p, int32_t split, float* sum_out,
                                      int32_t per_q_head, void* workspace, size_t workspace_bytes,
                                      void* stream) {
  if (p == nullptr || split <= 0 || split > p->N) return FAWS_EINVAL;
  return raw_col_sums(p, sum_out, per_q_head, workspace, workspace_bytes, stream, kForward, split, split);
}

int faws_attention_cross_token_softmax_sum(const faws_problem* p, int32_t split, float* sum_out,
                                           int32_t per_q_head, void* workspace,
                                           size_t workspace_bytes, void* stream) {
  if (p == nullptr || split <= 0 || split > p->N) return FAWS_EINVAL;
  return softmax_col_sums(p, sum_out, per_q_head, workspace, workspace_bytes, stream, split, split, 0,
                          kRoundRobin);
}

int faws_attention_cross_token_softmax_sum_buffered(const faws_problem* p, int32_t split,
                                                    float* sum_out, int32_t per_q_head,
                                                    void* workspace, size_t workspace_bytes,
                                                    void* stream) {
  if (p == nullptr || split <= 0 || split > p->N) return FAWS_EINVAL;
  return softmax_col_sums(p, sum_out, per_q_head, workspace, workspace_bytes, stream, split, split,
                          split, kForward);
}

int faws_total_attention(const faws_problem* p, float* total, void* stream) {
  int st = validate(p);
  if (st != FAWS_OK) return st;
  if (total == nullptr || p->log_normalizer == nullptr) return FAWS_EINVAL;
  ColSoftmaxParams c = make_cs(p, p->log_normalizer, total, 0, p->N);
  return run_colsoftmax(p, c, total, nullptr, 0, static_cast<cudaStream_t>(stream));
}

int faws_attention_backward(const faws_problem* p, const faws_grads* g, void* workspace,
                            size_t workspace_bytes, void* stream) {
  int st = validate(p);
  if (st != FAWS_OK) return st;
  if (g == nullptr || p->v.ptr == nullptr || p->out.ptr == nullptr || p->log_normalizer == nullptr ||
      g->dout.ptr == nullptr || g->dq.ptr == nullptr || g->dk.ptr == nullptr || g->dv.ptr == nullptr)
    return FAWS_EINVAL;
  if (p->m_begin != 0 || p->m_end != p->M) return FAWS_EINVAL;
  const size_t need = faws_workspace_bytes(FAWS_OP_ATTENTION_BACKWARD, p, 0);
  if (workspace == nullptr || workspace_bytes < need || misaligned_ws(workspace)) return FAWS_EWORKSPACE;
  BwdParams b{};
  b.q = p->q.ptr; b.k = p->k.ptr; b.v = p->v.ptr; b.o = p->out.ptr;
  b.dout = g->dout.ptr; b.dq = g->dq.ptr; b.dk = g->dk.ptr; b.dv = g->dv.ptr;
  b.q_sb = p->q.stride_b; b.q_sh = p->q.stride_h; b.q_ss = p->q.stride_s;
  b.k_sb = p->k.stride_b; b.k_sh = p->k.stride_h; b.k_ss = p->k.stride_s;
  b.v_sb = p->v.stride_b; b.v_sh = p->v.stride_h; b.v_ss = p->v.stride_s;
  b.o_sb = p->out.stride_b; b.o_sh = p->out.stride_h; b.o_ss = p->out.stride_s;
  b.do_sb = g->dout.stride_b; b.do_sh = g->dout.stride_h; b.do_ss = g->dout.stride_s;
  b.dq_sb = g->dq.stride_b; b.dq_sh = g->dq.stride_h; b.dq_ss = g->dq.stride_s;
  b.dk_sb = g->dk.stride_b; b.dk_sh = g->dk.stride_h; b.dk_ss = g->dk.stride_s;
  b.dv_sb = g->dv.stride_b; b.dv_sh = g->dv.stride_h; b.dv_ss = g->dv.stride_s;
  b.L = p->log_normalizer;
  b.delta = static_cast<float*>(workspace);
  b.B = p->B; b.Hq = p->Hq; b.Hk = p->Hk; b.G = p->Hq / p->Hk; b.M = p->M; b.N = p->N; b.D = p->D;
  b.p_seq = p->N - p->M; b.causal = p->causal ? 1 : 0; b.sm_scale = p->sm_scale;
  b.drop = make_drop(p);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  bool use_tc = false;
  if (p->backend != FAWS_BACKEND_GENERIC) use_tc = tc_bwd_supported(b, p->dtype);
  if (p->backend == FAWS_BACKEND_TCGEN05 && !use_tc) return FAWS_EBACKEND;
  // the tcgen05 path has its own pre-pass (delta and L into tile-padded arrays in the workspace)
  if (!use_tc && launch_bwd_delta(b, p->dtype, s) != cudaSuccess) return FAWS_ECUDA;
  const cudaError_t e = use_tc ? launch_tc_bwd(b, p->dtype, s) : launch_generic_bwd(b, p->dtype, s);
  if (e != cudaSuccess) {
    std::fprintf(stderr, "faws: backward launch failed: %s\n", cudaGetErrorString(e));
    return FAWS_ECUDA;
  }
  t_last_backend = use_tc ? FAWS_BACKEND_TCGEN05 : FAWS_BACKEND_GENERIC;
  return FAWS_OK;
}

size_t faws_workspace_bytes(int32_t op, const faws_problem* p, int32_t split) {
  if (validate(p) != FAWS_OK) return 0;
  switch (op) {
    case FAWS_OP_ATTENTION_SPLIT_KV:  // `split` carries the number of key ranges
      if (split < 1 || split > cdiv(p->N, kTcBlockN)) return 0;
      return split == 1 ? 0 : split_kv_bytes(p, split);
    case FAWS_OP_ATTENTION_BACKWARD:  // enough for either kernel family
      return tc_bwd_workspace_bytes(p->B, p->Hq, p->Hk, p->M, p->N, p->D);
    case FAWS_OP_COL_SUM:
    case FAWS_OP_COL_SUM_SEQUENTIAL:
      return align256(partial_floats(p, 0, p->N) * 4) + align256(qsum_floats(p) * 4);
    case FAWS_OP_CROSS_QK_SUM:
      if (split <= 0 || split > p->N) return 0;
      return align256(partial_floats(p, split, split) * 4) + align256(qsum_floats(p) * 4);
    case FAWS_OP_SOFTMAX_COL_SUM:
      return carve_softmax_ws(p, nullptr, p->N, 0).total;
    case FAWS_OP_CROSS_SOFTMAX_SUM:
      if (split <= 0 || split > p->N) return 0;
      return carve_softmax_ws(p, nullptr, split, 0).total;
    case FAWS_OP_CROSS_SOFTMAX_SUM_BUFFERED:
      if (split <= 0 || split > p->N) return 0;
      return carve_softmax_ws(p, nullptr, split, split).total;
    default:
      return 0;
  }
}

int faws_reduce_ranks(const float* parts, int32_t n_ranks, int64_t count, float* out, void* stream) {
  if (parts == nullptr || out == nullptr || n_ranks <= 0 || count < 0) return FAWS_EINVAL;
  return launch_reduce_ranks(parts, n_ranks, count, out, static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? FAWS_OK
             : FAWS_ECUDA;
}

int faws_device_status(int32_t reset) { return tc_read_status(reset); }

int faws_selftest_wait_give_up(void* stream) {
  return launch_wait_give_up(static_cast<cudaStream_t>(stream)) == cudaSuccess ? FAWS_OK : FAWS_ECUDA;
}

int faws_last_backend(void) { return t_last_backend; }
int64_t faws_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* faws_strerror(int status) {
  switch (status) {
    case FAWS_OK: return "ok";
    case FAWS_EINVAL: return "invalid argument (shape, pointer, window or split)";
    case FAWS_EUNSUPPORTED: return "unsupported head dimension or dtype";
    case FAWS_EWORKSPACE: return "workspace missing, too small or not on a 256-byte boundary";
    case FAWS_ECUDA: return "CUDA call failed";
    case FAWS_EBACKEND: return "requested kernel family cannot run this problem";
    case FAWS_ETOOLARGE: return "problem needs more scratch than the built-in array of the _noalloc entry point";
    default: return "unknown status";
  }
}

int faws_version(void) { return FAWS_VERSION; }

}  // extern "C"
