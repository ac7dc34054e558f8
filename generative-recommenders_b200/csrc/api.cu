// extern "C" entry points: argument validation, dispatch, error strings.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "attn_plan.cuh"
#include "common.cuh"

namespace b200hstu {

thread_local char g_err[512] = "";
std::atomic<long long> g_launches{0};

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
int check_cuda(cudaError_t e, const char *what) {
  if (e == cudaSuccess) return 0;
  snprintf(g_err, sizeof(g_err), "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
  return (int)e;
}

// ---------------------------------------------------------------------------------------
// per-kernel event timing (off by default)
// ---------------------------------------------------------------------------------------
namespace {
constexpr int PROF_RING = 512;
struct ProfileState {
  bool on = false;
  cudaEvent_t start[PROF_KINDS][PROF_RING];
  cudaEvent_t stop[PROF_KINDS][PROF_RING];
  bool created[PROF_KINDS][PROF_RING] = {};
  int count[PROF_KINDS] = {};
};
ProfileState g_prof;
}  // namespace

ProfileScope::ProfileScope(int kind_, cudaStream_t st_) : kind(kind_), st(st_), stop(nullptr) {
  if (!g_prof.on || kind < 0 || kind >= PROF_KINDS) return;
  int slot = g_prof.count[kind] % PROF_RING;
  if (!g_prof.created[kind][slot]) {
    cudaEventCreate(&g_prof.start[kind][slot]);
    cudaEventCreate(&g_prof.stop[kind][slot]);
    g_prof.created[kind][slot] = true;
  }
  cudaEventRecord(g_prof.start[kind][slot], st);
  stop = g_prof.stop[kind][slot];
  ++g_prof.count[kind];
}
ProfileScope::~ProfileScope() {
  if (stop != nullptr) cudaEventRecord(stop, st);
}

// implemented in the kernel translation units
int attn_simt(const b200_hstu_attn_args &a, cudaStream_t st, bool bwd);
bool attn_tc_applicable(const b200_hstu_attn_args &a, bool bwd, const char **why);
int attn_tc_fwd(const b200_hstu_attn_args &a, cudaStream_t st);
int attn_tc_bwd(const b200_hstu_attn_args &a, cudaStream_t st);
int64_t attn_tc_workspace_bytes(const b200_hstu_attn_args &a, int which);
int attn_tc_fwd_fp8(const b200_hstu_attn_fp8_args &a, cudaStream_t st);
int quantize_e4m3_block(const void *x, int dtype, int64_t row_stride, int64_t head_stride, void *x8, float *scale,
                        const int32_t *seq_offsets, const int32_t *block_offsets, int B, int H, int d,
                        int64_t total_L, int max_seq_len, cudaStream_t st);
int layer_norm_fwd(const void *x, int64_t x_rs, const void *w, const void *b, void *y, int64_t y_rs, float *mean,
                   float *rstd, int64_t rows, int D, float eps, int dtype, cudaStream_t st);
int layer_norm_bwd(const void *dy, int64_t dy_rs, const void *x, int64_t x_rs, const void *w, const float *mean,
                   const float *rstd, void *dx, int64_t dx_rs, void *dw, void *db, void *partial,
                   int64_t partial_bytes, int64_t rows, int D, int dtype, cudaStream_t st);
int64_t stage_bwd_workspace_bytes(int cols);
int jagged_concat_split(const b200_hstu_jagged_args &j, bool split, cudaStream_t st);
int ts_pos_fwd(const b200_hstu_ts_pos_args &p, cudaStream_t st);
int ts_pos_bwd(const b200_hstu_ts_pos_args &p, cudaStream_t st);
int ln_linear_fwd(const b200_hstu_ln_linear_args &a, cudaStream_t st);
int64_t ln_linear_workspace_bytes(int D, int N);
bool ln_linear_supported(int D, int N, int silu_cols, int dtype, const char **why);
int silu_launch(const void *dy, int64_t dy_rs, const void *x, int64_t x_rs, void *out, int64_t out_rs, int64_t rows,
                int width, bool bwd, int dtype, cudaStream_t st);
int norm_mul(const b200_hstu_norm_mul_args &a, bool bwd, cudaStream_t st);
int64_t norm_mul_dropout_mask_bytes(const b200_hstu_norm_mul_args &a);

namespace {

int validate_attn(const b200_hstu_attn_args *a, bool bwd) {
  if (a == nullptr) return fail(B200_HSTU_EINVAL, "args is NULL");
  if (a->B < 0 || a->H <= 0 || a->dqk <= 0 || a->dv <= 0 || a->total_L < 0)
    return fail(B200_HSTU_EINVAL, "bad sizes B=%d H=%d dqk=%d dv=%d total_L=%lld", a->B, a->H, a->dqk, a->dv,
                (long long)a->total_L);
  if (a->max_seq_len <= 0) return fail(B200_HSTU_EINVAL, "max_seq_len must be larger than 0");
  if (a->total_L >= (1ll << 31)) return fail(B200_HSTU_EUNSUPPORTED, "total_L must fit in int32");
  if (a->max_attn_len < 0 || a->contextual_seq_len < 0 || a->min_full_attn_seq_len < 0)
    return fail(B200_HSTU_EINVAL, "negative max_attn_len / contextual_seq_len / min_full_attn_seq_len");
  if (a->dtype != B200_HSTU_F32 && a->dtype != B200_HSTU_BF16 && a->dtype != B200_HSTU_F16)
    return fail(B200_HSTU_EINVAL, "dtype %d is not f32 / bf16 / f16", a->dtype);
  if (a->B == 0 || a->total_L == 0) return 0;
  if (!a->q || !a->k || !a->v || !a->seq_offsets) return fail(B200_HSTU_EINVAL, "q / k / v / seq_offsets is NULL");
  if (!bwd && !a->out) return fail(B200_HSTU_EINVAL, "out is NULL");
  if (bwd && (!a->dout || !a->dq || !a->dk || !a->dv_)) return fail(B200_HSTU_EINVAL, "dout / dq / dk / dv is NULL");
  if (a->attn_scale && a->attn_scale_numel != 1 && a->attn_scale_numel != a->total_L)
    return fail(B200_HSTU_EINVAL, "attn_scale must have 1 or total_L elements");
  if (a->bias_by_distance && a->bias_numel <= 0) return fail(B200_HSTU_EINVAL, "bias_numel must be positive");
  if (a->delta_size < 0) return fail(B200_HSTU_EINVAL, "delta_size must not be negative");
  if (a->delta_size > 0) {
    if (bwd) return fail(B200_HSTU_EUNSUPPORTED, "delta attention has no backward (it is the cached inference path)");
    if (a->attn_scale && a->attn_scale_numel != 1)
      return fail(B200_HSTU_EINVAL, "delta attention takes a scalar attn_scale only");
    if (a->plan_mode != B200_HSTU_PLAN_OWN) return fail(B200_HSTU_EINVAL, "delta attention plans for itself");
  }
  if (a->dropout_ratio < 0.f || !(a->dropout_ratio < 1.f))
    return fail(B200_HSTU_EINVAL, "dropout_ratio must be at least 0 and below 1");
  if (a->dropout_ratio > 0.f && a->dropout_seed != nullptr && a->delta_size > 0)
    return fail(B200_HSTU_EUNSUPPORTED, "delta attention is the inference path: no dropout");
  if (a->plan_mode != B200_HSTU_PLAN_OWN && a->plan_mode != (bwd ? B200_HSTU_PLAN_REUSE : B200_HSTU_PLAN_FOR_BACKWARD))
    return fail(B200_HSTU_EINVAL, "plan_mode %d is not valid for this call", (int)a->plan_mode);
  return 0;
}

}  // namespace
}  // namespace b200hstu

using namespace b200hstu;

extern "C" {

int b200_hstu_attn_fwd(const b200_hstu_attn_args *a, b200_hstu_stream_t stream) {
  int st = validate_attn(a, false);
  if (st != 0) return st;
  if (a->B == 0 || a->total_L == 0) return 0;
  const char *why = "";
  bool tc = attn_tc_applicable(*a, false, &why);
  if (a->impl == B200_HSTU_IMPL_TCGEN05 && !tc)
    return fail(B200_HSTU_EUNSUPPORTED, "tcgen05 forward not applicable: %s", why);
  if (tc && a->impl != B200_HSTU_IMPL_SIMT) return attn_tc_fwd(*a, (cudaStream_t)stream);
  return attn_simt(*a, (cudaStream_t)stream, false);
}

int b200_hstu_attn_bwd(const b200_hstu_attn_args *a, b200_hstu_stream_t stream) {
  int st = validate_attn(a, true);
  if (st != 0) return st;
  if (a->B == 0 || a->total_L == 0) return 0;
  const char *why = "";
  bool tc = attn_tc_applicable(*a, true, &why);
  if (a->impl == B200_HSTU_IMPL_TCGEN05 && !tc)
    return fail(B200_HSTU_EUNSUPPORTED, "tcgen05 backward not applicable: %s", why);
  if (tc && a->impl != B200_HSTU_IMPL_SIMT) return attn_tc_bwd(*a, (cudaStream_t)stream);
  return attn_simt(*a, (cudaStream_t)stream, true);
}

int64_t b200_hstu_attn_workspace_bytes(const b200_hstu_attn_args *a, int backward) {
  if (a == nullptr) return 0;
  const char *why = "";
  if (a->impl == B200_HSTU_IMPL_SIMT || !attn_tc_applicable(*a, backward == 1, &why)) return 0;
  return attn_tc_workspace_bytes(*a, backward);
}

int b200_hstu_attn_fwd_fp8(const b200_hstu_attn_fp8_args *a, b200_hstu_stream_t stream) {
  if (a == nullptr) return fail(B200_HSTU_EINVAL, "args is NULL");
  b200_hstu_attn_args base = a->base;
  base.dtype = B200_HSTU_BF16;
  int st = validate_attn(&base, false);
  if (st != 0) return st;
  if (base.B == 0 || base.total_L == 0) return 0;
  if (!a->q_scale || !a->k_scale || !a->v_scale || !a->block_offsets)
    return fail(B200_HSTU_EINVAL, "fp8 scales / block_offsets is NULL");
  if (base.dropout_ratio > 0.f && base.dropout_seed != nullptr)
    return fail(B200_HSTU_EUNSUPPORTED, "the fp8 forward has no dropout");
  return attn_tc_fwd_fp8(*a, (cudaStream_t)stream);
}

int b200_hstu_quantize_e4m3_block(const void *x, int32_t dtype, int64_t row_stride, int64_t head_stride, void *x8,
                                  float *scale, const int32_t *seq_offsets, const int32_t *block_offsets, int32_t B,
                                  int32_t H, int32_t d, int64_t total_L, int32_t max_seq_len,
                                  b200_hstu_stream_t stream) {
  if (B < 0 || H <= 0 || d <= 0 || total_L < 0) return fail(B200_HSTU_EINVAL, "bad sizes");
  if (B == 0 || total_L == 0) return 0;
  if (!x || !x8 || !scale || !seq_offsets || !block_offsets) return fail(B200_HSTU_EINVAL, "NULL pointer");
  return quantize_e4m3_block(x, dtype, row_stride, head_stride, x8, scale, seq_offsets, block_offsets, B, H, d,
                             total_L, max_seq_len, (cudaStream_t)stream);
}

int b200_hstu_layer_norm_fwd(const void *x, int64_t x_row_stride, const void *weight, const void *bias, void *y,
                             int64_t y_row_stride, float *mean, float *rstd, int64_t rows, int32_t D, float eps,
                             int32_t dtype, b200_hstu_stream_t stream) {
  if (rows < 0 || D <= 0) return fail(B200_HSTU_EINVAL, "layer_norm: bad sizes rows=%lld D=%d", (long long)rows, D);
  if (rows == 0) return 0;
  if (!x || !weight || !bias || !y) return fail(B200_HSTU_EINVAL, "layer_norm: NULL pointer");
  return layer_norm_fwd(x, x_row_stride, weight, bias, y, y_row_stride, mean, rstd, rows, D, eps, dtype,
                        (cudaStream_t)stream);
}

int b200_hstu_layer_norm_bwd(const void *dy, int64_t dy_row_stride, const void *x, int64_t x_row_stride,
                             const void *weight, const float *mean, const float *rstd, void *dx,
                             int64_t dx_row_stride, void *dweight, void *dbias, void *partial, int64_t partial_bytes,
                             int64_t rows, int32_t D, int32_t dtype, b200_hstu_stream_t stream) {
  if (rows < 0 || D <= 0) return fail(B200_HSTU_EINVAL, "layer_norm: bad sizes rows=%lld D=%d", (long long)rows, D);
  if (!weight || !dweight || !dbias || !partial) return fail(B200_HSTU_EINVAL, "layer_norm backward: NULL pointer");
  if (rows > 0 && (!dy || !x || !mean || !rstd || !dx)) return fail(B200_HSTU_EINVAL, "layer_norm backward: NULL pointer");
  return layer_norm_bwd(dy, dy_row_stride, x, x_row_stride, weight, mean, rstd, dx, dx_row_stride, dweight, dbias,
                        partial, partial_bytes, rows, D, dtype, (cudaStream_t)stream);
}

int64_t b200_hstu_layer_norm_bwd_workspace_bytes(int32_t D) { return stage_bwd_workspace_bytes(D); }

int b200_hstu_ln_linear_silu_fwd(const b200_hstu_ln_linear_args *args, b200_hstu_stream_t stream) {
  if (!args) return fail(B200_HSTU_EINVAL, "ln_linear: NULL args");
  return ln_linear_fwd(*args, (cudaStream_t)stream);
}
int64_t b200_hstu_ln_linear_workspace_bytes(int32_t D, int32_t N) {
  if (D <= 0 || N <= 0) return 0;
  return ln_linear_workspace_bytes(D, N);
}
int b200_hstu_ln_linear_supported(int32_t D, int32_t N, int32_t silu_cols, int32_t dtype) {
  const char *why = "";
  return ln_linear_supported(D, N, silu_cols, dtype, &why) ? 1 : 0;
}

int b200_hstu_concat_2d_jagged(const b200_hstu_jagged_args *args, b200_hstu_stream_t stream) {
  if (!args) return fail(B200_HSTU_EINVAL, "concat_2D_jagged: NULL args");
  return jagged_concat_split(*args, false, (cudaStream_t)stream);
}
int b200_hstu_split_2d_jagged(const b200_hstu_jagged_args *args, b200_hstu_stream_t stream) {
  if (!args) return fail(B200_HSTU_EINVAL, "split_2D_jagged: NULL args");
  return jagged_concat_split(*args, true, (cudaStream_t)stream);
}
int b200_hstu_add_timestamp_positional_embeddings_fwd(const b200_hstu_ts_pos_args *args, b200_hstu_stream_t stream) {
  if (!args) return fail(B200_HSTU_EINVAL, "add_timestamp_positional_embeddings: NULL args");
  return ts_pos_fwd(*args, (cudaStream_t)stream);
}
int b200_hstu_add_timestamp_positional_embeddings_bwd(const b200_hstu_ts_pos_args *args, b200_hstu_stream_t stream) {
  if (!args) return fail(B200_HSTU_EINVAL, "add_timestamp_positional_embeddings: NULL args");
  return ts_pos_bwd(*args, (cudaStream_t)stream);
}

int b200_hstu_silu_fwd(const void *x, int64_t x_row_stride, void *y, int64_t y_row_stride, int64_t rows,
                       int32_t width, int32_t dtype, b200_hstu_stream_t stream) {
  if (rows < 0 || width <= 0) return fail(B200_HSTU_EINVAL, "silu: bad sizes");
  if (rows == 0) return 0;
  if (!x || !y) return fail(B200_HSTU_EINVAL, "silu: NULL pointer");
  return silu_launch(nullptr, 0, x, x_row_stride, y, y_row_stride, rows, width, false, dtype, (cudaStream_t)stream);
}

int b200_hstu_silu_bwd(const void *dy, int64_t dy_row_stride, const void *x, int64_t x_row_stride, void *dx,
                       int64_t dx_row_stride, int64_t rows, int32_t width, int32_t dtype, b200_hstu_stream_t stream) {
  if (rows < 0 || width <= 0) return fail(B200_HSTU_EINVAL, "silu: bad sizes");
  if (rows == 0) return 0;
  if (!dy || !x || !dx) return fail(B200_HSTU_EINVAL, "silu: NULL pointer");
  return silu_launch(dy, dy_row_stride, x, x_row_stride, dx, dx_row_stride, rows, width, true, dtype,
                     (cudaStream_t)stream);
}

static int validate_norm_mul(const b200_hstu_norm_mul_args *a, bool bwd) {
  if (a == nullptr) return fail(B200_HSTU_EINVAL, "args is NULL");
  if (a->rows < 0 || a->H <= 0 || a->V <= 0) return fail(B200_HSTU_EINVAL, "norm_mul: bad sizes");
  if (a->act < 0 || a->act > 2) return fail(B200_HSTU_EINVAL, "norm_mul: act must be 0 (none), 1 (sigmoid), 2 (silu)");
  if (a->group_norm && a->act != 0)
    return fail(B200_HSTU_EINVAL, "norm_mul: the group-norm variant has no activation on u");
  if (a->group_norm && (a->concat_u != a->concat_x))
    return fail(B200_HSTU_EINVAL, "norm_mul: the group-norm variant concatenates both u and attn or neither");
  if (!a->weight || !a->bias) return fail(B200_HSTU_EINVAL, "norm_mul: NULL weight / bias");
  if (a->rows > 0 && (!a->attn || !a->u)) return fail(B200_HSTU_EINVAL, "norm_mul: NULL attn / u");
  if (!bwd && a->rows > 0 && !a->out) return fail(B200_HSTU_EINVAL, "norm_mul: NULL out");
  if (bwd) {
    if (!a->dweight || !a->dbias || !a->partial) return fail(B200_HSTU_EINVAL, "norm_mul backward: NULL pointer");
    if (a->rows > 0 && (!a->dout || !a->dattn || !a->du || !a->mean || !a->rstd))
      return fail(B200_HSTU_EINVAL, "norm_mul backward: NULL pointer");
  }
  return 0;
}

int b200_hstu_norm_mul_fwd(const b200_hstu_norm_mul_args *a, b200_hstu_stream_t stream) {
  int st = validate_norm_mul(a, false);
  if (st != 0) return st;
  if (a->rows == 0) return 0;
  return norm_mul(*a, false, (cudaStream_t)stream);
}

int b200_hstu_norm_mul_bwd(const b200_hstu_norm_mul_args *a, b200_hstu_stream_t stream) {
  int st = validate_norm_mul(a, true);
  if (st != 0) return st;
  return norm_mul(*a, true, (cudaStream_t)stream);
}

int64_t b200_hstu_norm_mul_bwd_workspace_bytes(int32_t H, int32_t V, int32_t group_norm) {
  return stage_bwd_workspace_bytes(group_norm ? H : H * V);
}

int64_t b200_hstu_norm_mul_dropout_mask_bytes(const b200_hstu_norm_mul_args *a) {
  if (a == nullptr || a->rows <= 0) return 0;
  return norm_mul_dropout_mask_bytes(*a);
}

void b200_hstu_profile_enable(int on) {
  g_prof.on = on != 0;
  for (int k = 0; k < PROF_KINDS; ++k) g_prof.count[k] = 0;
}

int b200_hstu_profile_collect(int kind, float *out_ms, int max_n) {
  if (kind < 0 || kind >= PROF_KINDS || out_ms == nullptr) return 0;
  int n = g_prof.count[kind] < PROF_RING ? g_prof.count[kind] : PROF_RING;
  if (n > max_n) n = max_n;
  int got = 0;
  for (int i = 0; i < n; ++i) {
    float ms = 0.f;
    if (g_prof.created[kind][i] && cudaEventElapsedTime(&ms, g_prof.start[kind][i], g_prof.stop[kind][i]) == cudaSuccess)
      out_ms[got++] = ms;
  }
  return got;
}

const char *b200_hstu_last_error(void) { return g_err; }
int b200_hstu_version(void) { return 103; }
int64_t b200_hstu_launch_count(void) { return (int64_t)g_launches.load(); }

/* Host utility for tooling and tests: the kv range a query tile visits (the block-skipping
   rule the kernels use).  Returns lo, hi and diag_lo (-1 when the diagonal block is not
   separate) through the pointers. */
void b200_hstu_host_kv_range(int32_t len, int32_t num_targets, int32_t max_seq_len, int32_t contextual_seq_len,
                             int32_t max_attn_len, int32_t min_full_attn_seq_len, int32_t m0, int32_t tile,
                             int32_t *lo, int32_t *hi, int32_t *diag_lo) {
  SeqMask m = make_seq_mask(len, max_seq_len, num_targets, contextual_seq_len, max_attn_len, min_full_attn_seq_len);
  KvRange r = kv_range_for_q_tile(m, len, num_targets, m0, tile);
  *lo = r.lo;
  *hi = r.hi;
  *diag_lo = r.diag_lo;
}

/* Host utility: the query tiles (128 rows each) that the backward's K/V-stationary kernel visits
   for kv tile `kt`: tiles [t_lo, t_lo + n_main) plus `extra_tile` when it is >= 0. */
void b200_hstu_host_bwd_q_tiles(int32_t len, int32_t num_targets, int32_t max_seq_len, int32_t contextual_seq_len,
                                int32_t max_attn_len, int32_t min_full_attn_seq_len, int32_t kt, int32_t *t_lo,
                                int32_t *n_main, int32_t *extra_tile) {
  AttnGeomParams g;
  g.seq_offsets = nullptr;
  g.num_targets = nullptr;
  g.B = 1;
  g.H = 1;
  g.max_seq_len = max_seq_len;
  g.W = max_attn_len;
  g.c = contextual_seq_len;
  g.F = min_full_attn_seq_len;
  g.delta = 0;
  TileItem it;
  fill_kv_item(it, g, 0, kt, 0, len, num_targets);
  *t_lo = it.t_lo;
  *n_main = it.n_main;
  *extra_tile = it.extra_tile;
}

/* Host utility: mask(i, j) from the closed-form per-row (transposed = 0) or per-column
   (transposed = 1) intervals the tensor-core kernels use on partially visible tiles; -1 when the
   sequence is outside the domain where the closed form applies (the kernels then evaluate the
   exact mask element by element). */
int b200_hstu_host_interval_mask(int32_t len, int32_t num_targets, int32_t max_seq_len, int32_t contextual_seq_len,
                                 int32_t max_attn_len, int32_t min_full_attn_seq_len, int32_t i, int32_t j,
                                 int32_t transposed) {
  AttnGeomParams g;
  g.seq_offsets = nullptr;
  g.num_targets = nullptr;
  g.B = 1;
  g.H = 1;
  g.max_seq_len = max_seq_len;
  g.W = max_attn_len;
  g.c = contextual_seq_len;
  g.F = min_full_attn_seq_len;
  g.delta = 0;
  TileItem it;
  fill_common(it, g, 0, 0, 0, len, num_targets);
  if (!it.regular) return -1;
  if (i >= it.m.L || j >= it.m.L) return 0;
  if (!transposed) {
    RowInterval r = row_interval(it, i);
    int base = j & ~31;
    return (row_mask_bits(r, base, it.m.L) >> (j - base)) & 1u;
  }
  ColInterval r = col_interval(it, j);
  int base = i & ~31;
  return (col_mask_bits(r, base, it.m.L) >> (i - base)) & 1u;
}

/* Host utility: mask(i, j) of one sequence, as the kernels evaluate it. */
int b200_hstu_host_mask(int32_t len, int32_t num_targets, int32_t max_seq_len, int32_t contextual_seq_len,
                        int32_t max_attn_len, int32_t min_full_attn_seq_len, int32_t i, int32_t j) {
  SeqMask m = make_seq_mask(len, max_seq_len, num_targets, contextual_seq_len, max_attn_len, min_full_attn_seq_len);
  return (i < m.L && j < m.L && m.valid(i, j)) ? 1 : 0;
}

}  // extern "C"
