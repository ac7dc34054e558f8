/*
 * b200_hstu.h - C ABI of the B200 (sm_100a) HSTU jagged-attention library.
 *
 * Every entry point takes plain pointers and sizes, launches on the stream it is
 * given, never synchronises the device and never throws.  Return value: 0 on
 * success, a negative B200_HSTU_E* code for a rejected argument, or a positive
 * cudaError_t if the CUDA runtime reported one.  b200_hstu_last_error() returns a
 * human-readable message for the calling thread's last non-zero status.
 *
 * All data pointers are device pointers unless stated otherwise.  "Jagged" tensors
 * are [total_L, H, d] with unit stride on d, `head_stride` elements between heads
 * and `row_stride` elements between tokens; sequence b owns rows
 * seq_offsets[b] .. seq_offsets[b+1].
 *
 * The comments cite the interface of meta-recsys/generative-recommenders that each
 * entry point stands in for (paths relative to that project).
 */
#ifndef B200_HSTU_H_
#define B200_HSTU_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define B200_HSTU_OK 0
#define B200_HSTU_EINVAL (-1)      /* bad or inconsistent argument                  */
#define B200_HSTU_EUNSUPPORTED (-2) /* valid in the reference, not implemented here */
#define B200_HSTU_EWORKSPACE (-3)  /* workspace missing or too small                */
#define B200_HSTU_EDEVICE (-4)     /* not an sm_100 device / driver entry missing   */

/* element types */
#define B200_HSTU_F32 0
#define B200_HSTU_BF16 1
#define B200_HSTU_F16 2
#define B200_HSTU_E4M3 3

/* who builds the work lists the tensor-core kernels walk (b200_hstu_attn_args.plan_mode) */
#define B200_HSTU_PLAN_OWN 0          /* every call builds its own lists in its workspace                  */
#define B200_HSTU_PLAN_FOR_BACKWARD 1 /* forward: also build the backward's lists (one planning launch for  */
                                      /* the whole training step); workspace of ..._workspace_bytes(a, 2)  */
#define B200_HSTU_PLAN_REUSE 2        /* backward: workspace is that forward workspace; plan nothing.  The  */
                                      /* lists serve one backward call; same sizes / offsets / semantics   */

/* which kernel family runs the attention */
#define B200_HSTU_IMPL_AUTO 0    /* tcgen05 when dtype/head-dim allow, else SIMT */
#define B200_HSTU_IMPL_SIMT 1    /* fp32-accumulating CUDA-core kernels          */
#define B200_HSTU_IMPL_TCGEN05 2 /* tensor-core kernels; error if not applicable */

typedef void *b200_hstu_stream_t; /* a cudaStream_t */

/*
 * Arguments of the jagged HSTU attention, forward and backward.
 *
 *   out[i] = sum_j mask(i, j) * SiLU(alpha * <q_i, k_j>) * scale * v_j
 *
 * with scale = 1 / max_seq_len, or attn_scale[0] / attn_scale[token] when
 * attn_scale is given.  The mask is the reference's causal HSTU mask with targets,
 * contextual prefix and local window
 * (generative_recommenders/ops/pytorch/pt_hstu_attention.py:33-84).
 */
typedef struct b200_hstu_attn_args {
  /* tensors */
  const void *q;          /* [total_L, H, dqk] */
  const void *k;          /* [total_L, H, dqk] */
  const void *v;          /* [total_L, H, dv]  */
  void *out;              /* fwd: written.  [total_L, H, dv]; bwd: unused (may be NULL) */
  const void *dout;       /* bwd only: [total_L, H, dv] */
  void *dq, *dk, *dv_;    /* bwd only: written, same shapes as q, k, v */
  const int32_t *seq_offsets; /* [B + 1] */
  const int32_t *num_targets; /* [B] or NULL */
  const float *attn_scale;    /* NULL, or fp32 [1] (scalar) or [total_L] (per query token) */
  int64_t attn_scale_numel;   /* 0, 1 or total_L */
  /* strides, in elements */
  int64_t q_row_stride, k_row_stride, v_row_stride, o_row_stride;
  int64_t q_head_stride, k_head_stride, v_head_stride, o_head_stride;
  int64_t do_row_stride, dq_row_stride, dk_row_stride, dv_row_stride;
  int64_t do_head_stride, dq_head_stride, dk_head_stride, dv_head_stride;
  /* sizes */
  int64_t total_L;
  int32_t B, H, dqk, dv;
  int32_t max_seq_len; /* N: scale 1/N, and rows beyond N of a sequence produce zeros */
  /* semantics */
  float alpha;
  int32_t max_attn_len;          /* 0 = unlimited */
  int32_t contextual_seq_len;    /* 0 = none */
  int32_t min_full_attn_seq_len; /* 0 = none */
  int32_t dtype;                 /* B200_HSTU_F32 / BF16 / F16 (q, k, v, out, dout, dq, dk, dv) */
  int32_t impl;                  /* B200_HSTU_IMPL_* */
  /* optional relative position bias added to alpha*<q,k> before SiLU, shared by all heads:
     bias_by_distance[|i - j|] when |i - j| < bias_numel, else 0 (fp32); NULL = none */
  const float *bias_by_distance;
  int32_t bias_numel;
  int32_t plan_mode;             /* B200_HSTU_PLAN_*; ignored by the CUDA-core kernels */
  /* scratch: see b200_hstu_attn_workspace_bytes(); contents need no initialisation */
  void *workspace;
  int64_t workspace_bytes;
  /* > 0 (forward only): q and out hold delta_size rows per sequence, [B * delta_size, H, d] - the
     last delta_size positions of each sequence attend to its full K/V (total_L counts K/V rows).
     Stands in for delta_hstu_mha (generative_recommenders/ops/hstu_attention.py:210-275,
     pt_hstu_attention.py:191-251).  Every sequence must be at least delta_size and at most
     max_seq_len long; attn_scale must be NULL or a scalar. */
  int32_t delta_size;
  /* > 0 (with dropout_seed): dropout on the attention weights - after scale and mask, before the
     product with V - as the reference's PyTorch path applies it
     (generative_recommenders/ops/pytorch/pt_hstu_attention.py:180-181); must be below 1.  The weight
     of query row r (a row of q), head h and key position j inside the sequence is element
     idx = (r * H + h) * max_seq_len + j of the mask: dropped when the (idx % 8)-th 16-bit piece of
     Philox4x32-10(key = *dropout_seed, counter = idx / 8) is below round(dropout_ratio * 65536), scaled by
     the inverse keep probability otherwise.  A backward call with the same ratio and seed regenerates
     the mask.  CUDA-core kernels only: impl = AUTO takes them, impl = TCGEN05 is refused; not with
     delta_size. */
  float dropout_ratio;
  /* bwd only, optional: gradient of bias_by_distance, fp32 [bias_numel].  The backward ADDS into this
     caller-zeroed buffer (fp32 atomics: the sum over pairs, heads and sequences of dL/dscore at each
     |i - j|; the order of the additions, and with it the last bits, varies from run to run).  NULL =
     not wanted.  The research model trains these tables
     (generative_recommenders/research/modeling/sequential/hstu.py:65-143, 203-211). */
  float *d_bias_by_distance;
  const uint64_t *dropout_seed;    /* device, one value; NULL = no dropout */
} b200_hstu_attn_args;

/*
 * Forward.  Stands in for hstu_mha / torch.ops.hstu.hstu_mha_fwd
 * (generative_recommenders/ops/hstu_attention.py:101-207,
 *  generative_recommenders/ops/cpp/hstu_attention/flash_api_cpu.cpp:142-235).
 */
int b200_hstu_attn_fwd(const b200_hstu_attn_args *args, b200_hstu_stream_t stream);

/*
 * Backward: fills dq, dk, dv from dout.  Stands in for
 * _AttentionFunction.backward / torch.ops.hstu.hstu_mha_bwd
 * (generative_recommenders/ops/triton/triton_hstu_attention.py:3031-3092,
 *  generative_recommenders/ops/cpp/hstu_attention/flash_common.cpp:851-1212).
 */
int b200_hstu_attn_bwd(const b200_hstu_attn_args *args, b200_hstu_stream_t stream);

/*
 * Forward for callers that cannot allocate device memory (a server that owns all of HBM through
 * its own arena, code running where the allocator must not be touched, a bare C caller with no
 * allocator at hand).  Same arguments and result as b200_hstu_attn_fwd(), but args->workspace is
 * ignored: the work list lives in a 1 MiB array inside the library's device image (held by every
 * context that loads the library until exit).  Batches needing more (total_L / 128 + B + 1 >
 * 32 767 items of 32 bytes; a bias_by_distance table takes 8 * (roundup128(max_seq_len) + 256)
 * bytes of the same array) are rejected with B200_HSTU_EWORKSPACE.  The first call on a device
 * looks the array up with cudaGetSymbolAddress - make it outside any stream capture; no call
 * allocates.
 * One array per device is shared by all calls: back-to-back calls on one stream are fine, calls
 * that may overlap on the GPU race.  This entry point has no counterpart in the reference (its
 * ops allocate their scratch per call through torch).
 */
int b200_hstu_attn_fwd_static_scratch(const b200_hstu_attn_args *args, b200_hstu_stream_t stream);
int64_t b200_hstu_attn_fwd_static_scratch_max_bytes(void);

/* Bytes of scratch that fwd (backward = 0), bwd (backward = 1) or a forward that also plans the
   backward (backward = 2, plan_mode FOR_BACKWARD / REUSE) need for these sizes.
   Host function; depends on B, H, dqk, dv, total_L, dtype, impl, and - through the table of a
   relative bias - on whether bias_by_distance is set and on max_seq_len. */
int64_t b200_hstu_attn_workspace_bytes(const b200_hstu_attn_args *args, int backward);

/*
 * Status of the tensor-core launches.  Every wait inside those kernels is bounded (2 s without
 * progress); a wait that gives up records its site id (> 0) in the status word of the launch's
 * work list and the kernel returns early, leaving its output incomplete.  This call queues, on
 * `stream`, copies of the status words of the launches that used args->workspace into
 * host_status[3] - [0] forward, [1] backward dK/dV launch, [2] backward dQ launch; entries that
 * the call does not cover are set to 0 - which the caller reads after synchronising the stream
 * (pinned host memory keeps the copies asynchronous).  `which`: 0 = a forward's workspace, 1 = a
 * backward's, 2 = the workspace of a forward that planned the backward (all three).  Same args as
 * the launch.  The CUDA-core kernels have no waits: all zeros.  No counterpart in the reference
 * (its kernels spin without a limit, generative_recommenders/ops/triton/triton_attention_utils.py:42-48).
 */
int b200_hstu_attn_status_async(const b200_hstu_attn_args *args, int which, int32_t *host_status,
                                b200_hstu_stream_t stream);

/*
 * Self-test of the bounded wait: a one-warp kernel waits, with the limit shortened to 1 ms, on a
 * barrier nobody arrives at; the wait expires, records site 777 in *status_dev (device int32,
 * cleared first) and the time it waited in *elapsed_ns_dev (device uint64), and the kernel returns.
 */
int b200_hstu_selftest_bounded_wait(int32_t *status_dev, uint64_t *elapsed_ns_dev, b200_hstu_stream_t stream);

/*
 * FP8 (e4m3) forward for inference with per-block scales: q8/k8/v8 are
 * [total_L, H, d] e4m3 (contiguous heads), *_scale are fp32 [n_blocks_total, H] where
 * sequence b owns rows block_offsets[b] .. block_offsets[b+1], one row per 128 tokens
 * counted from the sequence's first token.  Output is bf16.  The reference plumbs
 * per-(batch, head) descale tensors through torch.ops.hstu.hstu_mha_fwd
 * (generative_recommenders/ops/cpp/hstu_attention/flash_common.cpp:680-711) but
 * compiles FP8 out; per-block scales are an extension.
 */
typedef struct b200_hstu_attn_fp8_args {
  b200_hstu_attn_args base; /* q, k, v hold e4m3 data; out is bf16; dtype ignored */
  const float *q_scale, *k_scale, *v_scale;
  const int32_t *block_offsets; /* [B + 1] */
} b200_hstu_attn_fp8_args;
int b200_hstu_attn_fwd_fp8(const b200_hstu_attn_fp8_args *args, b200_hstu_stream_t stream);

/* Block quantiser producing the layout above: x [total_L, H, d] (bf16 / f16 / f32) ->
   x8 e4m3 + scale = absmax / 448 per (128-token block, head). */
int b200_hstu_quantize_e4m3_block(const void *x, int32_t dtype, int64_t row_stride, int64_t head_stride,
                                  void *x8, float *scale, const int32_t *seq_offsets,
                                  const int32_t *block_offsets, int32_t B, int32_t H, int32_t d,
                                  int64_t total_L, int32_t max_seq_len, b200_hstu_stream_t stream);

/*
 * Row LayerNorm with affine, fp32 statistics (generative_recommenders/ops/layer_norm.py:50-94,
 * generative_recommenders/ops/pytorch/pt_layer_norm.py:24-38).  x, y: [rows, D] with the given
 * row strides; mean, rstd: fp32 [rows] (written by fwd when non-NULL, read by bwd).
 */
int b200_hstu_layer_norm_fwd(const void *x, int64_t x_row_stride, const void *weight, const void *bias,
                             void *y, int64_t y_row_stride, float *mean, float *rstd, int64_t rows,
                             int32_t D, float eps, int32_t dtype, b200_hstu_stream_t stream);
/* dx [rows, D]; dweight, dbias [D] in `dtype`.  partial: fp32 scratch of
   b200_hstu_layer_norm_bwd_workspace_bytes(D) bytes. */
int b200_hstu_layer_norm_bwd(const void *dy, int64_t dy_row_stride, const void *x, int64_t x_row_stride,
                             const void *weight, const float *mean, const float *rstd, void *dx,
                             int64_t dx_row_stride, void *dweight, void *dbias, void *partial,
                             int64_t partial_bytes, int64_t rows, int32_t D, int32_t dtype,
                             b200_hstu_stream_t stream);
int64_t b200_hstu_layer_norm_bwd_workspace_bytes(int32_t D);

/*
 * u = SiLU(uvqk[:, :width]) - the gating half of hstu_compute_uqvk
 * (generative_recommenders/ops/hstu_compute.py:90-100).  q, k, v stay views of uvqk.
 */
int b200_hstu_silu_fwd(const void *x, int64_t x_row_stride, void *y, int64_t y_row_stride, int64_t rows,
                       int32_t width, int32_t dtype, b200_hstu_stream_t stream);
/* dx = dy * SiLU'(x) */
int b200_hstu_silu_bwd(const void *dy, int64_t dy_row_stride, const void *x, int64_t x_row_stride, void *dx,
                       int64_t dx_row_stride, int64_t rows, int32_t width, int32_t dtype,
                       b200_hstu_stream_t stream);

/*
 * y = act(u) * Norm(attn) with the optional [u, attn, y] concatenation that feeds the output
 * linear (generative_recommenders/ops/pytorch/pt_hstu_linear.py:23-82).  attn, u: [rows, H*V];
 * out: [rows, (1 + concat_u + concat_x) * H*V].  act: 0 none, 1 sigmoid, 2 silu.  group_norm: 0 =
 * LayerNorm over H*V (weight/bias [H*V]), 1 = per-head normalisation (weight/bias [H]).
 * Dropout (training; pt_hstu_linear.py:77-81 applies F.dropout to the concatenated row, the
 * reference's GPU path generates the mask inside its kernel, ops/triton/triton_hstu_linear.py:
 * 365-492): with dropout_seed != NULL and 0 < dropout_ratio < 1 every element of the output row is
 * zeroed with probability round(dropout_ratio * 65536) / 65536 and the others are scaled by the
 * inverse keep probability.  Element idx = row * width + column uses the (idx % 8)-th 16-bit piece
 * of Philox4x32-10(key = *dropout_seed, counter = idx / 8, 0, 0); the backward, given the same
 * seed, regenerates the mask (nothing is stored).  Not built for group_norm = 1.
 */
typedef struct b200_hstu_norm_mul_args {
  const void *attn, *u, *weight, *bias;
  void *out;
  float *mean, *rstd;     /* fp32 [rows * groups]; written by fwd if non-NULL, read by bwd */
  const void *dout;       /* bwd */
  void *dattn, *du, *dweight, *dbias; /* bwd */
  void *partial;          /* bwd scratch, b200_hstu_norm_mul_bwd_workspace_bytes() */
  int64_t partial_bytes;
  int64_t attn_row_stride, u_row_stride, out_row_stride, dout_row_stride, dattn_row_stride, du_row_stride;
  int64_t rows;
  int32_t H, V;
  int32_t concat_u, concat_x, act, group_norm;
  float eps;
  int32_t dtype;
  float dropout_ratio;               /* 0 = no dropout */
  int32_t reserved0;
  const int64_t *dropout_seed;       /* device, one int64 (read by the kernels); NULL = no dropout */
  /* optional, with dropout: the mask as bits, b200_hstu_norm_mul_dropout_mask_bytes() bytes (element
     idx = row * width + col is bit idx % 8 of byte idx / 8; set = kept).  The forward writes it next
     to the output; a backward that is given it reads it instead of running the generator again
     (ten dependent rounds per 8 elements: the regenerating backward takes twice as long).  NULL =
     nothing stored, the backward regenerates the mask from the seed. */
  uint8_t *dropout_mask;
} b200_hstu_norm_mul_args;
int b200_hstu_norm_mul_fwd(const b200_hstu_norm_mul_args *args, b200_hstu_stream_t stream);
int b200_hstu_norm_mul_bwd(const b200_hstu_norm_mul_args *args, b200_hstu_stream_t stream);
int64_t b200_hstu_norm_mul_bwd_workspace_bytes(int32_t H, int32_t V, int32_t group_norm);
/* Bytes of args->dropout_mask for the forward arguments given, or 0 where a stored mask cannot be used
   (group norm, 32-bit elements, rows not made of whole 16-byte aligned vectors, no dropout). */
int64_t b200_hstu_norm_mul_dropout_mask_bytes(const b200_hstu_norm_mul_args *args);

/*
 * The uvqk stage as one tensor-core kernel (generative_recommenders/ops/hstu_compute.py:54-104:
 * layer_norm -> addmm -> split -> silu):
 *   out = LayerNorm(x; norm_weight, norm_bias, eps) * weight + bias      [M, N]
 *   u   = SiLU(out[:, :silu_cols])                                       [M, silu_cols]  (if u != NULL)
 * x [M, D], weight [D, N] row-major and contiguous, bias [N] (may be NULL), all of `dtype` (bf16 or
 * f16).  mean / rstd (fp32 [M], may be NULL) receive the row statistics for the backward.
 * Supported: D a multiple of 64 up to 512, N a multiple of 64, silu_cols a multiple of 32,
 * 16-byte aligned tensors and row strides (b200_hstu_ln_linear_supported() tells; other shapes
 * return B200_HSTU_EUNSUPPORTED and the caller runs the three separate stages).  Row strides in
 * elements.  workspace: b200_hstu_ln_linear_workspace_bytes(D, N) bytes, contents need no
 * initialisation.
 */
typedef struct b200_hstu_ln_linear_args {
  const void *x, *norm_weight, *norm_bias, *weight, *bias;
  void *out, *u;
  float *mean, *rstd;
  void *workspace;
  int64_t workspace_bytes;
  int64_t x_row_stride, out_row_stride, u_row_stride;
  int64_t M;
  int32_t D, N, silu_cols;
  float eps;
  int32_t dtype;
  int32_t weights_prepared; /* 1: workspace still holds what an earlier call derived from the same
                               norm_weight / norm_bias / weight / bias values; skips that step */
  int32_t skip_pre_activation; /* 1 (needs u): out[:, :silu_cols] is left unwritten - only the backward
                                  reads those columns */
  int32_t reserved0;
} b200_hstu_ln_linear_args;
int b200_hstu_ln_linear_silu_fwd(const b200_hstu_ln_linear_args *args, b200_hstu_stream_t stream);
int64_t b200_hstu_ln_linear_workspace_bytes(int32_t D, int32_t N);
int b200_hstu_ln_linear_supported(int32_t D, int32_t N, int32_t silu_cols, int32_t dtype);

/*
 * concat_2D_jagged / split_2D_jagged (generative_recommenders/ops/jagged_tensors.py:55-162;
 * semantics of ops/pytorch/pt_jagged_tensors.py:32-160): sequence b of `combined` holds the rows
 * of `left` for b followed by the rows of `right` for b.  Rows are `row_bytes` bytes and
 * contiguous in all three tensors.  A side without offsets (NULL) is dense: every sequence has
 * dense_len_* rows there.  total_rows = rows of `combined`.  concat reads left/right and writes
 * combined; split reads combined and writes left/right.  Offsets are int64 device arrays [B + 1].
 * Each is the other's backward.  right_rows_first = c > 0 gives the layout of
 * hstu_split_l2_embeddings / hstu_concat_l2_embeddings (ops/jagged_tensors.py:165-227): the first c
 * rows of every sequence of `combined` are the first c rows of `right` for that sequence, then come
 * the rows of `left`, then the rest of `right` (every sequence needs at least c rows in `right`).
 */
typedef struct b200_hstu_jagged_args {
  void *left, *right, *combined;
  const int64_t *offsets_left, *offsets_right;
  int64_t dense_len_left, dense_len_right;
  int64_t total_rows;
  int64_t row_bytes;
  int32_t B;
  int32_t right_rows_first;
} b200_hstu_jagged_args;
int b200_hstu_concat_2d_jagged(const b200_hstu_jagged_args *args, b200_hstu_stream_t stream);
int b200_hstu_split_2d_jagged(const b200_hstu_jagged_args *args, b200_hstu_stream_t stream);

/*
 * add_timestamp_positional_embeddings (generative_recommenders/ops/position.py:40-118; semantics
 * of ops/pytorch/pt_position.py:40-160):
 *   out[t] = alpha * seq_embeddings[t] + (ts_weight[bucket(t)] + pos_weight[index(t)])
 * with index(t) counted back from the end of the history (targets share one index; the first
 * max_contextual_seq_len rows use their own position) and bucket(t) = sqrt or log of the time to
 * the sequence's last item in minutes, clamped to [0, ts_bucket_max] (the reference clamps to
 * ts_weight.size(1) - 1) and to the table.  Index tensors are int64 device arrays; tables are
 * [max_pos_ind, D] / [ts_rows, D], float32 or of the sequence dtype.  The backward writes
 * d_seq_embeddings = alpha * d_out and ADDS the table gradients into the caller-zeroed fp32
 * buffers d_pos_weight / d_ts_weight.  time_bucket_fn: 0 sqrt, 1 log.
 */
typedef struct b200_hstu_ts_pos_args {
  const void *seq_embeddings, *pos_weight, *ts_weight;
  void *out;
  const void *d_out;       /* bwd */
  void *d_seq_embeddings;  /* bwd */
  float *d_pos_weight, *d_ts_weight; /* bwd, fp32, accumulated into */
  const int64_t *seq_offsets, *seq_lengths, *num_targets, *timestamps;
  int64_t total_rows;
  int32_t B, D;
  int32_t max_contextual_seq_len, max_pos_ind, ts_rows, ts_bucket_max;
  int32_t interleave_targets, time_bucket_fn;
  float alpha;
  int32_t dtype, table_dtype;
  int32_t reserved0;
} b200_hstu_ts_pos_args;
int b200_hstu_add_timestamp_positional_embeddings_fwd(const b200_hstu_ts_pos_args *args, b200_hstu_stream_t stream);
int b200_hstu_add_timestamp_positional_embeddings_bwd(const b200_hstu_ts_pos_args *args, b200_hstu_stream_t stream);

/*
 * Optional per-kernel timing for benchmarks.  After b200_hstu_profile_enable(1) every launch of a
 * hot kernel is bracketed by a cudaEvent pair on its launch stream; once the caller has
 * synchronised the device, b200_hstu_profile_collect(kind, out_ms, max_n) writes up to max_n
 * durations (milliseconds, oldest first, at most the 512 most recent launches since the last
 * enable) and returns how many.  Kinds: 0 work-list planning, 1 attention forward, 2 backward
 * dK/dV, 3 backward dQ, 4 fp8 forward, 5 layer_norm forward, 6 layer_norm backward, 7 SiLU
 * gating, 8 norm_mul forward, 9 norm_mul backward, 10 e4m3 quantiser, 11 CUDA-core attention,
 * 12 jagged concat / split, 13 timestamp + position embeddings, 14 preparation of the fused uvqk
 * stage, 15 fused uvqk stage.
 * Enabling resets the counters; b200_hstu_profile_enable(0) turns the events off again.
 */
void b200_hstu_profile_enable(int on);
int b200_hstu_profile_collect(int kind, float *out_ms, int max_n);

/* Host helpers. */
const char *b200_hstu_last_error(void);
int b200_hstu_version(void);
/* Number of kernels this library has launched in the calling process since load. */
int64_t b200_hstu_launch_count(void);

/* Host utilities for tooling and tests (no device work).  b200_hstu_host_mask() evaluates the
   mask(i, j) of one sequence exactly as the kernels do; b200_hstu_host_kv_range() returns the kv
   positions [lo, hi) (+ a separate diagonal block at diag_lo, or -1) that the block-skipping rule
   makes the query tile starting at row m0 visit. */
void b200_hstu_host_kv_range(int32_t len, int32_t num_targets, int32_t max_seq_len, int32_t contextual_seq_len,
                             int32_t max_attn_len, int32_t min_full_attn_seq_len, int32_t m0, int32_t tile,
                             int32_t *lo, int32_t *hi, int32_t *diag_lo);
/* Query tiles (128 rows each) the backward's K/V-stationary kernel visits for kv tile kt:
   [t_lo, t_lo + n_main) plus extra_tile when it is >= 0. */
void b200_hstu_host_bwd_q_tiles(int32_t len, int32_t num_targets, int32_t max_seq_len, int32_t contextual_seq_len,
                                int32_t max_attn_len, int32_t min_full_attn_seq_len, int32_t kt, int32_t *t_lo,
                                int32_t *n_main, int32_t *extra_tile);
/* mask(i, j) from the closed-form row (transposed = 0) / column (transposed = 1) intervals used on
   partially visible tiles; -1 when the closed form does not apply to this sequence. */
int b200_hstu_host_interval_mask(int32_t len, int32_t num_targets, int32_t max_seq_len, int32_t contextual_seq_len,
                                 int32_t max_attn_len, int32_t min_full_attn_seq_len, int32_t i, int32_t j,
                                 int32_t transposed);
int b200_hstu_host_mask(int32_t len, int32_t num_targets, int32_t max_seq_len, int32_t contextual_seq_len,
                        int32_t max_attn_len, int32_t min_full_attn_seq_len, int32_t i, int32_t j);

#ifdef __cplusplus
}
#endif
#endif /* B200_HSTU_H_ */
