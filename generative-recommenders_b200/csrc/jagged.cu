// Jagged glue around the HSTU layer, all HBM-bound row movers:
//
//  * concat_2D_jagged / split_2D_jagged
//    (generative_recommenders/ops/jagged_tensors.py:55-162; PyTorch restatement
//    ops/pytorch/pt_jagged_tensors.py:32-160): sequence b of the combined tensor is the rows of
//    `left` for b followed by the rows of `right` for b.  One kernel does both directions: a CTA
//    takes 64 combined rows, one thread per row finds the row's sequence (binary search over
//    offsets_left + offsets_right) and its partner row, then all threads move the rows in 16-byte
//    pieces.  Either side may be dense (no offsets: every sequence has `dense_len` rows).  With
//    right_rows_first = c the first c rows of every sequence belong to `right`
//    (hstu_split_l2_embeddings / hstu_concat_l2_embeddings, ops/jagged_tensors.py:165-227).
//
//  * add_timestamp_positional_embeddings (ops/position.py:40-118;
//    ops/pytorch/pt_position.py:40-160): out = alpha * x + (ts_emb[bucket] + pos_emb[index]),
//    one warp per token; the backward accumulates the two table gradients with vector
//    reductions in fp32 and writes alpha * dy.
#include "common.cuh"

namespace b200hstu {

namespace {

constexpr int JAG_ROWS = 64;      // combined rows per CTA
constexpr int JAG_THREADS = 256;

struct JaggedArgs {
  const int64_t *off_l;  // [B + 1] or nullptr (dense: dense_l rows per sequence)
  const int64_t *off_r;
  int64_t dense_l, dense_r;
  int shift;             // rows of `right` that come BEFORE the rows of `left` in every sequence
  int B;
  int64_t total;  // combined rows
  char *left, *right, *comb;
  int64_t row_bytes;
};

__device__ __forceinline__ int64_t side_off(const int64_t *off, int64_t dense, int b) {
  return off ? off[b] : dense * b;
}

template <typename V, bool SPLIT>
__global__ void __launch_bounds__(JAG_THREADS) jagged_rows_kernel(JaggedArgs a) {
  __shared__ int64_t partner[JAG_ROWS];  // row index in left, or ~row index in right
  const int64_t g0 = (int64_t)blockIdx.x * JAG_ROWS;
  const int rows = (int)((a.total - g0) < JAG_ROWS ? (a.total - g0) : JAG_ROWS);
  if ((int)threadIdx.x < rows) {
    const int64_t g = g0 + threadIdx.x;
    int lo = 0, hi = a.B;  // largest b with combined offset(b) <= g
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if (side_off(a.off_l, a.dense_l, mid) + side_off(a.off_r, a.dense_r, mid) <= g) lo = mid; else hi = mid;
    }
    const int64_t ol = side_off(a.off_l, a.dense_l, lo), orr = side_off(a.off_r, a.dense_r, lo);
    const int64_t len_l = side_off(a.off_l, a.dense_l, lo + 1) - ol;
    const int64_t len_r = side_off(a.off_r, a.dense_r, lo + 1) - orr;
    const int64_t pos = g - ol - orr;
    // sequence layout: right[0, shift) | left | right[shift, ...)
    int64_t pr = pos < a.shift ? ~(orr + pos)
                               : (pos < a.shift + len_l ? ol + (pos - a.shift) : ~(orr + pos - len_l));
    // a row the offsets do not account for (inconsistent arguments) is skipped, never dereferenced
    if (pos < 0 || pos >= len_l + len_r) pr = INT64_MIN;
    partner[threadIdx.x] = pr;
  }
  __syncthreads();
  const int per_row = (int)(a.row_bytes / (int64_t)sizeof(V));
  const int n = rows * per_row;
  const V *__restrict__ comb_in = (const V *)(a.comb + g0 * a.row_bytes);
  V *__restrict__ comb_out = (V *)(a.comb + g0 * a.row_bytes);
  constexpr int UNROLL = 4;
  for (int base = threadIdx.x; base < n; base += JAG_THREADS * UNROLL) {
    V val[UNROLL];
    V *dst[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int i = base + u * JAG_THREADS;
      dst[u] = nullptr;
      if (i < n) {
        const int r = i / per_row, c = i - r * per_row;
        const int64_t p = partner[r];
        if (p == INT64_MIN) continue;
        char *side = p >= 0 ? a.left + p * a.row_bytes : a.right + (~p) * a.row_bytes;
        if (SPLIT) {
          val[u] = comb_in[i];
          dst[u] = (V *)side + c;
        } else {
          val[u] = ((const V *)side)[c];
          dst[u] = comb_out + i;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (dst[u]) *dst[u] = val[u];
  }
}

template <typename V>
int launch_jagged(const JaggedArgs &a, bool split, cudaStream_t st) {
  const unsigned grid = (unsigned)((a.total + JAG_ROWS - 1) / JAG_ROWS);
  if (split)
    jagged_rows_kernel<V, true><<<grid, JAG_THREADS, 0, st>>>(a);
  else
    jagged_rows_kernel<V, false><<<grid, JAG_THREADS, 0, st>>>(a);
  count_launch();
  B200_CHECK_LAUNCH("jagged_rows_kernel");
  return 0;
}

// ---------------------------------------------------------------------------------------
// timestamp + position embeddings
// ---------------------------------------------------------------------------------------
struct TsPosArgs {
  const int64_t *seq_offsets;  // [B + 1]
  const int64_t *seq_lengths;  // [B]
  const int64_t *num_targets;  // [B] or nullptr
  const int64_t *timestamps;   // [total]
  int B;
  int64_t total;
  int D;
  int max_contextual_seq_len;
  int max_pos_ind;     // rows of the position table
  int ts_rows;         // rows of the timestamp table
  int ts_bucket_max;   // largest bucket the reference's clamp allows
  int interleave_targets;
  int log_buckets;     // 0: sqrt, 1: log
  float alpha;
};

// position-table row and timestamp bucket of combined row g (pt_position.py:40-73, 96-125)
__device__ __forceinline__ void ts_pos_indices(const TsPosArgs &a, int64_t g, int &pos_ind, int &bucket) {
  int lo = 0, hi = a.B;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (a.seq_offsets[mid] <= g) lo = mid; else hi = mid;
  }
  const int64_t start = a.seq_offsets[lo];
  const int64_t p = g - start;
  const int64_t n = a.seq_lengths[lo];
  int64_t idx;
  if (a.num_targets) {
    const int64_t high = n - a.num_targets[lo] * (a.interleave_targets ? 2 : 1);
    idx = high - (p < high ? p : high);
  } else {
    idx = n - p;
  }
  idx += a.max_contextual_seq_len;
  if (idx > a.max_pos_ind - 1) idx = a.max_pos_ind - 1;
  if (p < a.max_contextual_seq_len) idx = p < a.max_pos_ind ? p : a.max_pos_ind - 1;
  if (idx < 0) idx = 0;  // only with seq_lengths smaller than the rows the offsets give: stay inside the table
  pos_ind = (int)idx;
  const int64_t rows_b = a.seq_offsets[lo + 1] - start;
  int64_t last = n - 1 > 0 ? n - 1 : 0;
  if (last > rows_b - 1) last = rows_b - 1;  // same: stay inside the sequence
  const int64_t dt = a.timestamps[start + last] - a.timestamps[g];
  float f = fmaxf((float)dt, 1e-6f);
  f = __fdiv_rn(f, 60.0f);
  f = a.log_buckets ? logf(f) : __fsqrt_rn(f);
  f = fmaxf(f, 0.f);
  int bk = (int)f;
  bk = bk < a.ts_bucket_max ? bk : a.ts_bucket_max;
  bucket = bk < a.ts_rows - 1 ? bk : a.ts_rows - 1;  // never past the table
}

constexpr int TSPOS_THREADS = 256;

// out = E(E(alpha x) + E(ts + pos)): the roundings of the reference's three tensor ops
template <typename E, typename TE>
__global__ void __launch_bounds__(TSPOS_THREADS)
ts_pos_fwd_kernel(TsPosArgs a, const E *__restrict__ x, const TE *__restrict__ pos_w, const TE *__restrict__ ts_w,
                  E *__restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (TSPOS_THREADS / 32) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (TSPOS_THREADS / 32);
  for (int64_t g = warp; g < a.total; g += nwarps) {
    int pi, bk;
    ts_pos_indices(a, g, pi, bk);
    const E *xr = x + g * a.D;
    const TE *pr = pos_w + (int64_t)pi * a.D;
    const TE *tr = ts_w + (int64_t)bk * a.D;
    E *orow = out + g * a.D;
    for (int c = lane; c < a.D; c += 32) {
      // explicit roundings: no contraction of the product into the sum
      const float scaled = to_f32(from_f32<E>(__fmul_rn(to_f32(xr[c]), a.alpha)));
      const TE emb = from_f32<TE>(__fadd_rn(to_f32(tr[c]), to_f32(pr[c])));
      const float add = to_f32(from_f32<E>(to_f32(emb)));
      orow[c] = from_f32<E>(__fadd_rn(scaled, add));
    }
  }
}

// dx = alpha dy; d_pos[index] += dy; d_ts[bucket] += dy (fp32 accumulators)
template <typename E>
__global__ void __launch_bounds__(TSPOS_THREADS)
ts_pos_bwd_kernel(TsPosArgs a, const E *__restrict__ dy, E *__restrict__ dx, float *__restrict__ d_pos,
                  float *__restrict__ d_ts) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (TSPOS_THREADS / 32) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (TSPOS_THREADS / 32);
  const bool vec4 = (a.D & 3) == 0;
  for (int64_t g = warp; g < a.total; g += nwarps) {
    int pi, bk;
    ts_pos_indices(a, g, pi, bk);
    const E *dr = dy + g * a.D;
    E *xr = dx + g * a.D;
    float *pr = d_pos + (int64_t)pi * a.D;
    float *tr = d_ts + (int64_t)bk * a.D;
    if (vec4) {
      for (int c = lane * 4; c < a.D; c += 128) {
        float4 v;
        v.x = to_f32(dr[c]); v.y = to_f32(dr[c + 1]); v.z = to_f32(dr[c + 2]); v.w = to_f32(dr[c + 3]);
        xr[c] = from_f32<E>(v.x * a.alpha);
        xr[c + 1] = from_f32<E>(v.y * a.alpha);
        xr[c + 2] = from_f32<E>(v.z * a.alpha);
        xr[c + 3] = from_f32<E>(v.w * a.alpha);
        atomicAdd((float4 *)(pr + c), v);
        atomicAdd((float4 *)(tr + c), v);
      }
    } else {
      for (int c = lane; c < a.D; c += 32) {
        const float v = to_f32(dr[c]);
        xr[c] = from_f32<E>(v * a.alpha);
        atomicAdd(pr + c, v);
        atomicAdd(tr + c, v);
      }
    }
  }
}

// ---- block versions for D % 8 == 0: a CTA takes 64 tokens, one thread per token finds the two
// table rows, then all threads move 8-element pieces ---------------------------------------------
constexpr int TSPOS_ROWS = 64;

template <typename E> struct Pack8 { uint4 raw; };  // 8 x 16-bit
template <> struct Pack8<float> { float4 lo, hi; };

template <typename E> __device__ __forceinline__ void unpack8(const Pack8<E> &p, float (&f)[8]) {
  const E *e = reinterpret_cast<const E *>(&p);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = to_f32(e[i]);
}
template <typename E> __device__ __forceinline__ void pack8(const float (&f)[8], Pack8<E> &p) {
  E *e = reinterpret_cast<E *>(&p);
#pragma unroll
  for (int i = 0; i < 8; ++i) e[i] = from_f32<E>(f[i]);
}

template <typename E, typename TE>
__global__ void __launch_bounds__(TSPOS_THREADS)
ts_pos_fwd_block_kernel(TsPosArgs a, const E *__restrict__ x, const TE *__restrict__ pos_w,
                        const TE *__restrict__ ts_w, E *__restrict__ out) {
  __shared__ int s_pos[TSPOS_ROWS], s_ts[TSPOS_ROWS];
  const int64_t g0 = (int64_t)blockIdx.x * TSPOS_ROWS;
  const int rows = (int)((a.total - g0) < TSPOS_ROWS ? (a.total - g0) : TSPOS_ROWS);
  if ((int)threadIdx.x < rows) ts_pos_indices(a, g0 + threadIdx.x, s_pos[threadIdx.x], s_ts[threadIdx.x]);
  __syncthreads();
  const int per_row = a.D >> 3;
  const int n = rows * per_row;
  const Pack8<E> *xin = reinterpret_cast<const Pack8<E> *>(x + g0 * a.D);
  Pack8<E> *xout = reinterpret_cast<Pack8<E> *>(out + g0 * a.D);
#pragma unroll 2
  for (int i = threadIdx.x; i < n; i += TSPOS_THREADS) {
    const int r = i / per_row, c = i - r * per_row;
    const Pack8<E> xv = xin[i];
    const Pack8<TE> pv = reinterpret_cast<const Pack8<TE> *>(pos_w + (int64_t)s_pos[r] * a.D)[c];
    const Pack8<TE> tv = reinterpret_cast<const Pack8<TE> *>(ts_w + (int64_t)s_ts[r] * a.D)[c];
    float xf[8], pf[8], tf[8], of[8];
    unpack8<E>(xv, xf);
    unpack8<TE>(pv, pf);
    unpack8<TE>(tv, tf);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float scaled = to_f32(from_f32<E>(__fmul_rn(xf[k], a.alpha)));
      const TE emb = from_f32<TE>(__fadd_rn(tf[k], pf[k]));
      of[k] = __fadd_rn(scaled, to_f32(from_f32<E>(to_f32(emb))));
    }
    Pack8<E> ov;
    pack8<E>(of, ov);
    xout[i] = ov;
  }
}

template <typename E> struct Quad { uint2 raw; };  // 4 x 16-bit
template <> struct Quad<float> { float4 raw; };
template <typename E> __device__ __forceinline__ float4 load4(const E *p) {
  const Quad<E> q = *reinterpret_cast<const Quad<E> *>(p);
  const E *e = reinterpret_cast<const E *>(&q);
  return make_float4(to_f32(e[0]), to_f32(e[1]), to_f32(e[2]), to_f32(e[3]));
}
template <typename E> __device__ __forceinline__ void store4(E *p, float4 v) {
  Quad<E> q;
  E *e = reinterpret_cast<E *>(&q);
  e[0] = from_f32<E>(v.x); e[1] = from_f32<E>(v.y); e[2] = from_f32<E>(v.z); e[3] = from_f32<E>(v.w);
  *reinterpret_cast<Quad<E> *>(p) = q;
}

// Backward: a thread owns one 4-column piece and walks a run of consecutive tokens, adding up dy
// for as long as the table row stays the same (time buckets change slowly along a sequence; all
// targets share one position row), so that one vector reduction goes out per run.
template <typename E>
__global__ void __launch_bounds__(TSPOS_THREADS)
ts_pos_bwd_block_kernel(TsPosArgs a, const E *__restrict__ dy, E *__restrict__ dx, float *__restrict__ d_pos,
                        float *__restrict__ d_ts) {
  __shared__ int s_pos[TSPOS_ROWS], s_ts[TSPOS_ROWS];
  const int64_t g0 = (int64_t)blockIdx.x * TSPOS_ROWS;
  const int rows = (int)((a.total - g0) < TSPOS_ROWS ? (a.total - g0) : TSPOS_ROWS);
  if ((int)threadIdx.x < rows) ts_pos_indices(a, g0 + threadIdx.x, s_pos[threadIdx.x], s_ts[threadIdx.x]);
  __syncthreads();
  const int chunks = a.D >> 2;
  // row groups: the largest power of two that fits the CTA's threads over the chunks
  int groups = 1;
  while (groups * 2 * chunks <= TSPOS_THREADS && groups * 2 <= TSPOS_ROWS) groups *= 2;
  const int rows_per_group = TSPOS_ROWS / groups;
  for (int item = threadIdx.x; item < groups * chunks; item += TSPOS_THREADS) {
    const int grp = item / chunks, c = item - grp * chunks;
    const int r0 = grp * rows_per_group;
    const int r1 = (r0 + rows_per_group) < rows ? (r0 + rows_per_group) : rows;
    float4 acc_p = make_float4(0.f, 0.f, 0.f, 0.f), acc_t = acc_p;
    for (int r = r0; r < r1; ++r) {
      const float4 v = load4(dy + (g0 + r) * a.D + c * 4);
      store4(dx + (g0 + r) * a.D + c * 4,
             make_float4(v.x * a.alpha, v.y * a.alpha, v.z * a.alpha, v.w * a.alpha));
      acc_p.x += v.x; acc_p.y += v.y; acc_p.z += v.z; acc_p.w += v.w;
      acc_t.x += v.x; acc_t.y += v.y; acc_t.z += v.z; acc_t.w += v.w;
      const bool last = r + 1 == r1;
      if (last || s_pos[r + 1] != s_pos[r]) {
        atomicAdd(reinterpret_cast<float4 *>(d_pos + (int64_t)s_pos[r] * a.D) + c, acc_p);
        acc_p = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      if (last || s_ts[r + 1] != s_ts[r]) {
        atomicAdd(reinterpret_cast<float4 *>(d_ts + (int64_t)s_ts[r] * a.D) + c, acc_t);
        acc_t = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
  }
}

inline unsigned ts_pos_grid(int64_t total) {
  int64_t want = (total + TSPOS_THREADS / 32 - 1) / (TSPOS_THREADS / 32);
  const int64_t cap = 148 * 8;
  return (unsigned)(want < cap ? (want > 0 ? want : 1) : cap);
}

template <typename E>
int ts_pos_fwd_t(const TsPosArgs &a, const void *x, const void *pos_w, const void *ts_w, int table_dtype, void *out,
                 cudaStream_t st) {
  const unsigned blocks = (unsigned)((a.total + TSPOS_ROWS - 1) / TSPOS_ROWS);
  const bool aligned = (((uintptr_t)x | (uintptr_t)pos_w | (uintptr_t)ts_w | (uintptr_t)out) & 15) == 0;
  if ((a.D & 7) == 0 && aligned) {
    if (table_dtype == B200_HSTU_F32)
      ts_pos_fwd_block_kernel<E, float><<<blocks, TSPOS_THREADS, 0, st>>>(a, (const E *)x, (const float *)pos_w,
                                                                          (const float *)ts_w, (E *)out);
    else
      ts_pos_fwd_block_kernel<E, E><<<blocks, TSPOS_THREADS, 0, st>>>(a, (const E *)x, (const E *)pos_w,
                                                                      (const E *)ts_w, (E *)out);
    count_launch();
    B200_CHECK_LAUNCH("ts_pos_fwd_block_kernel");
    return 0;
  }
  if (table_dtype == B200_HSTU_F32)
    ts_pos_fwd_kernel<E, float><<<ts_pos_grid(a.total), TSPOS_THREADS, 0, st>>>(
        a, (const E *)x, (const float *)pos_w, (const float *)ts_w, (E *)out);
  else
    ts_pos_fwd_kernel<E, E><<<ts_pos_grid(a.total), TSPOS_THREADS, 0, st>>>(a, (const E *)x, (const E *)pos_w,
                                                                             (const E *)ts_w, (E *)out);
  count_launch();
  B200_CHECK_LAUNCH("ts_pos_fwd_kernel");
  return 0;
}

template <typename E>
int ts_pos_bwd_t(const TsPosArgs &a, const void *dy, void *dx, float *d_pos, float *d_ts, cudaStream_t st) {
  const bool aligned = (((uintptr_t)d_pos | (uintptr_t)d_ts | (uintptr_t)dy | (uintptr_t)dx) & 15) == 0;
  if ((a.D & 3) == 0 && aligned) {
    const unsigned blocks = (unsigned)((a.total + TSPOS_ROWS - 1) / TSPOS_ROWS);
    ts_pos_bwd_block_kernel<E><<<blocks, TSPOS_THREADS, 0, st>>>(a, (const E *)dy, (E *)dx, d_pos, d_ts);
    count_launch();
    B200_CHECK_LAUNCH("ts_pos_bwd_block_kernel");
    return 0;
  }
  ts_pos_bwd_kernel<E><<<ts_pos_grid(a.total), TSPOS_THREADS, 0, st>>>(a, (const E *)dy, (E *)dx, d_pos, d_ts);
  count_launch();
  B200_CHECK_LAUNCH("ts_pos_bwd_kernel");
  return 0;
}

}  // namespace

int jagged_concat_split(const b200_hstu_jagged_args &j, bool split, cudaStream_t st) {
  if (j.B < 0 || j.total_rows < 0 || j.row_bytes <= 0 || j.right_rows_first < 0)
    return fail(B200_HSTU_EINVAL, "jagged: negative size");
  if (!j.offsets_left && !j.offsets_right && (j.dense_len_left < 0 || j.dense_len_right < 0))
    return fail(B200_HSTU_EINVAL, "jagged: a side without offsets needs its dense length");
  if (j.total_rows == 0 || j.B == 0) return 0;
  // a side that holds no rows may be a null pointer
  if (!j.combined || (!j.left && !j.right)) return fail(B200_HSTU_EINVAL, "jagged: null tensor");
  JaggedArgs a;
  a.off_l = j.offsets_left;
  a.off_r = j.offsets_right;
  a.dense_l = j.dense_len_left;
  a.dense_r = j.dense_len_right;
  a.shift = j.right_rows_first;
  a.B = j.B;
  a.total = j.total_rows;
  a.left = (char *)j.left;
  a.right = (char *)j.right;
  a.comb = (char *)j.combined;
  a.row_bytes = j.row_bytes;
  ProfileScope prof(PROF_JAGGED, st);
  const uintptr_t align = (uintptr_t)j.left | (uintptr_t)j.right | (uintptr_t)j.combined | (uintptr_t)j.row_bytes;
  if ((align & 15) == 0) return launch_jagged<uint4>(a, split, st);
  if ((align & 3) == 0) return launch_jagged<uint32_t>(a, split, st);
  if ((align & 1) == 0) return launch_jagged<uint16_t>(a, split, st);
  return launch_jagged<uint8_t>(a, split, st);
}

static int fill_ts_pos(const b200_hstu_ts_pos_args &p, TsPosArgs &a) {
  if (p.B < 0 || p.total_rows < 0 || p.D <= 0 || p.max_pos_ind <= 0 || p.ts_rows <= 0)
    return fail(B200_HSTU_EINVAL, "add_timestamp_positional_embeddings: bad size");
  if (p.total_rows > 0 && (!p.seq_offsets || !p.seq_lengths || !p.timestamps))
    return fail(B200_HSTU_EINVAL, "add_timestamp_positional_embeddings: null index tensor");
  a.seq_offsets = p.seq_offsets;
  a.seq_lengths = p.seq_lengths;
  a.num_targets = p.num_targets;
  a.timestamps = p.timestamps;
  a.B = p.B;
  a.total = p.total_rows;
  a.D = p.D;
  a.max_contextual_seq_len = p.max_contextual_seq_len;
  a.max_pos_ind = p.max_pos_ind;
  a.ts_rows = p.ts_rows;
  a.ts_bucket_max = p.ts_bucket_max;
  a.interleave_targets = p.interleave_targets;
  a.log_buckets = p.time_bucket_fn;
  a.alpha = p.alpha;
  return 0;
}

int ts_pos_fwd(const b200_hstu_ts_pos_args &p, cudaStream_t st) {
  TsPosArgs a;
  if (int rc = fill_ts_pos(p, a)) return rc;
  if (p.total_rows == 0) return 0;
  if (!p.seq_embeddings || !p.pos_weight || !p.ts_weight || !p.out)
    return fail(B200_HSTU_EINVAL, "add_timestamp_positional_embeddings: null tensor");
  if (p.table_dtype != B200_HSTU_F32 && p.table_dtype != p.dtype)
    return fail(B200_HSTU_EUNSUPPORTED, "embedding tables must be float32 or of the sequence dtype");
  ProfileScope prof(PROF_TS_POS, st);
  switch (p.dtype) {
    case B200_HSTU_F32: return ts_pos_fwd_t<float>(a, p.seq_embeddings, p.pos_weight, p.ts_weight, p.table_dtype, p.out, st);
    case B200_HSTU_BF16: return ts_pos_fwd_t<__nv_bfloat16>(a, p.seq_embeddings, p.pos_weight, p.ts_weight, p.table_dtype, p.out, st);
    case B200_HSTU_F16: return ts_pos_fwd_t<__half>(a, p.seq_embeddings, p.pos_weight, p.ts_weight, p.table_dtype, p.out, st);
    default: return fail(B200_HSTU_EINVAL, "unknown dtype %d", p.dtype);
  }
}

int ts_pos_bwd(const b200_hstu_ts_pos_args &p, cudaStream_t st) {
  TsPosArgs a;
  if (int rc = fill_ts_pos(p, a)) return rc;
  if (p.total_rows == 0) return 0;
  if (!p.d_out || !p.d_seq_embeddings || !p.d_pos_weight || !p.d_ts_weight)
    return fail(B200_HSTU_EINVAL, "add_timestamp_positional_embeddings backward: null tensor");
  ProfileScope prof(PROF_TS_POS, st);
  switch (p.dtype) {
    case B200_HSTU_F32: return ts_pos_bwd_t<float>(a, p.d_out, p.d_seq_embeddings, p.d_pos_weight, p.d_ts_weight, st);
    case B200_HSTU_BF16: return ts_pos_bwd_t<__nv_bfloat16>(a, p.d_out, p.d_seq_embeddings, p.d_pos_weight, p.d_ts_weight, st);
    case B200_HSTU_F16: return ts_pos_bwd_t<__half>(a, p.d_out, p.d_seq_embeddings, p.d_pos_weight, p.d_ts_weight, st);
    default: return fail(B200_HSTU_EINVAL, "unknown dtype %d", p.dtype);
  }
}

}  // namespace b200hstu
