// CUDA-core (SIMT) jagged HSTU attention, forward and backward, fp32 accumulation.
//
// This is the path for fp32 tensors and for head dimensions the tensor-core kernels do not
// cover (anything other than 64 / 128, or d_qk != d_v).  It is written for clarity and exact
// mask semantics, not for peak throughput: 32x32 tiles, one CTA of 128 threads per
// (query tile, head, sequence) in the forward and dQ kernels and per (kv tile, head, sequence)
// in the dK/dV kernel.  The backward uses two kernels so that every gradient element has a
// single owner: no atomics, no scratch, bit-reproducible.
//
// Math (generative_recommenders/ops/pytorch/pt_hstu_attention.py:146-187, backward as in
// generative_recommenders/ops/triton/triton_hstu_attention.py:1905-2020):
//   x = alpha * q.k (+ bias[|i-j|]);  P = silu(x) * scale * mask;  O = P V
//   dV = P^T dO;  dP = dO V^T;  dS = dP * silu'(x) * scale * mask;  dQ = alpha dS K;  dK = alpha dS^T Q
//   dbias[d] = sum of dS over the pairs with |i - j| = d (all heads and sequences), when asked for
// Optional dropout on P (pt_hstu_attention.py:180-181: after scale and mask, before P V): P and dP are
// multiplied by keep(i, h, j) / (1 - ratio), the mask a pure function of the seed and the element's
// index, so that the three kernels agree on it without storing it.
#include "common.cuh"

namespace b200hstu {

namespace {

constexpr int T = 32;          // tile edge
constexpr int NTHREADS = 128;  // 4 warps; thread t owns row t/4 and the 8 columns (t%4) + 4*jj

struct SimtParams {
  const void *q, *k, *v, *dout;
  void *out, *dq, *dk, *dv;
  const int32_t *seq_offsets, *num_targets;
  const float *attn_scale;
  int64_t attn_scale_numel;
  const float *bias;
  int bias_numel;
  float *dbias;   // backward, optional: gradient of `bias`, accumulated with atomics
  int64_t q_rs, k_rs, v_rs, o_rs, do_rs, dq_rs, dk_rs, dv_rs;
  int64_t q_hs, k_hs, v_hs, o_hs, do_hs, dq_hs, dk_hs, dv_hs;
  int H, dqk, dv_dim, max_seq_len;
  float alpha;
  int W, c, F;
  int delta;   // > 0 (forward only): q / out hold the last `delta` positions of each sequence, `delta` rows each
  const unsigned long long *drop_seed;   // device; NULL = no dropout
  uint32_t drop_thr;                      // a weight is dropped when its 16 random bits are below this
  float drop_scale;                       // 65536 / (65536 - drop_thr)
};

// Dropout factor of the weight of (query row `token` of the jagged tensor, head h, key position j).
struct DropMask {
  uint32_t k0, k1, thr;
  float scale;
  bool on;
  __device__ __forceinline__ void init(const SimtParams &p) {
    on = p.drop_seed != nullptr;
    thr = p.drop_thr;
    scale = p.drop_scale;
    const unsigned long long s = on ? *p.drop_seed : 0ull;
    k0 = (uint32_t)s;
    k1 = (uint32_t)(s >> 32);
  }
  __device__ __forceinline__ float factor(const SimtParams &p, int64_t token, int h, int j) const {
    if (!on) return 1.f;
    const uint64_t idx = ((uint64_t)token * (uint64_t)p.H + (uint64_t)h) * (uint64_t)p.max_seq_len + (uint64_t)j;
    return philox_keep(k0, k1, idx, thr) ? scale : 0.f;
  }
};

template <typename E>
__device__ __forceinline__ void load_tile(float *dst, int ld, const E *src, int64_t row_stride, int row0, int nrows,
                                          int d) {
  // dst[r][x] (leading dim ld) <- src[(row0 + r) * row_stride + x], zero beyond nrows
  for (int idx = threadIdx.x; idx < T * d; idx += NTHREADS) {
    int r = idx / d, x = idx - r * d;
    float val = 0.f;
    if (r < nrows) val = to_f32(src[(int64_t)(row0 + r) * row_stride + x]);
    dst[r * ld + x] = val;
  }
}

// acc[jj] = sum_x A[r][x] * Bm[(cg + 4 jj)][x]
__device__ __forceinline__ void dot_rows(float (&acc)[8], const float *A, const float *Bm, int ld, int d, int r,
                                         int cg) {
#pragma unroll
  for (int jj = 0; jj < 8; ++jj) acc[jj] = 0.f;
  const float *a = A + r * ld;
  for (int x = 0; x < d; ++x) {
    float av = a[x];
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) acc[jj] = fmaf(av, Bm[(cg + 4 * jj) * ld + x], acc[jj]);
  }
}

struct SeqGeom {
  int start, len, nt;
  SeqMask m;
};

__device__ __forceinline__ SeqGeom seq_geom(const SimtParams &p, int b) {
  SeqGeom g;
  g.start = p.seq_offsets[b];
  g.len = p.seq_offsets[b + 1] - g.start;
  g.nt = p.num_targets ? p.num_targets[b] : 0;
  g.m = make_seq_mask(g.len, p.max_seq_len, g.nt, p.c, p.W, p.F);
  return g;
}

__device__ __forceinline__ float row_scale(const SimtParams &p, int64_t token) {
  if (p.attn_scale == nullptr) return 1.f / (float)p.max_seq_len;
  return p.attn_scale_numel == 1 ? p.attn_scale[0] : p.attn_scale[token];
}

__device__ __forceinline__ bool tiles_overlap(const KvRange &r, int n0) {
  int n1 = n0 + T;
  bool in_main = n0 < r.hi && n1 > r.lo;
  bool in_diag = r.diag_lo >= 0 && n0 < r.diag_lo + T && n1 > r.diag_lo;
  return in_main || in_diag;
}

// Rows of a sequence at or beyond max_seq_len never take part; the reference returns zeros for
// them (its dense_to_jagged pads).  The grid only covers max_seq_len rows, so the CTA of the last
// tile also clears whatever lies beyond the grid.
template <typename E>
__device__ __forceinline__ void zero_rows_beyond_grid(E *base, int64_t row_stride, int64_t head_stride, int h,
                                                      int start, int len, int d) {
  if (blockIdx.x != gridDim.x - 1) return;
  int first = (int)gridDim.x * T;
  for (int64_t idx = (int64_t)first * d + threadIdx.x; idx < (int64_t)len * d; idx += NTHREADS) {
    int i = (int)(idx / d), x = (int)(idx - (int64_t)i * d);
    base[(int64_t)(start + i) * row_stride + (int64_t)h * head_stride + x] = from_f32<E>(0.f);
  }
}

// ---------------------------------------------------------------------------------------
// forward (MODE 0) and dQ (MODE 1): query-stationary
// ---------------------------------------------------------------------------------------
template <typename E, int MAXD, int MODE>
__global__ void __launch_bounds__(NTHREADS) attn_q_stationary_kernel(SimtParams p) {
  extern __shared__ float smem[];
  const int b = blockIdx.z, h = blockIdx.y;
  const SeqGeom g = seq_geom(p, b);
  const bool cached = MODE == 0 && p.delta > 0;
  if ((int)blockIdx.x * T >= (cached ? p.delta : g.len)) return;
  // position of the tile's first query inside the sequence, and its row in the q / out tensors
  const int m0 = (int)blockIdx.x * T + (cached ? g.m.L - p.delta : 0);
  const int64_t qrow0 = cached ? (int64_t)b * p.delta + (int)blockIdx.x * T : (int64_t)g.start + m0;
  const int dqk = p.dqk, dvd = p.dv_dim;
  const int dmax = dqk > dvd ? dqk : dvd;
  const int ld = dmax + 1;
  float *Qs = smem;               // [T][ld]   q rows
  float *Ks = Qs + T * ld;        // [T][ld]   k rows
  float *Vs = Ks + T * ld;        // [T][ld]   v rows
  float *Gs = Vs + T * ld;        // [T][ld]   dout rows (MODE 1)
  float *Ps = Gs + (MODE == 1 ? T * ld : 0);  // [T][T+1]
  const int r = threadIdx.x >> 2, cg = threadIdx.x & 3;
  const int out_d = MODE == 0 ? dvd : dqk;  // width of the accumulated output row
  float acc_o[MAXD / 4];
#pragma unroll
  for (int i = 0; i < MAXD / 4; ++i) acc_o[i] = 0.f;

  const int L = g.m.L;
  DropMask drop;
  drop.init(p);
  if (m0 < L) {
    const E *qp = (const E *)p.q + qrow0 * p.q_rs + (int64_t)h * p.q_hs;
    const E *kp = (const E *)p.k + (int64_t)g.start * p.k_rs + (int64_t)h * p.k_hs;
    const E *vp = (const E *)p.v + (int64_t)g.start * p.v_rs + (int64_t)h * p.v_hs;
    const int qrows = min(T, L - m0);
    load_tile(Qs, ld, qp, p.q_rs, 0, qrows, dqk);
    if (MODE == 1) {
      const E *gp = (const E *)p.dout + (int64_t)g.start * p.do_rs + (int64_t)h * p.do_hs;
      load_tile(Gs, ld, gp, p.do_rs, m0, qrows, dvd);
    }
    const KvRange range = kv_range_for_q_tile(g.m, g.len, g.nt, m0, T);
    const int i = m0 + r;
    const int id_i = g.m.id(i);
    const float sc = (i >= 0 && i < L) ? row_scale(p, (int64_t)g.start + i) : 0.f;
    for (int n0 = 0; n0 < L; n0 += T) {
      if (!tiles_overlap(range, n0)) continue;
      __syncthreads();
      const int krows = min(T, L - n0);
      load_tile(Ks, ld, kp, p.k_rs, n0, krows, dqk);
      load_tile(Vs, ld, vp, p.v_rs, n0, krows, dvd);
      __syncthreads();
      float s[8];
      dot_rows(s, Qs, Ks, ld, dqk, r, cg);
      float dp[8];
      if (MODE == 1) dot_rows(dp, Gs, Vs, ld, dvd, r, cg);
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        int j = n0 + cg + 4 * jj;
        bool ok = i >= 0 && i < L && j < L && g.m.valid_ids(i, j, id_i, g.m.id(j));
        float x = s[jj] * p.alpha;
        if (p.bias != nullptr) {
          int dist = i > j ? i - j : j - i;
          if (dist < p.bias_numel) x += p.bias[dist];
        }
        float val;
        if (MODE == 0) {
          val = ok ? siluf_(x) * sc : 0.f;
        } else {
          val = ok ? dp[jj] * dsiluf_(x) * sc : 0.f;   // dS; alpha is applied to the finished dQ row
        }
        if (ok && drop.on) val *= drop.factor(p, (int64_t)g.start + i, h, j);
        Ps[r * (T + 1) + cg + 4 * jj] = val;
      }
      __syncthreads();
      if (MODE == 1 && p.dbias != nullptr && threadIdx.x < 2 * T - 1) {
        // one thread per diagonal of the 32 x 32 tile: rows - columns = m
        const int m = (int)threadIdx.x - (T - 1);
        float sum = 0.f;
        for (int rr = m > 0 ? m : 0; rr < T && rr - m < T; ++rr) sum += Ps[rr * (T + 1) + rr - m];
        int dist = m0 - n0 + m;
        dist = dist < 0 ? -dist : dist;
        if (sum != 0.f && dist < p.bias_numel) atomicAdd(p.dbias + dist, sum);
      }
      const float *Bm = MODE == 0 ? Vs : Ks;
      for (int j = 0; j < T; ++j) {
        float pv = Ps[r * (T + 1) + j];
#pragma unroll
        for (int cc = 0; cc < MAXD / 4; ++cc) {
          int x = cg + 4 * cc;
          if (x < out_d) acc_o[cc] = fmaf(pv, Bm[j * ld + x], acc_o[cc]);
        }
      }
    }
  }
  // rows at or beyond max_seq_len produce zeros (the reference's dense_to_jagged pads them)
  if (MODE == 0) {
    if (!cached) zero_rows_beyond_grid((E *)p.out, p.o_rs, p.o_hs, h, g.start, g.len, dvd);
  } else {
    zero_rows_beyond_grid((E *)p.dq, p.dq_rs, p.dq_hs, h, g.start, g.len, dqk);
  }
  const int i = m0 + r;
  if (i >= 0 && i < g.len) {
    E *op;
    if (MODE == 0)
      op = (E *)p.out + (qrow0 + r) * p.o_rs + (int64_t)h * p.o_hs;
    else
      op = (E *)p.dq + (int64_t)(g.start + i) * p.dq_rs + (int64_t)h * p.dq_hs;
    const float fin = MODE == 1 ? p.alpha : 1.f;
#pragma unroll
    for (int cc = 0; cc < MAXD / 4; ++cc) {
      int x = cg + 4 * cc;
      if (x < out_d) op[x] = from_f32<E>(acc_o[cc] * fin);
    }
  }
}

// ---------------------------------------------------------------------------------------
// dK, dV: key/value-stationary
// ---------------------------------------------------------------------------------------
template <typename E, int MAXD>
__global__ void __launch_bounds__(NTHREADS) attn_kv_stationary_bwd_kernel(SimtParams p) {
  extern __shared__ float smem[];
  const int b = blockIdx.z, h = blockIdx.y, n0 = blockIdx.x * T;
  const SeqGeom g = seq_geom(p, b);
  if (n0 >= g.len) return;
  const int dqk = p.dqk, dvd = p.dv_dim;
  const int dmax = dqk > dvd ? dqk : dvd;
  const int ld = dmax + 1;
  float *Qs = smem;
  float *Ks = Qs + T * ld;
  float *Vs = Ks + T * ld;
  float *Gs = Vs + T * ld;
  float *Ps = Gs + T * ld;          // [T][T+1]  P
  float *Ss = Ps + T * (T + 1);     // [T][T+1]  dS
  const int r = threadIdx.x >> 2, cg = threadIdx.x & 3;
  float acc_dk[MAXD / 4], acc_dv[MAXD / 4];
#pragma unroll
  for (int i = 0; i < MAXD / 4; ++i) acc_dk[i] = acc_dv[i] = 0.f;
  const int L = g.m.L;
  DropMask drop;
  drop.init(p);
  if (n0 < L) {
    const E *qp = (const E *)p.q + (int64_t)g.start * p.q_rs + (int64_t)h * p.q_hs;
    const E *kp = (const E *)p.k + (int64_t)g.start * p.k_rs + (int64_t)h * p.k_hs;
    const E *vp = (const E *)p.v + (int64_t)g.start * p.v_rs + (int64_t)h * p.v_hs;
    const E *gp = (const E *)p.dout + (int64_t)g.start * p.do_rs + (int64_t)h * p.do_hs;
    const int krows = min(T, L - n0);
    load_tile(Ks, ld, kp, p.k_rs, n0, krows, dqk);
    load_tile(Vs, ld, vp, p.v_rs, n0, krows, dvd);
    for (int m0 = 0; m0 < L; m0 += T) {
      const KvRange range = kv_range_for_q_tile(g.m, g.len, g.nt, m0, T);
      if (!tiles_overlap(range, n0)) continue;
      __syncthreads();
      const int qrows = min(T, L - m0);
      load_tile(Qs, ld, qp, p.q_rs, m0, qrows, dqk);
      load_tile(Gs, ld, gp, p.do_rs, m0, qrows, dvd);
      __syncthreads();
      const int i = m0 + r;
      const int id_i = g.m.id(i);
      const float sc = i < L ? row_scale(p, (int64_t)g.start + i) : 0.f;
      float s[8], dp[8];
      dot_rows(s, Qs, Ks, ld, dqk, r, cg);
      dot_rows(dp, Gs, Vs, ld, dvd, r, cg);
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        int j = n0 + cg + 4 * jj;
        bool ok = i < L && j < L && g.m.valid_ids(i, j, id_i, g.m.id(j));
        float x = s[jj] * p.alpha;
        if (p.bias != nullptr) {
          int dist = i > j ? i - j : j - i;
          if (dist < p.bias_numel) x += p.bias[dist];
        }
        const float keep = (ok && drop.on) ? drop.factor(p, (int64_t)g.start + i, h, j) : 1.f;
        Ps[r * (T + 1) + cg + 4 * jj] = ok ? siluf_(x) * sc * keep : 0.f;
        Ss[r * (T + 1) + cg + 4 * jj] = ok ? dp[jj] * dsiluf_(x) * sc * p.alpha * keep : 0.f;
      }
      __syncthreads();
      // this thread now owns kv row `r` (of the stationary tile) and columns cg + 4 cc
      for (int qi = 0; qi < T; ++qi) {
        float pv = Ps[qi * (T + 1) + r];
        float ds = Ss[qi * (T + 1) + r];
#pragma unroll
        for (int cc = 0; cc < MAXD / 4; ++cc) {
          int x = cg + 4 * cc;
          if (x < dvd) acc_dv[cc] = fmaf(pv, Gs[qi * ld + x], acc_dv[cc]);
          if (x < dqk) acc_dk[cc] = fmaf(ds, Qs[qi * ld + x], acc_dk[cc]);
        }
      }
    }
  }
  zero_rows_beyond_grid((E *)p.dk, p.dk_rs, p.dk_hs, h, g.start, g.len, dqk);
  zero_rows_beyond_grid((E *)p.dv, p.dv_rs, p.dv_hs, h, g.start, g.len, dvd);
  const int j = n0 + r;
  if (j < g.len) {
    E *dkp = (E *)p.dk + (int64_t)(g.start + j) * p.dk_rs + (int64_t)h * p.dk_hs;
    E *dvp = (E *)p.dv + (int64_t)(g.start + j) * p.dv_rs + (int64_t)h * p.dv_hs;
#pragma unroll
    for (int cc = 0; cc < MAXD / 4; ++cc) {
      int x = cg + 4 * cc;
      if (x < dqk) dkp[x] = from_f32<E>(acc_dk[cc]);
      if (x < dvd) dvp[x] = from_f32<E>(acc_dv[cc]);
    }
  }
}

SimtParams make_params(const b200_hstu_attn_args &a) {
  SimtParams p;
  p.q = a.q; p.k = a.k; p.v = a.v; p.dout = a.dout;
  p.out = a.out; p.dq = a.dq; p.dk = a.dk; p.dv = a.dv_;
  p.seq_offsets = a.seq_offsets; p.num_targets = a.num_targets;
  p.attn_scale = a.attn_scale; p.attn_scale_numel = a.attn_scale_numel;
  p.bias = a.bias_by_distance; p.bias_numel = a.bias_numel;
  p.dbias = a.bias_by_distance != nullptr ? a.d_bias_by_distance : nullptr;
  p.q_rs = a.q_row_stride; p.k_rs = a.k_row_stride; p.v_rs = a.v_row_stride; p.o_rs = a.o_row_stride;
  p.do_rs = a.do_row_stride; p.dq_rs = a.dq_row_stride; p.dk_rs = a.dk_row_stride; p.dv_rs = a.dv_row_stride;
  p.q_hs = a.q_head_stride; p.k_hs = a.k_head_stride; p.v_hs = a.v_head_stride; p.o_hs = a.o_head_stride;
  p.do_hs = a.do_head_stride; p.dq_hs = a.dq_head_stride; p.dk_hs = a.dk_head_stride; p.dv_hs = a.dv_head_stride;
  p.H = a.H; p.dqk = a.dqk; p.dv_dim = a.dv; p.max_seq_len = a.max_seq_len;
  p.alpha = a.alpha; p.W = a.max_attn_len; p.c = a.contextual_seq_len; p.F = a.min_full_attn_seq_len;
  p.delta = a.delta_size;
  p.drop_seed = nullptr; p.drop_thr = 0; p.drop_scale = 1.f;
  if (a.dropout_ratio > 0.f && a.dropout_seed != nullptr) {   // (the ratio's range is checked by the caller)
    uint32_t thr = (uint32_t)(a.dropout_ratio * 65536.f + 0.5f);
    if (thr > 65535u) thr = 65535u;
    p.drop_seed = (const unsigned long long *)a.dropout_seed;
    p.drop_thr = thr;
    p.drop_scale = 65536.f / (float)(65536u - thr);
  }
  return p;
}

template <typename E, int MAXD>
int launch_fwd(const b200_hstu_attn_args &a, cudaStream_t st) {
  SimtParams p = make_params(a);
  int dmax = a.dqk > a.dv ? a.dqk : a.dv;
  size_t smem = (size_t)(3 * T * (dmax + 1) + T * (T + 1)) * sizeof(float);
  auto kern = attn_q_stationary_kernel<E, MAXD, 0>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return check_cuda(e, "simt fwd smem attribute");
  const int q_rows = a.delta_size > 0 ? a.delta_size : a.max_seq_len;
  dim3 grid((unsigned)((q_rows + T - 1) / T), (unsigned)a.H, (unsigned)a.B);
  kern<<<grid, NTHREADS, smem, st>>>(p);
  count_launch();
  B200_CHECK_LAUNCH("simt attention forward");
  return 0;
}

template <typename E, int MAXD>
int launch_bwd(const b200_hstu_attn_args &a, cudaStream_t st) {
  SimtParams p = make_params(a);
  int dmax = a.dqk > a.dv ? a.dqk : a.dv;
  dim3 grid((unsigned)((a.max_seq_len + T - 1) / T), (unsigned)a.H, (unsigned)a.B);
  {
    size_t smem = (size_t)(4 * T * (dmax + 1) + T * (T + 1)) * sizeof(float);
    auto kern = attn_q_stationary_kernel<E, MAXD, 1>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return check_cuda(e, "simt dq smem attribute");
    kern<<<grid, NTHREADS, smem, st>>>(p);
    count_launch();
    B200_CHECK_LAUNCH("simt attention backward (dq)");
  }
  {
    size_t smem = (size_t)(4 * T * (dmax + 1) + 2 * T * (T + 1)) * sizeof(float);
    auto kern = attn_kv_stationary_bwd_kernel<E, MAXD>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return check_cuda(e, "simt dkdv smem attribute");
    kern<<<grid, NTHREADS, smem, st>>>(p);
    count_launch();
    B200_CHECK_LAUNCH("simt attention backward (dk, dv)");
  }
  return 0;
}

template <typename E>
int dispatch_d(const b200_hstu_attn_args &a, cudaStream_t st, bool bwd) {
  int dmax = a.dqk > a.dv ? a.dqk : a.dv;
  if (dmax <= 32) return bwd ? launch_bwd<E, 32>(a, st) : launch_fwd<E, 32>(a, st);
  if (dmax <= 64) return bwd ? launch_bwd<E, 64>(a, st) : launch_fwd<E, 64>(a, st);
  if (dmax <= 128) return bwd ? launch_bwd<E, 128>(a, st) : launch_fwd<E, 128>(a, st);
  if (dmax <= 256) return bwd ? launch_bwd<E, 256>(a, st) : launch_fwd<E, 256>(a, st);
  return fail(B200_HSTU_EUNSUPPORTED, "head dimension %d > 256 is not supported", dmax);
}

}  // namespace

int attn_simt(const b200_hstu_attn_args &a, cudaStream_t st, bool bwd) {
  switch (a.dtype) {
    case B200_HSTU_F32: return dispatch_d<float>(a, st, bwd);
    case B200_HSTU_BF16: return dispatch_d<__nv_bfloat16>(a, st, bwd);
    case B200_HSTU_F16: return dispatch_d<__half>(a, st, bwd);
    default: return fail(B200_HSTU_EINVAL, "unknown dtype %d", a.dtype);
  }
}

}  // namespace b200hstu
