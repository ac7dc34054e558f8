// Memory-bound stages around the attention: row LayerNorm (fwd/bwd), SiLU gating of U (fwd/bwd)
// and the output-side  y = act(u) * Norm(attn)  with its [u, attn, y] concatenation (fwd/bwd).
//
// All kernels are "one warp per row, row held in registers": a lane owns 16-byte vectors
// lane, lane + 32, ... of the row, so global loads/stores are coalesced 512-byte warp
// transactions, statistics are fp32 warp shuffles, and every input element is read from
// HBM exactly once.  Rows are limited to 32 * MAXV vectors (bf16/fp16: 2048 elements, fp32: 1024).
// Backward kernels are persistent (a few CTAs per SM): each warp walks rows with a stride,
// keeps its share of dweight / dbias in registers, the CTA reduces them through shared memory
// into one fp32 partial row, and a second small kernel sums the partial rows.
#include "common.cuh"

namespace b200hstu {
namespace {

constexpr int WARPS = 8;  // warps per CTA

template <typename E> struct VecInfo { static constexpr int EV = 16 / sizeof(E); };

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// sum over the `width` (power of two <= 32) consecutive lanes this lane belongs to
__device__ __forceinline__ float group_sum(float v, int width) {
  for (int o = width >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename E, int MAXV>
struct Row {
  static constexpr int EV = VecInfo<E>::EV;
  float v[MAXV][EV];

  __device__ __forceinline__ void load(const E *row, int D, int lane, bool vec_ok) {
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      int e0 = (k * 32 + lane) * EV;
      if (vec_ok && e0 + EV <= D) {
        uint4 raw = *reinterpret_cast<const uint4 *>(row + e0);
        const E *pe = reinterpret_cast<const E *>(&raw);
#pragma unroll
        for (int t = 0; t < EV; ++t) v[k][t] = to_f32(pe[t]);
      } else {
#pragma unroll
        for (int t = 0; t < EV; ++t) v[k][t] = (e0 + t < D) ? to_f32(row[e0 + t]) : 0.f;
      }
    }
  }
  __device__ __forceinline__ void store(E *row, int D, int lane, bool vec_ok) const {
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      int e0 = (k * 32 + lane) * EV;
      if (vec_ok && e0 + EV <= D) {
        uint4 raw;
        E *pe = reinterpret_cast<E *>(&raw);
#pragma unroll
        for (int t = 0; t < EV; ++t) pe[t] = from_f32<E>(v[k][t]);
        *reinterpret_cast<uint4 *>(row + e0) = raw;
      } else {
#pragma unroll
        for (int t = 0; t < EV; ++t)
          if (e0 + t < D) row[e0 + t] = from_f32<E>(v[k][t]);
      }
    }
  }
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int k = 0; k < MAXV; ++k)
#pragma unroll
      for (int t = 0; t < EV; ++t) v[k][t] = 0.f;
  }
};

// A row as raw 16-byte vectors: loaded one row ahead of its use, so the global loads of row r+1 are
// in flight while row r is reduced and stored (vector path only: aligned pointers and strides).
template <typename E, int MAXV>
struct RawRow {
  static constexpr int EV = VecInfo<E>::EV;
  uint4 v[MAXV];
  __device__ __forceinline__ void load(const E *row, int D, int lane) {
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      int e0 = (k * 32 + lane) * EV;
      v[k] = (e0 + EV <= D) ? __ldg(reinterpret_cast<const uint4 *>(row + e0)) : make_uint4(0, 0, 0, 0);
    }
  }
  __device__ __forceinline__ void unpack(Row<E, MAXV> &r) const {
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const E *pe = reinterpret_cast<const E *>(&v[k]);
#pragma unroll
      for (int t = 0; t < EV; ++t) r.v[k][t] = to_f32(pe[t]);
    }
  }
};

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// mean / rstd of a row held in registers (two-pass: mean first, then centred second moment)
template <typename E, int MAXV>
__device__ __forceinline__ void row_stats(const Row<E, MAXV> &x, int D, int lane, float eps, float &mean,
                                          float &rstd) {
  constexpr int EV = VecInfo<E>::EV;
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < MAXV; ++k)
#pragma unroll
    for (int t = 0; t < EV; ++t) s += x.v[k][t];  // out-of-range slots hold 0
  mean = warp_sum(s) / (float)D;
  float q = 0.f;
#pragma unroll
  for (int k = 0; k < MAXV; ++k)
#pragma unroll
    for (int t = 0; t < EV; ++t) {
      int e = (k * 32 + lane) * EV + t;
      float d = e < D ? x.v[k][t] - mean : 0.f;
      q += d * d;
    }
  rstd = rsqrtf(warp_sum(q) / (float)D + eps);
}

// ---------------------------------------------------------------------------------------
// LayerNorm
// ---------------------------------------------------------------------------------------
// Registers bound the number of resident warps, and with it the bytes in flight: on the vector
// path weight and bias stay packed (16-byte vectors, converted where they are used) and the kernel
// is compiled for three resident CTAs (four cost more in spills than they gain).
template <typename E, int MAXV>
__global__ void __launch_bounds__(WARPS * 32, MAXV <= 2 ? 3 : (MAXV <= 4 ? 2 : 1)) layer_norm_fwd_kernel(
    const E *__restrict__ x, int64_t x_rs, const E *__restrict__ w, const E *__restrict__ b, E *__restrict__ y,
    int64_t y_rs, float *__restrict__ mean_out, float *__restrict__ rstd_out, int64_t rows, int D, float eps,
    bool vec_ok) {
  constexpr int EV = VecInfo<E>::EV;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t step = (int64_t)gridDim.x * WARPS;
  int64_t row = (int64_t)blockIdx.x * WARPS + warp;
  constexpr bool PF = MAXV <= 8;  // one-row-ahead prefetch (every width: the packed weights leave room for it)
  if (PF && vec_ok) {
    RawRow<E, PF ? MAXV : 1> wraw, braw, nxt;
    wraw.load(w, D, lane);
    braw.load(b, D, lane);
    if (row < rows) nxt.load(x + row * x_rs, D, lane);
    for (; row < rows; row += step) {
      Row<E, PF ? MAXV : 1> xr;
      nxt.unpack(xr);
      if (row + step < rows) nxt.load(x + (row + step) * x_rs, D, lane);
      float mean, rstd;
      row_stats(xr, D, lane, eps, mean, rstd);
#pragma unroll
      for (int k = 0; k < (PF ? MAXV : 1); ++k) {
        const E *pw = reinterpret_cast<const E *>(&wraw.v[k]);
        const E *pb = reinterpret_cast<const E *>(&braw.v[k]);
#pragma unroll
        for (int t = 0; t < EV; ++t) xr.v[k][t] = (xr.v[k][t] - mean) * rstd * to_f32(pw[t]) + to_f32(pb[t]);
      }
      xr.store(y + row * y_rs, D, lane, true);
      if (lane == 0) {
        if (mean_out) mean_out[row] = mean;
        if (rstd_out) rstd_out[row] = rstd;
      }
    }
    return;
  }
  Row<E, MAXV> wr, br;
  wr.load(w, D, lane, vec_ok);
  br.load(b, D, lane, vec_ok);
  for (; row < rows; row += step) {
    Row<E, MAXV> xr;
    xr.load(x + row * x_rs, D, lane, vec_ok);
    float mean, rstd;
    row_stats(xr, D, lane, eps, mean, rstd);
#pragma unroll
    for (int k = 0; k < MAXV; ++k)
#pragma unroll
      for (int t = 0; t < EV; ++t) xr.v[k][t] = (xr.v[k][t] - mean) * rstd * wr.v[k][t] + br.v[k][t];
    xr.store(y + row * y_rs, D, lane, vec_ok);
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
  }
}

// shared-memory reduction of the per-warp column accumulators into partial[blockIdx.x][which][D]
template <typename E, int MAXV>
__device__ __forceinline__ void reduce_columns_to_partial(const Row<E, MAXV> &acc, float *smem, float *partial_row,
                                                          int D, int lane, int warp) {
  constexpr int EV = VecInfo<E>::EV;
  __syncthreads();
#pragma unroll
  for (int k = 0; k < MAXV; ++k)
#pragma unroll
    for (int t = 0; t < EV; ++t) {
      int e = (k * 32 + lane) * EV + t;
      if (e < D) smem[warp * D + e] = acc.v[k][t];
    }
  __syncthreads();
  for (int e = threadIdx.x; e < D; e += WARPS * 32) {
    float s = 0.f;
#pragma unroll
    for (int wv = 0; wv < WARPS; ++wv) s += smem[wv * D + e];
    partial_row[e] = s;
  }
}

template <typename E, int MAXV>
__global__ void __launch_bounds__(WARPS * 32, 2) layer_norm_bwd_kernel(
    const E *__restrict__ dy, int64_t dy_rs, const E *__restrict__ x, int64_t x_rs, const E *__restrict__ w,
    const float *__restrict__ mean_in, const float *__restrict__ rstd_in, E *__restrict__ dx, int64_t dx_rs,
    float *__restrict__ partial, int64_t rows, int D, bool vec_ok) {
  constexpr int EV = VecInfo<E>::EV;
  extern __shared__ float smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  Row<E, MAXV> wr, dw, db;
  wr.load(w, D, lane, vec_ok);
  dw.zero();
  db.zero();
  const float invD = 1.f / (float)D;
  const int64_t step = (int64_t)gridDim.x * WARPS;
  int64_t row = (int64_t)blockIdx.x * WARPS + warp;
  constexpr bool PF = MAXV <= 2;
  const bool pf = PF && vec_ok;
  RawRow<E, PF ? MAXV : 1> nx, ng;
  float nmean = 0.f, nrstd = 0.f;
  if constexpr (PF) {
    if (pf && row < rows) {
      nx.load(x + row * x_rs, D, lane);
      ng.load(dy + row * dy_rs, D, lane);
      nmean = mean_in[row];
      nrstd = rstd_in[row];
    }
  }
  for (; row < rows; row += step) {
    Row<E, MAXV> xr, gr;
    float mean, rstd;
    bool loaded = false;
    if constexpr (PF) {
      if (pf) {
        nx.unpack(xr);
        ng.unpack(gr);
        mean = nmean;
        rstd = nrstd;
        if (row + step < rows) {
          nx.load(x + (row + step) * x_rs, D, lane);
          ng.load(dy + (row + step) * dy_rs, D, lane);
          nmean = mean_in[row + step];
          nrstd = rstd_in[row + step];
        }
        loaded = true;
      }
    }
    if (!loaded) {
      xr.load(x + row * x_rs, D, lane, vec_ok);
      gr.load(dy + row * dy_rs, D, lane, vec_ok);
      mean = mean_in[row];
      rstd = rstd_in[row];
    }
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int k = 0; k < MAXV; ++k)
#pragma unroll
      for (int t = 0; t < EV; ++t) {
        int e = (k * 32 + lane) * EV + t;
        float xhat = e < D ? (xr.v[k][t] - mean) * rstd : 0.f;
        float g = gr.v[k][t];
        dw.v[k][t] += g * xhat;
        db.v[k][t] += g;
        float gw = g * wr.v[k][t];
        xr.v[k][t] = xhat;
        gr.v[k][t] = gw;
        c1 += gw * xhat;
        c2 += gw;
      }
    c1 = warp_sum(c1) * invD;
    c2 = warp_sum(c2) * invD;
#pragma unroll
    for (int k = 0; k < MAXV; ++k)
#pragma unroll
      for (int t = 0; t < EV; ++t) gr.v[k][t] = (gr.v[k][t] - c2 - xr.v[k][t] * c1) * rstd;
    gr.store(dx + row * dx_rs, D, lane, vec_ok);
  }
  float *prow = partial + (int64_t)blockIdx.x * 2 * D;
  reduce_columns_to_partial(dw, smem, prow, D, lane, warp);
  reduce_columns_to_partial(db, smem, prow + D, D, lane, warp);
}

// The same backward with the two column accumulators (dweight, dbias) of every warp in shared
// memory instead of registers: 64 registers fewer per thread, so three CTAs instead of two fit an
// SM and more rows are in flight (two CTAs for rows of four vectors per lane, which without this
// would neither fit a prefetched row into the registers nor a second CTA onto the SM).  Vector path
// only (aligned pointers and strides); eight vectors per lane run one CTA per SM.
// Shared memory: [2][WARPS][MAXV * EV / 4][32] float4, each lane touching only its own entries.
template <typename E, int MAXV>
__global__ void __launch_bounds__(WARPS * 32, MAXV <= 2 ? 3 : (MAXV <= 4 ? 2 : 1)) layer_norm_bwd_smem_kernel(
    const E *__restrict__ dy, int64_t dy_rs, const E *__restrict__ x, int64_t x_rs, const E *__restrict__ w,
    const float *__restrict__ mean_in, const float *__restrict__ rstd_in, E *__restrict__ dx, int64_t dx_rs,
    float *__restrict__ partial, int64_t rows, int D) {
  constexpr int EV = VecInfo<E>::EV;
  constexpr int Q = EV / 4;
  constexpr int PER_WARP = MAXV * Q * 32;  // float4 entries per warp and accumulator
  extern __shared__ float smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float4 *accw = reinterpret_cast<float4 *>(smem) + (size_t)warp * PER_WARP;
  float4 *accb = reinterpret_cast<float4 *>(smem) + (size_t)(WARPS + warp) * PER_WARP;
#pragma unroll
  for (int i = 0; i < MAXV * Q; ++i) {
    accw[i * 32 + lane] = make_float4(0.f, 0.f, 0.f, 0.f);
    accb[i * 32 + lane] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  RawRow<E, MAXV> wraw, nx, ng;
  wraw.load(w, D, lane);
  const float invD = 1.f / (float)D;
  const int64_t step = (int64_t)gridDim.x * WARPS;
  int64_t row = (int64_t)blockIdx.x * WARPS + warp;
  float nmean = 0.f, nrstd = 0.f;
  if (row < rows) {
    nx.load(x + row * x_rs, D, lane);
    ng.load(dy + row * dy_rs, D, lane);
    nmean = mean_in[row];
    nrstd = rstd_in[row];
  }
  for (; row < rows; row += step) {
    Row<E, MAXV> xr, gr;
    nx.unpack(xr);
    ng.unpack(gr);
    const float mean = nmean, rstd = nrstd;
    if (row + step < rows) {
      nx.load(x + (row + step) * x_rs, D, lane);
      ng.load(dy + (row + step) * dy_rs, D, lane);
      nmean = mean_in[row + step];
      nrstd = rstd_in[row + step];
    }
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const E *pw = reinterpret_cast<const E *>(&wraw.v[k]);
#pragma unroll
      for (int q = 0; q < Q; ++q) {
        float4 aw = accw[(k * Q + q) * 32 + lane], ab = accb[(k * Q + q) * 32 + lane];
        float *paw = reinterpret_cast<float *>(&aw), *pab = reinterpret_cast<float *>(&ab);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int t = q * 4 + c;
          const int e = (k * 32 + lane) * EV + t;
          const float xhat = e < D ? (xr.v[k][t] - mean) * rstd : 0.f;
          const float g = gr.v[k][t];
          paw[c] += g * xhat;
          pab[c] += g;
          const float gw = g * to_f32(pw[t]);
          xr.v[k][t] = xhat;
          gr.v[k][t] = gw;
          c1 += gw * xhat;
          c2 += gw;
        }
        accw[(k * Q + q) * 32 + lane] = aw;
        accb[(k * Q + q) * 32 + lane] = ab;
      }
    }
    c1 = warp_sum(c1) * invD;
    c2 = warp_sum(c2) * invD;
#pragma unroll
    for (int k = 0; k < MAXV; ++k)
#pragma unroll
      for (int t = 0; t < EV; ++t) gr.v[k][t] = (gr.v[k][t] - c2 - xr.v[k][t] * c1) * rstd;
    gr.store(dx + row * dx_rs, D, lane, true);
  }
  __syncthreads();
  float *prow = partial + (int64_t)blockIdx.x * 2 * D;
  for (int i = threadIdx.x; i < 2 * D; i += WARPS * 32) {
    const int which = i >= D ? 1 : 0;
    const int e = i - which * D;
    const int t = e % EV, l = (e / EV) & 31, k = e / (EV * 32);
    const int idx = (((k * Q + t / 4) * 32 + l) << 2) + (t & 3);
    float sum = 0.f;
#pragma unroll
    for (int wv = 0; wv < WARPS; ++wv) sum += smem[(size_t)(which * WARPS + wv) * PER_WARP * 4 + idx];
    prow[i] = sum;
  }
}

// out[which][e] = sum_b partial[b][which][e]   (which in {0,1}).  A CTA takes 32 columns; its
// eight warps split the partial rows (four loads in flight each) and are added up in a fixed
// order, so the result does not depend on timing.
template <typename E>
__global__ void __launch_bounds__(256) reduce_partial_kernel(const float *__restrict__ partial, int nblocks, int D,
                                                             E *__restrict__ out0, E *__restrict__ out1) {
  __shared__ float part[8][33];
  const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
  const int e = blockIdx.x * 32 + lane;
  const int64_t stride = 2 * (int64_t)D;
  float s = 0.f;
  if (e < 2 * D) {
    int b = g;
    for (; b + 24 < nblocks; b += 32) {
      const float v0 = partial[(int64_t)b * stride + e], v1 = partial[(int64_t)(b + 8) * stride + e];
      const float v2 = partial[(int64_t)(b + 16) * stride + e], v3 = partial[(int64_t)(b + 24) * stride + e];
      s += (v0 + v1) + (v2 + v3);
    }
    for (; b < nblocks; b += 8) s += partial[(int64_t)b * stride + e];
  }
  part[g][lane] = s;
  __syncthreads();
  if (g == 0 && e < 2 * D) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += part[i][lane];
    if (e < D) {
      if (out0) out0[e] = from_f32<E>(t);
    } else {
      if (out1) out1[e - D] = from_f32<E>(t);
    }
  }
}

// ---------------------------------------------------------------------------------------
// SiLU gating
// ---------------------------------------------------------------------------------------
template <typename E, bool BWD>
__global__ void __launch_bounds__(256) silu_kernel(const E *__restrict__ dy, int64_t dy_rs, const E *__restrict__ x,
                                                   int64_t x_rs, E *__restrict__ out, int64_t out_rs, int64_t rows,
                                                   int width, bool vec_ok) {
  constexpr int EV = VecInfo<E>::EV;
  constexpr int UNR = 4;  // independent 16-byte vectors in flight per thread
  const int vec_per_row = (width + EV - 1) / EV;
  const int64_t total = rows * vec_per_row;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t base = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; base < total; base += nthreads * UNR) {
    uint4 xraw[UNR], graw[UNR];
    int64_t rowi[UNR];
    int e0[UNR];
    bool fast[UNR];
#pragma unroll
    for (int k = 0; k < UNR; ++k) {
      const int64_t idx = base + k * nthreads;
      fast[k] = false;
      if (idx < total) {
        rowi[k] = idx / vec_per_row;
        e0[k] = (int)(idx - rowi[k] * vec_per_row) * EV;
        fast[k] = vec_ok && e0[k] + EV <= width;
        if (fast[k]) {
          xraw[k] = __ldg(reinterpret_cast<const uint4 *>(x + rowi[k] * x_rs + e0[k]));
          if (BWD) graw[k] = __ldg(reinterpret_cast<const uint4 *>(dy + rowi[k] * dy_rs + e0[k]));
        }
      }
    }
#pragma unroll
    for (int k = 0; k < UNR; ++k) {
      const int64_t idx = base + k * nthreads;
      if (idx >= total) continue;
      E *op = out + rowi[k] * out_rs + e0[k];
      if (fast[k]) {
        const E *xe = reinterpret_cast<const E *>(&xraw[k]);
        const E *ge = reinterpret_cast<const E *>(&graw[k]);
        uint4 oraw;
        E *oe = reinterpret_cast<E *>(&oraw);
#pragma unroll
        for (int t = 0; t < EV; ++t)
          oe[t] = from_f32<E>(BWD ? to_f32(ge[t]) * dsiluf_(to_f32(xe[t])) : siluf_(to_f32(xe[t])));
        *reinterpret_cast<uint4 *>(op) = oraw;
      } else {
        const E *xp = x + rowi[k] * x_rs + e0[k];
        for (int t = 0; t < EV && e0[k] + t < width; ++t) {
          float xv = to_f32(xp[t]);
          op[t] = from_f32<E>(BWD ? to_f32(dy[rowi[k] * dy_rs + e0[k] + t]) * dsiluf_(xv) : siluf_(xv));
        }
      }
    }
  }
}

// Row-shaped variant (one warp per row, next row's vectors prefetched): used when a row fits the
// register budget and everything is 16-byte aligned - the usual case of slicing u out of uvqk.
template <typename E, int MAXV, bool BWD>
__global__ void __launch_bounds__(WARPS * 32) silu_rows_kernel(const E *__restrict__ dy, int64_t dy_rs,
                                                               const E *__restrict__ x, int64_t x_rs,
                                                               E *__restrict__ out, int64_t out_rs, int64_t rows,
                                                               int width) {
  constexpr int EV = VecInfo<E>::EV;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t step = (int64_t)gridDim.x * WARPS;
  int64_t row = (int64_t)blockIdx.x * WARPS + warp;
  RawRow<E, MAXV> nx, ng;
  if (row < rows) {
    nx.load(x + row * x_rs, width, lane);
    if (BWD) ng.load(dy + row * dy_rs, width, lane);
  }
  for (; row < rows; row += step) {
    Row<E, MAXV> xr, gr;
    nx.unpack(xr);
    if (BWD) ng.unpack(gr);
    if (row + step < rows) {
      nx.load(x + (row + step) * x_rs, width, lane);
      if (BWD) ng.load(dy + (row + step) * dy_rs, width, lane);
    }
#pragma unroll
    for (int k = 0; k < MAXV; ++k)
#pragma unroll
      for (int t = 0; t < EV; ++t)
        xr.v[k][t] = BWD ? gr.v[k][t] * dsiluf_(xr.v[k][t]) : siluf_(xr.v[k][t]);
    xr.store(out + row * out_rs, width, lane, true);
  }
}

// ---------------------------------------------------------------------------------------
// y = act(u) * Norm(attn), optional [u | attn | y] concat
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float act_f(float u, int act) {
  return act == 0 ? u : (act == 1 ? sigmoidf_(u) : siluf_(u));
}
__device__ __forceinline__ float dact_f(float u, int act) {
  if (act == 0) return 1.f;
  if (act == 1) {
    float s = sigmoidf_(u);
    return s * (1.f - s);
  }
  return dsiluf_(u);
}

struct NormMulParams {
  const void *attn, *u, *w, *b, *dout;
  void *out, *dattn, *du;
  float *mean, *rstd, *partial;
  int64_t attn_rs, u_rs, out_rs, dout_rs, dattn_rs, du_rs, rows;
  int H, V, concat_u, concat_x, act, group_norm;
  float eps;
  bool vec_ok;
  // dropout over the whole (concatenated) output row, generated in the kernel
  const unsigned long long *drop_seed;  // device; NULL = no dropout
  uint32_t drop_thr;                    // an element is dropped when its 16 random bits are below this
  float drop_scale;                     // 65536 / (65536 - drop_thr)
  // optional: the mask as bits (element idx = bit idx % 8 of byte idx / 8, set = kept), written by the
  // forward and read by the backward instead of running the generator again
  uint8_t *mask;
};

// ---------------------------------------------------------------------------------------
// Dropout mask: counter-based, so that the backward regenerates the forward's mask from the seed
// instead of reading it from memory.  Element idx of the [rows, width] output matrix takes the
// (idx % 8)-th 16-bit piece of Philox4x32-10(key = seed, counter = idx / 8): one generator call
// serves the eight 16-bit elements of a 16-byte vector, and the mask does not depend on the
// element type or on how rows are spread over threads.
// ---------------------------------------------------------------------------------------
struct Dropout {
  uint32_t k0, k1, thr;
  float scale;
  __device__ __forceinline__ void init(const NormMulParams &p) {
    const unsigned long long s = *p.drop_seed;
    k0 = (uint32_t)s;
    k1 = (uint32_t)(s >> 32);
    thr = p.drop_thr;
    scale = p.drop_scale;
  }
  __device__ __forceinline__ float one(float v, uint64_t idx) const {
    uint32_t o[4];
    const uint64_t g = idx >> 3;
    philox4x32_10(k0, k1, (uint32_t)g, (uint32_t)(g >> 32), o);
    const int j = (int)(idx & 7);
    const uint32_t r = (o[j >> 1] >> (16 * (j & 1))) & 0xffffu;
    return r >= thr ? v * scale : 0.f;
  }
  // the D elements of one part of a row, whose first element has index `base` in the output matrix.
  // WHOLE: D is a multiple of the vector width, so that every vector is one aligned group of the
  // generator (no element-wise path in the code at all - it is most of the code otherwise, and these
  // kernels run few enough warps to feel the instruction cache).  STORE (only with WHOLE and 8-element
  // vectors, see norm_mul_mask_bytes): the keep bits of every vector also go to memory, one byte each.
  template <bool WHOLE, bool STORE, typename E, int MAXV>
  __device__ __forceinline__ void apply(Row<E, MAXV> &r, uint64_t base, int D, int lane,
                                        uint8_t *mask_out = nullptr) const {
    constexpr int EV = VecInfo<E>::EV;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int e0 = (k * 32 + lane) * EV;
      if (e0 >= D) continue;
      const uint64_t idx0 = base + (uint64_t)e0;
      if (WHOLE || ((idx0 & (EV - 1)) == 0 && e0 + EV <= D)) {
        uint32_t o[4];
        const uint64_t g = idx0 >> 3;
        philox4x32_10(k0, k1, (uint32_t)g, (uint32_t)(g >> 32), o);
        if constexpr (EV == 8) {
          // two pieces per word: the high one compares in place, the low one after a shift
          const uint32_t thr_hi = thr << 16;
          uint32_t kept = 0;
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const bool lo = (o[w] << 16) >= thr_hi, hi = o[w] >= thr_hi;
            r.v[k][2 * w] = lo ? r.v[k][2 * w] * scale : 0.f;
            r.v[k][2 * w + 1] = hi ? r.v[k][2 * w + 1] * scale : 0.f;
            if (STORE) {
              if (lo) kept |= 1u << (2 * w);
              if (hi) kept |= 2u << (2 * w);
            }
          }
          if (STORE) mask_out[g] = (uint8_t)kept;
        } else {
          const int j0 = (int)(idx0 & 7);   // 0, or 4 for the second half of a group of 32-bit elements
#pragma unroll
          for (int t = 0; t < EV; ++t) {
            const int j = j0 + t;
            const uint32_t rr = (o[(j >> 1) & 3] >> (16 * (j & 1))) & 0xffffu;
            r.v[k][t] = rr >= thr ? r.v[k][t] * scale : 0.f;
          }
        }
      } else {
#pragma unroll
        for (int t = 0; t < EV; ++t)
          if (e0 + t < D) r.v[k][t] = one(r.v[k][t], idx0 + t);
      }
    }
  }
};

// The same from stored bits (whole 8-element vectors only).
template <typename E, int MAXV>
__device__ __forceinline__ void apply_stored_mask(Row<E, MAXV> &r, uint64_t base, int D, int lane, const uint8_t *mask,
                                                  float scale) {
  constexpr int EV = VecInfo<E>::EV;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int e0 = (k * 32 + lane) * EV;
    if (e0 >= D) continue;
    const uint32_t kept = mask[(base + (uint64_t)e0) >> 3];
#pragma unroll
    for (int t = 0; t < EV; ++t) r.v[k][t] = (kept >> t) & 1u ? r.v[k][t] * scale : 0.f;
  }
}

// The same with the bytes of a lane's vectors already in registers.  Each byte stays in a register of
// its own until it is used: any arithmetic on a loaded byte at the point of the load would make the
// warp wait for the load there, which is what prefetching the next row's bytes is meant to avoid.
template <int MAXV>
struct MaskBytes {
  uint32_t b[MAXV];
  __device__ __forceinline__ void load(const uint8_t *mask, uint64_t base, int D, int lane) {
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int e0 = (k * 32 + lane) * 8;
      b[k] = e0 < D ? (uint32_t)__ldg(mask + ((base + (uint64_t)e0) >> 3)) : 0u;
    }
  }
  template <typename E>
  __device__ __forceinline__ void apply(Row<E, MAXV> &r, float scale) const {
#pragma unroll
    for (int k = 0; k < MAXV; ++k)
#pragma unroll
      for (int t = 0; t < VecInfo<E>::EV; ++t) r.v[k][t] = (b[k] >> t) & 1u ? r.v[k][t] * scale : 0.f;
  }
};

// LayerNorm flavour: one warp per row of D = H * V elements.  With dropout the generator's ten
// dependent rounds make the kernel latency-bound; rows of up to two vectors per lane are compiled
// for two resident CTAs (128 registers instead of 158: 3.1 instead of 2.3 TB/s at D = 512; without
// dropout 128 instead of 161: 6.2 instead of 5.4 TB/s), wider rows would spill and are left to the
// compiler's own choice (0 = no minimum).
// DROPOUT: 0 = none, 1 = any row width, 2 = rows of whole vectors, 3 = the same and the mask bits stored
template <typename E, int MAXV, int DROPOUT>
__global__ void __launch_bounds__(WARPS * 32, MAXV <= 2 ? 2 : 0) norm_mul_fwd_kernel(NormMulParams p) {
  constexpr bool WHOLE = DROPOUT >= 2, STORE = DROPOUT == 3 && VecInfo<E>::EV == 8;
  constexpr int EV = VecInfo<E>::EV;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int D = p.H * p.V;
  Dropout drop;
  if (DROPOUT) drop.init(p);
  const int width = D * (1 + (p.concat_u ? 1 : 0) + (p.concat_x ? 1 : 0));
  Row<E, MAXV> wr, br;
  wr.load((const E *)p.w, D, lane, p.vec_ok);
  br.load((const E *)p.b, D, lane, p.vec_ok);
  const int64_t step = (int64_t)gridDim.x * WARPS;
  int64_t row = (int64_t)blockIdx.x * WARPS + warp;
  constexpr bool PF = MAXV <= 4;
  const bool pf = PF && p.vec_ok;
  RawRow<E, PF ? MAXV : 1> nx, nu;
  if constexpr (PF) {
    if (pf && row < p.rows) {
      nx.load((const E *)p.attn + row * p.attn_rs, D, lane);
      nu.load((const E *)p.u + row * p.u_rs, D, lane);
    }
  }
  for (; row < p.rows; row += step) {
    Row<E, MAXV> xr, ur;
    bool loaded = false;
    if constexpr (PF) {
      if (pf) {
        nx.unpack(xr);
        nu.unpack(ur);
        if (row + step < p.rows) {
          nx.load((const E *)p.attn + (row + step) * p.attn_rs, D, lane);
          nu.load((const E *)p.u + (row + step) * p.u_rs, D, lane);
        }
        loaded = true;
      }
    }
    if (!loaded) {
      xr.load((const E *)p.attn + row * p.attn_rs, D, lane, p.vec_ok);
      ur.load((const E *)p.u + row * p.u_rs, D, lane, p.vec_ok);
    }
    float mean, rstd;
    row_stats(xr, D, lane, p.eps, mean, rstd);
    E *orow = (E *)p.out + row * p.out_rs;
    const uint64_t rbase = (uint64_t)row * (uint64_t)width;   // index of the row's first element
    int off = 0;
    if (p.concat_u) {
      if (DROPOUT) {
        Row<E, MAXV> du_ = ur;
        drop.template apply<WHOLE, STORE>(du_, rbase, D, lane, p.mask);
        du_.store(orow, D, lane, p.vec_ok);
      } else {
        ur.store(orow, D, lane, p.vec_ok);
      }
      off += D;
    }
    if (p.concat_x) {
      if (DROPOUT) {
        Row<E, MAXV> dx_ = xr;
        drop.template apply<WHOLE, STORE>(dx_, rbase + off, D, lane, p.mask);
        dx_.store(orow + off, D, lane, p.vec_ok);
      } else {
        xr.store(orow + off, D, lane, p.vec_ok);
      }
      off += D;
    }
#pragma unroll
    for (int k = 0; k < MAXV; ++k)
#pragma unroll
      for (int t = 0; t < EV; ++t)
        xr.v[k][t] = act_f(ur.v[k][t], p.act) * ((xr.v[k][t] - mean) * rstd * wr.v[k][t] + br.v[k][t]);
    if (DROPOUT) drop.template apply<WHOLE, STORE>(xr, rbase + off, D, lane, p.mask);
    xr.store(orow + off, D, lane, p.vec_ok);
    if (lane == 0) {
      if (p.mean) p.mean[row] = mean;
      if (p.rstd) p.rstd[row] = rstd;
    }
  }
}

// The same forward for rows of eight vectors per lane (D = 2048 in 16-bit elements), which do not fit
// the registers as fp32 values next to a prefetched row: the row and the next one stay packed (raw
// 16-byte vectors) and are unpacked vector by vector - twice for the statistics, once for the
// output -, weight and bias are read where they are used (they stay in L1).  Vector path only
// (aligned pointers and strides, D a multiple of the vector width).  DROPOUT: 0 = none, 2 = on.
// Also used for rows of four vectors per lane with dropout, where this form needs 128 registers (two
// resident CTAs) against the 254 of the register-resident kernel: 3.5 instead of 2.8 TB/s at D = 1024.
template <typename E, int MAXV, int DROPOUT>
__global__ void __launch_bounds__(WARPS * 32, MAXV <= 4 ? 2 : 1) norm_mul_fwd_packed_kernel(NormMulParams p) {
  constexpr int EV = VecInfo<E>::EV;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int D = p.H * p.V;
  Dropout drop;
  if (DROPOUT) drop.init(p);
  const int width = D * (1 + (p.concat_u ? 1 : 0) + (p.concat_x ? 1 : 0));
  const float invD = 1.f / (float)D;
  const int64_t step = (int64_t)gridDim.x * WARPS;
  int64_t row = (int64_t)blockIdx.x * WARPS + warp;
  RawRow<E, MAXV> nx, nu;
  if (row < p.rows) {
    nx.load((const E *)p.attn + row * p.attn_rs, D, lane);
    nu.load((const E *)p.u + row * p.u_rs, D, lane);
  }
  for (; row < p.rows; row += step) {
    const RawRow<E, MAXV> cx = nx, cu = nu;
    if (row + step < p.rows) {
      nx.load((const E *)p.attn + (row + step) * p.attn_rs, D, lane);
      nu.load((const E *)p.u + (row + step) * p.u_rs, D, lane);
    }
    // statistics as in row_stats(): mean first, then the centred second moment
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const E *px = reinterpret_cast<const E *>(&cx.v[k]);
#pragma unroll
      for (int t = 0; t < EV; ++t) sum += to_f32(px[t]);   // vectors beyond the row hold zeros
    }
    const float mean = warp_sum(sum) * invD;
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const E *px = reinterpret_cast<const E *>(&cx.v[k]);
      const bool in = (k * 32 + lane) * EV < D;
#pragma unroll
      for (int t = 0; t < EV; ++t) {
        const float d = in ? to_f32(px[t]) - mean : 0.f;
        q += d * d;
      }
    }
    const float rstd = rsqrtf(warp_sum(q) * invD + p.eps);
    E *orow = (E *)p.out + row * p.out_rs;
    const uint64_t rbase = (uint64_t)row * (uint64_t)width;
    const int off_x = p.concat_u ? D : 0;
    const int off_y = off_x + (p.concat_x ? D : 0);
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int e0 = (k * 32 + lane) * EV;
      if (e0 >= D) continue;
      Row<E, 1> fx, fu, fy;
      const E *px = reinterpret_cast<const E *>(&cx.v[k]), *pu = reinterpret_cast<const E *>(&cu.v[k]);
      const uint4 wraw = __ldg(reinterpret_cast<const uint4 *>((const E *)p.w + e0));
      const uint4 braw = __ldg(reinterpret_cast<const uint4 *>((const E *)p.b + e0));
      const E *pw = reinterpret_cast<const E *>(&wraw), *pb = reinterpret_cast<const E *>(&braw);
#pragma unroll
      for (int t = 0; t < EV; ++t) {
        fx.v[0][t] = to_f32(px[t]);
        fu.v[0][t] = to_f32(pu[t]);
        fy.v[0][t] = act_f(fu.v[0][t], p.act) * ((fx.v[0][t] - mean) * rstd * to_f32(pw[t]) + to_f32(pb[t]));
      }
      // (Row<E, 1> places its one vector at lane * EV: the pointers below are shifted to vector k)
      if (p.concat_u) {
        if (DROPOUT) {
          drop.template apply<true, false>(fu, rbase + (uint64_t)(k * 32 * EV), D - k * 32 * EV, lane);
          fu.store(orow + k * 32 * EV, D - k * 32 * EV, lane, true);
        } else {
          *reinterpret_cast<uint4 *>(orow + e0) = cu.v[k];
        }
      }
      if (p.concat_x) {
        if (DROPOUT) {
          drop.template apply<true, false>(fx, rbase + (uint64_t)(off_x + k * 32 * EV), D - k * 32 * EV, lane);
          fx.store(orow + off_x + k * 32 * EV, D - k * 32 * EV, lane, true);
        } else {
          *reinterpret_cast<uint4 *>(orow + off_x + e0) = cx.v[k];
        }
      }
      if (DROPOUT) drop.template apply<true, false>(fy, rbase + (uint64_t)(off_y + k * 32 * EV), D - k * 32 * EV, lane);
      fy.store(orow + off_y + k * 32 * EV, D - k * 32 * EV, lane, true);
    }
    if (lane == 0) {
      if (p.mean) p.mean[row] = mean;
      if (p.rstd) p.rstd[row] = rstd;
    }
  }
}

// DROPOUT: 0 = none, 1 = the forward's mask regenerated from the seed, 2 = read from p.mask,
// 3 = regenerated, rows of whole vectors
template <typename E, int MAXV, int DROPOUT>
__global__ void __launch_bounds__(WARPS * 32) norm_mul_bwd_kernel(NormMulParams p) {
  constexpr int EV = VecInfo<E>::EV;
  constexpr bool REGEN = DROPOUT == 1 || DROPOUT == 3, WHOLE = DROPOUT == 3;
  extern __shared__ float smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int D = p.H * p.V;
  Dropout drop;
  if (REGEN) drop.init(p);
  const int width = D * (1 + (p.concat_u ? 1 : 0) + (p.concat_x ? 1 : 0));
  Row<E, MAXV> wr, br, dw, db;
  wr.load((const E *)p.w, D, lane, p.vec_ok);
  br.load((const E *)p.b, D, lane, p.vec_ok);
  dw.zero();
  db.zero();
  const float invD = 1.f / (float)D;
  const int off_x = p.concat_u ? D : 0;
  const int off_y = off_x + (p.concat_x ? D : 0);
  const int64_t step = (int64_t)gridDim.x * WARPS;
  int64_t row = (int64_t)blockIdx.x * WARPS + warp;
  constexpr bool PF = MAXV <= 2;
  const bool pf = PF && p.vec_ok;
  constexpr int RV = PF ? MAXV : 1;
  RawRow<E, RV> nx, nu, ngy, ngu, ngx;
  float nmean = 0.f, nrstd = 0.f;
  MaskBytes<RV> nmy, nmu, nmx;  // stored mask bytes of the prefetched row's parts (a dependent load otherwise)
  auto prefetch = [&](int64_t r) {
    if constexpr (PF) {
      const E *grow = (const E *)p.dout + r * p.dout_rs;
      if constexpr (DROPOUT == 2) {
        const uint64_t rb = (uint64_t)r * (uint64_t)width;
        nmy.load(p.mask, rb + off_y, D, lane);
        if (p.concat_u) nmu.load(p.mask, rb, D, lane);
        if (p.concat_x) nmx.load(p.mask, rb + off_x, D, lane);
      }
      nx.load((const E *)p.attn + r * p.attn_rs, D, lane);
      nu.load((const E *)p.u + r * p.u_rs, D, lane);
      ngy.load(grow + off_y, D, lane);
      if (p.concat_u) ngu.load(grow, D, lane);
      if (p.concat_x) ngx.load(grow + off_x, D, lane);
      nmean = p.mean[r];
      nrstd = p.rstd[r];
    }
  };
  if (pf && row < p.rows) prefetch(row);
  for (; row < p.rows; row += step) {
    Row<E, MAXV> xr, ur, gy, tmp;
    RawRow<E, RV> cgu, cgx;  // this row's concat gradients (the prefetch buffers get overwritten below)
    float mean, rstd;
    MaskBytes<RV> cmy, cmu, cmx;
    const E *grow = (const E *)p.dout + row * p.dout_rs;
    bool loaded = false;
    if constexpr (PF) {
      if (pf) {
        if constexpr (DROPOUT == 2) cmy = nmy, cmu = nmu, cmx = nmx;
        nx.unpack(xr);
        nu.unpack(ur);
        ngy.unpack(gy);
        cgu = ngu;
        cgx = ngx;
        mean = nmean;
        rstd = nrstd;
        if (row + step < p.rows) prefetch(row + step);
        loaded = true;
      }
    }
    if (!loaded) {
      xr.load((const E *)p.attn + row * p.attn_rs, D, lane, p.vec_ok);
      ur.load((const E *)p.u + row * p.u_rs, D, lane, p.vec_ok);
      gy.load(grow + off_y, D, lane, p.vec_ok);
      mean = p.mean[row];
      rstd = p.rstd[row];
    }
    // the forward's mask, regenerated: the gradient of a dropped element is zero, of a kept one scaled
    const uint64_t rbase = (uint64_t)row * (uint64_t)width;
    if (REGEN) drop.template apply<WHOLE, false>(gy, rbase + off_y, D, lane);
    if constexpr (DROPOUT == 2) {
      if (PF && loaded) { if constexpr (PF) cmy.apply(gy, p.drop_scale); }
      else apply_stored_mask(gy, rbase + off_y, D, lane, p.mask, p.drop_scale);
    }
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int k = 0; k < MAXV; ++k)
#pragma unroll
      for (int t = 0; t < EV; ++t) {
        int e = (k * 32 + lane) * EV + t;
        float xhat = e < D ? (xr.v[k][t] - mean) * rstd : 0.f;
        float ln = xhat * wr.v[k][t] + br.v[k][t];
        float uu = ur.v[k][t];
        float g = gy.v[k][t];
        float ga = g * act_f(uu, p.act);  // gradient w.r.t. the normalised value
        ur.v[k][t] = g * ln * dact_f(uu, p.act);  // du (y part)
        dw.v[k][t] += ga * xhat;
        db.v[k][t] += ga;
        float gw = ga * wr.v[k][t];
        xr.v[k][t] = xhat;
        gy.v[k][t] = gw;
        c1 += gw * xhat;
        c2 += gw;
      }
    c1 = warp_sum(c1) * invD;
    c2 = warp_sum(c2) * invD;
#pragma unroll
    for (int k = 0; k < MAXV; ++k)
#pragma unroll
      for (int t = 0; t < EV; ++t) gy.v[k][t] = (gy.v[k][t] - c2 - xr.v[k][t] * c1) * rstd;
    if (p.concat_u) {
      if (loaded) {
        if constexpr (PF) cgu.unpack(tmp);
      } else {
        tmp.load(grow, D, lane, p.vec_ok);
      }
      if (REGEN) drop.template apply<WHOLE, false>(tmp, rbase, D, lane);
      if constexpr (DROPOUT == 2) {
        if (PF && loaded) { if constexpr (PF) cmu.apply(tmp, p.drop_scale); }
        else apply_stored_mask(tmp, rbase, D, lane, p.mask, p.drop_scale);
      }
#pragma unroll
      for (int k = 0; k < MAXV; ++k)
#pragma unroll
        for (int t = 0; t < EV; ++t) ur.v[k][t] += tmp.v[k][t];
    }
    if (p.concat_x) {
      if (loaded) {
        if constexpr (PF) cgx.unpack(tmp);
      } else {
        tmp.load(grow + off_x, D, lane, p.vec_ok);
      }
      if (REGEN) drop.template apply<WHOLE, false>(tmp, rbase + off_x, D, lane);
      if constexpr (DROPOUT == 2) {
        if (PF && loaded) { if constexpr (PF) cmx.apply(tmp, p.drop_scale); }
        else apply_stored_mask(tmp, rbase + off_x, D, lane, p.mask, p.drop_scale);
      }
#pragma unroll
      for (int k = 0; k < MAXV; ++k)
#pragma unroll
        for (int t = 0; t < EV; ++t) gy.v[k][t] += tmp.v[k][t];
    }
    ur.store((E *)p.du + row * p.du_rs, D, lane, p.vec_ok);
    gy.store((E *)p.dattn + row * p.dattn_rs, D, lane, p.vec_ok);
  }
  float *prow = p.partial + (int64_t)blockIdx.x * 2 * D;
  reduce_columns_to_partial(dw, smem, prow, D, lane, warp);
  reduce_columns_to_partial(db, smem, prow + D, D, lane, warp);
}

// The same backward for rows of four vectors per lane (D = 1024 in 16-bit elements), which the kernel
// above can only run without its prefetch and at the edge of spilling: the column accumulators
// (dweight, dbias) of every warp live in shared memory, weight and bias are read from a packed copy
// in shared memory, and the registers so freed hold the next row's five raw inputs.  Vector path only
// (aligned pointers and strides, D a multiple of the vector width).  DROPOUT: 0 = none, 3 = the
// forward's mask regenerated from the seed.
// Shared memory: [2][WARPS][MAXV * EV / 4][32] float4 accumulators, then weight and bias as
// [2][MAXV * 32] 16-byte vectors.
template <typename E, int MAXV, int DROPOUT>
__global__ void __launch_bounds__(WARPS * 32) norm_mul_bwd_wide_kernel(NormMulParams p) {
  constexpr int EV = VecInfo<E>::EV;
  constexpr int Q = EV / 4;
  constexpr int PER_WARP = MAXV * Q * 32;  // float4 entries per warp and accumulator
  constexpr bool REGEN = DROPOUT == 3;
  extern __shared__ float smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int D = p.H * p.V;
  float4 *accw = reinterpret_cast<float4 *>(smem) + (size_t)warp * PER_WARP;
  float4 *accb = reinterpret_cast<float4 *>(smem) + (size_t)(WARPS + warp) * PER_WARP;
  uint4 *wb = reinterpret_cast<uint4 *>(reinterpret_cast<float4 *>(smem) + (size_t)2 * WARPS * PER_WARP);
#pragma unroll
  for (int i = 0; i < MAXV * Q; ++i) {
    accw[i * 32 + lane] = make_float4(0.f, 0.f, 0.f, 0.f);
    accb[i * 32 + lane] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int i = threadIdx.x; i < MAXV * 32; i += WARPS * 32) {
    const bool in = (i + 1) * EV <= D;
    wb[i] = in ? __ldg(reinterpret_cast<const uint4 *>((const E *)p.w + (size_t)i * EV)) : make_uint4(0, 0, 0, 0);
    wb[MAXV * 32 + i] = in ? __ldg(reinterpret_cast<const uint4 *>((const E *)p.b + (size_t)i * EV)) : make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  Dropout drop;
  if (REGEN) drop.init(p);
  const int width = D * (1 + (p.concat_u ? 1 : 0) + (p.concat_x ? 1 : 0));
  const float invD = 1.f / (float)D;
  const int off_x = p.concat_u ? D : 0;
  const int off_y = off_x + (p.concat_x ? D : 0);
  const int64_t step = (int64_t)gridDim.x * WARPS;
  int64_t row = (int64_t)blockIdx.x * WARPS + warp;
  RawRow<E, MAXV> nx, nu, ngy, ngu, ngx;
  float nmean = 0.f, nrstd = 0.f;
  auto prefetch = [&](int64_t r) {
    const E *grow = (const E *)p.dout + r * p.dout_rs;
    nx.load((const E *)p.attn + r * p.attn_rs, D, lane);
    nu.load((const E *)p.u + r * p.u_rs, D, lane);
    ngy.load(grow + off_y, D, lane);
    if (p.concat_u) ngu.load(grow, D, lane);
    if (p.concat_x) ngx.load(grow + off_x, D, lane);
    nmean = p.mean[r];
    nrstd = p.rstd[r];
  };
  if (row < p.rows) prefetch(row);
  for (; row < p.rows; row += step) {
    Row<E, MAXV> xr, ur, gy;
    nx.unpack(xr);
    nu.unpack(ur);
    ngy.unpack(gy);
    const RawRow<E, MAXV> cgu = ngu, cgx = ngx;  // this row's concat gradients (the prefetch overwrites the buffers)
    const float mean = nmean, rstd = nrstd;
    if (row + step < p.rows) prefetch(row + step);
    const uint64_t rbase = (uint64_t)row * (uint64_t)width;
    if (REGEN) drop.template apply<true, false>(gy, rbase + off_y, D, lane);
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const uint4 wraw = wb[k * 32 + lane], braw = wb[MAXV * 32 + k * 32 + lane];
      const E *pw = reinterpret_cast<const E *>(&wraw), *pb = reinterpret_cast<const E *>(&braw);
#pragma unroll
      for (int q = 0; q < Q; ++q) {
        float4 aw = accw[(k * Q + q) * 32 + lane], ab = accb[(k * Q + q) * 32 + lane];
        float *paw = reinterpret_cast<float *>(&aw), *pab = reinterpret_cast<float *>(&ab);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int t = q * 4 + c;
          const int e = (k * 32 + lane) * EV + t;
          const float w_ = to_f32(pw[t]);
          const float xhat = e < D ? (xr.v[k][t] - mean) * rstd : 0.f;
          const float ln = xhat * w_ + to_f32(pb[t]);
          const float uu = ur.v[k][t];
          const float g = gy.v[k][t];
          const float ga = g * act_f(uu, p.act);      // gradient w.r.t. the normalised value
          ur.v[k][t] = g * ln * dact_f(uu, p.act);    // du (y part)
          paw[c] += ga * xhat;
          pab[c] += ga;
          const float gw = ga * w_;
          xr.v[k][t] = xhat;
          gy.v[k][t] = gw;
          c1 += gw * xhat;
          c2 += gw;
        }
        accw[(k * Q + q) * 32 + lane] = aw;
        accb[(k * Q + q) * 32 + lane] = ab;
      }
    }
    c1 = warp_sum(c1) * invD;
    c2 = warp_sum(c2) * invD;
#pragma unroll
    for (int k = 0; k < MAXV; ++k)
#pragma unroll
      for (int t = 0; t < EV; ++t) gy.v[k][t] = (gy.v[k][t] - c2 - xr.v[k][t] * c1) * rstd;
    if (p.concat_u) {
      cgu.unpack(xr);   // (the normalised row is no longer needed)
      if (REGEN) drop.template apply<true, false>(xr, rbase, D, lane);
#pragma unroll
      for (int k = 0; k < MAXV; ++k)
#pragma unroll
        for (int t = 0; t < EV; ++t) ur.v[k][t] += xr.v[k][t];
    }
    if (p.concat_x) {
      cgx.unpack(xr);
      if (REGEN) drop.template apply<true, false>(xr, rbase + off_x, D, lane);
#pragma unroll
      for (int k = 0; k < MAXV; ++k)
#pragma unroll
        for (int t = 0; t < EV; ++t) gy.v[k][t] += xr.v[k][t];
    }
    ur.store((E *)p.du + row * p.du_rs, D, lane, true);
    gy.store((E *)p.dattn + row * p.dattn_rs, D, lane, true);
  }
  __syncthreads();
  float *prow = p.partial + (int64_t)blockIdx.x * 2 * D;
  for (int i = threadIdx.x; i < 2 * D; i += WARPS * 32) {
    const int which = i >= D ? 1 : 0;
    const int e = i - which * D;
    const int t = e % EV, l = (e / EV) & 31, k = e / (EV * 32);
    const int idx = (((k * Q + t / 4) * 32 + l) << 2) + (t & 3);
    float sum = 0.f;
#pragma unroll
    for (int wv = 0; wv < WARPS; ++wv) sum += smem[(size_t)(which * WARPS + wv) * PER_WARP * 4 + idx];
    prow[i] = sum;
  }
}

// Group-norm flavour (statistics per head; weight / bias are per-head scalars): one warp per
// (row, head), scalar loads.  Used by the `group_norm=True` variant of the output stage only.
template <typename E, bool BWD>
__global__ void __launch_bounds__(WARPS * 32) group_norm_mul_kernel(NormMulParams p) {
  extern __shared__ float smem[];  // BWD: [WARPS][2][H]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int H = p.H, V = p.V, D = H * V;
  const int off_x = p.concat_u ? D : 0;
  const int off_y = off_x + (p.concat_x ? D : 0);
  if (BWD) {
    for (int i = threadIdx.x; i < WARPS * 2 * H; i += WARPS * 32) smem[i] = 0.f;
    __syncthreads();
  }
  const int64_t items = p.rows * H;
  for (int64_t it = (int64_t)blockIdx.x * WARPS + warp; it < items; it += (int64_t)gridDim.x * WARPS) {
    const int64_t row = it / H;
    const int h = (int)(it - row * H);
    const E *xa = (const E *)p.attn + row * p.attn_rs + h * V;
    const E *ua = (const E *)p.u + row * p.u_rs + h * V;
    const float wv = to_f32(((const E *)p.w)[h]), bv = to_f32(((const E *)p.b)[h]);
    float mean, rstd;
    if (!BWD) {
      float s = 0.f;
      for (int e = lane; e < V; e += 32) s += to_f32(xa[e]);
      mean = warp_sum(s) / (float)V;
      float q = 0.f;
      for (int e = lane; e < V; e += 32) {
        float d = to_f32(xa[e]) - mean;
        q += d * d;
      }
      rstd = rsqrtf(warp_sum(q) / (float)V + p.eps);
      E *orow = (E *)p.out + row * p.out_rs + h * V;
      for (int e = lane; e < V; e += 32) {
        float xv = to_f32(xa[e]), uv = to_f32(ua[e]);
        // the group-norm branch multiplies by u itself (no activation) and concatenates only
        // when both flags are set (pt_hstu_linear.py:42-54)
        if (p.concat_u && p.concat_x) {
          orow[e] = from_f32<E>(uv);
          orow[D + e] = from_f32<E>(xv);
        }
        orow[off_y + e] = from_f32<E>(uv * ((xv - mean) * rstd * wv + bv));
      }
      if (lane == 0) {
        if (p.mean) p.mean[it] = mean;
        if (p.rstd) p.rstd[it] = rstd;
      }
    } else {
      mean = p.mean[it];
      rstd = p.rstd[it];
      const E *grow = (const E *)p.dout + row * p.dout_rs + h * V;
      float c1 = 0.f, c2 = 0.f, aw = 0.f, ab = 0.f;
      for (int e = lane; e < V; e += 32) {
        float xhat = (to_f32(xa[e]) - mean) * rstd;
        float ga = to_f32(grow[off_y + e]) * to_f32(ua[e]);
        aw += ga * xhat;
        ab += ga;
        c1 += ga * wv * xhat;
        c2 += ga * wv;
      }
      c1 = warp_sum(c1) / (float)V;
      c2 = warp_sum(c2) / (float)V;
      aw = warp_sum(aw);
      ab = warp_sum(ab);
      if (lane == 0) {
        smem[(warp * 2 + 0) * H + h] += aw;
        smem[(warp * 2 + 1) * H + h] += ab;
      }
      E *dxa = (E *)p.dattn + row * p.dattn_rs + h * V;
      E *dua = (E *)p.du + row * p.du_rs + h * V;
      for (int e = lane; e < V; e += 32) {
        float xhat = (to_f32(xa[e]) - mean) * rstd;
        float g = to_f32(grow[off_y + e]);
        float gw = g * to_f32(ua[e]) * wv;
        float dxv = (gw - c2 - xhat * c1) * rstd;
        float duv = g * (xhat * wv + bv);
        if (p.concat_u && p.concat_x) {
          duv += to_f32(grow[e]);
          dxv += to_f32(grow[D + e]);
        }
        dxa[e] = from_f32<E>(dxv);
        dua[e] = from_f32<E>(duv);
      }
    }
  }
  if (BWD) {
    __syncthreads();
    float *prow = p.partial + (int64_t)blockIdx.x * 2 * H;
    for (int i = threadIdx.x; i < 2 * H; i += WARPS * 32) {
      float s = 0.f;
      for (int wv = 0; wv < WARPS; ++wv) s += smem[wv * 2 * H + i];
      prow[i] = s;
    }
  }
}

int g_num_sms = 0;
int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

constexpr int BWD_BLOCKS_PER_SM = 3;
int bwd_blocks() { return num_sms() * BWD_BLOCKS_PER_SM; }
constexpr int MAX_BWD_BLOCKS = 512;  // workspace is sized for this many partial rows

template <typename E>
int max_row_elems() { return 32 * 8 * VecInfo<E>::EV; }

template <typename E>
int pick_maxv(int D) {
  int nvec = (D + VecInfo<E>::EV - 1) / VecInfo<E>::EV;
  int per_lane = (nvec + 31) / 32;
  return per_lane <= 1 ? 1 : per_lane <= 2 ? 2 : per_lane <= 4 ? 4 : 8;
}

#define DISPATCH_MAXV(maxv, ...)          \
  switch (maxv) {                         \
    case 1: { constexpr int MV = 1; __VA_ARGS__; } break; \
    case 2: { constexpr int MV = 2; __VA_ARGS__; } break; \
    case 4: { constexpr int MV = 4; __VA_ARGS__; } break; \
    default: { constexpr int MV = 8; __VA_ARGS__; } break; \
  }

template <typename E>
int ln_fwd_t(const void *x, int64_t x_rs, const void *w, const void *b, void *y, int64_t y_rs, float *mean,
             float *rstd, int64_t rows, int D, float eps, cudaStream_t st) {
  constexpr int EV = VecInfo<E>::EV;
  if (D > max_row_elems<E>()) return fail(B200_HSTU_EUNSUPPORTED, "layer_norm: D=%d exceeds %d", D, max_row_elems<E>());
  bool vec_ok = aligned16(x) && aligned16(y) && aligned16(w) && aligned16(b) && x_rs % EV == 0 && y_rs % EV == 0;
  int64_t nblk = (rows + WARPS - 1) / WARPS;
  int grid = (int)(nblk < (int64_t)num_sms() * 8 ? nblk : (int64_t)num_sms() * 8);
  if (grid == 0) return 0;
  ProfileScope prof(PROF_LN_FWD, st);
  DISPATCH_MAXV(pick_maxv<E>(D), (layer_norm_fwd_kernel<E, MV><<<grid, WARPS * 32, 0, st>>>(
                                     (const E *)x, x_rs, (const E *)w, (const E *)b, (E *)y, y_rs, mean, rstd,
                                     rows, D, eps, vec_ok)));
  count_launch();
  B200_CHECK_LAUNCH("layer_norm forward");
  return 0;
}

template <typename E>
int ln_bwd_t(const void *dy, int64_t dy_rs, const void *x, int64_t x_rs, const void *w, const float *mean,
             const float *rstd, void *dx, int64_t dx_rs, void *dw, void *db, void *partial, int64_t partial_bytes,
             int64_t rows, int D, cudaStream_t st) {
  constexpr int EV = VecInfo<E>::EV;
  if (D > max_row_elems<E>()) return fail(B200_HSTU_EUNSUPPORTED, "layer_norm: D=%d exceeds %d", D, max_row_elems<E>());
  int grid = bwd_blocks();
  if (grid > MAX_BWD_BLOCKS) grid = MAX_BWD_BLOCKS;
  if ((int64_t)grid * 2 * D * (int64_t)sizeof(float) > partial_bytes)
    return fail(B200_HSTU_EWORKSPACE, "layer_norm backward: scratch of %lld bytes is too small",
                (long long)partial_bytes);
  bool vec_ok = aligned16(x) && aligned16(dy) && aligned16(dx) && aligned16(w) && x_rs % EV == 0 &&
                dy_rs % EV == 0 && dx_rs % EV == 0;
  size_t smem = (size_t)WARPS * D * sizeof(float);
  ProfileScope prof(PROF_LN_BWD, st);
  const int maxv = pick_maxv<E>(D);
  if (vec_ok && D % EV == 0) {
    // accumulators in shared memory, three (two for four vectors per lane) resident CTAs
    const size_t acc_bytes = (size_t)2 * WARPS * maxv * (EV / 4) * 32 * sizeof(float4);
    if (maxv == 1) {
      layer_norm_bwd_smem_kernel<E, 1><<<grid, WARPS * 32, acc_bytes, st>>>(
          (const E *)dy, dy_rs, (const E *)x, x_rs, (const E *)w, mean, rstd, (E *)dx, dx_rs, (float *)partial, rows, D);
    } else if (maxv == 2) {
      layer_norm_bwd_smem_kernel<E, 2><<<grid, WARPS * 32, acc_bytes, st>>>(
          (const E *)dy, dy_rs, (const E *)x, x_rs, (const E *)w, mean, rstd, (E *)dx, dx_rs, (float *)partial, rows, D);
    } else {
      auto kern = maxv == 4 ? layer_norm_bwd_smem_kernel<E, 4> : layer_norm_bwd_smem_kernel<E, 8>;
      grid = num_sms() * (maxv == 4 ? 2 : 1);   // two / one resident CTAs: one wave of the grid-stride loop
      if (acc_bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)acc_bytes);
        if (e != cudaSuccess) return check_cuda(e, "layer_norm backward smem attribute");
      }
      kern<<<grid, WARPS * 32, acc_bytes, st>>>((const E *)dy, dy_rs, (const E *)x, x_rs, (const E *)w, mean, rstd,
                                                (E *)dx, dx_rs, (float *)partial, rows, D);
    }
    count_launch();
    B200_CHECK_LAUNCH("layer_norm backward");
    reduce_partial_kernel<E><<<(2 * D + 31) / 32, 256, 0, st>>>((const float *)partial, grid, D, (E *)dw, (E *)db);
    count_launch();
    B200_CHECK_LAUNCH("layer_norm backward (reduce)");
    return 0;
  }
  DISPATCH_MAXV(pick_maxv<E>(D), {
    auto kern = layer_norm_bwd_kernel<E, MV>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<grid, WARPS * 32, smem, st>>>((const E *)dy, dy_rs, (const E *)x, x_rs, (const E *)w, mean, rstd,
                                         (E *)dx, dx_rs, (float *)partial, rows, D, vec_ok);
  });
  count_launch();
  B200_CHECK_LAUNCH("layer_norm backward");
  reduce_partial_kernel<E><<<(2 * D + 31) / 32, 256, 0, st>>>((const float *)partial, grid, D, (E *)dw, (E *)db);
  count_launch();
  B200_CHECK_LAUNCH("layer_norm backward (reduce)");
  return 0;
}

template <typename E>
int silu_t(const void *dy, int64_t dy_rs, const void *x, int64_t x_rs, void *out, int64_t out_rs, int64_t rows,
           int width, bool bwd, cudaStream_t st) {
  constexpr int EV = VecInfo<E>::EV;
  bool vec_ok = aligned16(x) && aligned16(out) && x_rs % EV == 0 && out_rs % EV == 0 &&
                (!bwd || (aligned16(dy) && dy_rs % EV == 0));
  int64_t total = rows * ((width + EV - 1) / EV);
  if (total == 0) return 0;
  if (vec_ok && width % EV == 0 && width <= 32 * 4 * EV) {
    int64_t nblk = (rows + WARPS - 1) / WARPS;
    int grid = (int)(nblk < (int64_t)num_sms() * 8 ? nblk : (int64_t)num_sms() * 8);
    ProfileScope prof(PROF_SILU, st);
    int maxv = pick_maxv<E>(width);
    if (bwd) {
      DISPATCH_MAXV(maxv, (silu_rows_kernel<E, (MV > 4 ? 4 : MV), true><<<grid, WARPS * 32, 0, st>>>(
                              (const E *)dy, dy_rs, (const E *)x, x_rs, (E *)out, out_rs, rows, width)));
    } else {
      DISPATCH_MAXV(maxv, (silu_rows_kernel<E, (MV > 4 ? 4 : MV), false><<<grid, WARPS * 32, 0, st>>>(
                              nullptr, 0, (const E *)x, x_rs, (E *)out, out_rs, rows, width)));
    }
    count_launch();
    B200_CHECK_LAUNCH("silu (rows)");
    return 0;
  }
  int64_t nblk = (total + 256 * 4 - 1) / (256 * 4);
  int grid = (int)(nblk < (int64_t)num_sms() * 8 ? nblk : (int64_t)num_sms() * 8);
  if (grid < 1) grid = 1;
  ProfileScope prof(PROF_SILU, st);
  if (bwd)
    silu_kernel<E, true><<<grid, 256, 0, st>>>((const E *)dy, dy_rs, (const E *)x, x_rs, (E *)out, out_rs, rows,
                                               width, vec_ok);
  else
    silu_kernel<E, false><<<grid, 256, 0, st>>>(nullptr, 0, (const E *)x, x_rs, (E *)out, out_rs, rows, width,
                                                vec_ok);
  count_launch();
  B200_CHECK_LAUNCH("silu");
  return 0;
}

// Bytes of the optional dropout mask of these arguments: one bit per element of the [rows, width]
// output, or 0 where it cannot be used (group norm, 32-bit elements, rows that are not made of whole
// aligned 8-element vectors).
int64_t norm_mul_mask_bytes(const b200_hstu_norm_mul_args &a) {
  if (a.group_norm || a.dtype == B200_HSTU_F32 || !(a.dropout_ratio > 0.f)) return 0;
  const int64_t D = (int64_t)a.H * a.V;
  if (D % 8 != 0 || D > max_row_elems<__nv_bfloat16>()) return 0;
  if (!aligned16(a.attn) || !aligned16(a.u) || !aligned16(a.weight) || !aligned16(a.bias) || !aligned16(a.out) ||
      a.attn_row_stride % 8 || a.u_row_stride % 8 || a.out_row_stride % 8)
    return 0;
  const int64_t width = D * (1 + (a.concat_u ? 1 : 0) + (a.concat_x ? 1 : 0));
  return a.rows * width / 8;
}

template <typename E>
int norm_mul_t(const b200_hstu_norm_mul_args &a, bool bwd, cudaStream_t st) {
  constexpr int EV = VecInfo<E>::EV;
  NormMulParams p;
  p.attn = a.attn; p.u = a.u; p.w = a.weight; p.b = a.bias; p.dout = a.dout;
  p.out = a.out; p.dattn = a.dattn; p.du = a.du;
  p.mean = a.mean; p.rstd = a.rstd; p.partial = (float *)a.partial;
  p.attn_rs = a.attn_row_stride; p.u_rs = a.u_row_stride; p.out_rs = a.out_row_stride;
  p.dout_rs = a.dout_row_stride; p.dattn_rs = a.dattn_row_stride; p.du_rs = a.du_row_stride;
  p.rows = a.rows; p.H = a.H; p.V = a.V; p.concat_u = a.concat_u; p.concat_x = a.concat_x; p.act = a.act;
  p.group_norm = a.group_norm; p.eps = a.eps;
  p.drop_seed = nullptr; p.drop_thr = 0; p.drop_scale = 1.f;
  const bool dropout = a.dropout_seed != nullptr && a.dropout_ratio > 0.f;
  if (dropout) {
    if (a.group_norm) return fail(B200_HSTU_EUNSUPPORTED, "norm_mul: in-kernel dropout is not built for the group-norm variant");
    if (!(a.dropout_ratio < 1.f)) return fail(B200_HSTU_EINVAL, "norm_mul: dropout_ratio must be below 1");
    uint32_t thr = (uint32_t)(a.dropout_ratio * 65536.f + 0.5f);
    thr = thr > 65535u ? 65535u : thr;
    p.drop_seed = reinterpret_cast<const unsigned long long *>(a.dropout_seed);
    p.drop_thr = thr;
    p.drop_scale = 65536.f / (float)(65536u - thr);
  }
  p.mask = nullptr;
  const int D = a.H * a.V;
  if (a.rows == 0) {
    if (bwd) {  // dweight / dbias of an empty batch are zeros
      int n = a.group_norm ? a.H : D;
      cudaMemsetAsync(a.dweight, 0, (size_t)n * sizeof(E), st);
      cudaMemsetAsync(a.dbias, 0, (size_t)n * sizeof(E), st);
    }
    return 0;
  }
  if (a.group_norm) {
    int64_t items = a.rows * a.H;
    int64_t nblk = (items + WARPS - 1) / WARPS;
    if (!bwd) {
      int grid = (int)(nblk < (int64_t)num_sms() * 8 ? nblk : (int64_t)num_sms() * 8);
      group_norm_mul_kernel<E, false><<<grid, WARPS * 32, 0, st>>>(p);
      count_launch();
      B200_CHECK_LAUNCH("group_norm_mul forward");
      return 0;
    }
    int grid = bwd_blocks();
    if (grid > MAX_BWD_BLOCKS) grid = MAX_BWD_BLOCKS;
    if ((int64_t)grid * 2 * a.H * (int64_t)sizeof(float) > a.partial_bytes)
      return fail(B200_HSTU_EWORKSPACE, "norm_mul backward: scratch too small");
    size_t smem = (size_t)WARPS * 2 * a.H * sizeof(float);
    group_norm_mul_kernel<E, true><<<grid, WARPS * 32, smem, st>>>(p);
    count_launch();
    B200_CHECK_LAUNCH("group_norm_mul backward");
    reduce_partial_kernel<E><<<(2 * a.H + 31) / 32, 256, 0, st>>>(p.partial, grid, a.H, (E *)a.dweight,
                                                                    (E *)a.dbias);
    count_launch();
    B200_CHECK_LAUNCH("group_norm_mul backward (reduce)");
    return 0;
  }
  if (D > max_row_elems<E>()) return fail(B200_HSTU_EUNSUPPORTED, "norm_mul: H*V=%d exceeds %d", D, max_row_elems<E>());
  bool vec_ok = aligned16(a.attn) && aligned16(a.u) && aligned16(a.weight) && aligned16(a.bias) &&
                a.attn_row_stride % EV == 0 && a.u_row_stride % EV == 0 && D % EV == 0;
  if (!bwd) {
    vec_ok = vec_ok && aligned16(a.out) && a.out_row_stride % EV == 0;
    p.vec_ok = vec_ok;
    int64_t nblk = (a.rows + WARPS - 1) / WARPS;
    int grid = (int)(nblk < (int64_t)num_sms() * 8 ? nblk : (int64_t)num_sms() * 8);
    if (dropout && a.dropout_mask != nullptr) {
      if (norm_mul_mask_bytes(a) == 0)
        return fail(B200_HSTU_EUNSUPPORTED, "norm_mul: a stored dropout mask needs 16-bit elements, aligned rows and H*V %% 8 == 0");
      p.mask = a.dropout_mask;
    }
    ProfileScope prof(PROF_NORM_MUL_FWD, st);
    if (vec_ok && D % EV == 0 && pick_maxv<E>(D) == 8 && p.mask == nullptr) {
      // rows of eight vectors per lane: packed rows, unpacked vector by vector
      if (dropout) norm_mul_fwd_packed_kernel<E, 8, 2><<<grid, WARPS * 32, 0, st>>>(p);
      else norm_mul_fwd_packed_kernel<E, 8, 0><<<grid, WARPS * 32, 0, st>>>(p);
    } else if (vec_ok && D % EV == 0 && pick_maxv<E>(D) == 4 && dropout && p.mask == nullptr) {
      // four vectors per lane with dropout: the packed form fits two resident CTAs
      norm_mul_fwd_packed_kernel<E, 4, 2><<<grid, WARPS * 32, 0, st>>>(p);
    } else if (dropout && p.mask != nullptr) {
      DISPATCH_MAXV(pick_maxv<E>(D), (norm_mul_fwd_kernel<E, MV, 3><<<grid, WARPS * 32, 0, st>>>(p)));
    } else if (dropout && D % EV == 0) {
      DISPATCH_MAXV(pick_maxv<E>(D), (norm_mul_fwd_kernel<E, MV, 2><<<grid, WARPS * 32, 0, st>>>(p)));
    } else if (dropout) {
      DISPATCH_MAXV(pick_maxv<E>(D), (norm_mul_fwd_kernel<E, MV, 1><<<grid, WARPS * 32, 0, st>>>(p)));
    } else {
      DISPATCH_MAXV(pick_maxv<E>(D), (norm_mul_fwd_kernel<E, MV, 0><<<grid, WARPS * 32, 0, st>>>(p)));
    }
    count_launch();
    B200_CHECK_LAUNCH("norm_mul forward");
    return 0;
  }
  vec_ok = vec_ok && aligned16(a.dout) && aligned16(a.dattn) && aligned16(a.du) && a.dout_row_stride % EV == 0 &&
           a.dattn_row_stride % EV == 0 && a.du_row_stride % EV == 0;
  p.vec_ok = vec_ok;
  int grid = bwd_blocks();
  if (grid > MAX_BWD_BLOCKS) grid = MAX_BWD_BLOCKS;
  if ((int64_t)grid * 2 * D * (int64_t)sizeof(float) > a.partial_bytes)
    return fail(B200_HSTU_EWORKSPACE, "norm_mul backward: scratch too small");
  size_t smem = (size_t)WARPS * D * sizeof(float);
  ProfileScope prof(PROF_NORM_MUL_BWD, st);
  if (vec_ok && D % EV == 0 && pick_maxv<E>(D) == 4 && !(dropout && a.dropout_mask != nullptr)) {
    // rows of four vectors per lane: accumulators and weights in shared memory, prefetched rows.  (The same
    // kernel for rows of two vectors per lane, compiled for two resident CTAs, spills and is slower than
    // the register kernel below: 0.98 instead of 0.85 ms on 690 k rows of 512.)
    const size_t wide_smem = (size_t)2 * WARPS * 4 * (EV / 4) * 32 * sizeof(float4) + (size_t)2 * 4 * 32 * sizeof(uint4);
    auto kern = dropout ? norm_mul_bwd_wide_kernel<E, 4, 3> : norm_mul_bwd_wide_kernel<E, 4, 0>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)wide_smem);
    if (e != cudaSuccess) return check_cuda(e, "norm_mul backward smem attribute");
    kern<<<grid, WARPS * 32, wide_smem, st>>>(p);
  } else if (dropout && a.dropout_mask != nullptr) {
    if (!vec_ok || EV != 8 || norm_mul_mask_bytes(a) == 0)
      return fail(B200_HSTU_EUNSUPPORTED, "norm_mul backward: a stored dropout mask needs 16-bit elements, aligned rows and H*V %% 8 == 0");
    p.mask = a.dropout_mask;
    DISPATCH_MAXV(pick_maxv<E>(D), {
      auto kern = norm_mul_bwd_kernel<E, MV, 2>;
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      kern<<<grid, WARPS * 32, smem, st>>>(p);
    });
  } else if (dropout && D % EV == 0) {
    DISPATCH_MAXV(pick_maxv<E>(D), {
      auto kern = norm_mul_bwd_kernel<E, MV, 3>;
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      kern<<<grid, WARPS * 32, smem, st>>>(p);
    });
  } else if (dropout) {
    DISPATCH_MAXV(pick_maxv<E>(D), {
      auto kern = norm_mul_bwd_kernel<E, MV, 1>;
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      kern<<<grid, WARPS * 32, smem, st>>>(p);
    });
  } else {
    DISPATCH_MAXV(pick_maxv<E>(D), {
      auto kern = norm_mul_bwd_kernel<E, MV, 0>;
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      kern<<<grid, WARPS * 32, smem, st>>>(p);
    });
  }
  count_launch();
  B200_CHECK_LAUNCH("norm_mul backward");
  reduce_partial_kernel<E><<<(2 * D + 31) / 32, 256, 0, st>>>(p.partial, grid, D, (E *)a.dweight, (E *)a.dbias);
  count_launch();
  B200_CHECK_LAUNCH("norm_mul backward (reduce)");
  return 0;
}

}  // namespace

#define DISPATCH_DTYPE(dtype, CALL)                                          \
  switch (dtype) {                                                           \
    case B200_HSTU_F32: { using E = float; return CALL; }                    \
    case B200_HSTU_BF16: { using E = __nv_bfloat16; return CALL; }           \
    case B200_HSTU_F16: { using E = __half; return CALL; }                   \
    default: return fail(B200_HSTU_EINVAL, "unknown dtype %d", (int)(dtype)); \
  }

int layer_norm_fwd(const void *x, int64_t x_rs, const void *w, const void *b, void *y, int64_t y_rs, float *mean,
                   float *rstd, int64_t rows, int D, float eps, int dtype, cudaStream_t st) {
  DISPATCH_DTYPE(dtype, (ln_fwd_t<E>(x, x_rs, w, b, y, y_rs, mean, rstd, rows, D, eps, st)));
}
int layer_norm_bwd(const void *dy, int64_t dy_rs, const void *x, int64_t x_rs, const void *w, const float *mean,
                   const float *rstd, void *dx, int64_t dx_rs, void *dw, void *db, void *partial,
                   int64_t partial_bytes, int64_t rows, int D, int dtype, cudaStream_t st) {
  DISPATCH_DTYPE(dtype, (ln_bwd_t<E>(dy, dy_rs, x, x_rs, w, mean, rstd, dx, dx_rs, dw, db, partial, partial_bytes,
                                     rows, D, st)));
}
int64_t stage_bwd_workspace_bytes(int cols) { return (int64_t)MAX_BWD_BLOCKS * 2 * cols * (int64_t)sizeof(float); }
int silu_launch(const void *dy, int64_t dy_rs, const void *x, int64_t x_rs, void *out, int64_t out_rs, int64_t rows,
                int width, bool bwd, int dtype, cudaStream_t st) {
  DISPATCH_DTYPE(dtype, (silu_t<E>(dy, dy_rs, x, x_rs, out, out_rs, rows, width, bwd, st)));
}
int64_t norm_mul_dropout_mask_bytes(const b200_hstu_norm_mul_args &a) { return norm_mul_mask_bytes(a); }
int norm_mul(const b200_hstu_norm_mul_args &a, bool bwd, cudaStream_t st) {
  DISPATCH_DTYPE(a.dtype, (norm_mul_t<E>(a, bwd, st)));
}

}  // namespace b200hstu
