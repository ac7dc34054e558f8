// Shared device/host helpers for the HSTU kernels: element-type traits, the HSTU mask on
// clamped position ids, per-sequence geometry, and error plumbing for the C ABI.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/b200_hstu.h"

namespace b200hstu {

// ---------------------------------------------------------------------------------------
// error plumbing (host)
// ---------------------------------------------------------------------------------------
void set_error(const char *fmt, ...);
int fail(int code, const char *fmt, ...);
int check_cuda(cudaError_t e, const char *what);
extern std::atomic<long long> g_launches;
inline void count_launch(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// Optional per-kernel timing: when enabled (b200_hstu_profile_enable), every launch of a hot
// kernel is bracketed by a cudaEvent pair on the launch stream; b200_hstu_profile_collect() reads
// the durations back after the caller has synchronised.  Off by default (no events are created).
enum ProfileKind {
  PROF_PLAN = 0, PROF_ATTN_FWD = 1, PROF_ATTN_BWD_DKDV = 2, PROF_ATTN_BWD_DQ = 3, PROF_ATTN_FWD_FP8 = 4,
  PROF_LN_FWD = 5, PROF_LN_BWD = 6, PROF_SILU = 7, PROF_NORM_MUL_FWD = 8, PROF_NORM_MUL_BWD = 9,
  PROF_QUANT = 10, PROF_ATTN_SIMT = 11, PROF_JAGGED = 12, PROF_TS_POS = 13,
  PROF_LN_LINEAR_PREP = 14, PROF_LN_LINEAR = 15, PROF_KINDS = 16
};
struct ProfileScope {
  int kind;
  cudaStream_t st;
  cudaEvent_t stop;
  ProfileScope(int kind, cudaStream_t st);
  ~ProfileScope();
};

#define B200_CHECK_LAUNCH(what)                                   \
  do {                                                            \
    int _st = ::b200hstu::check_cuda(cudaGetLastError(), what);   \
    if (_st != 0) return _st;                                     \
  } while (0)

// ---------------------------------------------------------------------------------------
// element conversion
// ---------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

// (approximate reciprocal: 2 ulp, one MUFU operation and a multiply instead of the dozen instructions
// of an IEEE division - these run in memory-bound kernels with few warps, where instructions count)
__device__ __forceinline__ float sigmoidf_(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x * sigmoidf_(x); }
// d/dx [x * sigmoid(x)] = s * (1 + x * (1 - s))
__device__ __forceinline__ float dsiluf_(float x) {
  float s = sigmoidf_(x);
  return s * (1.f + x * (1.f - s));
}

// ---------------------------------------------------------------------------------------
// The HSTU mask of one sequence, on clamped position ids.
//
// id(p) = min(max(p - c + 1, 0), max_id)   (c = contextual_seq_len; the max() only if c > 0)
// max_id = L - max(c - 1, 0) - num_targets
// valid(i, j) = (i == j) or (d > 0 and (W == 0 or d <= W or (F > 0 and id_i >= max_id - F)))
//               or (c > 0 and id_i == 0 and id_j < max_id),   d = id_i - id_j
// which is the reference's construction
// (generative_recommenders/ops/pytorch/pt_hstu_attention.py:44-83) evaluated for one (row, col).
// ---------------------------------------------------------------------------------------
struct SeqMask {
  int L;       // rows/cols of this sequence that take part (already truncated at max_seq_len)
  int max_id;
  int c;       // contextual_seq_len
  int W;       // max_attn_len (0 = unlimited)
  int F;       // min_full_attn_seq_len
  __host__ __device__ __forceinline__ int id(int p) const {
    int v = p;
    if (c > 0) {
      v = p - c + 1;
      v = v < 0 ? 0 : v;
    }
    return v < max_id ? v : max_id;
  }
  __host__ __device__ __forceinline__ bool valid_ids(int i, int j, int id_i, int id_j) const {
    int d = id_i - id_j;
    bool v = d > 0;
    if (W > 0) v = v && (d <= W || (F > 0 && id_i >= max_id - F));
    v = v || (i == j);
    if (c > 0) v = v || (id_i == 0 && id_j < max_id);
    return v;
  }
  __host__ __device__ __forceinline__ bool valid(int i, int j) const { return valid_ids(i, j, id(i), id(j)); }
};

__host__ __device__ __forceinline__ SeqMask make_seq_mask(int len, int max_seq_len, int num_targets, int c, int W,
                                                          int F) {
  SeqMask m;
  m.L = len < max_seq_len ? len : max_seq_len;
  m.c = c;
  m.W = W;
  m.F = F;
  // the reference derives max_id from the untruncated length (seq_offsets difference)
  m.max_id = len - (c > 0 ? c - 1 : 0) - num_targets;
  return m;
}

// ---------------------------------------------------------------------------------------
// kv-tile range a query tile has to visit (tile edge `T` rows/cols), used for block skipping.
// Rows [m0, m0+T) of a sequence; returns a half-open range of kv positions [lo, hi) that
// contains every valid column of every row of the tile, plus (for tiles made only of target
// rows) the tile's own diagonal block, which lies outside [lo, hi).  Conservative (a superset)
// everywhere and exact on tile granularity for the regular domain
// (L - targets >= contextual + 1).
// ---------------------------------------------------------------------------------------
struct KvRange {
  int lo, hi;      // main range of kv positions
  int diag_lo;     // >= 0: an extra block [diag_lo, diag_lo + T) outside the main range
};

__host__ __device__ __forceinline__ KvRange kv_range_for_q_tile(const SeqMask &m, int len, int num_targets, int m0,
                                                                int T) {
  KvRange r;
  const int L = m.L;
  int m1 = m0 + T < L ? m0 + T : L;
  int u = len - num_targets;  // first target position
  r.diag_lo = -1;
  bool regular = (u >= m.c + 1) && (num_targets >= 0) && (len <= L);
  if (!regular) {  // degenerate sequence (or truncated): visit everything, the element mask decides
    r.lo = 0;
    r.hi = L;
    return r;
  }
  if (m0 < m.c) {  // contextual rows see all of [0, u); later rows of the tile see up to themselves
    r.lo = 0;
    r.hi = u > m1 ? u : m1;
    if (r.hi > L) r.hi = L;
    return r;
  }
  int first = m0 < u ? m0 : u;  // smallest effective row position in the tile
  int lo = 0;
  if (m.W > 0 && m.F == 0) {
    lo = first - m.W;
    if (lo < m.c) lo = 0;  // first - W <= c - 1: the row also sees the contextual prefix
  }
  r.lo = lo;
  if (m0 >= u) {  // only target rows: history/contextual columns + own diagonal block
    r.hi = u;
    r.diag_lo = m0;
  } else {
    r.hi = m1;
  }
  return r;
}

// Philox4x32-10 (counter c0, c1, 0, 0; key k0, k1): the counter-based generator behind both dropout
// masks (output stage and attention weights), so that a backward kernel regenerates the forward's
// mask from the seed.
__device__ __forceinline__ void philox4x32_10(uint32_t k0, uint32_t k1, uint32_t c0, uint32_t c1, uint32_t (&o)[4]) {
  uint32_t c2 = 0, c3 = 0;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    c0 = hi1 ^ c1 ^ k0;
    c1 = lo1;
    c2 = hi0 ^ c3 ^ k1;
    c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  o[0] = c0; o[1] = c1; o[2] = c2; o[3] = c3;
}

// Element idx of a mask takes the (idx % 8)-th 16-bit piece of the generator's output for counter
// idx / 8 and is kept when that piece is at least `thr` = round(ratio * 65536).
__device__ __forceinline__ bool philox_keep(uint32_t k0, uint32_t k1, uint64_t idx, uint32_t thr) {
  uint32_t o[4];
  const uint64_t g = idx >> 3;
  philox4x32_10(k0, k1, (uint32_t)g, (uint32_t)(g >> 32), o);
  const int j = (int)(idx & 7);
  return ((o[j >> 1] >> (16 * (j & 1))) & 0xffffu) >= thr;
}

}  // namespace b200hstu
