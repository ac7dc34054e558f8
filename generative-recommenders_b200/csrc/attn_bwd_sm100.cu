// Jagged HSTU attention backward on Blackwell tensor cores (tcgen05 + TMEM + TMA), bf16 / fp16,
// head dimension 64 or 128 (d_qk == d_v), constant attention scale.
//
// With x = alpha q.k (+ bias), s = sigmoid(x), P = x s scale mask:
//   dV = P^T dO          dP = dO V^T          dS = dP * (s + x s (1 - s)) * scale * mask
//   dK = alpha dS^T Q    dQ = alpha dS K
// (the math of generative_recommenders/ops/triton/triton_hstu_attention.py:1905-2020; no softmax
// statistics and no `out` are needed).
//
// Two launches of one persistent kernel template; each element of every gradient has exactly one
// owner, so there are no atomics, no fp32 dQ scratch, no convert pass, and the result is
// bit-reproducible:
//   * DKDV = true  - a work item is (sequence, 128-row K/V tile, head).  K and V stay in shared
//     memory; the Q and dO tiles of every query tile that can see the K/V tile stream through
//     2-stage TMA rings.  Stage 1: S^T = K Q^T and dP^T = V dO^T into TMEM.  The threads that
//     own one K/V row each turn them into bf16 P^T and dS^T written back over the same TMEM
//     columns.  Stage 2: dV += P^T dO and dK += dS^T Q with the TMEM tiles as A operands (dO and
//     Q are MN-major B operands).
//   * DKDV = false - a work item is (sequence, 128-row query tile, head): Q and dO stay, K and V
//     stream; stage 1: S = Q K^T, dP = dO V^T; stage 2: dQ += dS K.  Consecutive items alternate
//     between two dQ accumulators, so an item never waits for the previous one to be stored.
// Fourteen warps, specialised:
//   warp 0       TMA producer; claims the next item from an atomic counter and publishes it
//   warp 1       MMA issuer; owns TMEM.  Per streamed tile i four 128 x 128 x 128 products:
//                G1 = X0 Y0^T (scores), G2 = X1 Y1^T (dP), G3 (kv-stationary launch only) and G4
//                (stage 2), issued in the order  G3(i), G1(i+1), G4(i), G2(i+1):  the tensor pipe
//                computes the next tile's scores while the CUDA cores turn dP into dS, and the
//                next dP while they turn scores into P.  During the last tile of an item the
//                G1 / G2 of the next item's first tile are issued instead.  The stationary tiles
//                are released as soon as the item's last G2 is issued.
//   warps 2-9    activation, one row of the stationary tile per thread, 64 of the 128 columns per
//                warpgroup.  Phase A: scores -> P (16-bit, written over the scores) and silu',
//                which stays in registers as packed halves; phase B: dP -> dS = dP silu' (16-bit,
//                written over dP).  Every thread writes only over columns it has read itself
//                (warpgroup 0: columns [0,32), warpgroup 1: [64,96) of the 128-column region), so no
//                barrier between the warps is needed; stage 2 takes its K steps from those two
//                column ranges.
//   warps 10-13  epilogue: accumulators (fp32, TMEM) -> scale -> 16-bit -> global
// TMEM: scores / P [0,128), dP / dS [128,256), two 128-column accumulators.  Constant factors
// are folded into the epilogues: dV * scale, dK * scale*alpha, dQ * scale*alpha.
#include <stdlib.h>

#include "attn_plan.cuh"
#include "sm100_ptx.cuh"

namespace b200hstu {

using namespace ptx;

int make_tile_map_rows(CUtensorMap *m, const void *base, int64_t rows, int64_t cols, int64_t row_stride_elems,
                       int elem_bytes, bool is_bf16, int box_rows);
int device_sm_count();
void fill_pdl_config(cudaLaunchConfig_t *cfg, cudaLaunchAttribute *attr, int grid, int threads, size_t smem,
                     cudaStream_t st);

namespace {

constexpr int BWD_THREADS = 448;
constexpr int Y0_STAGES = 3;  // streamed operand read by G1 and by G4 (Q | K): longest lifetime
constexpr int Y1_STAGES = 2;  // streamed operand read by G2 (and G3): dO | V
constexpr int BWD_SCHED_CONSUMERS = 13;  // MMA warp, 8 activation warps, 4 epilogue warps: one arrival each

struct BwdParams {
  AttnGeomParams g;
  PlanHeader *plan;
  const ItemDesc *items;
  int *status;
  void *dq, *dk, *dv;
  int64_t dq_rs, dq_hs, dk_rs, dk_hs, dv_rs, dv_hs;
  const float *attn_scale;  // NULL or one fp32 on the device
  const float *bias;       // bias_by_distance as given (element-wise path)
  int bias_numel;
  const float *bias_ext;   // centre of the signed-distance table (see BiasTable); NULL = no bias
  float *dbias;            // q-stationary launch, optional: gradient of `bias` (fp32 [bias_numel], accumulated into)
  float half_alpha, alpha, inv_n;
  int H;
  int wide_stores;  // dq / dk / dv rows are 32-byte aligned
  ulonglong2 *trace;  // optional timeline of CTA 0 (see Tracer); NULL = off
};

template <int D>
struct BwdSmem {
  static constexpr int CHUNKS = D / 64;
  static constexpr int TILE_BYTES = TILE * D * 2;
  static constexpr int CHUNK_BYTES = TILE * 128;
  static constexpr int A_OFF = 0;                                 // stationary tile 0 (K or Q)
  static constexpr int B_OFF = A_OFF + TILE_BYTES;                // stationary tile 1 (V or dO)
  static constexpr int X_OFF = B_OFF + TILE_BYTES;                // streamed ring 0 (Q or K)
  static constexpr int Y_OFF = X_OFF + Y0_STAGES * TILE_BYTES;    // streamed ring 1 (dO or V)
  static constexpr int BAR_OFF = Y_OFF + Y1_STAGES * TILE_BYTES;
  static constexpr int NUM_BARS = 40;
  static constexpr int MISC_OFF = BAR_OFF + NUM_BARS * 8;
  static constexpr int SCHED_OFF = MISC_OFF + 64;
  static constexpr int TOTAL = SCHED_OFF + 4 * 64;   // ring of work items (GEOM_SLOTS x GEOM_SLOT_BYTES)
  static constexpr int DYN_BYTES = (TOTAL + 1024) > 116 * 1024 ? (TOTAL + 1024) : 116 * 1024;
};

__device__ __forceinline__ uint32_t pack2h(float a, float b, bool is_bf16) {
  if (is_bf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&v);
}

// silu(x) / silu'(x) from one tanh: h = x/2, t = tanh(h): silu = h + h t, sigma = .5 + .5 t,
// silu' = sigma + silu (.5 - .5 t)
__device__ __forceinline__ void silu_and_grad(float h, float &silu, float &dsilu) {
  float t = tanh_approx(h);
  silu = fmaf(h, t, h);
  float sg = fmaf(0.5f, t, 0.5f);
  float om = fmaf(-0.5f, t, 0.5f);
  dsilu = fmaf(silu, om, sg);
}

// silu' of a pair, kept between the two activation phases as packed fp16 (values in [-0.1, 1.1])
__device__ __forceinline__ uint32_t pack_keep(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&v);
}
__device__ __forceinline__ float2 unpack_keep(uint32_t u) {
  return __half22float2(*reinterpret_cast<__half2 *>(&u));
}

// Phase A on 32 score columns of one thread: P (kv-stationary launch) written over the scores,
// silu' (zero where masked) returned in `keep`.  `bits` marks the visible columns; with
// MASKED = false all of them are.
// BIAS: bp points at the signed-distance table entry (already halved) of this thread's row /
// column and the chunk's first streamed position; the streamed index grows along the chunk, so the
// distance q - k grows in the kv-stationary launch (entry bp[+k]) and shrinks in the q-stationary
// one (entry bp[-k]).
template <bool IS_BF16, bool DKDV, bool MASKED, bool BIAS>
__device__ __forceinline__ void phase_a_chunk(uint32_t t_in, uint32_t t_out, float half_alpha, uint32_t bits,
                                              uint32_t (&keep)[16], const float *bp) {
  uint32_t rs[32];
  tmem_ld32(t_in, rs);
  tc_wait_ld();
  uint32_t pk[16];
  if (DKDV) {
    // kv-stationary launch: packed fp32 arithmetic for SiLU and its derivative (half as many
    // instructions: this phase is bound by instruction issue), scalar selects for the mask (measured:
    // the byte-permute pair masks of the branch below make this launch slower, the q-stationary
    // one faster; the packed arithmetic alone takes 7 % off this launch)
#pragma unroll
    for (int x = 0; x < 16; ++x) {
      float sl0, dsl0, sl1, dsl1;
      float h0, h1, sg0, sg1, om0, om1;
      mul2(__uint_as_float(rs[2 * x]), __uint_as_float(rs[2 * x + 1]), half_alpha, h0, h1);
      if (BIAS) {
        h0 += __ldg(DKDV ? bp + 2 * x : bp - 2 * x);
        h1 += __ldg(DKDV ? bp + 2 * x + 1 : bp - 2 * x - 1);
      }
      const float t0 = tanh_approx(h0), t1 = tanh_approx(h1);
      fma2(h0, h1, t0, t1, h0, h1, sl0, sl1);
      fma2(0.5f, 0.5f, t0, t1, 0.5f, 0.5f, sg0, sg1);
      fma2(-0.5f, -0.5f, t0, t1, 0.5f, 0.5f, om0, om1);
      fma2(sl0, sl1, om0, om1, sg0, sg1, dsl0, dsl1);
      if (MASKED) {
        const bool v0 = bits & (1u << (2 * x)), v1 = bits & (1u << (2 * x + 1));
        sl0 = v0 ? sl0 : 0.f;
        sl1 = v1 ? sl1 : 0.f;
        dsl0 = v0 ? dsl0 : 0.f;
        dsl1 = v1 ? dsl1 : 0.f;
      }
      pk[x] = pack2h(sl0, sl1, IS_BF16);
      keep[x] = pack_keep(dsl0, dsl1);
    }
  } else {
    // q-stationary launch: the pair goes through packed fp32 arithmetic - the same operations as
    // silu_and_grad(), half as many instructions - and masked-out elements are cleared in the
    // packed result (P is not needed here)
    const PairMasks pm(bits);
#pragma unroll
    for (int x = 0; x < 16; ++x) {
      float h0, h1, sl0, sl1, sg0, sg1, om0, om1, dsl0, dsl1;
      mul2(__uint_as_float(rs[2 * x]), __uint_as_float(rs[2 * x + 1]), half_alpha, h0, h1);
      if (BIAS) {
        h0 += __ldg(DKDV ? bp + 2 * x : bp - 2 * x);
        h1 += __ldg(DKDV ? bp + 2 * x + 1 : bp - 2 * x - 1);
      }
      const float t0 = tanh_approx(h0), t1 = tanh_approx(h1);
      fma2(h0, h1, t0, t1, h0, h1, sl0, sl1);
      fma2(0.5f, 0.5f, t0, t1, 0.5f, 0.5f, sg0, sg1);
      fma2(-0.5f, -0.5f, t0, t1, 0.5f, 0.5f, om0, om1);
      fma2(sl0, sl1, om0, om1, sg0, sg1, dsl0, dsl1);
      const uint32_t lanes = MASKED ? pm.pair(x) : 0xffffffffu;
      keep[x] = pack_keep(dsl0, dsl1) & lanes;
    }
  }
  if (DKDV) tmem_st16(t_out, pk);
}

// Phase A, element-wise variant (sequences outside the regular domain, or a relative bias)
template <bool IS_BF16, bool DKDV>
__device__ __forceinline__ void phase_a_exact_chunk(uint32_t t_in, uint32_t t_out, float half_alpha, const SeqMask &m,
                                                    int own, int id_own, int c0, const float *bias, int bias_numel,
                                                    uint32_t (&keep)[16]) {
  const int L = m.L;
  uint32_t rs[32];
  tmem_ld32(t_in, rs);
  tc_wait_ld();
  uint32_t pk[16];
#pragma unroll
  for (int x = 0; x < 32; x += 2) {
    float pv[2], dv[2];
#pragma unroll
    for (int y = 0; y < 2; ++y) {
      const int other = c0 + x + y;
      const int qi_ = DKDV ? other : own, kj_ = DKDV ? own : other;
      float hh = __uint_as_float(rs[x + y]) * half_alpha;
      if (bias != nullptr) {
        int dist = qi_ > kj_ ? qi_ - kj_ : kj_ - qi_;
        if (dist < bias_numel) hh += 0.5f * bias[dist];
      }
      float sl, dsl;
      silu_and_grad(hh, sl, dsl);
      const int id_other = m.id(other);
      bool valid = qi_ < L && kj_ < L && m.valid_ids(qi_, kj_, DKDV ? id_other : id_own, DKDV ? id_own : id_other);
      pv[y] = valid ? sl : 0.f;
      dv[y] = valid ? dsl : 0.f;
    }
    pk[x / 2] = pack2h(pv[0], pv[1], IS_BF16);
    keep[x / 2] = pack_keep(dv[0], dv[1]);
  }
  if (DKDV) tmem_st16(t_out, pk);
}

// Phase B on 32 dP columns of one thread: dS = dP silu' written over dP as a 16-bit tile.
template <bool IS_BF16, bool PACKED>
__device__ __forceinline__ void phase_b_chunk(uint32_t t_in, uint32_t t_out, const uint32_t (&keep)[16]) {
  uint32_t rp[32];
  tmem_ld32(t_in, rp);
  tc_wait_ld();
  uint32_t dk[16];
#pragma unroll
  for (int x = 0; x < 16; ++x) {
    const float2 g = unpack_keep(keep[x]);
    float d0, d1;
    if (PACKED) {
      mul2v(__uint_as_float(rp[2 * x]), __uint_as_float(rp[2 * x + 1]), g.x, g.y, d0, d1);
    } else {
      d0 = __uint_as_float(rp[2 * x]) * g.x;
      d1 = __uint_as_float(rp[2 * x + 1]) * g.y;
    }
    dk[x] = pack2h(d0, d1, IS_BF16);
  }
  tmem_st16(t_out, dk);
}

// Phase B of the q-stationary launch when the gradient of the relative bias is wanted: the same dS,
// and its sums along the diagonals of the chunk (query - key distance constant).  Lane l of the
// warp owns query row l of 32 consecutive rows, register x holds key column x of the chunk, so the
// element (l, x) belongs to diagonal l - x.  Rotating register x by x lanes brings every element
// of diagonal m to lane m mod 32: lane l collects diagonal l (elements that did not wrap around) and
// diagonal l - 32 (those that did) - which are the distances of the lane's own row to the chunk's
// first column and to the column 32 before it.  Two fp32 atomics per lane and chunk then add the
// sums (times the attention scale, which the 16-bit dS does not carry) to the gradient.  Rows
// beyond the sequence hold scores of the next sequence's tokens: they are cleared first.
template <bool IS_BF16>
__device__ __forceinline__ void phase_b_chunk_dbias(uint32_t t_in, uint32_t t_out, const uint32_t (&keep)[16],
                                                    float *dbias, int bias_numel, int dist, bool row_valid, int lane,
                                                    float sc) {
  uint32_t rp[32];
  tmem_ld32(t_in, rp);
  tc_wait_ld();
  uint32_t dk[16];
  float pos = 0.f, neg = 0.f;
#pragma unroll
  for (int x = 0; x < 16; ++x) {
    const float2 g = unpack_keep(keep[x]);
    float d0, d1;
    mul2v(__uint_as_float(rp[2 * x]), __uint_as_float(rp[2 * x + 1]), g.x, g.y, d0, d1);
    dk[x] = pack2h(d0, d1, IS_BF16);
    d0 = row_valid ? d0 : 0.f;
    d1 = row_valid ? d1 : 0.f;
    const float r0 = __shfl_sync(0xffffffffu, d0, (lane + 2 * x) & 31);
    const float r1 = __shfl_sync(0xffffffffu, d1, (lane + 2 * x + 1) & 31);
    if (lane + 2 * x < 32) pos += r0; else neg += r0;
    if (lane + 2 * x + 1 < 32) pos += r1; else neg += r1;
  }
  tmem_st16(t_out, dk);
  const int a0 = dist < 0 ? -dist : dist, a1 = dist - 32 < 0 ? 32 - dist : dist - 32;
  if (pos != 0.f && a0 < bias_numel) atomicAdd(dbias + a0, pos * sc);
  if (neg != 0.f && a1 < bias_numel) atomicAdd(dbias + a1, neg * sc);
}

// What the activation warps do for one streamed tile: phase A, hand the score region back, phase
// B, hand the dP region back.  MODE 0: every element visible; 1: per-row / per-column bit masks;
// 2: element-wise mask and bias.
struct ActTile {
  uint32_t tS, tP;          // this thread's 64 score / dP columns in TMEM
  uint32_t t_full, w_full;  // barrier pairs
  uint32_t parity;
  float half_alpha;
  int lane;
  const float *bias_at;     // table entry of (this thread's row / column, first streamed position); NULL = no bias
  float *dbias;             // q-stationary launch: gradient of the bias wanted (NULL = no)
  int dbias_numel;
  const float *sc_ptr;      // attention scale on the device, or NULL (1 / max_seq_len, in inv_n)
  float inv_n;
  bool row_valid;           // this thread's query row lies inside the sequence
};

template <bool IS_BF16, bool DKDV, int MODE, bool BIAS>
__device__ __forceinline__ bool act_tile_body(const WaitCtx &wc, const ActTile &a, uint32_t bits0, uint32_t bits1,
                                              const SeqMask &m, int own, int c0, const float *bias, int bias_numel,
                                              Tracer &tr) {
  uint32_t keep0[16], keep1[16];
  tr.mark(30);
  if (!mbar_wait(wc, a.t_full, a.parity, 601)) return false;
  tc_fence_after();
  tr.mark(31);
  if (MODE == 0) {
    phase_a_chunk<IS_BF16, DKDV, false, false>(a.tS, a.tS, a.half_alpha, 0xffffffffu, keep0, nullptr);
    phase_a_chunk<IS_BF16, DKDV, false, false>(a.tS + 32, a.tS + 16, a.half_alpha, 0xffffffffu, keep1, nullptr);
  } else if (MODE == 1) {
    if (BIAS) {
      phase_a_chunk<IS_BF16, DKDV, true, true>(a.tS, a.tS, a.half_alpha, bits0, keep0, a.bias_at);
      phase_a_chunk<IS_BF16, DKDV, true, true>(a.tS + 32, a.tS + 16, a.half_alpha, bits1, keep1,
                                               DKDV ? a.bias_at + 32 : a.bias_at - 32);
    } else {
      phase_a_chunk<IS_BF16, DKDV, true, false>(a.tS, a.tS, a.half_alpha, bits0, keep0, nullptr);
      phase_a_chunk<IS_BF16, DKDV, true, false>(a.tS + 32, a.tS + 16, a.half_alpha, bits1, keep1, nullptr);
    }
  } else {
    const int id_own = m.id(own);
    phase_a_exact_chunk<IS_BF16, DKDV>(a.tS, a.tS, a.half_alpha, m, own, id_own, c0, bias, bias_numel, keep0);
    phase_a_exact_chunk<IS_BF16, DKDV>(a.tS + 32, a.tS + 16, a.half_alpha, m, own, id_own, c0 + 32, bias, bias_numel,
                                       keep1);
  }
  tr.mark(37);
  if (DKDV) tc_wait_st();
  tc_fence_before();
  __syncwarp();
  if (a.lane == 0) mbar_arrive(a.w_full);
  tr.mark(33);
  if (!mbar_wait(wc, a.t_full + 8, a.parity, 603)) return false;
  tc_fence_after();
  tr.mark(32);
  if (!DKDV && a.dbias != nullptr) {
    const float sc = a.sc_ptr != nullptr ? a.sc_ptr[0] : a.inv_n;
    phase_b_chunk_dbias<IS_BF16>(a.tP, a.tP, keep0, a.dbias, a.dbias_numel, own - c0, a.row_valid, a.lane, sc);
    phase_b_chunk_dbias<IS_BF16>(a.tP + 32, a.tP + 16, keep1, a.dbias, a.dbias_numel, own - c0 - 32, a.row_valid,
                                 a.lane, sc);
  } else {
    phase_b_chunk<IS_BF16, !DKDV>(a.tP, a.tP, keep0);
    phase_b_chunk<IS_BF16, !DKDV>(a.tP + 32, a.tP + 16, keep1);
  }
  tc_wait_st();
  tc_fence_before();
  __syncwarp();
  if (a.lane == 0) mbar_arrive(a.w_full + 8);
  tr.mark(34);
  return true;
}

// The element-wise variant stays out of line: it is several times the size of the interval path.
template <bool IS_BF16, bool DKDV>
__device__ __noinline__ bool act_tile_exact(WaitCtx wc, ActTile a, SeqMask m, int own, int c0, const float *bias,
                                            int bias_numel) {
  Tracer off;
  off.init(nullptr, 0, false);
  return act_tile_body<IS_BF16, DKDV, 2, false>(wc, a, 0u, 0u, m, own, c0, bias, bias_numel, off);
}

// Stores one 128 x D fp32 accumulator (TMEM) as scaled 16-bit rows of a jagged tensor.  One row
// per thread, so every lane of a store hits another 32-byte sector: `wide` (row pointers 32-byte
// aligned) writes whole sectors with 256-bit stores, half as many instructions.
template <int D, bool IS_BF16>
__device__ __forceinline__ void store_acc_rows(uint32_t tacc, float scale, uint16_t *row_ptr, bool row_valid,
                                               bool wide) {
  uint32_t r[2][32];
  tmem_ld32(tacc, r[0]);
#pragma unroll
  for (int c = 0; c < D / 32; ++c) {
    tc_wait_ld();
    if (c + 1 < D / 32) tmem_ld32(tacc + (c + 1) * 32, r[(c + 1) & 1]);
    if (row_valid) {
      const uint32_t(&v)[32] = r[c & 1];
      uint4 o4[4];
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        o4[x].x = pack2h(__uint_as_float(v[8 * x + 0]) * scale, __uint_as_float(v[8 * x + 1]) * scale, IS_BF16);
        o4[x].y = pack2h(__uint_as_float(v[8 * x + 2]) * scale, __uint_as_float(v[8 * x + 3]) * scale, IS_BF16);
        o4[x].z = pack2h(__uint_as_float(v[8 * x + 4]) * scale, __uint_as_float(v[8 * x + 5]) * scale, IS_BF16);
        o4[x].w = pack2h(__uint_as_float(v[8 * x + 6]) * scale, __uint_as_float(v[8 * x + 7]) * scale, IS_BF16);
      }
      if (wide) {
        st_global_256(row_ptr + c * 32, o4[0], o4[1]);
        st_global_256(row_ptr + c * 32 + 16, o4[2], o4[3]);
      } else {
#pragma unroll
        for (int x = 0; x < 4; ++x) *reinterpret_cast<uint4 *>(row_ptr + c * 32 + x * 8) = o4[x];
      }
    }
  }
}

template <int D>
__device__ __forceinline__ void zero_rows_beyond(uint16_t *base, int64_t rs, int64_t hs, int h, int start, int L,
                                                 int len, int row_in_tile) {
  for (int r2 = L + row_in_tile; r2 < len; r2 += TILE) {
    uint16_t *zr = base + (int64_t)(start + r2) * rs + (int64_t)h * hs;
    for (int x = 0; x < D; x += 8) *reinterpret_cast<uint4 *>(zr + x) = make_uint4(0, 0, 0, 0);
  }
}

template <bool DKDV>
__device__ __forceinline__ void fill_bwd_item(TileItem &it, const AttnGeomParams &g, const ItemDesc &d) {
  if (DKDV) fill_kv_item(it, g, d.b, d.t, d.start, d.len, d.nt);
  else fill_q_item(it, g, d.b, d.t, d.start, d.len, d.nt);
}

// ---------------------------------------------------------------------------------------
// Work items travel from the producer warp to the other warps as ready-made geometry (64 bytes
// in a 4-slot shared-memory ring): the tile ranges are worked out once per item, by the warp with
// the most slack, a whole item ahead of their use.  Code that runs once per item is fetched
// cold, so the less of it the consumers execute at an item boundary the shorter the boundary.
// ---------------------------------------------------------------------------------------
struct __align__(16) ItemGeom {
  int idx;                   // (item, head) index; >= number of (item, head) pairs: no more work
  int start, len, nt;        // first token row, untruncated length, number of targets
  int m0, n_tiles, t_lo, n_main;
  int extra_tile, L, u, regular;
  int max_id, pad0, pad1, pad2;
  __device__ __forceinline__ int tile_at(int j) const { return j < n_main ? t_lo + j : extra_tile; }
};
constexpr int GEOM_SLOTS = 4;
constexpr int GEOM_SLOT_BYTES = 64;

__device__ __forceinline__ void geom_from_item(ItemGeom &g, const TileItem &it, int idx) {
  g.idx = idx;
  g.start = it.start; g.len = it.len; g.nt = it.nt;
  g.m0 = it.m0; g.n_tiles = it.n_tiles; g.t_lo = it.t_lo; g.n_main = it.n_main;
  g.extra_tile = it.extra_tile; g.L = it.m.L; g.u = it.u; g.regular = it.regular ? 1 : 0;
  g.max_id = it.m.max_id; g.pad0 = g.pad1 = g.pad2 = 0;
}
// the fields the activation and epilogue code reads (no tile ranges are recomputed)
__device__ __forceinline__ void item_from_geom(TileItem &it, const ItemGeom &g, const AttnGeomParams &gp) {
  it.b = 0; it.mt = g.m0 / TILE;
  it.start = g.start; it.len = g.len; it.nt = g.nt;
  it.m0 = g.m0;
  it.m.L = g.L; it.m.max_id = g.max_id; it.m.c = gp.c; it.m.W = gp.W; it.m.F = gp.F;
  it.t_lo = g.t_lo; it.n_main = g.n_main; it.extra_tile = g.extra_tile; it.n_tiles = g.n_tiles;
  it.u = g.u; it.regular = g.regular != 0;
}
// item ordinals n = 0, 1, 2, ... use slot n % 4
__device__ __forceinline__ bool geom_publish(const WaitCtx &wc, uint8_t *ring, uint32_t full0, uint32_t empty0,
                                             uint32_t n, const ItemGeom &g) {
  const uint32_t slot = n & (GEOM_SLOTS - 1);
  if (!mbar_wait(wc, empty0 + 8 * slot, ((n / GEOM_SLOTS) & 1) ^ 1, 901)) return false;
  int4 *dst = reinterpret_cast<int4 *>(ring + slot * GEOM_SLOT_BYTES);
  const int4 *src = reinterpret_cast<const int4 *>(&g);
  dst[0] = src[0]; dst[1] = src[1]; dst[2] = src[2]; dst[3] = src[3];
  asm volatile("fence.acq_rel.cta;" ::: "memory");
  mbar_arrive(full0 + 8 * slot);
  return true;
}
__device__ __forceinline__ bool geom_fetch(const WaitCtx &wc, const uint8_t *ring, uint32_t full0, uint32_t empty0,
                                           uint32_t n, ItemGeom &g, bool arrive) {
  const uint32_t slot = n & (GEOM_SLOTS - 1);
  if (!mbar_wait(wc, full0 + 8 * slot, (n / GEOM_SLOTS) & 1, 902)) return false;
  const volatile int *src = reinterpret_cast<const volatile int *>(ring + slot * GEOM_SLOT_BYTES);
  int *dst = reinterpret_cast<int *>(&g);
#pragma unroll
  for (int i = 0; i < 13; ++i) dst[i] = src[i];
  __syncwarp();
  if (arrive) mbar_arrive(empty0 + 8 * slot);
  return true;
}

// The two kinds of tensor-core products of the MMA warp.
struct Stage1Args {
  uint32_t x_bar, x_par;   // stationary tile arrival to wait for (x_bar = 0: already waited for)
  uint32_t y_bar, y_par;   // streamed tile arrival
  uint64_t x_desc;
  uint32_t y_smem, d_tmem, idesc;
  uint32_t commit_t, commit_y, commit_x;  // barriers to signal on completion (0 = none)
};
template <int D>
__device__ __forceinline__ bool bwd_stage1(const WaitCtx &wc, const Stage1Args &a) {
  if (a.x_bar != 0 && !mbar_wait(wc, a.x_bar, a.x_par, 501)) return false;
  if (!mbar_wait(wc, a.y_bar, a.y_par, 502)) return false;
  tc_fence_after();
  const uint64_t y_desc = make_smem_desc(a.y_smem, 16, 1024);
  if (elect_one()) {
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const uint32_t off = (ks / 4) * (TILE * 128) + (ks % 4) * 32;
      mma_ss(a.d_tmem, desc_advance(a.x_desc, off), desc_advance(y_desc, off), a.idesc, ks > 0);
    }
    tc_commit(a.commit_t);
    if (a.commit_y != 0) tc_commit(a.commit_y);
    if (a.commit_x != 0) tc_commit(a.commit_x);
  }
  __syncwarp();
  return true;
}
// acc += A B with the 16-bit A tile in TMEM (K steps 0-3 in columns [0,32), 4-7 in [64,96) of its
// 128-column region) and the streamed tile as MN-major B: 64-column blocks 16 KB apart, 16 rows
// (one K step) = 2 KB.
__device__ __forceinline__ void bwd_stage2(uint32_t acc_tmem, uint32_t a_tmem, uint32_t y_smem, uint32_t idesc,
                                        uint32_t acc_on, uint32_t commit0, uint32_t commit1) {
  const uint64_t y_mn = make_smem_desc(y_smem, TILE * 128, 1024);
  if (elect_one()) {
#pragma unroll
    for (int ks = 0; ks < TILE / 16; ++ks)
      mma_ts(acc_tmem, a_tmem + (ks / 4) * 64 + (ks % 4) * 8, desc_advance(y_mn, ks * 2048), idesc,
             (acc_on || ks > 0) ? 1u : 0u);
    if (commit0 != 0) tc_commit(commit0);
    if (commit1 != 0) tc_commit(commit1);
  }
  __syncwarp();
}

template <int D, bool IS_BF16, bool DKDV, bool BIAS>
__global__ void __launch_bounds__(BWD_THREADS, 1)
    hstu_attn_bwd_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                               const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                               const BwdParams p) {
  using SM = BwdSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  // stationary pair X0 (K | Q), X1 (V | dO); streamed rings Y0 (Q | K), Y1 (dO | V)
  const uint32_t sX0 = smem_base + SM::A_OFF, sX1 = smem_base + SM::B_OFF;
  const uint32_t sY0 = smem_base + SM::X_OFF, sY1 = smem_base + SM::Y_OFF;
  const CUtensorMap *mapX0 = DKDV ? &tmap_k : &tmap_q;
  const CUtensorMap *mapX1 = DKDV ? &tmap_v : &tmap_do;
  const CUtensorMap *mapY0 = DKDV ? &tmap_q : &tmap_k;
  const CUtensorMap *mapY1 = DKDV ? &tmap_do : &tmap_v;
  const uint32_t bars = smem_base + SM::BAR_OFF;
  const uint32_t x_full = bars + 0, x_empty = bars + 16;   // [2]: stationary tile 0 (K | Q), tile 1 (V | dO)
  const uint32_t y0_full = bars + 32, y0_empty = y0_full + 8 * Y0_STAGES;
  const uint32_t y1_full = y0_empty + 8 * Y0_STAGES, y1_empty = y1_full + 8 * Y1_STAGES;
  const uint32_t t_full = y1_empty + 8 * Y1_STAGES;  // [2] scores ready, dP ready
  const uint32_t w_full = t_full + 16;               // [2] P written (scores consumed), dS written
  const uint32_t acc_full = w_full + 16;           // [2] accumulator set complete
  const uint32_t acc_empty = acc_full + 16;        // [2] accumulator set stored
  const uint32_t sched_full = acc_empty + 16;      // [SCHED_SLOTS] next work item published
  const uint32_t sched_empty = sched_full + 8 * SCHED_SLOTS;
  uint8_t *sched_ring = smem_gen + SM::SCHED_OFF;
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + SM::MISC_OFF);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + SM::MISC_OFF + 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  WaitCtx wc{abort_flag, p.status};
#ifdef B200_HSTU_TRACE_BUILD
  const uint64_t cta_t0 = p.trace != nullptr ? globaltimer_ns() : 0;
#endif

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int x = 0; x < 2; ++x) {
      mbar_init(x_full + 8 * x, 1);
      mbar_init(x_empty + 8 * x, 1);
    }
    for (int s = 0; s < Y0_STAGES; ++s) {
      mbar_init(y0_full + 8 * s, 1);
      mbar_init(y0_empty + 8 * s, 1);
    }
    for (int s = 0; s < Y1_STAGES; ++s) {
      mbar_init(y1_full + 8 * s, 1);
      mbar_init(y1_empty + 8 * s, 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(t_full + 8 * x, 1);
      mbar_init(w_full + 8 * x, 8);
      mbar_init(acc_full + 8 * x, 1);
      mbar_init(acc_empty + 8 * x, 4);
    }
    for (int x = 0; x < SCHED_SLOTS; ++x) {
      mbar_init(sched_full + 8 * x, 1);
      mbar_init(sched_empty + 8 * x, BWD_SCHED_CONSUMERS);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns: TS [0,128) scores (S^T | S) then P, TP [128,256) dP (dP^T | dP) then dS,
  //   ACC0 [256,384), ACC1 [384,512);  kv-stationary: ACC0 = dV, ACC1 = dK (one set);
  //   q-stationary: ACC0 / ACC1 = dQ of even / odd items (two sets)
  // Everything above overlapped with the kernel before this one in the stream.  The kv-stationary
  // launch follows the planning kernel and waits for its lists here.  The q-stationary launch
  // follows the kv-stationary one, whose outputs it does not touch and which has seen the lists
  // complete: it starts working at once, on SMs that the first launch's CTAs have left, and only
  // waits for that launch at its very end, so that the stream order of completion is kept.
  if (DKDV) grid_dependency_wait();
  allow_dependents();
  const int num_items = p.plan->num_items * p.H;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && (int)blockIdx.x < num_items) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v); prefetch_tmap(&tmap_do);
      uint32_t it_cnt = 0, cnt = 0;
      bool ok = true;
      Tracer tr;
      tr.init(p.trace, 0, true);
      ItemGeom g;
      {
        TileItem it;
        fill_bwd_item<DKDV>(it, p.g, load_desc(p.items, blockIdx.x / p.H));
        geom_from_item(g, it, blockIdx.x);
      }
      ok = geom_publish(wc, sched_ring, sched_full, sched_empty, 0, g);
      while (g.idx < num_items && ok) {
        // The next (item, head) index is claimed while this item's tiles are requested: the
        // atomic goes out after the first requests, its result is first read one tile later (to
        // fetch the item's descriptor) and the geometry is computed and published another tile
        // later - the round trips never sit between two items' requests.
        int nidx = num_items;
        ItemDesc nd;
        const int h = g.idx % p.H;
        const int n_req = g.n_tiles;
        const int j_desc = n_req > 1 ? 1 : 0, j_geom = n_req > 2 ? 2 : n_req - 1;
        ItemGeom ng = g;
        tr.mark(1);
        // order of requests = order of first use: X0, Y0(0) feed G1; X1, Y1(0) feed G2
        for (int j = 0; j < g.n_tiles; ++j, ++cnt) {
          const int s0 = cnt % Y0_STAGES, s1 = cnt % Y1_STAGES;
          const int row = g.start + g.tile_at(j) * TILE;
          if (j == 0) {
            ok = mbar_wait(wc, x_empty, (it_cnt & 1) ^ 1, 401);
            if (!ok) break;
            tr.mark(2);
            mbar_arrive_expect_tx(x_full, SM::TILE_BYTES);
#pragma unroll
            for (int c = 0; c < SM::CHUNKS; ++c)
              tma_load_2d(sX0 + c * SM::CHUNK_BYTES, mapX0, h * D + c * 64, g.start + g.m0, x_full);
          }
          ok = mbar_wait(wc, y0_empty + 8 * s0, ((cnt / Y0_STAGES) & 1) ^ 1, 402);
          if (!ok) break;
          tr.mark(3);
          mbar_arrive_expect_tx(y0_full + 8 * s0, SM::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < SM::CHUNKS; ++c)
            tma_load_2d(sY0 + s0 * SM::TILE_BYTES + c * SM::CHUNK_BYTES, mapY0, h * D + c * 64, row, y0_full + 8 * s0);
          if (j == 0) {
            ok = mbar_wait(wc, x_empty + 8, (it_cnt & 1) ^ 1, 404);
            if (!ok) break;
            tr.mark(4);
            mbar_arrive_expect_tx(x_full + 8, SM::TILE_BYTES);
#pragma unroll
            for (int c = 0; c < SM::CHUNKS; ++c)
              tma_load_2d(sX1 + c * SM::CHUNK_BYTES, mapX1, h * D + c * 64, g.start + g.m0, x_full + 8);
          }
          ok = mbar_wait(wc, y1_empty + 8 * s1, ((cnt / Y1_STAGES) & 1) ^ 1, 403);
          if (!ok) break;
          mbar_arrive_expect_tx(y1_full + 8 * s1, SM::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < SM::CHUNKS; ++c)
            tma_load_2d(sY1 + s1 * SM::TILE_BYTES + c * SM::CHUNK_BYTES, mapY1, h * D + c * 64, row, y1_full + 8 * s1);
          if (j == 0) nidx = atomicAdd(&p.plan->next, 1);
          if (j == j_desc && nidx < num_items) nd = load_desc(p.items, nidx / p.H);
          if (j == j_geom) {
            ng.idx = nidx;
            if (nidx < num_items) {
              TileItem ni;
              fill_bwd_item<DKDV>(ni, p.g, nd);
              geom_from_item(ng, ni, nidx);
            }
            ok = geom_publish(wc, sched_ring, sched_full, sched_empty, it_cnt + 1, ng);
            if (!ok) break;
          }
        }
        if (!ok) break;
        ++it_cnt;
        g = ng;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (warp-uniform)
    if ((int)blockIdx.x < num_items) {
      constexpr uint32_t FMT = IS_BF16 ? 1u : 0u;
      const uint32_t idesc_1 = make_idesc(FMT, FMT, 0, 0, TILE, TILE);  // 128 x 128, both operands K-major
      const uint32_t idesc_2 = make_idesc(FMT, FMT, 0, 1, TILE, D);     // 128 x D, TMEM A, MN-major B
      uint32_t it_cnt = 0, cnt = 0;
      bool ok = true;
      Tracer tr;
      tr.init(p.trace, 1, lane == 0);

      // G1 (which = 0: TS = X0 Y0^T) or G2 (which = 1: TP = X1 Y1^T) of streamed tile number
      // `tile_no`.  `first_of` >= 0: first tile of item number first_of, whose stationary tile has
      // to have arrived; `last`: last tile of its item, after which that tile has no reader left.
      auto stage1 = [&](int which, uint32_t tile_no, int first_of, bool last) -> bool {
        const int stages = which == 0 ? Y0_STAGES : Y1_STAGES;
        const int s = tile_no % stages;
        Stage1Args a;
        a.x_bar = first_of >= 0 ? x_full + 8 * which : 0u;
        a.x_par = first_of & 1;
        a.y_bar = (which == 0 ? y0_full : y1_full) + 8 * s;
        a.y_par = (tile_no / stages) & 1;
        a.x_desc = make_smem_desc(which == 0 ? sX0 : sX1, 16, 1024);
        a.y_smem = (which == 0 ? sY0 : sY1) + s * SM::TILE_BYTES;
        a.d_tmem = tmem_base + which * 128;
        a.idesc = idesc_1;
        a.commit_t = t_full + 8 * which;
        // q-stationary launch: stage 2 does not read V again, its slot can be refilled already
        a.commit_y = (!DKDV && which == 1) ? y1_empty + 8 * s : 0u;
        a.commit_x = last ? x_empty + 8 * which : 0u;
        return bwd_stage1<D>(wc, a);
      };

      ItemGeom g;
      ok = geom_fetch(wc, sched_ring, sched_full, sched_empty, 0, g, lane == 0);
      bool pre_issued = false;  // G1 / G2 of this item's first tile were issued while the previous item finished
      for (; ok && g.idx < num_items; ++it_cnt) {
        const int n = g.n_tiles;
        tr.mark(10);
        // accumulator of G4 and how often it has been used before: dK is always ACC1 (dV, from G3,
        // always ACC0); dQ alternates between the two
        const int aset = DKDV ? 1 : (int)(it_cnt & 1);
        const uint32_t ause = DKDV ? it_cnt : (it_cnt >> 1);
        if (!pre_issued) {
          ok = stage1(0, cnt, (int)it_cnt, n == 1) && stage1(1, cnt, (int)it_cnt, n == 1);
          if (!ok) break;
        }
        pre_issued = false;
        ItemGeom ng;
        ng.idx = num_items;
        bool next_item = false;
        for (int j = 0; j < n; ++j, ++cnt) {
          const int s0 = cnt % Y0_STAGES, s1 = cnt % Y1_STAGES;
          const bool has_next = j + 1 < n;
          const uint32_t acc_on = j > 0 ? 1u : 0u;
          // ---- scores consumed (P written): G3, then the next scores
          tr.mark(12);
          ok = mbar_wait(wc, w_full, cnt & 1, 505);
          if (!ok) break;
          tc_fence_after();
          tr.mark(14);
          if (DKDV) {
            if (j == 0) {  // dV of the previous item must have been stored
              ok = mbar_wait(wc, acc_empty, (it_cnt & 1) ^ 1, 504);
              if (!ok) break;
            }
            // dV += P^T dO; afterwards the dO tile has no reader left
            bwd_stage2(tmem_base + 256, tmem_base, sY1 + s1 * SM::TILE_BYTES, idesc_2, acc_on, y1_empty + 8 * s1,
                       has_next ? 0u : acc_full);
          }
          tr.mark(16);
          // What follows this tile: the item's next tile, or - at the item's last tile, when the
          // score region is free from here on - the first tile of the next item, whose stationary
          // tiles were requested as soon as this item's last G1 / G2 had been issued.  G1 of it is
          // issued now, G2 after this tile's G4.  The kv-stationary launch, whose code is the
          // largest, serves both cases from one issue site; the q-stationary launch is faster with
          // two.
          bool issue_next = has_next;
          int first_of = -1;
          bool next_last = j == n - 2;
          if (!has_next) {
            ok = geom_fetch(wc, sched_ring, sched_full, sched_empty, it_cnt + 1, ng, lane == 0);
            if (!ok) break;
            if (ng.idx < num_items) {
              next_item = true;
              issue_next = true;
              first_of = (int)it_cnt + 1;
              next_last = ng.n_tiles == 1;
            }
          }
          if (DKDV) {
            if (issue_next) {
              ok = stage1(0, cnt + 1, first_of, next_last);
              if (!ok) break;
            }
          } else if (has_next) {
            ok = stage1(0, cnt + 1, -1, j == n - 2);
            if (!ok) break;
          } else if (next_item) {
            ok = stage1(0, cnt + 1, (int)it_cnt + 1, ng.n_tiles == 1);
            if (!ok) break;
          }
          // ---- dS written: G4, then the next dP
          tr.mark(13);
          ok = mbar_wait(wc, w_full + 8, cnt & 1, 506);
          if (!ok) break;
          tc_fence_after();
          tr.mark(15);
          if (j == 0) {  // the previous user of this accumulator (dK | dQ of the item before last) must have been stored
            ok = mbar_wait(wc, acc_empty + 8 * aset, (ause & 1) ^ 1, 507);
            if (!ok) break;
          }
          // dK += dS^T Q  |  dQ += dS K; afterwards the Q | K tile has no reader left
          bwd_stage2(tmem_base + 256 + aset * 128, tmem_base + 128, sY0 + s0 * SM::TILE_BYTES, idesc_2, acc_on,
                     y0_empty + 8 * s0, has_next ? 0u : acc_full + 8 * aset);
          tr.mark(17);
          if (DKDV) {
            if (issue_next) {
              ok = stage1(1, cnt + 1, first_of, next_last);
              if (!ok) break;
              if (!has_next) pre_issued = true;
            }
          } else if (has_next) {
            ok = stage1(1, cnt + 1, -1, j == n - 2);
            if (!ok) break;
          } else if (next_item) {
            ok = stage1(1, cnt + 1, (int)it_cnt + 1, ng.n_tiles == 1);
            if (!ok) break;
            pre_issued = true;
          }
        }
        if (!ok) break;
        g = ng;
      }
    }
  } else if (warp < 10) {
    // ------------------------------------------------------------------ activation warps
    // thread = one row of the stationary tile; warps 2-5 take columns [0,64) of the streamed tile,
    // warps 6-9 columns [64,128), each in two chunks of 32
    const int wg = warp >= 6 ? 1 : 0;
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;  // stationary-tile row owned by this thread
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const uint32_t tS = tmem_base + lane_off + wg * 64;        // this thread's score columns; P goes over them
    const uint32_t tP = tmem_base + 128 + lane_off + wg * 64;  // this thread's dP columns; dS goes over them
    uint32_t cnt = 0, item_no = 0;
    bool ok = true;
    Tracer tr;
    tr.init(p.trace, 2, warp == 2 && lane == 0);
    if ((int)blockIdx.x < num_items) {
      ItemGeom g;
      ok = geom_fetch(wc, sched_ring, sched_full, sched_empty, 0, g, lane == 0);
      while (ok && g.idx < num_items) {
        TileItem it;
        item_from_geom(it, g, p.g);
        const int L = it.m.L;
        const int own = it.m0 + row_in_tile;  // kv position (DKDV) or query position
        const bool exact_only = !it.regular;
        for (int j = 0; j < it.n_tiles && ok; ++j, ++cnt) {
          // The thread's mask interval is worked out again for every tile although it only depends
          // on the item: code that runs once per item is fetched cold (several thousand cycles of
          // instruction-cache misses per item), code inside the tile loop stays resident.
          int own_j = own;
          asm volatile("" : "+r"(own_j));   // keeps the compiler from hoisting it out of the loop
          ColInterval ci;
          RowInterval ri;
          if (DKDV) ci = col_interval(it, own_j); else ri = row_interval(it, own_j);
          const int o0 = it.tile_at(j) * TILE;  // first position of the streamed tile
          const int c0 = o0 + wg * 64;  // first streamed position of this thread's 64 columns
          ActTile at;
          at.tS = tS;
          at.tP = tP;
          at.t_full = t_full;
          at.w_full = w_full;
          at.parity = cnt & 1;
          at.half_alpha = p.half_alpha;
          at.lane = lane;
          // signed distance query - key of (own row / column, first streamed position)
          at.bias_at = BIAS ? p.bias_ext + (DKDV ? c0 - own : own - c0) : nullptr;
          // only the bias instantiation of the q-stationary launch carries the bias-gradient code
          at.dbias = (BIAS && !DKDV) ? p.dbias : nullptr;
          at.dbias_numel = p.bias_numel;
          at.sc_ptr = p.attn_scale;
          at.inv_n = p.inv_n;
          at.row_valid = own < L;
          if (!exact_only) {
            // one code path for fully and partially visible tiles: the tensor pipe, not the
            // activation, bounds this kernel, and code that runs once per item is slow to fetch
            // kv-stationary launch: the interval mask is all ones on a fully visible tile, no separate
            // test for those (it would evaluate the tile pair); q-stationary launch: the test is
            // cheap and saves the mask words
            uint32_t b0, b1;
            if (DKDV) {
              b0 = col_mask_bits(ci, c0, L);
              b1 = col_mask_bits(ci, c0 + 32, L);
            } else {
              const bool full = tile_pair_is_full(it, o0);
              b0 = full ? 0xffffffffu : row_mask_bits(ri, c0, L);
              b1 = full ? 0xffffffffu : row_mask_bits(ri, c0 + 32, L);
            }
            ok = act_tile_body<IS_BF16, DKDV, 1, BIAS>(wc, at, b0, b1, it.m, own, c0, nullptr, 0, tr);
          } else {
            ok = act_tile_exact<IS_BF16, DKDV>(wc, at, it.m, own, c0, p.bias, p.bias_numel);
          }
        }
        if (!ok) break;
        ++item_no;
        ok = geom_fetch(wc, sched_ring, sched_full, sched_empty, item_no, g, lane == 0);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    // accumulators (fp32, TMEM) -> scale -> 16-bit -> global; thread = one row of the stationary tile
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    uint32_t it_cnt = 0;
    bool ok = true;
    Tracer tr;
    tr.init(p.trace, 3, warp == 10 && lane == 0);
    const float sc = p.attn_scale ? p.attn_scale[0] : p.inv_n;
    if ((int)blockIdx.x < num_items) {
      ItemGeom g;
      ok = geom_fetch(wc, sched_ring, sched_full, sched_empty, 0, g, lane == 0);
      while (ok && g.idx < num_items) {
        const int h = g.idx % p.H;
        const int L = g.L;
        const int own = g.m0 + row_in_tile;
        const bool rv = own < L;
        tr.mark(40);
        if (DKDV) {
          // dV (ACC0) is complete after the item's last G3, dK (ACC1) after its last G4; each is
          // handed back as soon as it has been stored
          uint16_t *dvrow = reinterpret_cast<uint16_t *>(p.dv) + (int64_t)(g.start + own) * p.dv_rs + (int64_t)h * p.dv_hs;
          uint16_t *dkrow = reinterpret_cast<uint16_t *>(p.dk) + (int64_t)(g.start + own) * p.dk_rs + (int64_t)h * p.dk_hs;
          // one copy of the store code serves both accumulators
#pragma unroll 1
          for (int acc = 0; acc < 2 && ok; ++acc) {
            ok = mbar_wait(wc, acc_full + 8 * acc, it_cnt & 1, 602 + acc);
            if (!ok) break;
            tc_fence_after();
            store_acc_rows<D, IS_BF16>(tmem_base + 256 + acc * 128 + lane_off, acc ? sc * p.alpha : sc,
                                       acc ? dkrow : dvrow, rv, p.wide_stores != 0);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + 8 * acc);
          }
          if (!ok) break;
        } else {
          const int aset = (int)(it_cnt & 1);
          uint16_t *dqrow = reinterpret_cast<uint16_t *>(p.dq) + (int64_t)(g.start + own) * p.dq_rs + (int64_t)h * p.dq_hs;
          ok = mbar_wait(wc, acc_full + 8 * aset, (it_cnt >> 1) & 1, 602);
          if (!ok) break;
          tc_fence_after();
          tr.mark(41);
          store_acc_rows<D, IS_BF16>(tmem_base + 256 + aset * 128 + lane_off, sc * p.alpha, dqrow, rv, p.wide_stores != 0);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty + 8 * aset);
        }
        tr.mark(42);
        if (g.len > L && g.m0 + TILE >= L) {
          if (DKDV) {
            zero_rows_beyond<D>(reinterpret_cast<uint16_t *>(p.dk), p.dk_rs, p.dk_hs, h, g.start, L, g.len, row_in_tile);
            zero_rows_beyond<D>(reinterpret_cast<uint16_t *>(p.dv), p.dv_rs, p.dv_hs, h, g.start, L, g.len, row_in_tile);
          } else {
            zero_rows_beyond<D>(reinterpret_cast<uint16_t *>(p.dq), p.dq_rs, p.dq_hs, h, g.start, L, g.len, row_in_tile);
          }
        }
        ++it_cnt;
        ok = geom_fetch(wc, sched_ring, sched_full, sched_empty, it_cnt, g, lane == 0);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 20000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (!DKDV) grid_dependency_wait();
#ifdef B200_HSTU_TRACE_BUILD
  // timeline: start and end time of every CTA (second half of the last role's records)
  if (p.trace != nullptr && threadIdx.x == 0 && blockIdx.x < TRACE_RECORDS / 2)
    p.trace[3 * TRACE_RECORDS + TRACE_RECORDS / 2 + blockIdx.x] = make_ulonglong2(cta_t0, globaltimer_ns());
#endif
}

}  // namespace

// scratch: two work lists (kv-stationary and q-stationary)
int64_t attn_tc_bwd_workspace_bytes(const b200_hstu_attn_args &a) {
  return bias_table_bytes(a.bias_by_distance, a.max_seq_len) + 2 * plan_bytes(a.total_L, a.B);
}

template <int D, bool IS_BF16, bool BIAS>
int launch_bwd_tc(const b200_hstu_attn_args &a, cudaStream_t st) {
  using SM = BwdSmem<D>;
  if (a.workspace == nullptr || a.workspace_bytes < attn_tc_bwd_workspace_bytes(a))
    return fail(B200_HSTU_EWORKSPACE, "attention backward needs %lld bytes of scratch, got %lld",
                (long long)attn_tc_bwd_workspace_bytes(a), (long long)a.workspace_bytes);
  CUtensorMap mq, mk, mv, mdo;
  int rc;
  const int64_t cols = (int64_t)a.H * D;
  if ((rc = make_tile_map_rows(&mq, a.q, a.total_L, cols, a.q_row_stride, 2, IS_BF16, TILE)) != 0) return rc;
  if ((rc = make_tile_map_rows(&mk, a.k, a.total_L, cols, a.k_row_stride, 2, IS_BF16, TILE)) != 0) return rc;
  if ((rc = make_tile_map_rows(&mv, a.v, a.total_L, cols, a.v_row_stride, 2, IS_BF16, TILE)) != 0) return rc;
  if ((rc = make_tile_map_rows(&mdo, a.dout, a.total_L, cols, a.do_row_stride, 2, IS_BF16, TILE)) != 0) return rc;
  BwdParams p;
  p.g.seq_offsets = a.seq_offsets;
  p.g.num_targets = a.num_targets;
  p.g.B = a.B;
  p.g.H = a.H;
  p.g.max_seq_len = a.max_seq_len;
  p.g.W = a.max_attn_len;
  p.g.c = a.contextual_seq_len;
  p.g.F = a.min_full_attn_seq_len;
  p.g.delta = 0;
  p.dq = a.dq; p.dk = a.dk; p.dv = a.dv_;
  p.dq_rs = a.dq_row_stride; p.dq_hs = a.dq_head_stride;
  p.dk_rs = a.dk_row_stride; p.dk_hs = a.dk_head_stride;
  p.dv_rs = a.dv_row_stride; p.dv_hs = a.dv_head_stride;
  p.attn_scale = a.attn_scale;
  p.bias = a.bias_by_distance;
  p.bias_numel = a.bias_numel;
  const int64_t eb = bias_table_bytes(a.bias_by_distance, a.max_seq_len);
  BiasTable bt{a.bias_by_distance, a.bias_numel, reinterpret_cast<float *>(a.workspace), a.max_seq_len};
  p.bias_ext = a.bias_by_distance ? bt.centre() : nullptr;
  p.dbias = a.bias_by_distance ? a.d_bias_by_distance : nullptr;
  p.half_alpha = 0.5f * a.alpha;
  p.alpha = a.alpha;
  p.inv_n = 1.f / (float)a.max_seq_len;
  p.H = a.H;
  {
    auto al32 = [](const void *q, int64_t rs, int64_t hs) {
      return (reinterpret_cast<uintptr_t>(q) & 31) == 0 && rs % 16 == 0 && hs % 16 == 0;
    };
    p.wide_stores = al32(a.dq, a.dq_row_stride, a.dq_head_stride) && al32(a.dk, a.dk_row_stride, a.dk_head_stride) &&
                    al32(a.dv_, a.dv_row_stride, a.dv_head_stride);
  }
  p.trace = nullptr;
  const int max_items = (int)plan_max_items(a.total_L, a.B);
  const int64_t one = plan_bytes(a.total_L, a.B);
  // B200_HSTU_TRACE=dkdv|dq and a scratch buffer with TRACE_BYTES of extra room: CTA 0 of that
  // launch records a timeline of its roles behind the work lists (a profiling aid, off by default)
  static const char *want_trace = getenv("B200_HSTU_TRACE");
  ulonglong2 *trace_buf = nullptr;
  if (want_trace != nullptr && a.plan_mode != B200_HSTU_PLAN_REUSE && a.workspace_bytes >= eb + 2 * one + TRACE_BYTES)
    trace_buf = reinterpret_cast<ulonglong2 *>(reinterpret_cast<uint8_t *>(a.workspace) + eb + 2 * one);
  const int64_t upper = (int64_t)max_items * a.H;
  const int grid = (int)(upper < device_sm_count() ? upper : device_sm_count());
  // own scratch: [bias table | kv list | q list]; planned by the forward: [bias table | forward
  // list | kv list | q list] (the table is the forward's too)
  const bool reuse = a.plan_mode == B200_HSTU_PLAN_REUSE;
  if (reuse && a.workspace_bytes < eb + 3 * one)
    return fail(B200_HSTU_EWORKSPACE, "backward reusing the forward's lists expects its %lld-byte scratch, got %lld",
                (long long)(eb + 3 * one), (long long)a.workspace_bytes);
  uint8_t *ws = reinterpret_cast<uint8_t *>(a.workspace) + eb + (reuse ? one : 0);
  PlanHeader *hdr_kv = reinterpret_cast<PlanHeader *>(ws);
  PlanHeader *hdr_q = reinterpret_cast<PlanHeader *>(ws + one);
  if (!reuse) {
    {
      ProfileScope prof(PROF_PLAN, st);
      attn_plan2_kernel<PLAN_KV_TILE, PLAN_Q_TILE><<<2, PLAN_THREADS, 0, st>>>(
          p.g, hdr_kv, reinterpret_cast<ItemDesc *>(hdr_kv + 1), hdr_q, reinterpret_cast<ItemDesc *>(hdr_q + 1),
          max_items, grid, bt);
    }
    count_launch();
    B200_CHECK_LAUNCH("attention plan (backward)");
  }
  {
    auto kern = hstu_attn_bwd_sm100_kernel<D, IS_BF16, true, BIAS>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::DYN_BYTES);
    if (e != cudaSuccess) return check_cuda(e, "backward smem attribute");
    BwdParams pk = p;
    pk.plan = hdr_kv;
    pk.items = reinterpret_cast<ItemDesc *>(hdr_kv + 1);
    pk.status = &hdr_kv->status;
    if (trace_buf != nullptr && want_trace[0] == 'd' && want_trace[1] == 'k') pk.trace = trace_buf;
    ProfileScope prof(PROF_ATTN_BWD_DKDV, st);
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr;
    fill_pdl_config(&cfg, &attr, grid, BWD_THREADS, SM::DYN_BYTES, st);
    e = cudaLaunchKernelEx(&cfg, kern, mq, mk, mv, mdo, pk);
    if (e != cudaSuccess) return check_cuda(e, "backward (dk, dv) launch");
    count_launch();
    B200_CHECK_LAUNCH("tcgen05 attention backward (dk, dv)");
  }
  {
    auto kern = hstu_attn_bwd_sm100_kernel<D, IS_BF16, false, BIAS>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::DYN_BYTES);
    if (e != cudaSuccess) return check_cuda(e, "backward smem attribute");
    BwdParams pq = p;
    pq.plan = hdr_q;
    pq.items = reinterpret_cast<ItemDesc *>(hdr_q + 1);
    pq.status = &hdr_q->status;
    if (trace_buf != nullptr && want_trace[0] == 'd' && want_trace[1] == 'q') pq.trace = trace_buf;
    ProfileScope prof(PROF_ATTN_BWD_DQ, st);
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr;
    fill_pdl_config(&cfg, &attr, grid, BWD_THREADS, SM::DYN_BYTES, st);
    e = cudaLaunchKernelEx(&cfg, kern, mq, mk, mv, mdo, pq);
    if (e != cudaSuccess) return check_cuda(e, "backward (dq) launch");
    count_launch();
    B200_CHECK_LAUNCH("tcgen05 attention backward (dq)");
  }
  return 0;
}

int attn_tc_bwd(const b200_hstu_attn_args &a, cudaStream_t st) {
  const bool bf = a.dtype == B200_HSTU_BF16;
  // a relative bias has its own instantiation, so that the common case carries none of its code
  if (a.bias_by_distance != nullptr) {
    if (a.dqk == 128) return bf ? launch_bwd_tc<128, true, true>(a, st) : launch_bwd_tc<128, false, true>(a, st);
    return bf ? launch_bwd_tc<64, true, true>(a, st) : launch_bwd_tc<64, false, true>(a, st);
  }
  if (a.dqk == 128) return bf ? launch_bwd_tc<128, true, false>(a, st) : launch_bwd_tc<128, false, false>(a, st);
  return bf ? launch_bwd_tc<64, true, false>(a, st) : launch_bwd_tc<64, false, false>(a, st);
}

}  // namespace b200hstu
