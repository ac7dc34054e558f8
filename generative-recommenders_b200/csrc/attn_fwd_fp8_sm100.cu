// Jagged HSTU attention forward with FP8 (e4m3) q / k / v and per-block scales, for inference.
//
// q8, k8, v8 are e4m3 with one fp32 scale per (128-token block counted from the start of the
// sequence, head); the output is bf16.  The kernel has the structure of the bf16 forward (pairs of
// 128-row query tiles per CTA, TMA rings, TMEM accumulators, two activation warpgroups), with:
//   * S = Q8 K8^T as kind::f8f6f4 MMAs (K = 32 per instruction).  Because a scale block is exactly
//     one 128-row tile, the de-scaling is one scalar per (query tile, kv tile):
//     x = alpha * sq[q block] * sk[k block] * S.
//   * P = SiLU(x) is written back to TMEM as a pair of e4m3 tiles, P ~ P_hi + P_lo (P_lo is the
//     e4m3 rounding of the residual), so that P keeps about 8 bits; O += P_hi V8 + P_lo V8 are two
//     fp8 MMAs on the same V tile (V8 is the MN-major B operand).
//   * V's block scale is folded into P before the split, relative to the scale of the query
//     tile's own block, times a constant that lifts typical activations into e4m3's normal range:
//     P' = SiLU(x) * (sv[k block] / sv_ref) * 16;  out = O * sv_ref / 16 / max_seq_len.
// Shared memory traffic per kv tile is about 60 % of the bf16 kernel's (1-byte operands).
#include <stdlib.h>

#include "attn_plan.cuh"
#include "sm100_ptx.cuh"

namespace b200hstu {

using namespace ptx;

int make_tile_map(CUtensorMap *m, const void *base, int64_t rows, int64_t cols, int64_t row_stride_elems,
                  int elem_bytes, bool is_bf16);
int device_sm_count();

namespace {

constexpr int FWD_THREADS = 320;
constexpr int KV_STAGES = 4;

struct Fp8Params {
  AttnGeomParams g;
  const PlanHeader *plan;
  const ItemDesc *items;
  int *status;
  void *out;
  int64_t o_rs, o_hs;
  const float *attn_scale;
  int64_t attn_scale_numel;
  const float *bias;
  int bias_numel;
  float half_alpha;   // alpha / 2
  float inv_n;        // 1 / max_seq_len
  int H;
  const float *q_scale, *k_scale, *v_scale;  // [n_blocks_total, H]
  const int32_t *block_offsets;              // [B + 1]
  // optional timeline of CTA 0 (4 roles x TRACE_RECORDS records of {ns, tag}); NULL = off
  ulonglong2 *trace;
};

constexpr int TRACE_RECORDS = 1024;
constexpr int64_t TRACE_BYTES = 4 * TRACE_RECORDS * (int64_t)sizeof(ulonglong2);

struct Tracer {
  ulonglong2 *buf;
  int n;
  __device__ __forceinline__ void init(ulonglong2 *base, int role, bool on) {
    buf = (base != nullptr && on && blockIdx.x == 0) ? base + role * TRACE_RECORDS : nullptr;
    n = 0;
  }
  __device__ __forceinline__ void mark(unsigned tag) {
    if (buf != nullptr && n < TRACE_RECORDS) buf[n++] = make_ulonglong2(globaltimer_ns(), tag);
  }
};

constexpr float P_LIFT = 16.f;   // constant that lifts activations into e4m3's normal range

template <int D>
struct FwdSmem {
  static_assert(D == 128, "the fp8 forward is built for head dimension 128");
  static constexpr int CHUNKS = 1;                      // a row is 128 bytes = one TMA box
  static constexpr int TILE_BYTES = TILE * D;           // one Q / K / V tile of e4m3
  static constexpr int CHUNK_BYTES = TILE * 128;        // 128 rows x 128 bytes
  static constexpr int Q_OFF = 0;                       // Q_A, Q_B
  static constexpr int K_OFF = Q_OFF + 2 * TILE_BYTES;
  static constexpr int V_OFF = K_OFF + KV_STAGES * TILE_BYTES;
  static constexpr int BAR_OFF = V_OFF + KV_STAGES * TILE_BYTES;
  static constexpr int NUM_BARS = 2 + 4 * KV_STAGES + 8;
  static constexpr int MISC_OFF = BAR_OFF + NUM_BARS * 8;
  static constexpr int TOTAL = MISC_OFF + 64;
  // slack for manual 1024-byte alignment; at least 116 KB so that two CTAs (each of which
  // allocates all 512 TMEM columns) can never share an SM
  static constexpr int DYN_BYTES = (TOTAL + 1024) > 116 * 1024 ? (TOTAL + 1024) : 116 * 1024;
};

__device__ __forceinline__ uint32_t pack2_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&v);
}

// two fp32 -> f16x2 (first argument in the low half)
__device__ __forceinline__ uint32_t to_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint16_t f16x2_to_e4m3x2(uint32_t v) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint16_t v) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
  return r;
}

// 32 scores -> 8 words of P_hi and 8 words of P_lo (4 e4m3 per word).
// silu(x) = h + h tanh(h), h = x / 2, on packed f16 pairs; `gain2` = f16x2 of the lift factor.
template <bool MASKED>
__device__ __forceinline__ void silu_chunk_fp8(const uint32_t (&r)[32], uint32_t (&hi)[8], uint32_t (&lo)[8],
                                               float half_alpha, uint32_t gain2, uint32_t bits) {
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    uint16_t h16[2], l16[2];
#pragma unroll
    for (int y = 0; y < 2; ++y) {
      const int x = 4 * w + 2 * y;
      float h0 = __uint_as_float(r[x]) * half_alpha;
      float h1 = __uint_as_float(r[x + 1]) * half_alpha;
      h0 = fminf(fmaxf(h0, -30000.f), 30000.f);
      h1 = fminf(fmaxf(h1, -30000.f), 30000.f);
      if (MASKED) {
        h0 = (bits & (1u << x)) ? h0 : 0.f;
        h1 = (bits & (1u << (x + 1))) ? h1 : 0.f;
      }
      uint32_t hh = to_f16x2(h0, h1), t, pp, back, res;
      asm("tanh.approx.f16x2 %0, %1;" : "=r"(t) : "r"(hh));
      asm("fma.rn.f16x2 %0, %1, %2, %1;" : "=r"(pp) : "r"(hh), "r"(t));
      asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(pp) : "r"(pp), "r"(gain2));
      h16[y] = f16x2_to_e4m3x2(pp);
      back = e4m3x2_to_f16x2(h16[y]);
      asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(res) : "r"(pp), "r"(back));
      l16[y] = f16x2_to_e4m3x2(res);
    }
    hi[w] = (uint32_t)h16[0] | ((uint32_t)h16[1] << 16);
    lo[w] = (uint32_t)l16[0] | ((uint32_t)l16[1] << 16);
  }
}

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

// D[tmem] (+)= A[tmem, e4m3] * B[smem desc, e4m3]
__device__ __forceinline__ void mma_ts_f8(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int D>
__global__ void __launch_bounds__(FWD_THREADS, 1)
    hstu_attn_fwd_fp8_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                               const __grid_constant__ CUtensorMap tmap_v, const Fp8Params p) {
  using SM = FwdSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base + SM::Q_OFF;   // Q_A at sQ, Q_B at sQ + TILE_BYTES
  const uint32_t sK = smem_base + SM::K_OFF;
  const uint32_t sV = smem_base + SM::V_OFF;
  const uint32_t bars = smem_base + SM::BAR_OFF;
  // barrier map
  const uint32_t q_full = bars + 0, q_empty = bars + 8;
  const uint32_t k_full = bars + 16, k_empty = k_full + 8 * KV_STAGES;
  const uint32_t v_full = k_empty + 8 * KV_STAGES, v_empty = v_full + 8 * KV_STAGES;
  const uint32_t s_full = v_empty + 8 * KV_STAGES;   // [2]: S_A, S_B ready
  const uint32_t p_full = s_full + 16;               // [2]: P_A, P_B written
  const uint32_t o_full = p_full + 16;               // [2]: O_A, O_B complete
  const uint32_t o_empty = o_full + 16;              // [2]: O_A, O_B read out
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + SM::MISC_OFF);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + SM::MISC_OFF + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  WaitCtx wc{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(k_full + 8 * s, 1);
      mbar_init(k_empty + 8 * s, 1);
      mbar_init(v_full + 8 * s, 1);
      mbar_init(v_empty + 8 * s, 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(s_full + 8 * x, 1);
      mbar_init(p_full + 8 * x, 4);
      mbar_init(o_full + 8 * x, 1);
      mbar_init(o_empty + 8 * x, 4);
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
  // TMEM columns: S_A [0,128)  S_B [128,256)  O_A [256,384)  O_B [384,512)
  const int num_items = p.plan->num_items * p.H;
  const int stride = gridDim.x;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && (int)blockIdx.x < num_items) {
      prefetch_tmap(&tmap_q);
      prefetch_tmap(&tmap_k);
      prefetch_tmap(&tmap_v);
      uint32_t it_cnt = 0, kv_cnt = 0;
      bool ok = true;
      Tracer tr;
      tr.init(p.trace, 0, true);
      ItemDesc nxt = load_desc(p.items, blockIdx.x / p.H);
      for (int idx = blockIdx.x; idx < num_items && ok; idx += stride, ++it_cnt) {
        const ItemDesc d = nxt;
        if (idx + stride < num_items) nxt = load_desc(p.items, (idx + stride) / p.H);
        const int h = idx % p.H;
        PairItem pr;
        fill_pair_item(pr, p.g, d.b, d.t, d.start, d.len, d.nt);
        tr.mark(1);
        ok = mbar_wait(wc, q_empty, (it_cnt & 1) ^ 1, 101);
        if (!ok) break;
        tr.mark(2);
        mbar_arrive_expect_tx(q_full, (pr.hasB ? 2 : 1) * SM::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < SM::CHUNKS; ++c)
          tma_load_2d(sQ + c * SM::CHUNK_BYTES, &tmap_q, h * D, d.start + pr.A.m0, q_full);
        if (pr.hasB) {
#pragma unroll
          for (int c = 0; c < SM::CHUNKS; ++c)
            tma_load_2d(sQ + SM::TILE_BYTES + c * SM::CHUNK_BYTES, &tmap_q, h * D, d.start + pr.B.m0, q_full);
        }
        for (int j = 0; j < pr.n_tiles; ++j, ++kv_cnt) {
          const int s = kv_cnt % KV_STAGES;
          const uint32_t par = ((kv_cnt / KV_STAGES) & 1) ^ 1;
          const int row = d.start + pr.tile_at(j) * TILE;
          ok = mbar_wait(wc, k_empty + 8 * s, par, 102);
          if (!ok) break;
          tr.mark(3);
          mbar_arrive_expect_tx(k_full + 8 * s, SM::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < SM::CHUNKS; ++c)
            tma_load_2d(sK + s * SM::TILE_BYTES + c * SM::CHUNK_BYTES, &tmap_k, h * D, row, k_full + 8 * s);
          ok = mbar_wait(wc, v_empty + 8 * s, par, 103);
          if (!ok) break;
          tr.mark(4);
          mbar_arrive_expect_tx(v_full + 8 * s, SM::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < SM::CHUNKS; ++c)
            tma_load_2d(sV + s * SM::TILE_BYTES + c * SM::CHUNK_BYTES, &tmap_v, h * D, row, v_full + 8 * s);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // All 32 lanes run the control flow and the barrier waits, so everything that feeds the MMA
    // descriptors stays warp-uniform; one elected lane issues the tcgen05 instructions.
    if ((int)blockIdx.x < num_items) {
      const uint32_t idesc_s = make_idesc(0, 0, 0, 0, TILE, TILE);   // e4m3 x e4m3, both K-major
      const uint32_t idesc_o = make_idesc(0, 0, 0, 1, TILE, D);      // e4m3 P (TMEM) x MN-major e4m3 V
      uint32_t it_cnt = 0, kv_cnt = 0;
      uint32_t tile_cnt[2] = {0, 0};   // S/P tiles processed so far per query tile (barrier phases)
      uint32_t item_cnt[2] = {0, 0};   // items in which the query tile took part
      bool ok = true;
      Tracer tr;
      tr.init(p.trace, 1, lane == 0);

      // S_X = Q_X K^T for kv ring slot of global tile counter g
      auto issue_s = [&](int X, uint32_t g) {
        const int s = g % KV_STAGES;
        const uint64_t q_desc = make_smem_desc(sQ + X * SM::TILE_BYTES, 16, 1024);
        const uint64_t k_desc = make_smem_desc(sK + s * SM::TILE_BYTES, 16, 1024);
        const uint32_t dcol = tmem_base + X * 128;
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < D / 32; ++ks)  // 32 e4m3 = 32 bytes per step inside the 128-byte row
            mma_ss_f8(dcol, desc_advance(q_desc, ks * 32), desc_advance(k_desc, ks * 32), idesc_s, ks > 0);
          tc_commit(s_full + 8 * X);
        }
        __syncwarp();
      };

      ItemDesc nxt = load_desc(p.items, blockIdx.x / p.H);
      for (int idx = blockIdx.x; idx < num_items && ok; idx += stride, ++it_cnt) {
        const ItemDesc d = nxt;
        if (idx + stride < num_items) nxt = load_desc(p.items, (idx + stride) / p.H);
        PairItem pr;
        fill_pair_item(pr, p.g, d.b, d.t, d.start, d.len, d.nt);
        tr.mark(10);
        ok = mbar_wait(wc, q_full, it_cnt & 1, 202);
        if (!ok) break;
        tr.mark(11);
        const int n = pr.n_tiles;
        int remaining[2] = {pr.A.n_tiles, pr.B.n_tiles};
        bool started[2] = {false, false};
        // first kv tile: both S
        {
          const int t0 = pr.tile_at(0);
          ok = mbar_wait(wc, k_full + 8 * (kv_cnt % KV_STAGES), (kv_cnt / KV_STAGES) & 1, 201);
          if (!ok) break;
          tc_fence_after();
          if (pr.A.visits(t0)) issue_s(0, kv_cnt);
          if (pr.hasB && pr.B.visits(t0)) issue_s(1, kv_cnt);
          if (elect_one()) tc_commit(k_empty + 8 * (kv_cnt % KV_STAGES));
          __syncwarp();
        }
        for (int j = 0; j < n; ++j, ++kv_cnt) {
          const int t = pr.tile_at(j);
          const bool has_next = j + 1 < n;
          const int tn = has_next ? pr.tile_at(j + 1) : -1;
          const int s = kv_cnt % KV_STAGES;
          const int sn = (kv_cnt + 1) % KV_STAGES;
          bool v_ready = false, kn_ready = false;
          if (j == n - 1) {  // every S of this item has been issued
            if (elect_one()) tc_commit(q_empty);
            __syncwarp();
          }
#pragma unroll
          for (int X = 0; X < 2; ++X) {
            const TileItem &ti = X == 0 ? pr.A : pr.B;
            const bool here = (X == 0 || pr.hasB) && ti.visits(t);
            const bool next = has_next && (X == 0 || pr.hasB) && ti.visits(tn);
            if (here) {
              if (!started[X]) {  // O_X of the previous item must have been read out
                ok = mbar_wait(wc, o_empty + 8 * X, (item_cnt[X] & 1) ^ 1, 203);
                if (!ok) break;
              }
              tr.mark(12 + X);
              ok = mbar_wait(wc, p_full + 8 * X, tile_cnt[X] & 1, 204);
              if (!ok) break;
              tr.mark(14 + X);
              if (!v_ready) {
                ok = mbar_wait(wc, v_full + 8 * s, (kv_cnt / KV_STAGES) & 1, 205);
                if (!ok) break;
                v_ready = true;
                tr.mark(20);
              }
              tc_fence_after();
              // V tile: [128 kv rows][128 bytes]; 32 kv rows per MMA = 4 KB
              const uint64_t v_desc = make_smem_desc(sV + s * SM::TILE_BYTES, SM::CHUNK_BYTES, 1024);
              const uint32_t a_tmem = tmem_base + X * 128;
              const uint32_t o_tmem = tmem_base + 256 + X * 128;
              const bool last = --remaining[X] == 0;
              if (elect_one()) {
#pragma unroll
                for (int ks = 0; ks < TILE / 32; ++ks)  // P_hi: TMEM columns [0,32) of the S region
                  mma_ts_f8(o_tmem, a_tmem + ks * 8, desc_advance(v_desc, ks * 4096), idesc_o,
                            (started[X] || ks > 0) ? 1u : 0u);
#pragma unroll
                for (int ks = 0; ks < TILE / 32; ++ks)  // P_lo: columns [32,64)
                  mma_ts_f8(o_tmem, a_tmem + 32 + ks * 8, desc_advance(v_desc, ks * 4096), idesc_o, 1u);
                if (last) tc_commit(o_full + 8 * X);
              }
              __syncwarp();
              started[X] = true;
              ++tile_cnt[X];
              if (last) ++item_cnt[X];
            }
            if (next) {
              if (!kn_ready) {
                tr.mark(16);
                ok = mbar_wait(wc, k_full + 8 * sn, ((kv_cnt + 1) / KV_STAGES) & 1, 206);
                if (!ok) break;
                kn_ready = true;
                tc_fence_after();
                tr.mark(17);
              }
              issue_s(X, kv_cnt + 1);
              tr.mark(18 + X);
            }
          }
          if (!ok) break;
          // keep the ring phases in step even if neither tile used this slot
          if (!v_ready) {
            ok = mbar_wait(wc, v_full + 8 * s, (kv_cnt / KV_STAGES) & 1, 207);
            if (!ok) break;
          }
          if (has_next && !kn_ready) {
            ok = mbar_wait(wc, k_full + 8 * sn, ((kv_cnt + 1) / KV_STAGES) & 1, 208);
            if (!ok) break;
          }
          if (elect_one()) {
            tc_commit(v_empty + 8 * s);
            if (has_next) tc_commit(k_empty + 8 * sn);
          }
          __syncwarp();
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ SiLU + epilogue warps
    const int X = warp >= 6 ? 1 : 0;           // query tile A or B
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may touch
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const uint32_t tS = tmem_base + X * 128 + lane_off;
    const uint32_t tO = tmem_base + 256 + X * 128 + lane_off;
    uint32_t my_tiles = 0, my_items = 0;
    bool ok = true;
    Tracer tr;
    tr.init(p.trace, 2 + X, quad == 2 && lane == 0);
    if ((int)blockIdx.x < num_items) {
      ItemDesc nxt = load_desc(p.items, blockIdx.x / p.H);
      for (int idx = blockIdx.x; idx < num_items && ok; idx += stride) {
        const ItemDesc d = nxt;
        if (idx + stride < num_items) nxt = load_desc(p.items, (idx + stride) / p.H);
        const int h = idx % p.H;
        PairItem pr;
        fill_pair_item(pr, p.g, d.b, d.t, d.start, d.len, d.nt);
        if (X == 1 && !pr.hasB) continue;
        const TileItem &it = X == 0 ? pr.A : pr.B;
        const int L = it.m.L;
        const int i = it.m0 + row_in_tile;
        const int id_i = it.m.id(i);
        const RowInterval ri = row_interval(it, i);
        const bool exact_only = !it.regular;
        // block scales: row of this sequence's first block, then one row per 128-token tile
        const int blk0 = p.block_offsets[d.b];
        const float sq = p.q_scale[(int64_t)(blk0 + it.mt) * p.H + h];
        const float sv_ref = p.v_scale[(int64_t)(blk0 + it.mt) * p.H + h];
        const float inv_sv_ref = 1.f / sv_ref;
        float sk_next = 0.f, sv_next = 0.f;
        {
          int jf = 0;
          while (jf < pr.n_tiles && !it.visits(pr.tile_at(jf))) ++jf;
          if (jf < pr.n_tiles) {
            sk_next = p.k_scale[(int64_t)(blk0 + pr.tile_at(jf)) * p.H + h];
            sv_next = p.v_scale[(int64_t)(blk0 + pr.tile_at(jf)) * p.H + h];
          }
        }
        for (int j = 0; j < pr.n_tiles; ++j) {
          const int t = pr.tile_at(j);
          if (!it.visits(t)) continue;
          const int n0 = t * TILE;
          const bool full = !exact_only && tile_pair_is_full(it, n0);
          const float sk = sk_next, sv = sv_next;
          {  // fetch the scales of the next kv tile this query tile visits while working on this one
            int jn = j + 1;
            while (jn < pr.n_tiles && !it.visits(pr.tile_at(jn))) ++jn;
            if (jn < pr.n_tiles) {
              sk_next = p.k_scale[(int64_t)(blk0 + pr.tile_at(jn)) * p.H + h];
              sv_next = p.v_scale[(int64_t)(blk0 + pr.tile_at(jn)) * p.H + h];
            }
          }
          const float ha = p.half_alpha * sq * sk;
          const float gain = sv * inv_sv_ref * P_LIFT;
          const uint32_t gain2 = to_f16x2(gain, gain);
          tr.mark(30);
          ok = mbar_wait(wc, s_full + 8 * X, my_tiles & 1, 301);
          if (!ok) break;
          tc_fence_after();
          tr.mark(31);
          {
            uint32_t sreg[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, sreg[c]);
            tc_wait_ld();
            tr.mark(32);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t hi[8], lo[8];
              uint32_t bits = 0xffffffffu;
              if (!full) {
                if (!exact_only) {
                  bits = row_mask_bits(ri, n0 + c * 32, L);
                } else {  // outside the closed form: evaluate the mask element by element
                  bits = 0;
                  for (int x = 0; x < 32; ++x) {
                    const int jj = n0 + c * 32 + x;
                    if (i < L && jj < L && it.m.valid_ids(i, jj, id_i, it.m.id(jj))) bits |= 1u << x;
                  }
                }
              }
              if (full)
                silu_chunk_fp8<false>(sreg[c], hi, lo, ha, gain2, bits);
              else
                silu_chunk_fp8<true>(sreg[c], hi, lo, ha, gain2, bits);
              tmem_st8(tS + c * 8, hi);
              tmem_st8(tS + 32 + c * 8, lo);
            }
          }
          tr.mark(37);
          tc_wait_st();
          tr.mark(38);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(p_full + 8 * X);
          tr.mark(33);
          ++my_tiles;
        }
        if (!ok) break;
        // epilogue: O (fp32, TMEM) -> scale -> 16-bit -> global, valid rows only
        tr.mark(34);
        ok = mbar_wait(wc, o_full + 8 * X, my_items & 1, 302);
        if (!ok) break;
        tc_fence_after();
        tr.mark(35);
        float scale = p.inv_n;
        if (p.attn_scale != nullptr && i < L)
          scale = p.attn_scale_numel == 1 ? p.attn_scale[0] : p.attn_scale[(int64_t)d.start + i];
        scale *= sv_ref * (1.f / P_LIFT);
        uint16_t *orow = reinterpret_cast<uint16_t *>(p.out) + (int64_t)(d.start + i) * p.o_rs + (int64_t)h * p.o_hs;
#pragma unroll
        for (int c0 = 0; c0 < D / 32; c0 += 2) {
          uint32_t r[2][32];
          tmem_ld32(tO + c0 * 32, r[0]);
          tmem_ld32(tO + c0 * 32 + 32, r[1]);
          tc_wait_ld();
          if (i < L) {
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
#pragma unroll
              for (int x = 0; x < 4; ++x) {
                uint4 o4;
                o4.x = pack2_bf16(__uint_as_float(r[cc][8 * x + 0]) * scale, __uint_as_float(r[cc][8 * x + 1]) * scale);
                o4.y = pack2_bf16(__uint_as_float(r[cc][8 * x + 2]) * scale, __uint_as_float(r[cc][8 * x + 3]) * scale);
                o4.z = pack2_bf16(__uint_as_float(r[cc][8 * x + 4]) * scale, __uint_as_float(r[cc][8 * x + 5]) * scale);
                o4.w = pack2_bf16(__uint_as_float(r[cc][8 * x + 6]) * scale, __uint_as_float(r[cc][8 * x + 7]) * scale);
                *reinterpret_cast<uint4 *>(orow + (c0 + cc) * 32 + x * 8) = o4;
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(o_empty + 8 * X);
        tr.mark(36);
        ++my_items;
        // rows at or beyond max_seq_len of an over-long sequence come back as zeros
        if (d.len > L && it.m0 + TILE >= L) {
          for (int r2 = L + row_in_tile; r2 < d.len; r2 += TILE) {
            uint16_t *zr = reinterpret_cast<uint16_t *>(p.out) + (int64_t)(d.start + r2) * p.o_rs + (int64_t)h * p.o_hs;
            for (int x = 0; x < D; x += 8) *reinterpret_cast<uint4 *>(zr + x) = make_uint4(0, 0, 0, 0);
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ common exit
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // a bounded wait gave up: let any TMA copy still in flight land before the CTA retires
    uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 20000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace

int attn_tc_fwd_fp8(const b200_hstu_attn_fp8_args &fa, cudaStream_t st) {
  constexpr int D = 128;
  using SM = FwdSmem<D>;
  const b200_hstu_attn_args &a = fa.base;
  auto al16 = [](const void *ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
  if (a.dqk != D || a.dv != D) return fail(B200_HSTU_EUNSUPPORTED, "the fp8 forward needs head dimension 128");
  if (a.q_head_stride != D || a.k_head_stride != D || a.v_head_stride != D || a.q_row_stride % 16 ||
      a.k_row_stride % 16 || a.v_row_stride % 16 || !al16(a.q) || !al16(a.k) || !al16(a.v))
    return fail(B200_HSTU_EINVAL, "fp8 q / k / v must have contiguous heads and 16-byte aligned rows");
  if (!al16(a.out) || a.o_row_stride % 8 || a.o_head_stride % 8)
    return fail(B200_HSTU_EINVAL, "out must be 16-byte aligned bf16");
  if (a.bias_by_distance != nullptr) return fail(B200_HSTU_EUNSUPPORTED, "the fp8 forward takes no relative bias");
  const int64_t need = plan_bytes(a.total_L, a.B);
  if (a.workspace == nullptr || a.workspace_bytes < need)
    return fail(B200_HSTU_EWORKSPACE, "fp8 attention forward needs %lld bytes of scratch, got %lld", (long long)need,
                (long long)a.workspace_bytes);
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = make_tile_map(&mq, a.q, a.total_L, (int64_t)a.H * D, a.q_row_stride, 1, false)) != 0) return rc;
  if ((rc = make_tile_map(&mk, a.k, a.total_L, (int64_t)a.H * D, a.k_row_stride, 1, false)) != 0) return rc;
  if ((rc = make_tile_map(&mv, a.v, a.total_L, (int64_t)a.H * D, a.v_row_stride, 1, false)) != 0) return rc;
  Fp8Params p;
  p.g.seq_offsets = a.seq_offsets;
  p.g.num_targets = a.num_targets;
  p.g.B = a.B;
  p.g.H = a.H;
  p.g.max_seq_len = a.max_seq_len;
  p.g.W = a.max_attn_len;
  p.g.c = a.contextual_seq_len;
  p.g.F = a.min_full_attn_seq_len;
  p.g.delta = 0;
  PlanHeader *hdr = reinterpret_cast<PlanHeader *>(a.workspace);
  ItemDesc *items = reinterpret_cast<ItemDesc *>(hdr + 1);
  p.plan = hdr;
  p.items = items;
  p.status = &hdr->status;
  p.out = a.out;
  p.o_rs = a.o_row_stride;
  p.o_hs = a.o_head_stride;
  p.attn_scale = a.attn_scale;
  p.attn_scale_numel = a.attn_scale_numel;
  p.bias = nullptr;
  p.bias_numel = 0;
  p.half_alpha = 0.5f * a.alpha;
  p.inv_n = 1.f / (float)a.max_seq_len;
  p.H = a.H;
  p.q_scale = fa.q_scale;
  p.k_scale = fa.k_scale;
  p.v_scale = fa.v_scale;
  p.block_offsets = fa.block_offsets;
  p.trace = nullptr;
  const int max_items = (int)plan_max_items(a.total_L, a.B);
  {
    ProfileScope prof(PROF_PLAN, st);
    attn_plan_kernel<PLAN_Q_PAIR><<<1, PLAN_THREADS, 0, st>>>(p.g, hdr, items, max_items, 0, BiasTable{nullptr, 0, nullptr, 0});
  }
  count_launch();
  B200_CHECK_LAUNCH("attention plan");
  auto kern = hstu_attn_fwd_fp8_sm100_kernel<D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::DYN_BYTES);
  if (e != cudaSuccess) return check_cuda(e, "fp8 forward smem attribute");
  int64_t upper = (int64_t)max_items * a.H;
  int grid = (int)(upper < device_sm_count() ? upper : device_sm_count());
  {
    ProfileScope prof(PROF_ATTN_FWD_FP8, st);
    kern<<<grid, FWD_THREADS, SM::DYN_BYTES, st>>>(mq, mk, mv, p);
  }
  count_launch();
  B200_CHECK_LAUNCH("tcgen05 fp8 attention forward");
  return 0;
}

}  // namespace b200hstu
