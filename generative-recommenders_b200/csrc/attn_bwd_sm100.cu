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
//   warp 1       MMA issuer; owns TMEM.  Every streamed tile is processed as two 64-column halves
//                (a, b) in the order  stage2_a(i), stage1_a(i+1), stage2_b(i), stage1_b(i+1),  so
//                the tensor pipe works on one half while the CUDA cores activate the other; during
//                the last tile of an item the stage-1 tiles of the next item are issued instead.
//                The stationary tiles are released as soon as the item's last stage 1 is issued.
//   warps 2-9    activation: all eight work on one half at a time, one row of the stationary tile
//                per thread, 32 of the half's 64 columns per warpgroup
//   warps 10-13  epilogue: accumulators (fp32, TMEM) -> scale -> 16-bit -> global
// TMEM: 4 x 64 columns of stage-1 tiles + two 128-column accumulators.  Constant factors are
// folded into the epilogues: dV * scale, dK * scale*alpha, dQ * scale*alpha.
#include <stdlib.h>

#include "attn_plan.cuh"
#include "sm100_ptx.cuh"

namespace b200hstu {

using namespace ptx;

int make_tile_map_rows(CUtensorMap *m, const void *base, int64_t rows, int64_t cols, int64_t row_stride_elems,
                       int elem_bytes, bool is_bf16, int box_rows);
int device_sm_count();

namespace {

constexpr int BWD_THREADS = 448;
constexpr int STAGES = 2;
constexpr int BWD_SCHED_CONSUMERS = 13;  // MMA warp, 8 activation warps, 4 epilogue warps: one arrival each

struct BwdParams {
  AttnGeomParams g;
  PlanHeader *plan;
  const ItemDesc *items;
  int *status;
  void *dq, *dk, *dv;
  int64_t dq_rs, dq_hs, dk_rs, dk_hs, dv_rs, dv_hs;
  const float *attn_scale;  // NULL or one fp32 on the device
  const float *bias;
  int bias_numel;
  float half_alpha, alpha, inv_n;
  int H;
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
  static constexpr int Y_OFF = X_OFF + STAGES * TILE_BYTES;       // streamed ring 1 (dO or V)
  static constexpr int BAR_OFF = Y_OFF + STAGES * TILE_BYTES;
  static constexpr int NUM_BARS = 40;
  static constexpr int MISC_OFF = BAR_OFF + NUM_BARS * 8;
  static constexpr int SCHED_OFF = MISC_OFF + 64;
  static constexpr int TOTAL = SCHED_OFF + SCHED_SLOTS * SCHED_SLOT_BYTES;
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

constexpr int HALF = 64;  // streamed-tile columns processed at a time

// One half of a streamed tile, 32 columns per thread: scores and dP from TMEM, P (kv-stationary
// launch only) and dS back over them as 16-bit tiles.  `bits` marks the visible columns; with
// MASKED = false all of them are.
template <bool IS_BF16, bool DKDV, bool MASKED>
__device__ __forceinline__ void act_half(uint32_t tT0, uint32_t tT1, int wg, float half_alpha, uint32_t bits) {
  uint32_t rs[32], rp[32];
  tmem_ld32(tT0 + wg * 32, rs);
  tmem_ld32(tT1 + wg * 32, rp);
  tc_wait_ld();
  // the 16-bit tiles are written over the first 32 columns of T0 / T1: every warp must hold its
  // scores in registers before anyone stores
  asm volatile("bar.sync 1, 256;" ::: "memory");
  uint32_t pk[16], dk[16];
#pragma unroll
  for (int x = 0; x < 16; ++x) {
    float sl0, dsl0, sl1, dsl1;
    silu_and_grad(__uint_as_float(rs[2 * x]) * half_alpha, sl0, dsl0);
    silu_and_grad(__uint_as_float(rs[2 * x + 1]) * half_alpha, sl1, dsl1);
    float ds0 = __uint_as_float(rp[2 * x]) * dsl0, ds1 = __uint_as_float(rp[2 * x + 1]) * dsl1;
    if (MASKED) {
      const bool v0 = bits & (1u << (2 * x)), v1 = bits & (1u << (2 * x + 1));
      sl0 = v0 ? sl0 : 0.f;
      sl1 = v1 ? sl1 : 0.f;
      ds0 = v0 ? ds0 : 0.f;
      ds1 = v1 ? ds1 : 0.f;
    }
    if (DKDV) pk[x] = pack2h(sl0, sl1, IS_BF16);
    dk[x] = pack2h(ds0, ds1, IS_BF16);
  }
  if (DKDV) tmem_st16(tT0 + wg * 16, pk);
  tmem_st16(tT1 + wg * 16, dk);
}

// The partially visible and the element-wise variants stay out of line: the loop over fully
// visible tiles is the hot one and should stay small.
template <bool IS_BF16, bool DKDV>
__device__ __noinline__ void act_half_masked(uint32_t tT0, uint32_t tT1, int wg, float half_alpha, uint32_t bits) {
  act_half<IS_BF16, DKDV, true>(tT0, tT1, wg, half_alpha, bits);
}

template <bool IS_BF16, bool DKDV>
__device__ __noinline__ void act_half_exact(uint32_t tT0, uint32_t tT1, int wg, float half_alpha, SeqMask m, int own,
                                            int c0, const float *bias, int bias_numel) {
  uint32_t rs[32], rp[32];
  tmem_ld32(tT0 + wg * 32, rs);
  tmem_ld32(tT1 + wg * 32, rp);
  tc_wait_ld();
  asm volatile("bar.sync 1, 256;" ::: "memory");
  const int L = m.L;
  const int id_own = m.id(own);
  uint32_t pk[16], dk[16];
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
      float ds = __uint_as_float(rp[x + y]) * dsl;
      const int id_other = m.id(other);
      bool valid = qi_ < L && kj_ < L && m.valid_ids(qi_, kj_, DKDV ? id_other : id_own, DKDV ? id_own : id_other);
      pv[y] = valid ? sl : 0.f;
      dv[y] = valid ? ds : 0.f;
    }
    pk[x / 2] = pack2h(pv[0], pv[1], IS_BF16);
    dk[x / 2] = pack2h(dv[0], dv[1], IS_BF16);
  }
  if (DKDV) tmem_st16(tT0 + wg * 16, pk);
  tmem_st16(tT1 + wg * 16, dk);
}

// Stores one 128 x D fp32 accumulator (TMEM) as scaled 16-bit rows of a jagged tensor.
template <int D, bool IS_BF16>
__device__ __forceinline__ void store_acc_rows(uint32_t tacc, float scale, uint16_t *row_ptr, bool row_valid) {
  uint32_t r[2][32];
  tmem_ld32(tacc, r[0]);
#pragma unroll
  for (int c = 0; c < D / 32; ++c) {
    tc_wait_ld();
    if (c + 1 < D / 32) tmem_ld32(tacc + (c + 1) * 32, r[(c + 1) & 1]);
    if (row_valid) {
      const uint32_t(&v)[32] = r[c & 1];
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        uint4 o4;
        o4.x = pack2h(__uint_as_float(v[8 * x + 0]) * scale, __uint_as_float(v[8 * x + 1]) * scale, IS_BF16);
        o4.y = pack2h(__uint_as_float(v[8 * x + 2]) * scale, __uint_as_float(v[8 * x + 3]) * scale, IS_BF16);
        o4.z = pack2h(__uint_as_float(v[8 * x + 4]) * scale, __uint_as_float(v[8 * x + 5]) * scale, IS_BF16);
        o4.w = pack2h(__uint_as_float(v[8 * x + 6]) * scale, __uint_as_float(v[8 * x + 7]) * scale, IS_BF16);
        *reinterpret_cast<uint4 *>(row_ptr + c * 32 + x * 8) = o4;
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

template <int D, bool IS_BF16, bool DKDV>
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
  const uint32_t x_full = bars + 0, x_empty = bars + 8;
  // the streamed rings are filled and released in half tiles (64 rows): index 2 * slot + half
  const uint32_t y0_full = bars + 16, y0_empty = y0_full + 16 * STAGES;
  const uint32_t y1_full = y0_empty + 16 * STAGES, y1_empty = y1_full + 16 * STAGES;
  const uint32_t t_full = y1_empty + 16 * STAGES;  // [2] stage-1 tiles of half a / b ready
  const uint32_t w_full = t_full + 16;             // [2] 16-bit tiles of half a / b written
  const uint32_t acc_full = w_full + 16;           // [2] accumulator set complete
  const uint32_t acc_empty = acc_full + 16;        // [2] accumulator set stored
  const uint32_t sched_full = acc_empty + 16;      // [SCHED_SLOTS] next work item published
  const uint32_t sched_empty = sched_full + 8 * SCHED_SLOTS;
  uint8_t *sched_ring = smem_gen + SM::SCHED_OFF;
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + SM::MISC_OFF);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + SM::MISC_OFF + 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  WaitCtx wc{abort_flag, p.status};
  const uint64_t cta_t0 = p.trace != nullptr ? globaltimer_ns() : 0;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(x_full, 1);
    mbar_init(x_empty, 1);
    for (int s = 0; s < 2 * STAGES; ++s) {
      mbar_init(y0_full + 8 * s, 1);
      mbar_init(y0_empty + 8 * s, 1);
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
  // TMEM columns: T0_a [0,64) T0_b [64,128) T1_a [128,192) T1_b [192,256) ACC0 [256,384) ACC1 [384,512)
  //   T0 = S^T | S,  T1 = dP^T | dP;  kv-stationary: ACC0 = dV, ACC1 = dK (one set);
  //   q-stationary: ACC0 / ACC1 = dQ of even / odd items (two sets)
  const int num_items = p.plan->num_items * p.H;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && (int)blockIdx.x < num_items) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v); prefetch_tmap(&tmap_do);
      uint32_t it_cnt = 0, cnt = 0;
      bool ok = true;
      Tracer tr;
      tr.init(p.trace, 0, true);
      ItemDesc d = load_desc(p.items, blockIdx.x / p.H);
      int idx = blockIdx.x;
      while (idx < num_items && ok) {
        const int nidx = atomicAdd(&p.plan->next, 1);
        const int h = idx % p.H;
        TileItem it;
        fill_bwd_item<DKDV>(it, p.g, d);
        tr.mark(1);
        ok = mbar_wait(wc, x_empty, (it_cnt & 1) ^ 1, 401);
        if (!ok) break;
        tr.mark(2);
        mbar_arrive_expect_tx(x_full, 2 * SM::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < SM::CHUNKS; ++c) {
          tma_load_2d(sX0 + c * SM::CHUNK_BYTES, mapX0, h * D + c * 64, it.start + it.m0, x_full);
          tma_load_2d(sX1 + c * SM::CHUNK_BYTES, mapX1, h * D + c * 64, it.start + it.m0, x_full);
        }
        for (int j = 0; j < it.n_tiles && ok; ++j, ++cnt) {
          const int s = cnt % STAGES;
          const uint32_t par = ((cnt / STAGES) & 1) ^ 1;
          const int row = it.start + it.tile_at(j) * TILE;
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const int b = 8 * (2 * s + hf);
            const uint32_t off = s * SM::TILE_BYTES + hf * HALF * 128;
            ok = mbar_wait(wc, y0_empty + b, par, 402);
            if (!ok) break;
            tr.mark(3);
            mbar_arrive_expect_tx(y0_full + b, SM::TILE_BYTES / 2);
#pragma unroll
            for (int c = 0; c < SM::CHUNKS; ++c)
              tma_load_2d(sY0 + off + c * SM::CHUNK_BYTES, mapY0, h * D + c * 64, row + hf * HALF, y0_full + b);
            ok = mbar_wait(wc, y1_empty + b, par, 403);
            if (!ok) break;
            mbar_arrive_expect_tx(y1_full + b, SM::TILE_BYTES / 2);
#pragma unroll
            for (int c = 0; c < SM::CHUNKS; ++c)
              tma_load_2d(sY1 + off + c * SM::CHUNK_BYTES, mapY1, h * D + c * 64, row + hf * HALF, y1_full + b);
          }
        }
        if (!ok) break;
        ItemDesc nd = d;
        if (nidx < num_items) nd = load_desc(p.items, nidx / p.H);
        ++it_cnt;
        sched_publish(wc, sched_ring, sched_full, sched_empty, it_cnt, nd.b, nd.t, nd.start, nd.len, nd.nt, nidx, ok);
        d = nd;
        idx = nidx;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (warp-uniform)
    if ((int)blockIdx.x < num_items) {
      constexpr uint32_t FMT = IS_BF16 ? 1u : 0u;
      const uint32_t idesc_1 = make_idesc(FMT, FMT, 0, 0, TILE, HALF);  // 128 x 64, both operands K-major
      const uint32_t idesc_2 = make_idesc(FMT, FMT, 0, 1, TILE, D);     // 128 x D, TMEM A, MN-major B
      const uint64_t x0_desc = make_smem_desc(sX0, 16, 1024);
      const uint64_t x1_desc = make_smem_desc(sX1, 16, 1024);
      uint32_t it_cnt = 0, cnt = 0;
      bool ok = true;
      Tracer tr;
      tr.init(p.trace, 1, lane == 0);

      // stage 1 of half hf of streamed tile number `tile_no` (ring slot tile_no % STAGES):
      // T0_hf = X0 Y0_hf^T, T1_hf = X1 Y1_hf^T
      auto stage1 = [&](int hf, uint32_t tile_no) -> bool {
        const int s = tile_no % STAGES;
        const uint32_t par = (tile_no / STAGES) & 1;
        const int b = 8 * (2 * s + hf);
        if (!mbar_wait(wc, y0_full + b, par, 502)) return false;
        if (!mbar_wait(wc, y1_full + b, par, 503)) return false;
        tc_fence_after();
        const uint64_t y0_desc = make_smem_desc(sY0 + s * SM::TILE_BYTES + hf * HALF * 128, 16, 1024);
        const uint64_t y1_desc = make_smem_desc(sY1 + s * SM::TILE_BYTES + hf * HALF * 128, 16, 1024);
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = (ks / 4) * SM::CHUNK_BYTES + (ks % 4) * 32;
            mma_ss(tmem_base + hf * HALF, desc_advance(x0_desc, off), desc_advance(y0_desc, off), idesc_1, ks > 0);
          }
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = (ks / 4) * SM::CHUNK_BYTES + (ks % 4) * 32;
            mma_ss(tmem_base + 128 + hf * HALF, desc_advance(x1_desc, off), desc_advance(y1_desc, off), idesc_1,
                   ks > 0);
          }
          tc_commit(t_full + 8 * hf);
          // q-stationary launch: stage 2 does not read V again, its half can be refilled already
          if (!DKDV) tc_commit(y1_empty + b);
        }
        __syncwarp();
        return true;
      };
      // the stationary tiles have no reader left once the item's last stage 1 has been issued
      auto release_x = [&]() {
        if (elect_one()) tc_commit(x_empty);
        __syncwarp();
      };

      ItemDesc d = load_desc(p.items, blockIdx.x / p.H);
      int idx = blockIdx.x;
      bool pre_issued = false;  // stage 1 of this item's first tile was issued while the previous item finished
      for (; idx < num_items && ok; ++it_cnt) {
        TileItem it;
        fill_bwd_item<DKDV>(it, p.g, d);
        const int n = it.n_tiles;
        tr.mark(10);
        // accumulator set of this item and how often it has been used before
        const int aset = DKDV ? 0 : (int)(it_cnt & 1);
        const uint32_t ause = DKDV ? it_cnt : (it_cnt >> 1);
        if (!pre_issued) {
          ok = mbar_wait(wc, x_full, it_cnt & 1, 501);
          if (!ok) break;
          tc_fence_after();
          ok = stage1(0, cnt) && stage1(1, cnt);
          if (!ok) break;
          if (n == 1) release_x();
        }
        pre_issued = false;
        ItemDesc nd = d;
        int nidx = idx;
        bool next_item = false;
        int next_n = 0;
        for (int j = 0; j < n; ++j, ++cnt) {
          const int s = cnt % STAGES;
          const bool has_next = j + 1 < n;
          if (j == 0) {  // the previous user of this accumulator set must have been stored
            ok = mbar_wait(wc, acc_empty + 8 * aset, (ause & 1) ^ 1, 504);
            if (!ok) break;
          }
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            tr.mark(12 + hf);
            ok = mbar_wait(wc, w_full + 8 * hf, cnt & 1, 505);
            if (!ok) break;
            tc_fence_after();
            tr.mark(14 + hf);
            // stage 2: the 64 rows of this half of the streamed tile are the contraction dimension.
            // MN-major B: 64-column blocks 16 KB apart, 16 rows (one MMA) = 2 KB, half b starts 8 KB in.
            const uint64_t y0_mn = make_smem_desc(sY0 + s * SM::TILE_BYTES + hf * HALF * 128, SM::CHUNK_BYTES, 1024);
            const uint64_t y1_mn = make_smem_desc(sY1 + s * SM::TILE_BYTES + hf * HALF * 128, SM::CHUNK_BYTES, 1024);
            const uint32_t acc_on = (j > 0 || hf > 0) ? 1u : 0u;
            if (elect_one()) {
              if (DKDV) {
#pragma unroll
                for (int ks = 0; ks < HALF / 16; ++ks)  // dV += P^T dO
                  mma_ts(tmem_base + 256, tmem_base + hf * HALF + ks * 8, desc_advance(y1_mn, ks * 2048), idesc_2,
                         (acc_on || ks > 0) ? 1u : 0u);
#pragma unroll
                for (int ks = 0; ks < HALF / 16; ++ks)  // dK += dS^T Q
                  mma_ts(tmem_base + 384, tmem_base + 128 + hf * HALF + ks * 8, desc_advance(y0_mn, ks * 2048),
                         idesc_2, (acc_on || ks > 0) ? 1u : 0u);
              } else {
#pragma unroll
                for (int ks = 0; ks < HALF / 16; ++ks)  // dQ += dS K
                  mma_ts(tmem_base + 256 + aset * 128, tmem_base + 128 + hf * HALF + ks * 8,
                         desc_advance(y0_mn, ks * 2048), idesc_2, (acc_on || ks > 0) ? 1u : 0u);
              }
              if (!has_next && hf == 1) tc_commit(acc_full + 8 * aset);
              // this half of the streamed tile has no readers left
              tc_commit(y0_empty + 8 * (2 * s + hf));
              if (DKDV) tc_commit(y1_empty + 8 * (2 * s + hf));
            }
            __syncwarp();
            tr.mark(16 + hf);
            if (has_next) {
              ok = stage1(hf, cnt + 1);
              if (!ok) break;
              tr.mark(18 + hf);
              if (hf == 1 && j == n - 2) release_x();
            } else if (hf == 0) {
              // Last tile of the item: the half-a tiles are free from here on.  Fetch the next
              // item and issue stage 1 of its first tile, half a now and half b after this
              // item's last stage 2; its stationary tiles were requested when this item's last
              // stage 1 was issued, its first streamed tile goes to the other ring slot.
              ok = sched_fetch(wc, sched_ring, sched_full, sched_empty, it_cnt + 1, nd.b, nd.t, nd.start, nd.len,
                               nd.nt, nidx, lane == 0);
              if (!ok) break;
              if (nidx < num_items) {
                TileItem ni;
                fill_bwd_item<DKDV>(ni, p.g, nd);
                next_n = ni.n_tiles;
                next_item = true;
                ok = mbar_wait(wc, x_full, (it_cnt + 1) & 1, 508);
                if (!ok) break;
                tc_fence_after();
                ok = stage1(0, cnt + 1);
                if (!ok) break;
                tr.mark(20);
              }
            } else if (next_item) {
              ok = stage1(1, cnt + 1);
              if (!ok) break;
              tr.mark(21);
              if (next_n == 1) release_x();
              pre_issued = true;
            }
          }
          if (!ok) break;
        }
        if (!ok) break;
        d = nd;
        idx = nidx;
      }
    }
  } else if (warp < 10) {
    // ------------------------------------------------------------------ activation warps
    // All eight warps work on one half of the streamed tile at a time (a, then b): the half is
    // finished - and handed back to the tensor pipe - soonest when every warp works on it.
    // Warps 2-5 take columns [0,32) of the half, warps 6-9 columns [32,64); thread = one row of
    // the stationary tile.
    const int wg = warp >= 6 ? 1 : 0;
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;  // stationary-tile row owned by this thread
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    uint32_t cnt = 0, item_no = 0;
    bool ok = true;
    Tracer tr;
    tr.init(p.trace, 2, warp == 2 && lane == 0);
    if ((int)blockIdx.x < num_items) {
      ItemDesc d = load_desc(p.items, blockIdx.x / p.H);
      int idx = blockIdx.x;
      while (idx < num_items && ok) {
        TileItem it;
        fill_bwd_item<DKDV>(it, p.g, d);
        const int L = it.m.L;
        const int own = it.m0 + row_in_tile;  // kv position (DKDV) or query position
        const bool exact_only = !it.regular || p.bias != nullptr;
        ColInterval ci;
        RowInterval ri;
        if (DKDV) ci = col_interval(it, own); else ri = row_interval(it, own);
        for (int j = 0; j < it.n_tiles && ok; ++j, ++cnt) {
          const int o0 = it.tile_at(j) * TILE;  // first position of the streamed tile
          bool full;
          if (DKDV) {  // streamed = query tile o0, stationary = kv tile it.m0; all query rows must exist
            TileItem qi = it;
            qi.m0 = o0;
            full = !exact_only && tile_pair_is_full(qi, it.m0) && (o0 + TILE <= L);
          } else {
            full = !exact_only && tile_pair_is_full(it, o0);
          }
#pragma unroll 1
          for (int hf = 0; hf < 2; ++hf) {
            const int c0 = o0 + hf * HALF + wg * 32;  // first streamed position of this thread's 32 columns
            const uint32_t tT0 = tmem_base + hf * HALF + lane_off;
            const uint32_t tT1 = tmem_base + 128 + hf * HALF + lane_off;
            tr.mark(30);
            ok = mbar_wait(wc, t_full + 8 * hf, cnt & 1, 601);
            if (!ok) break;
            tc_fence_after();
            tr.mark(31);
            if (full) {
              act_half<IS_BF16, DKDV, false>(tT0, tT1, wg, p.half_alpha, 0xffffffffu);
            } else if (!exact_only) {
              const uint32_t bits = DKDV ? col_mask_bits(ci, c0, L) : row_mask_bits(ri, c0, L);
              act_half_masked<IS_BF16, DKDV>(tT0, tT1, wg, p.half_alpha, bits);
            } else {
              act_half_exact<IS_BF16, DKDV>(tT0, tT1, wg, p.half_alpha, it.m, own, c0, p.bias, p.bias_numel);
            }
            tr.mark(37);
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(w_full + 8 * hf);
            tr.mark(33);
          }
        }
        if (!ok) break;
        ++item_no;
        ok = sched_fetch(wc, sched_ring, sched_full, sched_empty, item_no, d.b, d.t, d.start, d.len, d.nt, idx,
                         lane == 0);
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
      ItemDesc d = load_desc(p.items, blockIdx.x / p.H);
      int idx = blockIdx.x;
      while (idx < num_items && ok) {
        const int h = idx % p.H;
        TileItem it;
        fill_bwd_item<DKDV>(it, p.g, d);
        const int L = it.m.L;
        const int own = it.m0 + row_in_tile;
        const bool rv = own < L;
        const int aset = DKDV ? 0 : (int)(it_cnt & 1);
        const uint32_t ause = DKDV ? it_cnt : (it_cnt >> 1);
        tr.mark(34);
        ok = mbar_wait(wc, acc_full + 8 * aset, ause & 1, 602);
        if (!ok) break;
        tc_fence_after();
        tr.mark(35);
        if (DKDV) {
          uint16_t *dvrow = reinterpret_cast<uint16_t *>(p.dv) + (int64_t)(it.start + own) * p.dv_rs + (int64_t)h * p.dv_hs;
          uint16_t *dkrow = reinterpret_cast<uint16_t *>(p.dk) + (int64_t)(it.start + own) * p.dk_rs + (int64_t)h * p.dk_hs;
          store_acc_rows<D, IS_BF16>(tmem_base + 256 + lane_off, sc, dvrow, rv);
          store_acc_rows<D, IS_BF16>(tmem_base + 384 + lane_off, sc * p.alpha, dkrow, rv);
        } else {
          uint16_t *dqrow = reinterpret_cast<uint16_t *>(p.dq) + (int64_t)(it.start + own) * p.dq_rs + (int64_t)h * p.dq_hs;
          store_acc_rows<D, IS_BF16>(tmem_base + 256 + aset * 128 + lane_off, sc * p.alpha, dqrow, rv);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty + 8 * aset);
        tr.mark(36);
        if (it.len > L && it.m0 + TILE >= L) {
          if (DKDV) {
            zero_rows_beyond<D>(reinterpret_cast<uint16_t *>(p.dk), p.dk_rs, p.dk_hs, h, it.start, L, it.len, row_in_tile);
            zero_rows_beyond<D>(reinterpret_cast<uint16_t *>(p.dv), p.dv_rs, p.dv_hs, h, it.start, L, it.len, row_in_tile);
          } else {
            zero_rows_beyond<D>(reinterpret_cast<uint16_t *>(p.dq), p.dq_rs, p.dq_hs, h, it.start, L, it.len, row_in_tile);
          }
        }
        ++it_cnt;
        ok = sched_fetch(wc, sched_ring, sched_full, sched_empty, it_cnt, d.b, d.t, d.start, d.len, d.nt, idx,
                         lane == 0);
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
  // timeline: start and end time of every CTA (second half of the last role's records)
  if (p.trace != nullptr && threadIdx.x == 0 && blockIdx.x < TRACE_RECORDS / 2)
    p.trace[3 * TRACE_RECORDS + TRACE_RECORDS / 2 + blockIdx.x] = make_ulonglong2(cta_t0, globaltimer_ns());
}

}  // namespace

// scratch: two work lists (kv-stationary and q-stationary)
int64_t attn_tc_bwd_workspace_bytes(const b200_hstu_attn_args &a) {
  return 2 * plan_bytes(a.total_L, a.B);
}

template <int D, bool IS_BF16>
int launch_bwd_tc(const b200_hstu_attn_args &a, cudaStream_t st) {
  using SM = BwdSmem<D>;
  if (a.workspace == nullptr || a.workspace_bytes < attn_tc_bwd_workspace_bytes(a))
    return fail(B200_HSTU_EWORKSPACE, "attention backward needs %lld bytes of scratch, got %lld",
                (long long)attn_tc_bwd_workspace_bytes(a), (long long)a.workspace_bytes);
  CUtensorMap mq, mk, mv, mdo;
  int rc;
  // stationary operands are fetched as whole 128-row tiles, streamed ones in 64-row halves
  CUtensorMap mqh, mkh, mvh, mdoh;
  const int64_t cols = (int64_t)a.H * D;
  if ((rc = make_tile_map_rows(&mq, a.q, a.total_L, cols, a.q_row_stride, 2, IS_BF16, TILE)) != 0) return rc;
  if ((rc = make_tile_map_rows(&mk, a.k, a.total_L, cols, a.k_row_stride, 2, IS_BF16, TILE)) != 0) return rc;
  if ((rc = make_tile_map_rows(&mv, a.v, a.total_L, cols, a.v_row_stride, 2, IS_BF16, TILE)) != 0) return rc;
  if ((rc = make_tile_map_rows(&mdo, a.dout, a.total_L, cols, a.do_row_stride, 2, IS_BF16, TILE)) != 0) return rc;
  if ((rc = make_tile_map_rows(&mqh, a.q, a.total_L, cols, a.q_row_stride, 2, IS_BF16, HALF)) != 0) return rc;
  if ((rc = make_tile_map_rows(&mkh, a.k, a.total_L, cols, a.k_row_stride, 2, IS_BF16, HALF)) != 0) return rc;
  if ((rc = make_tile_map_rows(&mvh, a.v, a.total_L, cols, a.v_row_stride, 2, IS_BF16, HALF)) != 0) return rc;
  if ((rc = make_tile_map_rows(&mdoh, a.dout, a.total_L, cols, a.do_row_stride, 2, IS_BF16, HALF)) != 0) return rc;
  BwdParams p;
  p.g.seq_offsets = a.seq_offsets;
  p.g.num_targets = a.num_targets;
  p.g.B = a.B;
  p.g.H = a.H;
  p.g.max_seq_len = a.max_seq_len;
  p.g.W = a.max_attn_len;
  p.g.c = a.contextual_seq_len;
  p.g.F = a.min_full_attn_seq_len;
  p.dq = a.dq; p.dk = a.dk; p.dv = a.dv_;
  p.dq_rs = a.dq_row_stride; p.dq_hs = a.dq_head_stride;
  p.dk_rs = a.dk_row_stride; p.dk_hs = a.dk_head_stride;
  p.dv_rs = a.dv_row_stride; p.dv_hs = a.dv_head_stride;
  p.attn_scale = a.attn_scale;
  p.bias = a.bias_by_distance;
  p.bias_numel = a.bias_numel;
  p.half_alpha = 0.5f * a.alpha;
  p.alpha = a.alpha;
  p.inv_n = 1.f / (float)a.max_seq_len;
  p.H = a.H;
  p.trace = nullptr;
  const int max_items = (int)plan_max_items(a.total_L, a.B);
  const int64_t one = plan_bytes(a.total_L, a.B);
  // B200_HSTU_TRACE=dkdv|dq and a scratch buffer with TRACE_BYTES of extra room: CTA 0 of that
  // launch records a timeline of its roles behind the work lists (a profiling aid, off by default)
  static const char *want_trace = getenv("B200_HSTU_TRACE");
  ulonglong2 *trace_buf = nullptr;
  if (want_trace != nullptr && a.workspace_bytes >= 2 * one + TRACE_BYTES)
    trace_buf = reinterpret_cast<ulonglong2 *>(reinterpret_cast<uint8_t *>(a.workspace) + 2 * one);
  const int64_t upper = (int64_t)max_items * a.H;
  const int grid = (int)(upper < device_sm_count() ? upper : device_sm_count());
  PlanHeader *hdr_kv = reinterpret_cast<PlanHeader *>(a.workspace);
  PlanHeader *hdr_q = reinterpret_cast<PlanHeader *>(reinterpret_cast<uint8_t *>(a.workspace) + one);
  {
    ProfileScope prof(PROF_PLAN, st);
    attn_plan2_kernel<PLAN_KV_TILE, PLAN_Q_TILE><<<2, PLAN_THREADS, 0, st>>>(
        p.g, hdr_kv, reinterpret_cast<ItemDesc *>(hdr_kv + 1), hdr_q, reinterpret_cast<ItemDesc *>(hdr_q + 1),
        max_items, grid);
  }
  count_launch();
  B200_CHECK_LAUNCH("attention plan (backward)");
  {
    auto kern = hstu_attn_bwd_sm100_kernel<D, IS_BF16, true>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::DYN_BYTES);
    if (e != cudaSuccess) return check_cuda(e, "backward smem attribute");
    BwdParams pk = p;
    pk.plan = hdr_kv;
    pk.items = reinterpret_cast<ItemDesc *>(hdr_kv + 1);
    pk.status = &hdr_kv->status;
    if (trace_buf != nullptr && want_trace[0] == 'd' && want_trace[1] == 'k') pk.trace = trace_buf;
    ProfileScope prof(PROF_ATTN_BWD_DKDV, st);
    kern<<<grid, BWD_THREADS, SM::DYN_BYTES, st>>>(mqh, mk, mv, mdoh, pk);
    count_launch();
    B200_CHECK_LAUNCH("tcgen05 attention backward (dk, dv)");
  }
  {
    auto kern = hstu_attn_bwd_sm100_kernel<D, IS_BF16, false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::DYN_BYTES);
    if (e != cudaSuccess) return check_cuda(e, "backward smem attribute");
    BwdParams pq = p;
    pq.plan = hdr_q;
    pq.items = reinterpret_cast<ItemDesc *>(hdr_q + 1);
    pq.status = &hdr_q->status;
    if (trace_buf != nullptr && want_trace[0] == 'd' && want_trace[1] == 'q') pq.trace = trace_buf;
    ProfileScope prof(PROF_ATTN_BWD_DQ, st);
    kern<<<grid, BWD_THREADS, SM::DYN_BYTES, st>>>(mq, mkh, mvh, mdo, pq);
    count_launch();
    B200_CHECK_LAUNCH("tcgen05 attention backward (dq)");
  }
  return 0;
}

int attn_tc_bwd(const b200_hstu_attn_args &a, cudaStream_t st) {
  const bool bf = a.dtype == B200_HSTU_BF16;
  if (a.dqk == 128) return bf ? launch_bwd_tc<128, true>(a, st) : launch_bwd_tc<128, false>(a, st);
  return bf ? launch_bwd_tc<64, true>(a, st) : launch_bwd_tc<64, false>(a, st);
}

}  // namespace b200hstu
