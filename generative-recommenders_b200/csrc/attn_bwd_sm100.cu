// Jagged HSTU attention backward on Blackwell tensor cores (tcgen05 + TMEM + TMA), bf16 / fp16,
// head dimension 64 or 128 (d_qk == d_v), constant attention scale.
//
// With x = alpha q.k (+ bias), s = sigmoid(x), P = x s scale mask:
//   dV = P^T dO          dP = dO V^T          dS = dP * (s + x s (1 - s)) * scale * mask
//   dK = alpha dS^T Q    dQ = alpha dS K
// (the math of generative_recommenders/ops/triton/triton_hstu_attention.py:1905-2020; no softmax
// statistics and no `out` are needed).
//
// Two persistent kernels, each element of every gradient has exactly one owner, so there are no
// atomics, no fp32 dQ scratch, no convert pass, and the result is bit-reproducible:
//   * dkdv kernel - one work item per (sequence, 128-row K/V tile, head).  K and V stay in shared
//     memory; Q and dO tiles of every query tile that can see the K/V tile stream through 2-stage
//     TMA rings.  S^T = K Q^T and dP^T = V dO^T land in TMEM, 128 threads (one K/V row each) turn
//     them into bf16 P^T and dS^T written back over the same TMEM columns, and those feed
//     dV += P^T dO and dK += dS^T Q as TMEM A-operands (dO and Q are the MN-major B operands).
//   * dq kernel - one work item per (sequence, 128-row query tile, head), the forward's loop
//     structure: Q and dO stay, K and V stream; S = Q K^T and dP = dO V^T in TMEM, dS written over
//     dP, dQ += dS K with K as the MN-major B operand.
// Constant factors are folded into the epilogues: dV * scale, dK * scale*alpha, dQ * scale*alpha.
#include "attn_plan.cuh"
#include "sm100_ptx.cuh"

namespace b200hstu {

using namespace ptx;

int make_tile_map(CUtensorMap *m, const void *base, int64_t rows, int64_t cols, int64_t row_stride_elems,
                  int elem_bytes, bool is_bf16);
int device_sm_count();

namespace {

constexpr int BWD_THREADS = 192;
constexpr int STAGES = 2;

struct BwdParams {
  AttnGeomParams g;
  const PlanHeader *plan;
  const int2 *items;
  int *status;
  void *dq, *dk, *dv;
  int64_t dq_rs, dq_hs, dk_rs, dk_hs, dv_rs, dv_hs;
  const float *attn_scale;  // NULL or one fp32 on the device
  const float *bias;
  int bias_numel;
  float half_alpha, alpha, inv_n;
  int H;
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
  static constexpr int NUM_BARS = 24;
  static constexpr int MISC_OFF = BAR_OFF + NUM_BARS * 8;
  static constexpr int TOTAL = MISC_OFF + 64;
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

// Stores one 128 x D fp32 accumulator (TMEM) as scaled 16-bit rows of a jagged tensor.
template <int D, bool IS_BF16>
__device__ __forceinline__ void store_acc_rows(uint32_t tacc, float scale, uint16_t *row_ptr, bool row_valid) {
#pragma unroll 1
  for (int c = 0; c < D / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(tacc + c * 32, r);
    tc_wait_ld();
    if (row_valid) {
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        uint4 o4;
        o4.x = pack2h(__uint_as_float(r[8 * x + 0]) * scale, __uint_as_float(r[8 * x + 1]) * scale, IS_BF16);
        o4.y = pack2h(__uint_as_float(r[8 * x + 2]) * scale, __uint_as_float(r[8 * x + 3]) * scale, IS_BF16);
        o4.z = pack2h(__uint_as_float(r[8 * x + 4]) * scale, __uint_as_float(r[8 * x + 5]) * scale, IS_BF16);
        o4.w = pack2h(__uint_as_float(r[8 * x + 6]) * scale, __uint_as_float(r[8 * x + 7]) * scale, IS_BF16);
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

// =========================================================================================
// dK / dV kernel: K/V-stationary
// =========================================================================================
template <int D, bool IS_BF16>
__global__ void __launch_bounds__(BWD_THREADS, 1)
    hstu_attn_bwd_dkdv_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                                    const __grid_constant__ CUtensorMap tmap_v,
                                    const __grid_constant__ CUtensorMap tmap_do, const BwdParams p) {
  using SM = BwdSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sK = smem_base + SM::A_OFF, sV = smem_base + SM::B_OFF;
  const uint32_t sQ = smem_base + SM::X_OFF, sDO = smem_base + SM::Y_OFF;
  const uint32_t bars = smem_base + SM::BAR_OFF;
  const uint32_t kv_full = bars + 0, kv_empty = bars + 8;
  const uint32_t q_full = bars + 16, q_empty = q_full + 8 * STAGES;       // Q ring
  const uint32_t do_full = q_empty + 8 * STAGES, do_empty = do_full + 8 * STAGES;  // dO ring
  const uint32_t st_full = do_empty + 8 * STAGES;   // S^T and dP^T ready (MMA -> threads)
  const uint32_t pt_full = st_full + 8;             // P^T and dS^T written (threads -> MMA)
  const uint32_t acc_full = pt_full + 8;            // dK, dV complete
  const uint32_t acc_empty = acc_full + 8;          // dK, dV read out
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + SM::MISC_OFF);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + SM::MISC_OFF + 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  WaitCtx wc{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(kv_full, 1);
    mbar_init(kv_empty, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(q_full + 8 * s, 1);
      mbar_init(q_empty + 8 * s, 1);
      mbar_init(do_full + 8 * s, 1);
      mbar_init(do_empty + 8 * s, 1);
    }
    mbar_init(st_full, 1);
    mbar_init(pt_full, 4);
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 4);
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
  const uint32_t tST = tmem_base;          // S^T  -> P^T   (columns 0..127)
  const uint32_t tDPT = tmem_base + 128;   // dP^T -> dS^T
  const uint32_t tDV = tmem_base + 256;
  const uint32_t tDK = tmem_base + 384;
  const int num_items = p.plan->num_items * p.H;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v); prefetch_tmap(&tmap_do);
      uint32_t it_cnt = 0, cnt = 0;
      bool ok = true;
      for (int idx = blockIdx.x; idx < num_items && ok; idx += gridDim.x, ++it_cnt) {
        const int2 e = p.items[idx / p.H];
        const int h = idx % p.H;
        TileItem it;
        load_item<true>(it, p.g, e.x, e.y);
        ok = mbar_wait(wc, kv_empty, (it_cnt & 1) ^ 1, 401);
        if (!ok) break;
        mbar_arrive_expect_tx(kv_full, 2 * SM::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < SM::CHUNKS; ++c) {
          tma_load_2d(sK + c * SM::CHUNK_BYTES, &tmap_k, h * D + c * 64, it.start + it.m0, kv_full);
          tma_load_2d(sV + c * SM::CHUNK_BYTES, &tmap_v, h * D + c * 64, it.start + it.m0, kv_full);
        }
        for (int j = 0; j < it.n_tiles; ++j, ++cnt) {
          const int s = cnt % STAGES;
          const uint32_t par = ((cnt / STAGES) & 1) ^ 1;
          const int row = it.start + it.tile_at(j) * TILE;
          ok = mbar_wait(wc, q_empty + 8 * s, par, 402);
          if (!ok) break;
          mbar_arrive_expect_tx(q_full + 8 * s, SM::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < SM::CHUNKS; ++c)
            tma_load_2d(sQ + s * SM::TILE_BYTES + c * SM::CHUNK_BYTES, &tmap_q, h * D + c * 64, row, q_full + 8 * s);
          ok = mbar_wait(wc, do_empty + 8 * s, par, 403);
          if (!ok) break;
          mbar_arrive_expect_tx(do_full + 8 * s, SM::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < SM::CHUNKS; ++c)
            tma_load_2d(sDO + s * SM::TILE_BYTES + c * SM::CHUNK_BYTES, &tmap_do, h * D + c * 64, row, do_full + 8 * s);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t FMT = IS_BF16 ? 1u : 0u;
      const uint32_t idesc_kk = make_idesc(FMT, FMT, 0, 0, TILE, TILE);  // K-major x K-major -> 128 x 128
      const uint32_t idesc_mn = make_idesc(FMT, FMT, 0, 1, TILE, D);     // TMEM A x MN-major B -> 128 x D
      const uint64_t k_desc = make_smem_desc(sK, 16, 1024);
      const uint64_t v_desc = make_smem_desc(sV, 16, 1024);
      uint32_t it_cnt = 0, cnt = 0;
      bool ok = true;
      for (int idx = blockIdx.x; idx < num_items && ok; idx += gridDim.x, ++it_cnt) {
        const int2 e = p.items[idx / p.H];
        TileItem it;
        load_item<true>(it, p.g, e.x, e.y);
        ok = mbar_wait(wc, kv_full, it_cnt & 1, 501);
        if (!ok) break;
        const int n = it.n_tiles;
        for (int j = 0; j < n; ++j, ++cnt) {
          const int s = cnt % STAGES;
          const uint32_t par = (cnt / STAGES) & 1;
          ok = mbar_wait(wc, q_full + 8 * s, par, 502);
          if (!ok) break;
          tc_fence_after();
          const uint64_t q_desc = make_smem_desc(sQ + s * SM::TILE_BYTES, 16, 1024);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = (ks / 4) * SM::CHUNK_BYTES + (ks % 4) * 32;
            mma_ss(tST, desc_advance(k_desc, off), desc_advance(q_desc, off), idesc_kk, ks > 0);
          }
          ok = mbar_wait(wc, do_full + 8 * s, par, 503);
          if (!ok) break;
          tc_fence_after();
          const uint64_t do_desc = make_smem_desc(sDO + s * SM::TILE_BYTES, 16, 1024);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = (ks / 4) * SM::CHUNK_BYTES + (ks % 4) * 32;
            mma_ss(tDPT, desc_advance(v_desc, off), desc_advance(do_desc, off), idesc_kk, ks > 0);
          }
          tc_commit(st_full);
          if (j == 0) {  // previous item's dK / dV must have been read out before they are overwritten
            ok = mbar_wait(wc, acc_empty, (it_cnt & 1) ^ 1, 504);
            if (!ok) break;
          }
          ok = mbar_wait(wc, pt_full, cnt & 1, 505);
          if (!ok) break;
          tc_fence_after();
          // B operands: dO / Q tiles as [128 q rows][D] MN-major (q is the contraction dimension)
          const uint64_t do_mn = make_smem_desc(sDO + s * SM::TILE_BYTES, SM::CHUNK_BYTES, 1024);
          const uint64_t q_mn = make_smem_desc(sQ + s * SM::TILE_BYTES, SM::CHUNK_BYTES, 1024);
#pragma unroll
          for (int ks = 0; ks < TILE / 16; ++ks)
            mma_ts(tDV, tST + ks * 8, desc_advance(do_mn, ks * 2048), idesc_mn, (j > 0 || ks > 0) ? 1u : 0u);
          tc_commit(do_empty + 8 * s);
#pragma unroll
          for (int ks = 0; ks < TILE / 16; ++ks)
            mma_ts(tDK, tDPT + ks * 8, desc_advance(q_mn, ks * 2048), idesc_mn, (j > 0 || ks > 0) ? 1u : 0u);
          tc_commit(q_empty + 8 * s);
        }
        if (!ok) break;
        tc_commit(kv_empty);
        tc_commit(acc_full);
        if (n == 0) {
          // nothing visited this tile (cannot happen for a non-empty tile: the diagonal is always valid)
        }
      }
    }
  } else {
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;  // K/V row owned by this thread
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    uint32_t it_cnt = 0, cnt = 0;
    bool ok = true;
    const float sc = p.attn_scale ? p.attn_scale[0] : p.inv_n;
    for (int idx = blockIdx.x; idx < num_items && ok; idx += gridDim.x, ++it_cnt) {
      const int2 e = p.items[idx / p.H];
      const int h = idx % p.H;
      TileItem it;
      load_item<true>(it, p.g, e.x, e.y);
      const int L = it.m.L;
      const int jcol = it.m0 + row_in_tile;  // kv position
      const int id_j = it.m.id(jcol);
      for (int j = 0; j < it.n_tiles; ++j, ++cnt) {
        const int m0 = it.tile_at(j) * TILE;  // first query row of the streamed tile
        // mask can be skipped when the (query tile, kv tile) pair is fully visible and every query
        // row of the tile exists
        TileItem qi = it;
        qi.m0 = m0;
        const bool full = tile_pair_is_full(qi, it.m0) && (m0 + TILE <= L) && p.bias == nullptr;
        ok = mbar_wait(wc, st_full, cnt & 1, 601);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t rs[32], rp[32];
          tmem_ld32(tST + lane_off + c * 32, rs);
          tmem_ld32(tDPT + lane_off + c * 32, rp);
          tc_wait_ld();
          uint32_t pk[16], dk[16];
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            float pv[2], dv[2];
#pragma unroll
            for (int y = 0; y < 2; ++y) {
              const int i = m0 + c * 32 + x + y;  // query position
              float hh = __uint_as_float(rs[x + y]) * p.half_alpha;
              if (p.bias != nullptr) {
                int dist = i > jcol ? i - jcol : jcol - i;
                if (dist < p.bias_numel) hh += 0.5f * p.bias[dist];
              }
              float sl, dsl;
              silu_and_grad(hh, sl, dsl);
              float ds = __uint_as_float(rp[x + y]) * dsl;
              bool valid = full || (i < L && jcol < L && it.m.valid_ids(i, jcol, it.m.id(i), id_j));
              pv[y] = valid ? sl : 0.f;
              dv[y] = valid ? ds : 0.f;
            }
            pk[x / 2] = pack2h(pv[0], pv[1], IS_BF16);
            dk[x / 2] = pack2h(dv[0], dv[1], IS_BF16);
          }
          tmem_st16(tST + lane_off + c * 16, pk);
          tmem_st16(tDPT + lane_off + c * 16, dk);
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(pt_full);
      }
      if (!ok) break;
      ok = mbar_wait(wc, acc_full, it_cnt & 1, 602);
      if (!ok) break;
      tc_fence_after();
      const bool rv = jcol < L;
      uint16_t *dvrow = reinterpret_cast<uint16_t *>(p.dv) + (int64_t)(it.start + jcol) * p.dv_rs + (int64_t)h * p.dv_hs;
      uint16_t *dkrow = reinterpret_cast<uint16_t *>(p.dk) + (int64_t)(it.start + jcol) * p.dk_rs + (int64_t)h * p.dk_hs;
      store_acc_rows<D, IS_BF16>(tDV + lane_off, sc, dvrow, rv);
      store_acc_rows<D, IS_BF16>(tDK + lane_off, sc * p.alpha, dkrow, rv);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
      if (it.len > L && it.m0 + TILE >= L) {
        zero_rows_beyond<D>(reinterpret_cast<uint16_t *>(p.dk), p.dk_rs, p.dk_hs, h, it.start, L, it.len, row_in_tile);
        zero_rows_beyond<D>(reinterpret_cast<uint16_t *>(p.dv), p.dv_rs, p.dv_hs, h, it.start, L, it.len, row_in_tile);
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
}

// =========================================================================================
// dQ kernel: Q/dO-stationary
// =========================================================================================
template <int D, bool IS_BF16>
__global__ void __launch_bounds__(BWD_THREADS, 1)
    hstu_attn_bwd_dq_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                                  const __grid_constant__ CUtensorMap tmap_v,
                                  const __grid_constant__ CUtensorMap tmap_do, const BwdParams p) {
  using SM = BwdSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base + SM::A_OFF, sDO = smem_base + SM::B_OFF;
  const uint32_t sK = smem_base + SM::X_OFF, sV = smem_base + SM::Y_OFF;
  const uint32_t bars = smem_base + SM::BAR_OFF;
  const uint32_t qd_full = bars + 0, qd_empty = bars + 8;
  const uint32_t k_full = bars + 16, k_empty = k_full + 8 * STAGES;
  const uint32_t v_full = k_empty + 8 * STAGES, v_empty = v_full + 8 * STAGES;
  const uint32_t sp_full = v_empty + 8 * STAGES;    // S and dP ready
  const uint32_t ds_full = sp_full + 8;             // dS written
  const uint32_t acc_full = ds_full + 8, acc_empty = acc_full + 8;
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + SM::MISC_OFF);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + SM::MISC_OFF + 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  WaitCtx wc{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(qd_full, 1);
    mbar_init(qd_empty, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(k_full + 8 * s, 1);
      mbar_init(k_empty + 8 * s, 1);
      mbar_init(v_full + 8 * s, 1);
      mbar_init(v_empty + 8 * s, 1);
    }
    mbar_init(sp_full, 1);
    mbar_init(ds_full, 4);
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 4);
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
  const uint32_t tS = tmem_base;           // S
  const uint32_t tDP = tmem_base + 128;    // dP -> dS
  const uint32_t tDQ = tmem_base + 256;
  const int num_items = p.plan->num_items * p.H;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v); prefetch_tmap(&tmap_do);
      uint32_t it_cnt = 0, cnt = 0;
      bool ok = true;
      for (int idx = blockIdx.x; idx < num_items && ok; idx += gridDim.x, ++it_cnt) {
        const int2 e = p.items[idx / p.H];
        const int h = idx % p.H;
        TileItem it;
        load_item<false>(it, p.g, e.x, e.y);
        ok = mbar_wait(wc, qd_empty, (it_cnt & 1) ^ 1, 701);
        if (!ok) break;
        mbar_arrive_expect_tx(qd_full, 2 * SM::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < SM::CHUNKS; ++c) {
          tma_load_2d(sQ + c * SM::CHUNK_BYTES, &tmap_q, h * D + c * 64, it.start + it.m0, qd_full);
          tma_load_2d(sDO + c * SM::CHUNK_BYTES, &tmap_do, h * D + c * 64, it.start + it.m0, qd_full);
        }
        for (int j = 0; j < it.n_tiles; ++j, ++cnt) {
          const int s = cnt % STAGES;
          const uint32_t par = ((cnt / STAGES) & 1) ^ 1;
          const int row = it.start + it.tile_at(j) * TILE;
          ok = mbar_wait(wc, k_empty + 8 * s, par, 702);
          if (!ok) break;
          mbar_arrive_expect_tx(k_full + 8 * s, SM::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < SM::CHUNKS; ++c)
            tma_load_2d(sK + s * SM::TILE_BYTES + c * SM::CHUNK_BYTES, &tmap_k, h * D + c * 64, row, k_full + 8 * s);
          ok = mbar_wait(wc, v_empty + 8 * s, par, 703);
          if (!ok) break;
          mbar_arrive_expect_tx(v_full + 8 * s, SM::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < SM::CHUNKS; ++c)
            tma_load_2d(sV + s * SM::TILE_BYTES + c * SM::CHUNK_BYTES, &tmap_v, h * D + c * 64, row, v_full + 8 * s);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t FMT = IS_BF16 ? 1u : 0u;
      const uint32_t idesc_kk = make_idesc(FMT, FMT, 0, 0, TILE, TILE);
      const uint32_t idesc_mn = make_idesc(FMT, FMT, 0, 1, TILE, D);
      const uint64_t q_desc = make_smem_desc(sQ, 16, 1024);
      const uint64_t do_desc = make_smem_desc(sDO, 16, 1024);
      uint32_t it_cnt = 0, cnt = 0;
      bool ok = true;
      for (int idx = blockIdx.x; idx < num_items && ok; idx += gridDim.x, ++it_cnt) {
        const int2 e = p.items[idx / p.H];
        TileItem it;
        load_item<false>(it, p.g, e.x, e.y);
        ok = mbar_wait(wc, qd_full, it_cnt & 1, 801);
        if (!ok) break;
        const int n = it.n_tiles;
        for (int j = 0; j < n; ++j, ++cnt) {
          const int s = cnt % STAGES;
          const uint32_t par = (cnt / STAGES) & 1;
          ok = mbar_wait(wc, k_full + 8 * s, par, 802);
          if (!ok) break;
          tc_fence_after();
          const uint64_t k_desc = make_smem_desc(sK + s * SM::TILE_BYTES, 16, 1024);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = (ks / 4) * SM::CHUNK_BYTES + (ks % 4) * 32;
            mma_ss(tS, desc_advance(q_desc, off), desc_advance(k_desc, off), idesc_kk, ks > 0);
          }
          ok = mbar_wait(wc, v_full + 8 * s, par, 803);
          if (!ok) break;
          tc_fence_after();
          const uint64_t v_desc = make_smem_desc(sV + s * SM::TILE_BYTES, 16, 1024);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = (ks / 4) * SM::CHUNK_BYTES + (ks % 4) * 32;
            mma_ss(tDP, desc_advance(do_desc, off), desc_advance(v_desc, off), idesc_kk, ks > 0);
          }
          tc_commit(v_empty + 8 * s);
          tc_commit(sp_full);
          if (j == 0) {
            ok = mbar_wait(wc, acc_empty, (it_cnt & 1) ^ 1, 804);
            if (!ok) break;
          }
          ok = mbar_wait(wc, ds_full, cnt & 1, 805);
          if (!ok) break;
          tc_fence_after();
          const uint64_t k_mn = make_smem_desc(sK + s * SM::TILE_BYTES, SM::CHUNK_BYTES, 1024);
#pragma unroll
          for (int ks = 0; ks < TILE / 16; ++ks)
            mma_ts(tDQ, tDP + ks * 8, desc_advance(k_mn, ks * 2048), idesc_mn, (j > 0 || ks > 0) ? 1u : 0u);
          tc_commit(k_empty + 8 * s);
        }
        if (!ok) break;
        tc_commit(qd_empty);
        tc_commit(acc_full);
      }
    }
  } else {
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    uint32_t it_cnt = 0, cnt = 0;
    bool ok = true;
    const float sc = p.attn_scale ? p.attn_scale[0] : p.inv_n;
    for (int idx = blockIdx.x; idx < num_items && ok; idx += gridDim.x, ++it_cnt) {
      const int2 e = p.items[idx / p.H];
      const int h = idx % p.H;
      TileItem it;
      load_item<false>(it, p.g, e.x, e.y);
      const int L = it.m.L;
      const int i = it.m0 + row_in_tile;
      const int id_i = it.m.id(i);
      for (int j = 0; j < it.n_tiles; ++j, ++cnt) {
        const int n0 = it.tile_at(j) * TILE;
        const bool full = tile_pair_is_full(it, n0) && p.bias == nullptr;
        ok = mbar_wait(wc, sp_full, cnt & 1, 901);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t rs[32], rp[32];
          tmem_ld32(tS + lane_off + c * 32, rs);
          tmem_ld32(tDP + lane_off + c * 32, rp);
          tc_wait_ld();
          uint32_t dk[16];
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            float dv[2];
#pragma unroll
            for (int y = 0; y < 2; ++y) {
              const int jj = n0 + c * 32 + x + y;
              float hh = __uint_as_float(rs[x + y]) * p.half_alpha;
              if (p.bias != nullptr) {
                int dist = i > jj ? i - jj : jj - i;
                if (dist < p.bias_numel) hh += 0.5f * p.bias[dist];
              }
              float sl, dsl;
              silu_and_grad(hh, sl, dsl);
              float ds = __uint_as_float(rp[x + y]) * dsl;
              bool valid = full || (i < L && jj < L && it.m.valid_ids(i, jj, id_i, it.m.id(jj)));
              dv[y] = valid ? ds : 0.f;
            }
            dk[x / 2] = pack2h(dv[0], dv[1], IS_BF16);
          }
          tmem_st16(tDP + lane_off + c * 16, dk);
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(ds_full);
      }
      if (!ok) break;
      ok = mbar_wait(wc, acc_full, it_cnt & 1, 902);
      if (!ok) break;
      tc_fence_after();
      uint16_t *dqrow = reinterpret_cast<uint16_t *>(p.dq) + (int64_t)(it.start + i) * p.dq_rs + (int64_t)h * p.dq_hs;
      store_acc_rows<D, IS_BF16>(tDQ + lane_off, sc * p.alpha, dqrow, i < L);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
      if (it.len > L && it.m0 + TILE >= L)
        zero_rows_beyond<D>(reinterpret_cast<uint16_t *>(p.dq), p.dq_rs, p.dq_hs, h, it.start, L, it.len, row_in_tile);
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
}

}  // namespace

// scratch: two work lists (kv-stationary and q-stationary)
int64_t attn_tc_bwd_workspace_bytes(const b200_hstu_attn_args &a) {
  int64_t one = (plan_bytes(a.total_L, a.B) + 255) / 256 * 256;
  return 2 * one;
}

template <int D, bool IS_BF16>
int launch_bwd_tc(const b200_hstu_attn_args &a, cudaStream_t st) {
  using SM = BwdSmem<D>;
  if (a.workspace == nullptr || a.workspace_bytes < attn_tc_bwd_workspace_bytes(a))
    return fail(B200_HSTU_EWORKSPACE, "attention backward needs %lld bytes of scratch, got %lld",
                (long long)attn_tc_bwd_workspace_bytes(a), (long long)a.workspace_bytes);
  CUtensorMap mq, mk, mv, mdo;
  int rc;
  if ((rc = make_tile_map(&mq, a.q, a.total_L, (int64_t)a.H * D, a.q_row_stride, 2, IS_BF16)) != 0) return rc;
  if ((rc = make_tile_map(&mk, a.k, a.total_L, (int64_t)a.H * D, a.k_row_stride, 2, IS_BF16)) != 0) return rc;
  if ((rc = make_tile_map(&mv, a.v, a.total_L, (int64_t)a.H * D, a.v_row_stride, 2, IS_BF16)) != 0) return rc;
  if ((rc = make_tile_map(&mdo, a.dout, a.total_L, (int64_t)a.H * D, a.do_row_stride, 2, IS_BF16)) != 0) return rc;
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
  const int max_items = (int)plan_max_items(a.total_L, a.B);
  const int64_t one = (plan_bytes(a.total_L, a.B) + 255) / 256 * 256;
  PlanHeader *hdr_kv = reinterpret_cast<PlanHeader *>(a.workspace);
  PlanHeader *hdr_q = reinterpret_cast<PlanHeader *>(reinterpret_cast<uint8_t *>(a.workspace) + one);
  attn_plan_kernel<true><<<1, PLAN_THREADS, 0, st>>>(p.g, hdr_kv, reinterpret_cast<int2 *>(hdr_kv + 1), max_items);
  count_launch();
  B200_CHECK_LAUNCH("attention plan (kv)");
  attn_plan_kernel<false><<<1, PLAN_THREADS, 0, st>>>(p.g, hdr_q, reinterpret_cast<int2 *>(hdr_q + 1), max_items);
  count_launch();
  B200_CHECK_LAUNCH("attention plan (q)");
  int64_t upper = (int64_t)max_items * a.H;
  int grid = (int)(upper < device_sm_count() ? upper : device_sm_count());
  {
    auto kern = hstu_attn_bwd_dkdv_sm100_kernel<D, IS_BF16>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::DYN_BYTES);
    if (e != cudaSuccess) return check_cuda(e, "backward smem attribute");
    BwdParams pk = p;
    pk.plan = hdr_kv;
    pk.items = reinterpret_cast<int2 *>(hdr_kv + 1);
    pk.status = &hdr_kv->status;
    kern<<<grid, BWD_THREADS, SM::DYN_BYTES, st>>>(mq, mk, mv, mdo, pk);
    count_launch();
    B200_CHECK_LAUNCH("tcgen05 attention backward (dk, dv)");
  }
  {
    auto kern = hstu_attn_bwd_dq_sm100_kernel<D, IS_BF16>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::DYN_BYTES);
    if (e != cudaSuccess) return check_cuda(e, "backward smem attribute");
    BwdParams pq = p;
    pq.plan = hdr_q;
    pq.items = reinterpret_cast<int2 *>(hdr_q + 1);
    pq.status = &hdr_q->status;
    kern<<<grid, BWD_THREADS, SM::DYN_BYTES, st>>>(mq, mk, mv, mdo, pq);
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
