// Jagged HSTU attention forward on Blackwell tensor cores (tcgen05 + TMEM + TMA), bf16 / fp16,
// head dimension 64 or 128 (d_qk == d_v).
//
//   out[i] = scale_i * sum_j mask(i,j) * SiLU(alpha * q_i.k_j) * v_j
//
// One persistent CTA per SM takes work items from a longest-first list (the first one by CTA
// index, the rest through an atomic counter); an item is a pair of consecutive 128-row query
// tiles (A, B) of one sequence and one head, which share every K/V tile they visit.  Fourteen
// warps, specialised:
//   warp 0       TMA producer: the two Q tiles once per item, K and V tiles through 2-stage
//                rings; claims the next item and publishes it to the other warps
//   warp 1       MMA issuer (one lane): S_X = Q_X K^T into TMEM, O_X += P_X V with P_X read back
//                from TMEM (X = A, B); owns TMEM allocation.  While the last kv tile of an item
//                is being finished it already issues the first S tiles of the next item.
//   warps 2-9    activation: all eight work on one score tile at a time (A, B, A, ...), one query
//                row per thread, half the columns per warpgroup: tcgen05.ld S -> SiLU (one MUFU
//                tanh per pair of scores) -> mask (only on tiles that are not fully visible, from
//                a per-row bit mask) -> 16-bit P written over S in TMEM
//   warps 10-13  epilogue: O_X (fp32, TMEM) -> scale -> 16-bit -> global, valid rows only, while
//                the activation warps are already busy with the next item
// The issue order  PV_A(j), S_A(j+1), PV_B(j), S_B(j+1)  keeps the tensor pipe busy with tile B
// while the CUDA cores activate tile A and vice versa.  TMEM: S_A, S_B, O_A, O_B = 4 x 128
// columns.
//
// K/V tiles that straddle the end of a sequence pull rows of the next sequence (or TMA zero
// fill); their columns are zeroed by the mask.  Rows past the sequence end are computed and
// never stored.  Which kv tiles an item visits follows the block-skipping rule of attn_plan.cuh
// (causal bound, local-window bound, contextual prefix, target rows' own diagonal block).
#include <stdlib.h>

#include "attn_plan.cuh"
#include "sm100_ptx.cuh"

namespace b200hstu {

using namespace ptx;

int make_tile_map(CUtensorMap *m, const void *base, int64_t rows, int64_t cols, int64_t row_stride_elems,
                  int elem_bytes, bool is_bf16);
int device_sm_count();
void fill_pdl_config(cudaLaunchConfig_t *cfg, cudaLaunchAttribute *attr, int grid, int threads, size_t smem,
                     cudaStream_t st);

namespace {

constexpr int FWD_THREADS = 448;
constexpr int FWD_SCHED_CONSUMERS = 13;  // MMA warp, 8 activation warps, 4 epilogue warps: one arrival each
constexpr int KV_STAGES = 2;

struct FwdParams {
  AttnGeomParams g;
  PlanHeader *plan;
  const ItemDesc *items;
  int *status;
  void *out;
  int64_t o_rs, o_hs;
  const float *attn_scale;
  int64_t attn_scale_numel;
  const float *bias;       // bias_by_distance as given (element-wise path)
  int bias_numel;
  const float *bias_ext;   // centre of the signed-distance table (see BiasTable); NULL = no bias
  float half_alpha;   // alpha / 2
  float inv_n;        // 1 / max_seq_len
  int H;
  int wide_stores;    // out rows are 32-byte aligned
  // optional timeline of CTA 0 (4 roles x TRACE_RECORDS records of {SM clock, tag}); NULL = off
  ulonglong2 *trace;
};

template <int D>
struct FwdSmem {
  static constexpr int CHUNKS = D / 64;                 // 64-column (128-byte) TMA boxes per tile
  static constexpr int TILE_BYTES = TILE * D * 2;       // one Q / K / V tile
  static constexpr int CHUNK_BYTES = TILE * 128;        // 128 rows x 128 bytes
  static constexpr int Q_OFF = 0;                       // Q_A, Q_B
  static constexpr int K_OFF = Q_OFF + 2 * TILE_BYTES;
  static constexpr int V_OFF = K_OFF + KV_STAGES * TILE_BYTES;
  static constexpr int BAR_OFF = V_OFF + KV_STAGES * TILE_BYTES;
  static constexpr int NUM_BARS = 4 + 4 * KV_STAGES + 8 + 2 * SCHED_SLOTS;
  static constexpr int MISC_OFF = BAR_OFF + NUM_BARS * 8;
  static constexpr int SCHED_OFF = MISC_OFF + 64;
  static constexpr int TOTAL = SCHED_OFF + SCHED_SLOTS * 128;   // ring of work items (PairGeom slots)
  // slack for manual 1024-byte alignment; at least 116 KB so that two CTAs (each of which
  // allocates all 512 TMEM columns) can never share an SM
  static constexpr int DYN_BYTES = (TOTAL + 1024) > 116 * 1024 ? (TOTAL + 1024) : 116 * 1024;
};

template <bool IS_BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if (IS_BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&v);
}

// tanh and fma on two packed 16-bit values: one MUFU and one FMA-pipe instruction per pair
template <bool IS_BF16>
__device__ __forceinline__ uint32_t silu_pair(float h0, float h1, uint32_t keep = 0xffffffffu) {
  uint32_t hh, t, r;
  if (IS_BF16) {
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hh) : "f"(h1), "f"(h0));
    hh &= keep;
    asm("tanh.approx.bf16x2 %0, %1;" : "=r"(t) : "r"(hh));
    asm("fma.rn.bf16x2 %0, %1, %2, %1;" : "=r"(r) : "r"(hh), "r"(t));
  } else {
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(hh) : "f"(h1), "f"(h0));
    hh &= keep;
    asm("tanh.approx.f16x2 %0, %1;" : "=r"(t) : "r"(hh));
    asm("fma.rn.f16x2 %0, %1, %2, %1;" : "=r"(r) : "r"(hh), "r"(t));
  }
  return r;
}

// 32 scores -> 16 packed P values.  silu(x) = h + h tanh(h) with h = x / 2, evaluated on packed
// 16-bit pairs (the result is rounded to 16 bits for the tensor core anyway).  Masked-out scores
// are replaced by h = 0 before the activation: silu(0) = 0 exactly.  fp16 inputs are clamped so
// that the activation cannot overflow the format.
template <bool IS_BF16, bool MASKED>
__device__ __forceinline__ void silu_chunk(const uint32_t (&r)[32], uint32_t (&packed)[16], float half_alpha,
                                           uint32_t bits) {
  const PairMasks pm(bits);
#pragma unroll
  for (int x = 0; x < 16; ++x) {
    float h0, h1;
    mul2(__uint_as_float(r[2 * x]), __uint_as_float(r[2 * x + 1]), half_alpha, h0, h1);
    if (!IS_BF16) {
      h0 = fminf(fmaxf(h0, -30000.f), 30000.f);
      h1 = fminf(fmaxf(h1, -30000.f), 30000.f);
    }
    packed[x] = MASKED ? silu_pair<IS_BF16>(h0, h1, pm.pair(x)) : silu_pair<IS_BF16>(h0, h1);
  }
}

// The same with a relative position bias: bp points at the table entry of (this row, first column
// of the chunk); the entry of column k is bp[-k] (already halved).
template <bool IS_BF16>
__device__ __forceinline__ void silu_chunk_bias(const uint32_t (&r)[32], uint32_t (&packed)[16], float half_alpha,
                                                uint32_t bits, const float *bp) {
  const PairMasks pm(bits);
#pragma unroll
  for (int x = 0; x < 16; ++x) {
    float h0 = fmaf(__uint_as_float(r[2 * x]), half_alpha, __ldg(bp - 2 * x));
    float h1 = fmaf(__uint_as_float(r[2 * x + 1]), half_alpha, __ldg(bp - 2 * x - 1));
    if (!IS_BF16) {
      h0 = fminf(fmaxf(h0, -30000.f), 30000.f);
      h1 = fminf(fmaxf(h1, -30000.f), 30000.f);
    }
    packed[x] = silu_pair<IS_BF16>(h0, h1, pm.pair(x));
  }
}

// Exact element-wise path: sequences outside the regular domain (with or without a bias).
template <bool IS_BF16>
__device__ __forceinline__ void silu_chunk_exact(const uint32_t (&r)[32], uint32_t (&packed)[16], float half_alpha,
                                              const SeqMask m, int i, int id_i, int col0, const float *bias,
                                              int bias_numel) {
#pragma unroll
  for (int x = 0; x < 16; ++x) {
    float pv[2];
#pragma unroll
    for (int y = 0; y < 2; ++y) {
      const int jj = col0 + 2 * x + y;
      float hh = __uint_as_float(r[2 * x + y]) * half_alpha;
      if (bias != nullptr) {
        int dist = i > jj ? i - jj : jj - i;
        if (dist < bias_numel) hh += 0.5f * bias[dist];
      }
      float val = fmaf(hh, tanh_approx(hh), hh);
      bool valid = i < m.L && jj < m.L && m.valid_ids(i, jj, id_i, m.id(jj));
      pv[y] = valid ? val : 0.f;
    }
    packed[x] = pack2<IS_BF16>(pv[0], pv[1]);
  }
}

// ---------------------------------------------------------------------------------------
// Work items travel from the producer warp to the other warps as ready-made geometry (128 bytes
// in a 4-slot shared-memory ring): the tile ranges are worked out once per item, by the warp with
// the most slack, a whole item ahead of their use.  Code that runs once per item is fetched
// cold, so the less of it the consumers execute at an item boundary the shorter the boundary.
// ---------------------------------------------------------------------------------------
struct __align__(16) PairGeom {
  int idx;                   // (item, head) index; >= number of (item, head) pairs: no more work
  int start, len, nt;        // first token row, untruncated length, number of targets
  int m0, L, u, regular;     // first row of tile A, rows that take part, first target, closed forms valid
  int max_id, has_b, n_tiles, t_lo;
  int n_main, extra0, extra1, a_lo;      // union of the kv tiles of A and B: [t_lo, t_lo + n_main) + extras
  int a_hi, a_x, a_n, b_lo;              // kv tiles of A: [a_lo, a_hi) + a_x (a_n in total); likewise B
  int b_hi, b_x, b_n, fa_lo;             // fully visible kv tiles of A: [fa_lo, fa_hi); likewise B
  int fa_hi, fb_lo, fb_hi, q_row;        // q_row: row of tile A's first query in the q / out tensors
  int pad[4];
  __device__ __forceinline__ int tile_at(int j) const { return j < n_main ? t_lo + j : (j == n_main ? extra0 : extra1); }
  __device__ __forceinline__ bool visits(int X, int t) const {
    const int lo = X ? b_lo : a_lo, hi = X ? b_hi : a_hi, x = X ? b_x : a_x;
    return (t >= lo && t < hi) || t == x;
  }
};
constexpr int GEOM_INTS = 28;

__device__ __forceinline__ void geom_from_pair(PairGeom &g, const PairItem &pr, int idx, int delta) {
  g.idx = idx;
  g.start = pr.A.start; g.len = pr.A.len; g.nt = pr.A.nt;
  g.m0 = pr.A.m0; g.L = pr.A.m.L; g.u = pr.A.u; g.regular = pr.A.regular ? 1 : 0;
  g.max_id = pr.A.m.max_id; g.has_b = pr.hasB ? 1 : 0; g.n_tiles = pr.n_tiles; g.t_lo = pr.t_lo;
  g.n_main = pr.n_main; g.extra0 = pr.extra0; g.extra1 = pr.extra1;
  g.a_lo = pr.A.t_lo; g.a_hi = pr.A.t_lo + pr.A.n_main; g.a_x = pr.A.extra_tile; g.a_n = pr.A.n_tiles;
  g.b_lo = pr.B.t_lo; g.b_hi = pr.B.t_lo + pr.B.n_main; g.b_x = pr.B.extra_tile; g.b_n = pr.B.n_tiles;
  const FullRange fa = full_tile_range(pr.A), fb = full_tile_range(pr.B);
  g.fa_lo = fa.lo; g.fa_hi = fa.hi; g.fb_lo = fb.lo; g.fb_hi = fb.hi;
  // cached inference: q / out hold `delta` rows per sequence; otherwise they are jagged like k / v
  g.q_row = delta > 0 ? pr.A.b * delta + pr.A.mt * TILE : pr.A.start + pr.A.m0;
}
// item ordinals n = 0, 1, 2, ... use slot n % SCHED_SLOTS
__device__ __forceinline__ bool geom_publish(const WaitCtx &wc, uint8_t *ring, uint32_t full0, uint32_t empty0,
                                             uint32_t n, const PairGeom &g) {
  const uint32_t slot = n & (SCHED_SLOTS - 1);
  if (!mbar_wait(wc, empty0 + 8 * slot, ((n / SCHED_SLOTS) & 1) ^ 1, 901)) return false;
  int4 *dst = reinterpret_cast<int4 *>(ring + slot * 128);
  const int4 *src = reinterpret_cast<const int4 *>(&g);
#pragma unroll
  for (int i = 0; i < 7; ++i) dst[i] = src[i];
  asm volatile("fence.acq_rel.cta;" ::: "memory");
  mbar_arrive(full0 + 8 * slot);
  return true;
}
__device__ __forceinline__ bool geom_fetch(const WaitCtx &wc, const uint8_t *ring, uint32_t full0, uint32_t empty0,
                                           uint32_t n, PairGeom &g, bool arrive) {
  const uint32_t slot = n & (SCHED_SLOTS - 1);
  if (!mbar_wait(wc, full0 + 8 * slot, (n / SCHED_SLOTS) & 1, 902)) return false;
  const volatile int *src = reinterpret_cast<const volatile int *>(ring + slot * 128);
  int *dst = reinterpret_cast<int *>(&g);
#pragma unroll
  for (int i = 0; i < GEOM_INTS; ++i) dst[i] = src[i];
  __syncwarp();
  if (arrive) mbar_arrive(empty0 + 8 * slot);
  return true;
}

// One score tile on the element-wise path, kept out of line: it is rarely taken and several
// times the size of the interval paths, which should stay close together in the instruction
// cache.  Same steps as the inline path: scores to registers, P over the thread's own S columns.
template <bool IS_BF16>
__device__ __noinline__ void exact_tile(uint32_t tS, int wg, float half_alpha, SeqMask m, int i, int col0,
                                        const float *bias, int bias_numel) {
  uint32_t sreg[2][32];
  tmem_ld32(tS + wg * 64, sreg[0]);
  tmem_ld32(tS + wg * 64 + 32, sreg[1]);
  tc_wait_ld();
  const int id_i = m.id(i);
  uint32_t packed[16];
  silu_chunk_exact<IS_BF16>(sreg[0], packed, half_alpha, m, i, id_i, col0, bias, bias_numel);
  tmem_st16(tS + wg * 64, packed);
  silu_chunk_exact<IS_BF16>(sreg[1], packed, half_alpha, m, i, id_i, col0 + 32, bias, bias_numel);
  tmem_st16(tS + wg * 64 + 16, packed);
}

// One partially visible score tile on the regular domain (row intervals), also out of line: the
// loop over fully visible tiles is the hot one.
template <bool IS_BF16>
__device__ __noinline__ void masked_tile(uint32_t tS, int wg, float half_alpha, int lo, int hi, int ctx_hi, int self,
                                         int col0, int L) {
  uint32_t sreg[2][32];
  tmem_ld32(tS + wg * 64, sreg[0]);
  tmem_ld32(tS + wg * 64 + 32, sreg[1]);
  tc_wait_ld();
  RowInterval ri;
  ri.lo = lo;
  ri.hi = hi;
  ri.ctx_hi = ctx_hi;
  ri.self = self;
  const uint32_t b0 = row_mask_bits(ri, col0, L), b1 = row_mask_bits(ri, col0 + 32, L);
  uint32_t p0[16], p1[16];
  silu_chunk<IS_BF16, true>(sreg[0], p0, half_alpha, b0);
  tmem_st16(tS + wg * 64, p0);
  silu_chunk<IS_BF16, true>(sreg[1], p1, half_alpha, b1);
  tmem_st16(tS + wg * 64 + 16, p1);
}

template <int D, bool IS_BF16, bool ONE_PATH, bool BIAS>
__global__ void __launch_bounds__(FWD_THREADS, 1)
    hstu_attn_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                               const __grid_constant__ CUtensorMap tmap_v, const FwdParams p) {
  using SM = FwdSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base + SM::Q_OFF;   // Q_A at sQ, Q_B at sQ + TILE_BYTES
  const uint32_t sK = smem_base + SM::K_OFF;
  const uint32_t sV = smem_base + SM::V_OFF;
  const uint32_t bars = smem_base + SM::BAR_OFF;
  // barrier map
  const uint32_t q_full = bars + 0, q_empty = bars + 16;   // [2]: Q_A, Q_B
  const uint32_t k_full = bars + 32, k_empty = k_full + 8 * KV_STAGES;
  const uint32_t v_full = k_empty + 8 * KV_STAGES, v_empty = v_full + 8 * KV_STAGES;
  const uint32_t s_full = v_empty + 8 * KV_STAGES;   // [2]: S_A, S_B ready
  const uint32_t p_full = s_full + 16;               // [2]: P_A, P_B written
  const uint32_t o_full = p_full + 16;               // [2]: O_A, O_B complete
  const uint32_t o_empty = o_full + 16;              // [2]: O_A, O_B read out
  const uint32_t sched_full = o_empty + 16;          // [SCHED_SLOTS] next work item published
  const uint32_t sched_empty = sched_full + 8 * SCHED_SLOTS;
  uint8_t *sched_ring = smem_gen + SM::SCHED_OFF;
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + SM::MISC_OFF);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + SM::MISC_OFF + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  WaitCtx wc{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int x = 0; x < 2; ++x) {
      mbar_init(q_full + 8 * x, 1);
      mbar_init(q_empty + 8 * x, 1);
    }
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(k_full + 8 * s, 1);
      mbar_init(k_empty + 8 * s, 1);
      mbar_init(v_full + 8 * s, 1);
      mbar_init(v_empty + 8 * s, 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(s_full + 8 * x, 1);
      mbar_init(p_full + 8 * x, 8);
      mbar_init(o_full + 8 * x, 1);
      mbar_init(o_empty + 8 * x, 4);
    }
    for (int x = 0; x < SCHED_SLOTS; ++x) {
      mbar_init(sched_full + 8 * x, 1);
      mbar_init(sched_empty + 8 * x, FWD_SCHED_CONSUMERS);
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
  // everything above overlapped with the planning kernel; its list is read from here on
  grid_dependency_wait();
  const int num_items = p.plan->num_items * p.H;

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
      PairGeom g;
      {
        const ItemDesc d = load_desc(p.items, blockIdx.x / p.H);
        PairItem pr;
        fill_pair_item(pr, p.g, d.b, d.t, d.start, d.len, d.nt);
        geom_from_pair(g, pr, blockIdx.x, p.g.delta);
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
        PairGeom ng = g;
        tr.mark(1);
        // order of requests = order of first use: Q_A, K(0) feed S_A; Q_B feeds S_B; then V(0)
        for (int j = 0; j < g.n_tiles; ++j, ++kv_cnt) {
          const int s = kv_cnt % KV_STAGES;
          const uint32_t par = ((kv_cnt / KV_STAGES) & 1) ^ 1;
          const int row = g.start + g.tile_at(j) * TILE;
          if (j == 0) {
            ok = mbar_wait(wc, q_empty, (it_cnt & 1) ^ 1, 101);
            if (!ok) break;
            tr.mark(2);
            mbar_arrive_expect_tx(q_full, SM::TILE_BYTES);
#pragma unroll
            for (int c = 0; c < SM::CHUNKS; ++c)
              tma_load_2d(sQ + c * SM::CHUNK_BYTES, &tmap_q, h * D + c * 64, g.q_row, q_full);
          }
          ok = mbar_wait(wc, k_empty + 8 * s, par, 102);
          if (!ok) break;
          tr.mark(3);
          mbar_arrive_expect_tx(k_full + 8 * s, SM::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < SM::CHUNKS; ++c)
            tma_load_2d(sK + s * SM::TILE_BYTES + c * SM::CHUNK_BYTES, &tmap_k, h * D + c * 64, row, k_full + 8 * s);
          if (j == 0) {
            // Q_B is requested for every item (a pair without a second tile reads rows that are
            // never used), which keeps the barrier phases of the two Q buffers in step
            ok = mbar_wait(wc, q_empty + 8, (it_cnt & 1) ^ 1, 104);
            if (!ok) break;
            mbar_arrive_expect_tx(q_full + 8, SM::TILE_BYTES);
#pragma unroll
            for (int c = 0; c < SM::CHUNKS; ++c)
              tma_load_2d(sQ + SM::TILE_BYTES + c * SM::CHUNK_BYTES, &tmap_q, h * D + c * 64, g.q_row + TILE,
                          q_full + 8);
          }
          ok = mbar_wait(wc, v_empty + 8 * s, par, 103);
          if (!ok) break;
          tr.mark(4);
          mbar_arrive_expect_tx(v_full + 8 * s, SM::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < SM::CHUNKS; ++c)
            tma_load_2d(sV + s * SM::TILE_BYTES + c * SM::CHUNK_BYTES, &tmap_v, h * D + c * 64, row, v_full + 8 * s);
          if (j == 0) nidx = atomicAdd(&p.plan->next, 1);
          if (j == j_desc && nidx < num_items) nd = load_desc(p.items, nidx / p.H);
          if (j == j_geom) {
            ng.idx = nidx;
            if (nidx < num_items) {
              PairItem np;
              fill_pair_item(np, p.g, nd.b, nd.t, nd.start, nd.len, nd.nt);
              geom_from_pair(ng, np, nidx, p.g.delta);
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
    // ------------------------------------------------------------------ MMA issuer
    // All 32 lanes run the control flow and the barrier waits, so everything that feeds the MMA
    // descriptors stays warp-uniform; one elected lane issues the tcgen05 instructions.
    if ((int)blockIdx.x < num_items) {
      constexpr uint32_t FMT = IS_BF16 ? 1u : 0u;
      const uint32_t idesc_s = make_idesc(FMT, FMT, 0, 0, TILE, TILE);   // S = Q K^T  (both K-major)
      const uint32_t idesc_o = make_idesc(FMT, FMT, 0, 1, TILE, D);      // O = P V    (V is MN-major)
      uint32_t it_cnt = 0, kv_cnt = 0;
      uint32_t tile_cnt[2] = {0, 0};   // S/P tiles processed so far per query tile (barrier phases)
      uint32_t item_cnt[2] = {0, 0};   // items in which the query tile took part
      bool ok = true;
      Tracer tr;
      tr.init(p.trace, 1, lane == 0);

      // S_X = Q_X K^T for kv ring slot of global tile counter g; `last`: Q_X has no reader left
      auto issue_s = [&](int X, uint32_t g, bool last) {
        const int s = g % KV_STAGES;
        const uint64_t q_desc = make_smem_desc(sQ + X * SM::TILE_BYTES, 16, 1024);
        const uint64_t k_desc = make_smem_desc(sK + s * SM::TILE_BYTES, 16, 1024);
        const uint32_t dcol = tmem_base + X * 128;
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = (ks / 4) * SM::CHUNK_BYTES + (ks % 4) * 32;
            mma_ss(dcol, desc_advance(q_desc, off), desc_advance(k_desc, off), idesc_s, ks > 0);
          }
          tc_commit(s_full + 8 * X);
          if (last) tc_commit(q_empty + 8 * X);
        }
        __syncwarp();
      };
      // a query tile that takes no part in an item (a pair without a second tile) hands its Q buffer back at once
      auto release_q = [&](int X) {
        if (elect_one()) tc_commit(q_empty + 8 * X);
        __syncwarp();
      };

      PairGeom g;
      ok = geom_fetch(wc, sched_ring, sched_full, sched_empty, 0, g, lane == 0);
      bool pre_issued = false;   // the S tiles of this item's first kv tile were issued during the previous item
      for (; ok && g.idx < num_items; ++it_cnt) {
        tr.mark(10);
        const int n = g.n_tiles;
        int remaining[2] = {g.a_n, g.b_n};
        int s_left[2] = {g.a_n, g.b_n};      // S tiles of this item still to be issued per query tile
        bool started[2] = {false, false};
        if (!pre_issued) {
          // first kv tile: both S
          const int t0 = g.tile_at(0);
          ok = mbar_wait(wc, k_full + 8 * (kv_cnt % KV_STAGES), (kv_cnt / KV_STAGES) & 1, 201);
          if (!ok) break;
#pragma unroll
          for (int X = 0; X < 2; ++X) {
            ok = mbar_wait(wc, q_full + 8 * X, it_cnt & 1, 202);
            if (!ok) break;
            tc_fence_after();
            if (g.visits(X, t0)) {
              --s_left[X];
              issue_s(X, kv_cnt, s_left[X] == 0);
            } else if (s_left[X] == 0) {
              release_q(X);
            }
          }
          if (!ok) break;
          tr.mark(11);
          if (elect_one()) tc_commit(k_empty + 8 * (kv_cnt % KV_STAGES));
          __syncwarp();
        } else {
          // the first kv tile's S tiles were issued early: account for them
          const int t0 = g.tile_at(0);
          if (g.visits(0, t0)) --s_left[0];
          if (g.visits(1, t0)) --s_left[1];
        }
        pre_issued = false;
        PairGeom ng;
        ng.idx = num_items;
        bool next_item = false;
        for (int j = 0; j < n; ++j, ++kv_cnt) {
          const int t = g.tile_at(j);
          const bool has_next = j + 1 < n;
          const int tn = has_next ? g.tile_at(j + 1) : -1;
          const int s = kv_cnt % KV_STAGES;
          const int sn = (kv_cnt + 1) % KV_STAGES;
          bool v_ready = false, kn_ready = false;
#pragma unroll
          for (int X = 0; X < 2; ++X) {
            const bool here = g.visits(X, t);
            const bool next = has_next && g.visits(X, tn);
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
              // V tile: [128 kv rows][D], 64-column blocks 16 KB apart; 16 kv rows per MMA = 2 KB.
              // P: K steps 0-3 sit in columns [0,32) of the score region, 4-7 in [64,96).
              const uint64_t v_desc = make_smem_desc(sV + s * SM::TILE_BYTES, SM::CHUNK_BYTES, 1024);
              const uint32_t a_tmem = tmem_base + X * 128;
              const uint32_t o_tmem = tmem_base + 256 + X * 128;
              const bool last = --remaining[X] == 0;
              if (elect_one()) {
#pragma unroll
                for (int ks = 0; ks < TILE / 16; ++ks)
                  mma_ts(o_tmem, a_tmem + (ks / 4) * 64 + (ks % 4) * 8, desc_advance(v_desc, ks * 2048), idesc_o,
                         (started[X] || ks > 0) ? 1u : 0u);
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
              --s_left[X];
              issue_s(X, kv_cnt + 1, s_left[X] == 0);
              tr.mark(18 + X);
            }
            if (j == n - 1) {
              // Last kv tile: the S_X buffer is free from here on.  Take the next item (X = 0)
              // and issue its first S_X ahead of what remains of this item, so that the
              // activation warps find a score tile waiting when they finish this item.  Q_X of
              // the next item was requested when this item's last S_X was issued; its first K tile
              // goes to the ring slot after this one.
              if (X == 0) {
                ok = geom_fetch(wc, sched_ring, sched_full, sched_empty, it_cnt + 1, ng, lane == 0);
                if (!ok) break;
                next_item = ng.idx < num_items;
                if (next_item) {
                  ok = mbar_wait(wc, k_full + 8 * sn, ((kv_cnt + 1) / KV_STAGES) & 1, 210);
                  if (!ok) break;
                }
              }
              if (next_item) {
                ok = mbar_wait(wc, q_full + 8 * X, (it_cnt + 1) & 1, 209);
                if (!ok) break;
                tc_fence_after();
                const int nt0 = ng.tile_at(0);
                const int n_x = X ? ng.b_n : ng.a_n;
                if (ng.visits(X, nt0)) issue_s(X, kv_cnt + 1, n_x == 1);
                else if (n_x == 0) release_q(X);
                tr.mark(21);
              }
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
          if (j == n - 1 && next_item) pre_issued = true;
          if (elect_one()) {
            tc_commit(v_empty + 8 * s);
            if (has_next || (j == n - 1 && next_item)) tc_commit(k_empty + 8 * sn);
          }
          __syncwarp();
        }
        if (!ok) break;
        g = ng;
      }
    }
  } else if (warp < 10) {
    // ------------------------------------------------------------------ activation warps
    // All eight warps work on one score tile at a time (A, then B, then A ...): the activation is
    // bound by the MUFU rate of the whole SM, so a tile is finished soonest - and its P handed
    // back to the tensor pipe soonest - when every warp works on it.  Warps 2-5 take columns
    // [0,64) of the tile, warps 6-9 columns [64,128); thread = one query row.  P (16-bit) goes
    // over the first half of the columns the thread has read itself - [0,32) or [64,96) - so the
    // warps need no barrier among themselves.
    const int wg = warp >= 6 ? 1 : 0;
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may touch
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    uint32_t tiles_a = 0, tiles_b = 0;   // score tiles processed so far (barrier phases)
    bool ok = true;
    Tracer tr;
    tr.init(p.trace, 2 + wg, quad == 2 && lane == 0);
    if ((int)blockIdx.x < num_items) {
      PairGeom g;
      ok = geom_fetch(wc, sched_ring, sched_full, sched_empty, 0, g, lane == 0);
      uint32_t item_no = 0;
      while (ok && g.idx < num_items) {
        const int L = g.L;
        SeqMask m;
        m.L = g.L; m.max_id = g.max_id; m.c = p.g.c; m.W = p.g.W; m.F = p.g.F;
        const bool exact_only = !g.regular;
        const int iA = g.m0 + row_in_tile, iB = g.m0 + TILE + row_in_tile;
        RowInterval riA, riB;
        {
          TileItem ti;   // the fields row_interval() reads
          ti.m = m;
          ti.u = g.u;
          riA = row_interval(ti, iA);
          riB = row_interval(ti, iB);
        }
        const int n_tiles = g.n_tiles;
        for (int j = 0; j < n_tiles && ok; ++j) {
          const int t = g.tile_at(j);
          // the loop over the two query tiles stays rolled: one copy of the hot code
#pragma unroll 1
          for (int X = 0; X < 2; ++X) {
            const bool isb = X != 0;
            if (!g.visits(X, t)) continue;
            const int f_lo = isb ? g.fb_lo : g.fa_lo, f_hi = isb ? g.fb_hi : g.fa_hi;
            const bool full = !exact_only && t >= f_lo && t < f_hi;
            const uint32_t tS = tmem_base + X * 128 + lane_off;
            const int col0 = t * TILE + wg * 64;
            tr.mark(30);
            ok = mbar_wait(wc, s_full + 8 * X, (isb ? tiles_b : tiles_a) & 1, 301);
            if (!ok) break;
            tc_fence_after();
            tr.mark(31);
            if (!exact_only) {
              // Fully and partially visible tiles share everything but the activation block
              // itself.  ONE_PATH (short sequences, where every third tile is partially visible):
              // the masking variant serves both, so the loop has one block that stays in the
              // instruction cache; otherwise fully visible tiles take a variant without the
              // per-element selects, which is what long sequences mostly run.
              uint32_t b0 = 0xffffffffu, b1 = 0xffffffffu;
              if (!full) {
                RowInterval ri;
                ri.lo = isb ? riB.lo : riA.lo;
                ri.hi = isb ? riB.hi : riA.hi;
                ri.ctx_hi = isb ? riB.ctx_hi : riA.ctx_hi;
                ri.self = isb ? riB.self : riA.self;
                b0 = row_mask_bits(ri, col0, L);
                b1 = row_mask_bits(ri, col0 + 32, L);
              }
              uint32_t sreg[2][32];
              tmem_ld32(tS + wg * 64, sreg[0]);
              tmem_ld32(tS + wg * 64 + 32, sreg[1]);
              tc_wait_ld();
              tr.mark(32);
              // one straight-line block, so that the second half's MUFU work is scheduled under
              // the first half's packing and store
              uint32_t p0[16], p1[16];
              if (BIAS) {
                // signed distance of (this row, first column of the chunk)
                const float *bp = p.bias_ext + ((isb ? iB : iA) - col0);
                silu_chunk_bias<IS_BF16>(sreg[0], p0, p.half_alpha, b0, bp);
                tmem_st16(tS + wg * 64, p0);
                silu_chunk_bias<IS_BF16>(sreg[1], p1, p.half_alpha, b1, bp - 32);
                tmem_st16(tS + wg * 64 + 16, p1);
              } else if (!ONE_PATH && full) {
                silu_chunk<IS_BF16, false>(sreg[0], p0, p.half_alpha, b0);
                tmem_st16(tS + wg * 64, p0);
                silu_chunk<IS_BF16, false>(sreg[1], p1, p.half_alpha, b1);
                tmem_st16(tS + wg * 64 + 16, p1);
              } else {
                silu_chunk<IS_BF16, true>(sreg[0], p0, p.half_alpha, b0);
                tmem_st16(tS + wg * 64, p0);
                silu_chunk<IS_BF16, true>(sreg[1], p1, p.half_alpha, b1);
                tmem_st16(tS + wg * 64 + 16, p1);
              }
            } else {
              exact_tile<IS_BF16>(tS, wg, p.half_alpha, m, isb ? iB : iA, col0, p.bias, p.bias_numel);
            }
            tr.mark(37);
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + 8 * X);
            tr.mark(33);
            if (isb) ++tiles_b; else ++tiles_a;
          }
        }
        if (!ok) break;
        ++item_no;
        ok = geom_fetch(wc, sched_ring, sched_full, sched_empty, item_no, g, lane == 0);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    // O (fp32, TMEM) -> scale -> 16-bit -> global; thread = one query row, valid rows only
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    uint32_t items_a = 0, items_b = 0;   // items in which each query tile took part (barrier phases)
    bool ok = true;
    if ((int)blockIdx.x < num_items) {
      PairGeom g;
      ok = geom_fetch(wc, sched_ring, sched_full, sched_empty, 0, g, lane == 0);
      uint32_t item_no = 0;
      while (ok && g.idx < num_items) {
        const int h = g.idx % p.H;
        const int L = g.L;
        // rolled: one copy of the store code serves both query tiles
#pragma unroll 1
        for (int X = 0; X < 2; ++X) {
          if (X == 1 && !g.has_b) continue;
          const int m0 = g.m0 + X * TILE;
          const int i = m0 + row_in_tile;
          ok = mbar_wait(wc, o_full + 8 * X, (X ? items_b : items_a) & 1, 302);
          if (!ok) break;
          tc_fence_after();
          const bool row_ok = i >= 0 && i < L;
          float scale = p.inv_n;
          if (p.attn_scale != nullptr && row_ok)
            scale = p.attn_scale_numel == 1 ? p.attn_scale[0] : p.attn_scale[(int64_t)g.start + i];
          uint16_t *orow = reinterpret_cast<uint16_t *>(p.out) +
                           (int64_t)(g.q_row + X * TILE + row_in_tile) * p.o_rs + (int64_t)h * p.o_hs;
          const uint32_t tO = tmem_base + 256 + X * 128 + lane_off;
          uint32_t r[2][32];
          tmem_ld32(tO, r[0]);
#pragma unroll
          for (int cc = 0; cc < D / 32; ++cc) {
            tc_wait_ld();
            if (cc + 1 < D / 32) tmem_ld32(tO + (cc + 1) * 32, r[(cc + 1) & 1]);
            if (row_ok) {
              const uint32_t(&v)[32] = r[cc & 1];
              uint4 o4[4];
#pragma unroll
              for (int x = 0; x < 4; ++x) {
                o4[x].x = pack2<IS_BF16>(__uint_as_float(v[8 * x + 0]) * scale, __uint_as_float(v[8 * x + 1]) * scale);
                o4[x].y = pack2<IS_BF16>(__uint_as_float(v[8 * x + 2]) * scale, __uint_as_float(v[8 * x + 3]) * scale);
                o4[x].z = pack2<IS_BF16>(__uint_as_float(v[8 * x + 4]) * scale, __uint_as_float(v[8 * x + 5]) * scale);
                o4[x].w = pack2<IS_BF16>(__uint_as_float(v[8 * x + 6]) * scale, __uint_as_float(v[8 * x + 7]) * scale);
              }
              // one row per thread: every lane of a store hits another 32-byte sector, so rows
              // that are 32-byte aligned are written in whole sectors (256-bit stores)
              if (p.wide_stores) {
                st_global_256(orow + cc * 32, o4[0], o4[1]);
                st_global_256(orow + cc * 32 + 16, o4[2], o4[3]);
              } else {
#pragma unroll
                for (int x = 0; x < 4; ++x) *reinterpret_cast<uint4 *>(orow + cc * 32 + x * 8) = o4[x];
              }
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(o_empty + 8 * X);
          if (X) ++items_b; else ++items_a;
          // rows at or beyond max_seq_len of an over-long sequence come back as zeros
          if (g.len > L && m0 + TILE >= L) {
            for (int r2 = L + row_in_tile; r2 < g.len; r2 += TILE) {
              uint16_t *zr = reinterpret_cast<uint16_t *>(p.out) + (int64_t)(g.start + r2) * p.o_rs + (int64_t)h * p.o_hs;
              for (int x = 0; x < D; x += 8) *reinterpret_cast<uint4 *>(zr + x) = make_uint4(0, 0, 0, 0);
            }
          }
        }
        if (!ok) break;
        ++item_no;
        ok = geom_fetch(wc, sched_ring, sched_full, sched_empty, item_no, g, lane == 0);
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

// scratch: [bias table (if any) | work list]
int64_t attn_tc_fwd_workspace_bytes(const b200_hstu_attn_args &a) {
  return bias_table_bytes(a.bias_by_distance, a.max_seq_len) + plan_bytes(a.total_L, a.B);
}

template <int D, bool IS_BF16, bool ONE_PATH, bool BIAS>
int launch_fwd_tc(const b200_hstu_attn_args &a, cudaStream_t st) {
  using SM = FwdSmem<D>;
  if (a.workspace == nullptr || a.workspace_bytes < attn_tc_fwd_workspace_bytes(a))
    return fail(B200_HSTU_EWORKSPACE, "attention forward needs %lld bytes of scratch, got %lld",
                (long long)attn_tc_fwd_workspace_bytes(a), (long long)a.workspace_bytes);
  CUtensorMap mq, mk, mv;
  int rc;
  const int64_t q_rows = a.delta_size > 0 ? (int64_t)a.B * a.delta_size : a.total_L;
  if ((rc = make_tile_map(&mq, a.q, q_rows, (int64_t)a.H * D, a.q_row_stride, 2, IS_BF16)) != 0) return rc;
  if ((rc = make_tile_map(&mk, a.k, a.total_L, (int64_t)a.H * D, a.k_row_stride, 2, IS_BF16)) != 0) return rc;
  if ((rc = make_tile_map(&mv, a.v, a.total_L, (int64_t)a.H * D, a.v_row_stride, 2, IS_BF16)) != 0) return rc;
  FwdParams p;
  p.g.seq_offsets = a.seq_offsets;
  p.g.num_targets = a.num_targets;
  p.g.B = a.B;
  p.g.H = a.H;
  p.g.max_seq_len = a.max_seq_len;
  p.g.W = a.max_attn_len;
  p.g.c = a.contextual_seq_len;
  p.g.F = a.min_full_attn_seq_len;
  p.g.delta = a.delta_size;
  const int64_t eb = bias_table_bytes(a.bias_by_distance, a.max_seq_len);
  uint8_t *lists = reinterpret_cast<uint8_t *>(a.workspace) + eb;
  BiasTable bt{a.bias_by_distance, a.bias_numel, reinterpret_cast<float *>(a.workspace), a.max_seq_len};
  PlanHeader *hdr = reinterpret_cast<PlanHeader *>(lists);
  ItemDesc *items = reinterpret_cast<ItemDesc *>(hdr + 1);
  p.plan = hdr;
  p.items = items;
  p.status = &hdr->status;
  p.out = a.out;
  p.o_rs = a.o_row_stride;
  p.o_hs = a.o_head_stride;
  p.attn_scale = a.attn_scale;
  p.attn_scale_numel = a.attn_scale_numel;
  p.bias = a.bias_by_distance;
  p.bias_numel = a.bias_numel;
  p.bias_ext = a.bias_by_distance ? bt.centre() : nullptr;
  p.half_alpha = 0.5f * a.alpha;
  p.inv_n = 1.f / (float)a.max_seq_len;
  p.H = a.H;
  p.wide_stores = (reinterpret_cast<uintptr_t>(a.out) & 31) == 0 && a.o_row_stride % 16 == 0 && a.o_head_stride % 16 == 0;
  // B200_HSTU_TRACE=1 and a scratch buffer with TRACE_BYTES of extra room: CTA 0 records a
  // timeline of its roles behind the work list (a profiling aid, off by default)
  p.trace = nullptr;
  {
    static const bool want_trace = getenv("B200_HSTU_TRACE") != nullptr;
    const int64_t need = attn_tc_fwd_workspace_bytes(a);
    if (want_trace && a.plan_mode == B200_HSTU_PLAN_OWN && a.workspace_bytes >= need + TRACE_BYTES)
      p.trace = reinterpret_cast<ulonglong2 *>(reinterpret_cast<uint8_t *>(a.workspace) + need);
  }
  const int max_items = (int)plan_max_items(a.total_L, a.B);
  const int64_t upper = (int64_t)max_items * a.H;
  const int grid = (int)(upper < device_sm_count() ? upper : device_sm_count());
  {
    ProfileScope prof(PROF_PLAN, st);
    if (a.plan_mode == B200_HSTU_PLAN_FOR_BACKWARD) {
      // one planning launch for the whole training step: the backward's two lists go behind this one
      const int64_t one = plan_bytes(a.total_L, a.B);
      if (a.workspace_bytes < eb + 3 * one)
        return fail(B200_HSTU_EWORKSPACE, "forward that plans the backward needs %lld bytes of scratch, got %lld",
                    (long long)(eb + 3 * one), (long long)a.workspace_bytes);
      PlanHeader *hdr_kv = reinterpret_cast<PlanHeader *>(lists + one);
      PlanHeader *hdr_q = reinterpret_cast<PlanHeader *>(lists + 2 * one);
      attn_plan3_kernel<PLAN_Q_PAIR><<<3, PLAN_THREADS, 0, st>>>(p.g, hdr, items, hdr_kv, reinterpret_cast<ItemDesc *>(hdr_kv + 1),
                                                    hdr_q, reinterpret_cast<ItemDesc *>(hdr_q + 1), max_items, grid, bt);
    } else {
      attn_plan_kernel<PLAN_Q_PAIR><<<1, PLAN_THREADS, 0, st>>>(p.g, hdr, items, max_items, grid, bt);
    }
  }
  count_launch();
  B200_CHECK_LAUNCH("attention plan");
  auto kern = hstu_attn_fwd_sm100_kernel<D, IS_BF16, ONE_PATH, BIAS>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::DYN_BYTES);
  if (e != cudaSuccess) return check_cuda(e, "forward smem attribute");
  {
    ProfileScope prof(PROF_ATTN_FWD, st);
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr;
    fill_pdl_config(&cfg, &attr, grid, FWD_THREADS, SM::DYN_BYTES, st);
    e = cudaLaunchKernelEx(&cfg, kern, mq, mk, mv, p);
    if (e != cudaSuccess) return check_cuda(e, "forward launch");
  }
  count_launch();
  B200_CHECK_LAUNCH("tcgen05 attention forward");
  return 0;
}

int attn_tc_fwd(const b200_hstu_attn_args &a, cudaStream_t st) {
  const bool bf = a.dtype == B200_HSTU_BF16;
  // a relative bias has its own instantiation (always the single masking activation block), so that
  // the common case carries none of its code
  if (a.bias_by_distance != nullptr) {
    if (a.dqk == 128) return bf ? launch_fwd_tc<128, true, true, true>(a, st) : launch_fwd_tc<128, false, true, true>(a, st);
    return bf ? launch_fwd_tc<64, true, true, true>(a, st) : launch_fwd_tc<64, false, true, true>(a, st);
  }
  const bool one_path = a.max_seq_len <= 2048;   // see ONE_PATH in the activation loop
  if (a.dqk == 128) {
    if (one_path) return bf ? launch_fwd_tc<128, true, true, false>(a, st) : launch_fwd_tc<128, false, true, false>(a, st);
    return bf ? launch_fwd_tc<128, true, false, false>(a, st) : launch_fwd_tc<128, false, false, false>(a, st);
  }
  if (one_path) return bf ? launch_fwd_tc<64, true, true, false>(a, st) : launch_fwd_tc<64, false, true, false>(a, st);
  return bf ? launch_fwd_tc<64, true, false, false>(a, st) : launch_fwd_tc<64, false, false, false>(a, st);
}

}  // namespace b200hstu
