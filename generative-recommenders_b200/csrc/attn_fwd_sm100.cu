// Jagged HSTU attention forward on Blackwell tensor cores (tcgen05 + TMEM + TMA), bf16 / fp16,
// head dimension 64 or 128 (d_qk == d_v).
//
//   out[i] = scale_i * sum_j mask(i,j) * SiLU(alpha * q_i.k_j) * v_j
//
// One persistent CTA per SM walks a longest-first list of (sequence, 128-row query tile) items
// crossed with the heads.  Inside a CTA the warps are specialised:
//   warp 0      TMA producer: Q tile once per item, K and V tiles through two 2-stage rings
//   warp 1      MMA issuer (one elected lane): S = Q K^T into a double-buffered TMEM
//               accumulator, O += P V with P read back from TMEM; owns TMEM alloc / dealloc
//   warps 2-5   128 threads, one query row each: tcgen05.ld S -> SiLU (one MUFU tanh) -> mask
//               (only on tiles that are not fully visible) -> bf16 P written over S in TMEM;
//               after the last kv tile they scale O and store the valid rows
// S(j+1) is issued before the SiLU of S(j) finishes, so the tensor pipe works on the next score
// tile while the CUDA cores activate the current one.  K/V tiles that straddle the end of a
// sequence pull rows of the next sequence (or TMA zero fill); their columns are zeroed by the
// element mask.  Rows past the sequence end are computed and never stored.
//
// The kv tiles an item visits come from the same block-skipping rule as the planning kernel:
// causal upper bound, local-window lower bound, contextual prefix, and for target-only tiles the
// tile's own diagonal block.
#include "attn_plan.cuh"
#include "sm100_ptx.cuh"

namespace b200hstu {

using namespace ptx;

namespace {

constexpr int FWD_THREADS = 192;
constexpr int KV_STAGES = 2;

struct FwdParams {
  AttnGeomParams g;
  const PlanHeader *plan;
  const int2 *items;
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
};

template <int D>
struct FwdSmem {
  static constexpr int CHUNKS = D / 64;                 // 64-column (128-byte) TMA boxes per tile
  static constexpr int TILE_BYTES = TILE * D * 2;       // one Q / K / V tile
  static constexpr int CHUNK_BYTES = TILE * 128;        // 128 rows x 128 bytes
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + TILE_BYTES;
  static constexpr int V_OFF = K_OFF + KV_STAGES * TILE_BYTES;
  static constexpr int BAR_OFF = V_OFF + KV_STAGES * TILE_BYTES;
  static constexpr int NUM_BARS = 2 + 4 * KV_STAGES + 2 + 2 + 2;
  static constexpr int MISC_OFF = BAR_OFF + NUM_BARS * 8;
  static constexpr int TOTAL = MISC_OFF + 64;
  // slack for manual 1024-byte alignment; at least 116 KB so that two CTAs (each of which
  // allocates all 512 TMEM columns) can never share an SM
  static constexpr int DYN_BYTES = (TOTAL + 1024) > 116 * 1024 ? (TOTAL + 1024) : 116 * 1024;
};

__device__ __forceinline__ uint32_t pack2(float a, float b, bool is_bf16) {
  if (is_bf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&v);
}

template <int D, bool IS_BF16>
__global__ void __launch_bounds__(FWD_THREADS, 1)
    hstu_attn_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                               const __grid_constant__ CUtensorMap tmap_v, const FwdParams p) {
  using SM = FwdSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base + SM::Q_OFF;
  const uint32_t sK = smem_base + SM::K_OFF;
  const uint32_t sV = smem_base + SM::V_OFF;
  const uint32_t bars = smem_base + SM::BAR_OFF;
  // barrier map
  const uint32_t q_full = bars + 0, q_empty = bars + 8;
  const uint32_t k_full = bars + 16, k_empty = k_full + 8 * KV_STAGES;
  const uint32_t v_full = k_empty + 8 * KV_STAGES, v_empty = v_full + 8 * KV_STAGES;
  const uint32_t s_full = v_empty + 8 * KV_STAGES, p_full = s_full + 16;
  const uint32_t o_full = p_full + 16, o_empty = o_full + 8;
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
    for (int s = 0; s < 2; ++s) {
      mbar_init(s_full + 8 * s, 1);
      mbar_init(p_full + 8 * s, 4);
    }
    mbar_init(o_full, 1);
    mbar_init(o_empty, 4);
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
  const uint32_t tS0 = tmem_base;            // S / P buffers: columns [0,128) and [128,256)
  const uint32_t tO = tmem_base + 256;       // O accumulator: D columns

  const int num_items = p.plan->num_items * p.H;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&tmap_q);
      prefetch_tmap(&tmap_k);
      prefetch_tmap(&tmap_v);
      uint32_t it_cnt = 0, kv_cnt = 0;
      bool ok = true;
      for (int idx = blockIdx.x; idx < num_items && ok; idx += gridDim.x, ++it_cnt) {
        const int2 e = p.items[idx / p.H];
        const int h = idx % p.H;
        TileItem it;
        load_item<false>(it, p.g, e.x, e.y);
        ok = mbar_wait(wc, q_empty, (it_cnt & 1) ^ 1, 101);
        if (!ok) break;
        mbar_arrive_expect_tx(q_full, SM::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < SM::CHUNKS; ++c)
          tma_load_2d(sQ + c * SM::CHUNK_BYTES, &tmap_q, h * D + c * 64, it.start + it.m0, q_full);
        for (int j = 0; j < it.n_tiles; ++j, ++kv_cnt) {
          const int s = kv_cnt % KV_STAGES;
          const uint32_t par = ((kv_cnt / KV_STAGES) & 1) ^ 1;
          const int row = it.start + it.tile_at(j) * TILE;
          ok = mbar_wait(wc, k_empty + 8 * s, par, 102);
          if (!ok) break;
          mbar_arrive_expect_tx(k_full + 8 * s, SM::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < SM::CHUNKS; ++c)
            tma_load_2d(sK + s * SM::TILE_BYTES + c * SM::CHUNK_BYTES, &tmap_k, h * D + c * 64, row, k_full + 8 * s);
          ok = mbar_wait(wc, v_empty + 8 * s, par, 103);
          if (!ok) break;
          mbar_arrive_expect_tx(v_full + 8 * s, SM::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < SM::CHUNKS; ++c)
            tma_load_2d(sV + s * SM::TILE_BYTES + c * SM::CHUNK_BYTES, &tmap_v, h * D + c * 64, row, v_full + 8 * s);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t FMT = IS_BF16 ? 1u : 0u;
      const uint32_t idesc_s = make_idesc(FMT, FMT, 0, 0, TILE, TILE);   // S = Q K^T  (both K-major)
      const uint32_t idesc_o = make_idesc(FMT, FMT, 0, 1, TILE, D);      // O = P V    (V is MN-major)
      const uint64_t q_desc = make_smem_desc(sQ, 16, 1024);
      uint32_t it_cnt = 0, kv_cnt = 0;
      bool ok = true;

      auto issue_s = [&](uint32_t g) -> bool {
        const int s = g % KV_STAGES;
        if (!mbar_wait(wc, k_full + 8 * s, (g / KV_STAGES) & 1, 201)) return false;
        tc_fence_after();
        const uint64_t k_desc = make_smem_desc(sK + s * SM::TILE_BYTES, 16, 1024);
        const uint32_t d = tS0 + (g & 1) * 128;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks / 4) * SM::CHUNK_BYTES + (ks % 4) * 32;
          mma_ss(d, desc_advance(q_desc, off), desc_advance(k_desc, off), idesc_s, ks > 0);
        }
        tc_commit(k_empty + 8 * s);
        tc_commit(s_full + 8 * (g & 1));
        return true;
      };

      for (int idx = blockIdx.x; idx < num_items && ok; idx += gridDim.x, ++it_cnt) {
        const int2 e = p.items[idx / p.H];
        TileItem it;
        load_item<false>(it, p.g, e.x, e.y);
        ok = mbar_wait(wc, q_full, it_cnt & 1, 202);
        if (!ok) break;
        const int n = it.n_tiles;
        for (int j = 0; j < n; ++j, ++kv_cnt) {
          if (j == 0) {
            ok = issue_s(kv_cnt);
            if (!ok) break;
          }
          if (j + 1 < n) {
            ok = issue_s(kv_cnt + 1);
            if (!ok) break;
          }
          if (j == n - 1) tc_commit(q_empty);  // every S of this item has been issued
          if (j == 0) {
            ok = mbar_wait(wc, o_empty, (it_cnt & 1) ^ 1, 203);
            if (!ok) break;
          }
          ok = mbar_wait(wc, p_full + 8 * (kv_cnt & 1), (kv_cnt >> 1) & 1, 204);
          if (!ok) break;
          const int s = kv_cnt % KV_STAGES;
          ok = mbar_wait(wc, v_full + 8 * s, (kv_cnt / KV_STAGES) & 1, 205);
          if (!ok) break;
          tc_fence_after();
          // V tile: [128 kv rows][D], 64-column blocks 16 KB apart; 16 kv rows per MMA = 2 KB
          const uint64_t v_desc = make_smem_desc(sV + s * SM::TILE_BYTES, SM::CHUNK_BYTES, 1024);
          const uint32_t a_tmem = tS0 + (kv_cnt & 1) * 128;
#pragma unroll
          for (int ks = 0; ks < TILE / 16; ++ks)
            mma_ts(tO, a_tmem + ks * 8, desc_advance(v_desc, ks * 2048), idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
          tc_commit(v_empty + 8 * s);
        }
        if (!ok) break;
        tc_commit(o_full);
      }
    }
  } else {
    // ------------------------------------------------------------------ SiLU + epilogue warps
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may touch
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    uint32_t it_cnt = 0, kv_cnt = 0;
    bool ok = true;
    for (int idx = blockIdx.x; idx < num_items && ok; idx += gridDim.x, ++it_cnt) {
      const int2 e = p.items[idx / p.H];
      const int h = idx % p.H;
      TileItem it;
      load_item<false>(it, p.g, e.x, e.y);
      const int L = it.m.L;
      const int i = it.m0 + row_in_tile;
      const int id_i = it.m.id(i);
      for (int j = 0; j < it.n_tiles; ++j, ++kv_cnt) {
        const int n0 = it.tile_at(j) * TILE;
        const bool full = tile_pair_is_full(it, n0) && p.bias == nullptr;
        ok = mbar_wait(wc, s_full + 8 * (kv_cnt & 1), (kv_cnt >> 1) & 1, 301);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tS = tS0 + (kv_cnt & 1) * 128 + lane_off;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32(tS + c * 32, r);
          tc_wait_ld();
          uint32_t packed[16];
          if (full) {
#pragma unroll
            for (int x = 0; x < 16; ++x) {
              float h0 = __uint_as_float(r[2 * x]) * p.half_alpha;
              float h1 = __uint_as_float(r[2 * x + 1]) * p.half_alpha;
              float p0 = fmaf(h0, tanh_approx(h0), h0);
              float p1 = fmaf(h1, tanh_approx(h1), h1);
              packed[x] = pack2(p0, p1, IS_BF16);
            }
          } else {
#pragma unroll
            for (int x = 0; x < 32; x += 2) {
              float pv[2];
#pragma unroll
              for (int y = 0; y < 2; ++y) {
                const int jj = n0 + c * 32 + x + y;
                float hh = __uint_as_float(r[x + y]) * p.half_alpha;
                if (p.bias != nullptr) {
                  int dist = i > jj ? i - jj : jj - i;
                  if (dist < p.bias_numel) hh += 0.5f * p.bias[dist];
                }
                float val = fmaf(hh, tanh_approx(hh), hh);
                bool valid = i < L && jj < L && it.m.valid_ids(i, jj, id_i, it.m.id(jj));
                pv[y] = valid ? val : 0.f;
              }
              packed[x / 2] = pack2(pv[0], pv[1], IS_BF16);
            }
          }
          tmem_st16(tS + c * 16, packed);
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full + 8 * (kv_cnt & 1));
      }
      if (!ok) break;
      // epilogue: O (fp32, TMEM) -> scale -> 16-bit -> global, valid rows only
      ok = mbar_wait(wc, o_full, it_cnt & 1, 302);
      if (!ok) break;
      tc_fence_after();
      float scale = p.inv_n;
      if (p.attn_scale != nullptr && i < L)
        scale = p.attn_scale_numel == 1 ? p.attn_scale[0] : p.attn_scale[(int64_t)it.start + i];
      uint16_t *orow = reinterpret_cast<uint16_t *>(p.out) + (int64_t)(it.start + i) * p.o_rs + (int64_t)h * p.o_hs;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tO + lane_off + c * 32, r);
        tc_wait_ld();
        if (i < L) {
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            uint4 o4;
            o4.x = pack2(__uint_as_float(r[8 * x + 0]) * scale, __uint_as_float(r[8 * x + 1]) * scale, IS_BF16);
            o4.y = pack2(__uint_as_float(r[8 * x + 2]) * scale, __uint_as_float(r[8 * x + 3]) * scale, IS_BF16);
            o4.z = pack2(__uint_as_float(r[8 * x + 4]) * scale, __uint_as_float(r[8 * x + 5]) * scale, IS_BF16);
            o4.w = pack2(__uint_as_float(r[8 * x + 6]) * scale, __uint_as_float(r[8 * x + 7]) * scale, IS_BF16);
            *reinterpret_cast<uint4 *>(orow + c * 32 + x * 8) = o4;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_empty);
      // rows at or beyond max_seq_len of an over-long sequence come back as zeros
      if (it.len > L && it.m0 + TILE >= L) {
        for (int r2 = L + row_in_tile; r2 < it.len; r2 += TILE) {
          uint16_t *zr = reinterpret_cast<uint16_t *>(p.out) + (int64_t)(it.start + r2) * p.o_rs + (int64_t)h * p.o_hs;
          for (int x = 0; x < D; x += 8) *reinterpret_cast<uint4 *>(zr + x) = make_uint4(0, 0, 0, 0);
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

// ----------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = (EncodeTiledFn)ptr;
  }
  return fn;
}

}  // namespace

// 2-D map over a jagged [rows, H*d] tensor of 16-bit elements (or 8-bit with elem_bytes = 1):
// box = 128 rows x 128 bytes, 128-byte swizzle, zero fill outside.
int make_tile_map(CUtensorMap *m, const void *base, int64_t rows, int64_t cols, int64_t row_stride_elems,
                  int elem_bytes, bool is_bf16) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return fail(B200_HSTU_EDEVICE, "cuTensorMapEncodeTiled is not available from the driver");
  {
    // the driver call needs this thread to have the device's primary context current; a thread
    // that has only inherited its device index (an autograd worker, say) may not have bound it yet
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaSetDevice(dev);
  }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(row_stride_elems * elem_bytes)};
  cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), (cuuint32_t)TILE};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                           : (is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  CUresult r = fn(m, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B200_HSTU_EINVAL, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

int device_sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

bool device_is_sm100() {
  static int ok = -1;
  if (ok < 0) {
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    ok = (major == 10) ? 1 : 0;
  }
  return ok == 1;
}

bool attn_tc_layout_ok(const b200_hstu_attn_args &a, bool bwd, const char **why) {
  auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (a.dtype != B200_HSTU_BF16 && a.dtype != B200_HSTU_F16) { *why = "dtype is not bf16 / f16"; return false; }
  if (a.dqk != a.dv || (a.dqk != 64 && a.dqk != 128)) { *why = "head dims must be equal and 64 or 128"; return false; }
  if (a.q_head_stride != a.dqk || a.k_head_stride != a.dqk || a.v_head_stride != a.dv) { *why = "heads not contiguous"; return false; }
  if (a.q_row_stride % 8 || a.k_row_stride % 8 || a.v_row_stride % 8) { *why = "row strides not multiples of 16 bytes"; return false; }
  if (!al16(a.q) || !al16(a.k) || !al16(a.v)) { *why = "q / k / v not 16-byte aligned"; return false; }
  if (!bwd) {
    if (!al16(a.out) || a.o_row_stride % 8 || a.o_head_stride % 8) { *why = "out not 16-byte aligned"; return false; }
  } else {
    if (a.do_head_stride != a.dv || a.do_row_stride % 8 || !al16(a.dout)) { *why = "dout layout"; return false; }
    if (!al16(a.dq) || !al16(a.dk) || !al16(a.dv_) || a.dq_row_stride % 8 || a.dk_row_stride % 8 ||
        a.dv_row_stride % 8 || a.dq_head_stride % 8 || a.dk_head_stride % 8 || a.dv_head_stride % 8) {
      *why = "dq / dk / dv layout";
      return false;
    }
  }
  if (!device_is_sm100()) { *why = "device is not compute capability 10.x"; return false; }
  return true;
}

int64_t attn_tc_fwd_workspace_bytes(const b200_hstu_attn_args &a) { return plan_bytes(a.total_L, a.B); }

template <int D, bool IS_BF16>
int launch_fwd_tc(const b200_hstu_attn_args &a, cudaStream_t st) {
  using SM = FwdSmem<D>;
  if (a.workspace == nullptr || a.workspace_bytes < attn_tc_fwd_workspace_bytes(a))
    return fail(B200_HSTU_EWORKSPACE, "attention forward needs %lld bytes of scratch, got %lld",
                (long long)attn_tc_fwd_workspace_bytes(a), (long long)a.workspace_bytes);
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = make_tile_map(&mq, a.q, a.total_L, (int64_t)a.H * D, a.q_row_stride, 2, IS_BF16)) != 0) return rc;
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
  PlanHeader *hdr = reinterpret_cast<PlanHeader *>(a.workspace);
  int2 *items = reinterpret_cast<int2 *>(hdr + 1);
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
  p.half_alpha = 0.5f * a.alpha;
  p.inv_n = 1.f / (float)a.max_seq_len;
  p.H = a.H;
  const int max_items = (int)plan_max_items(a.total_L, a.B);
  attn_plan_kernel<false><<<1, PLAN_THREADS, 0, st>>>(p.g, hdr, items, max_items);
  count_launch();
  B200_CHECK_LAUNCH("attention plan");
  auto kern = hstu_attn_fwd_sm100_kernel<D, IS_BF16>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::DYN_BYTES);
  if (e != cudaSuccess) return check_cuda(e, "forward smem attribute");
  int64_t upper = (int64_t)max_items * a.H;
  int grid = (int)(upper < device_sm_count() ? upper : device_sm_count());
  kern<<<grid, FWD_THREADS, SM::DYN_BYTES, st>>>(mq, mk, mv, p);
  count_launch();
  B200_CHECK_LAUNCH("tcgen05 attention forward");
  return 0;
}

int attn_tc_fwd(const b200_hstu_attn_args &a, cudaStream_t st) {
  const bool bf = a.dtype == B200_HSTU_BF16;
  if (a.dqk == 128) return bf ? launch_fwd_tc<128, true>(a, st) : launch_fwd_tc<128, false>(a, st);
  return bf ? launch_fwd_tc<64, true>(a, st) : launch_fwd_tc<64, false>(a, st);
}

}  // namespace b200hstu
