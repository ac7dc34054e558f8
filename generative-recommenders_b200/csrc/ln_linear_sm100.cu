// Fused uvqk stage of the HSTU layer for sm_100a:
//
//     out = LayerNorm(x) W + bias          [M, N]   (16-bit)
//     u   = SiLU(out[:, :silu_cols])       [M, silu_cols]
//
// (generative_recommenders/ops/hstu_compute.py:54-104: layer_norm -> addmm -> split -> silu) as one
// tensor-core kernel instead of a LayerNorm pass, a library GEMM and a SiLU pass.
//
// The normalisation is moved behind the GEMM:
//     LN(x) W = rstd * (x W' - mean * c1) + c2,   W' = diag(gamma) W,  c1[n] = sum_k W'[k, n],
//                                                 c2[n] = sum_k beta[k] W[k, n] + bias[n]
// so the tensor cores multiply the raw rows of x (exact 16-bit products, fp32 accumulation) and the
// per-row statistics are only needed by the epilogue; they are computed from the x tile in shared
// memory while the first products run.  W', c1 and c2 come from two small preparation launches.
//
// One CTA per SM walks 128-row blocks of x:
//   warp 0      producer: TMA loads of the x block (all of K, D / 64 sub-tiles of 128 x 64) and of W'
//               in stages of 64 (K) x 256 (N), 128-byte swizzle
//   warp 1      one elected thread issues tcgen05.mma 128 x 256 x 16 (A = x, K-major; B = W', N
//               contiguous = MN-major) into one of two 256-column TMEM accumulators
//   warps 2-5   row statistics (one row per thread) and the epilogue: TMEM -> registers ->
//               rstd * (acc - mean * c1) + c2 -> 16-bit -> global (whole 32-byte sectors per thread),
//               SiLU for the first silu_cols columns; overlaps the next tile's products
// Every wait is bounded.
#include <cuda.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace b200hstu {

int make_tile_map_rows(CUtensorMap *m, const void *base, int64_t rows, int64_t cols, int64_t row_stride_elems,
                       int elem_bytes, bool is_bf16, int box_rows);
int device_sm_count();
bool device_is_sm100();

namespace {

using namespace ptx;

constexpr int LL_THREADS = 192;
constexpr int LL_BM = 128;            // rows of x per block
constexpr int LL_BN = 256;            // columns per accumulator
constexpr int LL_KC = 64;             // K per shared-memory sub-tile / stage
constexpr int LL_A_SUB = LL_BM * 128; // bytes of one x sub-tile (128 rows x 64 elements)
constexpr int LL_B_BOX = LL_KC * 128; // bytes of one W' box (64 k x 64 n)
constexpr int LL_B_STAGE = 4 * LL_B_BOX;
constexpr int LL_MAX_STAGES = 6;
constexpr int LL_MAX_KC = 8;          // D <= 512
constexpr int LL_MISC = 2048;         // barriers, TMEM slot, abort flag | per-warp c1 / c2 staging
constexpr int LL_SMEM_LIMIT = 232448;

struct LLParams {
  const float *c1, *c2;   // [N]
  void *out;
  int64_t out_rs;         // elements
  void *u;
  int64_t u_rs;
  float *mean, *rstd;
  int *status;
  int64_t M;
  int D, N, silu_cols;
  int kc;                 // D / 64
  int stages;
  int nsplit;             // CTAs sharing one row block, each with its own range of column tiles
  int skip_pre;           // leave out[:, :silu_cols] unwritten
  float eps;
};

template <bool IS_BF16> __device__ __forceinline__ uint32_t pack2(float a, float b) {
  if (IS_BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&v);
}
template <bool IS_BF16> __device__ __forceinline__ float round16(float a) {
  return IS_BF16 ? __bfloat162float(__float2bfloat16_rn(a)) : __half2float(__float2half_rn(a));
}
template <bool IS_BF16> __device__ __forceinline__ float2 unpack2(uint32_t w) {
  if (IS_BF16) return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&w));
  return __half22float2(*reinterpret_cast<__half2 *>(&w));
}

// element i of an 8-entry register array, without indexing it dynamically
__device__ __forceinline__ float pick8(const float (&a)[8], int i) {
  float v = a[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) v = (i == k) ? a[k] : v;
  return v;
}

// One 32-column chunk of the epilogue for one row: rstd * (acc - mean * c1) + c2 -> 16 bits -> out,
// and SiLU of the rounded value -> u for the first silu_cols columns.
template <bool IS_BF16> struct EpiChunk {
  float rstd, neg_mr;
  float *my_c1, *my_c2;   // this warp's staging area: c1[32], c2[32]
  uint16_t *orow, *urow;  // this row at the tile's first column (urow may be NULL)
  int silu_left;          // silu_cols - first column of the tile
  int lane;
  bool row_ok, wide, skip_pre;
  __device__ __forceinline__ void run(const uint32_t (&acc)[32], int cc, float c1_lane, float c2_lane) const {
    __syncwarp();
    my_c1[lane] = c1_lane;
    my_c2[lane] = c2_lane;
    __syncwarp();
    if (!row_ok) return;
    const float4 *c1v = reinterpret_cast<const float4 *>(my_c1);
    const float4 *c2v = reinterpret_cast<const float4 *>(my_c2);
    float val[32];
#pragma unroll
    for (int x = 0; x < 8; ++x) {
      const float4 a = c1v[x], b = c2v[x];
      val[4 * x + 0] = fmaf(rstd, __uint_as_float(acc[4 * x + 0]), fmaf(neg_mr, a.x, b.x));
      val[4 * x + 1] = fmaf(rstd, __uint_as_float(acc[4 * x + 1]), fmaf(neg_mr, a.y, b.y));
      val[4 * x + 2] = fmaf(rstd, __uint_as_float(acc[4 * x + 2]), fmaf(neg_mr, a.z, b.z));
      val[4 * x + 3] = fmaf(rstd, __uint_as_float(acc[4 * x + 3]), fmaf(neg_mr, a.w, b.w));
    }
    uint4 o4[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      o4[x].x = pack2<IS_BF16>(val[8 * x + 0], val[8 * x + 1]);
      o4[x].y = pack2<IS_BF16>(val[8 * x + 2], val[8 * x + 3]);
      o4[x].z = pack2<IS_BF16>(val[8 * x + 4], val[8 * x + 5]);
      o4[x].w = pack2<IS_BF16>(val[8 * x + 6], val[8 * x + 7]);
    }
    const bool is_u = urow != nullptr && cc * 32 < silu_left;
    if (!(skip_pre && is_u)) store64(orow + cc * 32, o4);
    if (is_u) {
      // SiLU of the value as stored (rounded to 16 bits), silu(v) = h + h tanh(h), h = v / 2
      uint4 u4[4];
      uint32_t *uw = reinterpret_cast<uint32_t *>(u4);
      const uint32_t *ow = reinterpret_cast<const uint32_t *>(o4);
#pragma unroll
      for (int x = 0; x < 16; ++x) {
        const float2 v2 = unpack2<IS_BF16>(ow[x]);
        const float h0 = 0.5f * v2.x, h1 = 0.5f * v2.y;
        uw[x] = pack2<IS_BF16>(fmaf(h0, tanh_approx(h0), h0), fmaf(h1, tanh_approx(h1), h1));
      }
      store64(urow + cc * 32, u4);
    }
  }
  // 64 bytes of one row: whole 32-byte sectors when the row is aligned for it
  __device__ __forceinline__ void store64(uint16_t *dst, const uint4 (&v)[4]) const {
    if (wide) {
      st_global_256(dst, v[0], v[1]);
      st_global_256(dst + 16, v[2], v[3]);
    } else {
#pragma unroll
      for (int x = 0; x < 4; ++x) *reinterpret_cast<uint4 *>(dst + x * 8) = v[x];
    }
  }
};

// ---------------------------------------------------------------------------------------
// preparation: W' = gamma (.) W, c1 = column sums of W', c2 = beta W + bias, in two small launches:
//   1. grid (N / 256, D / 32): a CTA takes 32 rows x 256 columns of W (16-byte vectors, 8 columns
//      per lane, 4 rows per warp), writes W' and its partial column sums part[split][{c1, c2}][N]
//   2. one thread per column adds the partial sums in a fixed order (and the bias)
// ---------------------------------------------------------------------------------------
constexpr int PREP_ROWS = 32, PREP_COLS = 256;

template <typename E>
__global__ void __launch_bounds__(256)
ln_linear_prep_kernel(const E *__restrict__ W, const E *__restrict__ gamma, const E *__restrict__ beta,
                      E *__restrict__ Wp, float *__restrict__ part, int D, int N) {
  __shared__ float s1[8][PREP_COLS], s2[8][PREP_COLS];
  const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
  const int col0 = blockIdx.x * PREP_COLS + lane * 8;
  const int k0 = blockIdx.y * PREP_ROWS;
  float a1[8], a2[8];
#pragma unroll
  for (int t = 0; t < 8; ++t) a1[t] = a2[t] = 0.f;
  if (col0 < N) {  // N is a multiple of 64, so a lane's 8 columns are all in or all out
    uint4 raw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + wp + 8 * i;
      raw[i] = k < D ? __ldg(reinterpret_cast<const uint4 *>(W + (int64_t)k * N + col0)) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + wp + 8 * i;
      if (k < D) {
        const float gk = to_f32(gamma[k]), bk = to_f32(beta[k]);
        const E *pe = reinterpret_cast<const E *>(&raw[i]);
        uint4 outv;
        E *po = reinterpret_cast<E *>(&outv);
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const float w = to_f32(pe[t]);
          po[t] = from_f32<E>(w * gk);
          a1[t] += to_f32(po[t]);
          a2[t] = fmaf(bk, w, a2[t]);
        }
        *reinterpret_cast<uint4 *>(Wp + (int64_t)k * N + col0) = outv;
      }
    }
  }
#pragma unroll
  for (int t = 0; t < 8; ++t) {
    s1[wp][lane * 8 + t] = a1[t];
    s2[wp][lane * 8 + t] = a2[t];
  }
  __syncthreads();
  const int c = threadIdx.x, col = blockIdx.x * PREP_COLS + c;
  if (col < N) {
    float t1 = 0.f, t2 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      t1 += s1[i][c];
      t2 += s2[i][c];
    }
    float *dst = part + (int64_t)blockIdx.y * 2 * N;
    dst[col] = t1;
    dst[N + col] = t2;
  }
}

template <typename E>
__global__ void __launch_bounds__(256)
ln_linear_prep_sum_kernel(const float *__restrict__ part, int splits, const E *__restrict__ bias,
                          float *__restrict__ c1, float *__restrict__ c2, int *status, int N) {
  const int col = blockIdx.x * 256 + threadIdx.x;
  if (col < N) {
    float t1 = 0.f, t2 = 0.f;
    for (int s = 0; s < splits; ++s) {
      t1 += part[(int64_t)s * 2 * N + col];
      t2 += part[(int64_t)s * 2 * N + N + col];
    }
    c1[col] = t1;
    c2[col] = t2 + (bias ? to_f32(bias[col]) : 0.f);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) *status = 0;
}

// ---------------------------------------------------------------------------------------
// main kernel
// ---------------------------------------------------------------------------------------
template <bool IS_BF16>
__global__ void __launch_bounds__(LL_THREADS, 1)
ln_linear_sm100_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                       const LLParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sA = base;
  const uint32_t sB = sA + p.kc * LL_A_SUB;
  const uint32_t misc = sB + p.stages * LL_B_STAGE;
  uint8_t *misc_gen = smem_gen + (misc - base);
  // barriers (8 bytes each)
  const uint32_t a_full = misc;                        // [LL_MAX_KC] x sub-tile landed
  const uint32_t a_empty = a_full + 8 * LL_MAX_KC;     // x block no longer needed
  const uint32_t b_full = a_empty + 8;                 // [LL_MAX_STAGES]
  const uint32_t b_empty = b_full + 8 * LL_MAX_STAGES; // [LL_MAX_STAGES]
  const uint32_t acc_full = b_empty + 8 * LL_MAX_STAGES;  // [2]
  const uint32_t acc_empty = acc_full + 16;               // [2]
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(misc_gen + 512);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(misc_gen + 520);
  float *s_c = reinterpret_cast<float *>(misc_gen + 1024);  // per epilogue warp: c1[32], c2[32]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  WaitCtx wc{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < LL_MAX_KC; ++i) mbar_init(a_full + 8 * i, 1);
    mbar_init(a_empty, 5);  // the MMA warp's commit + one arrival per statistics warp
    for (int s = 0; s < LL_MAX_STAGES; ++s) {
      mbar_init(b_full + 8 * s, 1);
      mbar_init(b_empty + 8 * s, 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(acc_full + 8 * x, 1);
      mbar_init(acc_empty + 8 * x, 4);
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

  // work units: (row block, split) - with fewer row blocks than SMs the column tiles of a block
  // are divided among nsplit CTAs (each loads the x block and computes the statistics itself)
  const int n_tiles = (p.N + LL_BN - 1) / LL_BN;
  const int num_units = (int)((p.M + LL_BM - 1) / LL_BM) * p.nsplit;
  auto tile_lo = [&](int unit) { return ((unit % p.nsplit) * n_tiles) / p.nsplit; };
  auto tile_hi = [&](int unit) { return ((unit % p.nsplit + 1) * n_tiles) / p.nsplit; };
  const int KC = p.kc, ST = p.stages;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (elect_one()) {
      prefetch_tmap(&tmap_x);
      prefetch_tmap(&tmap_w);
      uint32_t slot = 0, sphase = 0;  // ring position of the next W' stage and the parity of its round
      int it = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, ++it) {
        const int blk = unit / p.nsplit;
        const int total_b = (tile_hi(unit) - tile_lo(unit)) * KC;
        int issued = 0, bn = tile_lo(unit), bk = 0;
        auto issue_b = [&](int upto) {
          for (; issued < upto && ok; ++issued) {
            ok = mbar_wait(wc, b_empty + 8 * slot, sphase ^ 1, 1101);
            if (!ok) break;
            const int n0 = bn * LL_BN;
            const int boxes = (p.N - n0) >= LL_BN ? 4 : (p.N - n0) / 64;
            const uint32_t full = b_full + 8 * slot, dst = sB + slot * LL_B_STAGE;
            mbar_arrive_expect_tx(full, boxes * LL_B_BOX);
            for (int bx = 0; bx < boxes; ++bx) tma_load_2d(dst + bx * LL_B_BOX, &tmap_w, n0 + bx * 64, bk * LL_KC, full);
            if (++bk == KC) { bk = 0; ++bn; }
            if (++slot == (uint32_t)ST) { slot = 0; sphase ^= 1; }
          }
        };
        // the first stages of W' do not depend on the x buffer: request them before waiting for it
        issue_b(total_b < ST ? total_b : ST);
        if (!ok) break;
        ok = mbar_wait(wc, a_empty, (it & 1) ^ 1, 1102);
        if (!ok) break;
        for (int kc = 0; kc < KC; ++kc) {
          mbar_arrive_expect_tx(a_full + 8 * kc, LL_A_SUB);
          tma_load_2d(sA + kc * LL_A_SUB, &tmap_x, kc * LL_KC, blk * LL_BM, a_full + 8 * kc);
        }
        issue_b(total_b);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue
    if (elect_one()) {
      constexpr uint32_t FMT = IS_BF16 ? 1u : 0u;
      uint32_t slot = 0, sphase = 0, tcount = 0;
      int it = 0;
      bool ok = true;
      const uint64_t a_desc0 = make_smem_desc(sA, 16, 1024);
      const uint64_t b_desc0 = make_smem_desc(sB, LL_B_BOX, 1024);
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, ++it) {
        const int n_lo = tile_lo(unit), n_hi = tile_hi(unit);
        for (int n = n_lo; n < n_hi && ok; ++n, ++tcount) {
          const int n0 = n * LL_BN;
          const int nt = (p.N - n0) >= LL_BN ? LL_BN : (p.N - n0);
          const uint32_t idesc = make_idesc(FMT, FMT, 0, 1, LL_BM, (uint32_t)nt);
          const uint32_t buf = tcount & 1;
          ok = mbar_wait(wc, acc_empty + 8 * buf, ((tcount >> 1) & 1) ^ 1, 1201);
          if (!ok) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * LL_BN;
          for (int kc = 0; kc < KC; ++kc) {
            if (n == n_lo) {
              ok = mbar_wait(wc, a_full + 8 * kc, it & 1, 1202);
              if (!ok) break;
            }
            ok = mbar_wait(wc, b_full + 8 * slot, sphase, 1203);
            if (!ok) break;
            tc_fence_after();
            const uint64_t a_desc = desc_advance(a_desc0, kc * LL_A_SUB);
            const uint64_t b_desc = desc_advance(b_desc0, slot * LL_B_STAGE);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              mma_ss(d_tmem, desc_advance(a_desc, ks * 32), desc_advance(b_desc, ks * 2048), idesc,
                     (kc | ks) != 0);
            tc_commit(b_empty + 8 * slot);
            if (++slot == (uint32_t)ST) { slot = 0; sphase ^= 1; }
          }
          if (!ok) break;
          tc_commit(acc_full + 8 * buf);
        }
        // nobody waits for the x buffer after this CTA's last block
        if (ok && unit + (int)gridDim.x < num_units) tc_commit(a_empty);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ statistics + epilogue
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int row_in_blk = q * 32 + lane;
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    float *my_c1 = s_c + q * 64, *my_c2 = my_c1 + 32;
    float nxt1[LL_BN / 32], nxt2[LL_BN / 32];  // c1 / c2 of the next column tile, one column per lane
#pragma unroll
    for (int cc = 0; cc < LL_BN / 32; ++cc) {
      const int col = cc * 32 + lane;
      nxt1[cc] = col < p.N ? __ldg(p.c1 + col) : 0.f;
      nxt2[cc] = col < p.N ? __ldg(p.c2 + col) : 0.f;
    }
    uint32_t tcount = 0;
    int it = 0;
    bool ok = true;
    const bool wide = (reinterpret_cast<uintptr_t>(p.out) & 31) == 0 && (p.out_rs & 15) == 0 &&
                      (p.u == nullptr || ((reinterpret_cast<uintptr_t>(p.u) & 31) == 0 && (p.u_rs & 15) == 0));
    int nxt_tile = 0;  // the column tile whose c1 / c2 are in nxt1 / nxt2
    for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, ++it) {
      const int blk = unit / p.nsplit;
      const int n_lo = tile_lo(unit), n_hi = tile_hi(unit);
      const bool first_split = unit % p.nsplit == 0;
      const int64_t row = (int64_t)blk * LL_BM + row_in_blk;
      const bool row_ok = row < p.M;
      // ---- row statistics from the x block in shared memory (shifted sums; the order of the
      // elements inside the swizzled 128-byte line does not matter)
      float shift = 0.f, s1 = 0.f, s2 = 0.f;
      for (int kc = 0; kc < KC; ++kc) {
        ok = mbar_wait(wc, a_full + 8 * kc, it & 1, 1301);
        if (!ok) break;
        const uint4 *line = reinterpret_cast<const uint4 *>(smem_gen + (sA - base) + kc * LL_A_SUB + row_in_blk * 128);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint4 v = line[(j + lane) & 7];  // rows are 128 bytes apart: rotate to spread the banks
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
          if (kc == 0 && j == 0) shift = unpack2<IS_BF16>(w[0]).x;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = unpack2<IS_BF16>(w[e]);
            const float d0 = f.x - shift, d1 = f.y - shift;
            s1 += d0 + d1;
            s2 = fmaf(d0, d0, s2);
            s2 = fmaf(d1, d1, s2);
          }
        }
      }
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(a_empty);
      const float inv_d = 1.f / (float)p.D;
      const float m_sh = s1 * inv_d;
      const float mean = shift + m_sh;
      const float var = fmaxf(s2 * inv_d - m_sh * m_sh, 0.f);
      const float rstd = rsqrtf(var + p.eps);
      if (row_ok) {
        if (p.mean && first_split) p.mean[row] = mean;
        if (p.rstd && first_split) p.rstd[row] = rstd;
      }
      const float neg_mr = -mean * rstd;
      // ---- epilogue of every column tile of this block
      for (int n = n_lo; n < n_hi && ok; ++n, ++tcount) {
        const int n0 = n * LL_BN;
        const int nt = (p.N - n0) >= LL_BN ? LL_BN : (p.N - n0);
        const uint32_t buf = tcount & 1;
        if (nxt_tile != n) {  // first tile of a unit that does not continue the previous one
#pragma unroll
          for (int cc = 0; cc < LL_BN / 32; ++cc) {
            const int col = n0 + cc * 32 + lane;
            nxt1[cc] = col < p.N ? __ldg(p.c1 + col) : 0.f;
            nxt2[cc] = col < p.N ? __ldg(p.c2 + col) : 0.f;
          }
        }
        ok = mbar_wait(wc, acc_full + 8 * buf, (tcount >> 1) & 1, 1302);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tacc = tmem_base + buf * LL_BN + lane_off;
        uint16_t *orow = reinterpret_cast<uint16_t *>(p.out) + row * p.out_rs + n0;
        uint16_t *urow = p.u ? reinterpret_cast<uint16_t *>(p.u) + row * p.u_rs + n0 : nullptr;
        const int chunks = nt / 32;
        // c1 / c2: one column per lane and chunk, fetched a whole tile ahead (an L2 round trip is
        // longer than a chunk's work), broadcast to the warp through its own 256 bytes of shared memory
        float cur1[LL_BN / 32], cur2[LL_BN / 32];
#pragma unroll
        for (int cc = 0; cc < LL_BN / 32; ++cc) {
          cur1[cc] = nxt1[cc];
          cur2[cc] = nxt2[cc];
        }
        {
          nxt_tile = n + 1 < n_hi ? n + 1 : tile_lo(unit + (int)gridDim.x);
          const int nn0 = nxt_tile * LL_BN;
#pragma unroll
          for (int cc = 0; cc < LL_BN / 32; ++cc) {
            const int col = nn0 + cc * 32 + lane;
            nxt1[cc] = col < p.N ? __ldg(p.c1 + col) : 0.f;
            nxt2[cc] = col < p.N ? __ldg(p.c2 + col) : 0.f;
          }
        }
        // The loop stays rolled (two chunks per trip for the register double buffer): the epilogue
        // shares its instruction cache with the MMA and producer threads, whose loops must stay hot.
        EpiChunk<IS_BF16> ec{rstd, neg_mr, my_c1, my_c2, orow, urow, p.silu_cols - n0, lane, row_ok, wide,
                             p.skip_pre != 0};
        uint32_t r0[32], r1[32];
        tmem_ld32(tacc, r0);
        for (int cc = 0; cc < chunks; cc += 2) {
          tc_wait_ld();
          if (cc + 1 < chunks) tmem_ld32(tacc + (cc + 1) * 32, r1);
          ec.run(r0, cc, pick8(cur1, cc), pick8(cur2, cc));
          if (cc + 1 < chunks) {
            tc_wait_ld();
            if (cc + 2 < chunks) tmem_ld32(tacc + (cc + 2) * 32, r0);
            ec.run(r1, cc + 1, pick8(cur1, cc + 1), pick8(cur2, cc + 1));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty + 8 * buf);
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

int stages_for(int D) {
  const int a_bytes = (D / LL_KC) * LL_A_SUB;
  int st = (LL_SMEM_LIMIT - 1024 /*alignment slack*/ - LL_MISC - a_bytes) / LL_B_STAGE;
  return st > LL_MAX_STAGES ? LL_MAX_STAGES : st;
}

inline int64_t align256(int64_t x) { return (x + 255) & ~(int64_t)255; }

}  // namespace

bool ln_linear_supported(int D, int N, int silu_cols, int dtype, const char **why) {
  if (dtype != B200_HSTU_BF16 && dtype != B200_HSTU_F16) { *why = "dtype is not bf16 / f16"; return false; }
  if (D < 64 || D > 64 * LL_MAX_KC || D % 64) { *why = "D must be a multiple of 64 up to 512"; return false; }
  if (N < 64 || N % 64) { *why = "N must be a multiple of 64"; return false; }
  if (silu_cols < 0 || silu_cols > N || silu_cols % 32) { *why = "silu_cols must be a multiple of 32"; return false; }
  return true;
}

// workspace: [status (256 B) | W' | c1 | c2 | partial column sums of the preparation]
int64_t ln_linear_workspace_bytes(int D, int N) {
  const int splits = (D + PREP_ROWS - 1) / PREP_ROWS;
  return 256 + align256((int64_t)D * N * 2) + 2 * align256((int64_t)N * 4) + align256((int64_t)splits * 2 * N * 4);
}

template <typename E, bool IS_BF16>
static int ln_linear_t(const b200_hstu_ln_linear_args &a, cudaStream_t st) {
  uint8_t *ws = reinterpret_cast<uint8_t *>(a.workspace);
  int *status = reinterpret_cast<int *>(ws);
  E *Wp = reinterpret_cast<E *>(ws + 256);
  float *c1 = reinterpret_cast<float *>(ws + 256 + align256((int64_t)a.D * a.N * 2));
  float *c2 = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(c1) + align256((int64_t)a.N * 4));
  if (!a.weights_prepared) {
    ProfileScope prof(PROF_LN_LINEAR_PREP, st);
    float *part = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(c2) + align256((int64_t)a.N * 4));
    const int splits = (a.D + PREP_ROWS - 1) / PREP_ROWS;
    dim3 grid((a.N + PREP_COLS - 1) / PREP_COLS, splits);
    ln_linear_prep_kernel<E><<<grid, 256, 0, st>>>((const E *)a.weight, (const E *)a.norm_weight,
                                                   (const E *)a.norm_bias, Wp, part, a.D, a.N);
    count_launch();
    B200_CHECK_LAUNCH("ln_linear_prep_kernel");
    ln_linear_prep_sum_kernel<E><<<(a.N + 255) / 256, 256, 0, st>>>(part, splits, (const E *)a.bias, c1, c2, status,
                                                                    a.N);
    count_launch();
    B200_CHECK_LAUNCH("ln_linear_prep_sum_kernel");
  }
  CUtensorMap mx, mw;
  int rc;
  if ((rc = make_tile_map_rows(&mx, a.x, a.M, a.D, a.x_row_stride, 2, IS_BF16, LL_BM)) != 0) return rc;
  if ((rc = make_tile_map_rows(&mw, Wp, a.D, a.N, a.N, 2, IS_BF16, LL_KC)) != 0) return rc;
  LLParams p;
  p.c1 = c1;
  p.c2 = c2;
  p.out = a.out;
  p.out_rs = a.out_row_stride;
  p.u = a.u;
  p.u_rs = a.u_row_stride;
  p.mean = a.mean;
  p.rstd = a.rstd;
  p.status = status;
  p.M = a.M;
  p.D = a.D;
  p.N = a.N;
  p.silu_cols = a.u ? a.silu_cols : 0;
  p.kc = a.D / LL_KC;
  p.stages = stages_for(a.D);
  p.eps = a.eps;
  const int smem = 1024 + p.kc * LL_A_SUB + p.stages * LL_B_STAGE + LL_MISC;
  auto kern = ln_linear_sm100_kernel<IS_BF16>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return check_cuda(e, "ln_linear smem attribute");
  const int64_t blocks = (a.M + LL_BM - 1) / LL_BM;
  const int n_tiles = (a.N + LL_BN - 1) / LL_BN;
  int nsplit = 1;
  if (blocks < device_sm_count()) {
    nsplit = (int)(device_sm_count() / blocks);
    nsplit = nsplit > n_tiles ? n_tiles : nsplit;
  }
  p.nsplit = nsplit;
  p.skip_pre = (a.skip_pre_activation && a.u) ? 1 : 0;
  const int64_t units = blocks * nsplit;
  const int grid = (int)(units < device_sm_count() ? units : device_sm_count());
  {
    ProfileScope prof(PROF_LN_LINEAR, st);
    kern<<<grid, LL_THREADS, smem, st>>>(mx, mw, p);
    count_launch();
    B200_CHECK_LAUNCH("ln_linear_sm100_kernel");
  }
  return 0;
}

int ln_linear_fwd(const b200_hstu_ln_linear_args &a, cudaStream_t st) {
  const char *why = "";
  if (a.M < 0) return fail(B200_HSTU_EINVAL, "ln_linear: negative row count");
  if (!ln_linear_supported(a.D, a.N, a.u ? a.silu_cols : 0, a.dtype, &why))
    return fail(B200_HSTU_EUNSUPPORTED, "ln_linear: %s", why);
  if (a.M == 0) return 0;
  if (!a.x || !a.norm_weight || !a.norm_bias || !a.weight || !a.out)
    return fail(B200_HSTU_EINVAL, "ln_linear: NULL tensor");
  auto al16 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (!al16(a.x) || !al16(a.out) || (a.u && !al16(a.u)) || !al16(a.workspace) || !al16(a.weight) || a.x_row_stride % 8 ||
      a.out_row_stride % 8 || (a.u && a.u_row_stride % 8))
    return fail(B200_HSTU_EUNSUPPORTED, "ln_linear: tensors must be 16-byte aligned with 16-byte row strides");
  if (a.workspace == nullptr || a.workspace_bytes < ln_linear_workspace_bytes(a.D, a.N))
    return fail(B200_HSTU_EWORKSPACE, "ln_linear needs %lld bytes of scratch, got %lld",
                (long long)ln_linear_workspace_bytes(a.D, a.N), (long long)a.workspace_bytes);
  if (!device_is_sm100()) return fail(B200_HSTU_EDEVICE, "ln_linear: device is not compute capability 10.x");
  if (a.dtype == B200_HSTU_BF16) return ln_linear_t<__nv_bfloat16, true>(a, st);
  return ln_linear_t<__half, false>(a, st);
}

}  // namespace b200hstu
