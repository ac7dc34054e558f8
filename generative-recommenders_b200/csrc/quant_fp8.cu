// Block quantiser for the FP8 forward: x [total_L, H, d] (bf16 / f16 / f32) -> e4m3 with one fp32
// scale = absmax / 448 per (128-token block counted from the start of each sequence, head).
// One CTA per (block, head): a first pass finds the absolute maximum, a second pass scales and
// converts.  The block is at most 128 x d elements and is read twice back to back, so the second
// read comes from L1/L2; HBM traffic is one read of x plus one write of x8.
#include <cuda_fp8.h>

#include "common.cuh"

namespace b200hstu {
namespace {

constexpr int QBLOCK = 128;

template <typename E>
__global__ void __launch_bounds__(256) quantize_e4m3_block_kernel(const E *__restrict__ x, int64_t rs, int64_t hs,
                                                                  uint8_t *__restrict__ x8, float *__restrict__ scale,
                                                                  const int32_t *__restrict__ seq_offsets,
                                                                  const int32_t *__restrict__ block_offsets, int B,
                                                                  int H, int d, int max_seq_len) {
  __shared__ float red[8];
  __shared__ float s_scale;
  const int h = blockIdx.y;
  const int total_blocks = block_offsets[B];
  for (int blk = blockIdx.x; blk < total_blocks; blk += gridDim.x) {
    // sequence that owns this block: last b with block_offsets[b] <= blk
    int lo = 0, hi = B - 1;
    while (lo < hi) {
      int mid = (lo + hi + 1) >> 1;
      if (block_offsets[mid] <= blk) lo = mid; else hi = mid - 1;
    }
    const int b = lo;
    const int start = seq_offsets[b], len = seq_offsets[b + 1] - start;
    const int r0 = (blk - block_offsets[b]) * QBLOCK;
    const int nrows = min(QBLOCK, len - r0);
    const int n = nrows * d;
    float amax = 0.f;
    for (int idx = threadIdx.x; idx < n; idx += blockDim.x) {
      int r = idx / d, c = idx - r * d;
      amax = fmaxf(amax, fabsf(to_f32(x[(int64_t)(start + r0 + r) * rs + (int64_t)h * hs + c])));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
      float m = red[0];
      for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
      float sc = fmaxf(m, 1e-12f) / 448.f;
      s_scale = sc;
      scale[(int64_t)blk * H + h] = sc;
    }
    __syncthreads();
    const float sc = s_scale;  // true division below: bit-identical to x / scale on the host
    for (int idx = threadIdx.x; idx < n; idx += blockDim.x) {
      int r = idx / d, c = idx - r * d;
      float v = to_f32(x[(int64_t)(start + r0 + r) * rs + (int64_t)h * hs + c]) / sc;
      x8[((int64_t)(start + r0 + r) * H + h) * d + c] = (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
    }
    __syncthreads();
  }
}

}  // namespace

int quantize_e4m3_block(const void *x, int dtype, int64_t row_stride, int64_t head_stride, void *x8, float *scale,
                        const int32_t *seq_offsets, const int32_t *block_offsets, int B, int H, int d, int64_t total_L,
                        int max_seq_len, cudaStream_t st) {
  int64_t max_blocks = total_L / QBLOCK + B;
  int gx = (int)(max_blocks < 65535 ? max_blocks : 65535);
  if (gx < 1) gx = 1;
  dim3 grid((unsigned)gx, (unsigned)H);
  ProfileScope prof(PROF_QUANT, st);
  switch (dtype) {
    case B200_HSTU_F32:
      quantize_e4m3_block_kernel<float><<<grid, 256, 0, st>>>((const float *)x, row_stride, head_stride, (uint8_t *)x8,
                                                              scale, seq_offsets, block_offsets, B, H, d, max_seq_len);
      break;
    case B200_HSTU_BF16:
      quantize_e4m3_block_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16 *)x, row_stride, head_stride,
                                                                      (uint8_t *)x8, scale, seq_offsets, block_offsets,
                                                                      B, H, d, max_seq_len);
      break;
    case B200_HSTU_F16:
      quantize_e4m3_block_kernel<__half><<<grid, 256, 0, st>>>((const __half *)x, row_stride, head_stride,
                                                               (uint8_t *)x8, scale, seq_offsets, block_offsets, B, H,
                                                               d, max_seq_len);
      break;
    default:
      return fail(B200_HSTU_EINVAL, "unknown dtype %d", dtype);
  }
  count_launch();
  B200_CHECK_LAUNCH("e4m3 block quantiser");
  return 0;
}

}  // namespace b200hstu
