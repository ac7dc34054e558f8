// Host-side helpers shared by the tensor-core attention kernels: TMA descriptor creation through
// the driver entry point, device queries, and the layout test that decides whether the
// tensor-core kernels can run a request.
#include <cuda.h>

#include "attn_plan.cuh"

namespace b200hstu {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
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

// 2-D map over a jagged [rows, H*d] tensor of 16-bit elements (or 8-bit with elem_bytes = 1):
// box = box_rows rows x 128 bytes, 128-byte swizzle, zero fill outside.
int make_tile_map_rows(CUtensorMap *m, const void *base, int64_t rows, int64_t cols, int64_t row_stride_elems,
                       int elem_bytes, bool is_bf16, int box_rows) {
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
  cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                           : (is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  CUresult r = fn(m, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B200_HSTU_EINVAL, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

int make_tile_map(CUtensorMap *m, const void *base, int64_t rows, int64_t cols, int64_t row_stride_elems,
                  int elem_bytes, bool is_bf16) {
  return make_tile_map_rows(m, base, rows, cols, row_stride_elems, elem_bytes, is_bf16, TILE);
}

// Launch attribute that lets a kernel start before the previous kernel of the stream has finished
// (programmatic dependent launch); the kernel itself waits where it first needs that kernel's output.
void fill_pdl_config(cudaLaunchConfig_t *cfg, cudaLaunchAttribute *attr, int grid, int threads, size_t smem,
                     cudaStream_t st) {
  *cfg = cudaLaunchConfig_t{};
  cfg->gridDim = dim3((unsigned)grid);
  cfg->blockDim = dim3((unsigned)threads);
  cfg->dynamicSmemBytes = smem;
  cfg->stream = st;
  attr->id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr->val.programmaticStreamSerializationAllowed = 1;
  cfg->attrs = attr;
  cfg->numAttrs = 1;
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


}  // namespace b200hstu
