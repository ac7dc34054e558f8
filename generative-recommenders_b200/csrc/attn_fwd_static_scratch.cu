// An attention-forward entry point for callers that cannot allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: an inference server that hands
// every byte of HBM to its own arena at start-up and forbids later allocations, a plugin called
// from inside a region that must not touch the allocator (for example while another component is
// capturing work, or in a latency-critical loop where an allocator lock is unacceptable), or a
// thin C caller that simply has no allocator to borrow scratch from.  b200_hstu_attn_fwd() needs a
// scratch buffer for its work list and normally expects the caller to provide it.  This variant
// brings its own: a fixed-size array in the library's device image.
//
// Properties a user must know:
//   * The array is 1 MiB and lives in every CUDA context that loads the library, from load until
//     the process exits.
//   * It is big enough for total_L / 128 + B + 1 <= 32 767 work items (for example 4 M tokens in
//     up to ~1000 sequences).  With a relative bias (bias_by_distance) the signed-distance table
//     comes out of the same array, 8 * (roundup128(max_seq_len) + 256) bytes rounded up to 256, and
//     the item limit shrinks by that many bytes / 32.  Larger batches are rejected with
//     B200_HSTU_EWORKSPACE and must go through b200_hstu_attn_fwd() with caller scratch.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress) and remembers it for the life of the process; make that first call
//     outside any stream capture.  Every call queues one 16-byte memset (the list header) and the
//     two kernels.  Resetting the device (cudaDeviceReset) invalidates the remembered address:
//     a process that resets a device must not use this entry point on it afterwards.
//   * There is one array per device, shared by all calls and all streams.  Calls are safe back to
//     back on one stream; two calls that can overlap on the GPU (different streams without an
//     ordering between them) race on the work list.  The array keeps the previous call's list and
//     bias table; the header (item count, status word, claim counter) is cleared by every call and
//     rewritten by its planning kernel, the table is rebuilt, nothing else is carried over.
//   * No cudaMalloc / cudaFree / allocating library call is made, on the first call or later.
#include <mutex>

#include "attn_plan.cuh"

namespace {

constexpr long long kStaticScratchBytes = 1 << 20;
constexpr int kMaxDevices = 64;

// Scratch for the work list of one forward launch.  In host code this name is only a handle for
// cudaGetSymbolAddress; the kernels receive the address that call returns.
static __device__ __align__(256) unsigned char g_attn_fwd_scratch[kStaticScratchBytes];

std::mutex g_lookup_mutex;
void *g_scratch_ptr[kMaxDevices] = {};

// Device address of the array on the current device (looked up once per device).
int scratch_address(void **out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return b200hstu::check_cuda(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return b200hstu::fail(B200_HSTU_EDEVICE, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_lookup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void *ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_attn_fwd_scratch);
    if (e != cudaSuccess) return b200hstu::check_cuda(e, "cudaGetSymbolAddress(static attention scratch)");
    if (ptr == nullptr) return b200hstu::fail(B200_HSTU_EDEVICE, "static attention scratch has no device address");
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace

extern "C" {

int64_t b200_hstu_attn_fwd_static_scratch_max_bytes(void) { return kStaticScratchBytes; }

int b200_hstu_attn_fwd_static_scratch(const b200_hstu_attn_args *args, b200_hstu_stream_t stream) {
  if (args == nullptr) return b200hstu::fail(B200_HSTU_EINVAL, "args is NULL");
  b200_hstu_attn_args a = *args;
  a.workspace = nullptr;
  a.workspace_bytes = 0;
  a.plan_mode = B200_HSTU_PLAN_OWN;   // the built-in buffer holds the forward's list only
  // size check first, on the host, before anything touches the device
  const int64_t need = b200_hstu_attn_workspace_bytes(&a, 0);
  if (need > kStaticScratchBytes)
    return b200hstu::fail(B200_HSTU_EWORKSPACE,
                          "this batch needs %lld bytes of scratch but the built-in buffer holds %lld "
                          "(32 bytes per work item, total_L / 128 + B + 1 of them, plus the bias table if any); "
                          "use b200_hstu_attn_fwd with caller scratch",
                          (long long)need, (long long)kStaticScratchBytes);
  if (need > 0) {
    void *ptr = nullptr;
    int st = scratch_address(&ptr);
    if (st != 0) return st;
    // The list header (item count, status word, claim counter) must not carry over from the
    // previous call.  Layout of the scratch: [bias table (if any) | header | items].
    unsigned char *hdr = static_cast<unsigned char *>(ptr) + b200hstu::bias_table_bytes(a.bias_by_distance, a.max_seq_len);
    cudaError_t e = cudaMemsetAsync(hdr, 0, sizeof(b200hstu::PlanHeader), (cudaStream_t)stream);
    if (e != cudaSuccess) return b200hstu::check_cuda(e, "clearing the static scratch header");
    a.workspace = ptr;
    a.workspace_bytes = kStaticScratchBytes;
  }
  return b200_hstu_attn_fwd(&a, stream);
}

}  // extern "C"
