// Host-readable status of the attention launches, and a self-test of the bounded wait.
//
// Every mbarrier wait of the tensor-core kernels gives up after WAIT_LIMIT_NS without progress,
// records the site where it gave up in the status word of its work list and lets the CTA leave
// through the common exit (TMEM freed, context intact).  b200_hstu_attn_status_async() copies those
// status words back to the host; a caller that wants to know whether a launch ran to completion
// reads them after synchronising the stream (the Python ops do so when B200_HSTU_CHECK_STATUS=1).
//
// The self-test runs the same wait loop in a one-warp kernel on a barrier that nobody ever arrives
// at, with the limit shortened to one millisecond: the wait expires, the site is recorded, the
// kernel returns.  Nothing faults, traps or hangs; it shows that an expired wait ends the kernel
// and that the record reaches the host.
#include "attn_plan.cuh"
#include "sm100_ptx.cuh"

namespace b200hstu {

int64_t attn_tc_workspace_bytes(const b200_hstu_attn_args &a, int which);
bool attn_tc_applicable(const b200_hstu_attn_args &a, bool bwd, const char **why);

namespace {

constexpr uint64_t SELFTEST_LIMIT_NS = 1000000ull;   // 1 ms
constexpr int SELFTEST_SITE = 777;

__global__ void __launch_bounds__(32, 1) bounded_wait_selftest_kernel(int *status, unsigned long long *elapsed_ns) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  const uint32_t bar_addr = ptx::smem_u32(&bar);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    ptx::mbar_init(bar_addr, 1);
    ptx::fence_mbar_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const uint64_t t0 = ptx::globaltimer_ns();
    // phase 0 of a barrier that expects one arrival which never comes
    const bool ok = ptx::mbar_wait_loop<SELFTEST_LIMIT_NS>(&abort_flag, status, bar_addr, 0, SELFTEST_SITE);
    if (ok) atomicCAS(status, 0, -1);   // cannot happen: nobody arrives
    *elapsed_ns = ptx::globaltimer_ns() - t0;
  }
}

}  // namespace
}  // namespace b200hstu

using namespace b200hstu;

extern "C" {

int b200_hstu_attn_status_async(const b200_hstu_attn_args *a, int which, int32_t *host_status, b200_hstu_stream_t stream) {
  if (a == nullptr || host_status == nullptr) return fail(B200_HSTU_EINVAL, "args / host_status is NULL");
  if (which < 0 || which > 2) return fail(B200_HSTU_EINVAL, "which must be 0 (forward), 1 (backward) or 2 (forward that planned the backward)");
  host_status[0] = host_status[1] = host_status[2] = 0;
  const char *why = "";
  if (a->workspace == nullptr || a->impl == B200_HSTU_IMPL_SIMT || !attn_tc_applicable(*a, which == 1, &why))
    return 0;   // the CUDA-core kernels have no waits and no status
  if (a->workspace_bytes < attn_tc_workspace_bytes(*a, which))
    return fail(B200_HSTU_EWORKSPACE, "workspace is smaller than this call's scratch");
  const uint8_t *lists = reinterpret_cast<const uint8_t *>(a->workspace) + bias_table_bytes(a->bias_by_distance, a->max_seq_len);
  const int64_t one = plan_bytes(a->total_L, a->B);
  // forward: [fwd]; backward: [kv, q]; forward that planned the backward: [fwd, kv, q]
  const int n = which == 0 ? 1 : (which == 1 ? 2 : 3);
  const int first = which == 1 ? 1 : 0;
  for (int i = 0; i < n; ++i) {
    const PlanHeader *hdr = reinterpret_cast<const PlanHeader *>(lists + i * one);
    cudaError_t e = cudaMemcpyAsync(host_status + first + i, &hdr->status, sizeof(int32_t), cudaMemcpyDeviceToHost,
                                    (cudaStream_t)stream);
    if (e != cudaSuccess) return check_cuda(e, "reading an attention status word");
  }
  return 0;
}

int b200_hstu_selftest_bounded_wait(int32_t *status_dev, uint64_t *elapsed_ns_dev, b200_hstu_stream_t stream) {
  if (status_dev == nullptr || elapsed_ns_dev == nullptr) return fail(B200_HSTU_EINVAL, "NULL pointer");
  cudaError_t e = cudaMemsetAsync(status_dev, 0, sizeof(int32_t), (cudaStream_t)stream);
  if (e != cudaSuccess) return check_cuda(e, "clearing the self-test status");
  bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status_dev,
                                                                   reinterpret_cast<unsigned long long *>(elapsed_ns_dev));
  count_launch();
  B200_CHECK_LAUNCH("bounded-wait self-test");
  return 0;
}

}  // extern "C"
