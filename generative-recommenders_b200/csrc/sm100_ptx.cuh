// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the attention kernels use:
// mbarriers with bounded waits, TMA tiled loads, TMEM allocation, tcgen05 MMA / commit / ld / st,
// and the shared-memory matrix descriptors + instruction descriptors tcgen05.mma consumes.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200hstu {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred;
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Every wait in these kernels is bounded: after `WAIT_LIMIT_NS` without progress the waiter
// records where it gave up and raises the CTA-wide abort flag; all roles then fall through to
// the common exit (which frees TMEM) instead of spinning forever.
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;  // 2 s

struct WaitCtx {
  volatile int *abort_flag;  // shared memory, one per CTA
  int *status;               // global: first failing site is recorded here (0 = ok)
};

// The spinning part.  LIMIT_NS is a template argument so that the self-test kernel
// (selftest.cu) can run the very same loop with a millisecond limit.
template <uint64_t LIMIT_NS>
__device__ __forceinline__ bool mbar_wait_loop(volatile int *abort_flag, int *status, uint32_t bar, uint32_t parity,
                                               int site) {
  const WaitCtx ctx{abort_flag, status};
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 255u) == 0) {
      if (*ctx.abort_flag) return false;
      uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > LIMIT_NS) {
        *ctx.abort_flag = 1;
        if (ctx.status) atomicCAS(ctx.status, 0, site);
        return false;
      }
    }
  }
}

// In the kernels it is one out-of-line function: inlined at every wait it added ~10 KB to
// kernels that are about as large as the instruction cache (110-135 KB).
static __device__ __noinline__ bool mbar_wait_slow(volatile int *abort_flag, int *status, uint32_t bar, uint32_t parity,
                                            int site) {
  return mbar_wait_loop<WAIT_LIMIT_NS>(abort_flag, status, bar, parity, site);
}

__device__ __forceinline__ bool mbar_wait(const WaitCtx &ctx, uint32_t bar, uint32_t parity, int site) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(ctx.abort_flag, ctx.status, bar, parity, site);
}

// ------------------------------------------------------------------ work ring (see attn_plan.cuh)
// slot layout: int4 {b, t, start, len}, int4 {nt, idx, 0, 0}
__device__ __forceinline__ void sched_publish(const WaitCtx &wc, uint8_t *ring, uint32_t full0, uint32_t empty0,
                                              uint32_t n, int b, int t, int start, int len, int nt, int idx, bool &ok) {
  // item ordinals start at 1 here (item 0 of a CTA is blockIdx.x and never goes through the ring)
  const uint32_t m = n - 1, slot = m & 3u;
  ok = mbar_wait(wc, empty0 + 8 * slot, ((m >> 2) & 1) ^ 1, 901);
  if (!ok) return;
  int4 *dst = reinterpret_cast<int4 *>(ring + slot * 32);
  dst[0] = make_int4(b, t, start, len);
  dst[1] = make_int4(nt, idx, 0, 0);
  asm volatile("fence.acq_rel.cta;" ::: "memory");
  mbar_arrive(full0 + 8 * slot);
}
__device__ __forceinline__ bool sched_fetch(const WaitCtx &wc, const uint8_t *ring, uint32_t full0, uint32_t empty0,
                                            uint32_t n, int &b, int &t, int &start, int &len, int &nt, int &idx,
                                            bool arrive) {
  const uint32_t m = n - 1, slot = m & 3u;
  if (!mbar_wait(wc, full0 + 8 * slot, (m >> 2) & 1, 902)) return false;
  const volatile int4 *src = reinterpret_cast<const volatile int4 *>(ring + slot * 32);
  int4 a, c;
  a.x = src[0].x; a.y = src[0].y; a.z = src[0].z; a.w = src[0].w;
  c.x = src[1].x; c.y = src[1].y;
  b = a.x; t = a.y; start = a.z; len = a.w; nt = c.x; idx = c.y;
  __syncwarp();
  if (arrive) mbar_arrive(empty0 + 8 * slot);
  return true;
}

// ------------------------------------------------------------------ TMA
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap *m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load global -> shared of this CTA, completion on an mbarrier
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *m, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// 32-byte global store (one full sector per lane); the address must be 32-byte aligned
__device__ __forceinline__ void st_global_256(void *p, uint4 a, uint4 b) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z),
               "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
               : "memory");
}

// ------------------------------------------------------------------ programmatic dependent launch
// A kernel launched with the programmatic-serialization attribute may start while the kernel
// before it in the stream is still running; grid_dependency_wait() blocks until that kernel has
// completed and its writes are visible.  allow_dependents() lets the next such kernel start.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void allow_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ------------------------------------------------------------------ TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// mbarrier arrives once all tcgen05 operations issued so far by this thread have completed
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// fp8 (e4m3/e5m2) operands
__device__ __forceinline__ void mma_ss_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (quadrant*32 + t)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// ------------------------------------------------------------------ descriptors
// Shared-memory matrix descriptor (64-bit): start address, leading / stride byte offsets in
// 16-byte units, descriptor version 1 (Blackwell) at bit 46, swizzle mode in bits 61-63
// (2 = 128-byte swizzle).  Tiles are 128-byte-swizzled and 1024-byte aligned.
//   K-major operand  (rows of 64 16-bit elements along K): SBO = 1024 B between 8-row groups, LBO unused (1).
//   MN-major operand (rows of 64 elements along M/N, one row per k): LBO = bytes between 64-element
//   column blocks, SBO = 1024 B between groups of 8 k.
__host__ __device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__host__ __device__ __forceinline__ uint64_t desc_advance(uint64_t d, uint32_t bytes) { return d + (uint64_t)(bytes >> 4); }

// Instruction descriptor for kind::f16 / kind::f8f6f4, fp32 accumulation, dense.
//   ab_fmt: kind::f16 -> 0 = f16, 1 = bf16;  kind::f8f6f4 -> 0 = e4m3, 1 = e5m2
__host__ __device__ __forceinline__ uint32_t make_idesc(uint32_t a_fmt, uint32_t b_fmt, uint32_t a_mn_major,
                                                        uint32_t b_mn_major, uint32_t M, uint32_t N) {
  uint32_t d = 0;
  d |= 1u << 4;  // D format: f32
  d |= a_fmt << 7;
  d |= b_fmt << 10;
  d |= a_mn_major << 15;
  d |= b_mn_major << 16;
  d |= (N >> 3) << 17;
  d |= (M >> 4) << 24;
  return d;
}

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ------------------------------------------------------------------ timeline (profiling aid)
// Optional record of {SM clock, tag} pairs written by one thread per role of CTA 0; off (NULL)
// unless the caller of a launch asks for it and provides the room.
constexpr int TRACE_RECORDS = 1024;
constexpr int64_t TRACE_BYTES = 4 * TRACE_RECORDS * (int64_t)sizeof(ulonglong2);

// Compiled in only with -DB200_HSTU_TRACE_BUILD (build.py: B200_HSTU_TRACE_BUILD=1): the marks sit
// in the hot loops, and these kernels are as large as the instruction cache - every instruction
// that is not needed costs time.
#ifdef B200_HSTU_TRACE_BUILD
struct Tracer {
  ulonglong2 *buf;
  int n;
  __device__ __forceinline__ void init(ulonglong2 *base, int role, bool on) {
    buf = (base != nullptr && on && blockIdx.x == 0) ? base + role * TRACE_RECORDS : nullptr;
    n = 0;
  }
  __device__ __forceinline__ void mark(unsigned tag) {
    if (buf != nullptr && n < TRACE_RECORDS) buf[n++] = make_ulonglong2((unsigned long long)clock64(), tag);
  }
};
#else
struct Tracer {
  __device__ __forceinline__ void init(ulonglong2 *, int, bool) {}
  __device__ __forceinline__ void mark(unsigned) {}
};
#endif

}  // namespace ptx

// ------------------------------------------------------------------ activation helpers
// The 32 visibility bits of a chunk as eight shifted copies: copy s has bit 8i + 7 - s in the sign
// position of byte i, from where a byte permute in sign-replication mode turns two bits into the
// 16-bit lane masks of a packed pair - 3 instructions per pair instead of a test and a select per
// element.
struct PairMasks {
  uint32_t sh[8];
  __device__ __forceinline__ explicit PairMasks(uint32_t bits) {
#pragma unroll
    for (int s = 0; s < 8; ++s) sh[s] = bits << s;
  }
  // lane mask of elements (2x, 2x + 1): 0xffff in the half whose bit is set
  __device__ __forceinline__ uint32_t pair(int x) const {
    const int i = x / 4, s = 7 - (2 * x) % 8;
    const uint32_t sel = ((0xCu + i) << 12) | ((0xCu + i) << 8) | ((8u + i) << 4) | (8u + i);
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(sh[s]), "r"(sh[s - 1]), "r"(sel));
    return d;
  }
};

// two fp32 products in one instruction (packed fp32 arithmetic of sm_100): {a0, a1} * s
__device__ __forceinline__ void mul2(float a0, float a1, float s, float &d0, float &d1) {
  asm("{\n\t.reg .b64 ra, rb, rc;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\t"
      "mul.rn.f32x2 rc, ra, rb;\n\tmov.b64 {%0, %1}, rc;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(s));
}
// {a0, a1} * {b0, b1}
__device__ __forceinline__ void mul2v(float a0, float a1, float b0, float b1, float &d0, float &d1) {
  asm("{\n\t.reg .b64 ra, rb, rc;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rc, ra, rb;\n\tmov.b64 {%0, %1}, rc;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
// {a0, a1} * {b0, b1} + {c0, c1}
__device__ __forceinline__ void fma2(float a0, float a1, float b0, float b1, float c0, float c1, float &d0,
                                     float &d1) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mov.b64 rc, {%6, %7};\n\tfma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}

}  // namespace b200hstu
