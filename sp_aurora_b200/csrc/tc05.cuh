// Thin inline-PTX wrappers for the Blackwell (sm_100a) primitives the attention
// kernels use: mbarriers with BOUNDED waits, TMA tiled loads, tcgen05 tensor
// memory allocation, tcgen05.mma (operands from shared memory), tcgen05.ld/st
// and the fences that order the generic, async and tensor-core proxies.
//
// Every wait in this file gives up after a clock budget, records where it gave
// up in a global status word and lets the kernel run to its normal exit (TMEM
// freed, no trap), so that a protocol bug can never leave the GPU spinning.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace spa {

// ---------------------------------------------------------------------------
// Status word shared by all CTAs of a launch (device global memory, 4 ints):
//   [0] error code (0 = ok)   [1] blockIdx.x   [2] site id   [3] iteration
// ---------------------------------------------------------------------------
enum : int { ST_OK = 0, ST_WAIT_TIMEOUT = 1 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One arrival for a whole warp: the lanes' earlier writes (TMEM stores completed by
// tcgen05.wait::st, shared-memory stores) are ordered before lane 0's releasing arrive by
// the warp barrier. 32 lanes arriving one by one on the same word keep the shared-memory
// pipe busy for tens of cycles per warp; barriers that compute warps arrive on count warps.
// Every lane of the warp must reach the call.
__device__ __forceinline__ void warp_arrive(uint64_t* bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Per-CTA view of the abort machinery.
struct WaitCtx {
  int* status;            // global status word (4 ints)
  volatile int* cta_abort;  // shared-memory flag of this CTA
};

#ifndef SPA_WAIT_BUDGET_CYCLES
#define SPA_WAIT_BUDGET_CYCLES (4000000000ll)  // about two seconds of SM clock
#endif

// Wait for `parity` of `bar`. Returns false (and flags the launch as failed)
// when the budget runs out or when another CTA already flagged a failure, in
// which case the caller must skip its work and fall through to the exit path.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& w,
                                          int site, int iter) {
  // Fast path: one try_wait, no shared-memory read and no clock read (a clock read before
  // every wait costs ~15 % of kernel time, and every extra shared-memory round trip adds
  // to a latency that each pipeline hop pays). A CTA that has aborted reaches the slow
  // path at its next unsatisfied wait and leaves there.
  if (mbar_try_wait(bar, parity)) return true;
  if (*w.cta_abort) return false;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0x3ff) == 0) {
      if (*w.cta_abort) return false;
      if (*reinterpret_cast<volatile int*>(w.status) != 0) {
        *w.cta_abort = 1;
        return false;
      }
      if (clock64() - t0 > SPA_WAIT_BUDGET_CYCLES) {
        if (atomicCAS(w.status, 0, ST_WAIT_TIMEOUT) == 0) {
          w.status[1] = blockIdx.x;
          w.status[2] = site;
          w.status[3] = iter;
          __threadfence();
        }
        *w.cta_abort = 1;
        return false;
      }
    }
  }
}

// Whole-warp wait: every lane waits, then the warp agrees on one outcome so that
// warp-collective tcgen05.ld/st that follow are never executed by a partial warp.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, const WaitCtx& w,
                                          int site, int iter) {
  const bool ok = mbar_wait(bar, parity, w, site, iter);
  return __all_sync(0xffffffffu, ok);
}

// ---------------------------------------------------------------------------
// TMA: tiled bulk tensor loads global -> shared, completion on an mbarrier.
// The innermost coordinate times the element size must be a multiple of 16 B.
// No cluster multicast anywhere in this library.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Bulk tensor reduce-add shared -> global (fp32 tile added into global memory by
// the TMA unit; rows outside the tensor are clipped). Completion is tracked by
// the issuing thread's bulk async-group.
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* m, const void* src, int c0,
                                                  int c1, int c2, int c3) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group"
      " [%0, {%2, %3, %4, %5}], [%1];" ::"l"(reinterpret_cast<uint64_t>(m)),
      "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// Bulk tensor store shared -> global (rows outside the tensor are clipped), tracked by
// the issuing thread's bulk async-group like the reduction above.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, const void* src, int c0, int c1,
                                             int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group"
      " [%0, {%2, %3, %4, %5}], [%1];" ::"l"(reinterpret_cast<uint64_t>(m)),
      "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Wait until all committed bulk groups have completed (writes performed).
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// ---------------------------------------------------------------------------
// Tensor memory (TMEM) management. One warp allocates and the same warp frees.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------
// Descriptors.
//
// Shared-memory matrix descriptor (64 bit) for a 128-byte-swizzled tile whose
// rows are 128 bytes (64 two-byte elements) and whose 8-row groups are 1024 B:
//   bits  0-13 start address >> 4        bits 16-29 leading byte offset >> 4
//   bits 32-45 stride byte offset >> 4   bits 46-47 descriptor version (1)
//   bits 61-63 swizzle mode (2 = 128 B)
// K-major operand  (rows = M or N, row bytes = K): SBO = bytes between 8-row
//   groups (1024); LBO unused; advance K by 16 elements = +32 B.
// MN-major operand (rows = K, row bytes = 64 elements of M or N): SBO = bytes
//   between 8-row K groups (1024); LBO = bytes between successive 64-element
//   column slabs; advance K by 16 rows = +2048 B.
// ---------------------------------------------------------------------------
// The same descriptor split into its two 32-bit words, so that the issuing thread
// can step through a tile by adding a (compile-time) constant to the low word
// instead of rebuilding 64 bits per MMA: byte offset `off` -> lo + (off >> 4).
struct SmemDesc {
  uint32_t lo, hi;
};
__device__ __forceinline__ SmemDesc make_smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes) {
  SmemDesc d;
  d.lo = ((saddr & 0x3FFFF) >> 4) | (((lbo_bytes >> 4) & 0x3FFF) << 16);
  d.hi = ((sbo_bytes >> 4) & 0x3FFF) | (1u << 14) | (2u << 29);
  return d;
}

// Instruction descriptor for tcgen05.mma kind::f16 with fp32 accumulation:
//   bits 4-5 D format (1 = f32); bits 7-9 A format, bits 10-12 B format
//   (0 = f16, 1 = bf16); bit 15 A is MN-major; bit 16 B is MN-major;
//   bits 17-22 N >> 3; bits 24-28 M >> 4.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, bool bf16, bool a_mn, bool b_mn) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) |
         ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread. Operands are split descriptors
// plus offsets in 16-byte units.
__device__ __forceinline__ void mma_ss_d(uint32_t d_tmem, SmemDesc a, uint32_t a_off16, SmemDesc b,
                                         uint32_t b_off16, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
      "r"(a.lo + a_off16), "r"(a.hi), "r"(b.lo + b_off16), "r"(b.hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; A is read from tensor memory (rows = TMEM lanes, 16-bit
// elements packed two per 32-bit column, 8 columns per K=16 step).
__device__ __forceinline__ void mma_ts_d(uint32_t d_tmem, uint32_t a_tmem, SmemDesc b,
                                         uint32_t b_off16, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b.lo + b_off16), "r"(b.hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on `bar` when every tcgen05 operation issued so far by this thread
// has completed (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
          smem_u32(bar))
      : "memory");
}

// ---------------------------------------------------------------------------
// TMEM <-> registers, shape 32x32b: lane i of the warp reads/writes TMEM lane
// (32*(warp%4) + i), 32 consecutive 32-bit columns starting at taddr's column.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};" ::"r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31]), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};" ::"r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%8], {%0, %1, %2, %3, %4, %5, %6, %7};" ::"r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(taddr)
      : "memory");
}
// Shape 16x256b, 4 repetitions (32 columns) of 16 TMEM lanes starting at taddr's
// lane: with g = laneid / 4 and t = laneid % 4, r[4i+0], r[4i+1] are (lane g,
// columns 8i+2t, 8i+2t+1) and r[4i+2], r[4i+3] are (lane g+8, same columns).
__device__ __forceinline__ void tmem_ld_16x256b_x4(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// Shape 16x128b, 4 repetitions (16 columns) of 16 TMEM lanes: r[2i+0] is (lane g,
// column 4i+t), r[2i+1] is (lane g+8, column 4i+t).
__device__ __forceinline__ void tmem_st_16x128b_x4(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x128b.x4.b32 [%8], {%0, %1, %2, %3, %4, %5, %6, %7};" ::"r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Packed fp32 arithmetic (two lanes per instruction on the FMA pipe): the compute warps of
// the attention kernels are bound by instruction issue, and these halve the count of their
// multiply-adds. (d0, d1) = (a0, a1) * (b0, b1) + (c0, c1), and the add / multiply forms.
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b0, float b1,
                                     float c0, float c1) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void add2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ void mul2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace spa
