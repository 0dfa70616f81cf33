// Stand-alone micro-benchmark (not part of the library): cost of switching accumulator /
// instruction shape between short tcgen05.mma chains, and of per-chain commits. Build and run:
//   nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -o umma_switch sp_aurora_b200/csrc/umma_switch_microbench.cu && ./umma_switch
#include <cstdio>
#include <cuda_runtime.h>
#include "tc05.cuh"
using namespace spa;

// mode 0: one accumulator, chains of CH MMAs (first of each chain overwrites)
// mode 1: chains alternate between two accumulators
// mode 2: like 1, and a tcgen05.commit (to a barrier nobody waits on) after every chain
// mode 4: mode 3 plus a tcgen05.fence::after_thread_sync before each group of MMAs
// mode 5: mode 3 plus a (satisfied) mbarrier.try_wait + fence before each group
// mode 6: mode 3 with the stage offset read from memory each iteration (runtime descriptors)
// mode 3: the backward kernel's iteration: S^T(8,N64) dP^T(8,N64) dV(4,N128,TS) dK(4,N128,TS) dQ^T(8,N64,MN/MN), 3 commits
template <int N, int CH, int MODE>
__global__ void __launch_bounds__(128, 1) k(unsigned long long* out, int rounds, const int* rt) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar, bar2[4];
  __shared__ uint32_t slot;
  __shared__ volatile int abortf;
  __shared__ int status[4];
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    for (int i = 0; i < 4; ++i) mbar_init(&bar2[i], 1);
    fence_mbar_init(); abortf = 0; status[0] = 0;
  }
  for (int i = threadIdx.x; i < 128 * 1024 / 4; i += blockDim.x) ((uint32_t*)smem)[i] = 0x3c003c00u;
  fence_proxy_async_smem();
  if (threadIdx.x < 32) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tb = slot;
  WaitCtx wc{status, &abortf, nullptr};
  if (threadIdx.x == 0) {
    SmemDesc a = make_smem_desc(smem_u32(smem), 16, 1024);
    SmemDesc b = make_smem_desc(smem_u32(smem + 32768), 16, 1024);
    SmemDesc amn = make_smem_desc(smem_u32(smem), 16384, 1024);
    SmemDesc bmn = make_smem_desc(smem_u32(smem + 32768), 8192, 1024);
    const uint32_t i64 = make_idesc(128, 64, true, false, false);
    const uint32_t i128mn = make_idesc(128, 128, true, false, true);
    const uint32_t i64mnmn = make_idesc(128, 64, true, true, true);
    const uint32_t idn = make_idesc(128, N, true, false, false);
    long long t0 = clock64();
    for (int r = 0; r < rounds; ++r) {
      if (MODE >= 3) {
        const uint32_t rto = (MODE == 6) ? (uint32_t)((const volatile int*)rt)[r % 3] : 0u;   // 0 at run time
        if (MODE == 4 || MODE == 5) tc_fence_after();
        if (MODE == 5) { mbar_try_wait(&bar2[3], 1); tc_fence_after(); }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) mma_ss_d(tb + 0, a, ((kk / 4) * 16384 + (kk % 4) * 32) >> 4, b, rto + (((kk / 4) * 8192 + (kk % 4) * 32) >> 4), i64, kk > 0);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) mma_ss_d(tb + 64, a, ((kk / 4) * 16384 + (kk % 4) * 32) >> 4, b, rto + (((kk / 4) * 8192 + (kk % 4) * 32) >> 4), i64, kk > 0);
        mma_commit(&bar2[0]);
        if (MODE == 4 || MODE == 5) tc_fence_after();
        if (MODE == 5) { mbar_try_wait(&bar2[3], 1); tc_fence_after(); }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) mma_ts_d(tb + 128, tb + 448 + kk * 8, bmn, rto + ((kk * 2048) >> 4), i128mn, 1);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) mma_ts_d(tb + 256, tb + 480 + kk * 8, bmn, rto + ((kk * 2048) >> 4), i128mn, 1);
        if (MODE == 4 || MODE == 5) tc_fence_after();
        if (MODE == 5) { mbar_try_wait(&bar2[3], 1); tc_fence_after(); }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) mma_ss_d(tb + 384, amn, (kk * 2048) >> 4, bmn, (kk * 2048) >> 4, i64mnmn, kk > 0);
        mma_commit(&bar2[1]);
        mma_commit(&bar2[2]);
      } else {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const uint32_t acc = tb + ((MODE >= 1 && c) ? 256 : 0);
#pragma unroll
          for (int kk = 0; kk < CH; ++kk)
            mma_ss_d(acc, a, (((kk % 8) / 4) * 16384 + (kk % 4) * 32) >> 4, b, (((kk % 8) / 4) * 16384 + (kk % 4) * 32) >> 4, idn, kk > 0);
          if (MODE == 2) mma_commit(&bar2[c]);
        }
      }
    }
    mma_commit(&bar);
    mbar_wait(&bar, 0, wc, 0, 0);
    long long t1 = clock64();
    if (blockIdx.x == 0) out[0] = (unsigned long long)(t1 - t0);
  }
  tc_fence_before(); __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tb, 512); }
}

template <int N, int CH, int MODE>
void run(const char* name, unsigned long long* d) {
  int rounds = 1000;
  cudaFuncSetAttribute(k<N, CH, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 132 * 1024);
  static int* rt = nullptr;
  if (!rt) { cudaMalloc(&rt, 16); cudaMemset(rt, 0, 16); }
  k<N, CH, MODE><<<148, 128, 132 * 1024>>>(d, rounds, rt);
  cudaError_t e = cudaDeviceSynchronize();
  unsigned long long h = 0;
  cudaMemcpy(&h, d, 8, cudaMemcpyDeviceToHost);
  if (MODE >= 3)
    printf("%-44s : %8.1f cycles per iteration (MMA time at isolated rates 1664) %s\n", name, (double)h / rounds,
           e == cudaSuccess ? "" : cudaGetErrorString(e));
  else
    printf("%-44s N=%3d chain=%2d : %6.1f cycles/MMA %s\n", name, N, CH, (double)h / (rounds * 2.0 * CH),
           e == cudaSuccess ? "" : cudaGetErrorString(e));
}

int main() {
  unsigned long long* d; cudaMalloc(&d, 64);
  run<64, 8, 0>("one accumulator", d);        run<128, 8, 0>("one accumulator", d);
  run<64, 8, 1>("two accumulators alternating", d); run<128, 8, 1>("two accumulators alternating", d);
  run<64, 4, 1>("two accumulators alternating", d); run<128, 4, 1>("two accumulators alternating", d);
  run<64, 8, 2>("alternating + commit per chain", d); run<128, 8, 2>("alternating + commit per chain", d);
  run<64, 4, 2>("alternating + commit per chain", d);
  run<64, 8, 3>("backward iteration sequence (32 MMAs)", d);
  run<64, 8, 4>("  + fence::after_thread_sync x3", d);
  run<64, 8, 5>("  + try_wait + fences x3", d);
  run<64, 8, 6>("  + runtime stage offset in descriptors", d);
  return 0;
}
