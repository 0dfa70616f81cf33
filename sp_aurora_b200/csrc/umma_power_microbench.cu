// Stand-alone micro-benchmark (not part of the library): tcgen05.mma rate under sustained load
// with constant vs random operand data (switching power). Build and run:
//   nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -o umma_power sp_aurora_b200/csrc/umma_power_microbench.cu && ./umma_power
#include <cstdio>
#include <cuda_runtime.h>
#include "tc05.cuh"
using namespace spa;

template <int N>
__global__ void __launch_bounds__(128, 1) k(unsigned long long* out, int rounds, int random_data) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  __shared__ volatile int abortf;
  __shared__ int status[4];
  if (threadIdx.x == 0) { mbar_init(&bar, 1); fence_mbar_init(); abortf = 0; status[0] = 0; }
  uint32_t x = 0x9e3779b9u * (threadIdx.x + 1 + blockIdx.x * 131);
  for (int i = threadIdx.x; i < 96 * 1024 / 4; i += blockDim.x) {
    x = x * 1664525u + 1013904223u;
    // random bf16 pairs in [-2, 2): sign + exponent 0x3f/0x40 + random mantissa
    uint32_t v = random_data ? ((x & 0x807f807fu) | 0x3f803f80u) : 0x3c003c00u;
    ((uint32_t*)smem)[i] = v;
  }
  fence_proxy_async_smem();
  if (threadIdx.x < 32) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tb = slot;
  WaitCtx wc{status, &abortf, nullptr};
  if (threadIdx.x == 0) {
    const uint32_t idesc = make_idesc(128, N, true, false, false);
    SmemDesc a = make_smem_desc(smem_u32(smem), 16, 1024);
    SmemDesc b = make_smem_desc(smem_u32(smem + 32768), 16, 1024);
    long long t0 = clock64();
    long long tmid = 0;
    for (int r = 0; r < rounds; ++r) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t koff = ((kk / 4) * 16384 + (kk % 4) * 32) >> 4;
        mma_ss_d(tb + (r & 1) * 256, a, koff, b, koff, idesc, kk > 0);   // fresh accumulation every round
      }
      if (r == rounds / 2) tmid = clock64();
    }
    mma_commit(&bar);
    mbar_wait(&bar, 0, wc, 0, 0);
    long long t1 = clock64();
    if (blockIdx.x == 0) { out[0] = (unsigned long long)(t1 - t0); out[1] = (unsigned long long)(t1 - tmid); }
  }
  tc_fence_before(); __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tb, 512); }
}

template <int N>
void run(unsigned long long* d, int rounds, int random_data) {
  cudaFuncSetAttribute(k<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  cudaEventRecord(e0);
  k<N><<<148, 128, 100 * 1024>>>(d, rounds, random_data);
  cudaEventRecord(e1);
  cudaError_t e = cudaDeviceSynchronize();
  float ms = 0; cudaEventElapsedTime(&ms, e0, e1);
  unsigned long long h[2];
  cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost);
  double per = (double)h[0] / (rounds * 8.0), per2 = (double)h[1] / (rounds * 4.0);
  double tflops = 148.0 * rounds * 8.0 * 128 * N * 16 * 2 / (ms * 1e-3) / 1e12;
  printf("N=%3d %-8s rounds=%7d : %6.1f cycles/MMA (second half %6.1f)  %7.2f ms  %7.1f TFLOP/s  avg SM clock %.0f MHz %s\n",
         N, random_data ? "random" : "constant", rounds, per, per2, ms, tflops, (double)h[0] / (ms * 1e3),
         e == cudaSuccess ? "" : cudaGetErrorString(e));
}

int main() {
  unsigned long long* d; cudaMalloc(&d, 64);
  run<128>(d, 2000, 0); run<128>(d, 2000, 1);
  run<128>(d, 400000, 0); run<128>(d, 400000, 1);
  run<64>(d, 400000, 1); run<256>(d, 200000, 1);
  return 0;
}
