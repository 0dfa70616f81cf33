// Stand-alone micro-benchmark (not part of the library): cycles per tcgen05.mma for
// several shapes / operand sources. Build and run on a B200:
//   nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -o umma_rate sp_aurora_b200/csrc/umma_rate_microbench.cu && ./umma_rate
#include <cstdio>
#include <cuda_runtime.h>
#include "tc05.cuh"
using namespace spa;

// mode: 0 SS (A K-major, B K-major), 1 SS (A K-major, B MN-major), 2 TS (B K-major), 3 TS (B MN-major),
//       4 SS (A MN-major, B MN-major)
template <int N, int MODE>
__global__ void __launch_bounds__(128, 1) k(unsigned long long* out, int rounds) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  __shared__ volatile int abortf;
  __shared__ int status[4];
  if (threadIdx.x == 0) { mbar_init(&bar, 1); fence_mbar_init(); abortf = 0; status[0]=0; }
  for (int i = threadIdx.x; i < 96 * 1024 / 4; i += 128) ((uint32_t*)smem)[i] = 0x3c003c00u;
  fence_proxy_async_smem();
  if (threadIdx.x < 32) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  uint32_t tb = slot;
  WaitCtx wc{status, &abortf, nullptr};
  if (threadIdx.x == 0) {
    const bool a_mn = MODE == 4, b_mn = (MODE == 1 || MODE == 3 || MODE == 4);
    const uint32_t idesc = make_idesc(128, N, true, a_mn, b_mn);
    SmemDesc a = make_smem_desc(smem_u32(smem), a_mn ? 16384 : 16, 1024);
    SmemDesc b = make_smem_desc(smem_u32(smem + 32768), b_mn ? 16384 : 16, 1024);
    long long t0 = clock64();
    for (int r = 0; r < rounds; ++r) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t koff = ((kk / 4) * 16384 + (kk % 4) * 32) >> 4;   // K-major step
        const uint32_t moff = (kk * 2048) >> 4;                            // MN-major step
        if (MODE == 2 || MODE == 3)
          mma_ts_d(tb, tb + 256 + kk * 8, b, b_mn ? moff : koff, idesc, 1);
        else
          mma_ss_d(tb, a, a_mn ? moff : koff, b, b_mn ? moff : koff, idesc, 1);
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

template <int N, int MODE>
void run(const char* name, unsigned long long* d) {
  int rounds = 2000;
  cudaFuncSetAttribute(k<N, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  k<N, MODE><<<148, 128, 100 * 1024>>>(d, rounds);
  cudaError_t e = cudaDeviceSynchronize();
  unsigned long long h = 0;
  cudaMemcpy(&h, d, 8, cudaMemcpyDeviceToHost);
  double per = (double)h / (rounds * 8.0);
  double ideal = 128.0 * N * 16 * 2 / 8192.0;
  printf("%-28s N=%3d : %7.1f cycles/MMA (ideal %5.1f)  eff %.2f  %s\n", name, N, per, ideal, ideal / per,
         e == cudaSuccess ? "" : cudaGetErrorString(e));
}

int main() {
  unsigned long long* d; cudaMalloc(&d, 8);
  run<64, 0>("SS A:K  B:K", d);   run<128, 0>("SS A:K  B:K", d);   run<256, 0>("SS A:K  B:K", d);
  run<64, 1>("SS A:K  B:MN", d);  run<128, 1>("SS A:K  B:MN", d);
  run<64, 4>("SS A:MN B:MN", d);  run<128, 4>("SS A:MN B:MN", d);
  run<64, 2>("TS      B:K", d);   run<128, 2>("TS      B:K", d);   run<256, 2>("TS      B:K", d);
  run<64, 3>("TS      B:MN", d);  run<128, 3>("TS      B:MN", d);
  return 0;
}
