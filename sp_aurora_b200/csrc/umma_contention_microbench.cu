// Stand-alone micro-benchmark (not part of the library): cycles per tcgen05.mma while
// other warps of the CTA generate shared-memory or tensor-memory traffic. Build and run:
//   nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -o umma_cont sp_aurora_b200/csrc/umma_contention_microbench.cu && ./umma_cont
#include <cstdio>
#include <cuda_runtime.h>
#include "tc05.cuh"
using namespace spa;

// Warp 0 issues MMAs. Warps 1..NW run `noise`:
//  0 none, 1 STS.128 stream, 2 LDS.128 broadcast stream, 3 tcgen05.ld 32x32b.x32 stream,
//  4 tcgen05.st 32x32b.x32 stream, 5 STS.32 stream (128 B per warp instruction),
//  6 bulk async copies global->shared (32 KB each, one thread), 7 bulk async reduce-add f32
//  shared->global (32 KB each, one thread), 8 MUFU ex2 stream
template <int N, bool TS>
__global__ void __launch_bounds__(288, 1) k(unsigned long long* out, int rounds, int noise, int nwarps,
                                            float* gbuf) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  __shared__ volatile int abortf, stop;
  __shared__ int status[4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); fence_mbar_init(); abortf = 0; stop = 0; status[0] = 0; }
  for (int i = threadIdx.x; i < 128 * 1024 / 4; i += blockDim.x) ((uint32_t*)smem)[i] = 0x3c003c00u;
  fence_proxy_async_smem();
  if (warp == 0) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tb = slot;
  WaitCtx wc{status, &abortf, nullptr};
  if (warp == 0) {
    const uint32_t leader = lane == 0;
    const uint32_t idesc = make_idesc(128, N, true, false, false);
    SmemDesc a = make_smem_desc(smem_u32(smem), 16, 1024);
    SmemDesc b = make_smem_desc(smem_u32(smem + 32768), 16, 1024);
    long long t0 = clock64();
    for (int r = 0; r < rounds; ++r) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t koff = ((kk / 4) * 16384 + (kk % 4) * 32) >> 4;
        if (TS) mma_ts_u(tb, tb + 256 + kk * 8, b, koff, idesc, 1, leader);
        else mma_ss_u(tb, a, koff, b, koff, idesc, 1, leader);
      }
    }
    mma_commit_u(&bar, leader);
    mbar_wait(&bar, 0, wc, 0, 0);
    long long t1 = clock64();
    stop = 1;
    if (blockIdx.x == 0 && lane == 0) out[0] = (unsigned long long)(t1 - t0);
  } else if (warp <= nwarps && noise) {
    uint8_t* scratch = smem + 65536 + (warp - 1) * 4096;     // private 4 KB per noise warp
    const uint32_t tq = tb + (static_cast<uint32_t>((warp & 3) * 32) << 16) + 320;
    uint32_t v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = i + lane;
    unsigned long long n = 0;
    while (!stop) {
      if (noise == 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(smem_u32(scratch + ((lane + 32 * i) & 255) * 16)),
                       "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]) : "memory");
      } else if (noise == 2) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          uint32_t x0, x1, x2, x3;
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3)
                       : "r"(smem_u32(scratch + i * 16)));
          v[i] += x0 + x3;
        }
      } else if (noise == 3) {
        tmem_ld32(tq, v);
        tmem_ld_wait();
      } else if (noise == 4) {
        tmem_st32(tq, v);
        tmem_st_wait();
      } else if (noise == 6) {
        if (warp == 1 && lane == 0) {
          __shared__ uint64_t lbar;
          if (n == 0) { mbar_init(&lbar, 1); fence_mbar_init(); }
          mbar_arrive_expect_tx(&lbar, 32768);
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(smem_u32(smem + 98304)), "l"(gbuf + (size_t)blockIdx.x * 65536 + (n & 7) * 8192), "r"(32768),
                         "r"(smem_u32(&lbar)) : "memory");
          mbar_wait(&lbar, n & 1, wc, 1, 0);
        }
      } else if (noise == 7) {
        if (warp == 1 && lane == 0) {
          asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;"
                       ::"l"(gbuf + (size_t)blockIdx.x * 65536 + (n & 7) * 8192), "r"(smem_u32(smem + 98304)), "r"(32768)
                       : "memory");
          bulk_commit_group();
          bulk_wait_read_all();
        }
      } else if (noise == 8) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __float_as_uint(fast_exp2(__uint_as_float(v[i])));
      } else if (noise == 5) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          asm volatile("st.shared.u32 [%0], %1;" ::"r"(smem_u32(scratch + i * 128 + lane * 4)), "r"(v[i]) : "memory");
      }
      ++n;
    }
    if (noise == 7 && warp == 1 && lane == 0) bulk_wait_all();
    if (blockIdx.x == 0 && lane == 0) out[warp] = n * 8;   // noise instructions issued (x8 for 1,2,5)
    if (v[5] == 0xdeadbeef) out[40] = v[7];
  }
  tc_fence_before(); __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tb, 512); }
}

template <int N, bool TS>
void run(const char* name, unsigned long long* d, int noise, int nwarps) {
  int rounds = 1000;
  cudaMemset(d, 0, 64 * 8);
  cudaFuncSetAttribute(k<N, TS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 132 * 1024);
  static float* gbuf = nullptr;
  if (!gbuf) { cudaMalloc(&gbuf, (size_t)148 * 65536 * 4); cudaMemset(gbuf, 0, (size_t)148 * 65536 * 4); }
  k<N, TS><<<148, 288, 132 * 1024>>>(d, rounds, noise, nwarps, gbuf);
  cudaError_t e = cudaDeviceSynchronize();
  unsigned long long h[16];
  cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
  double per = (double)h[0] / (rounds * 8.0);
  double noise_per_cycle = 0;
  for (int w = 1; w <= nwarps; ++w) noise_per_cycle += (double)h[w];
  noise_per_cycle /= (double)h[0];
  static const char* nn[] = {"none", "STS.128", "LDS.128 bcast", "tcgen05.ld x32", "tcgen05.st x32", "STS.32",
                             "bulk load 32K", "bulk red.add 32K", "MUFU ex2"};
  printf("%-3s N=%3d  noise=%-15s x%d warps : %6.1f cycles/MMA   noise instr/clk %.3f %s\n", name, N,
         nn[noise], nwarps, per, noise_per_cycle, e == cudaSuccess ? "" : cudaGetErrorString(e));
}

int main() {
  unsigned long long* d; cudaMalloc(&d, 64 * 8);
  for (int noise = 0; noise <= 8; ++noise) {
    int nw = noise ? 8 : 0;
    run<64, false>("SS", d, noise, nw);
    run<128, false>("SS", d, noise, nw);
    run<128, true>("TS", d, noise, nw);
  }
  run<64, false>("SS", d, 1, 2); run<64, false>("SS", d, 1, 4);
  run<64, false>("SS", d, 3, 4); run<128, true>("TS", d, 3, 4);
  return 0;
}
