// extern "C" surface of libspaurora_sm100 plus the HBM-bound helper kernels
// (delta row sums, stand-alone out/lse merge, fp32 -> element-type cast,
// Ulysses pack/unpack row permutation) and host-side plumbing: argument
// validation, TMA descriptor encoding, the per-device status word.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "spa_internal.h"

namespace spa {

// ------------------------------------------------------------------ errors
static thread_local char g_err[512] = "";
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

static std::atomic<long long> g_launches{0};
static inline void note_launch(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// --------------------------------------------------------- device status word
// Four ints per device, part of the library image (zero until a bounded wait gives up);
// host code needs the device address, looked up once per device.
static __device__ int g_status_dev[4];
static std::mutex g_status_mu;
static int* g_status[64] = {nullptr};

int* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("cudaGetDevice failed");
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_status_mu);
  if (!g_status[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_status_dev);
    if (e != cudaSuccess || !p) {
      set_error("status word lookup: %s", cudaGetErrorString(e));
      return nullptr;
    }
    g_status[dev] = static_cast<int*>(p);
  }
  return g_status[dev];
}

// --------------------------------------------- per-device kernel attributes
namespace {
struct SmemAttrEntry {
  const void* kernel;
  int device;
  int bytes;
};
std::mutex g_attr_mu;
SmemAttrEntry g_attr[256];
int g_attr_n = 0;
}  // namespace

// Pure bookkeeping of ensure_dynamic_smem: true when (kernel, device) was already raised
// to at least `bytes`; otherwise records it and returns false.
bool smem_attr_seen(const void* kernel, int device, int bytes) {
  std::lock_guard<std::mutex> lk(g_attr_mu);
  for (int i = 0; i < g_attr_n; ++i)
    if (g_attr[i].kernel == kernel && g_attr[i].device == device) {
      if (g_attr[i].bytes >= bytes) return true;
      g_attr[i].bytes = bytes;
      return false;
    }
  if (g_attr_n < 256) g_attr[g_attr_n++] = SmemAttrEntry{kernel, device, bytes};
  return false;
}

int ensure_dynamic_smem(const void* kernel, int bytes, const char* what) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    set_error("cudaGetDevice failed");
    return SPA_ECUDA;
  }
  if (smem_attr_seen(kernel, dev, bytes)) return SPA_OK;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) {
    set_error("cudaFuncSetAttribute(%s, %d bytes): %s", what, bytes, cudaGetErrorString(e));
    return SPA_ECUDA;
  }
  return SPA_OK;
}

int device_sm_count() {
  static std::atomic<int> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int v = cache[dev].load(std::memory_order_relaxed);
  if (v > 0) return v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
  cache[dev].store(v, std::memory_order_relaxed);
  return v;
}

// ------------------------------------------------------- TMA descriptor encode
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e =
        cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = (EncodeTiledFn)sym;
  }
  return fn;
}

int encode_rows_map(CUtensorMap* map, const void* ptr, int is_bf16, int D, int64_t S, int H, int B,
                    int64_t stride_s, int64_t stride_h, int64_t stride_b, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled entry point not available");
    return -1;
  }
  // Size-1 dimensions may carry arbitrary strides; give them harmless ones.
  if (S == 1) stride_s = D;
  if (H == 1) stride_h = D;
  if (B == 1) stride_b = D;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)stride_s * 2, (cuuint64_t)stride_h * 2,
                           (cuuint64_t)stride_b * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if (((uintptr_t)ptr & 15) || (strides[0] & 15) || (strides[1] & 15) || (strides[2] & 15)) {
    set_error("tensor base and strides must be 16-byte aligned for TMA");
    return -1;
  }
  CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                  4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d (D=%d S=%lld H=%d B=%d)", (int)r, D,
              (long long)S, H, B);
    return -1;
  }
  return 0;
}

int encode_f32_rows_map(CUtensorMap* map, const void* ptr, int D, int64_t S, int H, int B,
                        int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled entry point not available");
    return -1;
  }
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)H * D * 4, (cuuint64_t)D * 4, (cuuint64_t)S * H * D * 4};
  cuuint32_t box[4] = {(cuuint32_t)D, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if ((uintptr_t)ptr & 15) {
    set_error("fp32 accumulator must be 16-byte aligned for TMA");
    return -1;
  }
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(ptr), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled(fp32) failed with code %d", (int)r);
    return -1;
  }
  return 0;
}

int encode_f32_slab_map(CUtensorMap* map, const void* ptr, int D, int64_t S, int H, int B,
                        int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled entry point not available");
    return -1;
  }
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)H * D * 4, (cuuint64_t)D * 4, (cuuint64_t)S * H * D * 4};
  cuuint32_t box[4] = {32u, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if ((uintptr_t)ptr & 15) {
    set_error("fp32 gradient buffer must be 16-byte aligned for TMA");
    return -1;
  }
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(ptr), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled(fp32 slab) failed with code %d", (int)r);
    return -1;
  }
  return 0;
}

// ---------------------------------------------------------------- helpers
namespace {

template <typename T>
__device__ __forceinline__ float4 ld4(const T* p);
template <>
__device__ __forceinline__ float4 ld4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 ld4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
template <>
__device__ __forceinline__ float4 ld4<__half>(const __half* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T>
__device__ __forceinline__ void st4(T* p, float4 v);
template <>
__device__ __forceinline__ void st4<float>(float* p, float4 v) {
  *reinterpret_cast<float4*>(p) = v;
}
template <>
__device__ __forceinline__ void st4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}
template <>
__device__ __forceinline__ void st4<__half>(__half* p, float4 v) {
  __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

// One thread per 4 elements; D/4 consecutive threads (<= 32, a power of two,
// inside one warp) share a [b,s,h] row. Rows are numbered (b*S + s)*H + h.
struct RowIdx {
  int b, s, h;
};
// Idx is uint32_t whenever the thread count allows: the 64-bit divisions of the general
// case cost more issue slots than these streaming kernels have to spare.
template <typename Idx>
__device__ __forceinline__ RowIdx decode_row(Idx row, int S, int H) {
  RowIdx r;
  r.h = (int)(row % (Idx)H);
  row /= (Idx)H;
  r.s = (int)(row % (Idx)S);
  r.b = (int)(row / (Idx)S);
  return r;
}

// The pack/unpack copy keeps kVecPerThread independent 16-byte accesses in flight per
// thread (a block sweeps kVecPerThread coalesced runs of blockDim vectors) with the
// streaming (evict-first) hint.
constexpr int kVecPerThread = 4;
constexpr int kStreamBlock = 256;

inline long long stream_grid(long long n_vec) {
  const long long per_block = (long long)kStreamBlock * kVecPerThread;
  return (n_vec + per_block - 1) / per_block;
}

// 16 bytes of 2-byte elements (or 32 bytes of fp32) of two rows -> their partial dot product.
template <typename T>
struct Vec8 {
  uint4 lo, hi;   // hi is used by fp32 only
};
template <typename T>
__device__ __forceinline__ Vec8<T> load8(const T* p) {
  Vec8<T> v;
  v.lo = __ldcs(reinterpret_cast<const uint4*>(p));
  if (sizeof(T) == 4) v.hi = __ldcs(reinterpret_cast<const uint4*>(p) + 1); else v.hi = v.lo;
  return v;
}
template <typename T>
__device__ __forceinline__ float dot8(const Vec8<T>& a, const Vec8<T>& b);
template <>
__device__ __forceinline__ float dot8<float>(const Vec8<float>& a, const Vec8<float>& b) {
  const float* x = reinterpret_cast<const float*>(&a.lo);
  const float* y = reinterpret_cast<const float*>(&b.lo);
  const float* z = reinterpret_cast<const float*>(&a.hi);
  const float* w = reinterpret_cast<const float*>(&b.hi);
  return x[0] * y[0] + x[1] * y[1] + x[2] * y[2] + x[3] * y[3] + z[0] * w[0] + z[1] * w[1] +
         z[2] * w[2] + z[3] * w[3];
}
template <>
__device__ __forceinline__ float dot8<__nv_bfloat16>(const Vec8<__nv_bfloat16>& a,
                                                     const Vec8<__nv_bfloat16>& b) {
  const uint32_t wa[4] = {a.lo.x, a.lo.y, a.lo.z, a.lo.w}, wb[4] = {b.lo.x, b.lo.y, b.lo.z, b.lo.w};
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // a bf16 is the upper half of an fp32: two shifts / masks per pair instead of conversions
    acc = fmaf(__uint_as_float(wa[i] << 16), __uint_as_float(wb[i] << 16), acc);
    acc = fmaf(__uint_as_float(wa[i] & 0xffff0000u), __uint_as_float(wb[i] & 0xffff0000u), acc);
  }
  return acc;
}
template <>
__device__ __forceinline__ float dot8<__half>(const Vec8<__half>& a, const Vec8<__half>& b) {
  const uint32_t wa[4] = {a.lo.x, a.lo.y, a.lo.z, a.lo.w}, wb[4] = {b.lo.x, b.lo.y, b.lo.z, b.lo.w};
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __half22float2(*reinterpret_cast<const __half2*>(&wa[i]));
    const float2 y = __half22float2(*reinterpret_cast<const __half2*>(&wb[i]));
    acc = fmaf(x.x, y.x, acc);
    acc = fmaf(x.y, y.y, acc);
  }
  return acc;
}

// delta: one thread per 8 elements, D/8 consecutive lanes share a row. A warp takes
// kRowsInFlight * (32 / (D/8)) consecutive sequence positions of one (batch, head): every load
// is issued before the first use, and the row sums are gathered into the low lanes so that the
// warp writes its part of delta ([B,H,S]) as one contiguous run instead of one 4-byte store
// per sector. Consecutive warps take consecutive heads: the rows a block reads at one sequence
// position are adjacent in memory.
constexpr int kRowsInFlight = 4;

template <typename T, typename Idx>
__global__ void __launch_bounds__(256)
delta_kernel(const T* __restrict__ out, int64_t o_sb, int64_t o_ss, int64_t o_sh,
             const T* __restrict__ dout, int64_t d_sb, int64_t d_ss, int64_t d_sh,
             float* __restrict__ delta, int B, int S, int H, int D) {
  const int tpr = D / 8;                 // lanes per row: 4, 8 or 16
  const int rpw = 32 / tpr;              // rows per warp and pass
  const int sblk = kRowsInFlight * rpw;  // sequence positions per warp
  const int lane = threadIdx.x & 31;
  const Idx warp = ((Idx)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const Idx nsb = (Idx)((S + sblk - 1) / sblk);
  if (warp >= (Idx)B * nsb * (Idx)H) return;
  const int h = (int)(warp % (Idx)H);
  const Idx t = warp / (Idx)H;
  const int s0 = (int)(t % nsb) * sblk;
  const int b = (int)(t / nsb);
  const int sub = lane / tpr, c = (lane % tpr) * 8;
  const T* o0 = out + (int64_t)b * o_sb + (int64_t)h * o_sh + c;
  const T* d0 = dout + (int64_t)b * d_sb + (int64_t)h * d_sh + c;
  Vec8<T> va[kRowsInFlight], vb[kRowsInFlight];
  bool ok[kRowsInFlight];
#pragma unroll
  for (int u = 0; u < kRowsInFlight; ++u) {
    const int sq = s0 + u * rpw + sub;
    ok[u] = sq < S;
    if (ok[u]) {
      va[u] = load8<T>(o0 + (int64_t)sq * o_ss);
      vb[u] = load8<T>(d0 + (int64_t)sq * d_ss);
    }
  }
  float res = 0.f;
#pragma unroll
  for (int u = 0; u < kRowsInFlight; ++u) {
    float acc = ok[u] ? dot8<T>(va[u], vb[u]) : 0.f;
    for (int o = tpr >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    // lane L of the low `sblk` lanes keeps the sum of position L = u * rpw + sub
    const float v = __shfl_sync(0xffffffffu, acc, (lane % rpw) * tpr);
    if (lane / rpw == u) res = v;
  }
  if (lane < sblk && s0 + lane < S) delta[((size_t)b * H + h) * S + s0 + lane] = res;
}

// merge: a warp takes kMergeRows consecutive sequence positions of one (batch, head). Lane i
// (< kMergeRows) first turns the two lse values of position i into (lse', w_old, w_blk) -- the
// exponentials, the logarithm and the divisions are done once per row, not once per element
// vector, and the lse values of a warp are one contiguous 32-byte sector ([B,H,S] layout) --
// then the warp sweeps its rows, 128 floats (32 lanes x float4) per pass, with the weights of
// each row broadcast by shuffles. Consecutive warps take consecutive heads, so the rows a block
// touches at one sequence position are adjacent in memory.
constexpr int kMergeRows = 8;
template <typename T, typename Idx>
__global__ void __launch_bounds__(256)
merge_kernel(float* __restrict__ out_acc, float* __restrict__ lse, const T* __restrict__ bo,
             int64_t bo_sb, int64_t bo_ss, int64_t bo_sh, const float* __restrict__ blse, int B,
             int S, int H, int D) {
  const int lane = threadIdx.x & 31;
  const Idx warp = ((Idx)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const Idx nsb = (Idx)((S + kMergeRows - 1) / kMergeRows);
  if (warp >= (Idx)B * nsb * (Idx)H) return;
  const int h = (int)(warp % (Idx)H);
  const Idx t = warp / (Idx)H;
  const int s0 = (int)(t % nsb) * kMergeRows;
  const int b = (int)(t / nsb);
  const int n = min(kMergeRows, S - s0);
  // phase 1: lane i owns sequence position s0 + i
  const bool mine = lane < n;
  const size_t li = ((size_t)b * H + h) * S + s0 + (mine ? lane : 0);
  float w_old = 0.f, w_blk = 0.f;
  if (mine) {
    const float lo = lse[li], lb = blse[li];
    const float mx = fmaxf(lo, lb);
    float lse_new = mx;
    if (mx != -INFINITY) {
      const float eo = expf(lo - mx), eb = expf(lb - mx);
      const float sum = eo + eb;
      lse_new = mx + logf(sum);
      w_old = eo / sum;
      w_blk = eb / sum;
    }
    lse[li] = lse_new;
  }
  float* acc0 = out_acc + (((size_t)b * S + s0) * H + h) * D;          // row r: + r * H * D
  const T* bo0 = bo + (int64_t)b * bo_sb + (int64_t)s0 * bo_ss + (int64_t)h * bo_sh;   // row r: + r * bo_ss
  const size_t acc_step = (size_t)H * D;
  // phase 2: `rpp` rows per pass (a row is D/4 lanes wide), two passes in flight
  const int lpr = D / 4, rpp = 32 / lpr;
  const int sub = lane / lpr, c = (lane % lpr) * 4;
  for (int i = 0; i < n; i += 2 * rpp) {
    float4 av[2], xv[2];
    float wo[2], wb[2];
    int rr[2];
    bool ok[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      rr[u] = i + u * rpp + sub;
      const int src = min(rr[u], kMergeRows - 1);
      wo[u] = __shfl_sync(0xffffffffu, w_old, src);
      wb[u] = __shfl_sync(0xffffffffu, w_blk, src);
      ok[u] = rr[u] < n;
      if (ok[u]) {
        av[u] = __ldcs(reinterpret_cast<const float4*>(acc0 + rr[u] * acc_step + c));
        xv[u] = ld4<T>(bo0 + (int64_t)rr[u] * bo_ss + c);
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u)
      if (ok[u])
        __stcs(reinterpret_cast<float4*>(acc0 + rr[u] * acc_step + c),
               make_float4(wo[u] * av[u].x + wb[u] * xv[u].x, wo[u] * av[u].y + wb[u] * xv[u].y,
                           wo[u] * av[u].z + wb[u] * xv[u].z, wo[u] * av[u].w + wb[u] * xv[u].w));
  }
}

// Two independent 16-byte streaming loads per thread (82 -> 87 % of the copy peak).
template <typename T, typename Idx>
__global__ void cast_kernel(const float* __restrict__ src, T* __restrict__ dst, int64_t d_sb,
                            int64_t d_ss, int64_t d_sh, int B, int S, int H, int D, float alpha) {
  const int tpr = D / 4;
  const Idx nvec = (Idx)B * S * H * (Idx)tpr;
  const Idx g0 = ((Idx)blockIdx.x * 2) * blockDim.x + threadIdx.x;
  const Idx g1 = g0 + blockDim.x;
  float4 v0 = make_float4(0, 0, 0, 0), v1 = v0;
  if (g0 < nvec) v0 = __ldcs(reinterpret_cast<const float4*>(src) + g0);
  if (g1 < nvec) v1 = __ldcs(reinterpret_cast<const float4*>(src) + g1);
  if (g0 < nvec) {
    const RowIdx r = decode_row<Idx>(g0 / (Idx)tpr, S, H);
    const int c = (int)(g0 % (Idx)tpr) * 4;
    v0.x *= alpha; v0.y *= alpha; v0.z *= alpha; v0.w *= alpha;
    st4<T>(dst + r.b * d_sb + r.s * d_ss + r.h * d_sh + c, v0);
  }
  if (g1 < nvec) {
    const RowIdx r = decode_row<Idx>(g1 / (Idx)tpr, S, H);
    const int c = (int)(g1 % (Idx)tpr) * 4;
    v1.x *= alpha; v1.y *= alpha; v1.z *= alpha; v1.w *= alpha;
    st4<T>(dst + r.b * d_sb + r.s * d_ss + r.h * d_sh + c, v1);
  }
}

struct PermuteParams {
  int64_t n[4];
  int64_t ss[4];
  int64_t ds[4];
  int64_t vec_per_row;
  int64_t total_vec;
};
// Thread = kVecPerThread 16-byte vectors; consecutive threads walk a row, then the next
// logical row, so both sides see full-line accesses. Idx is the integer type of the
// vector / row arithmetic: 32-bit whenever the vector count allows (the 64-bit
// divisions of the general case cost more issue slots than the copy has to spare).
template <typename Idx>
__global__ void __launch_bounds__(kStreamBlock)
permute_rows_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                    const PermuteParams p) {
  const Idx vpr = (Idx)p.vec_per_row, n1 = (Idx)p.n[1], n2 = (Idx)p.n[2], n3 = (Idx)p.n[3];
  const int64_t chunk = (int64_t)gridDim.x * blockDim.x * kVecPerThread;
  for (int64_t base = (int64_t)blockIdx.x * blockDim.x * kVecPerThread; base < p.total_vec;
       base += chunk) {
    uint4 val[kVecPerThread];
    int64_t dof[kVecPerThread];
    bool ok[kVecPerThread];
#pragma unroll
    for (int u = 0; u < kVecPerThread; ++u) {
      const int64_t i64 = base + (int64_t)u * blockDim.x + threadIdx.x;
      ok[u] = i64 < p.total_vec;
      const Idx i = (Idx)(ok[u] ? i64 : 0);
      const Idx v = i % vpr;
      Idx r = i / vpr;
      const Idx i3 = r % n3; r /= n3;
      const Idx i2 = r % n2; r /= n2;
      const Idx i1 = r % n1; r /= n1;
      const Idx i0 = r;
      const int64_t so = (int64_t)i0 * p.ss[0] + (int64_t)i1 * p.ss[1] + (int64_t)i2 * p.ss[2] +
                         (int64_t)i3 * p.ss[3] + (int64_t)v * 16;
      dof[u] = (int64_t)i0 * p.ds[0] + (int64_t)i1 * p.ds[1] + (int64_t)i2 * p.ds[2] +
               (int64_t)i3 * p.ds[3] + (int64_t)v * 16;
      if (ok[u]) val[u] = __ldcs(reinterpret_cast<const uint4*>(src + so));
    }
#pragma unroll
    for (int u = 0; u < kVecPerThread; ++u)
      if (ok[u]) __stcs(reinterpret_cast<uint4*>(dst + dof[u]), val[u]);
  }
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s launch: %s", what, cudaGetErrorString(e));
    return SPA_ECUDA;
  }
  return SPA_OK;
}

bool valid_head_dim(int D) { return D == 32 || D == 64 || D == 128; }

bool force_simt() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("SPA_FORCE_CUDA_CORE");
    v = (e && e[0] == '1') ? 1 : 0;
  }
  return v == 1;
}

}  // namespace
// ---------------------------------------------------------------------------
// Rotary position embedding fused into a strided row copy (the Ulysses pack of q and k, or a
// plain in-layout rotation): dst[..., :D/2] = x1*cos - x2*sin, dst[..., D/2:] = x2*cos + x1*sin
// with x1, x2 the two halves of a head row ("rotate-half" convention) and cos/sin fp32 tables
// [table_rows, D/2] indexed by the token position = pos_offset + index along logical dim
// pos_dim. `inverse` negates sin (the gradient of the rotation). A thread moves one 16-byte
// vector of each half; HBM-bound: 2*N*elt bytes plus the (L2-resident) tables.
struct RopeParams {
  int64_t n[4];
  int64_t ss[4];   // element strides
  int64_t ds[4];
  int64_t total;   // vector pairs
  int64_t pos_off;
  int pos_dim, D;
  float sin_sign;
};

template <typename T>
struct RopeVec {
  static constexpr int kElts = 16 / sizeof(T);
  __device__ static void unpack(const uint4& v, float* f);
  __device__ static uint4 pack(const float* f);
};
template <>
__device__ void RopeVec<float>::unpack(const uint4& v, float* f) {
  f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
  f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
}
template <>
__device__ uint4 RopeVec<float>::pack(const float* f) {
  return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
}
template <>
__device__ void RopeVec<__nv_bfloat16>::unpack(const uint4& v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <>
__device__ uint4 RopeVec<__nv_bfloat16>::pack(const float* f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
template <>
__device__ void RopeVec<__half>::unpack(const uint4& v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}
template <>
__device__ uint4 RopeVec<__half>::pack(const float* f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

template <typename T>
__global__ void __launch_bounds__(kStreamBlock)
rope_rows_kernel(const T* __restrict__ src, T* __restrict__ dst, const float* __restrict__ cos_t,
                 const float* __restrict__ sin_t, const RopeParams p) {
  constexpr int E = RopeVec<T>::kElts;
  const int half = p.D / 2;
  const int64_t ppr = half / E;                       // vector pairs per row
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % ppr) * E;
    int64_t r = i / ppr;
    int64_t idx[4];
    idx[3] = r % p.n[3]; r /= p.n[3];
    idx[2] = r % p.n[2]; r /= p.n[2];
    idx[1] = r % p.n[1]; r /= p.n[1];
    idx[0] = r;
    int64_t so = c, dof = c;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      so += idx[k] * p.ss[k];
      dof += idx[k] * p.ds[k];
    }
    const int64_t pos = p.pos_off + idx[p.pos_dim];
    const uint4 lo = __ldcs(reinterpret_cast<const uint4*>(src + so));
    const uint4 hi = __ldcs(reinterpret_cast<const uint4*>(src + so + half));
    float x1[E], x2[E], cs[E], sn[E], y1[E], y2[E];
    RopeVec<T>::unpack(lo, x1);
    RopeVec<T>::unpack(hi, x2);
    const float4* c4 = reinterpret_cast<const float4*>(cos_t + pos * half + c);
    const float4* s4 = reinterpret_cast<const float4*>(sin_t + pos * half + c);
#pragma unroll
    for (int k = 0; k < E / 4; ++k) {
      const float4 cv = __ldg(c4 + k), sv = __ldg(s4 + k);
      cs[4 * k] = cv.x; cs[4 * k + 1] = cv.y; cs[4 * k + 2] = cv.z; cs[4 * k + 3] = cv.w;
      sn[4 * k] = sv.x; sn[4 * k + 1] = sv.y; sn[4 * k + 2] = sv.z; sn[4 * k + 3] = sv.w;
    }
#pragma unroll
    for (int k = 0; k < E; ++k) {
      const float sk = sn[k] * p.sin_sign;
      y1[k] = x1[k] * cs[k] - x2[k] * sk;
      y2[k] = x2[k] * cs[k] + x1[k] * sk;
    }
    __stcs(reinterpret_cast<uint4*>(dst + dof), RopeVec<T>::pack(y1));
    __stcs(reinterpret_cast<uint4*>(dst + dof + half), RopeVec<T>::pack(y2));
  }
}


}  // namespace spa

using namespace spa;

extern "C" {

const char* spa_last_error(void) { return g_err; }

int64_t spa_launch_count(void) { return g_launches.load(); }

int spa_device_info(int32_t device, int64_t info[6]) {
  cudaDeviceProp prop;
  cudaError_t e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) {
    set_error("cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    return SPA_ECUDA;
  }
  info[0] = prop.multiProcessorCount;
  info[1] = prop.major;
  info[2] = prop.minor;
  info[3] = (int64_t)prop.sharedMemPerBlockOptin;
  info[4] = prop.l2CacheSize;
  info[5] = (int64_t)(prop.totalGlobalMem >> 20);
  return SPA_OK;
}

int spa_check_status(void) {
  int* st = device_status_word();
  if (!st) return SPA_ECUDA;
  int h[4] = {0, 0, 0, 0};
  cudaError_t e = cudaMemcpy(h, st, sizeof(h), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) {
    set_error("status read: %s", cudaGetErrorString(e));
    return SPA_ECUDA;
  }
  if (h[0] != 0) {
    set_error("device-side bounded wait gave up: code %d block %d site %d iteration %d", h[0], h[1],
              h[2], h[3]);
    cudaMemset(st, 0, sizeof(h));
    return SPA_ETIMEOUT;
  }
  return SPA_OK;
}

static int validate_common(int B, int Sq, int Sk, int Hq, int Hkv, int D, int dtype, float scale) {
  if (B <= 0 || Sq <= 0 || Sk <= 0 || Hq <= 0 || Hkv <= 0) {
    set_error("sizes must be positive (B=%d Sq=%d Sk=%d Hq=%d Hkv=%d)", B, Sq, Sk, Hq, Hkv);
    return SPA_EINVAL;
  }
  if (Hq % Hkv != 0) {
    set_error("query heads (%d) must be a multiple of kv heads (%d)", Hq, Hkv);
    return SPA_EINVAL;
  }
  if (!valid_head_dim(D)) {
    set_error("head_dim must be 32, 64 or 128, got %d", D);
    return SPA_EUNSUPPORTED;
  }
  if (dtype != SPA_DTYPE_F32 && dtype != SPA_DTYPE_BF16 && dtype != SPA_DTYPE_F16) {
    set_error("unknown dtype %d", dtype);
    return SPA_EINVAL;
  }
  if (!(scale > 0.f) || !isfinite(scale)) {
    set_error("softmax scale must be positive and finite");
    return SPA_EINVAL;
  }
  return SPA_OK;
}

static bool misaligned(const void* p, int64_t sb, int64_t ss, int64_t sh, int elt, int vec_bytes) {
  return ((uintptr_t)p % vec_bytes) || ((sb * elt) % vec_bytes) || ((ss * elt) % vec_bytes) ||
         ((sh * elt) % vec_bytes);
}
static int elt_size(int dtype) { return dtype == SPA_DTYPE_F32 ? 4 : 2; }

int spa_attn_fwd(const spa_fwd_args* args) {
  if (!args || !args->q || !args->k || !args->v || !args->lse) {
    set_error("spa_attn_fwd: null pointer argument");
    return SPA_EINVAL;
  }
  spa_fwd_args n = *args;
  const spa_fwd_args* a = &n;
  int rc = validate_common(a->B, a->Sq, a->Sk, a->Hq, a->Hkv, a->D, a->dtype, a->scale);
  if (rc) return rc;
  if (!a->out && !a->out_acc) {
    set_error("spa_attn_fwd: at least one of out / out_acc is required");
    return SPA_EINVAL;
  }
  if (a->merge_prev && !a->out_acc) {
    set_error("spa_attn_fwd: merge_prev needs out_acc");
    return SPA_EINVAL;
  }
  if (n.lse_sb == 0 && n.lse_sh == 0) {
    n.lse_sh = a->Sq;
    n.lse_sb = (int64_t)a->Hq * a->Sq;
  }
  // Rows are read and written as 16-byte vectors by every kernel.
  const int es = elt_size(a->dtype);
  if (misaligned(a->q, a->q_sb, a->q_ss, a->q_sh, es, 16) ||
      misaligned(a->k, a->k_sb, a->k_ss, a->k_sh, es, 16) ||
      misaligned(a->v, a->v_sb, a->v_ss, a->v_sh, es, 16) ||
      (a->out && misaligned(a->out, a->o_sb, a->o_ss, a->o_sh, es, 16)) ||
      (a->out_acc && ((uintptr_t)a->out_acc & 15))) {
    set_error("spa_attn_fwd: tensor bases and strides must be multiples of 16 bytes");
    return SPA_EINVAL;
  }
  const bool tensor_core = a->dtype != SPA_DTYPE_F32 && a->D != 32 && !force_simt();
  rc = tensor_core ? launch_fwd_sm100(a) : launch_fwd_simt(a);
  if (rc == SPA_OK) note_launch(1);
  return rc;
}

// Checks shared by spa_attn_bwd and spa_attn_bwd_noalloc, after the zero stride
// triples have been replaced by the contiguous ones.
static int validate_bwd(const spa_bwd_args* a) {
  if (a->passes != SPA_BWD_BOTH && a->passes != SPA_BWD_DQ_ONLY && a->passes != SPA_BWD_DKV_ONLY) {
    set_error("spa_attn_bwd: unknown passes value %d", a->passes);
    return SPA_EINVAL;
  }
  const bool want_dq = a->passes != SPA_BWD_DKV_ONLY, want_dkv = a->passes != SPA_BWD_DQ_ONLY;
  if (want_dq && !a->dq && !a->dq_acc) {
    set_error("spa_attn_bwd: at least one of dq / dq_acc is required");
    return SPA_EINVAL;
  }
  if (want_dq && !a->dq_overwrite && !a->dq_acc) {
    set_error("spa_attn_bwd: dq_overwrite == 0 needs dq_acc (the earlier steps' sum)");
    return SPA_EINVAL;
  }
  if (want_dkv && (!a->dk || !a->dv)) {
    set_error("spa_attn_bwd: null dk / dv");
    return SPA_EINVAL;
  }
  if (want_dkv && a->dkv_fp32 && (a->dkv_ss != (int64_t)a->Hkv * a->D || a->dkv_sh != a->D ||
                      a->dkv_sb != (int64_t)a->Sk * a->Hkv * a->D)) {
    set_error("spa_attn_bwd: fp32 dk/dv must be contiguous [B,Sk,Hkv,D]");
    return SPA_EINVAL;
  }
  const int es = elt_size(a->dtype);
  if (misaligned(a->q, a->q_sb, a->q_ss, a->q_sh, es, 16) ||
      misaligned(a->k, a->k_sb, a->k_ss, a->k_sh, es, 16) ||
      misaligned(a->v, a->v_sb, a->v_ss, a->v_sh, es, 16) ||
      misaligned(a->dout, a->do_sb, a->do_ss, a->do_sh, es, 16) ||
      (want_dq && a->dq && misaligned(a->dq, a->dq_sb, a->dq_ss, a->dq_sh, es, 16)) ||
      (want_dq && a->dq_acc && ((uintptr_t)a->dq_acc & 15)) ||
      (want_dkv && (misaligned(a->dk, a->dkv_sb, a->dkv_ss, a->dkv_sh, a->dkv_fp32 ? 4 : es, 16) ||
                    misaligned(a->dv, a->dkv_sb, a->dkv_ss, a->dkv_sh, a->dkv_fp32 ? 4 : es, 16)))) {
    set_error("spa_attn_bwd: tensor bases and strides must be multiples of 16 bytes");
    return SPA_EINVAL;
  }
  return SPA_OK;
}

static void normalise_bwd(spa_bwd_args* n) {
  if (n->dtype == SPA_DTYPE_F32) n->dkv_fp32 = 0;   // fp32 is the element type: strided like any other
  if (n->lse_sb == 0 && n->lse_sh == 0) {
    n->lse_sh = n->Sq;
    n->lse_sb = (int64_t)n->Hq * n->Sq;
  }
  if (n->dq_sb == 0 && n->dq_ss == 0 && n->dq_sh == 0) {
    n->dq_sh = n->D;
    n->dq_ss = (int64_t)n->Hq * n->D;
    n->dq_sb = (int64_t)n->Sq * n->dq_ss;
  }
  if (n->dkv_sb == 0 && n->dkv_ss == 0 && n->dkv_sh == 0) {
    n->dkv_sh = n->D;
    n->dkv_ss = (int64_t)n->Hkv * n->D;
    n->dkv_sb = (int64_t)n->Sk * n->dkv_ss;
  }
}

// Both passes of the backward on the stream of `a` (already normalised and validated).
static int run_bwd(const spa_bwd_args* a) {
  const bool tensor_core = a->dtype != SPA_DTYPE_F32 && a->D != 32 && !force_simt();
  const bool want_dq = a->passes != SPA_BWD_DKV_ONLY, want_dkv = a->passes != SPA_BWD_DQ_ONLY;
  int rc = SPA_OK;
  if (tensor_core) {
    if (want_dq) rc = launch_bwd_dq_sm100(a);
    if (rc == SPA_OK && want_dkv) rc = launch_bwd_dkv_sm100(a);
  } else {
    rc = launch_bwd_simt(a);
  }
  if (rc == SPA_OK) note_launch((want_dq ? 1 : 0) + (want_dkv ? 1 : 0));
  return rc;
}

int spa_attn_bwd(const spa_bwd_args* args) {
  if (!args || !args->q || !args->k || !args->v || !args->dout || !args->lse || !args->delta) {
    set_error("spa_attn_bwd: null pointer argument");
    return SPA_EINVAL;
  }
  spa_bwd_args n = *args;
  int rc = validate_common(n.B, n.Sq, n.Sk, n.Hq, n.Hkv, n.D, n.dtype, n.scale);
  if (rc) return rc;
  normalise_bwd(&n);
  rc = validate_bwd(&n);
  if (rc) return rc;
  return run_bwd(&n);
}

#define SPA_DISPATCH_T(dtype, ...)                                 \
  switch (dtype) {                                                 \
    case SPA_DTYPE_F32: { using T = float; __VA_ARGS__; } break;   \
    case SPA_DTYPE_BF16: { using T = __nv_bfloat16; __VA_ARGS__; } break; \
    case SPA_DTYPE_F16: { using T = __half; __VA_ARGS__; } break;  \
    default: set_error("unknown dtype %d", dtype); return SPA_EINVAL; \
  }

int spa_bwd_delta(const void* out, int64_t o_sb, int64_t o_ss, int64_t o_sh, const void* dout,
                  int64_t do_sb, int64_t do_ss, int64_t do_sh, float* delta, int32_t B, int32_t S,
                  int32_t H, int32_t D, int32_t dtype, void* stream) {
  if (!out || !dout || !delta || B <= 0 || S <= 0 || H <= 0 || !valid_head_dim(D)) {
    set_error("spa_bwd_delta: bad argument");
    return SPA_EINVAL;
  }
  {
    const int es = elt_size(dtype), vec = 16;   // rows are read as 16-byte vectors
    if (misaligned(out, o_sb, o_ss, o_sh, es, vec) || misaligned(dout, do_sb, do_ss, do_sh, es, vec)) {
      set_error("spa_bwd_delta: tensor bases and strides must be multiples of %d bytes", vec);
      return SPA_EINVAL;
    }
  }
  const int sblk = kRowsInFlight * (32 / (D / 8));                        // positions per warp
  const long long threads = (long long)B * ((S + sblk - 1) / sblk) * H * 32;
  const int block = 256;
  const long long grid = (threads + block - 1) / block;
  const bool small = grid * block < (1ll << 31);
  SPA_DISPATCH_T(dtype, if (small) delta_kernel<T, uint32_t><<<(unsigned)grid, block, 0, (cudaStream_t)stream>>>(
                            (const T*)out, o_sb, o_ss, o_sh, (const T*)dout, do_sb, do_ss, do_sh,
                            delta, B, S, H, D);
                        else delta_kernel<T, long long><<<(unsigned)grid, block, 0, (cudaStream_t)stream>>>(
                            (const T*)out, o_sb, o_ss, o_sh, (const T*)dout, do_sb, do_ss, do_sh,
                            delta, B, S, H, D));
  int rc = check_launch("delta");
  if (rc == SPA_OK) note_launch();
  return rc;
}

int spa_merge(float* out_acc, float* lse, const void* block_out, int64_t bo_sb, int64_t bo_ss,
              int64_t bo_sh, const float* block_lse, int32_t B, int32_t S, int32_t H, int32_t D,
              int32_t dtype, void* stream) {
  if (!out_acc || !lse || !block_out || !block_lse || B <= 0 || S <= 0 || H <= 0 ||
      !valid_head_dim(D)) {
    set_error("spa_merge: bad argument");
    return SPA_EINVAL;
  }
  if (((uintptr_t)out_acc & 15) || misaligned(block_out, bo_sb, bo_ss, bo_sh, elt_size(dtype), 4 * elt_size(dtype))) {
    set_error("spa_merge: out_acc must be 16-byte aligned, block_out base and strides multiples of 4 elements");
    return SPA_EINVAL;
  }
  const long long threads = (long long)B * ((S + kMergeRows - 1) / kMergeRows) * H * 32;   // a warp per kMergeRows positions of a (b, h)
  const int block = 256;
  const long long grid = (threads + block - 1) / block;
  const bool small = grid * block < (1ll << 31);
  SPA_DISPATCH_T(dtype, if (small) merge_kernel<T, uint32_t><<<(unsigned)grid, block, 0, (cudaStream_t)stream>>>(
                            out_acc, lse, (const T*)block_out, bo_sb, bo_ss, bo_sh, block_lse, B, S,
                            H, D);
                        else merge_kernel<T, long long><<<(unsigned)grid, block, 0, (cudaStream_t)stream>>>(
                            out_acc, lse, (const T*)block_out, bo_sb, bo_ss, bo_sh, block_lse, B, S,
                            H, D));
  int rc = check_launch("merge");
  if (rc == SPA_OK) note_launch();
  return rc;
}

int spa_cast_from_f32(const float* src, void* dst, int64_t d_sb, int64_t d_ss, int64_t d_sh,
                      int32_t B, int32_t S, int32_t H, int32_t D, int32_t dtype, float alpha,
                      void* stream) {
  if (!src || !dst || B <= 0 || S <= 0 || H <= 0 || !valid_head_dim(D)) {
    set_error("spa_cast_from_f32: bad argument");
    return SPA_EINVAL;
  }
  if (((uintptr_t)src & 15) || misaligned(dst, d_sb, d_ss, d_sh, elt_size(dtype), 4 * elt_size(dtype))) {
    set_error("spa_cast_from_f32: src must be 16-byte aligned, dst base and strides multiples of 4 elements");
    return SPA_EINVAL;
  }
  const long long threads = (long long)B * S * H * (D / 4);
  const int block = 256;
  const long long grid = (threads + 2 * block - 1) / (2 * block);
  const bool small = grid * block * 2 < (1ll << 31);
  SPA_DISPATCH_T(dtype, if (small) cast_kernel<T, uint32_t><<<(unsigned)grid, block, 0, (cudaStream_t)stream>>>(
                            src, (T*)dst, d_sb, d_ss, d_sh, B, S, H, D, alpha);
                        else cast_kernel<T, long long><<<(unsigned)grid, block, 0, (cudaStream_t)stream>>>(
                            src, (T*)dst, d_sb, d_ss, d_sh, B, S, H, D, alpha));
  int rc = check_launch("cast");
  if (rc == SPA_OK) note_launch();
  return rc;
}

int spa_permute_rows(const void* src, void* dst, const int64_t n[4], const int64_t src_stride[4],
                     const int64_t dst_stride[4], int64_t row_bytes, void* stream) {
  if (!src || !dst || !n || !src_stride || !dst_stride || row_bytes <= 0 || (row_bytes & 15)) {
    set_error("spa_permute_rows: bad argument (row_bytes must be a positive multiple of 16)");
    return SPA_EINVAL;
  }
  if (((uintptr_t)src & 15) || ((uintptr_t)dst & 15)) {
    set_error("spa_permute_rows: base pointers must be 16-byte aligned");
    return SPA_EINVAL;
  }
  PermuteParams p;
  int64_t rows = 1;
  for (int i = 0; i < 4; ++i) {
    if (n[i] <= 0 || (src_stride[i] & 15) || (dst_stride[i] & 15)) {
      set_error("spa_permute_rows: extents must be positive and strides 16-byte multiples");
      return SPA_EINVAL;
    }
    p.n[i] = n[i];
    p.ss[i] = src_stride[i];
    p.ds[i] = dst_stride[i];
    rows *= n[i];
  }
  p.vec_per_row = row_bytes / 16;
  p.total_vec = rows * p.vec_per_row;
  const int block = kStreamBlock;
  // A few waves of 148 SMs x 8 resident blocks; the kernel grid-strides.
  int64_t grid = stream_grid(p.total_vec);
  const int64_t cap = 148 * 8 * 4;
  if (grid > cap) grid = cap;
  if (p.total_vec < (1ll << 31))
    permute_rows_kernel<uint32_t><<<(unsigned)grid, block, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)src, (uint8_t*)dst, p);
  else
    permute_rows_kernel<int64_t><<<(unsigned)grid, block, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)src, (uint8_t*)dst, p);
  int rc = check_launch("permute_rows");
  if (rc == SPA_OK) note_launch();
  return rc;
}


int spa_rope_rows(const void* src, void* dst, const int64_t n[4], const int64_t src_stride[4],
                             const int64_t dst_stride[4], int32_t D, int32_t dtype, const float* cos_table,
                             const float* sin_table, int64_t table_rows, int32_t pos_dim,
                             int64_t pos_offset, int32_t inverse, void* stream) {
  if (!src || !dst || !n || !src_stride || !dst_stride || !cos_table || !sin_table ||
      !valid_head_dim(D) || pos_dim < 0 || pos_dim > 3 || pos_offset < 0) {
    set_error("spa_rope_rows: bad argument");
    return SPA_EINVAL;
  }
  const int es = elt_size(dtype);
  if (es == 0) {
    set_error("spa_rope_rows: unknown dtype %d", dtype);
    return SPA_EINVAL;
  }
  if (((uintptr_t)src & 15) || ((uintptr_t)dst & 15) || ((uintptr_t)cos_table & 15) ||
      ((uintptr_t)sin_table & 15)) {
    set_error("spa_rope_rows: base pointers must be 16-byte aligned");
    return SPA_EINVAL;
  }
  RopeParams p;
  int64_t rows = 1;
  for (int i = 0; i < 4; ++i) {
    if (n[i] <= 0 || ((src_stride[i] * es) & 15) || ((dst_stride[i] * es) & 15)) {
      set_error("spa_rope_rows: extents must be positive and strides multiples of 16 bytes");
      return SPA_EINVAL;
    }
    p.n[i] = n[i];
    p.ss[i] = src_stride[i];
    p.ds[i] = dst_stride[i];
    rows *= n[i];
  }
  if (pos_offset + n[pos_dim] > table_rows) {
    set_error("spa_rope_rows: positions %lld..%lld exceed the %lld rows of the cos/sin tables",
              (long long)pos_offset, (long long)(pos_offset + n[pos_dim] - 1), (long long)table_rows);
    return SPA_EINVAL;
  }
  p.D = D;
  p.pos_dim = pos_dim;
  p.pos_off = pos_offset;
  p.sin_sign = inverse ? -1.f : 1.f;
  p.total = rows * ((D / 2) / (16 / es));
  int64_t grid = (p.total + kStreamBlock - 1) / kStreamBlock;
  const int64_t cap = 148 * 8 * 8;
  if (grid > cap) grid = cap;
  SPA_DISPATCH_T(dtype, rope_rows_kernel<T><<<(unsigned)grid, kStreamBlock, 0, (cudaStream_t)stream>>>(
                            (const T*)src, (T*)dst, cos_table, sin_table, p));
  int rc = check_launch("rope_rows");
  if (rc == SPA_OK) note_launch();
  return rc;
}


// ---------------------------------------------------------------------------
// Allocation-free backward.
//
// Some callers may not allocate device memory at all: code running inside a
// memory pool that already owns the whole GPU, a service with a fixed memory
// budget, or a host thread that must not take the allocator's locks. For them
// the scratch of the backward pass (the delta row sums, rowsum(dO * O)) lives in
// the fixed array below instead of in a caller-provided buffer. The array is
// part of the library image: every GPU that loads the library holds
// SPA_NOALLOC_SCRATCH_BYTES of it until the process exits.
// ---------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_noalloc_scratch[SPA_NOALLOC_SCRATCH_BYTES];

// In host code `g_noalloc_scratch` is only a handle; the device address has to
// be asked for, once per device, with that device current.
static std::mutex g_noalloc_mu;
static unsigned char* g_noalloc_ptr[64] = {nullptr};

static unsigned char* noalloc_scratch_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("cudaGetDevice failed");
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (!g_noalloc_ptr[dev]) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || !ptr) {
      set_error("cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
      return nullptr;
    }
    g_noalloc_ptr[dev] = static_cast<unsigned char*>(ptr);
  }
  return g_noalloc_ptr[dev];
}

int64_t spa_noalloc_scratch_bytes(void) { return (int64_t)SPA_NOALLOC_SCRATCH_BYTES; }

int spa_attn_bwd_noalloc(const spa_bwd_noalloc_args* a) {
  if (!a || !a->q || !a->k || !a->v || !a->out || !a->dout || !a->lse || !a->dq || !a->dk ||
      !a->dv) {
    set_error("spa_attn_bwd_noalloc: null pointer argument");
    return SPA_EINVAL;
  }
  int rc = validate_common(a->B, a->Sq, a->Sk, a->Hq, a->Hkv, a->D, a->dtype, a->scale);
  if (rc) return rc;
  const size_t delta_bytes = (size_t)a->B * a->Sq * a->Hq * sizeof(float);
  if (delta_bytes > (size_t)SPA_NOALLOC_SCRATCH_BYTES) {
    set_error("spa_attn_bwd_noalloc: B*Sq*Hq*4 = %zu bytes of scratch needed, the built-in "
              "scratch holds %zu; use spa_attn_bwd with a caller-provided delta buffer",
              delta_bytes, (size_t)SPA_NOALLOC_SCRATCH_BYTES);
    return SPA_EINVAL;
  }
  unsigned char* base = noalloc_scratch_ptr();
  if (!base) return SPA_ECUDA;
  // Every element of delta this call reads is written by its own delta kernel first, so
  // nothing in the shared array has to start at zero.
  float* delta = reinterpret_cast<float*>(base);
  rc = spa_bwd_delta(a->out, a->o_sb, a->o_ss, a->o_sh, a->dout, a->do_sb, a->do_ss, a->do_sh, delta,
                     a->B, a->Sq, a->Hq, a->D, a->dtype, a->stream);
  if (rc) return rc;
  spa_bwd_args b;
  memset(&b, 0, sizeof(b));
  b.q = a->q; b.q_sb = a->q_sb; b.q_ss = a->q_ss; b.q_sh = a->q_sh;
  b.k = a->k; b.k_sb = a->k_sb; b.k_ss = a->k_ss; b.k_sh = a->k_sh;
  b.v = a->v; b.v_sb = a->v_sb; b.v_ss = a->v_ss; b.v_sh = a->v_sh;
  b.dout = a->dout; b.do_sb = a->do_sb; b.do_ss = a->do_ss; b.do_sh = a->do_sh;
  b.lse = a->lse; b.delta = delta;
  // dq is written once, in the element type, by the CTA that owns its rows: no fp32
  // accumulator is needed. dk/dv likewise (a K/V tile belongs to one CTA).
  b.dq_acc = nullptr; b.dq = a->dq; b.dq_overwrite = 1;
  b.dk = a->dk; b.dv = a->dv;
  b.dkv_fp32 = 0; b.dkv_accumulate = 0; b.deterministic = 1;
  b.B = a->B; b.Sq = a->Sq; b.Sk = a->Sk; b.Hq = a->Hq; b.Hkv = a->Hkv; b.D = a->D;
  b.dtype = a->dtype; b.causal = a->causal; b.causal_off = a->causal_off; b.scale = a->scale;
  b.stream = a->stream;
  normalise_bwd(&b);
  rc = validate_bwd(&b);
  if (rc) return rc;
  // The tensor-core kernels (bf16/fp16, head_dim 64/128) and the CUDA-core kernels
  // (fp32, head_dim 32) both run without any allocation: TMA descriptors travel as
  // kernel parameters and the status word is part of the library image too.
  return run_bwd(&b);
}

// Test hook (not part of include/spa.h): the bookkeeping behind the per-device
// shared-memory attribute cache, callable without a GPU.
int spa_internal_smem_attr_seen(const void* kernel, int device, int bytes) {
  return smem_attr_seen(kernel, device, bytes) ? 1 : 0;
}

}  // extern "C"
