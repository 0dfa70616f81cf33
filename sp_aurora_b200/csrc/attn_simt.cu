// CUDA-core (fp32 FMA) flash-attention forward and backward.
//
// This is the path fp32 tensors take: every product and accumulation is fp32,
// so results agree with the reference's fp32 PyTorch math
// (sp_aurora/intel_flash_attn.py:95-126) to ~1e-6, inside the 1e-4 budget that
// tensor-core bf16/tf32 products cannot meet. It also accepts bf16/fp16 data
// (converted on load) so tests can cross-check the tcgen05 kernels on the GPU.
//
// Thread layout everywhere: four threads (a "quad") share one row; thread s of
// the quad owns the float4 chunks f with f % 4 == s of the head dimension, so
// the quad's shared-memory reads of a K/V/Q row are four consecutive float4s
// (conflict-free) and a dot product is finished with two shuffles.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include "spa_internal.h"

namespace spa {
namespace {

constexpr int kRows = 64;      // rows per CTA (256 threads)
constexpr int kTile = 32;      // rows of the streamed operand per shared-memory tile
constexpr int kThreadsSimt = 256;

template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
  const float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
  return make_float4(fa.x, fa.y, fb.x, fb.y);
}
template <>
__device__ __forceinline__ float4 load4<__half>(const __half* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const __half2 a = *reinterpret_cast<const __half2*>(&u.x);
  const __half2 b = *reinterpret_cast<const __half2*>(&u.y);
  const float2 fa = __half22float2(a), fb = __half22float2(b);
  return make_float4(fa.x, fa.y, fb.x, fb.y);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* p, float4 v) {
  *reinterpret_cast<float4*>(p) = v;
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}
template <>
__device__ __forceinline__ void store4<__half>(__half* p, float4 v) {
  __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

__device__ __forceinline__ float quad_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  return x;
}

// Cooperative load of `kTile` rows x D (element type T, row stride `stride`
// elements, rows >= n_valid zero-filled) into fp32 shared memory [kTile][D].
template <int D, typename T>
__device__ __forceinline__ void load_tile(float* dst, const T* src, int64_t stride, int n_valid) {
  constexpr int kVec = D / 4;
  for (int i = threadIdx.x; i < kTile * kVec; i += kThreadsSimt) {
    const int r = i / kVec, f = i % kVec;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < n_valid) v = load4<T>(src + (int64_t)r * stride + 4 * f);
    *reinterpret_cast<float4*>(dst + r * D + 4 * f) = v;
  }
}

struct SimtFwdParams {
  const void *q, *k, *v;
  int64_t q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh;
  void* out;
  int64_t o_sb, o_ss, o_sh;
  float* out_acc;
  float* lse;
  int64_t lse_sb, lse_sh;
  int B, Sq, Sk, Hq, Hkv, causal, causal_off, merge_prev;
  float scale;
};

template <int D, typename T>
__global__ void __launch_bounds__(kThreadsSimt)
attn_fwd_simt_kernel(const SimtFwdParams p) {
  constexpr int NF = D / 16;  // float4 chunks per thread
  __shared__ __align__(16) float k_s[kTile * D];
  __shared__ __align__(16) float v_s[kTile * D];
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int r0 = blockIdx.x * kRows;
  const int row = r0 + (threadIdx.x >> 2);
  const int sl = threadIdx.x & 3;
  const bool row_ok = row < p.Sq;
  const T* qp = reinterpret_cast<const T*>(p.q) + b * p.q_sb + (int64_t)min(row, p.Sq - 1) * p.q_ss +
                h * p.q_sh;
  float4 qv[NF], o[NF];
#pragma unroll
  for (int i = 0; i < NF; ++i) {
    qv[i] = load4<T>(qp + 4 * (4 * i + sl));
    o[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float m = -INFINITY, l = 0.f;

  int n_keys = p.Sk;
  if (p.causal) {
    const long long last = (long long)min(r0 + kRows, p.Sq) - 1 + p.causal_off;
    n_keys = (int)max(0ll, min((long long)p.Sk, last + 1));
  }
  const T* kbase = reinterpret_cast<const T*>(p.k) + b * p.k_sb + hk * p.k_sh;
  const T* vbase = reinterpret_cast<const T*>(p.v) + b * p.v_sb + hk * p.v_sh;
  const long long my_last = p.causal ? (long long)row + p.causal_off : (long long)p.Sk;

  for (int k0 = 0; k0 < n_keys; k0 += kTile) {
    __syncthreads();
    const int nv = min(kTile, p.Sk - k0);
    load_tile<D, T>(k_s, kbase + (int64_t)k0 * p.k_ss, p.k_ss, nv);
    load_tile<D, T>(v_s, vbase + (int64_t)k0 * p.v_ss, p.v_ss, nv);
    __syncthreads();
#pragma unroll 1
    for (int c0 = 0; c0 < kTile; c0 += 8) {
      float s[8];
      float cmax = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float* kr = k_s + (c0 + j) * D;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < NF; ++i) {
          const float4 kv = *reinterpret_cast<const float4*>(kr + 4 * (4 * i + sl));
          acc = fmaf(qv[i].x, kv.x, acc);
          acc = fmaf(qv[i].y, kv.y, acc);
          acc = fmaf(qv[i].z, kv.z, acc);
          acc = fmaf(qv[i].w, kv.w, acc);
        }
        acc = quad_sum(acc) * p.scale;
        const int kidx = k0 + c0 + j;
        if (kidx >= p.Sk || (long long)kidx > my_last) acc = -INFINITY;
        s[j] = acc;
        cmax = fmaxf(cmax, acc);
      }
      const float m_new = fmaxf(m, cmax);
      if (m_new == -INFINITY) continue;  // nothing visible yet
      const float alpha = __expf(m - m_new);  // m = -inf -> 0
      float psum = 0.f;
      float pj[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        pj[j] = expf(s[j] - m_new);
        psum += pj[j];
      }
      l = l * alpha + psum;
      m = m_new;
#pragma unroll
      for (int i = 0; i < NF; ++i) {
        float4 a = o[i];
        a.x *= alpha; a.y *= alpha; a.z *= alpha; a.w *= alpha;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 vv = *reinterpret_cast<const float4*>(v_s + (c0 + j) * D + 4 * (4 * i + sl));
          a.x = fmaf(pj[j], vv.x, a.x);
          a.y = fmaf(pj[j], vv.y, a.y);
          a.z = fmaf(pj[j], vv.z, a.z);
          a.w = fmaf(pj[j], vv.w, a.w);
        }
        o[i] = a;
      }
    }
  }

  if (!row_ok) return;
  const bool have = l > 0.f;
  const float inv_l = have ? 1.f / l : 0.f;
  const float lse_blk = have ? m + logf(l) : -INFINITY;
  const size_t lse_idx = (size_t)b * p.lse_sb + (size_t)h * p.lse_sh + row;
  float w_old = 0.f, w_blk = have ? 1.f : 0.f, lse_new = lse_blk;
  if (p.merge_prev) {
    const float lse_old = p.lse[lse_idx];
    const float mx = fmaxf(lse_old, lse_blk);
    if (mx == -INFINITY) {
      w_blk = 0.f;
      lse_new = -INFINITY;
    } else {
      const float e_old = expf(lse_old - mx), e_blk = expf(lse_blk - mx);
      const float sum = e_old + e_blk;
      lse_new = mx + logf(sum);
      w_old = e_old / sum;
      w_blk = e_blk / sum;
    }
  }
  if (sl == 0) p.lse[lse_idx] = lse_new;
  float* acc_row = p.out_acc ? p.out_acc + (((size_t)b * p.Sq + row) * p.Hq + h) * D : nullptr;
  T* out_row = p.out ? reinterpret_cast<T*>(p.out) + b * p.o_sb + (int64_t)row * p.o_ss + h * p.o_sh
                     : nullptr;
  const float osc = inv_l * w_blk;
#pragma unroll
  for (int i = 0; i < NF; ++i) {
    const int e = 4 * (4 * i + sl);
    float4 a = o[i];
    a.x *= osc; a.y *= osc; a.z *= osc; a.w *= osc;
    if (p.merge_prev) {
      const float4 ov = *reinterpret_cast<const float4*>(acc_row + e);
      a.x = fmaf(w_old, ov.x, a.x);
      a.y = fmaf(w_old, ov.y, a.y);
      a.z = fmaf(w_old, ov.z, a.z);
      a.w = fmaf(w_old, ov.w, a.w);
    }
    if (acc_row) *reinterpret_cast<float4*>(acc_row + e) = a;
    if (out_row) store4<T>(out_row + e, a);
  }
}

struct SimtBwdParams {
  const void *q, *k, *v, *dout;
  int64_t q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh, do_sb, do_ss, do_sh;
  const float* lse;
  const float* delta;
  int64_t lse_sb, lse_sh;
  float* dq_acc;
  void* dq;
  int64_t dq_sb, dq_ss, dq_sh;
  int dq_overwrite;
  void* dk;
  void* dv;
  int64_t dkv_sb, dkv_ss, dkv_sh;
  int dkv_fp32, dkv_accumulate;
  int B, Sq, Sk, Hq, Hkv, causal, causal_off;
  float scale;
};

// dQ: query rows stationary, keys streamed. The CTA owns its dq rows, so the
// accumulation into dq_acc is a plain read-modify-write.
template <int D, typename T>
__global__ void __launch_bounds__(kThreadsSimt)
attn_bwd_dq_simt_kernel(const SimtBwdParams p) {
  constexpr int NF = D / 16;
  __shared__ __align__(16) float k_s[kTile * D];
  __shared__ __align__(16) float v_s[kTile * D];
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int r0 = blockIdx.x * kRows;
  const int row = r0 + (threadIdx.x >> 2);
  const int sl = threadIdx.x & 3;
  const bool row_ok = row < p.Sq;
  const int rowc = min(row, p.Sq - 1);
  const T* qp = reinterpret_cast<const T*>(p.q) + b * p.q_sb + (int64_t)rowc * p.q_ss + h * p.q_sh;
  const T* dop =
      reinterpret_cast<const T*>(p.dout) + b * p.do_sb + (int64_t)rowc * p.do_ss + h * p.do_sh;
  float4 qv[NF], dov[NF], dq[NF];
#pragma unroll
  for (int i = 0; i < NF; ++i) {
    qv[i] = load4<T>(qp + 4 * (4 * i + sl));
    dov[i] = load4<T>(dop + 4 * (4 * i + sl));
    dq[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const size_t sidx = (size_t)b * p.lse_sb + (size_t)h * p.lse_sh + rowc;
  const float lse = p.lse[sidx];
  const float delta = p.delta[sidx];

  int n_keys = p.Sk;
  if (p.causal) {
    const long long last = (long long)min(r0 + kRows, p.Sq) - 1 + p.causal_off;
    n_keys = (int)max(0ll, min((long long)p.Sk, last + 1));
  }
  const T* kbase = reinterpret_cast<const T*>(p.k) + b * p.k_sb + hk * p.k_sh;
  const T* vbase = reinterpret_cast<const T*>(p.v) + b * p.v_sb + hk * p.v_sh;
  const long long my_last = p.causal ? (long long)row + p.causal_off : (long long)p.Sk;

  for (int k0 = 0; k0 < n_keys; k0 += kTile) {
    __syncthreads();
    const int nv = min(kTile, p.Sk - k0);
    load_tile<D, T>(k_s, kbase + (int64_t)k0 * p.k_ss, p.k_ss, nv);
    load_tile<D, T>(v_s, vbase + (int64_t)k0 * p.v_ss, p.v_ss, nv);
    __syncthreads();
#pragma unroll 2
    for (int j = 0; j < kTile; ++j) {
      const float* kr = k_s + j * D;
      const float* vr = v_s + j * D;
      float s = 0.f, dp = 0.f;
#pragma unroll
      for (int i = 0; i < NF; ++i) {
        const float4 kv = *reinterpret_cast<const float4*>(kr + 4 * (4 * i + sl));
        const float4 vv = *reinterpret_cast<const float4*>(vr + 4 * (4 * i + sl));
        s = fmaf(qv[i].x, kv.x, s); s = fmaf(qv[i].y, kv.y, s);
        s = fmaf(qv[i].z, kv.z, s); s = fmaf(qv[i].w, kv.w, s);
        dp = fmaf(dov[i].x, vv.x, dp); dp = fmaf(dov[i].y, vv.y, dp);
        dp = fmaf(dov[i].z, vv.z, dp); dp = fmaf(dov[i].w, vv.w, dp);
      }
      s = quad_sum(s) * p.scale;
      dp = quad_sum(dp);
      const int kidx = k0 + j;
      float pe = expf(s - lse);
      if (kidx >= p.Sk || (long long)kidx > my_last) pe = 0.f;
      const float ds = pe * (dp - delta);
#pragma unroll
      for (int i = 0; i < NF; ++i) {
        const float4 kv = *reinterpret_cast<const float4*>(kr + 4 * (4 * i + sl));
        dq[i].x = fmaf(ds, kv.x, dq[i].x);
        dq[i].y = fmaf(ds, kv.y, dq[i].y);
        dq[i].z = fmaf(ds, kv.z, dq[i].z);
        dq[i].w = fmaf(ds, kv.w, dq[i].w);
      }
    }
  }
  if (!row_ok) return;
  // total = (earlier ring steps' sum, unless this is the first) + this block; it goes to
  // dq in the element type and / or back to the fp32 accumulator, whichever is given.
  float* acc = p.dq_acc ? p.dq_acc + (((size_t)b * p.Sq + row) * p.Hq + h) * D : nullptr;
  T* dst = p.dq ? reinterpret_cast<T*>(p.dq) + b * p.dq_sb + (int64_t)row * p.dq_ss + h * p.dq_sh
                : nullptr;
#pragma unroll
  for (int i = 0; i < NF; ++i) {
    const int e = 4 * (4 * i + sl);
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!p.dq_overwrite) a = *reinterpret_cast<const float4*>(acc + e);
    a.x = fmaf(p.scale, dq[i].x, a.x);
    a.y = fmaf(p.scale, dq[i].y, a.y);
    a.z = fmaf(p.scale, dq[i].z, a.z);
    a.w = fmaf(p.scale, dq[i].w, a.w);
    if (dst) store4<T>(dst + e, a);
    if (acc) *reinterpret_cast<float4*>(acc + e) = a;
  }
}

// dK/dV: key rows stationary, queries (of every head of the GQA group) streamed.
template <int D, typename T>
__global__ void __launch_bounds__(kThreadsSimt)
attn_bwd_dkv_simt_kernel(const SimtBwdParams p) {
  constexpr int NF = D / 16;
  __shared__ __align__(16) float q_s[kTile * D];
  __shared__ __align__(16) float do_s[kTile * D];
  __shared__ float lse_s[kTile];
  __shared__ float dl_s[kTile];
  const int g = blockIdx.y, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int r0 = blockIdx.x * kRows;
  const int krow = r0 + (threadIdx.x >> 2);
  const int sl = threadIdx.x & 3;
  const bool row_ok = krow < p.Sk;
  const int rowc = min(krow, p.Sk - 1);
  const T* kp = reinterpret_cast<const T*>(p.k) + b * p.k_sb + (int64_t)rowc * p.k_ss + g * p.k_sh;
  const T* vp = reinterpret_cast<const T*>(p.v) + b * p.v_sb + (int64_t)rowc * p.v_ss + g * p.v_sh;
  float4 kv[NF], vv[NF], dk[NF], dv[NF];
#pragma unroll
  for (int i = 0; i < NF; ++i) {
    kv[i] = load4<T>(kp + 4 * (4 * i + sl));
    vv[i] = load4<T>(vp + 4 * (4 * i + sl));
    dk[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    dv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  int q_begin = 0;
  if (p.causal) {
    const long long first = (long long)r0 - p.causal_off;
    q_begin = (int)max(0ll, min((long long)p.Sq, first));
    q_begin = (q_begin / kTile) * kTile;
  }
  for (int hh = 0; hh < G; ++hh) {
    const int h = g * G + hh;
    const T* qbase = reinterpret_cast<const T*>(p.q) + b * p.q_sb + h * p.q_sh;
    const T* dobase = reinterpret_cast<const T*>(p.dout) + b * p.do_sb + h * p.do_sh;
    const size_t sbase = (size_t)b * p.lse_sb + (size_t)h * p.lse_sh;
    for (int q0 = q_begin; q0 < p.Sq; q0 += kTile) {
      __syncthreads();
      const int nv = min(kTile, p.Sq - q0);
      load_tile<D, T>(q_s, qbase + (int64_t)q0 * p.q_ss, p.q_ss, nv);
      load_tile<D, T>(do_s, dobase + (int64_t)q0 * p.do_ss, p.do_ss, nv);
      if (threadIdx.x < kTile) {
        const int qi = q0 + threadIdx.x;
        lse_s[threadIdx.x] = qi < p.Sq ? p.lse[sbase + qi] : INFINITY;
        dl_s[threadIdx.x] = qi < p.Sq ? p.delta[sbase + qi] : 0.f;
      }
      __syncthreads();
#pragma unroll 2
      for (int j = 0; j < kTile; ++j) {
        const float* qr = q_s + j * D;
        const float* dr = do_s + j * D;
        float s = 0.f, dp = 0.f;
#pragma unroll
        for (int i = 0; i < NF; ++i) {
          const float4 qq = *reinterpret_cast<const float4*>(qr + 4 * (4 * i + sl));
          const float4 dd = *reinterpret_cast<const float4*>(dr + 4 * (4 * i + sl));
          s = fmaf(kv[i].x, qq.x, s); s = fmaf(kv[i].y, qq.y, s);
          s = fmaf(kv[i].z, qq.z, s); s = fmaf(kv[i].w, qq.w, s);
          dp = fmaf(vv[i].x, dd.x, dp); dp = fmaf(vv[i].y, dd.y, dp);
          dp = fmaf(vv[i].z, dd.z, dp); dp = fmaf(vv[i].w, dd.w, dp);
        }
        s = quad_sum(s) * p.scale;
        dp = quad_sum(dp);
        const int qi = q0 + j;
        float pe = expf(s - lse_s[j]);
        if (qi >= p.Sq || (p.causal && (long long)krow > (long long)qi + p.causal_off)) pe = 0.f;
        const float ds = pe * (dp - dl_s[j]);
#pragma unroll
        for (int i = 0; i < NF; ++i) {
          const float4 qq = *reinterpret_cast<const float4*>(qr + 4 * (4 * i + sl));
          const float4 dd = *reinterpret_cast<const float4*>(dr + 4 * (4 * i + sl));
          dv[i].x = fmaf(pe, dd.x, dv[i].x); dv[i].y = fmaf(pe, dd.y, dv[i].y);
          dv[i].z = fmaf(pe, dd.z, dv[i].z); dv[i].w = fmaf(pe, dd.w, dv[i].w);
          dk[i].x = fmaf(ds, qq.x, dk[i].x); dk[i].y = fmaf(ds, qq.y, dk[i].y);
          dk[i].z = fmaf(ds, qq.z, dk[i].z); dk[i].w = fmaf(ds, qq.w, dk[i].w);
        }
      }
    }
  }
  if (!row_ok) return;
  const size_t off = (((size_t)b * p.Sk + krow) * p.Hkv + g) * D;                   // fp32: contiguous
  const int64_t off_t = b * p.dkv_sb + (int64_t)krow * p.dkv_ss + g * p.dkv_sh;     // element type: strided
#pragma unroll
  for (int i = 0; i < NF; ++i) {
    const int e = 4 * (4 * i + sl);
    float4 a = dk[i], c = dv[i];
    a.x *= p.scale; a.y *= p.scale; a.z *= p.scale; a.w *= p.scale;
    if (p.dkv_fp32) {
      float* pk = reinterpret_cast<float*>(p.dk) + off + e;
      float* pv = reinterpret_cast<float*>(p.dv) + off + e;
      if (p.dkv_accumulate) {
        const float4 x = *reinterpret_cast<float4*>(pk), y = *reinterpret_cast<float4*>(pv);
        a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
        c.x += y.x; c.y += y.y; c.z += y.z; c.w += y.w;
      }
      *reinterpret_cast<float4*>(pk) = a;
      *reinterpret_cast<float4*>(pv) = c;
    } else {
      T* pk = reinterpret_cast<T*>(p.dk) + off_t + e;
      T* pv = reinterpret_cast<T*>(p.dv) + off_t + e;
      if (p.dkv_accumulate) {
        const float4 x = load4<T>(pk), y = load4<T>(pv);
        a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
        c.x += y.x; c.y += y.y; c.z += y.z; c.w += y.w;
      }
      store4<T>(pk, a);
      store4<T>(pv, c);
    }
  }
}

template <int D, typename T>
int launch_fwd_simt_typed(const spa_fwd_args* a) {
  SimtFwdParams p;
  p.q = a->q; p.k = a->k; p.v = a->v;
  p.q_sb = a->q_sb; p.q_ss = a->q_ss; p.q_sh = a->q_sh;
  p.k_sb = a->k_sb; p.k_ss = a->k_ss; p.k_sh = a->k_sh;
  p.v_sb = a->v_sb; p.v_ss = a->v_ss; p.v_sh = a->v_sh;
  p.out = a->out; p.o_sb = a->o_sb; p.o_ss = a->o_ss; p.o_sh = a->o_sh;
  p.out_acc = a->out_acc; p.lse = a->lse;
  p.lse_sb = a->lse_sb; p.lse_sh = a->lse_sh;
  p.B = a->B; p.Sq = a->Sq; p.Sk = a->Sk; p.Hq = a->Hq; p.Hkv = a->Hkv;
  p.causal = a->causal; p.causal_off = a->causal_off; p.merge_prev = a->merge_prev;
  p.scale = a->scale;
  dim3 grid(ceil_div(a->Sq, kRows), a->Hq, a->B);
  attn_fwd_simt_kernel<D, T><<<grid, kThreadsSimt, 0, (cudaStream_t)a->stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("fwd simt launch: %s", cudaGetErrorString(e));
    return SPA_ECUDA;
  }
  return SPA_OK;
}

template <int D, typename T>
int launch_bwd_simt_typed(const spa_bwd_args* a) {
  SimtBwdParams p;
  p.q = a->q; p.k = a->k; p.v = a->v; p.dout = a->dout;
  p.q_sb = a->q_sb; p.q_ss = a->q_ss; p.q_sh = a->q_sh;
  p.k_sb = a->k_sb; p.k_ss = a->k_ss; p.k_sh = a->k_sh;
  p.v_sb = a->v_sb; p.v_ss = a->v_ss; p.v_sh = a->v_sh;
  p.do_sb = a->do_sb; p.do_ss = a->do_ss; p.do_sh = a->do_sh;
  p.lse = a->lse; p.delta = a->delta; p.lse_sb = a->lse_sb; p.lse_sh = a->lse_sh;
  p.dq_acc = a->dq_acc; p.dq = a->dq; p.dq_sb = a->dq_sb; p.dq_ss = a->dq_ss; p.dq_sh = a->dq_sh;
  p.dq_overwrite = a->dq_overwrite;
  p.dk = a->dk; p.dv = a->dv; p.dkv_sb = a->dkv_sb; p.dkv_ss = a->dkv_ss; p.dkv_sh = a->dkv_sh;
  p.dkv_fp32 = a->dkv_fp32; p.dkv_accumulate = a->dkv_accumulate;
  p.B = a->B; p.Sq = a->Sq; p.Sk = a->Sk; p.Hq = a->Hq; p.Hkv = a->Hkv;
  p.causal = a->causal; p.causal_off = a->causal_off; p.scale = a->scale;
  cudaStream_t st = (cudaStream_t)a->stream;
  dim3 gq(ceil_div(a->Sq, kRows), a->Hq, a->B);
  if (a->passes != SPA_BWD_DKV_ONLY) attn_bwd_dq_simt_kernel<D, T><<<gq, kThreadsSimt, 0, st>>>(p);
  dim3 gk(ceil_div(a->Sk, kRows), a->Hkv, a->B);
  if (a->passes != SPA_BWD_DQ_ONLY) attn_bwd_dkv_simt_kernel<D, T><<<gk, kThreadsSimt, 0, st>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("bwd simt launch: %s", cudaGetErrorString(e));
    return SPA_ECUDA;
  }
  return SPA_OK;
}

template <typename F32, typename BF, typename HF>
int dispatch_dtype(int dtype, F32 f32, BF bf, HF hf) {
  switch (dtype) {
    case SPA_DTYPE_F32: return f32();
    case SPA_DTYPE_BF16: return bf();
    case SPA_DTYPE_F16: return hf();
  }
  set_error("unknown dtype %d", dtype);
  return SPA_EINVAL;
}

}  // namespace

int launch_fwd_simt(const spa_fwd_args* a) {
  switch (a->D) {
    case 32:
      return dispatch_dtype(a->dtype, [&] { return launch_fwd_simt_typed<32, float>(a); },
                            [&] { return launch_fwd_simt_typed<32, __nv_bfloat16>(a); },
                            [&] { return launch_fwd_simt_typed<32, __half>(a); });
    case 64:
      return dispatch_dtype(a->dtype, [&] { return launch_fwd_simt_typed<64, float>(a); },
                            [&] { return launch_fwd_simt_typed<64, __nv_bfloat16>(a); },
                            [&] { return launch_fwd_simt_typed<64, __half>(a); });
    case 128:
      return dispatch_dtype(a->dtype, [&] { return launch_fwd_simt_typed<128, float>(a); },
                            [&] { return launch_fwd_simt_typed<128, __nv_bfloat16>(a); },
                            [&] { return launch_fwd_simt_typed<128, __half>(a); });
  }
  set_error("CUDA-core forward supports head_dim 32, 64, 128, got %d", a->D);
  return SPA_EUNSUPPORTED;
}

int launch_bwd_simt(const spa_bwd_args* a) {
  switch (a->D) {
    case 32:
      return dispatch_dtype(a->dtype, [&] { return launch_bwd_simt_typed<32, float>(a); },
                            [&] { return launch_bwd_simt_typed<32, __nv_bfloat16>(a); },
                            [&] { return launch_bwd_simt_typed<32, __half>(a); });
    case 64:
      return dispatch_dtype(a->dtype, [&] { return launch_bwd_simt_typed<64, float>(a); },
                            [&] { return launch_bwd_simt_typed<64, __nv_bfloat16>(a); },
                            [&] { return launch_bwd_simt_typed<64, __half>(a); });
    case 128:
      return dispatch_dtype(a->dtype, [&] { return launch_bwd_simt_typed<128, float>(a); },
                            [&] { return launch_bwd_simt_typed<128, __nv_bfloat16>(a); },
                            [&] { return launch_bwd_simt_typed<128, __half>(a); });
  }
  set_error("CUDA-core backward supports head_dim 32, 64, 128, got %d", a->D);
  return SPA_EUNSUPPORTED;
}

}  // namespace spa
