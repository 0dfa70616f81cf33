// Flash-attention forward for sm_100a: tcgen05.mma with TMEM accumulators, TMA
// staged K/V tiles, two 128-row query tiles per CTA in ping-pong, online
// softmax in registers (one query row per thread), and the ring-step out/lse
// merge fused into the epilogue.
//
// Math follows sp_aurora/intel_flash_attn.py:95-126 (scores = scale*QK^T, causal
// triu(diagonal=1) mask, lse = logsumexp, out = softmax*V) and the merge follows
// sp_aurora/utils.py:99-104.
//
// CTA = 10 warps:
//   warps 0-3  softmax group of query tile 0 (thread = one query row)
//   warps 4-7  softmax group of query tile 1
//   warp  8    TMA producer (lane 0)
//   warp  9    tcgen05.mma issuer (lane 0); also owns the TMEM allocation
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D).
// The probabilities P (bf16/fp16, two per 32-bit column) overwrite the first 64
// columns of their S tile and feed the PV MMA as operand A straight from TMEM:
// P never goes through shared memory, whose bandwidth (128 B/clk) is what
// bounds this kernel. Shared memory holds Q (2 tiles) and a ring of K/V tiles.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include <type_traits>

#include "spa_internal.h"
#include "tc05.cuh"

namespace spa {

namespace {

constexpr int kTileM = 128;          // query rows per tile
constexpr int kTileN = 128;          // keys per K/V tile
constexpr int kThreads = 320;
constexpr float kRescaleThreshold = 8.0f;  // in log2 units
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kLog2e = 1.4426950408889634f;

struct FwdParams {
  int B, Sq, Sk, Hq, Hkv;
  int causal, causal_off, merge_prev;
  int n_qblk;
  int chunk;   // query blocks per scheduling chunk (n_qblk or 1)
  float scale_log2;
  void* out;
  int64_t o_sb, o_ss, o_sh;
  float* out_acc;
  float* lse;
  int64_t lse_sb, lse_sh;
  int* status;
};

template <int D>
struct FwdSmem {
  static constexpr int kSlabBytes = kTileM * 128;           // 128 rows x 128 B
  static constexpr int kTileBytes = (D / 64) * kSlabBytes;   // one Q/K/V tile
  static constexpr int kStages = 4;   // K_j -> slots 0,2 ; V_j -> slots 1,3 (period of two key tiles)
  static constexpr int kQOff = 0;
  static constexpr int kKVOff = kQOff + 2 * kTileBytes;
  static constexpr int kBarOff = kKVOff + kStages * kTileBytes;
  static constexpr int kNumBars = 1 + 2 * kStages + 6;
  static constexpr int kTotal = kBarOff + kNumBars * 8 + 16;
};

template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int D, typename T>
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tm_q,
                      const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  using L = FwdSmem<D>;
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzle needs 1024-byte aligned tiles.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + L::kStages;
  uint64_t* s_full = kv_empty + L::kStages;  // [2]
  uint64_t* p_full = s_full + 2;             // [2]
  uint64_t* o_done = p_full + 2;             // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Work decode: query blocks of one chunk fastest (longest first under a causal mask),
  // then heads, batch, chunks. The host picks the chunk: all query blocks (CTAs resident
  // together then stream the K/V of one kv head, which stays in L2: S=131072 causal
  // 993 -> 1036 TFLOP/s), or one block for small causal problems, where
  // longest-block-first over all heads matters more.
  int w = blockIdx.x;
  const int q_lo = w % p.chunk;
  w /= p.chunk;
  const int h = w % p.Hq;
  w /= p.Hq;
  const int b = w % p.B;
  const int qblk = p.n_qblk - 1 - ((w / p.B) * p.chunk + q_lo);
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qblk * 2 * kTileM;

  // Number of K/V tiles each query tile attends to.
  int n_t[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int r0 = q0 + t * kTileM;
    int n = 0;
    if (r0 < p.Sq) {
      n = (p.Sk + kTileN - 1) / kTileN;
      if (p.causal) {
        const int last_row = min(r0 + kTileM, p.Sq) - 1;
        const long long last_key = (long long)last_row + p.causal_off;  // inclusive
        const int nc = last_key < 0 ? 0 : (int)(last_key / kTileN) + 1;
        n = min(n, nc);
      }
    }
    n_t[t] = n;
  }
  const int nmax = max(n_t[0], n_t[1]);

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    mbar_init(q_full, 1);
    for (int i = 0; i < L::kStages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 128 / 32);
      mbar_init(&o_done[t], 1);
    }
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  WaitCtx wc{p.status, cta_abort};

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA
    if (lane == 0 && nmax > 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      const int q_tiles = (n_t[1] > 0 || q0 + kTileM < p.Sq) ? 2 : 1;
      mbar_arrive_expect_tx(q_full, q_tiles * L::kTileBytes);
      for (int t = 0; t < q_tiles; ++t)
        for (int s = 0; s < D / 64; ++s)
          tma_load_4d(smem + L::kQOff + t * L::kTileBytes + s * L::kSlabBytes, &tm_q, q_full,
                      s * 64, q0 + t * kTileM, h, b);
      const int nfill = 2 * nmax;
      for (int n = 0; n < nfill; ++n) {
        const int slot = n % L::kStages;
        const uint32_t ph = (n / L::kStages) & 1;
        if (!mbar_wait(&kv_empty[slot], ph ^ 1, wc, 0, n)) break;
        mbar_arrive_expect_tx(&kv_full[slot], L::kTileBytes);
        const CUtensorMap* tm = (n & 1) ? &tm_v : &tm_k;
        const int j = n >> 1;
        for (int s = 0; s < D / 64; ++s)
          tma_load_4d(smem + L::kKVOff + slot * L::kTileBytes + s * L::kSlabBytes, tm,
                      &kv_full[slot], s * 64, j * kTileN, hk, b);
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA
    // One elected lane issues every MMA (measured faster than predicated
    // warp-uniform issue); descriptors are precomputed, offsets are constants.
    if (lane == 0 && nmax > 0) {
      constexpr uint32_t idesc_qk = make_idesc(128, 128, kBf16, false, false);
      constexpr uint32_t idesc_pv = make_idesc(128, D, kBf16, false, true);
      const uint32_t q_base = smem_u32(smem + L::kQOff);
      const uint32_t kv_base = smem_u32(smem + L::kKVOff);
      bool ok = mbar_wait(q_full, 0, wc, 1, 0);
      tc_fence_after();

      // Descriptors are built once; stepping through a tile only adds constants
      // to the low word (the issuing thread is latency bound otherwise).
      const SmemDesc q_desc = make_smem_desc(q_base, 16, 1024);
      const SmemDesc k_desc = make_smem_desc(kv_base, 16, 1024);             // K-major
      const SmemDesc v_desc = make_smem_desc(kv_base, L::kSlabBytes, 1024);  // MN-major
      // S_t = Q_t * K_j^T : A = Q (K-major), B = K tile (K-major).
      // `slot` is a compile-time constant at every call site (the key-tile loop is
      // unrolled over the ring period): runtime descriptor words cost issue time.
      auto issue_qk = [&](int t, int j, const int slot) -> bool {
        const int n = 2 * j;
        if (!mbar_wait(&kv_full[slot], (n / L::kStages) & 1, wc, 2, j)) return false;
        tc_fence_after();
        const uint32_t a0 = (t * L::kTileBytes) >> 4;
        const uint32_t b0 = (slot * L::kTileBytes) >> 4;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = ((kk / 4) * L::kSlabBytes + (kk % 4) * 32) >> 4;
          mma_ss_d(tmem_base + t * 128, q_desc, a0 + off, k_desc, b0 + off, idesc_qk, kk > 0);
        }
        mma_commit(&s_full[t]);
        return true;
      };
      // O_t (+)= P_t * V_j : A = P read from TMEM (columns of S_t), B = V tile
      // (MN-major: rows are keys = K dimension, D contiguous).
      auto issue_pv = [&](int t, int j, const int slot) -> bool {
        const int n = 2 * j + 1;
        if (!mbar_wait(&kv_full[slot], (n / L::kStages) & 1, wc, 3, j)) return false;
        tc_fence_after();
        const uint32_t b0 = (slot * L::kTileBytes) >> 4;
#pragma unroll
        for (int kk = 0; kk < kTileN / 16; ++kk)
          mma_ts_d(tmem_base + 256 + t * D, tmem_base + t * 128 + kk * 8, v_desc,
                   b0 + ((kk * 2048) >> 4), idesc_pv, (j > 0 || kk > 0));
        mma_commit(&o_done[t]);
        return true;
      };

      static_assert(L::kStages == 4, "slot constants below assume a 4-stage ring");
#pragma unroll
      for (int t = 0; t < 2; ++t)
        if (ok && n_t[t] > 0) ok = issue_qk(t, 0, 0);
      if (ok) mma_commit(&kv_empty[0]);  // K_0 slot free once both S(0) are done
      for (int j0 = 0; j0 < nmax && ok; j0 += 2) {
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          const int j = j0 + jj;
          if (j >= nmax || !ok) break;
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (!ok || j >= n_t[t]) continue;
            ok = mbar_wait(&p_full[t], j & 1, wc, 4, j);
            if (!ok) break;
            tc_fence_after();
            // PV(j) first: the pipe executes in order, so S(j+1) cannot overwrite
            // the columns P(j) lives in before PV(j) has read them.
            ok = issue_pv(t, j, 2 * jj + 1);
            if (ok && j + 1 < n_t[t]) ok = issue_qk(t, j + 1, (2 * jj + 2) % 4);
          }
          if (!ok) break;
          if (j + 1 < nmax) mma_commit(&kv_empty[(2 * jj + 2) % 4]);
          mma_commit(&kv_empty[2 * jj + 1]);
        }
      }
    }
  } else {
    // -------------------------------------------------------------- softmax
    const int t = warp >> 2;
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const int qrow = q0 + t * kTileM + row_in_tile;
    const uint32_t lane_field = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tmem_s = tmem_base + lane_field + t * 128;
    const uint32_t tmem_o = tmem_base + lane_field + 256 + t * D;
    const int nt = n_t[t];
    const int tile_row_min = q0 + t * kTileM;
    const float ninf = -INFINITY;

    float m_used = ninf;
    float l = 0.f;
    bool ok = true;

    for (int j = 0; j < nt; ++j) {
      ok = warp_wait(&s_full[t], j & 1, wc, 8 + t, j);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(tmem_s + c * 32, sr + c * 32);
      tmem_ld_wait();
      float* s = reinterpret_cast<float*>(sr);

      const int k0 = j * kTileN;
      const bool need_mask = (k0 + kTileN > p.Sk) ||
                             (p.causal && ((long long)k0 + kTileN - 1 >
                                           (long long)tile_row_min + p.causal_off));
      if (need_mask) {
        long long lim = p.Sk - 1;
        if (p.causal) lim = min(lim, (long long)qrow + p.causal_off);
        const int limit = (int)max(-1ll, min(lim - k0, 127ll));  // last visible column
#pragma unroll
        for (int c = 0; c < 128; ++c)
          if (c > limit) s[c] = ninf;
      }
      float mx = ninf;
#pragma unroll
      for (int c = 0; c < 128; ++c) mx = fmaxf(mx, s[c]);
      const float m_new = fmaxf(m_used, mx * p.scale_log2);
      const bool resc = m_new > m_used + kRescaleThreshold;
      const bool resc_any = __any_sync(0xffffffffu, resc);
      float alpha = 1.f;
      if (resc_any) {
        alpha = (m_new == ninf) ? 1.f : fast_exp2(m_used - m_new);
        m_used = m_new;
        l *= alpha;
      }
      const float m_eff = (m_used == ninf) ? 0.f : m_used;

      // P row -> TMEM, packed two per column, over the first 64 columns of S_t.
      uint32_t pk[64];
      float ls0 = 0.f, ls1 = 0.f;
      const float nm = -m_eff;
#pragma unroll
      for (int c = 0; c < 128; c += 2) {
        float x0, x1;
        fma2(x0, x1, s[c], s[c + 1], p.scale_log2, p.scale_log2, nm, nm);
        const float p0 = fast_exp2(x0);
        const float p1 = fast_exp2(x1);
        add2(ls0, ls1, ls0, ls1, p0, p1);
        pk[c >> 1] = pack2<T>(p0, p1);
      }
      l += ls0 + ls1;
      // PV(j-1) is complete here: S(j) was committed behind it on the in-order tensor pipe,
      // so O may be rescaled and the P columns overwritten without another wait.
      if (j > 0 && resc_any) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t orr[32];
          tmem_ld32(tmem_o + c * 32, orr);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float y0, y1;
            mul2(y0, y1, __uint_as_float(orr[i]), __uint_as_float(orr[i + 1]), alpha, alpha);
            orr[i] = __float_as_uint(y0);
            orr[i + 1] = __float_as_uint(y1);
          }
          tmem_st32(tmem_o + c * 32, orr);
        }
      }
      tmem_st32(tmem_s, pk);
      tmem_st32(tmem_s + 32, pk + 32);
      tmem_st_wait();
      tc_fence_before();
      warp_arrive(&p_full[t]);
    }

    // ------------------------------------------------------------- epilogue
    if (ok && nt > 0) {
      ok = warp_wait(&o_done[t], (nt - 1) & 1, wc, 12 + t, nt);
      tc_fence_after();
    }
    if (ok) {
      const bool row_ok = qrow < p.Sq;
      const bool have = (nt > 0) && (l > 0.f);
      const float inv_l = have ? 1.f / l : 0.f;
      const float lse_blk = have ? (m_used + log2f(l)) * kLn2 : ninf;
      const size_t lse_idx = (size_t)b * p.lse_sb + (size_t)h * p.lse_sh + qrow;
      float w_old = 0.f, w_blk = have ? 1.f : 0.f, lse_new = lse_blk;
      if (p.merge_prev && row_ok) {
        const float lse_old = p.lse[lse_idx];
        const float mx2 = fmaxf(lse_old, lse_blk);
        if (mx2 == ninf) {
          w_old = 0.f;
          w_blk = 0.f;
          lse_new = ninf;
        } else {
          const float e_old = __expf(lse_old - mx2);
          const float e_blk = __expf(lse_blk - mx2);
          const float sum = e_old + e_blk;
          lse_new = mx2 + __logf(sum);
          w_old = e_old / sum;
          w_blk = e_blk / sum;
        }
      }
      if (row_ok) p.lse[lse_idx] = lse_new;
      const float o_scale = inv_l * w_blk;
      float* acc_row =
          p.out_acc ? p.out_acc + (((size_t)b * p.Sq + qrow) * p.Hq + h) * D : nullptr;
      T* out_row = p.out ? reinterpret_cast<T*>(p.out) + (size_t)b * p.o_sb +
                               (size_t)qrow * p.o_ss + (size_t)h * p.o_sh
                         : nullptr;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t orr[32];
        float o[32];
        if (nt > 0) {
          tmem_ld32(tmem_o + c * 32, orr);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __uint_as_float(orr[i]) * o_scale;
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0.f;
        }
        if (p.merge_prev && row_ok) {
          const float4* old4 = reinterpret_cast<const float4*>(acc_row + c * 32);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 ov = old4[i];
            o[4 * i + 0] = fmaf(w_old, ov.x, o[4 * i + 0]);
            o[4 * i + 1] = fmaf(w_old, ov.y, o[4 * i + 1]);
            o[4 * i + 2] = fmaf(w_old, ov.z, o[4 * i + 2]);
            o[4 * i + 3] = fmaf(w_old, ov.w, o[4 * i + 3]);
          }
        }
        if (acc_row && row_ok) {
          float4* dst4 = reinterpret_cast<float4*>(acc_row + c * 32);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst4[i] = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        }
        if (out_row && row_ok) {
          uint4* dst4 = reinterpret_cast<uint4*>(out_row + c * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            dst4[i] = make_uint4(pack2<T>(o[8 * i], o[8 * i + 1]), pack2<T>(o[8 * i + 2], o[8 * i + 3]),
                                 pack2<T>(o[8 * i + 4], o[8 * i + 5]),
                                 pack2<T>(o[8 * i + 6], o[8 * i + 7]));
        }
      }
    }
  }

  // Common exit: give in-flight copies/MMAs of an aborted CTA time to land,
  // then free TMEM.
  tc_fence_before();
  __syncthreads();
  if (*cta_abort) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    __syncthreads();
  }
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int D, typename T>
int launch_fwd_typed(const spa_fwd_args* a, int is_bf16) {
  using L = FwdSmem<D>;
  CUtensorMap tq, tk, tv;
  if (encode_rows_map(&tq, a->q, is_bf16, D, a->Sq, a->Hq, a->B, a->q_ss, a->q_sh, a->q_sb, kTileM))
    return SPA_ECUDA;
  if (encode_rows_map(&tk, a->k, is_bf16, D, a->Sk, a->Hkv, a->B, a->k_ss, a->k_sh, a->k_sb, kTileN))
    return SPA_ECUDA;
  if (encode_rows_map(&tv, a->v, is_bf16, D, a->Sk, a->Hkv, a->B, a->v_ss, a->v_sh, a->v_sb, kTileN))
    return SPA_ECUDA;
  FwdParams p;
  p.B = a->B; p.Sq = a->Sq; p.Sk = a->Sk; p.Hq = a->Hq; p.Hkv = a->Hkv;
  p.causal = a->causal; p.causal_off = a->causal_off; p.merge_prev = a->merge_prev;
  p.n_qblk = ceil_div(a->Sq, 2 * kTileM);
  p.chunk = (!a->causal || p.n_qblk >= 256) ? p.n_qblk : 1;
  p.scale_log2 = a->scale * kLog2e;
  p.out = a->out; p.o_sb = a->o_sb; p.o_ss = a->o_ss; p.o_sh = a->o_sh;
  p.out_acc = a->out_acc; p.lse = a->lse; p.lse_sb = a->lse_sb; p.lse_sh = a->lse_sh;
  p.status = device_status_word();
  if (!p.status) return SPA_ECUDA;
  const int smem_bytes = L::kTotal + 1024;
  auto kern = attn_fwd_sm100_kernel<D, T>;
  int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes, "fwd sm100");
  if (rc) return rc;
  const long long grid = (long long)p.n_qblk * a->B * a->Hq;
  if (grid <= 0 || grid > 0x7fffffffll) {
    set_error("fwd grid out of range");
    return SPA_EINVAL;
  }
  kern<<<(unsigned)grid, kThreads, smem_bytes, (cudaStream_t)a->stream>>>(tq, tk, tv, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("fwd sm100 launch: %s", cudaGetErrorString(e));
    return SPA_ECUDA;
  }
  return SPA_OK;
}

}  // namespace

int launch_fwd_sm100(const spa_fwd_args* a) {
  const bool bf = a->dtype == SPA_DTYPE_BF16;
  if (a->D == 128) {
    return bf ? launch_fwd_typed<128, __nv_bfloat16>(a, 1) : launch_fwd_typed<128, __half>(a, 0);
  } else if (a->D == 64) {
    return bf ? launch_fwd_typed<64, __nv_bfloat16>(a, 1) : launch_fwd_typed<64, __half>(a, 0);
  }
  set_error("tensor-core forward supports head_dim 64 and 128, got %d", a->D);
  return SPA_EUNSUPPORTED;
}

}  // namespace spa
