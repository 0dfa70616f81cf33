// Flash-attention backward, dQ pass, for sm_100a (tcgen05 + TMEM + TMA).
//
// One CTA owns a 128-row query tile of one query head and streams every K/V tile
// (128 keys) those rows can see:
//     S  = Q K^T            dP = dO V^T
//     P  = exp2(S*scale*log2e - lse*log2e)        (global lse of the full sequence)
//     dS = P * (dP - delta)
//     dQ += dS K            (accumulated in TMEM over the whole walk)
// The CTA is the only writer of its dQ rows: no reduction across CTAs, no atomics,
// and the summation order is fixed by the loop, so results are bitwise reproducible.
// Together with attn_bwd_dkv_sm100.cu (the K/V-stationary pass) this is the
// per-step backward that the ring loop of sp_aurora/ring_flash_attn.py:97-152 expects
// (the reference's own sp_aurora/intel_flash_attn.py:129 is a stub); formulas as in
// the manual backward of sp_aurora/intel_ulysses_attn.py:403-426.
//
// CTA = 18 warps:
//   warps 0-15  four compute groups of four warps: query row per thread, group g works on
//               key columns [32g, 32g+32) of a tile (four warps per scheduler hide the
//               latency of the TMEM loads and of the exponentials)
//   warp  16    TMA producer (lane 0)     warp 17  MMA issuer (lane 0), TMEM owner
// TMEM columns: S [0,128)  dP [128,256)  dQ [256,256+D)  dS [384,448) (16-bit, two
// per column)  Q [448,448+D/2) (16-bit). Q and dS are the TMEM A operands of the S
// and dQ products, so per K/V tile shared memory is read only for dO (A of dP) and
// for K, V, K as B operands. Shared memory: the dO tile and a 3-stage ring of K|V.
//
// Tensor-pipe order per tile j:  S(j+1), dP(j+1), dQ(j)  -- the compute warps take S(j)
// and dP(j) into registers as soon as they exist, so the next tile's scores are on the
// pipe while S(j), dP(j) are turned into dS(j).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include <type_traits>

#include "spa_internal.h"
#include "tc05.cuh"

namespace spa {
namespace {

constexpr int kTileM = 128;   // query rows per CTA
constexpr int kTileN = 128;   // keys per K/V tile
constexpr int kThreads = 576;
constexpr int kComputeThreads = 512;
constexpr int kWarpTma = 16, kWarpMma = 17;
constexpr int kStages = 3;
constexpr float kLog2e = 1.4426950408889634f;
constexpr uint32_t kColS = 0, kColDP = 128, kColDQ = 256, kColDS = 384, kColQ = 448;

struct DqParams {
  int B, Sq, Sk, Hq, Hkv;
  int causal, causal_off;
  int dq_overwrite;
  int n_qblk;
  int chunk;   // query tiles per scheduling chunk (n_qblk or 1)
  float scale, scale_log2;
  const void* q;
  int64_t q_sb, q_ss, q_sh;
  const float* lse;
  const float* delta;
  int64_t lse_sb, lse_sh;
  float* dq_acc;
  void* dq;
  int64_t dq_sb, dq_ss, dq_sh;
  int* status;
};

template <int D>
struct DqSmem {
  static constexpr int kSlab = kTileN * 128;                 // 128 rows x 128 B
  static constexpr int kTile = (D / 64) * kSlab;             // one dO / K / V tile
  static constexpr int kStageBytes = 2 * kTile;              // K + V
  static constexpr int kDoOff = 0;
  static constexpr int kKVOff = kDoOff + kTile;
  static constexpr int kBarOff = kKVOff + kStages * kStageBytes;
  static constexpr int kNumBars = 2 + 2 * kStages + 4;
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
attn_bwd_dq_sm100_kernel(const __grid_constant__ CUtensorMap tm_k,
                         const __grid_constant__ CUtensorMap tm_v,
                         const __grid_constant__ CUtensorMap tm_do, const DqParams p) {
  using L = DqSmem<D>;
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* do_full = bars;
  uint64_t* q_ready = bars + 1;
  uint64_t* kv_full = bars + 2;
  uint64_t* kv_empty = kv_full + kStages;
  uint64_t* sdp_full = kv_empty + kStages;    // S(j) and dP(j) are complete
  uint64_t* sdp_free = sdp_full + 1;          // S(j) and dP(j) are in registers
  uint64_t* ds_full = sdp_free + 1;
  uint64_t* dq_done = ds_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Work decode: query tiles of one chunk fastest (longest first under a causal mask),
  // then heads, batch, chunks; the CTAs resident together stream the K/V of one kv head.
  int w = blockIdx.x;
  const int q_lo = w % p.chunk;
  w /= p.chunk;
  const int h = w % p.Hq;
  w /= p.Hq;
  const int b = w % p.B;
  const int qblk = p.n_qblk - 1 - ((w / p.B) * p.chunk + q_lo);
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qblk * kTileM;

  // K/V tiles this query tile can see.
  int n_kv = (p.Sk + kTileN - 1) / kTileN;
  if (p.causal) {
    const long long last_key = (long long)min(q0 + kTileM, p.Sq) - 1 + p.causal_off;  // inclusive
    const int nc = last_key < 0 ? 0 : (int)(last_key / kTileN) + 1;
    n_kv = min(n_kv, nc);
  }

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    mbar_init(do_full, 1);
    mbar_init(q_ready, kComputeThreads / 32);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(sdp_free, kComputeThreads / 32);
    mbar_init(ds_full, kComputeThreads / 32);
    mbar_init(dq_done, 1);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == kWarpMma) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  WaitCtx wc{p.status, cta_abort};

  if (warp == kWarpTma) {
    // ------------------------------------------------------------------ TMA
    if (lane == 0 && n_kv > 0) {
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_do);
      mbar_arrive_expect_tx(do_full, L::kTile);
      for (int s = 0; s < D / 64; ++s)
        tma_load_4d(smem + L::kDoOff + s * L::kSlab, &tm_do, do_full, s * 64, q0, h, b);
      for (int j = 0; j < n_kv; ++j) {
        const int slot = j % kStages;
        const uint32_t ph = (j / kStages) & 1;
        if (!mbar_wait(&kv_empty[slot], ph ^ 1, wc, 0, j)) break;
        uint8_t* st = smem + L::kKVOff + slot * L::kStageBytes;
        mbar_arrive_expect_tx(&kv_full[slot], L::kStageBytes);
        for (int s = 0; s < D / 64; ++s) {
          tma_load_4d(st + s * L::kSlab, &tm_k, &kv_full[slot], s * 64, j * kTileN, hk, b);
          tma_load_4d(st + L::kTile + s * L::kSlab, &tm_v, &kv_full[slot], s * 64, j * kTileN, hk, b);
        }
      }
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------------ MMA
    if (lane == 0 && n_kv > 0) {
      constexpr uint32_t idesc_s = make_idesc(128, kTileN, kBf16, false, false);
      constexpr uint32_t idesc_dq = make_idesc(128, D, kBf16, false, true);
      const uint32_t do_base = smem_u32(smem + L::kDoOff);
      const uint32_t kv_base = smem_u32(smem + L::kKVOff);
      const SmemDesc do_km = make_smem_desc(do_base, 16, 1024);          // dO, K-major (A of dP)
      const SmemDesc kv_km = make_smem_desc(kv_base, 16, 1024);          // K / V, K-major (B of S, dP)
      const SmemDesc k_mn = make_smem_desc(kv_base, L::kSlab, 1024);     // K, MN-major (B of dQ)
      bool ok = mbar_wait(do_full, 0, wc, 1, 0);
      if (ok) ok = mbar_wait(q_ready, 0, wc, 2, 0);
      tc_fence_after();

      // `slot` is a compile-time constant at every call site (the tile loop is unrolled
      // over the ring period): runtime descriptor words cost issue time.
      // S(j) = Q K_j^T : A = Q from TMEM, B = K tile (K-major).
      auto issue_s = [&](int j, const int slot) -> bool {
        if (!mbar_wait(&kv_full[slot], (j / kStages) & 1, wc, 3, j)) return false;
        tc_fence_after();
        const uint32_t b0 = (slot * L::kStageBytes) >> 4;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = ((kk / 4) * L::kSlab + (kk % 4) * 32) >> 4;
          mma_ts_d(tmem_base + kColS, tmem_base + kColQ + kk * 8, kv_km, b0 + off, idesc_s, kk > 0);
        }
        return true;
      };
      // dP(j) = dO V_j^T : A = dO tile (shared memory), B = V tile (K-major).
      auto issue_dp = [&](const int slot) {
        const uint32_t b0 = (slot * L::kStageBytes + L::kTile) >> 4;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = ((kk / 4) * L::kSlab + (kk % 4) * 32) >> 4;
          mma_ss_d(tmem_base + kColDP, do_km, off, kv_km, b0 + off, idesc_s, kk > 0);
        }
        mma_commit(sdp_full);
      };

      if (ok) ok = issue_s(0, 0);
      if (ok) issue_dp(0);
      for (int j0 = 0; j0 < n_kv && ok; j0 += kStages) {
#pragma unroll
        for (int sl = 0; sl < kStages; ++sl) {
          const int j = j0 + sl;
          if (j >= n_kv || !ok) break;
          if (j + 1 < n_kv) {
            ok = mbar_wait(sdp_free, j & 1, wc, 4, j);    // S(j) and dP(j) are in registers
            if (!ok) break;
            tc_fence_after();
            ok = issue_s(j + 1, (sl + 1) % kStages);
            if (!ok) break;
            issue_dp((sl + 1) % kStages);
          }
          ok = mbar_wait(ds_full, j & 1, wc, 6, j);
          if (!ok) break;
          tc_fence_after();
          // dQ += dS(j) K_j : A = dS from TMEM, B = K tile MN-major (rows = keys).
          const uint32_t b0 = (sl * L::kStageBytes) >> 4;
#pragma unroll
          for (int kk = 0; kk < kTileN / 16; ++kk)
            mma_ts_d(tmem_base + kColDQ, tmem_base + kColDS + kk * 8, k_mn, b0 + ((kk * 2048) >> 4),
                     idesc_dq, (j > 0 || kk > 0));
          mma_commit(&kv_empty[sl]);
          mma_commit(dq_done);
        }
      }
    }
  } else {
    // -------------------------------------------------------------- compute
    const int grp = warp >> 2;                 // key-column quarter of the tile
    const int quad = warp & 3;
    const int r = quad * 32 + lane;            // query row in tile = TMEM lane
    const int qrow = q0 + r;
    const bool row_ok = qrow < p.Sq;
    const int c_base = grp * 32;
    constexpr int kOutCols = D / 4;            // dQ columns (and Q elements) per group
    const uint32_t lane_field = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_s = tmem_base + lane_field + kColS + c_base;
    const uint32_t t_dp = tmem_base + lane_field + kColDP + c_base;
    const uint32_t t_ds = tmem_base + lane_field + kColDS + grp * 16;
    const uint32_t t_dq = tmem_base + lane_field + kColDQ + grp * kOutCols;
    const uint32_t t_q = tmem_base + lane_field + kColQ + grp * (D / 8);
    bool ok = true;

    // Q row -> TMEM (the A operand of S): each group stores a quarter of the row.
    if (n_kv > 0) {
      constexpr int kWords = D / 8;            // 32-bit words (two elements each) per group
      uint32_t qw[kWords];
      if (row_ok) {
        const uint4* src = reinterpret_cast<const uint4*>(
            reinterpret_cast<const T*>(p.q) + (size_t)b * p.q_sb + (size_t)qrow * p.q_ss +
            (size_t)h * p.q_sh + grp * (D / 4));
#pragma unroll
        for (int i = 0; i < kWords / 4; ++i) {
          const uint4 v = src[i];
          qw[4 * i] = v.x; qw[4 * i + 1] = v.y; qw[4 * i + 2] = v.z; qw[4 * i + 3] = v.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < kWords; ++i) qw[i] = 0u;
      }
      if constexpr (D == 128) tmem_st16(t_q, qw); else tmem_st8(t_q, qw);
      tmem_st_wait();
      tc_fence_before();
      warp_arrive(q_ready);
    }
    // Row statistics, negated for the packed multiply-adds: -inf in place of -lse makes
    // out-of-range rows give P = 0.
    const size_t sidx = (size_t)b * p.lse_sb + (size_t)h * p.lse_sh + (row_ok ? qrow : 0);
    const float nlse2 = row_ok ? -p.lse[sidx] * kLog2e : -INFINITY;
    const float ndlt = row_ok ? -p.delta[sidx] : 0.f;

    for (int j = 0; j < n_kv; ++j) {
      // dP(j) follows S(j) on the in-order tensor pipe, so its completion covers both. Both are
      // taken into registers before the exponentials: the issuer can then put S(j+1) and
      // dP(j+1) on the pipe back to back while this tile is turned into dS.
      ok = warp_wait(sdp_full, j & 1, wc, 8, j);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[32], dpr[32];
      tmem_ld32(t_s, sr);
      tmem_ld32(t_dp, dpr);
      tmem_ld_wait();
      tc_fence_before();
      warp_arrive(sdp_free);
      float* pr = reinterpret_cast<float*>(sr);   // scores, then probabilities, in place

      const int k0 = j * kTileN;
      const bool need_mask =
          (k0 + kTileN > p.Sk) ||
          (p.causal && ((long long)k0 + kTileN - 1 > (long long)q0 + p.causal_off));
      if (!need_mask) {                            // tiles below the diagonal: no selects
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float x0, x1;
          fma2(x0, x1, pr[c], pr[c + 1], p.scale_log2, p.scale_log2, nlse2, nlse2);
          pr[c] = fast_exp2(x0);
          pr[c + 1] = fast_exp2(x1);
        }
      } else {
        long long lim = p.Sk - 1;
        if (p.causal) lim = min(lim, (long long)qrow + p.causal_off);
        const int limit = (int)max(0ll, min(lim - k0 - c_base + 1, 32ll));   // first masked column
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float x0, x1;
          fma2(x0, x1, pr[c], pr[c + 1], p.scale_log2, p.scale_log2, nlse2, nlse2);
          pr[c] = c < limit ? fast_exp2(x0) : 0.f;
          pr[c + 1] = c + 1 < limit ? fast_exp2(x1) : 0.f;
        }
      }
      uint32_t dsp[16];
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        float e0, e1, d0, d1;
        add2(e0, e1, __uint_as_float(dpr[c]), __uint_as_float(dpr[c + 1]), ndlt, ndlt);
        mul2(d0, d1, pr[c], pr[c + 1], e0, e1);
        dsp[c >> 1] = pack2<T>(d0, d1);
      }
      if (j > 0) {
        // dQ(j-1) has finished reading the dS columns.
        ok = warp_wait(dq_done, (j - 1) & 1, wc, 10, j);
        if (!ok) break;
        tc_fence_after();
      }
      tmem_st16(t_ds, dsp);
      tmem_st_wait();
      tc_fence_before();
      warp_arrive(ds_full);
    }

    // ------------------------------------------------------------- epilogue
    if (ok && n_kv > 0) {
      ok = warp_wait(dq_done, (n_kv - 1) & 1, wc, 11, n_kv);
      if (ok) tc_fence_after();
    }
    if (ok) {
      // total = (earlier ring steps' sum unless dq_overwrite) + scale * dQ; it goes to dq in
      // the element type and / or back to the fp32 accumulator, whichever is given.
      const size_t acc_off = (((size_t)b * p.Sq + qrow) * p.Hq + h) * D + grp * kOutCols;
      const float* acc_in = (!p.dq_overwrite && p.dq_acc) ? p.dq_acc + acc_off : nullptr;
      float* acc_out = p.dq_acc ? p.dq_acc + acc_off : nullptr;
      T* out_row = p.dq ? reinterpret_cast<T*>(p.dq) + (size_t)b * p.dq_sb + (size_t)qrow * p.dq_ss +
                              (size_t)h * p.dq_sh + grp * kOutCols
                        : nullptr;
      const bool skip = (n_kv == 0) && !p.dq_overwrite && !p.dq;   // the accumulator already holds the total
      float o[kOutCols];
      if (n_kv > 0) {
        uint32_t v[kOutCols];
        if constexpr (kOutCols == 32) tmem_ld32(t_dq, v); else tmem_ld16(t_dq, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < kOutCols; ++i) o[i] = __uint_as_float(v[i]) * p.scale;
      } else {
#pragma unroll
        for (int i = 0; i < kOutCols; ++i) o[i] = 0.f;
      }
      if (row_ok && !skip) {
        if (acc_in) {
          const float4* a4 = reinterpret_cast<const float4*>(acc_in);
#pragma unroll
          for (int i = 0; i < kOutCols / 4; ++i) {
            const float4 a = a4[i];
            o[4 * i] += a.x; o[4 * i + 1] += a.y; o[4 * i + 2] += a.z; o[4 * i + 3] += a.w;
          }
        }
        if (out_row) {
          uint4* dst = reinterpret_cast<uint4*>(out_row);
#pragma unroll
          for (int i = 0; i < kOutCols / 8; ++i)
            dst[i] = make_uint4(pack2<T>(o[8 * i], o[8 * i + 1]), pack2<T>(o[8 * i + 2], o[8 * i + 3]),
                                pack2<T>(o[8 * i + 4], o[8 * i + 5]),
                                pack2<T>(o[8 * i + 6], o[8 * i + 7]));
        }
        if (acc_out) {
          float4* dst = reinterpret_cast<float4*>(acc_out);
#pragma unroll
          for (int i = 0; i < kOutCols / 4; ++i)
            dst[i] = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        }
      }
    }
  }

  // Common exit: give in-flight copies/MMAs of an aborted CTA time to land, then free TMEM.
  tc_fence_before();
  __syncthreads();
  if (*cta_abort) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    __syncthreads();
  }
  if (warp == kWarpMma) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int D, typename T>
int launch_dq_typed(const spa_bwd_args* a, int is_bf16) {
  using L = DqSmem<D>;
  CUtensorMap tk, tv, tdo;
  if (encode_rows_map(&tdo, a->dout, is_bf16, D, a->Sq, a->Hq, a->B, a->do_ss, a->do_sh, a->do_sb,
                      kTileM))
    return SPA_ECUDA;
  if (encode_rows_map(&tk, a->k, is_bf16, D, a->Sk, a->Hkv, a->B, a->k_ss, a->k_sh, a->k_sb, kTileN))
    return SPA_ECUDA;
  if (encode_rows_map(&tv, a->v, is_bf16, D, a->Sk, a->Hkv, a->B, a->v_ss, a->v_sh, a->v_sb, kTileN))
    return SPA_ECUDA;
  DqParams p;
  p.B = a->B; p.Sq = a->Sq; p.Sk = a->Sk; p.Hq = a->Hq; p.Hkv = a->Hkv;
  p.causal = a->causal; p.causal_off = a->causal_off;
  p.dq_overwrite = a->dq_overwrite;
  p.n_qblk = ceil_div(a->Sq, kTileM);
  p.chunk = (!a->causal || p.n_qblk >= 512) ? p.n_qblk : 1;
  p.scale = a->scale; p.scale_log2 = a->scale * kLog2e;
  p.q = a->q; p.q_sb = a->q_sb; p.q_ss = a->q_ss; p.q_sh = a->q_sh;
  p.lse = a->lse; p.delta = a->delta; p.lse_sb = a->lse_sb; p.lse_sh = a->lse_sh;
  p.dq_acc = a->dq_acc; p.dq = a->dq; p.dq_sb = a->dq_sb; p.dq_ss = a->dq_ss; p.dq_sh = a->dq_sh;
  p.status = device_status_word();
  if (!p.status) return SPA_ECUDA;
  const int smem_bytes = L::kTotal + 1024;
  auto kern = attn_bwd_dq_sm100_kernel<D, T>;
  int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes, "bwd dq sm100");
  if (rc) return rc;
  const long long grid = (long long)p.n_qblk * a->B * a->Hq;
  if (grid <= 0 || grid > 0x7fffffffll) {
    set_error("bwd dq grid out of range");
    return SPA_EINVAL;
  }
  kern<<<(unsigned)grid, kThreads, smem_bytes, (cudaStream_t)a->stream>>>(tk, tv, tdo, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("bwd dq sm100 launch: %s", cudaGetErrorString(e));
    return SPA_ECUDA;
  }
  return SPA_OK;
}

}  // namespace

int launch_bwd_dq_sm100(const spa_bwd_args* a) {
  const bool bf = a->dtype == SPA_DTYPE_BF16;
  if (((uintptr_t)a->q & 15) || ((a->q_ss * 2) & 15) || ((a->q_sh * 2) & 15) || ((a->q_sb * 2) & 15)) {
    set_error("q base and strides must be 16-byte aligned");
    return SPA_EINVAL;
  }
  if (a->D == 128) {
    return bf ? launch_dq_typed<128, __nv_bfloat16>(a, 1) : launch_dq_typed<128, __half>(a, 0);
  } else if (a->D == 64) {
    return bf ? launch_dq_typed<64, __nv_bfloat16>(a, 1) : launch_dq_typed<64, __half>(a, 0);
  }
  set_error("tensor-core backward supports head_dim 64 and 128, got %d", a->D);
  return SPA_EUNSUPPORTED;
}

}  // namespace spa
