// Flash-attention backward, dK/dV pass, for sm_100a (tcgen05 + TMEM + TMA).
//
// One CTA owns a 128-key K/V tile of one kv head and walks over every 128-row
// query tile (of every query head in its GQA group) that can see those keys.
// Scores are computed TRANSPOSED (rows = keys, columns = queries) so that the
// probabilities P^T and dS^T are already the A operands of the dV / dK products:
//     S^T  = K  Q^T          dP^T = V dO^T
//     P^T  = exp2(S^T*scale*log2e - lse*log2e)      (global lse of the full sequence)
//     dS^T = P^T * (dP^T - delta)
//     dV  += P^T dO          dK  += dS^T Q
// dV/dK stay in TMEM for the whole walk; every product is an N=128 MMA. dQ is not
// computed here: attn_bwd_dq_sm100.cu does it with the query tile stationary, so no
// kernel reduces across CTAs. The softmax scale is applied once on the way out.
//
// Algorithm source: the per-step flash backward that the ring loop of
// sp_aurora/ring_flash_attn.py:97-152 expects (the reference's own
// sp_aurora/intel_flash_attn.py:129 is a stub); formulas as in the manual
// backward of sp_aurora/intel_ulysses_attn.py:403-426.
//
// CTA = 18 warps:
//   warps 0-15  four compute groups of four warps: key row per thread, group g works on
//               query columns [32g, 32g+32) (four warps per scheduler hide the latency of
//               the TMEM loads and of the exponentials); the first 256 compute threads also
//               fetch lse*log2e and delta of the next query tile into shared memory
//   warp  16    TMA producer     warp 17  MMA issuer and TMEM owner
// TMEM columns: S^T [0,128) dP^T [128,256) dV [256,256+D) dK [384,384+D). P^T (16-bit,
// two per column) of group g overwrites columns [32g, 32g+16) of S^T, dS^T the same
// columns of dP^T: each compute thread overwrites only columns it has already read, and the
// in-order tensor pipe lets S^T(i+1) be issued right behind dV(i), dP^T(i+1) behind dK(i).
// Shared memory: K, V tiles and a ring of four Q / dO tiles (Q in slots 0,2; dO in 1,3).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>
#include <stdlib.h>

#include <type_traits>

#include "spa_internal.h"
#include "tc05.cuh"

namespace spa {
namespace {

constexpr int kTileKV = 128;
constexpr int kTileQ = 128;
constexpr int kThreads = 576;
constexpr int kComputeThreads = 512;
constexpr int kWarpTma = 16, kWarpMma = 17;
constexpr int kStatBufs = 3;   // row-statistics buffers (see the compute loop)
constexpr int kRing = 4;
constexpr float kLog2e = 1.4426950408889634f;
constexpr uint32_t kColS = 0, kColDP = 128, kColDV = 256, kColDK = 384;

struct DkvParams {
  int B, Sq, Sk, Hq, Hkv;
  int causal, causal_off;
  int dkv_fp32, dkv_accumulate;
  int q_split;     // CTAs sharing one K/V tile, each over a slice of the query tiles (dK/dV reduce-added)
  int n_kvblk;
  int chunk;       // K/V tiles per scheduling chunk (n_kvblk or 1)
  float scale, scale_log2;
  const float* lse;
  const float* delta;
  int64_t lse_sb, lse_sh;
  void* dk;
  void* dv;
  int64_t dkv_sb, dkv_ss, dkv_sh;
  int* status;
};

template <int D>
struct DkvSmem {
  static constexpr int kSlab = kTileKV * 128;                // 128 rows x 128 B
  static constexpr int kTile = (D / 64) * kSlab;             // one K / V / Q / dO tile
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kKOff + kTile;
  static constexpr int kRingOff = kVOff + kTile;
  static constexpr int kRowOff = kRingOff + kRing * kTile;   // [3 bufs][lse2|delta][128] floats
  static constexpr int kBarOff = kRowOff + kStatBufs * 2 * kTileQ * 4;
  static constexpr int kNumBars = 1 + 2 * kRing + 6 + kStatBufs;
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
attn_bwd_dkv_sm100_kernel(const __grid_constant__ CUtensorMap tm_q,
                          const __grid_constant__ CUtensorMap tm_k,
                          const __grid_constant__ CUtensorMap tm_v,
                          const __grid_constant__ CUtensorMap tm_do,
                          const __grid_constant__ CUtensorMap tm_dk,
                          const __grid_constant__ CUtensorMap tm_dv, const DkvParams p) {
  using L = DkvSmem<D>;
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* kv_full = bars;
  uint64_t* tile_full = bars + 1;              // [kRing]
  uint64_t* tile_empty = tile_full + kRing;    // [kRing]
  uint64_t* s_full = tile_empty + kRing;
  uint64_t* dp_full = s_full + 1;
  uint64_t* p_full = dp_full + 1;
  uint64_t* ds_full = p_full + 1;
  uint64_t* mma_done = ds_full + 1;
  uint64_t* row_ready = mma_done + 1;          // [kStatBufs]
  uint64_t* epi_full = row_ready + kStatBufs;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* row_buf = reinterpret_cast<float*>(smem + L::kRowOff);  // [buf][lse2|delta][128]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Work decode: query slices, then K/V tiles of one chunk fastest, then kv heads, batch,
  // chunks. The host picks the chunk: all tiles (CTAs resident together then walk the Q / dO
  // tiles of the same query heads a few tiles apart and share every HBM fetch through L2),
  // or one tile for small causal problems, where longest-tile-first over all heads matters
  // more.
  int w = blockIdx.x;
  const int qs = w % p.q_split;
  w /= p.q_split;
  const int kv_lo = w % p.chunk;
  w /= p.chunk;
  const int g = w % p.Hkv;
  w /= p.Hkv;
  const int b = w % p.B;
  const int kvblk = (w / p.B) * p.chunk + kv_lo;
  const int kv0 = kvblk * kTileKV;
  const int G = p.Hq / p.Hkv;

  // Query tiles that can see this K/V tile.
  int i_end = (p.Sq + kTileQ - 1) / kTileQ;
  int i_start = 0;
  if (p.causal) {
    const long long first_q = (long long)kv0 - p.causal_off;  // smallest query index seeing kv0
    if (first_q > 0) i_start = (int)min((long long)i_end, first_q / kTileQ);
  }
  if (p.q_split > 1) {  // this CTA's slice of the visible query tiles
    const int vis = i_end - i_start;
    const int lo = i_start + (int)((long long)vis * qs / p.q_split);
    i_end = i_start + (int)((long long)vis * (qs + 1) / p.q_split);
    i_start = lo;
  }
  const int n_q = i_end - i_start;
  const int n_it = n_q * G;

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    mbar_init(kv_full, 1);
    for (int i = 0; i < kRing; ++i) {
      mbar_init(&tile_full[i], 1);
      mbar_init(&tile_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_full, kComputeThreads / 32);
    mbar_init(ds_full, kComputeThreads / 32);
    mbar_init(mma_done, 1);
    for (int i = 0; i < kStatBufs; ++i) mbar_init(&row_ready[i], 256 / 32);
    mbar_init(epi_full, kComputeThreads / 32);
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
    if (lane == 0 && n_it > 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_do);
      mbar_arrive_expect_tx(kv_full, 2 * L::kTile);
      for (int s = 0; s < D / 64; ++s) {
        tma_load_4d(smem + L::kKOff + s * L::kSlab, &tm_k, kv_full, s * 64, kv0, g, b);
        tma_load_4d(smem + L::kVOff + s * L::kSlab, &tm_v, kv_full, s * 64, kv0, g, b);
      }
      for (int n = 0; n < 2 * n_it; ++n) {       // n even: Q tile, n odd: dO tile
        const int slot = n % kRing;
        const uint32_t ph = (n / kRing) & 1;
        if (!mbar_wait(&tile_empty[slot], ph ^ 1, wc, 0, n)) break;
        const int it = n >> 1;
        const int hq = g * G + it / n_q;
        const int q0 = (i_start + it % n_q) * kTileQ;
        uint8_t* st = smem + L::kRingOff + slot * L::kTile;
        const CUtensorMap* tm = (n & 1) ? &tm_do : &tm_q;
        mbar_arrive_expect_tx(&tile_full[slot], L::kTile);
        for (int s = 0; s < D / 64; ++s)
          tma_load_4d(st + s * L::kSlab, tm, &tile_full[slot], s * 64, q0, hq, b);
      }
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------------ MMA
    // One elected lane issues every MMA; descriptors are precomputed, offsets are constants.
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idesc_sdp = make_idesc(128, kTileQ, kBf16, false, false);
      constexpr uint32_t idesc_dkv = make_idesc(128, D, kBf16, false, true);
      const uint32_t k_base = smem_u32(smem + L::kKOff);
      const uint32_t v_base = smem_u32(smem + L::kVOff);
      const uint32_t ring_base = smem_u32(smem + L::kRingOff);
      const SmemDesc k_km = make_smem_desc(k_base, 16, 1024);             // K tile, K-major (A of S^T)
      const SmemDesc v_km = make_smem_desc(v_base, 16, 1024);             // V tile, K-major (A of dP^T)
      const SmemDesc ring_km = make_smem_desc(ring_base, 16, 1024);       // Q / dO, K-major (B of S^T, dP^T)
      const SmemDesc ring_mn = make_smem_desc(ring_base, L::kSlab, 1024); // Q / dO, MN-major (B of dK, dV)
      bool ok = mbar_wait(kv_full, 0, wc, 1, 0);
      tc_fence_after();

      // `slot` is a compile-time constant at every call site (the iteration loop is
      // unrolled over the ring period): runtime descriptor words cost issue time.
      // S^T(it) = K Q^T (slot even) or dP^T(it) = V dO^T (slot odd).
      auto issue_scores = [&](int it, const int slot) -> bool {
        const int n = 2 * it + (slot & 1);
        if (!mbar_wait(&tile_full[slot], (n / kRing) & 1, wc, 2, n)) return false;
        tc_fence_after();
        const uint32_t b0 = (slot * L::kTile) >> 4;
        const SmemDesc& a_desc = (slot & 1) ? v_km : k_km;
        const uint32_t d_col = (slot & 1) ? kColDP : kColS;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = ((kk / 4) * L::kSlab + (kk % 4) * 32) >> 4;
          mma_ss_d(tmem_base + d_col, a_desc, off, ring_km, b0 + off, idesc_sdp, kk > 0);
        }
        mma_commit((slot & 1) ? dp_full : s_full);
        return true;
      };
      // dV += P^T dO (slot odd) or dK += dS^T Q (slot even): A from TMEM (16 queries = 8
      // columns per step; the 32 queries of compute group g sit at column 32g of the score
      // region), B = the dO / Q tile read MN-major (rows = queries).
      auto issue_grad = [&](int it, const int slot) {
        const uint32_t b0 = (slot * L::kTile) >> 4;
        const uint32_t a_col = (slot & 1) ? kColS : kColDP;
        const uint32_t d_col = (slot & 1) ? kColDV : kColDK;
#pragma unroll
        for (int kk = 0; kk < kTileQ / 16; ++kk)
          mma_ts_d(tmem_base + d_col, tmem_base + a_col + (kk / 2) * 32 + (kk % 2) * 8, ring_mn,
                   b0 + ((kk * 2048) >> 4), idesc_dkv, (it > 0 || kk > 0));
      };

      if (ok) ok = issue_scores(0, 0);
      if (ok) ok = issue_scores(0, 1);
      for (int it0 = 0; it0 < n_it && ok; it0 += 2) {
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          const int it = it0 + jj;
          if (it >= n_it || !ok) break;
          ok = mbar_wait(p_full, it & 1, wc, 3, it);
          if (!ok) break;
          tc_fence_after();
          issue_grad(it, 2 * jj + 1);                                    // dV(it)
          if (it + 1 < n_it) {
            ok = issue_scores(it + 1, (2 * jj + 2) % kRing);             // S^T(it+1)
            if (!ok) break;
          }
          ok = mbar_wait(ds_full, it & 1, wc, 4, it);
          if (!ok) break;
          tc_fence_after();
          issue_grad(it, 2 * jj);                                        // dK(it)
          mma_commit(&tile_empty[2 * jj]);
          mma_commit(&tile_empty[2 * jj + 1]);
          if (it + 1 < n_it) {
            ok = issue_scores(it + 1, (2 * jj + 3) % kRing);             // dP^T(it+1)
            if (!ok) break;
          }
        }
      }
      if (ok) mma_commit(mma_done);
    }
  } else {
    // -------------------------------------------------------------- compute
    // Loop layout (TMEM shape 16x256b): the warp's 32 key rows are read as two 16-row
    // halves; in half hh, lane (g8, t4) = (lane / 4, lane % 4) holds rows
    // 16*hh + g8 and 16*hh + g8 + 8 of the warp's quadrant and the query columns
    // {8i + 2*t4, 8i + 2*t4 + 1 : i = 0..3} of the group's 32. A thread thus needs the
    // statistics (lse, delta) of 8 query columns for its 4 rows x 8 columns, instead of 32
    // for 1 row x 32 columns in the row-per-thread shape: the shared-memory broadcast
    // reads of the statistics were more than a third of this kernel's shared-memory
    // traffic, which is what bounds it. The epilogue uses the row-per-thread shape.
    const int grp = warp >> 2;               // query-column quarter of the tile
    const int quad = warp & 3;
    const int r = quad * 32 + lane;          // key row in tile = TMEM lane (epilogue)
    const int kidx = kv0 + r;
    const int g8 = lane >> 2, t4 = lane & 3;
    const int c_base = grp * 32;
    const uint32_t lane_field = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t half_step = 16u << 16;    // second 16-row half of the quadrant
    const uint32_t t_s = tmem_base + lane_field + kColS + c_base;      // scores, then P^T in [0,16)
    const uint32_t t_dp = tmem_base + lane_field + kColDP + c_base;    // dP^T, then dS^T in [0,16)
    const uint32_t t_dv = tmem_base + lane_field + kColDV;
    const uint32_t t_dk = tmem_base + lane_field + kColDK;
    const bool key_ok = kidx < p.Sk;
    bool ok = true;

    // Row statistics of a query tile, fetched by the first 256 compute threads and stored
    // NEGATED (the packed multiply-adds below add them): threads 0-127 -lse*log2(e), threads
    // 128-255 -delta. -inf in place of -lse makes out-of-range query rows give P = 0. Iteration `it` reads buffer it % 3 and fills
    // buffer (it + 1) % 3: a thread can be at most one iteration ahead of the slowest one
    // (it cannot pass the scores of iteration it before every thread has handed in P^T of
    // iteration it - 1), so the buffer being filled is never one that is still being read.
    const int stat_tid = threadIdx.x;
    auto fetch_rowstat = [&](int it) -> float {
      const int hq = g * G + it / n_q;
      const int qi = (i_start + it % n_q) * kTileQ + (stat_tid & 127);
      const size_t idx = (size_t)b * p.lse_sb + (size_t)hq * p.lse_sh + qi;
      if (stat_tid < 128) return qi < p.Sq ? -p.lse[idx] * kLog2e : -INFINITY;
      return qi < p.Sq ? -p.delta[idx] : 0.f;
    };
    if (n_it > 0 && stat_tid < 256) {
      row_buf[(0 * 2 + (stat_tid >> 7)) * kTileQ + (stat_tid & 127)] = fetch_rowstat(0);
      warp_arrive(&row_ready[0]);
    }

    for (int it = 0; it < n_it; ++it) {
      const int buf = it % kStatBufs;
      float next_stat = 0.f;
      if (stat_tid < 256 && it + 1 < n_it) next_stat = fetch_rowstat(it + 1);

      ok = warp_wait(&row_ready[buf], (it / kStatBufs) & 1, wc, 8, it);
      if (!ok) break;
      const float* lse2 = row_buf + (buf * 2 + 0) * kTileQ + c_base + 2 * t4;
      const float* dlt = row_buf + (buf * 2 + 1) * kTileQ + c_base + 2 * t4;
      float2 lv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) lv[i] = *reinterpret_cast<const float2*>(lse2 + 8 * i);
      const int q0 = (i_start + it % n_q) * kTileQ;
      // warp-uniform: does any row of this tile mask a column of this group?
      // (key kidx is visible to query column c iff c >= kidx - off - q0 - c_base)
      const bool need_mask = !(kv0 + kTileKV <= p.Sk) ||
                             (p.causal && (long long)kv0 + kTileKV - 1 - p.causal_off > (long long)q0 + c_base);

      ok = warp_wait(s_full, it & 1, wc, 9, it);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[32];                        // [half][16]: scores, then probabilities, in place
      tmem_ld_16x256b_x4(t_s, sr);
      tmem_ld_16x256b_x4(t_s + half_step, sr + 16);
      tmem_ld_wait();
      float* pr = reinterpret_cast<float*>(sr);
#pragma unroll
      for (int hh = 0; hh < 2; ++hh)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float* e = pr + hh * 16 + 4 * i;    // rows g8 (e[0], e[1]) and g8 + 8 (e[2], e[3])
          float x0, x1, x2, x3;
          fma2(x0, x1, e[0], e[1], p.scale_log2, p.scale_log2, lv[i].x, lv[i].y);
          fma2(x2, x3, e[2], e[3], p.scale_log2, p.scale_log2, lv[i].x, lv[i].y);
          e[0] = fast_exp2(x0);
          e[1] = fast_exp2(x1);
          e[2] = fast_exp2(x2);
          e[3] = fast_exp2(x3);
        }
      if (need_mask) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh)
#pragma unroll
          for (int rr = 0; rr < 2; ++rr) {
            const int krow = kv0 + quad * 32 + hh * 16 + rr * 8 + g8;
            long long cm = 0;
            if (p.causal) cm = (long long)krow - p.causal_off - q0 - c_base;
            int c_min = (int)max(0ll, min(cm, 32ll));
            if (krow >= p.Sk) c_min = 32;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float* e = pr + hh * 16 + 4 * i + 2 * rr;
              const int c = 8 * i + 2 * t4;
              if (c < c_min) e[0] = 0.f;
              if (c + 1 < c_min) e[1] = 0.f;
            }
          }
      }
      uint32_t pk[16];
#pragma unroll
      for (int hh = 0; hh < 2; ++hh)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float* e = pr + hh * 16 + 4 * i;
          pk[hh * 8 + 2 * i] = pack2<T>(e[0], e[1]);
          pk[hh * 8 + 2 * i + 1] = pack2<T>(e[2], e[3]);
        }
      tmem_st_16x128b_x4(t_s, pk);
      tmem_st_16x128b_x4(t_s + half_step, pk + 8);
      tmem_st_wait();
      tc_fence_before();
      warp_arrive(p_full);

      float2 dl[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) dl[i] = *reinterpret_cast<const float2*>(dlt + 8 * i);
      ok = warp_wait(dp_full, it & 1, wc, 10, it);
      if (!ok) break;
      tc_fence_after();
      uint32_t dsp[16];
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {        // one half at a time keeps the registers in bounds
        uint32_t dpr[16];
        tmem_ld_16x256b_x4(t_dp + hh * half_step, dpr);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float* e = pr + hh * 16 + 4 * i;
          float t0, t1, t2, t3, d0, d1, d2, d3;
          add2(t0, t1, __uint_as_float(dpr[4 * i]), __uint_as_float(dpr[4 * i + 1]), dl[i].x, dl[i].y);
          add2(t2, t3, __uint_as_float(dpr[4 * i + 2]), __uint_as_float(dpr[4 * i + 3]), dl[i].x, dl[i].y);
          mul2(d0, d1, e[0], e[1], t0, t1);
          mul2(d2, d3, e[2], e[3], t2, t3);
          dsp[hh * 8 + 2 * i] = pack2<T>(d0, d1);
          dsp[hh * 8 + 2 * i + 1] = pack2<T>(d2, d3);
        }
      }
      tmem_st_16x128b_x4(t_dp, dsp);
      tmem_st_16x128b_x4(t_dp + half_step, dsp + 8);
      tmem_st_wait();
      if (stat_tid < 256 && it + 1 < n_it) {
        row_buf[(((it + 1) % kStatBufs) * 2 + (stat_tid >> 7)) * kTileQ + (stat_tid & 127)] = next_stat;
        warp_arrive(&row_ready[(it + 1) % kStatBufs]);
      }
      tc_fence_before();
      warp_arrive(ds_full);
    }

    if (ok && n_it > 0) {
      ok = warp_wait(mma_done, 0, wc, 11, n_it);
      if (ok) tc_fence_after();
    }

    // ------------------------------------------------------------- epilogue
    // dV and dK rows: group g handles head-dim columns [g*D/4, (g+1)*D/4).
    constexpr int kCols = D / 4;           // 32 (D = 128) or 16 (D = 64) columns per thread
    auto load_cols = [&](uint32_t taddr, float scale, float* o) {
      if (n_it > 0) {
        uint32_t v[kCols];
        if constexpr (kCols == 32) tmem_ld32(taddr + grp * kCols, v); else tmem_ld16(taddr + grp * kCols, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < kCols; ++i) o[i] = __uint_as_float(v[i]) * scale;
      } else {
#pragma unroll
        for (int i = 0; i < kCols; ++i) o[i] = 0.f;
      }
    };
    if (p.dkv_fp32) {
      // fp32 gradients leave through shared memory: each 32-column chunk is a
      // [128 keys][128 B] slab in the 128-byte swizzle (thread = key row, conflict-free
      // 16-byte stores) over the K/V tiles (dV) and the Q/dO ring (dK), all idle now;
      // one thread then issues a bulk tensor store per slab, or a bulk reduce-add when
      // the destination already holds a partial sum or is shared with other CTAs.
      uint8_t* stg_dv = smem + L::kKOff;
      uint8_t* stg_dk = smem + L::kRingOff;
      if (ok) {
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          float o[kCols];
          load_cols(which == 0 ? t_dv : t_dk, which == 0 ? 1.f : p.scale, o);
          uint8_t* stg = which == 0 ? stg_dv : stg_dk;
          const int col0 = grp * kCols;                       // first head-dim column of this thread
          uint8_t* row = stg + (col0 / 32) * (kTileKV * 128) + r * 128;
          const int j0 = (col0 % 32) / 4;                     // first 16-byte chunk inside the slab row
#pragma unroll
          for (int j = 0; j < kCols / 4; ++j)
            *reinterpret_cast<float4*>(row + (((j0 + j) ^ (r & 7)) << 4)) =
                make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
        }
      }
      fence_proxy_async_smem();
      warp_arrive(epi_full);
      if (threadIdx.x == 0) {
        bool go = mbar_wait(epi_full, 0, wc, 12, 0);
        go = go && !*cta_abort && !(p.q_split > 1 && n_it == 0);
        if (go) {
          const bool add = p.dkv_accumulate || p.q_split > 1;
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            if (add) {
              tma_reduce_add_4d(&tm_dv, stg_dv + c * (kTileKV * 128), c * 32, kv0, g, b);
              tma_reduce_add_4d(&tm_dk, stg_dk + c * (kTileKV * 128), c * 32, kv0, g, b);
            } else {
              tma_store_4d(&tm_dv, stg_dv + c * (kTileKV * 128), c * 32, kv0, g, b);
              tma_store_4d(&tm_dk, stg_dk + c * (kTileKV * 128), c * 32, kv0, g, b);
            }
          }
          bulk_commit_group();
          bulk_wait_all();
        }
      }
    } else if (ok) {
      const size_t row_off = (size_t)b * p.dkv_sb + (size_t)kidx * p.dkv_ss + (size_t)g * p.dkv_sh +
                             grp * kCols;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        float o[kCols];
        load_cols(which == 0 ? t_dv : t_dk, which == 0 ? 1.f : p.scale, o);
        if (!key_ok) continue;
        T* drow = reinterpret_cast<T*>(which == 0 ? p.dv : p.dk) + row_off;
        if (p.dkv_accumulate) {
#pragma unroll
          for (int i = 0; i < kCols; ++i) o[i] += static_cast<float>(drow[i]);
        }
        uint4* dst = reinterpret_cast<uint4*>(drow);
#pragma unroll
        for (int i = 0; i < kCols / 8; ++i)
          dst[i] = make_uint4(pack2<T>(o[8 * i], o[8 * i + 1]), pack2<T>(o[8 * i + 2], o[8 * i + 3]),
                              pack2<T>(o[8 * i + 4], o[8 * i + 5]),
                              pack2<T>(o[8 * i + 6], o[8 * i + 7]));
      }
    }
  }

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

// One CTA per (K/V tile, kv head, batch) leaves the last wave partly empty when that count
// is a small non-multiple of the SM count (one CTA fits per SM). With fp32 dK/dV the query
// tiles of a K/V tile can be shared by 2, 4 or 8 CTAs that reduce-add their parts:
// take the smallest split whose wave efficiency reaches 95 %, else the most efficient.
// Under a causal mask CTAs differ in length and are issued longest first, which already
// fills the tail, so only grids of less than two waves are split there. The reduce-adds of
// a split arrive in scheduling order, so a deterministic call never splits.
// SPA_BWD_QSPLIT=n forces n.
int choose_q_split(const spa_bwd_args* a, long long base_grid) {
  if (!a->dkv_fp32 || a->deterministic) return 1;
  static int forced = -1;
  if (forced < 0) {
    const char* e = getenv("SPA_BWD_QSPLIT");
    forced = e ? atoi(e) : 0;
  }
  const int q_tiles = ceil_div(a->Sq, kTileQ);
  if (forced > 0) return forced > q_tiles ? (q_tiles > 0 ? q_tiles : 1) : forced;
  const int n_sm = device_sm_count();
  if (a->causal && base_grid >= 2ll * n_sm) return 1;
  int best = 1;
  double best_eff = 0.0;
  for (int s = 1; s <= 8; s *= 2) {
    if (s > 1 && q_tiles / s < 4) break;          // keep every slice long enough to pipeline
    const long long ctas = base_grid * s;
    const long long waves = (ctas + n_sm - 1) / n_sm;
    const double eff = (double)ctas / ((double)waves * n_sm);
    if (eff > best_eff + 1e-9) { best = s; best_eff = eff; }
    if (eff >= 0.95) break;
  }
  return best;
}

template <int D, typename T>
int launch_dkv_typed(const spa_bwd_args* a, int is_bf16) {
  using L = DkvSmem<D>;
  CUtensorMap tq, tk, tv, tdo, tdk, tdv;
  if (encode_rows_map(&tq, a->q, is_bf16, D, a->Sq, a->Hq, a->B, a->q_ss, a->q_sh, a->q_sb, kTileQ))
    return SPA_ECUDA;
  if (encode_rows_map(&tdo, a->dout, is_bf16, D, a->Sq, a->Hq, a->B, a->do_ss, a->do_sh, a->do_sb,
                      kTileQ))
    return SPA_ECUDA;
  if (encode_rows_map(&tk, a->k, is_bf16, D, a->Sk, a->Hkv, a->B, a->k_ss, a->k_sh, a->k_sb, kTileKV))
    return SPA_ECUDA;
  if (encode_rows_map(&tv, a->v, is_bf16, D, a->Sk, a->Hkv, a->B, a->v_ss, a->v_sh, a->v_sb, kTileKV))
    return SPA_ECUDA;
  if (a->dkv_fp32) {
    if (encode_f32_slab_map(&tdk, a->dk, D, a->Sk, a->Hkv, a->B, kTileKV)) return SPA_ECUDA;
    if (encode_f32_slab_map(&tdv, a->dv, D, a->Sk, a->Hkv, a->B, kTileKV)) return SPA_ECUDA;
  } else {
    tdk = tq;   // never used by the kernel
    tdv = tq;
  }
  DkvParams p;
  p.B = a->B; p.Sq = a->Sq; p.Sk = a->Sk; p.Hq = a->Hq; p.Hkv = a->Hkv;
  p.causal = a->causal; p.causal_off = a->causal_off;
  p.dkv_fp32 = a->dkv_fp32; p.dkv_accumulate = a->dkv_accumulate;
  p.n_kvblk = ceil_div(a->Sk, kTileKV);
  p.chunk = (!a->causal || p.n_kvblk >= 256) ? p.n_kvblk : 1;
  p.q_split = choose_q_split(a, (long long)p.n_kvblk * a->B * a->Hkv);
  p.scale = a->scale; p.scale_log2 = a->scale * kLog2e;
  p.lse = a->lse; p.delta = a->delta; p.lse_sb = a->lse_sb; p.lse_sh = a->lse_sh;
  p.dk = a->dk; p.dv = a->dv; p.dkv_sb = a->dkv_sb; p.dkv_ss = a->dkv_ss; p.dkv_sh = a->dkv_sh;
  p.status = device_status_word();
  if (!p.status) return SPA_ECUDA;
  const int smem_bytes = L::kTotal + 1024;
  auto kern = attn_bwd_dkv_sm100_kernel<D, T>;
  int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes, "bwd dkv sm100");
  if (rc) return rc;
  const long long grid = (long long)p.n_kvblk * a->B * a->Hkv * p.q_split;
  if (grid <= 0 || grid > 0x7fffffffll) {
    set_error("bwd dkv grid out of range");
    return SPA_EINVAL;
  }
  if (p.q_split > 1 && !a->dkv_accumulate) {   // the slices add into zeroed gradients
    const size_t bytes = (size_t)a->B * a->Sk * a->Hkv * D * sizeof(float);
    cudaError_t e = cudaMemsetAsync(a->dk, 0, bytes, (cudaStream_t)a->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(a->dv, 0, bytes, (cudaStream_t)a->stream);
    if (e != cudaSuccess) {
      set_error("bwd dkv memset: %s", cudaGetErrorString(e));
      return SPA_ECUDA;
    }
  }
  kern<<<(unsigned)grid, kThreads, smem_bytes, (cudaStream_t)a->stream>>>(tq, tk, tv, tdo, tdk, tdv, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("bwd dkv sm100 launch: %s", cudaGetErrorString(e));
    return SPA_ECUDA;
  }
  return SPA_OK;
}

}  // namespace

int launch_bwd_dkv_sm100(const spa_bwd_args* a) {
  const bool bf = a->dtype == SPA_DTYPE_BF16;
  if (!a->dkv_fp32 &&
      (((uintptr_t)a->dk & 15) || ((uintptr_t)a->dv & 15) || ((a->dkv_ss * 2) & 15) ||
       ((a->dkv_sh * 2) & 15) || ((a->dkv_sb * 2) & 15))) {
    set_error("dk/dv base and strides must be 16-byte aligned");
    return SPA_EINVAL;
  }
  if (a->D == 128) {
    return bf ? launch_dkv_typed<128, __nv_bfloat16>(a, 1) : launch_dkv_typed<128, __half>(a, 0);
  } else if (a->D == 64) {
    return bf ? launch_dkv_typed<64, __nv_bfloat16>(a, 1) : launch_dkv_typed<64, __half>(a, 0);
  }
  set_error("tensor-core backward supports head_dim 64 and 128, got %d", a->D);
  return SPA_EUNSUPPORTED;
}

}  // namespace spa
