// Flash-attention backward for sm_100a, head_dim 128, 128x128 tiles.
//
// Same mathematics and work decomposition as attn_bwd_sm100.cu (one CTA per
// 128-key K/V tile of a kv head, walking the visible query tiles of its GQA
// group, transposed scores), but with 128-row query tiles so that every product
// is an N=128 MMA: 40 tcgen05.mma per 21 MFLOP instead of 64. The kernel is
// bound by the issue cost of its MMAs, so instruction count is what matters.
//
// The 512 TMEM columns are time-shared; overwrites are protected by the
// in-order execution of one thread's tcgen05.mma stream plus mbarriers:
//   R0 [  0,128) S^T(i) fp32, then P^T(i) 16-bit in [0,32) and [64,96)
//   R1 [128,256) dP^T(i) fp32, then dS^T(i) 16-bit in [128,160) and [192,224),
//                then dQ^T(i) fp32 (all 128 columns)
//   R2 [256,384) dV accumulator          R3 [384,512) dK accumulator
// Issue order per query tile i (single issuing thread):
//   wait P/dS(i) -> dV(i) [A=P^T TMEM] -> S^T(i+1) -> dK(i) [A=dS^T TMEM]
//   -> dQ^T(i) -> wait dQ^T(i) drained -> dP^T(i+1)
// Shared memory (no slack: 224 KB of tiles): K, V (32 KB each), a ring of four
// 32 KB Q/dO tiles, and one 32 KB buffer that holds dS^T (B operand of dQ^T) and
// is then reused as the fp32 staging tile of the dQ reduce-add.
//
// Warps: 0-3 compute A (query columns 0-63), 4-7 compute B (64-127), 8-11 dQ
// drain, 12 TMA producer, 13 MMA issuer / TMEM owner.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>
#include <stdlib.h>

#include <type_traits>

#include "spa_internal.h"
#include "tc05.cuh"

namespace spa {
namespace {

constexpr int kT = 128;              // tile edge (keys and queries)
constexpr int kD = 128;              // head dim
constexpr int kThreads = 448;
constexpr int kWarpTma = 12, kWarpMma = 13;
constexpr int kRing = 4;             // Q/dO tile ring: Q_i -> slots 0,2 ; dO_i -> slots 1,3
constexpr float kLog2e = 1.4426950408889634f;
constexpr uint32_t kR0 = 0, kR1 = 128, kR2 = 256, kR3 = 384;

struct Bwd128Params {
  int B, Sq, Sk, Hq, Hkv;
  int causal, causal_off;
  int dkv_fp32, dkv_accumulate;
  float scale, scale_log2;
  const float* lse;
  const float* delta;
  void* dk;
  void* dv;
  int* status;
};

struct Smem128 {
  static constexpr int kSlab = kT * 128;                 // 128 rows x 128 B
  static constexpr int kTile = 2 * kSlab;                // 32 KB
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kKOff + kTile;
  static constexpr int kRingOff = kVOff + kTile;
  static constexpr int kDSOff = kRingOff + kRing * kTile;   // dS^T, then dQ staging
  static constexpr int kRowOff = kDSOff + kTile;            // lse2/delta [2 bufs][2][128] floats
  static constexpr int kBarOff = kRowOff + 2 * 2 * kT * 4;
  static constexpr int kNumBars = 1 + 2 * kRing + 9;
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

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
attn_bwd128_sm100_kernel(const __grid_constant__ CUtensorMap tm_q,
                         const __grid_constant__ CUtensorMap tm_k,
                         const __grid_constant__ CUtensorMap tm_v,
                         const __grid_constant__ CUtensorMap tm_do,
                         const __grid_constant__ CUtensorMap tm_dq, const Bwd128Params p) {
  using L = Smem128;
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* kv_full = bars;
  uint64_t* tile_full = bars + 1;               // [kRing]
  uint64_t* tile_empty = tile_full + kRing;     // [kRing]
  uint64_t* s_full = tile_empty + kRing;
  uint64_t* dp_full = s_full + 1;
  uint64_t* pds_full = dp_full + 1;
  uint64_t* mma_done = pds_full + 1;
  uint64_t* dq_free = mma_done + 1;
  uint64_t* stage_free = dq_free + 1;           // dS/staging buffer free for the next dS^T
  uint64_t* half_free = stage_free + 1;         // drain-internal: staging half consumed
  uint64_t* stage_full = half_free + 1;
  uint64_t* row_ready = stage_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* row_buf = reinterpret_cast<float*>(smem + L::kRowOff);   // [buf][lse2|delta][128]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  int w = blockIdx.x;
  const int g = w % p.Hkv;
  w /= p.Hkv;
  const int b = w % p.B;
  w /= p.B;
  const int kv0 = w * kT;
  const int G = p.Hq / p.Hkv;

  const int i_end = (p.Sq + kT - 1) / kT;
  int i_start = 0;
  if (p.causal) {
    const long long first_q = (long long)kv0 - p.causal_off;
    if (first_q > 0) i_start = (int)min((long long)i_end, first_q / kT);
  }
  const int n_q = i_end - i_start;
  const int n_it = n_q * G;

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    if (smem_u32(smem) & 1023u) {   // swizzled tiles need a 1024-byte aligned base
      if (atomicCAS(p.status, 0, 2) == 0) p.status[1] = blockIdx.x;
      *cta_abort = 1;
    }
    mbar_init(kv_full, 1);
    for (int i = 0; i < kRing; ++i) {
      mbar_init(&tile_full[i], 1);
      mbar_init(&tile_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(pds_full, 256);
    mbar_init(mma_done, 1);
    mbar_init(dq_free, 128);
    mbar_init(stage_free, 1);
    mbar_init(half_free, 1);
    mbar_init(stage_full, 128);
    mbar_init(row_ready, 128);
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
  WaitCtx wc{p.status, cta_abort, nullptr};
  const bool run = n_it > 0 && !*cta_abort;

  auto tile_hq = [&](int it) { return g * G + it / n_q; };
  auto tile_q0 = [&](int it) { return (i_start + it % n_q) * kT; };

  if (warp == kWarpTma) {
    // ------------------------------------------------------------------ TMA
    if (lane == 0 && run) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_do);
      mbar_arrive_expect_tx(kv_full, 2 * L::kTile);
      for (int s = 0; s < 2; ++s) {
        tma_load_4d(smem + L::kKOff + s * L::kSlab, &tm_k, kv_full, s * 64, kv0, g, b);
        tma_load_4d(smem + L::kVOff + s * L::kSlab, &tm_v, kv_full, s * 64, kv0, g, b);
      }
      for (int n = 0; n < 2 * n_it; ++n) {       // n = 2*it: Q tile, 2*it+1: dO tile
        const int slot = n % kRing;
        if (!mbar_wait(&tile_empty[slot], ((n / kRing) & 1) ^ 1, wc, 0, n)) break;
        const int it = n >> 1;
        uint8_t* dst = smem + L::kRingOff + slot * L::kTile;
        mbar_arrive_expect_tx(&tile_full[slot], L::kTile);
        const CUtensorMap* tm = (n & 1) ? &tm_do : &tm_q;
        for (int s = 0; s < 2; ++s)
          tma_load_4d(dst + s * L::kSlab, tm, &tile_full[slot], s * 64, tile_q0(it), tile_hq(it), b);
      }
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------------ MMA
    if (lane == 0 && run) {
      constexpr uint32_t id_kk = make_idesc(128, 128, kBf16, false, false);   // S^T, dP^T
      constexpr uint32_t id_kmn = make_idesc(128, 128, kBf16, false, true);   // dV, dK (A from TMEM)
      constexpr uint32_t id_mnmn = make_idesc(128, 128, kBf16, true, true);   // dQ^T
      const uint32_t ring_base = smem_u32(smem + L::kRingOff);
      const SmemDesc k_km = make_smem_desc(smem_u32(smem + L::kKOff), 16, 1024);
      const SmemDesc v_km = make_smem_desc(smem_u32(smem + L::kVOff), 16, 1024);
      const SmemDesc k_mn = make_smem_desc(smem_u32(smem + L::kKOff), L::kSlab, 1024);
      const SmemDesc ring_km = make_smem_desc(ring_base, 16, 1024);
      const SmemDesc ring_mn = make_smem_desc(ring_base, L::kSlab, 1024);
      const SmemDesc ds_mn = make_smem_desc(smem_u32(smem + L::kDSOff), L::kSlab, 1024);
      bool ok = mbar_wait(kv_full, 0, wc, 1, 0);
      tc_fence_after();

      // `slot` arguments are compile-time constants at every call site.
      auto wait_tile = [&](int n, const int slot) -> bool {
        const bool r = mbar_wait(&tile_full[slot], (n / kRing) & 1, wc, 2, n);
        tc_fence_after();
        return r;
      };
      auto issue_st = [&](int it, const int slot) -> bool {      // S^T(it) = K Q^T
        if (!wait_tile(2 * it, slot)) return false;
        const uint32_t tb = (slot * L::kTile) >> 4;
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t off = ((kk / 4) * L::kSlab + (kk % 4) * 32) >> 4;
          mma_ss_d(tmem_base + kR0, k_km, off, ring_km, tb + off, id_kk, kk > 0);
        }
        mma_commit(s_full);
        return true;
      };
      auto issue_dpt = [&](int it, const int slot) -> bool {     // dP^T(it) = V dO^T
        if (!wait_tile(2 * it + 1, slot)) return false;
        const uint32_t tb = (slot * L::kTile) >> 4;
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t off = ((kk / 4) * L::kSlab + (kk % 4) * 32) >> 4;
          mma_ss_d(tmem_base + kR1, v_km, off, ring_km, tb + off, id_kk, kk > 0);
        }
        mma_commit(dp_full);
        return true;
      };

      if (ok) ok = issue_st(0, 0);
      if (ok) ok = issue_dpt(0, 1);
      for (int it0 = 0; it0 < n_it && ok; it0 += 2) {
#pragma unroll
        for (int ii = 0; ii < 2; ++ii) {
          const int it = it0 + ii;
          if (it >= n_it || !ok) break;
          const int q_slot = 2 * ii, do_slot = 2 * ii + 1;
          ok = mbar_wait(pds_full, it & 1, wc, 4, it);
          if (!ok) break;
          tc_fence_after();
          // dV += P^T dO : A = P^T in R0 [0,32) (queries 0-63) and [64,96) (64-127)
          {
            const uint32_t tb = (do_slot * L::kTile) >> 4;
#pragma unroll
            for (int kk = 0; kk < kT / 16; ++kk)
              mma_ts_d(tmem_base + kR2, tmem_base + kR0 + (kk / 4) * 64 + (kk % 4) * 8, ring_mn,
                       tb + ((kk * 2048) >> 4), id_kmn, (it > 0 || kk > 0));
          }
          // S^T(it+1) may now overwrite R0: dV(it) is ahead of it in the pipe.
          if (it + 1 < n_it) {
            ok = issue_st(it + 1, (2 * ii + 2) % kRing);
            if (!ok) break;
          }
          // dK += dS^T Q : A = dS^T in R1 [0,32) and [64,96)
          {
            const uint32_t tb = (q_slot * L::kTile) >> 4;
#pragma unroll
            for (int kk = 0; kk < kT / 16; ++kk)
              mma_ts_d(tmem_base + kR3, tmem_base + kR1 + (kk / 4) * 64 + (kk % 4) * 8, ring_mn,
                       tb + ((kk * 2048) >> 4), id_kmn, (it > 0 || kk > 0));
          }
          // dQ^T = K^T dS into R1 (dK(it) is ahead of it in the pipe).
#pragma unroll
          for (int kk = 0; kk < kT / 16; ++kk)
            mma_ss_d(tmem_base + kR1, k_mn, (kk * 2048) >> 4, ds_mn, (kk * 2048) >> 4, id_mnmn, kk > 0);
          mma_commit(mma_done);
          mma_commit(&tile_empty[q_slot]);
          mma_commit(&tile_empty[do_slot]);
          if (it + 1 < n_it) {
            ok = mbar_wait(dq_free, it & 1, wc, 5, it);     // dQ^T(it) is in the drain's registers
            if (!ok) break;
            tc_fence_after();
            ok = issue_dpt(it + 1, (2 * ii + 3) % kRing);
            if (!ok) break;
          }
        }
      }
    }
  } else if (warp >= 8) {
    // ---------------------------------------------------------------- drain
    const int quad = warp & 3;
    const int d = quad * 32 + lane;                       // head-dim index = TMEM lane
    const int tid = threadIdx.x - 8 * 32;
    const uint32_t t_dq = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + kR1;
    float* stage = reinterpret_cast<float*>(smem + L::kDSOff);     // fp32 [64 queries][128]
    bool ok = run;
    int halves = 0;                                       // completed staging halves
    for (int it = 0; ok && it < n_it; ++it) {
      ok = warp_wait(mma_done, it & 1, wc, 16, it);
      if (!ok) break;
      tc_fence_after();
      uint32_t v[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(t_dq + c * 32, v + c * 32);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(dq_free);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        if (halves > 0) {   // previous reduce must have read the staging tile
          ok = warp_wait(half_free, (halves - 1) & 1, wc, 17, it);
          if (!ok) break;
        }
#pragma unroll
        for (int i = 0; i < 64; ++i) stage[i * kD + d] = __uint_as_float(v[half * 64 + i]) * p.scale;
        fence_proxy_async_smem();
        mbar_arrive(stage_full);
        if (tid == 0) {
          ok = mbar_wait(stage_full, halves & 1, wc, 18, it);
          if (ok) {
            tma_reduce_add_4d(&tm_dq, stage, 0, tile_q0(it) + half * 64, tile_hq(it), b);
            bulk_commit_group();
            bulk_wait_read_all();
            mbar_arrive(half_free);
            if (half == 1) mbar_arrive(stage_free);
          }
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ++halves;
      }
    }
    if (tid == 0) bulk_wait_all();
  } else {
    // -------------------------------------------------------------- compute
    const int grp = warp >> 2;               // 0: query columns 0-63, 1: 64-127
    const int quad = warp & 3;
    const int r = quad * 32 + lane;          // key row in tile
    const int kidx = kv0 + r;
    const int cb = grp * 64;
    const uint32_t lane_field = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_s = tmem_base + lane_field + kR0 + cb;    // S^T columns of this group
    const uint32_t t_dp = tmem_base + lane_field + kR1 + cb;
    const uint32_t t_p = tmem_base + lane_field + kR0 + cb;    // P^T goes over the group's own S^T
    const uint32_t t_ds = tmem_base + lane_field + kR1 + cb;
    uint8_t* ds_slab = smem + L::kDSOff + grp * L::kSlab;      // [128 keys][64 queries] 16-bit
    const bool key_ok = kidx < p.Sk;
    bool ok = run;

    // Row statistics of a query tile, fetched by group A (thread r -> query q0 + r).
    float nl = 0.f, nd = 0.f;
    auto fetch_rowstat = [&](int it) {
      const int qi = tile_q0(it) + r;
      const size_t idx = ((size_t)b * p.Hq + tile_hq(it)) * p.Sq + qi;
      nl = qi < p.Sq ? p.lse[idx] * kLog2e : INFINITY;   // +inf: out-of-range rows give P = 0
      nd = qi < p.Sq ? p.delta[idx] : 0.f;
    };
    if (ok && grp == 0) {
      fetch_rowstat(0);
      row_buf[(0 * 2 + 0) * kT + r] = nl;
      row_buf[(0 * 2 + 1) * kT + r] = nd;
      mbar_arrive(row_ready);
    }

    for (int it = 0; ok && it < n_it; ++it) {
      if (grp == 0 && it + 1 < n_it) fetch_rowstat(it + 1);
      const float* lse2 = row_buf + ((it & 1) * 2 + 0) * kT + cb;
      const float* dlt = row_buf + ((it & 1) * 2 + 1) * kT + cb;
      // Visible iff key <= q + off  <=>  column c >= key - off - q0 - cb.
      int c_min = 0;
      if (p.causal) {
        const long long cm = (long long)kidx - p.causal_off - tile_q0(it) - cb;
        c_min = (int)max(0ll, min(cm, 64ll));
      }
      if (!key_ok) c_min = 64;

      ok = warp_wait(s_full, it & 1, wc, 8, it);
      if (!ok) break;
      tc_fence_after();
      float pf[64];
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t sr[32];
        tmem_ld32(t_s + ch * 32, sr);
        tmem_ld_wait();
        if (ch == 0) {
          ok = warp_wait(row_ready, it & 1, wc, 9, it);
          if (!ok) break;
        }
        uint32_t pk[16];
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const float4 l4 = *reinterpret_cast<const float4*>(lse2 + ch * 32 + 4 * c4);
          const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int c = ch * 32 + 4 * c4 + u;
            float pe = fast_exp2(fmaf(__uint_as_float(sr[4 * c4 + u]), p.scale_log2, -lv[u]));
            if (c < c_min) pe = 0.f;
            pf[c] = pe;
          }
          pk[2 * c4] = pack2<T>(pf[ch * 32 + 4 * c4], pf[ch * 32 + 4 * c4 + 1]);
          pk[2 * c4 + 1] = pack2<T>(pf[ch * 32 + 4 * c4 + 2], pf[ch * 32 + 4 * c4 + 3]);
        }
        // packed P^T of columns [32ch, 32ch+32) -> 16 columns inside the part of
        // S^T this thread has already consumed
        tmem_st16(t_p + ch * 16, pk);
      }
      if (!ok) break;

      ok = warp_wait(dp_full, it & 1, wc, 10, it);
      if (!ok) break;
      tc_fence_after();
      if (it > 0) {   // the drain is done with the shared dS / staging buffer
        ok = warp_wait(stage_free, (it - 1) & 1, wc, 11, it);
        if (!ok) break;
      }
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t dr[32];
        tmem_ld32(t_dp + ch * 32, dr);
        tmem_ld_wait();
        uint32_t dk_[16];
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const float4 d4 = *reinterpret_cast<const float4*>(dlt + ch * 32 + 4 * c4);
          const float dv[4] = {d4.x, d4.y, d4.z, d4.w};
          float ds[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            ds[u] = pf[ch * 32 + 4 * c4 + u] * (__uint_as_float(dr[4 * c4 + u]) - dv[u]);
          dk_[2 * c4] = pack2<T>(ds[0], ds[1]);
          dk_[2 * c4 + 1] = pack2<T>(ds[2], ds[3]);
        }
        tmem_st16(t_ds + ch * 16, dk_);
#pragma unroll
        for (int c = 0; c < 4; ++c)
          *reinterpret_cast<uint4*>(ds_slab + sw128_chunk_off(r, ch * 4 + c)) =
              make_uint4(dk_[4 * c], dk_[4 * c + 1], dk_[4 * c + 2], dk_[4 * c + 3]);
      }
      if (grp == 0 && it + 1 < n_it) {
        row_buf[(((it + 1) & 1) * 2 + 0) * kT + r] = nl;
        row_buf[(((it + 1) & 1) * 2 + 1) * kT + r] = nd;
        mbar_arrive(row_ready);
      }
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(pds_full);
    }

    if (ok && n_it > 0) {
      ok = warp_wait(mma_done, (n_it - 1) & 1, wc, 12, n_it);
      if (ok) tc_fence_after();
    }

    // dV (R2) and dK (R3) rows: group A writes head-dim columns [0,64), group B the rest.
    if (ok || (n_it == 0 && !*cta_abort)) {
      const size_t row_off = (((size_t)b * p.Sk + kidx) * p.Hkv + g) * kD;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint32_t taddr = tmem_base + lane_field + (which == 0 ? kR2 : kR3);
        void* dst_base = which == 0 ? p.dv : p.dk;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int c = grp * 2 + cc;
          float o[32];
          if (n_it > 0) {
            uint32_t v[32];
            tmem_ld32(taddr + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __uint_as_float(v[i]) * (which == 0 ? 1.f : p.scale);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0.f;
          }
          if (!key_ok) continue;
          if (p.dkv_fp32) {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(dst_base) + row_off + c * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float4 x = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
              if (p.dkv_accumulate) {
                const float4 y = dst[i];
                x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
              }
              dst[i] = x;
            }
          } else {
            T* drow = reinterpret_cast<T*>(dst_base) + row_off + c * 32;
            if (p.dkv_accumulate) {
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] += static_cast<float>(drow[i]);
            }
            uint4* dst = reinterpret_cast<uint4*>(drow);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              dst[i] = make_uint4(pack2<T>(o[8 * i], o[8 * i + 1]), pack2<T>(o[8 * i + 2], o[8 * i + 3]),
                                  pack2<T>(o[8 * i + 4], o[8 * i + 5]),
                                  pack2<T>(o[8 * i + 6], o[8 * i + 7]));
          }
        }
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

template <typename T>
int launch_typed(const spa_bwd_args* a, int is_bf16) {
  using L = Smem128;
  CUtensorMap tq, tk, tv, tdo, tdq;
  if (encode_f32_rows_map(&tdq, a->dq_acc, kD, a->Sq, a->Hq, a->B, 64)) return SPA_ECUDA;
  if (encode_rows_map(&tq, a->q, is_bf16, kD, a->Sq, a->Hq, a->B, a->q_ss, a->q_sh, a->q_sb, kT))
    return SPA_ECUDA;
  if (encode_rows_map(&tdo, a->dout, is_bf16, kD, a->Sq, a->Hq, a->B, a->do_ss, a->do_sh, a->do_sb, kT))
    return SPA_ECUDA;
  if (encode_rows_map(&tk, a->k, is_bf16, kD, a->Sk, a->Hkv, a->B, a->k_ss, a->k_sh, a->k_sb, kT))
    return SPA_ECUDA;
  if (encode_rows_map(&tv, a->v, is_bf16, kD, a->Sk, a->Hkv, a->B, a->v_ss, a->v_sh, a->v_sb, kT))
    return SPA_ECUDA;
  Bwd128Params p;
  p.B = a->B; p.Sq = a->Sq; p.Sk = a->Sk; p.Hq = a->Hq; p.Hkv = a->Hkv;
  p.causal = a->causal; p.causal_off = a->causal_off;
  p.dkv_fp32 = a->dkv_fp32; p.dkv_accumulate = a->dkv_accumulate;
  p.scale = a->scale; p.scale_log2 = a->scale * kLog2e;
  p.lse = a->lse; p.delta = a->delta; p.dk = a->dk; p.dv = a->dv;
  p.status = device_status_word();
  if (!p.status) return SPA_ECUDA;
  const int smem_bytes = L::kTotal;
  auto kern = attn_bwd128_sm100_kernel<T>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) {
      set_error("cudaFuncSetAttribute(bwd128 sm100, %d bytes): %s", smem_bytes, cudaGetErrorString(e));
      return SPA_ECUDA;
    }
    attr_set = true;
  }
  const long long grid = (long long)ceil_div(a->Sk, kT) * a->B * a->Hkv;
  if (grid <= 0 || grid > 0x7fffffffll) {
    set_error("bwd grid out of range");
    return SPA_EINVAL;
  }
  kern<<<(unsigned)grid, kThreads, smem_bytes, (cudaStream_t)a->stream>>>(tq, tk, tv, tdo, tdq, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("bwd128 sm100 launch: %s", cudaGetErrorString(e));
    return SPA_ECUDA;
  }
  return SPA_OK;
}

}  // namespace

int launch_bwd128_sm100(const spa_bwd_args* a) {
  return a->dtype == SPA_DTYPE_BF16 ? launch_typed<__nv_bfloat16>(a, 1) : launch_typed<__half>(a, 0);
}

}  // namespace spa
