// Flash-attention backward for sm_100a (tcgen05 + TMEM + TMA), fp32 dK/dV build: the
// ring steps, whose dK|dV partial sums travel in fp32. Same main loop as
// attn_bwd_sm100.cu (which writes dK/dV in the input dtype); on top of it the query
// tiles of a K/V tile can be shared between CTAs, and dK/dV leave through shared
// memory as bulk tensor stores / reduce-adds. It is a translation unit of its own
// because the speed of these kernels proved sensitive to unrelated code compiled into
// them (S=131072 causal single-GPU backward: 770 vs 580 TFLOP/s with this epilogue merely
// present), so each file stays as measured.
//
// One CTA owns a 128-key K/V tile of one kv head and walks over every 64-row
// query tile (of every query head in its GQA group) that can see those keys.
// Scores are computed TRANSPOSED (rows = keys, columns = queries) so that the
// probabilities P^T and dS^T land in shared memory already K-major for the
// dV / dK products:
//     S^T  = K  Q^T          dP^T = V dO^T
//     P^T  = exp2(S^T*scale*log2e - lse*log2e)      (global lse)
//     dS^T = P^T * (dP^T - delta)
//     dV  += P^T dO          dK  += dS^T Q          dQ^T = K^T dS   (-> atomics)
// dV/dK stay in TMEM for the whole walk; dQ^T (rows = head dim, columns =
// queries) is drained each iteration with coalesced fp32 reductions into the
// caller's dq accumulator. The softmax scale is applied once on the way out.
//
// Algorithm source: the per-step flash backward that the ring loop of
// sp_aurora/ring_flash_attn.py:97-152 expects (the reference's own
// sp_aurora/intel_flash_attn.py:129 is a stub); formulas as in the manual
// backward of sp_aurora/intel_ulysses_attn.py:403-426.
//
// CTA = 14 warps:
//   warps 0-3   compute group A: key row per thread, query columns  0-31
//   warps 4-7   compute group B: key row per thread, query columns 32-63
//   warps 8-11  dQ drain group: head-dim lane per thread; TMEM -> shared memory
//               (fp32 [64 queries][D]) -> one TMA reduce-add into the dq accumulator
//   warp  12    TMA producer          warp 13  MMA issuer and TMEM owner
// TMEM columns: S^T [0,64) dP^T [64,128) dV [128,128+D) dK [256,256+D) dQ^T [384,448)
// P^T [448,480) dS^T [480,512) (16-bit, two per column): the A operands of the dV and
// dK products are read from TMEM, so P never touches shared memory and dS is
// written there only once (as the B operand of dQ^T). Shared-memory bandwidth
// (128 B/clk) is what bounds this kernel.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>
#include <stdlib.h>

#include <type_traits>

#include "spa_internal.h"
#include "tc05.cuh"

namespace spa {
namespace {

// Debug timeline (compile with -DSPA_TRACE, run with SPA_WAIT_PROFILE=1): block 0
// records clock64 at event `ev` of iterations [64, 72) into p.prof[ev * 8 + it - 64].
#ifdef SPA_TRACE
#define SPA_TRACE_EV(ev, it)                                                              \
  do {                                                                                    \
    if (p.prof && blockIdx.x == 0 && (it) >= 64 && (it) < 72 && (threadIdx.x & 31) == 0)  \
      p.prof[32 + (ev) * 8 + (it) - 64] = (unsigned long long)clock64();                  \
  } while (0)
#else
#define SPA_TRACE_EV(ev, it) do { } while (0)
#endif

constexpr int kTileKV = 128;
constexpr int kTileQ = 64;
constexpr int kThreads = 448;
constexpr int kWarpTma = 12, kWarpMma = 13;
constexpr int kStages = 3;
constexpr float kLog2e = 1.4426950408889634f;

constexpr uint32_t kColS = 0, kColDP = 64, kColDV = 128, kColDK = 256, kColDQ = 384;
constexpr uint32_t kColP = 448, kColDS = 480;

struct BwdParams {
  int B, Sq, Sk, Hq, Hkv;
  int causal, causal_off;
  int dkv_fp32, dkv_accumulate;
  int drain_red;   // 1: dQ leaves by per-thread red.global.add, 0: shared staging + TMA reduce
  int tmem_ops;    // 1: P^T / dS^T feed dV / dK from TMEM, 0: from shared memory
  int n_kvblk;
  int chunk;       // K/V tiles per scheduling chunk (n_kvblk or 1)
  int q_split;     // CTAs sharing one K/V tile, each over a slice of the query tiles (dK/dV by atomics)
  float scale, scale_log2;
  const float* lse;
  const float* delta;
  float* dq_acc;
  void* dk;
  void* dv;
  int* status;
  unsigned long long* prof;  // optional global array [32] of blocked cycles per wait site
};

template <int D>
struct BwdSmem {
  static constexpr int kKVSlab = kTileKV * 128;             // 16 KB
  static constexpr int kKVTile = (D / 64) * kKVSlab;         // K or V tile
  static constexpr int kQSlab = kTileQ * 128;                // 8 KB
  static constexpr int kQTile = (D / 64) * kQSlab;           // Q or dO tile
  static constexpr int kStageBytes = 2 * kQTile;             // Q + dO
  static constexpr int kPBytes = kTileKV * 128;              // 128 keys x 64 q (2 B)
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kKOff + kKVTile;
  static constexpr int kStageOff = kVOff + kKVTile;
  static constexpr int kPOff = kStageOff + kStages * kStageBytes;
  static constexpr int kDSOff = kPOff + kPBytes;
  static constexpr int kDQOff = kDSOff + kPBytes;            // dQ staging fp32 [64][D]
  static constexpr int kRowOff = kDQOff + kTileQ * D * 4;    // lse2/delta [2][2][64] floats
  static constexpr int kBarOff = kRowOff + 2 * 2 * 64 * 4;
  static constexpr int kNumBars = 1 + 2 * kStages + 9;
  static constexpr int kProfOff = kBarOff + kNumBars * 8 + 16;   // 32 x u64 wait profile
  static constexpr int kTotal = kProfOff + 32 * 8;
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
attn_bwd_f32out_sm100_kernel(const __grid_constant__ CUtensorMap tm_q,
                      const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v,
                      const __grid_constant__ CUtensorMap tm_do,
                      const __grid_constant__ CUtensorMap tm_dq,
                      const __grid_constant__ CUtensorMap tm_dk,
                      const __grid_constant__ CUtensorMap tm_dv, const BwdParams p) {
  using L = BwdSmem<D>;
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;
  uint64_t* qdo_empty = qdo_full + kStages;
  uint64_t* sdp_full = qdo_empty + kStages;
  uint64_t* sdp_free = sdp_full + 1;
  uint64_t* pds_full = sdp_free + 1;
  uint64_t* mma_done = pds_full + 1;
  uint64_t* dq_free = mma_done + 1;
  uint64_t* row_ready = dq_free + 1;
  uint64_t* stage_full = row_ready + 1;
  uint64_t* stage_free = stage_full + 1;
  uint64_t* epi_full = stage_free + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* row_buf = reinterpret_cast<float*>(smem + L::kRowOff);  // [buf][lse2|delta][64]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Work decode: K/V tiles of one chunk fastest, then kv heads, batch, chunks. The host
  // picks the chunk: all tiles (CTAs resident together then walk the Q / dO / dQ tiles of
  // the same query heads a few tiles apart and share every HBM fetch through L2:
  // S=65536 non-causal 584 -> 743 TFLOP/s), or one tile for small causal problems, where
  // longest-tile-first over all heads matters more (S=8192 causal: 807 vs 605).
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

  if (threadIdx.x < 32) reinterpret_cast<unsigned long long*>(smem + L::kProfOff)[threadIdx.x] = 0;
  if (threadIdx.x == 0) {
    *cta_abort = 0;
    mbar_init(kv_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(sdp_free, 256);
    mbar_init(pds_full, 256);
    mbar_init(mma_done, 1);
    mbar_init(dq_free, 128);
    mbar_init(row_ready, 128);
    mbar_init(stage_full, 128);
    mbar_init(stage_free, 1);
    mbar_init(epi_full, 256);
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
  unsigned long long* prof_s = reinterpret_cast<unsigned long long*>(smem + L::kProfOff);
  WaitCtx wc{p.status, cta_abort, p.prof ? prof_s : nullptr};
  const long long t_start = clock64();

  if (warp == kWarpTma) {
    // ------------------------------------------------------------------ TMA
    if (lane == 0 && n_it > 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_do);
      mbar_arrive_expect_tx(kv_full, 2 * L::kKVTile);
      for (int s = 0; s < D / 64; ++s) {
        tma_load_4d(smem + L::kKOff + s * L::kKVSlab, &tm_k, kv_full, s * 64, kv0, g, b);
        tma_load_4d(smem + L::kVOff + s * L::kKVSlab, &tm_v, kv_full, s * 64, kv0, g, b);
      }
      for (int it = 0; it < n_it; ++it) {
        const int slot = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        if (!mbar_wait(&qdo_empty[slot], ph ^ 1, wc, 0, it)) break;
        const int hq = g * G + it / n_q;
        const int q0 = (i_start + it % n_q) * kTileQ;
        uint8_t* st = smem + L::kStageOff + slot * L::kStageBytes;
        mbar_arrive_expect_tx(&qdo_full[slot], L::kStageBytes);
        for (int s = 0; s < D / 64; ++s) {
          tma_load_4d(st + s * L::kQSlab, &tm_q, &qdo_full[slot], s * 64, q0, hq, b);
          tma_load_4d(st + L::kQTile + s * L::kQSlab, &tm_do, &qdo_full[slot], s * 64, q0, hq, b);
        }
      }
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------------ MMA
    // One elected lane issues every MMA (measured faster than predicated
    // warp-uniform issue); descriptors are precomputed, offsets are constants.
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idesc_sdp = make_idesc(128, kTileQ, kBf16, false, false);
      constexpr uint32_t idesc_dkv = make_idesc(128, D, kBf16, false, true);
      constexpr uint32_t idesc_dq = make_idesc(128, kTileQ, kBf16, true, true);
      constexpr uint32_t kLboK = (D == 128) ? L::kKVSlab : 0;  // D=64: lanes 64-127 mirror 0-63
      const uint32_t k_base = smem_u32(smem + L::kKOff);
      const uint32_t v_base = smem_u32(smem + L::kVOff);
      const uint32_t st_base = smem_u32(smem + L::kStageOff);
      const uint32_t p_base = smem_u32(smem + L::kPOff);
      const uint32_t ds_base = smem_u32(smem + L::kDSOff);
      bool ok = mbar_wait(kv_full, 0, wc, 1, 0);
      tc_fence_after();

      const SmemDesc k_km = make_smem_desc(k_base, 16, 1024);        // K tile, K-major (S^T)
      const SmemDesc v_km = make_smem_desc(v_base, 16, 1024);        // V tile, K-major (dP^T)
      const SmemDesc k_mn = make_smem_desc(k_base, kLboK, 1024);     // K tile, MN-major (dQ^T)
      const SmemDesc st_km = make_smem_desc(st_base, 16, 1024);      // Q / dO stage, K-major
      const SmemDesc st_mn = make_smem_desc(st_base, L::kQSlab, 1024);  // Q / dO stage, MN-major
      const SmemDesc p_km = make_smem_desc(p_base, 16, 1024);        // P^T (shared-memory variant)
      const SmemDesc ds_km = make_smem_desc(ds_base, 16, 1024);      // dS^T as A of dK
      const SmemDesc ds_mn = make_smem_desc(ds_base, 16, 1024);      // dS^T as B of dQ^T
      // `slot` is a compile-time constant at every call site (the iteration loop is
      // unrolled over the ring period): runtime descriptor words cost issue time.
      auto issue_sdp = [&](int it, const int slot) -> bool {
        if (!mbar_wait(&qdo_full[slot], (it / kStages) & 1, wc, 2, it)) return false;
        tc_fence_after();
        const uint32_t qb = (slot * L::kStageBytes) >> 4;
        const uint32_t dob = qb + (L::kQTile >> 4);
        SPA_TRACE_EV(11, it);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t aoff = ((kk / 4) * L::kKVSlab + (kk % 4) * 32) >> 4;
          const uint32_t boff = ((kk / 4) * L::kQSlab + (kk % 4) * 32) >> 4;
          mma_ss_d(tmem_base + kColS, k_km, aoff, st_km, qb + boff, idesc_sdp, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t aoff = ((kk / 4) * L::kKVSlab + (kk % 4) * 32) >> 4;
          const uint32_t boff = ((kk / 4) * L::kQSlab + (kk % 4) * 32) >> 4;
          mma_ss_d(tmem_base + kColDP, v_km, aoff, st_km, dob + boff, idesc_sdp, kk > 0);
        }
        SPA_TRACE_EV(12, it);
        mma_commit(sdp_full);
        SPA_TRACE_EV(0, it);
        return true;
      };

      if (ok) ok = issue_sdp(0, 0);
      for (int it0 = 0; it0 < n_it && ok; it0 += kStages) {
#pragma unroll
       for (int sl = 0; sl < kStages; ++sl) {
        const int it = it0 + sl;
        if (it >= n_it || !ok) break;
        if (it + 1 < n_it) {
          ok = mbar_wait(sdp_free, it & 1, wc, 3, it);
          if (!ok) break;
          tc_fence_after();
          ok = issue_sdp(it + 1, (sl + 1) % kStages);
          if (!ok) break;
        }
        ok = mbar_wait(pds_full, it & 1, wc, 4, it);
        if (!ok) break;
        tc_fence_after();
        SPA_TRACE_EV(1, it);
        const int slot = sl;
        const uint32_t qb = (slot * L::kStageBytes) >> 4;
        const uint32_t dob = qb + (L::kQTile >> 4);
        // dV += P^T dO ; dK += dS^T Q : B = dO / Q stage read MN-major; A = P^T / dS^T
        // from TMEM (tmem_ops) or from shared memory.
        if (p.tmem_ops) {
#pragma unroll
          for (int kk = 0; kk < kTileQ / 16; ++kk)
            mma_ts_d(tmem_base + kColDV, tmem_base + kColP + kk * 8, st_mn, dob + ((kk * 2048) >> 4),
                     idesc_dkv, (it > 0 || kk > 0));
#pragma unroll
          for (int kk = 0; kk < kTileQ / 16; ++kk)
            mma_ts_d(tmem_base + kColDK, tmem_base + kColDS + kk * 8, st_mn, qb + ((kk * 2048) >> 4),
                     idesc_dkv, (it > 0 || kk > 0));
        } else {
#pragma unroll
          for (int kk = 0; kk < kTileQ / 16; ++kk)
            mma_ss_d(tmem_base + kColDV, p_km, (kk * 32) >> 4, st_mn, dob + ((kk * 2048) >> 4),
                     idesc_dkv, (it > 0 || kk > 0));
#pragma unroll
          for (int kk = 0; kk < kTileQ / 16; ++kk)
            mma_ss_d(tmem_base + kColDK, ds_km, (kk * 32) >> 4, st_mn, qb + ((kk * 2048) >> 4),
                     idesc_dkv, (it > 0 || kk > 0));
        }
        // dQ^T = K^T dS : A = K tile read MN-major (M = head dim), B = dS^T tile
        // read MN-major (N = queries), contraction over the 128 keys.
        SPA_TRACE_EV(13, it);
        if (it > 0) {
          ok = mbar_wait(dq_free, (it - 1) & 1, wc, 5, it);
          if (!ok) break;
          tc_fence_after();
        }
        SPA_TRACE_EV(14, it);
#pragma unroll
        for (int kk = 0; kk < kTileKV / 16; ++kk)
          mma_ss_d(tmem_base + kColDQ, k_mn, (kk * 2048) >> 4, ds_mn, (kk * 2048) >> 4, idesc_dq,
                   kk > 0);
        SPA_TRACE_EV(15, it);
        mma_commit(mma_done);
        SPA_TRACE_EV(2, it);
        mma_commit(&qdo_empty[slot]);
       }
      }
    }
  } else if (warp >= 8) {
    // ---------------------------------------------------------------- drain
    // dQ^T tile (TMEM lanes = head dim, columns = queries) -> shared memory as
    // fp32 [query][head dim] -> one bulk tensor reduce-add into dq_acc.
    const int quad = warp & 3;
    const int d = quad * 32 + lane;
    const int tid = threadIdx.x - 8 * 32;
    const uint32_t t_dq = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + kColDQ;
    float* stage = reinterpret_cast<float*>(smem + L::kDQOff);
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      ok = warp_wait(mma_done, it & 1, wc, 16, it);
      if (!ok) break;
      tc_fence_after();
      if (warp == 8) SPA_TRACE_EV(8, it);
      uint32_t v0[32], v1[32];
      tmem_ld32(t_dq, v0);
      tmem_ld32(t_dq + 32, v1);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(dq_free);
      if (warp == 8) SPA_TRACE_EV(9, it);
      if (p.drain_red) {
        // straight from registers: lane = head-dim index, one coalesced 128-byte
        // reduction per query row and warp
        if (d < D) {
          const int hq = g * G + it / n_q;
          const int q0 = (i_start + it % n_q) * kTileQ;
          float* base = p.dq_acc + (((size_t)b * p.Sq + q0) * p.Hq + hq) * D + d;
          const size_t rs = (size_t)p.Hq * D;
          const int nvalid = p.Sq - q0;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i < nvalid) atomicAdd(base + i * rs, __uint_as_float(v0[i]) * p.scale);
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (32 + i < nvalid) atomicAdd(base + (32 + i) * rs, __uint_as_float(v1[i]) * p.scale);
        }
        continue;
      }
      // staging buffer must have been read by the previous reduce
      ok = warp_wait(stage_free, (it & 1) ^ 1, wc, 17, it);
      if (!ok) break;
      if (d < D) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          stage[i * D + d] = __uint_as_float(v0[i]) * p.scale;
          stage[(32 + i) * D + d] = __uint_as_float(v1[i]) * p.scale;
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(stage_full);
      if (warp == 8) SPA_TRACE_EV(10, it);
      if (tid == 0) {
        ok = mbar_wait(stage_full, it & 1, wc, 18, it);
        if (ok) {
          const int hq = g * G + it / n_q;
          const int q0 = (i_start + it % n_q) * kTileQ;
          tma_reduce_add_4d(&tm_dq, stage, 0, q0, hq, b);
          bulk_commit_group();
          bulk_wait_read_all();
          mbar_arrive(stage_free);
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
    }
    if (tid == 0) bulk_wait_all();
  } else {
    // -------------------------------------------------------------- compute
    const int grp = warp >> 2;               // 0: query columns 0-31, 1: columns 32-63
    const int quad = warp & 3;
    const int r = quad * 32 + lane;          // key row in tile
    const int kidx = kv0 + r;
    const int c_base = grp * 32;
    const uint32_t lane_field = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_s = tmem_base + lane_field + kColS + c_base;
    const uint32_t t_dp = tmem_base + lane_field + kColDP + c_base;
    const uint32_t t_dv = tmem_base + lane_field + kColDV;
    const uint32_t t_dk = tmem_base + lane_field + kColDK;
    const uint32_t t_p = tmem_base + lane_field + kColP + grp * 16;
    const uint32_t t_ds = tmem_base + lane_field + kColDS + grp * 16;
    uint8_t* p_row = smem + L::kPOff;
    uint8_t* ds_row = smem + L::kDSOff;
    const bool key_ok = kidx < p.Sk;
    bool ok = true;

    // Row statistics of a query tile, fetched by group A: threads 0-63 lse
    // (pre-multiplied by log2 e), threads 64-127 delta. +inf lse makes
    // out-of-range rows give P = 0.
    auto fetch_rowstat = [&](int it) -> float {
      const int hq = g * G + it / n_q;
      const int q0 = (i_start + it % n_q) * kTileQ;
      const int c = r & 63;
      const int qi = q0 + c;
      const size_t idx = ((size_t)b * p.Hq + hq) * p.Sq + qi;
      if (r < 64) return qi < p.Sq ? p.lse[idx] * kLog2e : INFINITY;
      return qi < p.Sq ? p.delta[idx] : 0.f;
    };

    if (n_it > 0 && grp == 0) {
      row_buf[(0 * 2 + (r >> 6)) * 64 + (r & 63)] = fetch_rowstat(0);
      mbar_arrive(row_ready);
    }

    for (int it = 0; it < n_it; ++it) {
      float next_stat = 0.f;
      if (grp == 0 && it + 1 < n_it) next_stat = fetch_rowstat(it + 1);

      ok = warp_wait(sdp_full, it & 1, wc, 8, it);
      if (!ok) break;
      tc_fence_after();
      if (warp == 0) SPA_TRACE_EV(3, it);
      uint32_t sr[32], dpr[32];
      tmem_ld32(t_s, sr);
      tmem_ld32(t_dp, dpr);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(sdp_free);
      if (warp == 0) SPA_TRACE_EV(4, it);

      // Row statistics of this iteration are in shared memory once group A's
      // 128 threads have arrived (bounded, unlike a bar.sync).
      ok = warp_wait(row_ready, it & 1, wc, 9, it);
      if (!ok) break;
      const float* lse2 = row_buf + ((it & 1) * 2 + 0) * 64 + c_base;
      const float* dlt = row_buf + ((it & 1) * 2 + 1) * 64 + c_base;
      const int q0 = (i_start + it % n_q) * kTileQ;
      // Visible iff kidx <= q + off  <=>  column c >= kidx - off - q0.
      int c_min = 0;
      if (p.causal) {
        const long long cm = (long long)kidx - p.causal_off - q0 - c_base;
        c_min = (int)max(0ll, min(cm, 32ll));
      }
      if (!key_ok) c_min = 32;

      uint32_t pp[16], dsp[16];
#pragma unroll
      for (int c4 = 0; c4 < 8; ++c4) {
        const float4 l4 = *reinterpret_cast<const float4*>(lse2 + 4 * c4);
        const float4 d4 = *reinterpret_cast<const float4*>(dlt + 4 * c4);
        const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
        const float dv[4] = {d4.x, d4.y, d4.z, d4.w};
        float pv[4], dsv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = 4 * c4 + u;
          float pe = fast_exp2(fmaf(__uint_as_float(sr[c]), p.scale_log2, -lv[u]));
          if (c < c_min) pe = 0.f;
          pv[u] = pe;
          dsv[u] = pe * (__uint_as_float(dpr[c]) - dv[u]);
        }
        pp[2 * c4] = pack2<T>(pv[0], pv[1]);
        pp[2 * c4 + 1] = pack2<T>(pv[2], pv[3]);
        dsp[2 * c4] = pack2<T>(dsv[0], dsv[1]);
        dsp[2 * c4 + 1] = pack2<T>(dsv[2], dsv[3]);
      }

      if (warp == 0) SPA_TRACE_EV(5, it);
      if (it > 0) {
        // dV/dK/dQ MMAs of the previous iteration have finished reading P^T/dS^T.
        ok = warp_wait(mma_done, (it - 1) & 1, wc, 10, it);
        if (!ok) break;
        tc_fence_after();
      }
      if (warp == 0) SPA_TRACE_EV(6, it);
      if (p.tmem_ops) {
        tmem_st16(t_p, pp);
        tmem_st16(t_ds, dsp);
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t off = sw128_chunk_off(r, grp * 4 + c);
        if (!p.tmem_ops)
          *reinterpret_cast<uint4*>(p_row + off) =
              make_uint4(pp[4 * c], pp[4 * c + 1], pp[4 * c + 2], pp[4 * c + 3]);
        *reinterpret_cast<uint4*>(ds_row + off) =
            make_uint4(dsp[4 * c], dsp[4 * c + 1], dsp[4 * c + 2], dsp[4 * c + 3]);
      }
      if (p.tmem_ops) tmem_st_wait();
      if (grp == 0 && it + 1 < n_it) {
        row_buf[(((it + 1) & 1) * 2 + (r >> 6)) * 64 + (r & 63)] = next_stat;
        mbar_arrive(row_ready);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(pds_full);
      if (warp == 0) SPA_TRACE_EV(7, it);
    }

    if (ok && n_it > 0) {
      ok = warp_wait(mma_done, (n_it - 1) & 1, wc, 11, n_it);
      if (ok) tc_fence_after();
    }

    // ------------------------------------------------------------- epilogue
    // dV and dK rows: group A handles head-dim columns [0, D/2), group B the rest.
    constexpr int kHalfChunks = D / 64;  // 32-column chunks per group
    if (p.dkv_fp32) {
      // fp32 gradients leave through shared memory: each 32-column chunk is a
      // [128 keys][128 B] slab in the 128-byte swizzle (thread = key row, conflict-free
      // 16-byte stores) over the K/V tiles (dV) and the Q/dO ring (dK), all idle now;
      // one thread then issues a bulk tensor store per slab, or a bulk reduce-add when
      // the destination already holds a partial sum or is shared with other CTAs.
      uint8_t* stg_dv = smem + L::kKOff;
      uint8_t* stg_dk = smem + L::kStageOff;
      if (ok) {
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          const uint32_t taddr = which == 0 ? t_dv : t_dk;
          uint8_t* stg = which == 0 ? stg_dv : stg_dk;
#pragma unroll
          for (int cc = 0; cc < kHalfChunks; ++cc) {
            const int c = grp * kHalfChunks + cc;
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
            uint8_t* row = stg + c * (kTileKV * 128) + r * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<float4*>(row + ((j ^ (r & 7)) << 4)) =
                  make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
          }
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(epi_full);
      if (threadIdx.x == 0) {
        bool go = mbar_wait(epi_full, 0, wc, 19, 0);
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
      const size_t row_off = (((size_t)b * p.Sk + kidx) * p.Hkv + g) * D;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint32_t taddr = which == 0 ? t_dv : t_dk;
        void* dst_base = which == 0 ? p.dv : p.dk;
#pragma unroll
        for (int cc = 0; cc < kHalfChunks; ++cc) {
          const int c = grp * kHalfChunks + cc;
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

  tc_fence_before();
  __syncthreads();
  if (*cta_abort) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    __syncthreads();
  }
  if (p.prof && threadIdx.x < 32) {
    if (threadIdx.x == 31) prof_s[31] = (unsigned long long)(clock64() - t_start);  // CTA lifetime
    __syncwarp();
    atomicAdd(&p.prof[threadIdx.x], prof_s[threadIdx.x]);
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
// fills the tail, so only grids of less than two waves are split there (measured:
// S=8192, 32/8 heads: non-causal 742 -> 835 TFLOP/s with a split of 2, causal 809 -> 777).
// SPA_BWD_QSPLIT=n forces n.
int choose_q_split(const spa_bwd_args* a, long long base_grid) {
  if (!a->dkv_fp32) return 1;
  static int forced = -1;
  if (forced < 0) {
    const char* e = getenv("SPA_BWD_QSPLIT");
    forced = e ? atoi(e) : 0;
  }
  const int q_tiles = ceil_div(a->Sq, kTileQ);
  if (forced > 0) return forced > q_tiles ? (q_tiles > 0 ? q_tiles : 1) : forced;
  static int n_sm = 0;
  if (n_sm == 0) {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
      v = 148;
    n_sm = v;
  }
  if (a->causal && base_grid >= 2ll * n_sm) return 1;
  int best = 1;
  double best_eff = 0.0;
  for (int s = 1; s <= 8; s *= 2) {
    if (s > 1 && q_tiles / s < 8) break;          // keep every slice long enough to pipeline
    const long long ctas = base_grid * s;
    const long long waves = (ctas + n_sm - 1) / n_sm;
    const double eff = (double)ctas / ((double)waves * n_sm);
    if (eff > best_eff + 1e-9) { best = s; best_eff = eff; }
    if (eff >= 0.95) break;
  }
  return best;
}

template <int D, typename T>
int launch_bwd_typed(const spa_bwd_args* a, int is_bf16) {
  using L = BwdSmem<D>;
  CUtensorMap tq, tk, tv, tdo, tdq, tdk, tdv;
  if (encode_f32_rows_map(&tdq, a->dq_acc, D, a->Sq, a->Hq, a->B, kTileQ)) return SPA_ECUDA;
  if (a->dkv_fp32) {
    if (encode_f32_slab_map(&tdk, a->dk, D, a->Sk, a->Hkv, a->B, kTileKV)) return SPA_ECUDA;
    if (encode_f32_slab_map(&tdv, a->dv, D, a->Sk, a->Hkv, a->B, kTileKV)) return SPA_ECUDA;
  } else {
    tdk = tdq;   // never used by the kernel
    tdv = tdq;
  }
  if (encode_rows_map(&tq, a->q, is_bf16, D, a->Sq, a->Hq, a->B, a->q_ss, a->q_sh, a->q_sb, kTileQ))
    return SPA_ECUDA;
  if (encode_rows_map(&tdo, a->dout, is_bf16, D, a->Sq, a->Hq, a->B, a->do_ss, a->do_sh, a->do_sb,
                      kTileQ))
    return SPA_ECUDA;
  if (encode_rows_map(&tk, a->k, is_bf16, D, a->Sk, a->Hkv, a->B, a->k_ss, a->k_sh, a->k_sb, kTileKV))
    return SPA_ECUDA;
  if (encode_rows_map(&tv, a->v, is_bf16, D, a->Sk, a->Hkv, a->B, a->v_ss, a->v_sh, a->v_sb, kTileKV))
    return SPA_ECUDA;
  BwdParams p;
  p.B = a->B; p.Sq = a->Sq; p.Sk = a->Sk; p.Hq = a->Hq; p.Hkv = a->Hkv;
  p.causal = a->causal; p.causal_off = a->causal_off;
  p.dkv_fp32 = a->dkv_fp32; p.dkv_accumulate = a->dkv_accumulate;
  {
    static int mode = -1;   // SPA_BWD_DRAIN=red selects per-thread reductions instead of TMA reduce-add
    if (mode < 0) {
      const char* e = getenv("SPA_BWD_DRAIN");
      mode = (e && e[0] == 'r') ? 1 : 0;
    }
    p.drain_red = mode;
    static int tm = -1;     // SPA_BWD_TMEM=0 feeds dV/dK from shared-memory operands instead of TMEM
    if (tm < 0) {
      const char* e = getenv("SPA_BWD_TMEM");
      tm = (e && e[0] == '0') ? 0 : 1;
    }
    p.tmem_ops = tm;
  }
  p.n_kvblk = ceil_div(a->Sk, kTileKV);
  p.chunk = (!a->causal || p.n_kvblk >= 256) ? p.n_kvblk : 1;
  p.q_split = choose_q_split(a, (long long)p.n_kvblk * a->B * a->Hkv);
  p.scale = a->scale; p.scale_log2 = a->scale * kLog2e;
  p.lse = a->lse; p.delta = a->delta; p.dq_acc = a->dq_acc; p.dk = a->dk; p.dv = a->dv;
  p.status = device_status_word();
  if (!p.status) return SPA_ECUDA;
  p.prof = wait_profile_buffer();   // nullptr unless SPA_WAIT_PROFILE=1
  const int smem_bytes = L::kTotal + 1024;
  auto kern = attn_bwd_f32out_sm100_kernel<D, T>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) {
      set_error("cudaFuncSetAttribute(bwd sm100): %s", cudaGetErrorString(e));
      return SPA_ECUDA;
    }
    attr_set = true;
  }
  const long long grid = (long long)p.n_kvblk * a->B * a->Hkv * p.q_split;
  if (grid <= 0 || grid > 0x7fffffffll) {
    set_error("bwd grid out of range");
    return SPA_EINVAL;
  }
  if (p.q_split > 1 && !a->dkv_accumulate) {   // the slices add into zeroed gradients
    const size_t bytes = (size_t)a->B * a->Sk * a->Hkv * D * sizeof(float);
    cudaError_t e = cudaMemsetAsync(a->dk, 0, bytes, (cudaStream_t)a->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(a->dv, 0, bytes, (cudaStream_t)a->stream);
    if (e != cudaSuccess) {
      set_error("bwd sm100 memset: %s", cudaGetErrorString(e));
      return SPA_ECUDA;
    }
  }
  kern<<<(unsigned)grid, kThreads, smem_bytes, (cudaStream_t)a->stream>>>(tq, tk, tv, tdo, tdq, tdk, tdv, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("bwd sm100 launch: %s", cudaGetErrorString(e));
    return SPA_ECUDA;
  }
  if (p.prof) wait_profile_report("bwd", (cudaStream_t)a->stream);
  return SPA_OK;
}

}  // namespace

int launch_bwd_f32out_sm100(const spa_bwd_args* a) {
  const bool bf = a->dtype == SPA_DTYPE_BF16;
  if (!a->dkv_fp32) {
    set_error("launch_bwd_f32out_sm100 needs fp32 dk/dv");
    return SPA_EINVAL;
  }
  if (a->D == 128) {
    return bf ? launch_bwd_typed<128, __nv_bfloat16>(a, 1) : launch_bwd_typed<128, __half>(a, 0);
  } else if (a->D == 64) {
    return bf ? launch_bwd_typed<64, __nv_bfloat16>(a, 1) : launch_bwd_typed<64, __half>(a, 0);
  }
  set_error("tensor-core backward supports head_dim 64 and 128, got %d", a->D);
  return SPA_EUNSUPPORTED;
}

}  // namespace spa
