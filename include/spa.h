/*
 * libspaurora_sm100 -- C ABI of the B200 (sm_100a) sequence-parallel attention
 * hot path. Plain pointers, sizes and a cudaStream_t passed as void*; no torch
 * types. Every function returns 0 on success or a negative SPA_E* code and
 * leaves a message for spa_last_error(). Nothing here allocates device memory
 * except the 16-byte per-device status word created on first use.
 *
 * Tensors are [B, S, H, D] with the last dimension contiguous; the other
 * three strides are given in ELEMENTS so packed views (kv[:, :, 0], qkv[:, :, i])
 * are passed without a copy. lse/delta are fp32 [B, Hq, Sq], rows contiguous, with
 * batch and head strides in elements (both zero = contiguous).
 *
 * Each entry point names the reference interface it stands in for
 * (paths are relative to the sp-aurora project root).
 */
#ifndef SPA_H_
#define SPA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPA_OK 0
#define SPA_EINVAL (-1)     /* bad argument, nothing was launched            */
#define SPA_ECUDA (-2)      /* a CUDA runtime/driver call failed             */
#define SPA_ETIMEOUT (-3)   /* a bounded device-side wait gave up            */
#define SPA_EUNSUPPORTED (-4)

#define SPA_DTYPE_F32 0
#define SPA_DTYPE_BF16 1
#define SPA_DTYPE_F16 2

/*
 * Local flash-attention forward for one ring step, with the out/lse merge of
 * the previous steps fused into the epilogue.
 *
 * Replaces: sp_aurora/intel_flash_attn.py:18 intel_flash_attn_forward,
 *           sp_aurora/intel_flash_attn_sycl.py:40 intel_flash_attn_forward_sycl
 *           -> sp_aurora/sycl_bindings/bindings.cpp:50 flash_attn_forward_py,
 *           and the merge sp_aurora/utils.py:47 _update_out_and_lse.
 *
 * out = softmax(scale * Q K^T + mask) V ; lse = logsumexp(scale * Q K^T + mask).
 * causal != 0: key j is visible to query i iff j <= i + causal_off (causal_off
 * = 0 is the reference's top-left-aligned triu(diagonal=1) mask).
 * merge_prev != 0: (out_acc, lse) hold the running result of earlier ring
 * steps and are combined with this block:
 *     lse' = logaddexp(lse, lse_blk)
 *     out' = exp(lse - lse') * out_acc + exp(lse_blk - lse') * out_blk
 * The combined rows are written to out_acc (fp32, if non-NULL) and to out
 * (element type `dtype`, if non-NULL); lse is always written.
 * fp32 inputs run on the CUDA-core kernel (1e-4 parity), bf16/fp16 on the
 * tcgen05 tensor-core kernel.
 */
typedef struct spa_fwd_args {
  const void* q; int64_t q_sb, q_ss, q_sh;
  const void* k; int64_t k_sb, k_ss, k_sh;
  const void* v; int64_t v_sb, v_ss, v_sh;
  void* out;     int64_t o_sb, o_ss, o_sh;   /* may be NULL                       */
  float* out_acc;                            /* [B,Sq,Hq,D] contiguous, may be NULL */
  float* lse;                                /* [B,Hq,Sq], see lse_sb / lse_sh    */
  int64_t lse_sb, lse_sh;                    /* lse strides in elements; 0,0 = contiguous */
  int32_t B, Sq, Sk, Hq, Hkv, D;
  int32_t dtype;
  int32_t causal;
  int32_t causal_off;
  int32_t merge_prev;
  float scale;                               /* softmax scale, > 0                */
  void* stream;                              /* cudaStream_t                      */
} spa_fwd_args;

int spa_attn_fwd(const spa_fwd_args* args);

/*
 * delta[b,h,s] = sum_d dout[b,s,h,d] * out[b,s,h,d]  (fp32), the row term of
 * the softmax backward. No reference counterpart as a separate function: the
 * reference obtains it implicitly through autograd
 * (sp_aurora/intel_ring_flash_attn.py:229-248).
 */
int spa_bwd_delta(const void* out, int64_t o_sb, int64_t o_ss, int64_t o_sh,
                  const void* dout, int64_t do_sb, int64_t do_ss, int64_t do_sh,
                  float* delta, int32_t B, int32_t S, int32_t H, int32_t D, int32_t dtype,
                  void* stream);

/*
 * Local flash-attention backward for one ring step, using the GLOBAL lse and
 * delta of the full sequence.
 *
 * Replaces: sp_aurora/intel_flash_attn.py:129 intel_flash_attn_backward (a stub
 *           in the reference), sp_aurora/sycl_bindings/bindings.cpp:275
 *           flash_attn_backward_py (returns zeros), and the per-step body of
 *           sp_aurora/intel_ring_flash_attn.py:153 intel_ring_flash_attn_backward
 *           (intended algorithm: sp_aurora/ring_flash_attn.py:97-152).
 *
 * P = exp(scale * Q K^T + mask - lse);  dV = P^T dO;  dP = dO V^T;
 * dS = P * (dP - delta);  dQ = scale * dS K;  dK = scale * dS^T Q.
 *
 * dQ: the block's dQ is combined with the running sum of earlier ring steps.
 *   dq_overwrite == 0: total = dq_acc + dQ (dq_acc holds the earlier steps' sum);
 *   dq_overwrite != 0: total = dQ (dq_acc is not read and need not be initialised).
 *   The total is written to dq (element type `dtype`, strided) if dq is non-NULL and
 *   to dq_acc (fp32 [B,Sq,Hq,D] contiguous) if dq_acc is non-NULL. At least one of the
 *   two is required; dq_acc is required when dq_overwrite == 0.
 * dK/dV are [B,Sk,Hkv,D]: fp32 contiguous when dkv_fp32 != 0 (the ring's travelling
 * partial sums), else element type `dtype` with the strides dkv_sb/ss/sh (all zero =
 * contiguous). With dkv_accumulate != 0 the block result is added to what dk/dv
 * already hold (sp_aurora/ring_flash_attn.py:139-141), otherwise it overwrites them.
 * deterministic != 0 restricts the launcher to paths whose floating-point summation
 * order does not depend on scheduling (results are then bitwise reproducible).
 * The backward runs as two kernels, a K/V-stationary pass (dK, dV) and a
 * query-stationary pass (dQ). passes selects them: SPA_BWD_BOTH, SPA_BWD_DQ_ONLY (dk, dv
 * may be NULL) or SPA_BWD_DKV_ONLY (dq, dq_acc may be NULL), so that a ring step can
 * run its dQ pass while the travelling dK|dV partial is still in flight.
 */
#define SPA_BWD_BOTH 0
#define SPA_BWD_DQ_ONLY 1
#define SPA_BWD_DKV_ONLY 2

typedef struct spa_bwd_args {
  const void* q;    int64_t q_sb, q_ss, q_sh;
  const void* k;    int64_t k_sb, k_ss, k_sh;
  const void* v;    int64_t v_sb, v_ss, v_sh;
  const void* dout; int64_t do_sb, do_ss, do_sh;
  const float* lse;      /* [B,Hq,Sq], strides lse_sb / lse_sh */
  const float* delta;    /* same layout as lse */
  int64_t lse_sb, lse_sh;
  float* dq_acc;         /* [B,Sq,Hq,D] fp32 contiguous, may be NULL (see above) */
  void* dq;              /* [B,Sq,Hq,D] element type `dtype`, may be NULL */
  int64_t dq_sb, dq_ss, dq_sh;
  int32_t dq_overwrite;
  void* dk;              /* [B,Sk,Hkv,D] */
  void* dv;
  int64_t dkv_sb, dkv_ss, dkv_sh;
  int32_t dkv_fp32;
  int32_t dkv_accumulate;
  int32_t deterministic;
  int32_t passes;
  int32_t B, Sq, Sk, Hq, Hkv, D;
  int32_t dtype;
  int32_t causal;
  int32_t causal_off;
  float scale;
  void* stream;
} spa_bwd_args;

int spa_attn_bwd(const spa_bwd_args* args);

/*
 * Backward pass for callers that cannot allocate device memory.
 *
 * No counterpart in the reference. Who needs it: code that runs where every
 * byte of the GPU already belongs to someone else's pool, or that may not call
 * into the CUDA allocator at all (a fixed-budget service, a thread that must
 * not block on allocator locks). spa_attn_bwd makes such a caller bring a
 * scratch buffer (delta, the row sums of dO * O); this entry keeps it in a fixed
 * array inside the library instead. The caller passes only inputs
 * (q, k, v, out, dout, lse) and outputs (dq, dk, dv: element type `dtype`,
 * contiguous [B,Sq,Hq,D] / [B,Sk,Hkv,D], overwritten).
 *
 * - It calls no cudaMalloc/cudaFree and no allocating library routine.
 * - Limit: B*Sq*Hq*4 bytes must fit in SPA_NOALLOC_SCRATCH_BYTES; larger problems
 *   are rejected with SPA_EINVAL. Every GPU that loads the library holds that
 *   array until the process exits.
 * - The first call on a device looks up the array's device address; make that
 *   first call before starting any stream capture.
 * - All calls share the one array, which keeps the last call's contents. Nothing in
 *   it has to start at zero (each call writes every delta value it later reads), but
 *   calls that overlap on the same GPU, e.g. from two streams, race. Serialise them.
 * - bf16/fp16 with head_dim 64 or 128 run on the tensor-core kernels, everything
 *   else on the fp32 CUDA-core kernels, as in spa_attn_bwd; results are bitwise
 *   reproducible.
 */
#define SPA_NOALLOC_SCRATCH_BYTES (16u << 20)

typedef struct spa_bwd_noalloc_args {
  const void* q;    int64_t q_sb, q_ss, q_sh;
  const void* k;    int64_t k_sb, k_ss, k_sh;
  const void* v;    int64_t v_sb, v_ss, v_sh;
  const void* out;  int64_t o_sb, o_ss, o_sh;
  const void* dout; int64_t do_sb, do_ss, do_sh;
  const float* lse;      /* [B,Hq,Sq] */
  void* dq;              /* [B,Sq,Hq,D] contiguous */
  void* dk;              /* [B,Sk,Hkv,D] contiguous */
  void* dv;
  int32_t B, Sq, Sk, Hq, Hkv, D;
  int32_t dtype;
  int32_t causal;
  int32_t causal_off;
  float scale;
  void* stream;
} spa_bwd_noalloc_args;

int spa_attn_bwd_noalloc(const spa_bwd_noalloc_args* args);

/* Size of the built-in scratch array, in bytes. */
int64_t spa_noalloc_scratch_bytes(void);

/*
 * Stand-alone out/lse merge (the fused epilogue of spa_attn_fwd does the same
 * arithmetic; this entry exists for callers that hold two partial results).
 * Replaces: sp_aurora/utils.py:109 update_out_and_lse / :47 _update_out_and_lse.
 * out_acc fp32 [B,S,H,D] and lse fp32 [B,H,S] are updated in place from
 * block_out (element type `dtype`, strided) and block_lse [B,H,S].
 */
int spa_merge(float* out_acc, float* lse, const void* block_out, int64_t bo_sb, int64_t bo_ss,
              int64_t bo_sh, const float* block_lse, int32_t B, int32_t S, int32_t H, int32_t D,
              int32_t dtype, void* stream);

/*
 * y = (dtype) (alpha * x) for a contiguous fp32 buffer of n elements: the final
 * cast of the fp32 accumulators (sp_aurora/intel_ring_flash_attn.py:141-150,:271).
 * The destination is [B,S,H,D] with strides in elements.
 */
int spa_cast_from_f32(const float* src, void* dst, int64_t d_sb, int64_t d_ss, int64_t d_sh,
                      int32_t B, int32_t S, int32_t H, int32_t D, int32_t dtype, float alpha,
                      void* stream);

/*
 * Ulysses reshard pack/unpack: a strided permutation copy of 16-byte vectors.
 * Replaces the reshape/transpose/.contiguous() pairs around all_to_all_single in
 * sp_aurora/intel_ulysses_attn.py:95-110,:122-138 and
 * sp_aurora/comm/all_to_all.py:17-180,:228-335.
 * Copies a logical 5-D array [n0,n1,n2,n3,row] of `row_bytes`-byte rows from
 * src (strides in BYTES per logical dim) to dst (strides in BYTES); row_bytes
 * must be a multiple of 16 and both bases/strides 16-byte aligned.
 */
int spa_permute_rows(const void* src, void* dst, const int64_t n[4], const int64_t src_stride[4],
                     const int64_t dst_stride[4], int64_t row_bytes, void* stream);

/*
 * Rotary position embedding fused into the same kind of strided row copy (no counterpart in the
 * reference: its example block, examples/example_mpi_integration.py:38-86, applies no position
 * embedding; a caller with RoPE would otherwise pay one more full pass over q and k before the
 * Ulysses pack of sp_aurora/intel_ulysses_attn.py:95-110).
 * Logical array [n0,n1,n2,n3] of head rows of D elements; strides in ELEMENTS per logical dim
 * (multiples of 16 bytes); dst[:D/2] = x1*cos - x2*sin, dst[D/2:] = x2*cos + x1*sin ("rotate
 * half"), cos/sin fp32 [table_rows, D/2] indexed by pos_offset + index along logical dim
 * pos_dim. inverse != 0 negates sin (the gradient of the rotation). src == dst is allowed.
 */
int spa_rope_rows(const void* src, void* dst, const int64_t n[4], const int64_t src_stride[4],
                  const int64_t dst_stride[4], int32_t D, int32_t dtype, const float* cos_table,
                  const float* sin_table, int64_t table_rows, int32_t pos_dim, int64_t pos_offset,
                  int32_t inverse, void* stream);

/*
 * Device facts. Replaces sp_aurora/sycl_bindings/bindings.cpp:298 get_device_info_py
 * and :362 is_available. Fills: [0] SM count, [1] cc major, [2] cc minor,
 * [3] max opt-in shared memory per block, [4] L2 bytes, [5] global memory MiB.
 */
int spa_device_info(int32_t device, int64_t info[6]);

/* Reads the device status word of the current device (synchronises the
 * device). Returns SPA_OK, or SPA_ETIMEOUT with the site in spa_last_error(). */
int spa_check_status(void);

/* Number of kernels this library has launched in this process. */
int64_t spa_launch_count(void);

const char* spa_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* SPA_H_ */
