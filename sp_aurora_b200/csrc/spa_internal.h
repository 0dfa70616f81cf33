// Internal declarations shared by the kernels and the C-ABI translation unit.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/spa.h"

namespace spa {

// Error text for spa_last_error(); thread-local.
void set_error(const char* fmt, ...);

// Device-global status word (4 ints) of the current device; allocated lazily,
// zero while no bounded wait has ever given up.
int* device_status_word();

// Encode a 4-D TMA descriptor (dims D, S, H, B; 128-byte swizzle; box of
// `box_rows` sequence rows by 64 two-byte elements). Returns 0 on success.
int encode_rows_map(CUtensorMap* map, const void* ptr, int is_bf16, int D, int64_t S, int H, int B,
                    int64_t stride_s, int64_t stride_h, int64_t stride_b, int box_rows);

// 4-D TMA descriptor over a contiguous fp32 [B,S,H,D] tensor (dims D, S, H, B; no
// swizzle; box of `box_rows` sequence rows by D), used for bulk reduce-add.
int encode_f32_rows_map(CUtensorMap* map, const void* ptr, int D, int64_t S, int H, int B,
                        int box_rows);

// Same tensor, box of `box_rows` sequence rows by 32 floats with the 128-byte swizzle:
// shared-memory slabs of [box_rows][128 B] that a thread per row fills without bank
// conflicts. Used to store or reduce-add dK/dV tiles.
int encode_f32_slab_map(CUtensorMap* map, const void* ptr, int D, int64_t S, int H, int B,
                        int box_rows);

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) applies to the current device only:
// done once per (kernel, device), remembered in a small table. Returns a spa status code.
int ensure_dynamic_smem(const void* kernel, int bytes, const char* what);

// SM count of the current device (cached per device; 148 if the query fails).
int device_sm_count();

// Launchers (return a spa status code). Arguments arrive normalised: zero stride
// triples of spa.h are already replaced by the contiguous strides.
int launch_fwd_sm100(const spa_fwd_args* a);
int launch_bwd_dq_sm100(const spa_bwd_args* a);       // query-stationary pass: dQ
int launch_bwd_dkv_sm100(const spa_bwd_args* a);      // K/V-stationary pass: dK, dV
int launch_fwd_simt(const spa_fwd_args* a);
int launch_bwd_simt(const spa_bwd_args* a);

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

}  // namespace spa
