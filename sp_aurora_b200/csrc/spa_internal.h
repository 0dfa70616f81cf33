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

// Debug aid (library built with -DSPA_PROFILE_WAITS and env SPA_WAIT_PROFILE=1): a zeroed device array of 32 counters that
// the tensor-core kernels fill with cycles blocked per wait site, and a
// synchronous dump of it to stderr. Returns nullptr when the aid is off.
unsigned long long* wait_profile_buffer();
void wait_profile_report(const char* tag, cudaStream_t stream);

// Launchers (return a spa status code).
int launch_fwd_sm100(const spa_fwd_args* a);
int launch_bwd_sm100(const spa_bwd_args* a);          // dK/dV in the input dtype
int launch_bwd_f32out_sm100(const spa_bwd_args* a);   // fp32 dK/dV (ring steps)
int launch_bwd128_sm100(const spa_bwd_args* a);   // head_dim 128, 128x128 tiles
int launch_fwd_simt(const spa_fwd_args* a);
int launch_bwd_simt(const spa_bwd_args* a);

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

}  // namespace spa
