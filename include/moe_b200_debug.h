/*
 * moe_b200_debug.h - test hooks of libmoe_b200.so.  Not part of the drop-in
 * boundary: these entries have no counterpart in the reference crate; they let the
 * parity tests drive one kernel at a time.
 */
#ifndef MOE_B200_DEBUG_H
#define MOE_B200_DEBUG_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* One grouped tensor-core GEMM on caller-provided device buffers (bf16 operands).
 * variant 0: out0[r, N]  = A[r, K] * B_g[N, K]^T                         (bf16 out)
 *         1: as 0 with the SwiGLU epilogue: out0 = h [r, N/2], out1 = (g|u) [r, N] or null
 *         2: out0[r, N]  = A[r, K] * B_g[K, N]                           (bf16 out)
 *         3: as 2 with the SwiGLU-backward epilogue: aux = (g|u) [r, 2N], out0 = (dg|du) [r, 2N]
 *         4: out0_g[M, N] (+)= A[rows_g, M]^T * B[rows_g, N]             (f32 out)
 * group_row0 / tile_start are device arrays of n_groups+1 ints (row groups padded to 128).
 * error_flag is a device int that receives a non-zero code if a bounded wait gives up. */
int32_t moe_debug_tc_gemm(int32_t variant, const void* a, const void* b, void* out0, void* out1, const void* aux,
                          const int32_t* group_row0, const int32_t* tile_start, int32_t n_groups, int32_t rows,
                          int32_t m, int32_t n, int32_t k, int32_t accumulate, int32_t* error_flag, void* stream);

/* Per-kernel timing.  While enabled, the library brackets each stage of forward / backward
 * with CUDA events on the caller's stream.  moe_debug_profile_read synchronises, adds the
 * elapsed milliseconds and the number of bracketed stages per category into the two arrays
 * of MOE_PROFILE_CATEGORIES entries, and clears the record.  Categories:
 *  0 router+finalize  1 permute  2 gate|up GEMM  3 down GEMM  4 combine  5 gradient gather
 *  6 down dgrad  7 down wgrad  8 gate|up dgrad  9 gate|up wgrad  10 router backward
 *  11 un-permute  12 router wgrad  13 shared expert forward  14 shared expert backward  15 Adam */
#define MOE_PROFILE_CATEGORIES 16
struct moe_layer;
int32_t moe_debug_profile(struct moe_layer* layer, int32_t enable);
int32_t moe_debug_profile_read(struct moe_layer* layer, float* milliseconds, int32_t* stages);

/* Selects the tile variant of the grouped tensor-core GEMM for later launches: 0 one-SM 128x256 tiles,
 * 1 two-SM (cta_group::2) 256x256 tiles, 2 one-SM 256x256 tiles, 3 a choice per launch between 0 and 2 (the default). */
int32_t moe_debug_set_tc_pair(int32_t mode);

/* The polling wait behind moe_ep_set_deadline_ms, driven by a clock instead of a stream (needs no device):
 * the condition becomes true `ready_after_ms` after the call starts; returns MOE_OK (0) if that happens within
 * `deadline_ms`, else MOE_TIMEOUT (6) with *gave_up = 1.  deadline_ms = 0 waits for ever. */
int32_t moe_debug_deadline_wait(int32_t ready_after_ms, int32_t deadline_ms, int32_t* gave_up);

/* Failure-path hook of the grouped tensor-core GEMM: the NEXT launch (one launch only) runs with a producer
 * that issues no load and with `wait_limit_cycles` (about 2,000,000 = 1 ms) as the limit of every barrier
 * wait.  The consumers' waits run out, the kernel records a code in its error flag, every role leaves its
 * loop, the CTA frees its tensor memory and returns: the next moe_synchronize / moe_get_* on the handle
 * returns MOE_TIMEOUT and, after moe_clear_error, the handle works as before.  Nothing is in flight when
 * the waits give up, and no wait is unbounded. */
int32_t moe_debug_starve_next_gemm(int64_t wait_limit_cycles);

/* Number of kernel launches issued by this library in the calling process. */
int64_t moe_debug_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* MOE_B200_DEBUG_H */
