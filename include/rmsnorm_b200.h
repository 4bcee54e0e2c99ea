/* C ABI of RMSNorm forward / backward (libmoe_b200.so, sm_100a): the normalisation in front of the MoE
 * layer in every decoder block (reference norm.rs:41-129; its device kernels cuda_training.rs:141-184).
 *
 *   y[r, c]  = x[r, c] * inverse_rms(r) * weight[c],   inverse_rms = 1 / sqrt(mean_c(x^2) + eps)
 *   dx[r, c] = dy[r, c] * weight[c] * inverse_rms - x[r, c] * (sum_c dy * weight * x) * inverse_rms^3 / d
 *   dweight[c] += sum_r dy[r, c] * x[r, c] * inverse_rms(r)     (rows summed in tiles of 32 in row order, the
 *                                                                reference's tiles, norm.rs:8-14; tile totals in a
 *                                                                fixed order: independent of scheduling)
 *
 * Stateless: all pointers are device pointers owned by the caller; activations are f32
 * (MOE_PRECISION_F32) or bf16 (MOE_PRECISION_BF16), weight and its gradient f32.  Status codes are the
 * moe_status values of moe_b200.h; on failure `message` (optional) receives the reason.
 */
#ifndef RMSNORM_B200_H
#define RMSNORM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* RmsNorm::forward.  d must be a multiple of 8. */
int32_t rmsnorm_forward(const void* x, const float* weight, void* y, int32_t rows, int32_t d, float eps,
                        int32_t precision, void* stream, char* message, int32_t message_len);

/* Bytes of scratch rmsnorm_backward needs: one partial weight gradient per tile of 32 rows. */
int64_t rmsnorm_scratch_bytes(int32_t rows, int32_t d);

/* RmsNorm::backward: writes grad_x, ADDS the weight gradient to grad_weight (pass null for a frozen
 * weight, norm.rs:112).  The inverse RMS is recomputed from x, as in the reference. */
int32_t rmsnorm_backward(const void* x, const float* weight, const void* grad_y, void* grad_x, float* grad_weight,
                         void* scratch, int32_t rows, int32_t d, float eps, int32_t precision, void* stream,
                         char* message, int32_t message_len);

#ifdef __cplusplus
}
#endif
#endif
