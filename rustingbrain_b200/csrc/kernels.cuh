// Launchers of the non-tensor-core kernels (route.cu, combine.cu, gemm_simt.cu,
// backward.cu, optim.cu).  `precision` selects the activation type: f32 or bf16.
#pragma once
#include "common.cuh"

namespace moe {

// When the whole batch fits one router block the routing tables are finalized by that block (no second launch).
struct RouterFinalize {
  int enabled;              // set by the caller; honoured when tokens <= rows of one router block
  float aux_w, z_w;
  RouteMeta meta;
  float* stats;
  float* losses;
  int align;
};

struct RouterArgs {
  const void* x;            // [tokens, d] activations (f32 or bf16); unused when logits_in is set
  const float* w_router;    // [E, d]
  const float* logits_in;   // optional [tokens, E]: skip the projection (test hook)
  const uint8_t* valid;     // optional [tokens] padding mask (0 = padding row)
  int tokens, d, E, k;
  float* logits_out;        // optional [tokens, E]
  float* probs;             // [tokens, E]
  float* lse;               // [tokens]
  int* expert_of;           // [tokens*k], -1 on padding rows
  float* gates;             // [tokens*k]
  float* partial;           // [blocks, E+2]
  int* hist;                // [blocks, E]; after finalize: padded-row write cursors
  RouterFinalize fin;       // optional, see above
};

struct PermuteArgs {
  const void* x;
  const int* expert_of;
  const float* gates;
  const int* cursor;
  RouteMeta meta;
  int tokens, d, E, k;
  RowSpace x_perm;    // destination rows (local buffer, or the owners' receive buffers)
  const int* dest_base;  // optional [E]: row id of this rank's first row of each expert (expert parallel)
  int* slot_pos;      // [tokens*k] row id of each slot, -1 when unrouted
  int* row_token;     // [padded rows] token of each row, -1 for padding rows
  float* row_gate;    // [padded rows] gate of each row
  int* token_of;      // [R] compact, stable expert-major order (the reference's permutation)
  int* slot_of;       // [R]
  int skip_pad;       // do not zero the padding rows at the end of each expert's group
};

cudaError_t launch_router(const RouterArgs& a, int precision, cudaStream_t stream);
// bf16 logits product for decode-sized batches (d a multiple of 8): one CTA per token row
cudaError_t launch_router_logits_rows(const void* x, const void* w_bf16, float* logits, int tokens, int d, int E,
                                      cudaStream_t stream);
// Routing of a decode-sized batch (at most 64 rows and 64 experts, one GPU) in one launch: logits, softmax / top-k,
// finalize and the placement (slot_pos, row_token, ...) WITHOUT the row copy; ra.logits_in names the buffer the logits
// go through, `done` a zeroed device counter.  MOE_B200_DECODE_ROUTE=0 turns it off.
bool decode_route_supported(const RouterArgs& ra, const PermuteArgs& pa);
cudaError_t launch_decode_route_rows(const RouterArgs& ra, const PermuteArgs& pa, const void* w_router_bf16, int* done,
                                     cudaStream_t stream);
// `align`: every expert's row group starts at a multiple of this many rows (128 for the
// local expert GEMMs, 1 for the compact send layout of an expert-parallel rank).
cudaError_t launch_finalize(const RouterArgs& a, RouteMeta meta, float aux_w, float z_w, float* stats, float* losses,
                            int align, cudaStream_t stream);
cudaError_t launch_ep_plan(const int* gathered, int ranks, int E, int rank, int cap, int* dest_base, int* local_meta,
                           int* error_flag, cudaStream_t stream);
cudaError_t launch_ep_pack_stats(const float* stats, const int* counts, int E, int* out, cudaStream_t stream);
cudaError_t launch_ep_losses(const int* gathered, int ranks, int E, int k, float aux_w, float z_w, float* ext_stats,
                             int* ext_counts, float* losses, cudaStream_t stream);
cudaError_t launch_permute(const PermuteArgs& a, int precision, cudaStream_t stream);
cudaError_t launch_pad_rows(void* buf, int d, RouteMeta meta, int E, int precision, cudaStream_t stream);

// y[t] (+)= sum over the token's slots in ascending expert order of gate * y_perm[row] (+ shared[t]).
struct CombineArgs {
  RowSpace y_perm;          // expert output rows
  const void* shared;       // optional [tokens, d]
  const int* expert_of;     // [tokens*k]
  const float* gates;       // [tokens*k]
  const int* slot_pos;      // [tokens*k]
  void* y;                  // [tokens, d]
  int tokens, d, k, accumulate;
  int split = 0;            // set by launch_combine: warps that share one token (decode-sized batches)
};
cudaError_t launch_combine(const CombineArgs& a, int precision, cudaStream_t stream);

// ----- f32 path: grouped SIMT GEMMs over the padded row groups -----
struct SimtGemmArgs {
  const float* A;
  const float* B;
  float* C;
  const int* group_row0;   // [G+1] device
  int n_groups;
  int max_rows;            // capacity of the row-indexed operands (bounds the grid)
  int a_rows, b_rows;      // readable rows of A (and of B when B is row-indexed); rows beyond read as zero
  int N, K, M;
  long long b_group_stride, c_group_stride;
  int accumulate;
};
// C[row, n] = sum_k A[row,k] * B_g[n,k]
cudaError_t simt_gemm_nt(const SimtGemmArgs& a, cudaStream_t stream);
// C[row, n] = sum_k A[row,k] * B_g[k,n]
cudaError_t simt_gemm_nn(const SimtGemmArgs& a, cudaStream_t stream);
// C_g[m, n] (+)= sum_{row in g} A[row,m] * B[row,n]
cudaError_t simt_gemm_tn(const SimtGemmArgs& a, cudaStream_t stream);

// h[r, f] = silu(g) * u from the interleaved (g|u) rows; f32 path only (the bf16
// path fuses this into the GEMM epilogue).
// f32 [rows, cols] -> bf16 [rows, 6 * cols]: three bf16 pieces per value in the A or B segment pattern (gemm_simt.cu)
cudaError_t launch_expand3(const float* src, bf16* dst, long long rows, int cols, int b_pattern, cudaStream_t stream);
cudaError_t launch_swiglu_fwd_f32(const float* gu, float* h, long long rows, int f_pad, cudaStream_t stream);
cudaError_t launch_swiglu_bwd_f32(const float* dh, const float* gu, float* dgu, long long rows, int f_pad,
                                  cudaStream_t stream);

// ----- backward, non-GEMM -----
struct GatherGradArgs {
  const void* grad_y;     // [tokens, d]
  RowSpace y_perm;        // pre-gate expert output rows
  const int* slot_pos;    // [tokens*k]
  const float* gates;     // [tokens*k]
  RowSpace grad_y_perm;   // rows receiving gate * grad_y[token]
  float* grad_gates;      // [tokens*k] = <grad_y[token], y_perm[row]>
  int tokens, d, k;
};
cudaError_t launch_gather_grad(const GatherGradArgs& a, int precision, cudaStream_t stream);

// Expert-parallel peer transport: gate gradient computed on the expert owner.  `aux_off` is the byte
// offset, inside every rank's gradient receive buffer, of three 4-byte arrays of `rows.cap` entries:
// the gates pushed with the rows, the dots the owner computes, and (with dedup) the staging row of each row.
struct PushGradArgs {
  const void* grad_y;     // [tokens, d]
  RowSpace rows;          // the owners' gradient receive buffers
  const int* slot_pos;    // [tokens*k]
  const float* gates;     // [tokens*k]
  size_t aux_off;
  int tokens, d, k;
  // One crossing per (token, destination rank) instead of one per slot: the row goes once into a staging area on
  // every rank that owns one of the token's experts (row stage_base + token of `stage`, which is the owners'
  // input-gradient receive buffer, idle until their GEMMs write it), and each slot's row of the receive buffer gets
  // the gate and the staging row's index; the owner's scale_dot pass reads the staged row and writes the scaled one.
  RowSpace stage;
  int stage_base;         // this rank's first staging row on every owner (rank * max_tokens)
  int dedup;
};
cudaError_t launch_push_grad(const PushGradArgs& a, int precision, cudaStream_t stream);
struct ScaleDotArgs {
  void* grad_y;           // local receive buffer, scaled in place
  const void* y;          // local pre-gate expert outputs, same row layout
  const float* gate_in;   // [rows]
  float* dot_out;         // [rows]
  const void* stage;      // optional: the unscaled rows come from here, row src_index[row], instead of grad_y itself
  const int* src_index;   // [rows]
  const int* row0;        // [groups+1] padded group starts
  const int* counts;      // [groups]
  int groups, d;
};
cudaError_t launch_scale_dot(const ScaleDotArgs& a, int precision, int sm_count, cudaStream_t stream);
struct PullDotsArgs {
  RowSpace rows;
  size_t aux_off;
  const int* slot_pos;
  float* grad_gates;
  int slots;
};
cudaError_t launch_pull_dots(const PullDotsArgs& a, cudaStream_t stream);

struct RouterBwdArgs {
  const float* probs;       // [tokens, E]
  const float* lse;         // [tokens]
  const int* expert_of;     // [tokens*k]
  const float* grad_gates;  // [tokens*k]
  const int* counts;        // [E]   (whole batch)
  const int* total;         // meta.total ([3] = valid tokens) unless valid_override >= 0
  const float* ext_stats;   // optional: whole-batch statistics (expert parallel), [E+1] = V
  const int* ext_counts;
  int tokens, E, k;
  float aux_w, z_w;
  float* grad_logits;       // [tokens, E]
  bf16* grad_logits_bf16;   // optional bf16 copy (operand of the tensor-core router products)
};
cudaError_t launch_router_bwd(const RouterBwdArgs& a, cudaStream_t stream);

// grad_x[t] (+)= sum over slots (ascending expert) grad_x_perm[row] (+ shared) + grad_logits[t] W_r
struct UnpermuteArgs {
  RowSpace grad_x_perm;      // expert input-gradient rows
  const void* shared;        // optional [tokens, d]
  const void* extra;         // optional [tokens, d]: router input gradient computed elsewhere
  const float* grad_logits;  // [tokens, E]; null when `extra` already holds grad_logits W_r
  const float* w_router;     // [E, d]
  const int* expert_of;
  const int* slot_pos;
  void* grad_x;
  int tokens, d, E, k, accumulate;
};
// max_blocks > 0 caps the grid (the kernel strides over the tokens)
cudaError_t launch_unpermute(const UnpermuteArgs& a, int precision, cudaStream_t stream, int max_blocks = 0);

// dW_r[e, c] (+)= sum_t grad_logits[t,e] * x[t,c]; deterministic two-stage reduction.
struct RouterWgradArgs {
  const float* grad_logits;
  const void* x;
  float* grad_w;       // [E, d]
  float* scratch;      // [splits, E, d]
  int tokens, d, E, splits, accumulate;
};
cudaError_t launch_router_wgrad(const RouterWgradArgs& a, int precision, cudaStream_t stream);
cudaError_t launch_router_wgrad_sum(const RouterWgradArgs& a, cudaStream_t stream);

// ----- int8 expert weights for decode-sized batches (decode_q8.cu) -----
// out[row, n] = (sum_k x[row,k] * q_g[n,k]) * scale_g[n], rows of group g < E taken from the
// padded expert-major buffers, group E (optional) = the shared expert over every token row.
// swiglu: q holds the interleaved gate|up rows [2N, K]; out = silu(gate) * up, N hidden columns.
struct Q8Args {
  const bf16* x_rows;      // [padded rows, K]; with x_row_index: [tokens, K], row r of a group is x_rows[x_row_index[r]]
  const int* x_row_index;  // optional [padded rows]: gather the routed rows instead of reading them in place
  const bf16* x_shared;    // optional [tokens, K]
  bf16* out_rows;          // [padded rows, ldo]
  bf16* out_shared;        // [tokens, ldo]
  const int8_t* w;         // [groups][rows][K]
  const float* scale;      // [groups][rows]
  const int* counts;       // [E]
  const int* pad_off;      // [E+1]
  long long w_group_stride, s_group_stride;
  int E, tokens, K, N, ldo;
  int sm_count;            // grid = two CTAs per SM
  // tensor-core variant only (decode_q8_tc.cu)
  long long x_rows_cap;    // readable rows of x_rows
  long long x_shared_rows; // readable rows of x_shared
  int* error_flag;         // bounded waits report here
};
cudaError_t launch_q8_rows(const Q8Args& a, bool swiglu, cudaStream_t stream);
// tcgen05 variant: the weights are the 128-row MMA operand, widened to f16 in shared memory
bool q8_tc_supported(const Q8Args& a, bool swiglu);
cudaError_t launch_q8_rows_tc(const Q8Args& a, bool swiglu, cudaStream_t stream);

// ----- optimizer and casts -----
struct AdamArgs {
  float* w; float* g; float* m; float* v;
  bf16* w_bf16;        // optional compute copy refreshed in the same pass
  long long n;
  float lr, beta1, beta2, eps, wd, c1, c2, scale;
};
cudaError_t launch_adam(const AdamArgs& a, cudaStream_t stream);
cudaError_t launch_sgd(const AdamArgs& a, cudaStream_t stream);    // uses lr, scale
cudaError_t launch_lion(const AdamArgs& a, cudaStream_t stream);   // uses lr, beta1, beta2, wd, scale and the first moment
cudaError_t launch_cast_f32_to_bf16(const float* src, bf16* dst, long long n, cudaStream_t stream);
cudaError_t launch_cast_bf16_to_f32(const bf16* src, float* dst, long long n, cudaStream_t stream);
cudaError_t launch_fill_f32(float* dst, float v, long long n, cudaStream_t stream);

}  // namespace moe
