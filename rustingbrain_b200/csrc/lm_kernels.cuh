// Row kernels of the language model around the MoE layer (lm.cu): everything between the tensor-core
// products.  All of them are bound by HBM (or tiny); activations are bf16, arithmetic f32.
//
// Attention layouts.  Token rows are r = b * S + s.  For the tensor-core products the heads are regrouped so
// that one key/value head and the `g` query heads that share it form one row group of the grouped GEMM:
//   group  grp = b * Hkv + kvh,   query head h = kvh * g + gi
//   q_hm / o_hm / dq_hm / do_hm   [G * GR, hd]        row = grp * GR + gi * S + s     (GR = g * S rounded up to 128)
//   k_hm / v_hm                   [G][S_pad][hd]      row = grp * S_pad + s           (S_pad = S rounded up to 32)
//   scores / probabilities        [G * GR, S_pad]
// Rows and columns past the real ones stay zero, so the products over padded extents are exact.
#pragma once
#include "common.cuh"

namespace moe {
namespace lm {

struct AttnShape {
  int B, S, H, Hkv, hd;   // batch, sequence length, query heads, key/value heads, head_dim
  int g;                  // H / Hkv
  int GR;                 // rows of one (batch, kv head) group in the head-major layouts
  int S_pad;              // keys per group, padded
  int G;                  // groups = B * Hkv
};

cudaError_t launch_embed_gather(const uint32_t* ids, const bf16* table, bf16* x, int rows, int d, cudaStream_t st);
// next[r]: the next row with the same id (-1: none); first[r]: no earlier row has it (both made on the host, where
// the ids come from).  One block per first occurrence walks its chain in row order and adds the sum to the
// gradient row: deterministic, no atomics.
cudaError_t launch_embed_scatter(const uint32_t* ids, const bf16* grad_x, float* grad_table, const int* first, const int* next,
                                 int rows, int d, cudaStream_t st);

cudaError_t launch_rope_pack(const bf16* qkv, const float* cos_t, const float* sin_t, bf16* q_hm, bf16* k_hm, bf16* v_hm,
                             AttnShape a, cudaStream_t st);
// causal: only the visible prefix of a row is read.  bounded_tail: zeros are written only as far behind the prefix as
// the causal tensor-core products read (up to the next multiple of 128 from the query position); otherwise the whole
// rest of the row is written.
cudaError_t launch_softmax_causal(const bf16* scores, bf16* probs, AttnShape a, float scale, int causal, int bounded_tail,
                                  cudaStream_t st);
cudaError_t launch_softmax_backward(const bf16* probs, bf16* grad_probs_to_scores, AttnShape a, float scale, int causal,
                                    int bounded_tail, cudaStream_t st);
cudaError_t launch_heads_to_tokens(const bf16* o_hm, bf16* merged, AttnShape a, cudaStream_t st);
cudaError_t launch_tokens_to_heads(const bf16* grad_merged, bf16* do_hm, AttnShape a, cudaStream_t st);
cudaError_t launch_qkv_grad_unpack(const bf16* dq_hm, const float* dk_hm, const float* dv_hm, const float* cos_t,
                                   const float* sin_t, bf16* dqkv, AttnShape a, cudaStream_t st);
cudaError_t launch_attn_meta(int* meta, int groups, int group_rows, cudaStream_t st);

// packed [rows, qn + 2 kn] -> q [rows, qn], k [rows, kn], v [rows, kn] (the cached-decode attention takes them apart)
cudaError_t launch_split_qkv(const bf16* qkv, bf16* q, bf16* k, bf16* v, int rows, int qn, int kn, cudaStream_t st);
cudaError_t launch_add(const bf16* a, const bf16* b, bf16* out, long long n, cudaStream_t st);
cudaError_t launch_cast_rows_to_f32(const bf16* src, long long ld, float* dst, int rows, int cols, cudaStream_t st);

// Cross-entropy over the rows of `logits` [rows, ld] (first `vocab` columns), in place: the row becomes
// dL/dlogits = (softmax - onehot) / predicted for a row with a target, zero otherwise; row_loss[r] = -ln p[target].
cudaError_t launch_cross_entropy(bf16* logits, const int* targets, float* row_loss, int rows, int vocab, int ld,
                                 float inv_predicted, cudaStream_t st);
// out[0] = (sum of row_loss in a fixed order) / predicted
cudaError_t launch_loss_sum(const float* row_loss, int rows, float inv_predicted, float* out, cudaStream_t st);

// f32 [rows, cols] -> arena rows (f32 master + bf16 mirror) with leading dimension ld, starting at row0;
// kind 0 plain, 1 / 2 the gate / up rows of the interleaved gate|up matrix (blocks of 32).
cudaError_t launch_pack(const float* src, float* dst, bf16* dst_bf16, int rows, int cols, int ld, int row0, int kind,
                        cudaStream_t st);
cudaError_t launch_unpack(const float* src, float* dst, int rows, int cols, int ld, int row0, int kind, cudaStream_t st);

}  // namespace lm
}  // namespace moe
