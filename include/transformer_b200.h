/* C ABI of the language model around the MoE layer (libmoe_b200.so, sm_100a): everything
 * TransformerLm::train_step_batch runs on the device besides the MoE feed-forward itself, so that the
 * reference's 55M-parameter configuration steps as a whole model.
 *
 * What it replaces (reference, by the file's path within its project):
 *   TransformerLm::{forward_batch, backward, train_step_batch, accumulate_step, step, zero_grad}
 *                                        src/transformer.rs:676-735, 1214-1246, 1394-1425, 1519-1545, 1576-1606
 *   device drivers of the same           src/gpu_model.rs:2100-2346 (forward_block), 2683-2772 (chunked head + loss),
 *                                        3084-3530 (backward_block)
 *   TransformerBlock forward / backward  src/transformer_block.rs:205-270
 *   MultiHeadAttention forward_train / backward (packed QKV, rotate-half RoPE, causal GQA)
 *                                        src/attention.rs:305-341, 404-556; src/rope.rs:12-18, 129-146
 *   SwiGlu (dense layers)                src/ffn.rs:56-120
 *   Embedding gather / scatter / tied head   src/embedding.rs:49-152
 *   causal_lm_loss_batch                 src/causal_lm_loss.rs:66-150
 *   Param::step (Sgd, Adam, Lion)        src/param.rs:547-617
 *
 * Arithmetic: bf16 tensor-core products over f32 master weights (the reference's mixed_precision mode),
 * f32 normalisation, softmax, loss and optimizer.  Every matrix product runs on the grouped tcgen05 GEMM of
 * this library; the MoE blocks are moe_layer_t handles of moe_b200.h owned by the model.
 * Shape rules of that kernel: d_model, head_dim and the feed-forward widths are multiples of 32.
 * Status codes are the moe_status values of moe_b200.h.  A handle is not thread safe.
 */
#ifndef TRANSFORMER_B200_H
#define TRANSFORMER_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct lm_model lm_model_t;

/* TransformerConfig (transformer.rs:28-58; defaults :99-125). */
typedef struct lm_config {
  int32_t vocab_size, d_model, n_layers, n_heads, n_kv_heads, head_dim;
  int32_t d_ff;                 /* dense layers */
  int32_t moe_d_ff, num_experts, experts_per_token, shared_expert;
  uint64_t moe_layer_mask;      /* bit l set: layer l has a MoE feed-forward (moe_layers; at most 64 layers) */
  int32_t max_seq_len;
  float rope_base, rmsnorm_eps;
  int32_t tie_embeddings;
  float aux_loss_weight, router_z_loss_weight;
  int32_t max_batch_rows;       /* largest batch * seq_len a step will see (sizes the workspace) */
  int32_t device;
} lm_config_t;

/* Parameters, addressed like the reference's modules.  `layer` is the block index, ignored for the model-level
 * ones; `expert` is used by the per-expert MoE matrices only.  All matrices are [out, in] row-major f32. */
typedef enum lm_param {
  LM_EMBEDDING = 0,        /* [vocab, d_model]; also the output head when tied */
  LM_FINAL_NORM = 1,       /* [d_model] */
  LM_HEAD = 2,             /* [vocab, d_model], untied models only */
  LM_ATTENTION_NORM = 3,   /* [d_model] */
  LM_WQ = 4,               /* [n_heads * head_dim, d_model] */
  LM_WK = 5,               /* [n_kv_heads * head_dim, d_model] */
  LM_WV = 6,
  LM_WO = 7,               /* [d_model, n_heads * head_dim] */
  LM_FFN_NORM = 8,         /* [d_model] */
  LM_FFN_GATE = 9,         /* dense layers: [d_ff, d_model] */
  LM_FFN_UP = 10,
  LM_FFN_DOWN = 11,        /* [d_model, d_ff] */
  LM_MOE_ROUTER = 12,      /* MoE layers: the moe_weight ids of moe_b200.h, in the same order */
  LM_MOE_GATE = 13,
  LM_MOE_UP = 14,
  LM_MOE_DOWN = 15,
  LM_MOE_SHARED_GATE = 16,
  LM_MOE_SHARED_UP = 17,
  LM_MOE_SHARED_DOWN = 18
} lm_param;

/* TransformerConfig::validate (transformer.rs:132-172) plus the shape rules above. */
int32_t lm_config_validate(const lm_config_t* config, char* message, int32_t message_len);
/* TransformerConfig::parameter_counts (transformer.rs:195-235). */
int32_t lm_parameter_counts(const lm_config_t* config, int64_t* total, int64_t* active);

/* TransformerLm::from_builder + to_cuda: allocates weights (zero), gradients, Adam moments and the workspace.
 * Weight initialisation stays with the caller (lm_set_param), so the host language keeps its own RNG. */
int32_t lm_create(const lm_config_t* config, lm_model_t** out);
void lm_destroy(lm_model_t* model);
const char* lm_last_error(const lm_model_t* model);

int32_t lm_set_param(lm_model_t* model, int32_t layer, int32_t which, int32_t expert, const float* host, int32_t rows, int32_t cols);
int32_t lm_get_param(lm_model_t* model, int32_t layer, int32_t which, int32_t expert, float* host, int32_t rows, int32_t cols);
/* Plain dL/dW as accumulated since the last lm_zero_grad / lm_step. */
int32_t lm_get_grad(lm_model_t* model, int32_t layer, int32_t which, int32_t expert, float* host, int32_t rows, int32_t cols);

/* A packed batch (TokenBatch, batch.rs:22-75): ids_host [batch * seq_len] right-padded, lengths_host [batch]
 * (null: every sequence is seq_len long), loss_mask_host optional [batch * seq_len] bytes (with_loss_mask). */

/* forward_batch: logits_host [batch * seq_len, vocab] f32 (test and evaluation hook: the training entries
 * below never materialise them on the host).  moe_logits_host, optional: per MoE layer in ascending order,
 * [batch * seq_len, num_experts] f32, receives the router logits of that layer. */
int32_t lm_forward_logits(lm_model_t* model, const uint32_t* ids_host, const int32_t* lengths_host, int32_t batch,
                          int32_t seq_len, float* logits_host, float* moe_logits_host);

/* accumulate_step: forward, fused head + loss, backward into the gradients (no optimizer step). */
int32_t lm_accumulate_step(lm_model_t* model, const uint32_t* ids_host, const int32_t* lengths_host,
                           const uint8_t* loss_mask_host, int32_t batch, int32_t seq_len, float* lm_loss,
                           float* auxiliary_loss);
/* zero_grad (a flag, as DeviceParam::zero_grad) and step with Adam; `scale` multiplies the gradients. */
int32_t lm_zero_grad(lm_model_t* model);
int32_t lm_step_adam(lm_model_t* model, float lr, float beta1, float beta2, float eps, float weight_decay, float scale);
/* step with Optimizer::Sgd / Optimizer::Lion (param.rs:557-561, 590-613). */
int32_t lm_step_sgd(lm_model_t* model, float lr, float scale);
int32_t lm_step_lion(lm_model_t* model, float lr, float beta1, float beta2, float weight_decay, float scale);
/* train_step_batch: zero_grad, accumulate_step, step(1.0).  Returns TotalLoss{lm_loss, auxiliary_loss}. */
int32_t lm_train_step(lm_model_t* model, const uint32_t* ids_host, const int32_t* lengths_host,
                      const uint8_t* loss_mask_host, int32_t batch, int32_t seq_len, float lr, float beta1, float beta2,
                      float eps, float weight_decay, float* lm_loss, float* auxiliary_loss);
/* optimizer_step / set_optimizer_step (transformer.rs:1608-1618). */
int64_t lm_optimizer_step(const lm_model_t* model);
int32_t lm_set_optimizer_step(lm_model_t* model, int64_t step);

/* KV-cached decode (TransformerLm::new_kv_caches + forward_cached, transformer.rs:649-660, 737-770), for
 * `sequences` independent sequences that advance together: one batched cache per layer (kv_attention_b200.h,
 * bf16), `capacity` positions each (at most max_seq_len).  lm_forward_cached feeds rows_per_sequence new token ids
 * to each of the sequences first_sequence .. first_sequence + n_sequences - 1 (the whole prompt for a prefill, one
 * id per sequence for a decode step; ids_host is sequence-major) and returns the logits of every new row,
 * logits_host [n_sequences * rows_per_sequence, vocab] f32.  SequenceTooLong -> MOE_INVALID_INPUT, nothing appended. */
typedef struct lm_decoder lm_decoder_t;
int32_t lm_decoder_create(lm_model_t* model, int32_t sequences, int32_t capacity, lm_decoder_t** out);
void lm_decoder_destroy(lm_decoder_t* decoder);
/* KvCache::clear for every layer: one sequence, or all of them when sequence < 0. */
int32_t lm_decoder_clear(lm_model_t* model, lm_decoder_t* decoder, int32_t sequence);
int32_t lm_forward_cached(lm_model_t* model, lm_decoder_t* decoder, const uint32_t* ids_host, int32_t first_sequence,
                          int32_t n_sequences, int32_t rows_per_sequence, float* logits_host);

/* Kernel launches since creation and CUDA-event milliseconds of the last step's phases, for the benchmark:
 * ms[0] embedding + blocks forward, ms[1] head + loss (three products over the vocabulary), ms[2] blocks backward
 * + embedding scatter, ms[3] optimizer. */
int32_t lm_last_step_ms(lm_model_t* model, float* ms4);
int32_t lm_synchronize(lm_model_t* model);

#ifdef __cplusplus
}
#endif
#endif
