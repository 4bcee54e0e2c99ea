/*
 * moe_b200.h - C ABI of the sm_100a mixture-of-experts feed-forward layer.
 *
 * This is the boundary a host language binds (Rust `extern "C"`, Python ctypes,
 * C++).  It stands in for the Rust-internal interface of the reference crate
 * `rusting_brain` 2.0.2, which has no FFI of its own for this path: each entry
 * names the reference item it replaces (file:line inside the crate).
 *
 * Conventions
 *   - every function returns a moe_status (0 = ok) unless stated otherwise;
 *     moe_last_error() gives the text of the last failure on a handle
 *   - a handle belongs to one device and one layer and is not thread safe
 *   - "dev" pointers are device memory of that device, "host" pointers are host
 *     memory; activations are row-major [tokens, d_model], f32 for
 *     MOE_PRECISION_F32 handles and bf16 for MOE_PRECISION_BF16 / _Q8 handles
 *   - weights cross the boundary in the reference's layout: f32, row-major
 *     [out_features, in_features] (param.rs:620-625); the library repacks them
 *   - gradients are plain dL/dW (the reference's device buffers hold -dL/dW,
 *     gpu_transformer.rs:18-22; that sign convention does not cross this ABI)
 *   - there is no CPU fallback: without a usable device every call fails
 */
#ifndef MOE_B200_H
#define MOE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct moe_layer moe_layer_t;

/* NetworkError variants this path can raise (network.rs:19-83). */
typedef enum {
  MOE_OK = 0,
  MOE_INVALID_CONFIG = 1,
  MOE_INVALID_INPUT = 2,
  MOE_CUDA_ERROR = 3,
  MOE_OUT_OF_MEMORY = 4,
  MOE_UNSUPPORTED = 5,
  MOE_TIMEOUT = 6,
  MOE_COMM_ERROR = 7,
  MOE_POISONED = 8
} moe_status;

typedef enum {
  MOE_PRECISION_F32 = 0,  /* f32 storage and f32 FMA products (TransformerBuilder::mixed_precision(false)) */
  MOE_PRECISION_BF16 = 1, /* bf16 activations and weights on the tensor cores, f32 accumulate and f32 master weights */
  MOE_PRECISION_Q8 = 2    /* inference only: int8 expert weights with one f32 scale per output row, bf16 activations */
} moe_precision;

/* Which projection of the layer; order follows MoeLayer::params_mut (moe.rs:516-525). */
typedef enum {
  MOE_W_ROUTER = 0,      /* [num_experts, d_model] */
  MOE_W_GATE = 1,        /* [d_ff, d_model], per expert */
  MOE_W_UP = 2,          /* [d_ff, d_model], per expert */
  MOE_W_DOWN = 3,        /* [d_model, d_ff], per expert */
  MOE_W_SHARED_GATE = 4,
  MOE_W_SHARED_UP = 5,
  MOE_W_SHARED_DOWN = 6
} moe_weight;

/* MoeConfig (moe.rs:26-39) plus what the builder passes around it
 * (TransformerBuilder::experts / moe_d_ff / shared_expert / aux_loss_weight /
 * router_z_loss_weight / mixed_precision, transformer.rs:320-437). */
typedef struct {
  int32_t d_model;
  int32_t num_experts;
  int32_t experts_per_token;
  int32_t d_ff;
  int32_t shared_expert;          /* 0 / 1 */
  float aux_loss_weight;          /* DEFAULT_AUX_LOSS_WEIGHT = 0.01 */
  float router_z_loss_weight;     /* DEFAULT_ROUTER_Z_LOSS_WEIGHT = 1e-3, 0 disables */
  int32_t precision;              /* moe_precision */
  int32_t max_tokens;             /* largest `tokens` any call will pass; sizes the workspace */
  int32_t device;                 /* CUDA device ordinal */
  int32_t training;               /* 0: forward only (no gradient or optimizer state is allocated) */
  /* Expert parallelism: this handle owns experts [ep_rank*E/ep_size, (ep_rank+1)*E/ep_size).
   * ep_size = 1 is the single-device layer. */
  int32_t ep_rank;
  int32_t ep_size;
  /* Receive-buffer rows of an expert-parallel rank as a multiple of max_tokens * experts_per_token
   * (its share under uniform routing); 0 selects 1.25.  Routing is dropless, so a pass that sends
   * a rank more rows than this fails with MOE_INVALID_INPUT instead of dropping tokens. */
  float ep_capacity_factor;
} moe_config_t;

/* MoeConfig::validate (moe.rs:68-86) and the shape rules of the chosen precision. */
int32_t moe_config_validate(const moe_config_t* cfg, char* message, int32_t message_len);

/* Device bytes moe_create will allocate; lets a caller apply the reference's
 * budget check before upload (TransformerLm::to_cuda, transformer.rs:1265-1277). */
int64_t moe_workspace_bytes(const moe_config_t* cfg);

/* MoeLayer::new (moe.rs:215-231) + Param::move_to_cuda: allocates weights (zeroed),
 * gradients, Adam moments and the workspace.  Weight initialisation stays with
 * the caller (moe_set_weight_f32). */
int32_t moe_create(const moe_config_t* cfg, moe_layer_t** out);
void moe_destroy(moe_layer_t* layer);
const char* moe_last_error(const moe_layer_t* layer);
/* Clears a sticky failure (the reference's poisoned GpuContext has to be rebuilt;
 * here the handle can be reused once the cause is gone). */
int32_t moe_clear_error(moe_layer_t* layer);

/* Param upload / download (Param::move_to_cuda, DeviceParam::download,
 * gpu_transformer.rs:393-556).  `expert` is ignored for router and shared weights;
 * in an expert-parallel handle it is the GLOBAL expert index and must be owned. */
int32_t moe_set_weight_f32(moe_layer_t* layer, int32_t which, int32_t expert, const float* host, int32_t rows, int32_t cols);
int32_t moe_get_weight_f32(moe_layer_t* layer, int32_t which, int32_t expert, float* host, int32_t rows, int32_t cols);
int32_t moe_get_grad_f32(moe_layer_t* layer, int32_t which, int32_t expert, float* host, int32_t rows, int32_t cols);
int32_t moe_get_moments_f32(moe_layer_t* layer, int32_t which, int32_t expert, float* m_host, float* v_host, int32_t rows, int32_t cols);
int32_t moe_set_moments_f32(moe_layer_t* layer, int32_t which, int32_t expert, const float* m_host, const float* v_host, int32_t rows, int32_t cols);
/* Quantized (quantized.rs:17-24): int8 [rows, cols] + f32 scale[rows], w ~ q * scale. MOE_PRECISION_Q8 handles only.
 * MOE_W_ROUTER is accepted too (TransformerLm::quantize quantizes the router as well, transformer.rs:899-910): the
 * router then computes with the values q * scale. */
int32_t moe_set_weight_q8(moe_layer_t* layer, int32_t which, int32_t expert, const int8_t* q_host, const float* scale_host, int32_t rows, int32_t cols);

/* MoeLayer::forward_train / forward (moe.rs:237-341), device pointers.
 *   x_dev       [tokens, d_model]
 *   valid_dev   optional [tokens] bytes, 0 = padding row (Layout::valid, batch.rs:225-269)
 *   y_dev       [tokens, d_model]; accumulate != 0 adds into it (the reference's device
 *               path accumulates into the residual stream, gpu_model.rs:2314-2346)
 *   save_for_backward  keep what moe_backward needs (forward_train) or not (forward)
 *   stream      a cudaStream_t (0 = default stream) */
int32_t moe_forward(moe_layer_t* layer, const void* x_dev, int32_t tokens, int32_t cols, const uint8_t* valid_dev,
                    void* y_dev, int32_t accumulate, int32_t save_for_backward, void* stream);
/* Test hook: as moe_forward, but the router projection is replaced by the given
 * f32 logits [tokens, num_experts]; used for the bit-exact routing checks. */
int32_t moe_forward_from_logits(moe_layer_t* layer, const void* x_dev, const float* logits_dev, int32_t tokens,
                                int32_t cols, const uint8_t* valid_dev, void* y_dev, int32_t accumulate,
                                int32_t save_for_backward, void* stream);
/* MoeLayer::backward (moe.rs:348-489): weight gradients accumulate into the handle
 * (moe_zero_grad clears them), the auxiliary-loss gradients are included, and
 * grad_x_dev receives dL/dx (added to it when accumulate != 0). */
int32_t moe_backward(moe_layer_t* layer, const void* grad_y_dev, void* grad_x_dev, int32_t accumulate, void* stream);
int32_t moe_zero_grad(moe_layer_t* layer, void* stream);
/* Param::step with Optimizer::Adam over every weight of the layer (param.rs:562-589);
 * `step` is the already incremented global step, `scale` multiplies the gradient. Clears gradients. */
int32_t moe_step_adam(moe_layer_t* layer, float lr, float beta1, float beta2, float eps, float weight_decay,
                      int32_t step, float scale, void* stream);
/* Param::step with Optimizer::Sgd (param.rs:557-561): value -= lr * grad * scale.  Clears gradients. */
int32_t moe_step_sgd(moe_layer_t* layer, float lr, float scale, void* stream);
/* Param::step with Optimizer::Lion (param.rs:590-613): the sign of beta1 * m + (1 - beta1) * grad, decoupled weight
 * decay; the first-moment buffer is the one Adam uses (as the reference's Param::m).  Clears gradients. */
int32_t moe_step_lion(moe_layer_t* layer, float lr, float beta1, float beta2, float weight_decay, float scale, void* stream);

/* The same calls with HOST buffers: f32 [tokens, d_model] in and out, copies included
 * (what TransformerLm::forward_batch does around the device path). valid_host may be null. */
int32_t moe_forward_host(moe_layer_t* layer, const float* x_host, int32_t tokens, int32_t cols, const uint8_t* valid_host,
                         float* y_host, int32_t save_for_backward);
int32_t moe_backward_host(moe_layer_t* layer, const float* grad_y_host, float* grad_x_host);

/* MoeCache accessors (moe.rs:131-188), copied to host after synchronising the
 * stream of the last forward.  Any pointer may be null. */
int32_t moe_get_losses(moe_layer_t* layer, float* aux_loss, float* z_loss);
/* expert_of / gates: [tokens*k] (expert -1 and gate 0 on padding rows);
 * counts: [num_experts]; token_of / slot_of: the stable expert-major permutation,
 * length sum(counts).  Returns the number of routed rows through *routed. */
int32_t moe_get_routing(moe_layer_t* layer, int32_t* expert_of, float* gates, int32_t* counts, int32_t* token_of,
                        int32_t* slot_of, int32_t* routed);
/* logits / probabilities [tokens, E] and log-sum-exp [tokens] of the last forward. */
int32_t moe_get_router_cache(moe_layer_t* layer, float* logits, float* probabilities, float* log_sum_exp);

/* Expert parallelism (no counterpart in the reference, which is single-device; README.md:29-31).
 * Rank r of ep_size owns experts [r*E/ep_size, (r+1)*E/ep_size); router and shared expert are
 * replicated.  One rank obtains an id with moe_ep_unique_id and passes it to the others by any
 * host channel; every rank then calls moe_ep_init (collective).  After that moe_forward /
 * moe_backward on these handles are collectives: every rank must call them in the same order.
 * The row exchange is NCCL send/recv on the caller's stream. */
#define MOE_EP_UNIQUE_ID_BYTES 128
int32_t moe_ep_unique_id(void* out, int32_t len);
int32_t moe_ep_init(moe_layer_t* layer, const void* unique_id, int32_t len);
/* Deadline of the host-side waits that can sit behind a collective (moe_synchronize, moe_get_losses,
 * moe_get_routing, moe_get_grad_f32, the *_host entries, the count read-back of the ncclSend/ncclRecv
 * transport).  Such a wait polls the stream; when `milliseconds` pass without it finishing (a rank of the
 * group never arrived or is stuck), the library aborts the communicator, so that the NCCL kernels waiting
 * for the missing rank end, poisons the handle and returns MOE_TIMEOUT: fail closed, as the reference's
 * device context does after any error (gpu_transformer.rs:160-195).  Default 600000 (ten minutes); 0 waits
 * for ever.  The reference is single-device and has no counterpart. */
int32_t moe_ep_set_deadline_ms(moe_layer_t* layer, int64_t milliseconds);
/* Optional peer transport.  Each rank exports CUDA IPC handles of its four receive buffers
 * (MOE_EP_EXPORT_BYTES bytes); every rank imports the handles of every rank, its own included.
 * Once all are imported, the dispatch kernels store rows straight into the owner's buffer and the
 * combine kernels load rows straight from it over NVLink, with NCCL only for the count exchange,
 * the barriers and the gradient all-reduce.  Without it the rows travel by ncclSend/ncclRecv. */
#define MOE_EP_EXPORT_BYTES 256
int32_t moe_ep_export_buffers(moe_layer_t* layer, void* out, int32_t len);
int32_t moe_ep_import_buffers(moe_layer_t* layer, int32_t rank, const void* handles, int32_t len);
/* Host-only helper (no device needed): the exchange plan of `rank` from the gathered
 * count matrix counts_all[ranks][num_experts].  Outputs: send_off[E+1], recv_row[ranks*E/ranks],
 * local_row0 / local_tiles / local_counts [E/ranks + 1].  Returns the padded local row total, -1 on bad arguments. */
int32_t moe_ep_plan(const int32_t* counts_all, int32_t ranks, int32_t num_experts, int32_t rank, int32_t* send_off,
                    int32_t* recv_row, int32_t* local_row0, int32_t* local_tiles, int32_t* local_counts);

/* Routing without allocation.  This entry has no counterpart in the reference; it exists for
 * callers that may not let a library allocate device memory: a runtime that gave the whole device
 * to its own arena and works under a fixed budget, or a serving loop that cannot afford the
 * device-wide synchronisation a cudaMalloc implies.  It performs the routing step only, from given
 * router logits: softmax + log-sum-exp, dropless top-k with renormalised gates, per-expert counts,
 * and the weighted load-balancing and z losses (same results as moe_forward_from_logits followed by
 * moe_get_routing / moe_get_losses).  Every input and output is a caller-owned device buffer:
 *   logits [tokens, E] f32, valid optional [tokens] bytes;
 *   probabilities [tokens, E], log_sum_exp [tokens], expert_of / gates [tokens*k], counts [E], losses [2].
 * The scratch between its two kernels is a static array inside the library image (about 134 KB on
 * every GPU that loads the library, until the process exits), hence the limits below; a larger
 * problem is rejected with MOE_INVALID_INPUT.  It calls no allocation routine.  The first call on a
 * device looks up the array's device address (cudaGetSymbolAddress); make that call before any
 * stream capture begins.  All calls on one device share the array: two calls that overlap on the GPU
 * (different streams, no dependency) race on it.  Nothing in it has to be cleared between calls,
 * because each call writes every word it later reads.  Host side: the entry is not thread safe in the
 * sense above (callers serialise their launches); the one piece of host state, the per-device table of the
 * array's address, is written without a lock, which is harmless because every thread that fills an entry
 * stores the same value.  `message` (optional) receives the error text. */
#define MOE_ROUTE_NOALLOC_MAX_TOKENS 16384
#define MOE_ROUTE_NOALLOC_MAX_EXPERTS 64
int32_t moe_route_noalloc(const float* logits_dev, const uint8_t* valid_dev, int32_t tokens, int32_t num_experts,
                          int32_t experts_per_token, float aux_loss_weight, float router_z_loss_weight,
                          float* probabilities_dev, float* log_sum_exp_dev, int32_t* expert_of_dev, float* gates_dev,
                          int32_t* counts_dev, float* losses_dev, void* stream, char* message, int32_t message_len);

/* ---- low-rank adapters (LoRA) on the expert projections ------------------------------------------
 * TransformerLm::add_lora / merge_lora over this layer (transformer.rs, `Lora` in param.rs:635-714,
 * MoeLayer::lora_linears_mut in moe.rs:502-514): every gate, up and down projection of the routed
 * experts this handle owns and of the shared expert gets an adapter
 *     W_eff = W + (alpha / rank) * up * down,   down [rank, in],  up [out, rank]   (f32, host pointers)
 * the router gets none, and while adapters are attached the base weights are frozen: moe_step_adam
 * moves the adapters only.  The adapter is folded into the compute copy of the weights when it or a
 * base weight changed (once per optimizer step), as the reference's device path does
 * (gpu_model.rs:1390-1428); forward and backward run the same kernels as without adapters.
 * moe_get_grad_f32 keeps returning dL/dW_eff; moe_lora_get_grad returns
 *     d down = scale * up^T * dL/dW_eff        d up = scale * dL/dW_eff * down^T
 * (what Lora::backward accumulates, param.rs:690-709).  Adapters start as zeros: set `down` (the
 * reference initialises it He-uniform from its own RNG) and leave `up` zero to start from the base
 * model.  moe_lora_merge adds the adapters into the master weights and removes them.
 * Errors: MOE_INVALID_CONFIG for an int8 or inference-only handle, rank outside 1..64, a second attach
 * or a call without adapters; MOE_INVALID_INPUT for the router or an expert this handle does not own. */
int32_t moe_lora_attach(moe_layer_t* layer, int32_t rank, float alpha);
int32_t moe_lora_set(moe_layer_t* layer, int32_t which, int32_t expert, const float* down, const float* up);
int32_t moe_lora_get(moe_layer_t* layer, int32_t which, int32_t expert, float* down, float* up);
int32_t moe_lora_get_grad(moe_layer_t* layer, int32_t which, int32_t expert, float* grad_down, float* grad_up);
int32_t moe_lora_merge(moe_layer_t* layer);

/* Device synchronisation for timing (TransformerLm::synchronize, transformer.rs:1323-1334). */
int32_t moe_synchronize(moe_layer_t* layer);

/* ---- binary snapshots -------------------------------------------------------------------------
 * Readers for the two files the reference writes beside a model, so that a MoE layer can be filled
 * straight from them (no whole-model load, no dequantize-then-requantize detour for int8 files):
 *   weights   "RBWTS001"  TransformerLm::save_bin / load_bin (transformer.rs:1809-1932):
 *             magic, u64 header length, JSON header {config, optimizer, optimizer_step, precision},
 *             u64 parameter count, then per parameter u64 rows, u64 cols and either rows*cols f32
 *             (precision "F32") or, per row, an f32 scale followed by `cols` int8 values ("Q8");
 *   moments   "RBOPT001"  save_optimizer_state / load_optimizer_state (transformer.rs:1675-1753):
 *             magic, u64 parameter count, u64 step, then per parameter u64 rows, u64 cols and the
 *             first and second Adam moment as f32 (a frozen parameter is written as 0 x 0).
 * All integers and floats are little endian.  Parameters come in TransformerLm::params_mut order
 * (transformer.rs:1620-1630): embedding; per block attention norm, query, key, value, output,
 * feed-forward norm, then the feed-forward (dense: gate, up, down — or up, down for the GELU
 * variant; MoE: router, every expert's gate, up, down, then the shared expert's); final norm;
 * the LM head unless the embeddings are tied.  In the file of a model with LoRA adapters attached
 * (config.lora set) every adapted projection (attention and feed-forward, not the router, embedding or
 * LM head) is followed by its `down` [rank, in] and `up` [out, rank]. */
typedef struct moe_snapshot_info {
  int64_t vocab_size, d_model, n_layers, n_heads, n_kv_heads, head_dim, d_ff, moe_d_ff;
  int64_t num_experts, experts_per_token, max_seq_len;
  int32_t shared_expert, tie_embeddings, causal;
  float aux_loss_weight, router_z_loss_weight, rope_base, rmsnorm_eps;
  int32_t precision;            /* MOE_PRECISION_F32 or MOE_PRECISION_Q8: how the file stores weights */
  int32_t n_moe_layers;         /* entries used in moe_layers */
  int32_t moe_layers[256];      /* block indices with a MoE feed-forward, ascending */
  int64_t optimizer_step;
  int64_t parameter_count;      /* as written in the file */
  int32_t dense_ffn_params;     /* 3 (SwiGLU) or 2 (GELU) projections per dense feed-forward, 0 if none */
  int32_t lora_rank;            /* 0, or config.lora.rank: every adapted projection is followed by its down and up */
  float lora_alpha;
} moe_snapshot_info_t;

/* Parses the header of a weight file.  Host only (no GPU needed).  `message` (optional) receives
 * the error text: InvalidSnapshot for a wrong magic, truncated file or inconsistent counts. */
int32_t moe_snapshot_info(const char* weights_path, moe_snapshot_info_t* out, char* message, int32_t message_len);

/* Fills the layer from block `block_index` of a weight file.  The handle's shape (d_model, experts,
 * d_ff, shared expert) must match the file's configuration.  Any combination of file precision and
 * handle precision works: an int8 file feeds an int8 handle row for row (scales and bytes as stored;
 * the router, which stays f32 in an int8 handle, is dequantized), an int8 file is dequantized for an
 * f32 / bf16 handle exactly as load_bin does (value = int8 * scale), an f32 file is quantized for an
 * int8 handle on the reference's grid (scale = max|row| / 127, round half away from zero, clamp to
 * +-127; transformer.rs:514-519, quantized.rs:8-12).  An expert-parallel handle takes its own experts only.
 * Adapters in the file are loaded into the layer's adapters when it has some of the same rank and alpha
 * (moe_lora_attach first), otherwise only the base weights are taken. */
int32_t moe_load_snapshot_layer(moe_layer_t* layer, const char* weights_path, int32_t block_index);

/* Restores the Adam moments of block `block_index` from a moments file; `info` is the configuration
 * of the matching weight file (the moments file has no header of its own).  Returns the file's step
 * counter in *step (optional). */
int32_t moe_load_optimizer_layer(moe_layer_t* layer, const char* moments_path, const moe_snapshot_info_t* info,
                                 int32_t block_index, int64_t* step);

/* Fills the adapters of block `block_index` from an adapter file ("RBLOR001", TransformerLm::save_lora /
 * load_lora, transformer.rs:1109-1202): magic, u64 header length, JSON LoraConfig {rank, alpha, seed}, u64
 * parameter count, then per adapter matrix u64 rows, u64 cols and f32 data; the adapters of a model are
 * written block by block, four attention projections then the feed-forward ones (for a MoE block every
 * expert's gate, up, down and the shared expert's; never the router), `down` before `up`.  As load_lora
 * does, the layer must already carry adapters of the file's rank and alpha (moe_lora_attach), and any
 * mismatch fails without loading part of an adapter file's block.  `info` as for the moments file. */
int32_t moe_load_lora_layer(moe_layer_t* layer, const char* lora_path, const moe_snapshot_info_t* info,
                            int32_t block_index);

#ifdef __cplusplus
}
#endif
#endif /* MOE_B200_H */
