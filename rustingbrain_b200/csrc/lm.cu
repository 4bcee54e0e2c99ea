// The language model around the MoE layer (C ABI of include/transformer_b200.h): embedding, decoder blocks
// (RMSNorm -> causal grouped-query attention -> residual -> RMSNorm -> dense SwiGLU or MoE -> residual), final
// norm, output head fused with the cross-entropy, the backward pass of all of it, and Adam.
//
// Every matrix product is a launch of the grouped tcgen05 GEMM (gemm_tc.cu); the MoE blocks are moe_layer_t
// handles (moe_api.cu) created and driven from here.  Attention runs as products over head-major row groups
// (one group per batch entry and key/value head, see lm_kernels.cuh) with the probabilities kept for the
// backward pass, which is the reference's own formulation (attention.rs:305-341, 404-556): scores and
// probabilities cross HBM once each per direction, a few hundred MB per layer at the 55M model's shapes.
// Nothing here falls back to the host.

#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <cmath>
#include <new>
#include <string>
#include <vector>

#include "../../include/moe_b200.h"
#include "../../include/rmsnorm_b200.h"
#include "../../include/transformer_b200.h"
#include "gemm_tc.cuh"
#include "kernels.cuh"
#include "lm_kernels.cuh"

using namespace moe;

struct lm_block {
  bool is_moe = false;
  moe_layer_t* moe = nullptr;
  // arena offsets (floats)
  long long attn_norm = 0, wqkv = 0, wo = 0, ffn_norm = 0, wgu = 0, wd = 0;
  // saved activations (bf16)
  bf16 *xn1 = nullptr, *res = nullptr, *xn2 = nullptr, *merged = nullptr, *gu = nullptr, *h = nullptr;
  bf16 *q_hm = nullptr, *k_hm = nullptr, *v_hm = nullptr, *probs = nullptr;   // sized per batch shape
};

struct lm_model {
  lm_config_t cfg{};
  int device = 0, sm_count = 0;
  std::string err;
  int status = 0;
  int d = 0, H = 0, Hkv = 0, hd = 0, V = 0, V_pad = 0, L = 0, QN = 0, Fd = 0, Fd_pad = 0, R = 0;
  long long n_params = 0, off_emb = 0, off_final_norm = 0, off_head = 0;
  float *w = nullptr, *g = nullptr, *m = nullptr, *v = nullptr;
  bf16* wb = nullptr;
  bool grad_valid = false;
  long long step = 0;
  std::vector<lm_block> blocks;
  std::vector<bf16*> xs;            // block inputs: xs[l], and the last block's output xs[L]
  float *cos_t = nullptr, *sin_t = nullptr;
  // temporaries
  bf16 *qkv = nullptr, *tmp = nullptr, *dqkv = nullptr, *d_merged = nullptr, *dgu = nullptr;
  bf16 *dxa = nullptr, *dxb = nullptr, *dxn = nullptr, *xf = nullptr, *dxf = nullptr, *logits = nullptr;
  bf16 *scores = nullptr, *o_hm = nullptr, *do_hm = nullptr, *dq_hm = nullptr;
  float *dk_hm = nullptr, *dv_hm = nullptr;
  long long attn_q_rows = 0, attn_s_pad = 0, attn_kv_rows = 0;   // current capacity of the attention buffers
  float *row_loss = nullptr, *loss_dev = nullptr, *stage = nullptr;
  long long stage_elems = 0;
  int *targets = nullptr, *first = nullptr, *next = nullptr, *meta_table = nullptr, *attn_meta = nullptr, *error_flag = nullptr;
  uint32_t* ids = nullptr;
  uint8_t* valid = nullptr;
  void* rms_scratch = nullptr;
  uint32_t* ids_pin = nullptr; int* targets_pin = nullptr; uint8_t* valid_pin = nullptr; float* loss_pin = nullptr;
  int *first_pin = nullptr, *next_pin = nullptr;
  std::vector<int> last_seen;       // per vocabulary id: last row that held it (host scratch of the scatter chains)
  float* split_scratch = nullptr;   // partial weight gradients of the row-split products
  long long split_elems = 0;
  int* split_meta = nullptr;        // group tables of the row-split products: SPLIT_SLOTS tables of 32 entries
  struct SplitKey { int splits, chunk, padded; };
  std::vector<SplitKey> split_keys; // which (splits, chunk, padded) each filled slot holds
  cudaStream_t st = nullptr;
  cudaEvent_t ev[5] = {};
  float last_ms[4] = {0, 0, 0, 0};
  std::vector<void*> allocations;
  std::vector<void*> attn_allocations;
};

namespace {

int lfail(lm_model* M, int status, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (M) { M->err = buf; if (status == MOE_CUDA_ERROR || status == MOE_TIMEOUT || status == MOE_OUT_OF_MEMORY) M->status = status; }
  return status;
}

#define LCK(call)                                                                                   \
  do {                                                                                              \
    cudaError_t e_ = (call);                                                                        \
    if (e_ != cudaSuccess)                                                                          \
      return lfail(M, e_ == cudaErrorMemoryAllocation ? MOE_OUT_OF_MEMORY : MOE_CUDA_ERROR,         \
                   "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__);     \
  } while (0)

#define LENTER(M)                                                                                   \
  do {                                                                                              \
    if (!(M)) return MOE_INVALID_INPUT;                                                             \
    if ((M)->status != MOE_OK) return MOE_POISONED;                                                 \
    if (cudaSetDevice((M)->device) != cudaSuccess) return lfail((M), MOE_CUDA_ERROR, "cudaSetDevice failed"); \
  } while (0)

long long align_up(long long v, long long a) { return (v + a - 1) / a * a; }

int lalloc(lm_model* M, void** p, long long bytes, bool zero, std::vector<void*>* list = nullptr) {
  if (bytes <= 0) bytes = 16;
  LCK(cudaMalloc(p, (size_t)bytes));
  (list ? *list : M->allocations).push_back(*p);
  if (zero) LCK(cudaMemset(*p, 0, (size_t)bytes));
  return MOE_OK;
}
#define LA(ptr, bytes, zero)                                           \
  do {                                                                 \
    int rc_ = lalloc(M, (void**)&(ptr), (long long)(bytes), (zero));   \
    if (rc_ != MOE_OK) return rc_;                                     \
  } while (0)

int validate(const lm_config_t* c, char* msg, int len) {
  auto say = [&](const char* fmt, ...) {
    if (msg && len > 0) { va_list ap; va_start(ap, fmt); vsnprintf(msg, len, fmt, ap); va_end(ap); }
    return (int)MOE_INVALID_CONFIG;
  };
  if (!c) return say("null config");
  // TransformerConfig::validate, transformer.rs:132-172
  const struct { const char* name; int v; } nz[] = {{"vocab_size", c->vocab_size}, {"d_model", c->d_model}, {"n_layers", c->n_layers},
      {"n_heads", c->n_heads}, {"n_kv_heads", c->n_kv_heads}, {"head_dim", c->head_dim}, {"d_ff", c->d_ff}, {"max_seq_len", c->max_seq_len}};
  for (auto& f : nz) if (f.v <= 0) return say("%s must be non-zero", f.name);
  if (c->n_heads % c->n_kv_heads != 0 || c->n_kv_heads > c->n_heads)
    return say("n_heads (%d) must be a multiple of n_kv_heads (%d)", c->n_heads, c->n_kv_heads);
  if (c->head_dim % 2 != 0) return say("head_dim must be even for rotary embeddings, got %d", c->head_dim);
  if (c->n_layers > 64) return say("at most 64 layers");
  if (c->n_layers < 64 && (c->moe_layer_mask >> c->n_layers) != 0) {
    int layer = c->n_layers;
    while (!((c->moe_layer_mask >> layer) & 1)) ++layer;
    return say("moe_layers names layer %d, but the model has %d layers", layer, c->n_layers);
  }
  if (c->moe_layer_mask != 0) {
    if (c->num_experts <= 0) return say("a MoE layer needs at least one expert");
    if (c->experts_per_token <= 0 || c->experts_per_token > c->num_experts)
      return say("experts_per_token must be between 1 and num_experts (%d), got %d", c->num_experts, c->experts_per_token);
    if (c->moe_d_ff <= 0) return say("expert d_ff must be non-zero");
  }
  // shape rules of the tensor-core products
  if (c->d_model % 32 != 0 || c->head_dim % 32 != 0 || c->d_ff % 32 != 0)
    return say("d_model, head_dim and d_ff must be multiples of 32 (got %d, %d, %d)", c->d_model, c->head_dim, c->d_ff);
  if (c->max_batch_rows < 2) return say("max_batch_rows must be at least 2");
  return MOE_OK;
}

bool layer_is_moe(const lm_config_t& c, int l) { return ((c.moe_layer_mask >> l) & 1) != 0; }

// group table of a dense product over `rows` token rows: {row0[0], row0[1], tile_start[0], tile_start[1]}
__global__ void meta_table_kernel(int* table, int max_rows) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t > max_rows) return;
  const int rows = round_up(t, GROUP_ALIGN);
  table[4 * t] = 0; table[4 * t + 1] = rows; table[4 * t + 2] = 0; table[4 * t + 3] = rows / GROUP_ALIGN;
}

// ---------------------------------------------------------------------------
// product wrappers (one group over the token rows unless a meta is given)
// ---------------------------------------------------------------------------
struct Meta { const int* row0; const int* tstart; int groups; };
Meta dense_meta(lm_model* M, int rows) { return Meta{M->meta_table + 4 * rows, M->meta_table + 4 * rows + 2, 1}; }

// out[rows, N] = A[rows, K] * B_g[N, K]^T
int mm_nt(lm_model* M, const void* A, long long a_rows, int K, const void* B, int N, Meta mt, void* out, long long ld,
          int epi = tc::EPI_STORE, void* out1 = nullptr, long long ld1 = 0, int causal = 0, int causal_kind = 0) {
  tc::GemmArgs a{};
  a.group_row0 = mt.row0; a.tile_start = mt.tstart; a.n_groups = mt.groups; a.error_flag = M->error_flag;
  a.N = N; a.K = K; a.out0 = out; a.ld0 = ld; a.out1 = out1; a.ld1 = ld1; a.causal = causal; a.causal_kind = causal_kind;
  LCK(tc::gemm_rows_nt(tc::Operand{A, a_rows, K, 1}, tc::Operand{B, N, K, mt.groups}, a, epi, M->sm_count, M->st));
  return MOE_OK;
}
// out[rows, N] = A[rows, K] * B_g[K, N]
int mm_nn(lm_model* M, const void* A, long long a_rows, int K, const void* B, int N, Meta mt, void* out, long long ld,
          int epi = tc::EPI_STORE, const void* aux = nullptr, long long ldaux = 0, int causal = 0, int causal_kind = 0) {
  tc::GemmArgs a{};
  a.group_row0 = mt.row0; a.tile_start = mt.tstart; a.n_groups = mt.groups; a.error_flag = M->error_flag;
  a.N = N; a.K = K; a.out0 = out; a.ld0 = ld; a.aux = aux; a.ldaux = ldaux; a.causal = causal; a.causal_kind = causal_kind;
  LCK(tc::gemm_rows_nn(tc::Operand{A, a_rows, K, 1}, tc::Operand{B, K, N, mt.groups}, a, epi, M->sm_count, M->st));
  return MOE_OK;
}
// C_g[Mo, N] (+)= A[rows_g, Mo]^T * B[rows_g, N]   (f32 out)
int mm_tn(lm_model* M, const void* A, long long a_rows, int Mo, const void* B, long long b_rows, int N, Meta mt, float* out,
          long long ld, long long group_stride, int accumulate, int causal = 0) {
  tc::GemmArgs a{};
  a.group_row0 = mt.row0; a.n_groups = mt.groups; a.error_flag = M->error_flag;
  a.M = Mo; a.N = N; a.out0 = out; a.ld0 = ld; a.group_stride0 = group_stride; a.accumulate = accumulate; a.causal = causal;
  LCK(tc::gemm_rows_tn(tc::Operand{A, a_rows, Mo, 1}, tc::Operand{B, b_rows, N, 1}, a, M->sm_count, M->st));
  return MOE_OK;
}
#define RC_(call)                        \
  do {                                   \
    const int rc_ = (call);              \
    if (rc_ != MOE_OK) return rc_;       \
  } while (0)
constexpr int SPLIT_SLOTS = 16;
// Row ranges of a product whose rows are the reduction, cut into `splits` chunks: meta[g] = min(g * chunk, padded).
__global__ void split_rows_kernel(int* meta, int splits, int chunk, int padded) {
  const int g = threadIdx.x;
  if (g <= splits) meta[g] = min(g * chunk, padded);
}
// dst[i] += sum over s (ascending) of part[s][i]
__global__ void add_partials_kernel(float* __restrict__ dst, const float* __restrict__ part, long long n, int splits) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = 0.f;
  for (int s = 0; s < splits; ++s) acc += part[(long long)s * n + i];
  dst[i] += acc;
}

// Weight gradient of a dense projection over the token rows: out[Mo, N] += A[rows, Mo]^T * B[rows, N].
// The output is a handful of tiles and the token rows are the reduction, so with one group most SMs idle.  The
// rows are cut into chunks (one group each, partial results in scratch) so that every SM has a tile; the chunks
// are then added in order, which keeps the result independent of scheduling.
int mm_tn_dense(lm_model* M, const void* A, int rows, int Mo, const void* B, int N, float* out, long long ld) {
  const int tiles = ceil_div(Mo, tc::BM) * ceil_div(N, tc::BN);
  const int padded = round_up(rows, GROUP_ALIGN);
  int splits = std::min(16, std::max(1, M->sm_count / std::max(1, tiles)));
  const int chunk = round_up(ceil_div(padded, splits), GROUP_ALIGN);
  splits = ceil_div(padded, chunk);
  if (splits <= 1 || ld != N || (long long)splits * Mo * N > M->split_elems)
    return mm_tn(M, A, rows, Mo, B, rows, N, dense_meta(M, rows), out, ld, 0, 1);
  // the table depends on (splits, chunk, padded) only: a step uses a handful of them, each written once
  int slot = -1;
  for (size_t i = 0; i < M->split_keys.size(); ++i) {
    const auto& k = M->split_keys[i];
    if (k.splits == splits && k.chunk == chunk && k.padded == padded) { slot = (int)i; break; }
  }
  if (slot < 0) {
    slot = M->split_keys.size() < (size_t)SPLIT_SLOTS - 1 ? (int)M->split_keys.size() : SPLIT_SLOTS - 1;   // the last slot is rewritten
    split_rows_kernel<<<1, 32, 0, M->st>>>(M->split_meta + 32 * slot, splits, chunk, padded); count_launch();
    if (slot < SPLIT_SLOTS - 1) M->split_keys.push_back({splits, chunk, padded});
  }
  RC_(mm_tn(M, A, rows, Mo, B, rows, N, Meta{M->split_meta + 32 * slot, nullptr, splits}, M->split_scratch, N, (long long)Mo * N, 0));
  const long long n = (long long)Mo * N;
  add_partials_kernel<<<(unsigned)((n + 255) / 256), 256, 0, M->st>>>(out, M->split_scratch, n, splits); count_launch();
  LCK(cudaGetLastError());
  return MOE_OK;
}
#define RC(call)                         \
  do {                                   \
    const int rc_ = (call);              \
    if (rc_ != MOE_OK) return rc_;       \
  } while (0)

int norm_fwd(lm_model* M, const bf16* x, long long w_off, bf16* y, int rows) {
  char msg[160];
  const int rc = rmsnorm_forward(x, M->w + w_off, y, rows, M->d, M->cfg.rmsnorm_eps, MOE_PRECISION_BF16, M->st, msg, sizeof msg);
  return rc == MOE_OK ? MOE_OK : lfail(M, rc, "rmsnorm_forward: %s", msg);
}
int norm_bwd(lm_model* M, const bf16* x, long long w_off, const bf16* gy, bf16* gx, int rows) {
  char msg[160];
  const int rc = rmsnorm_backward(x, M->w + w_off, gy, gx, M->g + w_off, M->rms_scratch, rows, M->d, M->cfg.rmsnorm_eps,
                                  MOE_PRECISION_BF16, M->st, msg, sizeof msg);
  return rc == MOE_OK ? MOE_OK : lfail(M, rc, "rmsnorm_backward: %s", msg);
}

int moe_rc(lm_model* M, lm_block& b, int rc) {
  if (rc == MOE_OK) return MOE_OK;
  return lfail(M, rc, "MoE layer: %s", moe_last_error(b.moe));
}

}  // namespace

// ---------------------------------------------------------------------------
// life cycle
// ---------------------------------------------------------------------------
extern "C" {

int32_t lm_config_validate(const lm_config_t* config, char* message, int32_t message_len) {
  if (message && message_len > 0) message[0] = 0;
  return validate(config, message, message_len);
}

int32_t lm_parameter_counts(const lm_config_t* c, int64_t* total_out, int64_t* active_out) {
  if (!c) return MOE_INVALID_INPUT;
  // TransformerConfig::parameter_counts, transformer.rs:195-235
  const int64_t d = c->d_model;
  const int64_t query = d * c->n_heads * c->head_dim, key_value = 2 * d * c->n_kv_heads * c->head_dim;
  const int64_t attention = 2 * query + key_value, norms = 2 * d;
  const int64_t dense_ffn = 3 * d * c->d_ff, expert = 3 * d * c->moe_d_ff, shared = c->shared_expert ? expert : 0;
  const int64_t router = (int64_t)c->num_experts * d;
  const int64_t moe_total = router + c->num_experts * expert + shared, moe_active = router + c->experts_per_token * expert + shared;
  int64_t total = (int64_t)c->vocab_size * d + d + (c->tie_embeddings ? 0 : (int64_t)c->vocab_size * d);
  int64_t active = total;
  for (int l = 0; l < c->n_layers; ++l) {
    total += attention + norms; active += attention + norms;
    if (layer_is_moe(*c, l)) { total += moe_total; active += moe_active; }
    else { total += dense_ffn; active += dense_ffn; }
  }
  if (total_out) *total_out = total;
  if (active_out) *active_out = active;
  return MOE_OK;
}

int32_t lm_create(const lm_config_t* config, lm_model_t** out) {
  if (!out) return MOE_INVALID_INPUT;
  *out = nullptr;
  lm_model* M = new (std::nothrow) lm_model;
  if (!M) return MOE_OUT_OF_MEMORY;
  *out = M;   // returned even on failure so that the caller can read lm_last_error, then destroy
  char msg[256];
  if (validate(config, msg, sizeof msg) != MOE_OK) { M->err = std::string("InvalidConfig: ") + msg; return MOE_INVALID_CONFIG; }
  M->cfg = *config;
  const lm_config_t& c = M->cfg;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0 || c.device < 0 || c.device >= ndev) {
    cudaGetLastError();
    return lfail(M, MOE_UNSUPPORTED, "Unsupported: no usable CUDA device (there is no host fallback)");
  }
  cudaDeviceProp prop;
  LCK(cudaGetDeviceProperties(&prop, c.device));
  if (prop.major != 10) return lfail(M, MOE_UNSUPPORTED, "Unsupported: built for sm_100a only");
  M->device = c.device; M->sm_count = prop.multiProcessorCount;
  LCK(cudaSetDevice(c.device));
  LCK(cudaStreamCreateWithFlags(&M->st, cudaStreamNonBlocking));
  for (auto& e : M->ev) LCK(cudaEventCreate(&e));

  M->d = c.d_model; M->H = c.n_heads; M->Hkv = c.n_kv_heads; M->hd = c.head_dim; M->V = c.vocab_size;
  M->V_pad = round_up(c.vocab_size, 32); M->L = c.n_layers; M->QN = (c.n_heads + 2 * c.n_kv_heads) * c.head_dim;
  M->Fd = c.d_ff; M->Fd_pad = round_up(c.d_ff, GU_BLOCK); M->R = round_up(c.max_batch_rows, GROUP_ALIGN);
  const long long d = M->d, R = M->R, QN = M->QN, HD = (long long)M->H * M->hd, Fp = M->Fd_pad;

  // parameter arena of everything that is not inside a MoE handle
  long long o = 0;
  M->off_emb = o; o = align_up(o + (long long)M->V_pad * d, 128);
  M->off_final_norm = o; o = align_up(o + d, 128);
  M->off_head = o; if (!c.tie_embeddings) o = align_up(o + (long long)M->V_pad * d, 128);
  M->blocks.resize(M->L);
  for (int l = 0; l < M->L; ++l) {
    lm_block& b = M->blocks[l];
    b.is_moe = layer_is_moe(c, l);
    b.attn_norm = o; o = align_up(o + d, 128);
    b.wqkv = o; o = align_up(o + QN * d, 128);
    b.wo = o; o = align_up(o + d * HD, 128);
    b.ffn_norm = o; o = align_up(o + d, 128);
    if (!b.is_moe) {
      b.wgu = o; o = align_up(o + 2 * Fp * d, 128);
      b.wd = o; o = align_up(o + d * Fp, 128);
    }
  }
  M->n_params = o;
  LA(M->w, o * 4, true); LA(M->g, o * 4, true); LA(M->m, o * 4, true); LA(M->v, o * 4, true); LA(M->wb, o * 2, true);
  M->stage_elems = std::max<long long>((long long)M->V_pad * d, std::max(QN * d, 2 * Fp * d));
  LA(M->stage, M->stage_elems * 4, false);

  // RoPE tables, f32 arithmetic as Rope::new (rope.rs:77-90)
  {
    const int half = M->hd / 2;
    std::vector<float> co((size_t)c.max_seq_len * half), si((size_t)c.max_seq_len * half);
    for (int p = 0; p < c.max_seq_len; ++p)
      for (int ch = 0; ch < half; ++ch) {
        const float frequency = powf(c.rope_base, -2.0f * (float)ch / (float)M->hd);
        const float angle = (float)p * frequency;
        co[(size_t)p * half + ch] = cosf(angle);
        si[(size_t)p * half + ch] = sinf(angle);
      }
    LA(M->cos_t, co.size() * 4, false); LA(M->sin_t, si.size() * 4, false);
    LCK(cudaMemcpy(M->cos_t, co.data(), co.size() * 4, cudaMemcpyHostToDevice));
    LCK(cudaMemcpy(M->sin_t, si.data(), si.size() * 4, cudaMemcpyHostToDevice));
  }

  // activations kept for the backward pass, and temporaries (rows padded to the tile height, zeroed once:
  // rows past a batch's own stay zero, the products over padded extents are exact)
  M->xs.resize(M->L + 1);
  for (int l = 0; l <= M->L; ++l) LA(M->xs[l], R * d * 2, true);
  for (int l = 0; l < M->L; ++l) {
    lm_block& b = M->blocks[l];
    LA(b.xn1, R * d * 2, true); LA(b.res, R * d * 2, true); LA(b.xn2, R * d * 2, true); LA(b.merged, R * HD * 2, true);
    if (!b.is_moe) { LA(b.gu, R * 2 * Fp * 2, true); LA(b.h, R * Fp * 2, true); }
  }
  const long long wide = std::max<long long>(std::max(d, HD), 2 * Fp);
  LA(M->qkv, R * QN * 2, true); LA(M->tmp, R * wide * 2, true); LA(M->dqkv, R * QN * 2, true); LA(M->d_merged, R * HD * 2, true);
  LA(M->dgu, R * 2 * Fp * 2, true);
  LA(M->dxa, R * d * 2, true); LA(M->dxb, R * d * 2, true); LA(M->dxn, R * d * 2, true); LA(M->xf, R * d * 2, true); LA(M->dxf, R * d * 2, true);
  LA(M->logits, R * (long long)M->V_pad * 2, true);
  LA(M->row_loss, R * 4, true); LA(M->loss_dev, 16, true);
  LA(M->targets, R * 4, true); LA(M->first, R * 4, true); LA(M->next, R * 4, true); LA(M->ids, R * 4, true); LA(M->valid, R, true);
  LA(M->meta_table, (R + 1) * 16, false); LA(M->attn_meta, 2 * (MAX_EXPERTS + 2) * 4, true); LA(M->error_flag, 4, true);
  LA(M->rms_scratch, std::max<long long>(16, rmsnorm_scratch_bytes((int)R, (int)d)), false);
  meta_table_kernel<<<(unsigned)((R + 256) / 256), 256>>>(M->meta_table, (int)R);
  LCK(cudaGetLastError());
  LCK(cudaMallocHost((void**)&M->ids_pin, (size_t)R * 4)); LCK(cudaMallocHost((void**)&M->targets_pin, (size_t)R * 4));
  LCK(cudaMallocHost((void**)&M->valid_pin, (size_t)R)); LCK(cudaMallocHost((void**)&M->loss_pin, 16));
  LCK(cudaMallocHost((void**)&M->first_pin, (size_t)R * 4)); LCK(cudaMallocHost((void**)&M->next_pin, (size_t)R * 4));
  M->last_seen.assign(M->V, -1);
  M->split_elems = 16ll * std::max<long long>(std::max(QN, HD) * d, 2 * Fp * d);   // at most 16 partial results of the widest matrix
  LA(M->split_scratch, M->split_elems * 4, false); LA(M->split_meta, SPLIT_SLOTS * 32 * 4, true);

  // the MoE blocks: handles of the layer library, bf16 products over f32 master weights
  for (int l = 0; l < M->L; ++l) {
    lm_block& b = M->blocks[l];
    if (!b.is_moe) continue;
    moe_config_t mc{};
    mc.d_model = c.d_model; mc.num_experts = c.num_experts; mc.experts_per_token = c.experts_per_token; mc.d_ff = c.moe_d_ff;
    mc.shared_expert = c.shared_expert; mc.aux_loss_weight = c.aux_loss_weight; mc.router_z_loss_weight = c.router_z_loss_weight;
    mc.precision = MOE_PRECISION_BF16; mc.max_tokens = (int)R; mc.device = c.device; mc.training = 1; mc.ep_rank = 0; mc.ep_size = 1;
    const int rc = moe_create(&mc, &b.moe);
    if (rc != MOE_OK) return lfail(M, rc, "MoE layer %d: %s", l, b.moe ? moe_last_error(b.moe) : "moe_create failed");
  }
  LCK(cudaDeviceSynchronize());
  return MOE_OK;
}

void lm_destroy(lm_model_t* M) {
  if (!M) return;
  cudaSetDevice(M->device);
  cudaDeviceSynchronize();
  for (auto& b : M->blocks) if (b.moe) moe_destroy(b.moe);
  for (void* p : M->allocations) cudaFree(p);
  for (void* p : M->attn_allocations) cudaFree(p);
  if (M->ids_pin) cudaFreeHost(M->ids_pin);
  if (M->targets_pin) cudaFreeHost(M->targets_pin);
  if (M->valid_pin) cudaFreeHost(M->valid_pin);
  if (M->loss_pin) cudaFreeHost(M->loss_pin);
  if (M->first_pin) cudaFreeHost(M->first_pin);
  if (M->next_pin) cudaFreeHost(M->next_pin);
  for (auto& e : M->ev) if (e) cudaEventDestroy(e);
  if (M->st) cudaStreamDestroy(M->st);
  delete M;
}

const char* lm_last_error(const lm_model_t* M) { return M ? M->err.c_str() : "null model"; }

}  // extern "C"

// ---------------------------------------------------------------------------
// parameters
// ---------------------------------------------------------------------------
namespace {

struct Slot { long long off; int rows, cols, ld, row0, kind; };

// Where a parameter of the non-MoE part lives.  Returns MOE_OK, or an error with the reason set.
int find_slot(lm_model* M, int layer, int which, Slot* s) {
  const int d = M->d, HD = M->H * M->hd, KD = M->Hkv * M->hd;
  if (which == LM_EMBEDDING) { *s = {M->off_emb, M->V, d, d, 0, 0}; return MOE_OK; }
  if (which == LM_FINAL_NORM) { *s = {M->off_final_norm, 1, d, d, 0, 0}; return MOE_OK; }
  if (which == LM_HEAD) {
    if (M->cfg.tie_embeddings) return lfail(M, MOE_INVALID_INPUT, "InvalidInput: the output head is tied to the embedding");
    *s = {M->off_head, M->V, d, d, 0, 0};
    return MOE_OK;
  }
  if (layer < 0 || layer >= M->L) return lfail(M, MOE_INVALID_INPUT, "InvalidInput: layer %d of %d", layer, M->L);
  const lm_block& b = M->blocks[layer];
  switch (which) {
    case LM_ATTENTION_NORM: *s = {b.attn_norm, 1, d, d, 0, 0}; return MOE_OK;
    case LM_FFN_NORM: *s = {b.ffn_norm, 1, d, d, 0, 0}; return MOE_OK;
    case LM_WQ: *s = {b.wqkv, HD, d, d, 0, 0}; return MOE_OK;
    case LM_WK: *s = {b.wqkv, KD, d, d, HD, 0}; return MOE_OK;
    case LM_WV: *s = {b.wqkv, KD, d, d, HD + KD, 0}; return MOE_OK;
    case LM_WO: *s = {b.wo, d, HD, HD, 0, 0}; return MOE_OK;
    case LM_FFN_GATE:
    case LM_FFN_UP:
    case LM_FFN_DOWN:
      if (b.is_moe) return lfail(M, MOE_INVALID_INPUT, "InvalidInput: layer %d has a MoE feed-forward", layer);
      if (which == LM_FFN_DOWN) *s = {b.wd, d, M->Fd, M->Fd_pad, 0, 0};
      else *s = {b.wgu, M->Fd, d, d, 0, which == LM_FFN_GATE ? 1 : 2};
      return MOE_OK;
  }
  return lfail(M, MOE_INVALID_INPUT, "InvalidInput: unknown parameter id %d", which);
}

bool is_moe_param(int which) { return which >= LM_MOE_ROUTER && which <= LM_MOE_SHARED_DOWN; }

int moe_block(lm_model* M, int layer, lm_block** out) {
  if (layer < 0 || layer >= M->L || !M->blocks[layer].is_moe)
    return lfail(M, MOE_INVALID_INPUT, "InvalidInput: layer %d has no MoE feed-forward", layer);
  *out = &M->blocks[layer];
  return MOE_OK;
}

int read_slot(lm_model* M, const float* arena, int layer, int which, float* host, int rows, int cols, bool zero) {
  Slot s;
  RC(find_slot(M, layer, which, &s));
  if ((long long)rows * cols != (long long)s.rows * s.cols || (s.rows > 1 && (rows != s.rows || cols != s.cols)))
    return lfail(M, MOE_INVALID_INPUT, "InvalidInput: parameter shape mismatch (expected %d x %d)", s.rows, s.cols);
  if (!host) return lfail(M, MOE_INVALID_INPUT, "InvalidInput: null destination");
  LCK(cudaStreamSynchronize(M->st));
  if (zero) { memset(host, 0, (size_t)rows * cols * 4); return MOE_OK; }
  LCK(lm::launch_unpack(arena + s.off, M->stage, s.rows, s.cols, s.ld, s.row0, s.kind, M->st));
  LCK(cudaMemcpyAsync(host, M->stage, (size_t)s.rows * s.cols * 4, cudaMemcpyDeviceToHost, M->st));
  LCK(cudaStreamSynchronize(M->st));
  return MOE_OK;
}

}  // namespace

extern "C" {

int32_t lm_set_param(lm_model_t* M, int32_t layer, int32_t which, int32_t expert, const float* host, int32_t rows, int32_t cols) {
  LENTER(M);
  if (!host) return lfail(M, MOE_INVALID_INPUT, "InvalidInput: null source");
  if (is_moe_param(which)) {
    lm_block* b;
    RC(moe_block(M, layer, &b));
    LCK(cudaStreamSynchronize(M->st));
    return moe_rc(M, *b, moe_set_weight_f32(b->moe, which - LM_MOE_ROUTER, expert, host, rows, cols));
  }
  Slot s;
  RC(find_slot(M, layer, which, &s));
  if ((long long)rows * cols != (long long)s.rows * s.cols || (s.rows > 1 && (rows != s.rows || cols != s.cols)))
    return lfail(M, MOE_INVALID_INPUT, "InvalidInput: parameter shape mismatch (expected %d x %d)", s.rows, s.cols);
  LCK(cudaStreamSynchronize(M->st));   // a step may still be reading the weights
  LCK(cudaMemcpyAsync(M->stage, host, (size_t)s.rows * s.cols * 4, cudaMemcpyHostToDevice, M->st));
  LCK(lm::launch_pack(M->stage, M->w + s.off, M->wb + s.off, s.rows, s.cols, s.ld, s.row0, s.kind, M->st));
  LCK(cudaStreamSynchronize(M->st));
  return MOE_OK;
}

int32_t lm_get_param(lm_model_t* M, int32_t layer, int32_t which, int32_t expert, float* host, int32_t rows, int32_t cols) {
  LENTER(M);
  if (is_moe_param(which)) {
    lm_block* b;
    RC(moe_block(M, layer, &b));
    LCK(cudaStreamSynchronize(M->st));
    return moe_rc(M, *b, moe_get_weight_f32(b->moe, which - LM_MOE_ROUTER, expert, host, rows, cols));
  }
  return read_slot(M, M->w, layer, which, host, rows, cols, false);
}

int32_t lm_get_grad(lm_model_t* M, int32_t layer, int32_t which, int32_t expert, float* host, int32_t rows, int32_t cols) {
  LENTER(M);
  if (is_moe_param(which)) {
    lm_block* b;
    RC(moe_block(M, layer, &b));
    LCK(cudaStreamSynchronize(M->st));
    return moe_rc(M, *b, moe_get_grad_f32(b->moe, which - LM_MOE_ROUTER, expert, host, rows, cols));
  }
  return read_slot(M, M->g, layer, which, host, rows, cols, !M->grad_valid);
}

int64_t lm_optimizer_step(const lm_model_t* M) { return M ? M->step : -1; }
int32_t lm_set_optimizer_step(lm_model_t* M, int64_t step) {
  LENTER(M);
  if (step < 0) return lfail(M, MOE_INVALID_INPUT, "InvalidInput: negative step");
  M->step = step;
  return MOE_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// one pass
// ---------------------------------------------------------------------------
namespace {

struct Batch {
  int B = 0, S = 0, rows = 0, predicted = 0;
  bool padded = false;
  lm::AttnShape a{};
  long long TQ = 0, KV = 0;
};

// TokenBatch::new / with_loss_mask / predicts (batch.rs:35-160) on the caller's arrays; uploads ids, targets, valid.
int prepare_batch(lm_model* M, const uint32_t* ids, const int32_t* lengths, const uint8_t* mask, int B, int S, bool need_targets, Batch* out) {
  if (!ids || B <= 0 || S <= 0) return lfail(M, MOE_INVALID_INPUT, "InvalidInput: empty batch");
  if ((long long)B * S > M->cfg.max_batch_rows)
    return lfail(M, MOE_INVALID_INPUT, "InvalidInput: %d x %d rows exceed max_batch_rows %d", B, S, M->cfg.max_batch_rows);
  if (S > M->cfg.max_seq_len) return lfail(M, MOE_INVALID_INPUT, "SequenceTooLong: length %d, max_seq_len %d", S, M->cfg.max_seq_len);
  if ((long long)B * M->Hkv > MAX_EXPERTS) return lfail(M, MOE_UNSUPPORTED, "Unsupported: batch x kv heads above %d", MAX_EXPERTS);
  Batch b;
  b.B = B; b.S = S; b.rows = B * S;
  for (int i = 0; i < B; ++i) {
    const int len = lengths ? lengths[i] : S;
    if (len < 2 && need_targets) return lfail(M, MOE_INVALID_CONFIG, "InvalidConfig: a causal language-modelling loss needs at least two tokens per sequence, got %d", len);
    if (len < 1 || len > S) return lfail(M, MOE_INVALID_INPUT, "InvalidInput: sequence %d has length %d of %d", i, len, S);
    if (len != S) b.padded = true;
    for (int s = 0; s < S; ++s) {
      const int r = i * S + s;
      const uint32_t id = s < len ? ids[r] : 0u;
      if (id >= (uint32_t)M->V) return lfail(M, MOE_INVALID_INPUT, "TokenOutOfRange: id %u, vocab_size %d", id, M->V);
      M->ids_pin[r] = id;
      M->valid_pin[r] = s < len ? 1 : 0;
      const bool predicts = s + 1 < len && (!mask || mask[r + 1]);
      M->targets_pin[r] = predicts ? (int)ids[r + 1] : -1;
      b.predicted += predicts ? 1 : 0;
    }
  }
  if (need_targets && b.predicted == 0)
    return lfail(M, MOE_INVALID_CONFIG, mask ? "InvalidConfig: a loss mask left no position to predict"
                                             : "InvalidConfig: a causal language-modelling loss needs at least two tokens");
  lm::AttnShape& a = b.a;
  a.B = B; a.S = S; a.H = M->H; a.Hkv = M->Hkv; a.hd = M->hd; a.g = M->H / M->Hkv;
  a.GR = round_up(a.g * S, GROUP_ALIGN); a.S_pad = round_up(S, 32); a.G = B * M->Hkv;
  b.TQ = (long long)a.G * a.GR; b.KV = (long long)a.G * a.S_pad;
  if (need_targets) {
    // chains of the rows that hold the same id, for the deterministic scatter of the embedding gradient
    for (int r = 0; r < b.rows; ++r) {
      const uint32_t id = M->ids_pin[r];
      const int prev = M->last_seen[id];
      M->first_pin[r] = prev < 0 ? 1 : 0;
      M->next_pin[r] = -1;
      if (prev >= 0) M->next_pin[prev] = r;
      M->last_seen[id] = r;
    }
    for (int r = 0; r < b.rows; ++r) M->last_seen[M->ids_pin[r]] = -1;
    LCK(cudaMemcpyAsync(M->first, M->first_pin, (size_t)b.rows * 4, cudaMemcpyHostToDevice, M->st));
    LCK(cudaMemcpyAsync(M->next, M->next_pin, (size_t)b.rows * 4, cudaMemcpyHostToDevice, M->st));
  }
  LCK(cudaMemcpyAsync(M->ids, M->ids_pin, (size_t)b.rows * 4, cudaMemcpyHostToDevice, M->st));
  LCK(cudaMemcpyAsync(M->targets, M->targets_pin, (size_t)b.rows * 4, cudaMemcpyHostToDevice, M->st));
  LCK(cudaMemcpyAsync(M->valid, M->valid_pin, (size_t)b.rows, cudaMemcpyHostToDevice, M->st));
  *out = b;
  return MOE_OK;
}

// The head-major attention buffers depend on (batch, seq_len): padding rows inside them must be zero, so a new
// shape gets fresh zeroed buffers (a training loop keeps one shape; this runs on its first step only).
int ensure_attention(lm_model* M, const Batch& b) {
  if (M->attn_q_rows == b.TQ && M->attn_s_pad == b.a.S_pad && M->attn_kv_rows == b.KV) return MOE_OK;
  LCK(cudaStreamSynchronize(M->st));
  for (void* p : M->attn_allocations) cudaFree(p);
  M->attn_allocations.clear();
  M->attn_q_rows = M->attn_s_pad = M->attn_kv_rows = 0;
  const long long hd = M->hd, TQ = b.TQ, KV = b.KV, SP = b.a.S_pad;
  auto get = [&](void** p, long long bytes) { return lalloc(M, p, bytes, true, &M->attn_allocations); };
  for (auto& blk : M->blocks) {
    RC(get((void**)&blk.q_hm, TQ * hd * 2)); RC(get((void**)&blk.k_hm, KV * hd * 2)); RC(get((void**)&blk.v_hm, KV * hd * 2));
    RC(get((void**)&blk.probs, TQ * SP * 2));
  }
  RC(get((void**)&M->scores, TQ * SP * 2)); RC(get((void**)&M->o_hm, TQ * hd * 2)); RC(get((void**)&M->do_hm, TQ * hd * 2));
  RC(get((void**)&M->dq_hm, TQ * hd * 2)); RC(get((void**)&M->dk_hm, KV * hd * 4)); RC(get((void**)&M->dv_hm, KV * hd * 4));
  M->attn_q_rows = TQ; M->attn_s_pad = SP; M->attn_kv_rows = KV;
  return MOE_OK;
}

int forward_blocks(lm_model* M, const Batch& bt, bool save) {
  const int rows = bt.rows, d = M->d, HD = M->H * M->hd, Fp = M->Fd_pad;
  const lm::AttnShape& a = bt.a;
  const Meta dm = dense_meta(M, rows);
  const Meta am{M->attn_meta, M->attn_meta + a.G + 1, a.G};
  const float scale = 1.0f / sqrtf((float)M->hd);   // attention.rs:294-296
  LCK(lm::launch_attn_meta(M->attn_meta, a.G, a.GR, M->st));
  LCK(lm::launch_embed_gather(M->ids, M->wb + M->off_emb, M->xs[0], rows, d, M->st));
  for (int l = 0; l < M->L; ++l) {
    lm_block& b = M->blocks[l];
    // x + attn(norm(x))   (transformer_block.rs:205-216)
    RC(norm_fwd(M, M->xs[l], b.attn_norm, b.xn1, rows));
    RC(mm_nt(M, b.xn1, rows, d, M->wb + b.wqkv, M->QN, dm, M->qkv, M->QN));
    LCK(lm::launch_rope_pack(M->qkv, M->cos_t, M->sin_t, b.q_hm, b.k_hm, b.v_hm, a, M->st));
    // the half of the square above the diagonal is never computed: score tiles there are skipped (the softmax reads
    // the visible prefix only and writes the rest of the row as zeros), and P V stops at the last visible key
    RC(mm_nt(M, b.q_hm, bt.TQ, M->hd, b.k_hm, a.S_pad, am, M->scores, a.S_pad, tc::EPI_STORE, nullptr, 0, a.S, tc::CAUSAL_COLS));
    LCK(lm::launch_softmax_causal(M->scores, b.probs, a, scale, 1, tc::causal_skipping(), M->st));   // only the default tiles skip the masked part
    RC(mm_nn(M, b.probs, bt.TQ, a.S_pad, b.v_hm, M->hd, am, M->o_hm, M->hd, tc::EPI_STORE, nullptr, 0, a.S, tc::CAUSAL_K));
    LCK(lm::launch_heads_to_tokens(M->o_hm, b.merged, a, M->st));
    RC(mm_nt(M, b.merged, rows, HD, M->wb + b.wo, d, dm, M->tmp, d));
    LCK(lm::launch_add(M->tmp, M->xs[l], b.res, (long long)rows * d, M->st));
    // y + ffn(norm(y))    (transformer_block.rs:218-226)
    RC(norm_fwd(M, b.res, b.ffn_norm, b.xn2, rows));
    if (b.is_moe) {
      LCK(cudaMemcpyAsync(M->xs[l + 1], b.res, (size_t)rows * d * 2, cudaMemcpyDeviceToDevice, M->st));
      RC(moe_rc(M, b, moe_forward(b.moe, b.xn2, rows, d, bt.padded ? M->valid : nullptr, M->xs[l + 1], 1, save ? 1 : 0, M->st)));
    } else {
      RC(mm_nt(M, b.xn2, rows, d, M->wb + b.wgu, 2 * Fp, dm, b.h, Fp, tc::EPI_SWIGLU, save ? b.gu : nullptr, 2 * Fp));
      RC(mm_nt(M, b.h, rows, Fp, M->wb + b.wd, d, dm, M->tmp, d));
      LCK(lm::launch_add(M->tmp, b.res, M->xs[l + 1], (long long)rows * d, M->st));
    }
  }
  RC(norm_fwd(M, M->xs[M->L], M->off_final_norm, M->xf, rows));
  return MOE_OK;
}

long long head_offset(const lm_model* M) { return M->cfg.tie_embeddings ? M->off_emb : M->off_head; }

// logits = xf * head^T, cross-entropy in place (the logits become dL/dlogits), then both products of the
// head's backward: the loss is fused into the step and the logits never leave the device
// (gpu_model.rs:2683-2772, causal_lm_loss.rs:66-150, embedding.rs:130-146).
int head_and_loss(lm_model* M, const Batch& bt) {
  const int rows = bt.rows, d = M->d;
  const Meta dm = dense_meta(M, rows);
  const long long ho = head_offset(M);
  const float inv = 1.0f / (float)bt.predicted;
  RC(mm_nt(M, M->xf, rows, d, M->wb + ho, M->V_pad, dm, M->logits, M->V_pad));
  LCK(lm::launch_cross_entropy(M->logits, M->targets, M->row_loss, rows, M->V, M->V_pad, inv, M->st));
  LCK(lm::launch_loss_sum(M->row_loss, rows, inv, M->loss_dev, M->st));
  RC(mm_nn(M, M->logits, rows, M->V_pad, M->wb + ho, d, dm, M->dxf, d));
  RC(mm_tn(M, M->logits, rows, M->V_pad, M->xf, rows, d, dm, M->g + ho, d, 0, 1));
  return MOE_OK;
}

int backward_blocks(lm_model* M, const Batch& bt) {
  const int rows = bt.rows, d = M->d, HD = M->H * M->hd, Fp = M->Fd_pad;
  const long long n = (long long)rows * d;
  const lm::AttnShape& a = bt.a;
  const Meta dm = dense_meta(M, rows);
  const Meta am{M->attn_meta, M->attn_meta + a.G + 1, a.G};
  const float scale = 1.0f / sqrtf((float)M->hd);
  const long long kv_stride = (long long)a.S_pad * M->hd;
  bf16 *cur = M->dxa, *other = M->dxb;
  RC(norm_bwd(M, M->xs[M->L], M->off_final_norm, M->dxf, cur, rows));
  for (int l = M->L - 1; l >= 0; --l) {
    lm_block& b = M->blocks[l];
    // feed-forward branch (transformer_block.rs:247-254)
    if (b.is_moe) {
      RC(moe_rc(M, b, moe_backward(b.moe, cur, M->dxn, 0, M->st)));
    } else {
      RC(mm_nn(M, cur, rows, d, M->wb + b.wd, Fp, dm, M->dgu, 2 * Fp, tc::EPI_SWIGLU_BWD, b.gu, 2 * Fp));
      RC(mm_tn_dense(M, cur, rows, d, b.h, Fp, M->g + b.wd, Fp));
      RC(mm_nn(M, M->dgu, rows, 2 * Fp, M->wb + b.wgu, d, dm, M->dxn, d));
      RC(mm_tn_dense(M, M->dgu, rows, 2 * Fp, b.xn2, d, M->g + b.wgu, d));
    }
    RC(norm_bwd(M, b.res, b.ffn_norm, M->dxn, M->tmp, rows));
    LCK(lm::launch_add(M->tmp, cur, other, n, M->st));            // dL/dresidual
    // attention branch (attention.rs:404-556)
    RC(mm_nn(M, other, rows, d, M->wb + b.wo, HD, dm, M->d_merged, HD));
    RC(mm_tn_dense(M, other, rows, d, b.merged, HD, M->g + b.wo, HD));
    LCK(lm::launch_tokens_to_heads(M->d_merged, M->do_hm, a, M->st));
    // as in the forward pass, nothing above the diagonal is computed: dL/dP tiles there are skipped (the softmax
    // backward reads the visible prefix and writes zeros behind it), the two reductions over keys stop at the last
    // visible key, and the two reductions over queries skip the queries that come before the tile's keys
    RC(mm_nt(M, M->do_hm, bt.TQ, M->hd, b.v_hm, a.S_pad, am, M->scores, a.S_pad, tc::EPI_STORE, nullptr, 0, a.S, tc::CAUSAL_COLS));   // dL/dP
    RC(mm_tn(M, b.probs, bt.TQ, a.S_pad, M->do_hm, bt.TQ, M->hd, am, M->dv_hm, M->hd, kv_stride, 0, a.S));    // dL/dV, summed over the group
    LCK(lm::launch_softmax_backward(b.probs, M->scores, a, scale, 1, tc::causal_skipping(), M->st));                      // dL/dscore
    RC(mm_nn(M, M->scores, bt.TQ, a.S_pad, b.k_hm, M->hd, am, M->dq_hm, M->hd, tc::EPI_STORE, nullptr, 0, a.S, tc::CAUSAL_K));   // dL/dQ
    RC(mm_tn(M, M->scores, bt.TQ, a.S_pad, b.q_hm, bt.TQ, M->hd, am, M->dk_hm, M->hd, kv_stride, 0, a.S));    // dL/dK
    LCK(lm::launch_qkv_grad_unpack(M->dq_hm, M->dk_hm, M->dv_hm, M->cos_t, M->sin_t, M->dqkv, a, M->st));
    RC(mm_nn(M, M->dqkv, rows, M->QN, M->wb + b.wqkv, d, dm, M->dxn, d));
    RC(mm_tn_dense(M, M->dqkv, rows, M->QN, b.xn1, d, M->g + b.wqkv, d));
    RC(norm_bwd(M, M->xs[l], b.attn_norm, M->dxn, M->tmp, rows));
    LCK(lm::launch_add(M->tmp, other, cur, n, M->st));            // dL/dinput of the block
  }
  LCK(lm::launch_embed_scatter(M->ids, cur, M->g + M->off_emb, M->first, M->next, rows, d, M->st));
  return MOE_OK;
}

int check_device_flag(lm_model* M) {
  int flag = 0;
  LCK(cudaMemcpy(&flag, M->error_flag, sizeof flag, cudaMemcpyDeviceToHost));
  if (flag != 0) {
    cudaMemset(M->error_flag, 0, sizeof flag);
    return lfail(M, MOE_TIMEOUT, "Timeout: a bounded device-side wait gave up (code %d)", flag);
  }
  return MOE_OK;
}

int accumulate_impl(lm_model* M, const uint32_t* ids, const int32_t* lengths, const uint8_t* mask, int B, int S, float* lm_loss,
                    float* aux_loss) {
  Batch bt;
  RC(prepare_batch(M, ids, lengths, mask, B, S, true, &bt));
  RC(ensure_attention(M, bt));
  if (!M->grad_valid) {
    LCK(cudaMemsetAsync(M->g, 0, (size_t)M->n_params * 4, M->st));
    M->grad_valid = true;
  }
  LCK(cudaEventRecord(M->ev[0], M->st));
  RC(forward_blocks(M, bt, true));
  LCK(cudaEventRecord(M->ev[1], M->st));
  RC(head_and_loss(M, bt));
  LCK(cudaEventRecord(M->ev[2], M->st));
  RC(backward_blocks(M, bt));
  LCK(cudaEventRecord(M->ev[3], M->st));
  LCK(cudaMemcpyAsync(M->loss_pin, M->loss_dev, 4, cudaMemcpyDeviceToHost, M->st));
  LCK(cudaStreamSynchronize(M->st));
  for (int i = 0; i < 3; ++i) cudaEventElapsedTime(&M->last_ms[i], M->ev[i], M->ev[i + 1]);
  RC(check_device_flag(M));
  float aux_total = 0.f;                                   // summed in layer order (transformer.rs:700-705)
  for (auto& b : M->blocks) {
    if (!b.is_moe) continue;
    float a = 0.f, z = 0.f;
    RC(moe_rc(M, b, moe_get_losses(b.moe, &a, &z)));
    aux_total += a + z;
  }
  if (lm_loss) *lm_loss = M->loss_pin[0];
  if (aux_loss) *aux_loss = aux_total;
  return MOE_OK;
}

// kind 0 Adam, 1 Sgd, 2 Lion (Param::step, param.rs:547-617); the step counter advances for all three
// (TransformerLm::step, transformer.rs:1576-1606).
int step_impl(lm_model* M, int kind, float lr, float b1, float b2, float eps, float wd, float scale) {
  M->step += 1;
  LCK(cudaEventRecord(M->ev[3], M->st));
  if (!M->grad_valid) LCK(cudaMemsetAsync(M->g, 0, (size_t)M->n_params * 4, M->st));
  AdamArgs a{};
  a.w = M->w; a.g = M->g; a.m = M->m; a.v = M->v; a.w_bf16 = M->wb; a.n = M->n_params;
  a.lr = lr; a.beta1 = b1; a.beta2 = b2; a.eps = eps; a.wd = wd; a.scale = scale;
  a.c1 = 1.0f - powf(b1, (float)M->step);
  a.c2 = 1.0f - powf(b2, (float)M->step);
  LCK(kind == 0 ? launch_adam(a, M->st) : kind == 1 ? launch_sgd(a, M->st) : launch_lion(a, M->st));
  for (auto& b : M->blocks) {
    if (!b.is_moe) continue;
    const int rc = kind == 0   ? moe_step_adam(b.moe, lr, b1, b2, eps, wd, (int)M->step, scale, M->st)
                   : kind == 1 ? moe_step_sgd(b.moe, lr, scale, M->st)
                               : moe_step_lion(b.moe, lr, b1, b2, wd, scale, M->st);
    RC(moe_rc(M, b, rc));
  }
  LCK(cudaEventRecord(M->ev[4], M->st));
  M->grad_valid = false;   // the optimizer kernels cleared the gradients
  return MOE_OK;
}

int step_and_time(lm_model* M, int kind, float lr, float b1, float b2, float eps, float wd, float scale) {
  RC(step_impl(M, kind, lr, b1, b2, eps, wd, scale));
  LCK(cudaStreamSynchronize(M->st));
  cudaEventElapsedTime(&M->last_ms[3], M->ev[3], M->ev[4]);
  return MOE_OK;
}

}  // namespace

extern "C" {

int32_t lm_forward_logits(lm_model_t* M, const uint32_t* ids, const int32_t* lengths, int32_t B, int32_t S, float* logits_host,
                          float* moe_logits_host) {
  LENTER(M);
  if (!logits_host) return lfail(M, MOE_INVALID_INPUT, "InvalidInput: null logits buffer");
  Batch bt;
  RC(prepare_batch(M, ids, lengths, nullptr, B, S, false, &bt));
  RC(ensure_attention(M, bt));
  RC(forward_blocks(M, bt, false));
  RC(mm_nt(M, M->xf, bt.rows, M->d, M->wb + head_offset(M), M->V_pad, dense_meta(M, bt.rows), M->logits, M->V_pad));
  // bf16 device logits -> f32 host rows, a slab of rows at a time through the staging buffer
  const int slab = (int)std::max<long long>(1, M->stage_elems / M->V);
  for (int r0 = 0; r0 < bt.rows; r0 += slab) {
    const int n = std::min(slab, bt.rows - r0);
    LCK(lm::launch_cast_rows_to_f32(M->logits + (size_t)r0 * M->V_pad, M->V_pad, M->stage, n, M->V, M->st));
    LCK(cudaMemcpyAsync(logits_host + (size_t)r0 * M->V, M->stage, (size_t)n * M->V * 4, cudaMemcpyDeviceToHost, M->st));
    LCK(cudaStreamSynchronize(M->st));
  }
  RC(check_device_flag(M));
  if (moe_logits_host) {
    size_t k = 0;
    for (auto& b : M->blocks) {
      if (!b.is_moe) continue;
      RC(moe_rc(M, b, moe_get_router_cache(b.moe, moe_logits_host + k * (size_t)bt.rows * M->cfg.num_experts, nullptr, nullptr)));
      ++k;
    }
  }
  return MOE_OK;
}

int32_t lm_accumulate_step(lm_model_t* M, const uint32_t* ids, const int32_t* lengths, const uint8_t* mask, int32_t B, int32_t S,
                           float* lm_loss, float* aux_loss) {
  LENTER(M);
  return accumulate_impl(M, ids, lengths, mask, B, S, lm_loss, aux_loss);
}

int32_t lm_zero_grad(lm_model_t* M) {
  LENTER(M);
  M->grad_valid = false;
  for (auto& b : M->blocks)
    if (b.is_moe) RC(moe_rc(M, b, moe_zero_grad(b.moe, M->st)));
  return MOE_OK;
}

int32_t lm_step_adam(lm_model_t* M, float lr, float b1, float b2, float eps, float wd, float scale) {
  LENTER(M);
  return step_and_time(M, 0, lr, b1, b2, eps, wd, scale);
}

int32_t lm_step_sgd(lm_model_t* M, float lr, float scale) {
  LENTER(M);
  return step_and_time(M, 1, lr, 0.f, 0.f, 0.f, 0.f, scale);
}

int32_t lm_step_lion(lm_model_t* M, float lr, float b1, float b2, float wd, float scale) {
  LENTER(M);
  return step_and_time(M, 2, lr, b1, b2, 0.f, wd, scale);
}

int32_t lm_train_step(lm_model_t* M, const uint32_t* ids, const int32_t* lengths, const uint8_t* mask, int32_t B, int32_t S,
                      float lr, float b1, float b2, float eps, float wd, float* lm_loss, float* aux_loss) {
  LENTER(M);
  RC(lm_zero_grad(M));
  RC(accumulate_impl(M, ids, lengths, mask, B, S, lm_loss, aux_loss));
  return lm_step_adam(M, lr, b1, b2, eps, wd, 1.0f);
}

int32_t lm_last_step_ms(lm_model_t* M, float* ms4) {
  LENTER(M);
  if (!ms4) return MOE_INVALID_INPUT;
  for (int i = 0; i < 4; ++i) ms4[i] = M->last_ms[i];
  return MOE_OK;
}

int32_t lm_synchronize(lm_model_t* M) {
  LENTER(M);
  LCK(cudaStreamSynchronize(M->st));
  return check_device_flag(M);
}

}  // extern "C"

// ---------------------------------------------------------------------------
// KV-cached decode
// ---------------------------------------------------------------------------
#include "../../include/kv_attention_b200.h"

struct lm_decoder {
  std::vector<kv_cache_t*> layers;
  int sequences = 0, capacity = 0;
};

extern "C" {

int32_t lm_decoder_create(lm_model_t* M, int32_t sequences, int32_t capacity, lm_decoder_t** out) {
  LENTER(M);
  if (!out) return MOE_INVALID_INPUT;
  *out = nullptr;
  if (sequences <= 0 || capacity <= 0 || capacity > M->cfg.max_seq_len)
    return lfail(M, MOE_INVALID_CONFIG, "InvalidConfig: %d sequences of %d positions (max_seq_len %d)", sequences, capacity, M->cfg.max_seq_len);
  lm_decoder* D = new (std::nothrow) lm_decoder;
  if (!D) return MOE_OUT_OF_MEMORY;
  D->sequences = sequences; D->capacity = capacity;
  for (int l = 0; l < M->L; ++l) {
    kv_cache_config_t kc{};
    kc.sequences = sequences; kc.num_heads = M->H; kc.kv_heads = M->Hkv; kc.head_dim = M->hd; kc.capacity = capacity;
    kc.max_seq_len = M->cfg.max_seq_len; kc.rope_base = M->cfg.rope_base; kc.rope = 1; kc.precision = MOE_PRECISION_BF16; kc.device = M->device;
    kv_cache_t* c = nullptr;
    const int rc = kv_cache_create(&kc, &c);
    if (rc != MOE_OK) {
      lfail(M, rc, "layer %d cache: %s", l, c ? kv_cache_last_error(c) : "kv_cache_create failed");
      if (c) kv_cache_destroy(c);
      for (auto* p : D->layers) kv_cache_destroy(p);
      delete D;
      return rc;
    }
    D->layers.push_back(c);
  }
  *out = D;
  return MOE_OK;
}

void lm_decoder_destroy(lm_decoder_t* D) {
  if (!D) return;
  for (auto* p : D->layers) kv_cache_destroy(p);
  delete D;
}

int32_t lm_decoder_clear(lm_model_t* M, lm_decoder_t* D, int32_t sequence) {
  LENTER(M);
  if (!D || sequence >= D->sequences) return lfail(M, MOE_INVALID_INPUT, "InvalidInput: no such sequence");
  for (auto* c : D->layers) {
    const int rc = kv_cache_clear(c, sequence, M->st);
    if (rc != MOE_OK) return lfail(M, rc, "%s", kv_cache_last_error(c));
  }
  return MOE_OK;
}

int32_t lm_forward_cached(lm_model_t* M, lm_decoder_t* D, const uint32_t* ids, int32_t first, int32_t n_seq, int32_t per,
                          float* logits_host) {
  LENTER(M);
  if (!D || (int)D->layers.size() != M->L)
    return lfail(M, MOE_INVALID_CONFIG, "InvalidConfig: expected one kv cache per layer (%d)", M->L);   // transformer.rs:742-748
  if (!ids || !logits_host || n_seq <= 0 || per <= 0 || first < 0 || first + n_seq > D->sequences)
    return lfail(M, MOE_INVALID_INPUT, "InvalidInput: sequences %d .. %d of %d, %d rows each", first, first + n_seq - 1, D->sequences, per);
  const int rows = n_seq * per, d = M->d, HD = M->H * M->hd, KD = M->Hkv * M->hd, Fp = M->Fd_pad;
  if (rows > M->cfg.max_batch_rows) return lfail(M, MOE_INVALID_INPUT, "InvalidInput: %d rows exceed max_batch_rows %d", rows, M->cfg.max_batch_rows);
  for (int r = 0; r < rows; ++r) {
    if (ids[r] >= (uint32_t)M->V) return lfail(M, MOE_INVALID_INPUT, "TokenOutOfRange: id %u, vocab_size %d", ids[r], M->V);
    M->ids_pin[r] = ids[r];
  }
  LCK(cudaMemcpyAsync(M->ids, M->ids_pin, (size_t)rows * 4, cudaMemcpyHostToDevice, M->st));
  const Meta dm = dense_meta(M, rows);
  // temporaries of the training pass double as the decode pass's scratch (the two never overlap in time)
  bf16 *x = M->dxa, *y = M->dxb, *nrm = M->dxn, *q = M->dqkv, *k = q + (size_t)rows * HD, *v = k + (size_t)rows * KD;
  LCK(lm::launch_embed_gather(M->ids, M->wb + M->off_emb, x, rows, d, M->st));
  for (int l = 0; l < M->L; ++l) {
    lm_block& b = M->blocks[l];
    // transformer_block.rs:232-244
    RC(norm_fwd(M, x, b.attn_norm, nrm, rows));
    RC(mm_nt(M, nrm, rows, d, M->wb + b.wqkv, M->QN, dm, M->qkv, M->QN));
    LCK(lm::launch_split_qkv(M->qkv, q, k, v, rows, HD, KD, M->st));
    const int rc = kv_attention_forward_cached(D->layers[l], first, n_seq, q, k, v, per, M->d_merged, M->st);
    if (rc != MOE_OK) return lfail(M, rc, "%s", kv_cache_last_error(D->layers[l]));
    RC(mm_nt(M, M->d_merged, rows, HD, M->wb + b.wo, d, dm, M->tmp, d));
    LCK(lm::launch_add(M->tmp, x, y, (long long)rows * d, M->st));                 // residual
    RC(norm_fwd(M, y, b.ffn_norm, nrm, rows));
    if (b.is_moe) {
      RC(moe_rc(M, b, moe_forward(b.moe, nrm, rows, d, nullptr, y, 1, 0, M->st)));   // adds into the residual
      std::swap(x, y);
    } else {
      RC(mm_nt(M, nrm, rows, d, M->wb + b.wgu, 2 * Fp, dm, M->dgu, Fp, tc::EPI_SWIGLU, nullptr, 0));
      RC(mm_nt(M, M->dgu, rows, Fp, M->wb + b.wd, d, dm, M->tmp, d));
      LCK(lm::launch_add(M->tmp, y, x, (long long)rows * d, M->st));
    }
  }
  RC(norm_fwd(M, x, M->off_final_norm, M->xf, rows));
  RC(mm_nt(M, M->xf, rows, d, M->wb + head_offset(M), M->V_pad, dm, M->logits, M->V_pad));
  const int slab = (int)std::max<long long>(1, M->stage_elems / M->V);
  for (int r0 = 0; r0 < rows; r0 += slab) {
    const int n = std::min(slab, rows - r0);
    LCK(lm::launch_cast_rows_to_f32(M->logits + (size_t)r0 * M->V_pad, M->V_pad, M->stage, n, M->V, M->st));
    LCK(cudaMemcpyAsync(logits_host + (size_t)r0 * M->V, M->stage, (size_t)n * M->V * 4, cudaMemcpyDeviceToHost, M->st));
    LCK(cudaStreamSynchronize(M->st));
  }
  return check_device_flag(M);
}

}  // extern "C"
