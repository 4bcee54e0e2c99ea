// The layer handle behind the C ABI: owned device memory and the per-pass plans.
#pragma once
#include <string>
#include <vector>

#include "common.cuh"
#include "gemm_tc.cuh"
#include "kernels.cuh"

struct moe_layer {
  // configuration
  int d = 0, E = 0, k = 0, F = 0, F_pad = 0;
  int E_local = 0, e0 = 0, ep_rank = 0, ep_size = 1;
  bool shared = false, training = false;
  float aux_w = 0.f, z_w = 0.f;
  int precision = 0;       // moe_precision
  int act = 0;             // moe::PREC_F32 or PREC_BF16: element type of activations
  int max_tokens = 0, rows_cap = 0, shared_rows_cap = 0;
  int device = 0, sm_count = 0;
  size_t esz = 4;          // bytes per activation element

  // error state (sticky, like the reference's poisoned context)
  std::string err;
  int status = 0;

  // parameters: one arena per role so the optimizer is a single launch
  long long n_params = 0;
  long long off_router = 0, off_gu = 0, off_d = 0, off_sgu = 0, off_sd = 0;
  float* w = nullptr;      // f32 master
  float* g = nullptr;      // dL/dW
  float* m = nullptr;
  float* v = nullptr;
  moe::bf16* wb = nullptr; // bf16 compute copy (bf16 precision)
  bool grad_valid = false; // false: the next backward overwrites instead of accumulating
  float* stage = nullptr;  // staging for weight upload / download (one matrix)
  long long stage_elems = 0;

  // low-rank adapters on the expert projections (moe_lora_attach); base weights are frozen meanwhile
  int lora_rank = 0, lora_slots = 0;
  float lora_scale = 0.f;            // alpha / rank
  float lora_alpha = 0.f;
  long long lora_n = 0;              // floats in the adapter arenas
  float *la = nullptr, *lg = nullptr, *lm = nullptr, *lv = nullptr;   // adapters, their gradients, Adam moments
  void* lora_table = nullptr;        // device array of LoraSlot
  float* w_eff = nullptr;            // f32 handles: W + scale * up * down for the expert GEMMs
  float* wc = nullptr;               // f32 weights the expert GEMMs read: w, or w_eff with adapters
  bool lora_dirty = false;           // adapters or base weights changed since the last fold
  // f32 handles whose shapes fit the tensor-core tiles run their FORWARD expert products on tcgen05 with every
  // operand split into three bf16 pieces (f32-level accuracy, six cross terms in one product): expanded weights
  // [.., 6 * in] at 6 x the arena offsets, refreshed when `w3_dirty`; expanded activations per call
  moe::bf16* w3 = nullptr;
  moe::bf16 *xa3 = nullptr, *ha3 = nullptr;
  bool w3_dirty = true;

  // int8 inference weights (Q8 precision)
  int8_t* q_gu = nullptr; float* s_gu = nullptr;   // [E][2F_pad][d], [E][2F_pad]
  int8_t* q_d = nullptr;  float* s_d = nullptr;    // [E][d][F_pad],  [E][d]
  int8_t* q_sgu = nullptr; float* s_sgu = nullptr;
  int8_t* q_sd = nullptr;  float* s_sd = nullptr;

  // router cache
  float *logits = nullptr, *probs = nullptr, *lse = nullptr, *gates = nullptr;
  int* expert_of = nullptr;
  float* partial = nullptr;
  int* hist = nullptr;
  moe::RouteMeta meta{};
  int* meta_block = nullptr;
  float *stats = nullptr, *losses = nullptr;
  int *slot_pos = nullptr, *row_token = nullptr, *token_of = nullptr, *slot_of = nullptr;
  float* row_gate = nullptr;
  int* shared_meta = nullptr;   // [4]: row0[0..1], tstart[0..1] of the dense (shared expert) group: entry `tokens` of the table
  int* shared_meta_table = nullptr;   // [max_tokens + 1][4]
  int* error_flag = nullptr;
  int* route_done = nullptr;    // counter of the decode routing kernel (zero between launches)

  // activations (element type `act`)
  void *x_perm = nullptr, *gu = nullptr, *h = nullptr, *y_perm = nullptr;
  void *dy_perm = nullptr, *dgu = nullptr, *dx_perm = nullptr, *dh = nullptr;
  void *gu_s = nullptr, *h_s = nullptr, *y_s = nullptr, *dgu_s = nullptr, *dx_s = nullptr, *dh_s = nullptr;
  float *grad_gates = nullptr, *grad_logits = nullptr, *rw_scratch = nullptr;
  moe::bf16* gl_bf16 = nullptr;   // [max_tokens, E]
  void* dx_r = nullptr;           // [shared_rows_cap, d] router input gradient
  bool tc_router = false;         // router products on the tensor cores (bf16, E % 8 == 0)
  int rw_splits = 1;
  float* sh_scratch = nullptr;    // partial weight gradients of the row-split shared-expert products
  long long sh_scratch_elems = 0;
  int* sh_meta = nullptr;         // [splits + 1] token-chunk boundaries of those products
  int* rw_meta = nullptr;         // [splits + 1] token-chunk boundaries of the split router weight gradient

  // expert parallelism (ep_size > 1): the send side keeps the compact expert-major
  // layout in x_perm / y_perm / dy_perm / dx_perm; rows received for the local experts
  // live in the *_recv buffers in the padded layout the grouped GEMMs want.
  void* comm = nullptr;            // ncclComm_t
  bool ep_ready = false;
  long long ep_deadline_ms = 600000;   // how long a host-side wait behind a collective may take before the group is aborted (0 = for ever)
  float ep_capacity = 1.25f;
  int rows_cap_l = 0;              // capacity (rows) of the local-expert buffers
  int *ep_pack = nullptr, *ep_gathered = nullptr, *ep_gathered_host = nullptr;
  float* ext_stats = nullptr;      // whole-batch sum p[e], sum lse^2, valid tokens
  int* ext_counts = nullptr;       // whole-batch rows per expert
  int *local_meta = nullptr, *local_meta_host = nullptr;   // row0[El+1], tiles[El+1], counts[El+1]
  std::vector<int> cnt_all, send_off, recv_row;
  void *x_recv = nullptr, *y_recv = nullptr, *dy_recv = nullptr, *dx_recv = nullptr;
  // peer transport: every rank's four receive buffers mapped into this process (CUDA IPC);
  // dispatch pushes rows straight into the owner's x_recv / dy_recv and combine / un-permute
  // pull rows straight from the owner's y_recv / dx_recv over NVLink.
  void* peer_base[4][moe::MAX_RANKS] = {};   // [x, y, dy, dx][rank]
  bool peer_ready = false;
  int *dest_base = nullptr, *dest_base_host = nullptr;   // [E] first row id (rank*cap+row) of my rows per expert
  int* barrier_word = nullptr;
  float* g_rep_save = nullptr;     // replicated gradients (router, shared expert) of earlier passes, set aside while a pass's own are all-reduced
  bool rep_overwrite = false;      // the running backward writes the replicated gradients without accumulating

  // host-call staging
  float* host_stage_f32 = nullptr;   // [max_tokens, d]
  void* host_x = nullptr;            // [max_tokens, d] act type
  void* host_y = nullptr;
  void* host_gx = nullptr;
  uint8_t* host_valid = nullptr;
  void* pinned = nullptr;            // pinned bounce buffer, [max_tokens, d] f32
  cudaStream_t own_stream = nullptr;
  // The routed experts' weight-gradient GEMMs feed nothing else in the pass, so backward leaves them
  // on a side stream and returns; the HBM/NVLink-bound tail of backward and the router + dispatch of
  // the next forward run beside them.  Whatever they read that the next forward rewrites before its
  // first expert GEMM is double-buffered (dispatched rows, group tables), selected by `parity`.
  cudaStream_t side_stream = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  bool side_pending = false;            // deferred work not yet joined by a later call
  int parity = 0;
  void* x_perm2[2] = {nullptr, nullptr};
  void* x_recv2[2] = {nullptr, nullptr};
  int* meta_block2[2] = {nullptr, nullptr};
  int* local_meta2[2] = {nullptr, nullptr};

  // last forward
  int last_tokens = 0;
  bool have_cache = false;
  const void* last_x = nullptr;
  cudaStream_t last_stream = nullptr;

  // optional per-kernel timing with CUDA events on the launching stream
  struct ProfSpan { int cat; cudaEvent_t begin, end; };
  bool prof_on = false;
  std::vector<ProfSpan> prof_spans;
  std::vector<cudaEvent_t> prof_pool;

  std::vector<void*> allocations;
  long long allocated_bytes = 0;
};
