// C ABI of the layer (declared in include/moe_b200.h): handle life cycle, weight
// transfer, and the forward / backward / optimizer plans that sequence the kernels.
// Nothing here falls back to the host: without a device every entry fails.

#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <chrono>
#include <cmath>
#include <new>
#include <thread>

#include "../../include/moe_b200.h"
#include "../../include/moe_b200_debug.h"
#include <nccl.h>

#include "layer.cuh"

using namespace moe;

namespace {

int fail(moe_layer* L, int status, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (L) {
    L->err = buf;
    L->status = status;
  }
  return status;
}

#define CK(call)                                                                                   \
  do {                                                                                             \
    cudaError_t e_ = (call);                                                                       \
    if (e_ != cudaSuccess)                                                                         \
      return fail(L, e_ == cudaErrorMemoryAllocation ? MOE_OUT_OF_MEMORY : MOE_CUDA_ERROR,         \
                  "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__);     \
  } while (0)

#define ENTER(L)                                                                                   \
  do {                                                                                             \
    if (!(L)) return MOE_INVALID_INPUT;                                                            \
    if ((L)->status != MOE_OK) return MOE_POISONED;                                                \
    cudaError_t e_ = cudaSetDevice((L)->device);                                                   \
    if (e_ != cudaSuccess) return fail((L), MOE_CUDA_ERROR, "cudaSetDevice: %s", cudaGetErrorString(e_)); \
  } while (0)

// ---------------------------------------------------------------------------
// Deadlines.  A collective whose peer never arrives would leave cudaStreamSynchronize waiting for ever,
// so an expert-parallel handle waits by polling: `ready()` is asked until it says yes or `deadline_ms`
// has passed (0 = no deadline).  The poll sleeps 50 us at first and backs off to 1 ms.
// Returns true when ready, false when the deadline passed.
// ---------------------------------------------------------------------------
template <typename Ready>
bool poll_until(Ready ready, long long deadline_ms) {
  const auto t0 = std::chrono::steady_clock::now();
  long long sleep_us = 50;
  for (;;) {
    if (ready()) return true;
    if (deadline_ms > 0) {
      const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
      if (ms >= deadline_ms) return false;
    }
    std::this_thread::sleep_for(std::chrono::microseconds(sleep_us));
    if (sleep_us < 1000) sleep_us *= 2;
  }
}

// Waits for `st` (or the whole device when st_is_device).  Handles without a communicator wait the plain
// way.  An expert-parallel handle gives up after its deadline: it aborts the communicator (which ends the
// NCCL kernels that were waiting for the missing rank), poisons the handle and returns MOE_TIMEOUT; the
// caller destroys the handle and builds a new group, as after any fail-closed error.
int wait_for(moe_layer* L, cudaStream_t st, bool whole_device) {
  if (L->ep_size <= 1 || !L->comm) {
    CK(whole_device ? cudaDeviceSynchronize() : cudaStreamSynchronize(st));
    return MOE_OK;
  }
  cudaError_t bad = cudaSuccess;
  const bool done = poll_until([&]() {
    const cudaError_t q = whole_device ? cudaStreamQuery(cudaStreamLegacy) : cudaStreamQuery(st);
    if (q == cudaErrorNotReady) return false;
    bad = q;
    return true;
  }, L->ep_deadline_ms);
  if (!done) {
    ncclCommAbort((ncclComm_t)L->comm);
    L->comm = nullptr;
    L->ep_ready = false;
    return fail(L, MOE_TIMEOUT, "Timeout: the stream did not finish within %lld ms; a rank of the expert-parallel group is missing or stuck (communicator aborted)",
                L->ep_deadline_ms);
  }
  if (bad != cudaSuccess) return fail(L, MOE_CUDA_ERROR, "stream failed: %s", cudaGetErrorString(bad));
  if (whole_device) CK(cudaDeviceSynchronize());   // the legacy stream has drained; non-blocking streams follow at once
  return MOE_OK;
}
#define WAIT(L, st, dev)                         \
  do {                                           \
    const int w_ = wait_for((L), (st), (dev));   \
    if (w_ != MOE_OK) return w_;                 \
  } while (0)

// Brackets a stage with two events when profiling is on.
struct Span {
  moe_layer* L; cudaStream_t st; int idx = -1;
  Span(moe_layer* layer, int cat, cudaStream_t stream) : L(layer), st(stream) {
    if (!L->prof_on || cat < 0) return;
    cudaEvent_t ev[2];
    for (int i = 0; i < 2; ++i) {
      if (!L->prof_pool.empty()) { ev[i] = L->prof_pool.back(); L->prof_pool.pop_back(); }
      else if (cudaEventCreate(&ev[i]) != cudaSuccess) return;
    }
    cudaEventRecord(ev[0], st);
    L->prof_spans.push_back({cat, ev[0], ev[1]});
    idx = (int)L->prof_spans.size() - 1;
  }
  ~Span() { if (idx >= 0) cudaEventRecord(L->prof_spans[idx].end, st); }
};

long long align_up(long long v, long long a) { return (v + a - 1) / a * a; }

// How backward overlaps its HBM-bound tail with the tensor-core work (MOE_B200_OVERLAP):
//   0 none; 1 un-permute on a side stream beside the gate|up weight gradient;
//   2 both routed weight-gradient GEMMs deferred to the side stream past the end of the call.
// Unset (-1 here): 0 on one GPU and on two ranks, 1 from four ranks on.  Measured on cfg 4 the three modes give the
// same step time at 1 and 2 GPUs (the step runs at the board's power cap, and work that overlaps the GEMMs slows
// them by what it saves); from 4 ranks on, where each GPU's GEMMs are shorter and the exchange tail relatively
// longer, mode 1 is faster: 33.8 against 34.3 ms at 4 ranks, 35.8 against 37.8 ms at 8.
int overlap_mode() {
  static const int mode = [] {
    const char* e = getenv("MOE_B200_OVERLAP");
    return e && *e >= '0' && *e <= '2' ? *e - '0' : -1;
  }();
  return mode;
}

// Makes `st` wait for weight gradients still running on the side stream.
int join_side(moe_layer* L, cudaStream_t st) {
  if (!L->side_pending) return MOE_OK;
  CK(cudaStreamWaitEvent(st, L->ev_join, 0));
  L->side_pending = false;
  return MOE_OK;
}

void select_parity(moe_layer* L, int p) {
  const long long E = L->E;
  L->parity = p;
  L->meta_block = L->meta_block2[p];
  L->meta.counts = L->meta_block; L->meta.offsets = L->meta_block + (E + 1); L->meta.pad_off = L->meta_block + 2 * (E + 1);
  L->meta.tile_start = L->meta_block + 3 * (E + 1); L->meta.total = L->meta_block + 4 * (E + 1);
  L->x_perm = L->x_perm2[p];
  if (L->ep_size > 1) { L->x_recv = L->x_recv2[p]; L->local_meta = L->local_meta2[p]; }
}

int validate(const moe_config_t* c, char* msg, int len) {
  auto say = [&](const char* fmt, ...) {
    if (msg && len > 0) {
      va_list ap;
      va_start(ap, fmt);
      vsnprintf(msg, len, fmt, ap);
      va_end(ap);
    }
    return (int)MOE_INVALID_CONFIG;
  };
  if (!c) return say("null config");
  // MoeConfig::validate, moe.rs:68-86
  if (c->num_experts <= 0) return say("a MoE layer needs at least one expert");
  if (c->experts_per_token <= 0 || c->experts_per_token > c->num_experts)
    return say("experts_per_token must be between 1 and num_experts (%d), got %d", c->num_experts,
               c->experts_per_token);
  if (c->d_ff <= 0) return say("expert d_ff must be non-zero");
  if (c->d_model <= 0) return say("d_model must be non-zero");
  if (c->num_experts > MAX_EXPERTS) return say("at most %d experts are supported", MAX_EXPERTS);
  if (c->experts_per_token > MAX_TOPK) return say("at most %d experts per token are supported", MAX_TOPK);
  if (c->max_tokens <= 0) return say("max_tokens must be positive");
  if (c->precision < MOE_PRECISION_F32 || c->precision > MOE_PRECISION_Q8) return say("unknown precision");
  if (c->ep_size < 1 || c->ep_rank < 0 || c->ep_rank >= c->ep_size || c->num_experts % c->ep_size != 0)
    return say("num_experts must divide evenly over ep_size ranks");
  if (c->precision != MOE_PRECISION_F32 && c->d_model % 32 != 0)
    return say("the bf16 and int8 paths need d_model to be a multiple of 32 (got %d); use MOE_PRECISION_F32",
               c->d_model);
  if (c->precision == MOE_PRECISION_Q8 && c->training) return say("a quantized layer cannot be trained");
  if (c->precision == MOE_PRECISION_Q8 && c->d_model % 64 != 0) return say("the int8 path needs d_model to be a multiple of 64");
  if (c->precision == MOE_PRECISION_Q8 && c->ep_size != 1) return say("the int8 path is single-device");
  if ((long long)c->max_tokens * c->experts_per_token > (1ll << 30)) return say("max_tokens * experts_per_token too large");
  return MOE_OK;
}

struct Sizes {
  int F_pad, E_local, rows_cap, shared_rows_cap;
  long long off_router, off_gu, off_d, off_sgu, off_sd, n_params;
};

Sizes sizes_of(const moe_config_t* c) {
  Sizes s;
  s.F_pad = round_up(c->d_ff, c->precision == MOE_PRECISION_Q8 ? 2 * GU_BLOCK : GU_BLOCK);
  s.E_local = c->num_experts / c->ep_size;
  s.rows_cap = round_up(c->max_tokens * c->experts_per_token + c->num_experts * (GROUP_ALIGN - 1), GROUP_ALIGN);
  s.shared_rows_cap = round_up(c->max_tokens, GROUP_ALIGN);
  long long o = 0;
  s.off_router = o; o = align_up(o + (long long)c->num_experts * c->d_model, 128);
  s.off_gu = o;     o = align_up(o + (long long)s.E_local * 2 * s.F_pad * c->d_model, 128);
  s.off_d = o;      o = align_up(o + (long long)s.E_local * c->d_model * s.F_pad, 128);
  s.off_sgu = o;    if (c->shared_expert) o = align_up(o + 2ll * s.F_pad * c->d_model, 128);
  s.off_sd = o;     if (c->shared_expert) o = align_up(o + (long long)c->d_model * s.F_pad, 128);
  s.n_params = o;
  return s;
}

long long workspace_bytes(const moe_config_t* c) {
  const Sizes s = sizes_of(c);
  const long long esz = c->precision == MOE_PRECISION_F32 ? 4 : 2;
  const long long T = c->max_tokens, d = c->d_model, E = c->num_experts, k = c->experts_per_token;
  long long b = 0;
  if (c->precision == MOE_PRECISION_Q8) {
    b += (long long)c->num_experts * d * 4;                          // router
    b += (s.n_params - s.off_gu) + (s.E_local + 1ll) * (2 * s.F_pad + d) * 4;  // int8 values and scales
  } else {
    b += s.n_params * 4 * (c->training ? 4 : 1);
    if (c->precision == MOE_PRECISION_BF16) b += s.n_params * 2;
  }
  const long long act_rows = (long long)s.rows_cap * (2 * d + 3 * s.F_pad) + (c->shared_expert ? (long long)s.shared_rows_cap * (d + 3 * s.F_pad) : 0);
  b += act_rows * esz * (c->training ? 2 : 1);
  if (c->training && overlap_mode() == 2) b += (long long)s.rows_cap * d * esz;   // second half of the double-buffered dispatched rows
  b += T * E * 4 * 4 + T * k * 4 * 6 + (long long)s.rows_cap * 8;
  return b;
}

int dalloc(moe_layer* L, void** p, long long bytes, bool zero) {
  if (bytes <= 0) bytes = 16;
  CK(cudaMalloc(p, (size_t)bytes));
  L->allocations.push_back(*p);
  L->allocated_bytes += bytes;
  if (zero) CK(cudaMemset(*p, 0, (size_t)bytes));
  return MOE_OK;
}
#define DA(ptr, bytes, zero)                                         \
  do {                                                               \
    int rc_ = dalloc(L, (void**)&(ptr), (long long)(bytes), (zero)); \
    if (rc_ != MOE_OK) return rc_;                                   \
  } while (0)

// ---------------------------------------------------------------------------
// weight packing
// ---------------------------------------------------------------------------
struct WeightSlot {
  long long offset;     // into the parameter arenas
  int rows, cols;       // caller's [out, in]
  int ld;               // leading dimension inside the arena
  int kind;             // 0 plain rows, 1 gate rows of the interleaved matrix, 2 up rows
};

int slot_of_weight(moe_layer* L, int which, int expert, WeightSlot* s) {
  const int d = L->d, F = L->F, Fp = L->F_pad;
  int le = expert - L->e0;
  switch (which) {
    case MOE_W_ROUTER: *s = {L->off_router, L->E, d, d, 0}; return MOE_OK;
    case MOE_W_GATE:
    case MOE_W_UP:
      if (le < 0 || le >= L->E_local) return fail(L, MOE_INVALID_INPUT, "expert %d is not owned by this handle", expert);
      *s = {L->off_gu + (long long)le * 2 * Fp * d, F, d, d, which == MOE_W_GATE ? 1 : 2};
      return MOE_OK;
    case MOE_W_DOWN:
      if (le < 0 || le >= L->E_local) return fail(L, MOE_INVALID_INPUT, "expert %d is not owned by this handle", expert);
      *s = {L->off_d + (long long)le * d * Fp, d, F, Fp, 0};
      return MOE_OK;
    case MOE_W_SHARED_GATE:
    case MOE_W_SHARED_UP:
      if (!L->shared) return fail(L, MOE_INVALID_INPUT, "the layer has no shared expert");
      *s = {L->off_sgu, F, d, d, which == MOE_W_SHARED_GATE ? 1 : 2};
      return MOE_OK;
    case MOE_W_SHARED_DOWN:
      if (!L->shared) return fail(L, MOE_INVALID_INPUT, "the layer has no shared expert");
      *s = {L->off_sd, d, F, Fp, 0};
      return MOE_OK;
  }
  return fail(L, MOE_INVALID_INPUT, "unknown weight id %d", which);
}

__global__ void pack_kernel(const float* __restrict__ src, float* __restrict__ dst, bf16* __restrict__ dst_bf16,
                            int rows, int cols, int ld, int kind) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)rows * cols) return;
  const int r = (int)(i / cols), c = (int)(i - (long long)r * cols);
  const int pr = kind == 0 ? r : gu_row(kind - 1, r);
  const float v = src[i];
  dst[(long long)pr * ld + c] = v;
  if (dst_bf16) dst_bf16[(long long)pr * ld + c] = __float2bfloat16_rn(v);
}
__global__ void unpack_kernel(const float* __restrict__ src, float* __restrict__ dst, int rows, int cols, int ld,
                              int kind, int zero) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)rows * cols) return;
  const int r = (int)(i / cols), c = (int)(i - (long long)r * cols);
  const int pr = kind == 0 ? r : gu_row(kind - 1, r);
  dst[i] = zero ? 0.f : src[(long long)pr * ld + c];
}
__global__ void pack_q8_kernel(const int8_t* __restrict__ src, const float* __restrict__ scale_src,
                               int8_t* __restrict__ dst, float* __restrict__ scale_dst, int rows, int cols, int ld,
                               int kind) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)rows * cols) return;
  const int r = (int)(i / cols), c = (int)(i - (long long)r * cols);
  const int pr = kind == 0 ? r : gu_row(kind - 1, r);
  // fragment-major: blocks of 8 rows x 64 reduction values are contiguous (512 bytes, row-major inside),
  // blocks of one 8-row stripe follow each other along the reduction: a warp of the decode kernel reads
  // one block per load and streams a stripe front to back
  // and every byte has its sign bit flipped (value + 128 as an unsigned byte), which is the form the
  // kernel's int8 -> f16 widening wants; padding bytes of the arena are written as 0x80 at allocation
  dst[(long long)(pr / 8) * 8 * ld + (long long)(c / 64) * 512 + (pr % 8) * 64 + (c % 64)] = (int8_t)(src[i] ^ (int8_t)0x80);
  if (c == 0) scale_dst[pr] = scale_src[r];
}
// Row ranges of the token chunks the router weight gradient is split into (rows are the reduction of
// that GEMM): meta[g] = min(g * chunk, padded), g = 0..splits.
__global__ void split_meta_kernel(int* meta, int splits, int chunk, int padded) {
  const int g = threadIdx.x;
  if (g <= splits) meta[g] = min(g * chunk, padded);
}
// Group table of the dense (shared expert, router) GEMMs for every possible token count: entry t is
// {row0[0], row0[1], tile_start[0], tile_start[1]} of one group of t rows.  Filled once, so a pass only
// picks a pointer instead of launching a kernel.
__global__ void shared_meta_table_kernel(int* table, int max_tokens) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t > max_tokens) return;
  const int rows = round_up(t, GROUP_ALIGN);
  table[4 * t] = 0; table[4 * t + 1] = rows; table[4 * t + 2] = 0; table[4 * t + 3] = rows / GROUP_ALIGN;
}

__global__ void add_inplace_kernel(float* __restrict__ dst, const float* __restrict__ src, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] += src[i];
}

bool is_device_pointer(const void* p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

// MOE_B200_Q8_TC=1 selects the tcgen05 variant of the int8 decode projections (decode_q8_tc.cu).
bool q8_tc_mode() {
  static const bool on = [] { const char* v = getenv("MOE_B200_Q8_TC"); return v && atoi(v) != 0; }();
  return on;
}

int check_flag(moe_layer* L) {
  int flag = 0;
  CK(cudaMemcpy(&flag, L->error_flag, sizeof(int), cudaMemcpyDeviceToHost));
  if (flag != 0) {
    cudaMemset(L->error_flag, 0, sizeof(int));
    if (flag == 300) {
      L->err = "InvalidInput: more rows were routed to one rank's experts than its receive buffers hold; raise ep_capacity_factor (nothing was sent)";
      return MOE_INVALID_INPUT;
    }
    return fail(L, MOE_TIMEOUT, "a bounded device-side wait gave up (code %d)", flag);
  }
  return MOE_OK;
}

// ---------------------------------------------------------------------------
// expert stacks: one set of row groups through gate|up -> SwiGLU -> down
// ---------------------------------------------------------------------------
struct Groups {
  const int* row0;
  const int* tstart;
  int n_groups;
  int cap_rows;       // rows of the internal row-indexed buffers
  int in_rows;        // readable rows of the external input operand
};
struct ExpertIO {
  const void* x;          // input rows [*, d]
  void *gu, *h, *y;       // [cap, 2Fp], [cap, Fp], [cap, d]
  const void* dy;         // upstream gradient rows [*, d]
  void *dgu, *dx, *dh;    // [cap, 2Fp], [cap, d], [cap, Fp] (dh: f32 path only)
  long long w_gu, w_d;    // arena offsets
};

int experts_forward(moe_layer* L, const Groups& G, const ExpertIO& io, bool save, cudaStream_t st, bool routed) {
  const int d = L->d, Fp = L->F_pad;
  Span whole(L, routed ? -1 : 13, st);
  if (L->act == PREC_BF16) {
    tc::GemmArgs a{};
    a.group_row0 = G.row0; a.tile_start = G.tstart; a.n_groups = G.n_groups; a.error_flag = L->error_flag;
    a.N = 2 * Fp; a.K = d;
    a.out0 = io.h; a.ld0 = Fp; a.out1 = save ? io.gu : nullptr; a.ld1 = 2 * Fp;
    tc::Operand A{io.x, G.in_rows, d, 1};
    tc::Operand B{L->wb + io.w_gu, 2 * Fp, d, G.n_groups};
    { Span sp(L, routed ? 2 : -1, st); CK(tc::gemm_rows_nt(A, B, a, tc::EPI_SWIGLU, L->sm_count, st)); }
    tc::GemmArgs b{};
    b.group_row0 = G.row0; b.tile_start = G.tstart; b.n_groups = G.n_groups; b.error_flag = L->error_flag;
    b.N = d; b.K = Fp; b.out0 = io.y; b.ld0 = d;
    tc::Operand A2{io.h, G.cap_rows, Fp, 1};
    tc::Operand B2{L->wb + io.w_d, d, Fp, G.n_groups};
    { Span sp(L, routed ? 3 : -1, st); CK(tc::gemm_rows_nt(A2, B2, b, tc::EPI_STORE, L->sm_count, st)); }
  } else if (L->w3) {
    // f32 on the tensor cores: three bf16 pieces per operand, six cross terms along a reduction six times as long
    if (L->w3_dirty) {
      const int El = L->E_local;
      CK(launch_expand3(L->wc + L->off_gu, L->w3 + 6 * L->off_gu, (long long)El * 2 * Fp, d, 1, st));
      CK(launch_expand3(L->wc + L->off_d, L->w3 + 6 * L->off_d, (long long)El * d, Fp, 1, st));
      if (L->shared) {
        CK(launch_expand3(L->wc + L->off_sgu, L->w3 + 6 * L->off_sgu, 2ll * Fp, d, 1, st));
        CK(launch_expand3(L->wc + L->off_sd, L->w3 + 6 * L->off_sd, (long long)d, Fp, 1, st));
      }
      L->w3_dirty = false;
    }
    tc::GemmArgs a{};
    a.group_row0 = G.row0; a.tile_start = G.tstart; a.n_groups = G.n_groups; a.error_flag = L->error_flag;
    a.N = 2 * Fp; a.K = 6 * d; a.M = G.cap_rows; a.out0 = io.gu; a.ld0 = 2 * Fp;
    { Span sp(L, routed ? 2 : -1, st);
      CK(launch_expand3((const float*)io.x, L->xa3, G.in_rows, d, 0, st));
      // The tensor core adds into its accumulator with truncation, a bias that grows with the number of additions:
      // the leading term (hi x hi, first segment) therefore gets a product of its own over the short reduction, and
      // the five small cross terms are accumulated apart and added to it in f32 by the epilogue.
      a.K = d; a.accumulate = 0;
      CK(tc::gemm_rows_nt(tc::Operand{L->xa3, G.in_rows, d, 1, 6 * d}, tc::Operand{L->w3 + 6 * io.w_gu, 2 * Fp, d, G.n_groups, 6 * d}, a,
                          tc::EPI_STORE_F32, L->sm_count, st));
      a.K = 5 * d; a.accumulate = 1;
      CK(tc::gemm_rows_nt(tc::Operand{L->xa3 + d, G.in_rows, 5 * d, 1, 6 * d},
                          tc::Operand{L->w3 + 6 * io.w_gu + d, 2 * Fp, 5 * d, G.n_groups, 6 * d}, a, tc::EPI_STORE_F32, L->sm_count, st));
      CK(launch_swiglu_fwd_f32((const float*)io.gu, (float*)io.h, G.cap_rows, Fp, st)); }
    tc::GemmArgs b{};
    b.group_row0 = G.row0; b.tile_start = G.tstart; b.n_groups = G.n_groups; b.error_flag = L->error_flag;
    b.N = d; b.K = 6 * Fp; b.M = G.cap_rows; b.out0 = io.y; b.ld0 = d;
    { Span sp(L, routed ? 3 : -1, st);
      CK(launch_expand3((const float*)io.h, L->ha3, G.cap_rows, Fp, 0, st));
      b.K = Fp; b.accumulate = 0;
      CK(tc::gemm_rows_nt(tc::Operand{L->ha3, G.cap_rows, Fp, 1, 6 * Fp}, tc::Operand{L->w3 + 6 * io.w_d, d, Fp, G.n_groups, 6 * Fp}, b,
                          tc::EPI_STORE_F32, L->sm_count, st));
      b.K = 5 * Fp; b.accumulate = 1;
      CK(tc::gemm_rows_nt(tc::Operand{L->ha3 + Fp, G.cap_rows, 5 * Fp, 1, 6 * Fp},
                          tc::Operand{L->w3 + 6 * io.w_d + Fp, d, 5 * Fp, G.n_groups, 6 * Fp}, b, tc::EPI_STORE_F32, L->sm_count, st)); }
  } else {
    SimtGemmArgs a{};
    a.A = (const float*)io.x; a.B = L->wc + io.w_gu; a.C = (float*)io.gu;
    a.group_row0 = G.row0; a.n_groups = G.n_groups; a.max_rows = G.cap_rows; a.a_rows = G.in_rows; a.b_rows = 0;
    a.N = 2 * Fp; a.K = d; a.b_group_stride = 2ll * Fp * d;
    { Span sp(L, routed ? 2 : -1, st); CK(simt_gemm_nt(a, st));
    CK(launch_swiglu_fwd_f32((const float*)io.gu, (float*)io.h, G.cap_rows, Fp, st)); }
    SimtGemmArgs b{};
    b.A = (const float*)io.h; b.B = L->wc + io.w_d; b.C = (float*)io.y;
    b.group_row0 = G.row0; b.n_groups = G.n_groups; b.max_rows = G.cap_rows; b.a_rows = G.cap_rows;
    b.N = d; b.K = Fp; b.b_group_stride = (long long)d * Fp;
    { Span sp(L, routed ? 3 : -1, st); CK(simt_gemm_nt(b, st)); }
  }
  return MOE_OK;
}

// Weight gradient of the dense (shared expert) group: the output is a handful of tiles and the token rows are the
// reduction, so as one group it would keep a dozen SMs busy.  When the tiles do not fill the GPU the rows are cut
// into chunks (one group each, partial results in scratch) and the chunks are added in order afterwards.
__global__ void split_rows_kernel(int* meta, int splits, int chunk, int padded) {
  const int g = threadIdx.x;
  if (g <= splits) meta[g] = min(g * chunk, padded);
}
__global__ void add_partials_kernel(float* __restrict__ dst, const float* __restrict__ part, long long n, int splits, int accumulate) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = accumulate ? dst[i] : 0.f;
  for (int s = 0; s < splits; ++s) acc += part[(long long)s * n + i];
  dst[i] = acc;
}
int dense_wgrad(moe_layer* L, const tc::Operand& A, const tc::Operand& B, int rows, int M, int N, float* out, int acc, cudaStream_t st) {
  const int tiles = ceil_div(M, tc::BM) * ceil_div(N, tc::BN);
  const int padded = round_up(rows, GROUP_ALIGN);
  int splits = std::min(16, std::max(1, L->sm_count / std::max(1, tiles)));
  const int chunk = round_up(ceil_div(padded, splits), GROUP_ALIGN);
  splits = ceil_div(padded, chunk);
  tc::GemmArgs w{};
  w.error_flag = L->error_flag; w.M = M; w.N = N; w.ld0 = N;
  if (splits <= 1 || !L->sh_scratch || (long long)splits * M * N > L->sh_scratch_elems) {
    w.group_row0 = L->shared_meta; w.n_groups = 1; w.out0 = out; w.group_stride0 = (long long)M * N; w.accumulate = acc;
    CK(tc::gemm_rows_tn(A, B, w, L->sm_count, st));
    return MOE_OK;
  }
  split_rows_kernel<<<1, 32, 0, st>>>(L->sh_meta, splits, chunk, padded); count_launch();
  w.group_row0 = L->sh_meta; w.n_groups = splits; w.out0 = L->sh_scratch; w.group_stride0 = (long long)M * N; w.accumulate = 0;
  CK(tc::gemm_rows_tn(A, B, w, L->sm_count, st));
  const long long n = (long long)M * N;
  add_partials_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(out, L->sh_scratch, n, splits, acc); count_launch();
  CK(cudaGetLastError());
  return MOE_OK;
}

// phase 0: everything; 1: everything except the gate|up weight gradient; 2: only that gradient
// (it does not feed the input gradient, so the un-permute can run beside it).
// parts: 1 = the input-gradient chain (dgrad down + SwiGLU backward, dgrad gate|up), 2 = dW_down, 4 = dW_gate|up
int experts_backward(moe_layer* L, const Groups& G, const ExpertIO& io, cudaStream_t st, bool routed, int parts = 7) {
  const int d = L->d, Fp = L->F_pad;
  Span whole(L, routed ? -1 : 14, st);
  // replicated parameters of an expert-parallel layer: this pass's contribution is written alone, summed
  // over the ranks, and only then added to what earlier passes left (see backward_impl)
  const int acc = L->grad_valid && (routed || !L->rep_overwrite) ? 1 : 0;
  if (L->act == PREC_BF16) {
    // dgu = swiglu'(dy W_d) ; dW_d += dy^T h ; dx = dgu W_gu ; dW_gu += dgu^T x
    if (parts & 1) {
    tc::GemmArgs a{};
    a.group_row0 = G.row0; a.tile_start = G.tstart; a.n_groups = G.n_groups; a.error_flag = L->error_flag;
    a.N = Fp; a.K = d; a.out0 = io.dgu; a.ld0 = 2 * Fp; a.aux = io.gu; a.ldaux = 2 * Fp;
    tc::Operand A{io.dy, G.in_rows, d, 1};
    tc::Operand B{L->wb + io.w_d, d, Fp, G.n_groups};
    { Span sp(L, routed ? 6 : -1, st); CK(tc::gemm_rows_nn(A, B, a, tc::EPI_SWIGLU_BWD, L->sm_count, st)); }
    }
    if (parts & 2) {
    tc::GemmArgs wd{};
    wd.group_row0 = G.row0; wd.n_groups = G.n_groups; wd.error_flag = L->error_flag;
    wd.M = d; wd.N = Fp; wd.out0 = L->g + io.w_d; wd.ld0 = Fp; wd.group_stride0 = (long long)d * Fp; wd.accumulate = acc;
    tc::Operand Ad{io.dy, G.in_rows, d, 1};
    tc::Operand Bd{io.h, G.cap_rows, Fp, 1};
    { Span sp(L, routed ? 7 : -1, st);
      if (routed) CK(tc::gemm_rows_tn(Ad, Bd, wd, L->sm_count, st));
      else { const int r_ = dense_wgrad(L, Ad, Bd, G.in_rows, d, Fp, L->g + io.w_d, acc, st); if (r_ != MOE_OK) return r_; } }
    }
    if (parts & 1) {
    tc::GemmArgs b{};
    b.group_row0 = G.row0; b.tile_start = G.tstart; b.n_groups = G.n_groups; b.error_flag = L->error_flag;
    b.N = d; b.K = 2 * Fp; b.out0 = io.dx; b.ld0 = d;
    tc::Operand A2{io.dgu, G.cap_rows, 2 * Fp, 1};
    tc::Operand B2{L->wb + io.w_gu, 2 * Fp, d, G.n_groups};
    { Span sp(L, routed ? 8 : -1, st); CK(tc::gemm_rows_nn(A2, B2, b, tc::EPI_STORE, L->sm_count, st)); }
    }
    if (parts & 4) {
    tc::GemmArgs wg{};
    wg.group_row0 = G.row0; wg.n_groups = G.n_groups; wg.error_flag = L->error_flag;
    wg.M = 2 * Fp; wg.N = d; wg.out0 = L->g + io.w_gu; wg.ld0 = d; wg.group_stride0 = 2ll * Fp * d; wg.accumulate = acc;
    tc::Operand Ag{io.dgu, G.cap_rows, 2 * Fp, 1};
    tc::Operand Bg{io.x, G.in_rows, d, 1};
    { Span sp(L, routed ? 9 : -1, st);
      if (routed) CK(tc::gemm_rows_tn(Ag, Bg, wg, L->sm_count, st));
      else { const int r_ = dense_wgrad(L, Ag, Bg, G.in_rows, 2 * Fp, d, L->g + io.w_gu, acc, st); if (r_ != MOE_OK) return r_; } }
    }
  } else {
    if (parts & 1) {
    SimtGemmArgs a{};
    a.A = (const float*)io.dy; a.B = L->wc + io.w_d; a.C = (float*)io.dh;
    a.group_row0 = G.row0; a.n_groups = G.n_groups; a.max_rows = G.cap_rows; a.a_rows = G.in_rows;
    a.N = Fp; a.K = d; a.b_group_stride = (long long)d * Fp;
    { Span sp(L, routed ? 6 : -1, st); CK(simt_gemm_nn(a, st));
    CK(launch_swiglu_bwd_f32((const float*)io.dh, (const float*)io.gu, (float*)io.dgu, G.cap_rows, Fp, st)); }
    }
    if (parts & 2) {
    SimtGemmArgs wd{};
    wd.A = (const float*)io.dy; wd.B = (const float*)io.h; wd.C = L->g + io.w_d;
    wd.group_row0 = G.row0; wd.n_groups = G.n_groups; wd.a_rows = G.in_rows; wd.b_rows = G.cap_rows;
    wd.M = d; wd.N = Fp; wd.c_group_stride = (long long)d * Fp; wd.accumulate = acc;
    { Span sp(L, routed ? 7 : -1, st); CK(simt_gemm_tn(wd, st)); }
    }
    if (parts & 1) {
    SimtGemmArgs b{};
    b.A = (const float*)io.dgu; b.B = L->wc + io.w_gu; b.C = (float*)io.dx;
    b.group_row0 = G.row0; b.n_groups = G.n_groups; b.max_rows = G.cap_rows; b.a_rows = G.cap_rows;
    b.N = d; b.K = 2 * Fp; b.b_group_stride = 2ll * Fp * d;
    { Span sp(L, routed ? 8 : -1, st); CK(simt_gemm_nn(b, st)); }
    }
    if (parts & 4) {
    SimtGemmArgs wg{};
    wg.A = (const float*)io.dgu; wg.B = (const float*)io.x; wg.C = L->g + io.w_gu;
    wg.group_row0 = G.row0; wg.n_groups = G.n_groups; wg.a_rows = G.cap_rows; wg.b_rows = G.in_rows;
    wg.M = 2 * Fp; wg.N = d; wg.c_group_stride = 2ll * Fp * d; wg.accumulate = acc;
    { Span sp(L, routed ? 9 : -1, st); CK(simt_gemm_tn(wg, st)); }
    }
  }
  return MOE_OK;
}

#include "ep_impl.inc"
#include "lora_impl.inc"

int forward_impl(moe_layer* L, const void* x, const float* logits_in, int tokens, int cols, const uint8_t* valid,
                 void* y, int accumulate, int save, cudaStream_t st) {
  if (cols != L->d) {   // moe.rs:248-253
    L->err = "InvalidInput: expected " + std::to_string(L->d) + " columns, got " + std::to_string(cols);
    return MOE_INVALID_INPUT;
  }
  if (tokens < 0 || tokens > L->max_tokens) {
    L->err = "InvalidInput: " + std::to_string(tokens) + " tokens exceed max_tokens " + std::to_string(L->max_tokens);
    return MOE_INVALID_INPUT;
  }
  if (tokens > 0 && (!x || !y)) { L->err = "InvalidInput: null activation pointer"; return MOE_INVALID_INPUT; }
  if (save && !L->training) { L->err = "InvalidConfig: save_for_backward needs a handle created with training = 1"; return MOE_INVALID_CONFIG; }
  const bool ep = L->ep_size > 1;
  if (ep && !L->ep_ready) { L->err = "InvalidConfig: expert-parallel handle without a communicator (call moe_ep_init)"; return MOE_INVALID_CONFIG; }
  L->have_cache = false;
  L->last_tokens = tokens;
  L->last_stream = st;
  if (tokens == 0 && !ep) return MOE_OK;   // an expert-parallel rank with no tokens still serves its experts
  { const int fr = lora_fold(L, st); if (fr != MOE_OK) return fr; }   // adapters into the compute weights, if they changed
  if (L->training && overlap_mode() == 2) select_parity(L, L->parity ^ 1);   // deferred weight gradients may still read the other half

  RouterArgs ra{};
  ra.x = x; ra.w_router = L->w + L->off_router; ra.logits_in = logits_in; ra.valid = valid;
  ra.tokens = tokens; ra.d = L->d; ra.E = L->E; ra.k = L->k;
  ra.logits_out = L->logits; ra.probs = L->probs; ra.lse = L->lse; ra.expert_of = L->expert_of; ra.gates = L->gates;
  ra.partial = L->partial; ra.hist = L->hist;
  ra.fin = RouterFinalize{1, L->aux_w, L->z_w, L->meta, L->stats, L->losses, ep ? 1 : GROUP_ALIGN};
  L->shared_meta = L->shared_meta_table + 4 * tokens;
  PermuteArgs pa{};
  pa.x = x; pa.expert_of = L->expert_of; pa.gates = L->gates; pa.cursor = L->hist; pa.meta = L->meta;
  pa.tokens = tokens; pa.d = L->d; pa.E = L->E; pa.k = L->k;
  pa.x_perm = ep ? ep_rows(L, 0, L->x_perm) : local_rows(L->x_perm); pa.slot_pos = L->slot_pos;
  pa.dest_base = (ep && L->peer_ready) ? L->dest_base : nullptr; pa.row_token = L->row_token; pa.row_gate = L->row_gate;
  pa.token_of = L->token_of; pa.slot_of = L->slot_of;
  pa.skip_pad = L->precision == MOE_PRECISION_Q8 ? 1 : 0;   // the int8 kernels never read padding rows
  // int8 decode layer on a decode-sized batch: the whole routing in one launch, and no row copy (the first int8
  // pass gathers its token rows through row_token); not with the tcgen05 variant, whose loads want the rows in place
  bool gather_rows = false;
  { Span sp(L, 0, st);
  RouterArgs fa = ra;
  fa.logits_in = L->logits; fa.logits_out = nullptr;
  if (L->precision == MOE_PRECISION_Q8 && L->tc_router && !logits_in && !ep && !L->prof_on && !q8_tc_mode() &&
      decode_route_supported(fa, pa)) {
    CK(launch_decode_route_rows(fa, pa, L->wb + L->off_router, L->route_done, st));
    gather_rows = true;
  } else if (L->tc_router && !logits_in && tokens <= 256 && L->d % 8 == 0 && ((uintptr_t)x & 15) == 0) {
    // decode-sized batch: a CTA per token row beats one tensor-core tile on one SM
    CK(launch_router_logits_rows(x, L->wb + L->off_router, L->logits, tokens, L->d, L->E, st));
    ra.logits_in = L->logits;
    ra.logits_out = nullptr;
  } else if (L->tc_router && !logits_in) {
    // logits = x W_r^T on the tensor cores, f32 out; softmax/top-k then read them back
    tc::GemmArgs g{};
    g.group_row0 = L->shared_meta; g.tile_start = L->shared_meta + 2; g.n_groups = 1; g.error_flag = L->error_flag;
    g.N = L->E; g.K = L->d; g.M = tokens; g.out0 = L->logits; g.ld0 = L->E;
    tc::Operand A{x, tokens, L->d, 1};
    tc::Operand B{L->wb + L->off_router, L->E, L->d, 1};
    CK(tc::gemm_rows_nt(A, B, g, tc::EPI_STORE_F32, L->sm_count, st));
    ra.logits_in = L->logits;
    ra.logits_out = nullptr;
  }
  if (!gather_rows) {
    CK(launch_router(ra, L->act, st));
    CK(launch_finalize(ra, L->meta, L->aux_w, L->z_w, L->stats, L->losses, ep ? 1 : GROUP_ALIGN, st));
  } }

  if (ep) {
    Span sp(L, 1, st);
    int rc0 = ep_dispatch(L, st);
    if (rc0 != MOE_OK) return rc0;
  }
  if (!gather_rows) { Span sp(L, 1, st); CK(launch_permute(pa, L->act, st)); }

  int rc;
  if (L->precision == MOE_PRECISION_Q8) {
    // decode: stream each active expert's int8 rows once; the shared expert rides along as group E
    Span sp(L, 2, st);
    const int d = L->d, Fp = L->F_pad;
    Q8Args qa{};
    qa.x_rows = (const bf16*)L->x_perm; qa.x_shared = L->shared ? (const bf16*)x : nullptr;
    if (gather_rows) { qa.x_rows = (const bf16*)x; qa.x_row_index = L->row_token; }
    qa.out_rows = (bf16*)L->h; qa.out_shared = (bf16*)L->h_s;
    qa.w = L->q_gu; qa.scale = L->s_gu; qa.counts = L->meta.counts; qa.pad_off = L->meta.pad_off;
    qa.w_group_stride = 2ll * Fp * d; qa.s_group_stride = 2ll * Fp;
    qa.sm_count = L->sm_count; qa.E = L->E; qa.tokens = tokens; qa.K = d; qa.N = Fp; qa.ldo = Fp;
    qa.x_rows_cap = L->rows_cap; qa.x_shared_rows = tokens; qa.error_flag = L->error_flag;
    const bool tc = q8_tc_mode();
    if (tc && q8_tc_supported(qa, true)) CK(launch_q8_rows_tc(qa, true, st)); else CK(launch_q8_rows(qa, true, st));
    Q8Args qb{};
    qb.x_rows = (const bf16*)L->h; qb.x_shared = L->shared ? (const bf16*)L->h_s : nullptr;
    qb.out_rows = (bf16*)L->y_perm; qb.out_shared = (bf16*)L->y_s;
    qb.w = L->q_d; qb.scale = L->s_d; qb.counts = L->meta.counts; qb.pad_off = L->meta.pad_off;
    qb.w_group_stride = (long long)d * Fp; qb.s_group_stride = d;
    qb.sm_count = L->sm_count; qb.E = L->E; qb.tokens = tokens; qb.K = Fp; qb.N = d; qb.ldo = d;
    qb.x_rows_cap = L->rows_cap; qb.x_shared_rows = L->shared_rows_cap; qb.error_flag = L->error_flag;
    if (tc && q8_tc_supported(qb, false)) CK(launch_q8_rows_tc(qb, false, st)); else CK(launch_q8_rows(qb, false, st));
    rc = MOE_OK;
  } else if (ep) {
    rc = ep_forward_experts(L, save != 0, st);
  } else {
    if ((rc = join_side(L, st)) != MOE_OK) return rc;   // the expert GEMMs rewrite what deferred gradients read
    Groups G{L->meta.pad_off, L->meta.tile_start, L->E, L->rows_cap, L->rows_cap};
    ExpertIO io{};
    io.x = L->x_perm; io.gu = L->gu; io.h = L->h; io.y = L->y_perm; io.w_gu = L->off_gu; io.w_d = L->off_d;
    rc = experts_forward(L, G, io, save != 0, st, true);
  }
  if (rc != MOE_OK) return rc;

  if (L->shared && tokens > 0 && L->precision != MOE_PRECISION_Q8) {
    Groups S{L->shared_meta, L->shared_meta + 2, 1, L->shared_rows_cap, tokens};
    ExpertIO sio{};
    sio.x = x; sio.gu = L->gu_s; sio.h = L->h_s; sio.y = L->y_s; sio.w_gu = L->off_sgu; sio.w_d = L->off_sd;
    rc = experts_forward(L, S, sio, save != 0, st, false);
    if (rc != MOE_OK) return rc;
  }

  CombineArgs ca{};
  ca.y_perm = ep ? ep_rows(L, 1, L->y_perm) : local_rows(L->y_perm); ca.shared = L->shared ? L->y_s : nullptr; ca.expert_of = L->expert_of; ca.gates = L->gates;
  ca.slot_pos = L->slot_pos; ca.y = y; ca.tokens = tokens; ca.d = L->d; ca.k = L->k; ca.accumulate = accumulate;
  { Span sp(L, 4, st); CK(launch_combine(ca, L->act, st)); }
  CK(cudaGetLastError());
  L->have_cache = save != 0;
  L->last_x = x;
  return MOE_OK;
}

// force_mode 3 (host entry point, one GPU): like overlap mode 2 but the fork comes as late as possible
// (every tensor-core launch that feeds grad_x goes first, so nothing on the caller's stream queues behind
// the weight-gradient GEMMs) and the caller joins the side stream before it returns.
int backward_impl(moe_layer* L, const void* gy, void* gx, int accumulate, cudaStream_t st, int force_mode = -1) {
  if (!L->training) { L->err = "InvalidConfig: the handle was created with training = 0"; return MOE_INVALID_CONFIG; }
  if (!L->have_cache) { L->err = "InvalidInput: moe_backward needs a preceding moe_forward with save_for_backward"; return MOE_INVALID_INPUT; }
  if (!gy || !gx) { L->err = "InvalidInput: null gradient pointer"; return MOE_INVALID_INPUT; }
  const int tokens = L->last_tokens;
  const bool ep = L->ep_size > 1;
  if (tokens == 0 && !ep) return MOE_OK;
  // Gradient accumulation over several passes (accumulate_step, transformer.rs:1519) on an expert-parallel
  // handle: the experts' gradients accumulate in place as on one GPU.  The replicated ones (router, shared
  // expert) hold a sum over ranks already, so this pass's local contribution must not be added to them before
  // the all-reduce: the old values are set aside, the pass overwrites, the all-reduce sums the ranks, and the
  // old values are added back.
  const bool ep_accum = ep && L->grad_valid;
  const long long rep_router = (long long)L->E * L->d, rep_shared = L->shared ? L->n_params - L->off_sgu : 0;
  if (ep_accum) {
    CK(cudaMemcpyAsync(L->g_rep_save, L->g + L->off_router, (size_t)rep_router * 4, cudaMemcpyDeviceToDevice, st));
    if (rep_shared > 0)
      CK(cudaMemcpyAsync(L->g_rep_save + rep_router, L->g + L->off_sgu, (size_t)rep_shared * 4, cudaMemcpyDeviceToDevice, st));
  }
  L->rep_overwrite = ep_accum;
  const int rep_acc = L->grad_valid && !ep_accum ? 1 : 0;

  const bool owner_dots = ep && L->peer_ready;   // gate gradient computed where the expert output lives
  const size_t aux_off = (size_t)L->rows_cap_l * L->d * L->esz;
  if (owner_dots) {
    PushGradArgs pa{};
    pa.grad_y = gy; pa.rows = ep_rows(L, 2, L->dy_perm); pa.slot_pos = L->slot_pos; pa.gates = L->gates;
    pa.aux_off = aux_off; pa.tokens = tokens; pa.d = L->d; pa.k = L->k;
    pa.dedup = ep_push_dedup(L) ? 1 : 0;
    pa.stage = ep_rows(L, 3, L->dx_perm); pa.stage_base = L->ep_rank * L->max_tokens;
    Span sp(L, 5, st); CK(launch_push_grad(pa, L->act, st));
  } else {
    GatherGradArgs ga{};
    ga.grad_y = gy; ga.y_perm = ep ? ep_rows(L, 1, L->y_perm) : local_rows(L->y_perm); ga.slot_pos = L->slot_pos; ga.gates = L->gates;
    ga.grad_y_perm = ep ? ep_rows(L, 2, L->dy_perm) : local_rows(L->dy_perm); ga.grad_gates = L->grad_gates; ga.tokens = tokens; ga.d = L->d; ga.k = L->k;
    Span sp(L, 5, st); CK(launch_gather_grad(ga, L->act, st));
    if (!ep) CK(launch_pad_rows(L->dy_perm, L->d, L->meta, L->E, L->act, st));
  }

  tc::Operand RA{L->gl_bf16, tokens, L->E, 1};
  auto router_backward = [&]() -> int {
    RouterBwdArgs rb{};
    rb.probs = L->probs; rb.lse = L->lse; rb.expert_of = L->expert_of; rb.grad_gates = L->grad_gates;
    rb.counts = L->meta.counts; rb.total = L->meta.total; rb.tokens = tokens; rb.E = L->E; rb.k = L->k;
    rb.aux_w = L->aux_w; rb.z_w = L->z_w; rb.grad_logits = L->grad_logits;
    rb.grad_logits_bf16 = L->tc_router ? L->gl_bf16 : nullptr;
    if (ep) { rb.ext_stats = L->ext_stats; rb.ext_counts = L->ext_counts; }
    { Span sp(L, 10, st); CK(launch_router_bwd(rb, st)); }
    if (L->tc_router && tokens > 0) {
      // router input gradient grad_logits W_r: one more launch of the grouped tensor-core GEMM
      Span sp(L, 12, st);
      tc::GemmArgs g{};
      g.group_row0 = L->shared_meta; g.tile_start = L->shared_meta + 2; g.n_groups = 1; g.error_flag = L->error_flag;
      g.N = L->d; g.K = L->E; g.out0 = L->dx_r; g.ld0 = L->d;
      tc::Operand B{L->wb + L->off_router, L->E, L->d, 1};
      CK(tc::gemm_rows_nn(RA, B, g, tc::EPI_STORE, L->sm_count, st));
    }
    return MOE_OK;
  };
  auto router_weight_gradient = [&](cudaStream_t s) -> int {
    if (L->tc_router && tokens > 0) {
      // E x d output = a handful of tiles, tokens = the reduction: split the tokens into chunks (one
      // group each, partial results in scratch) so that every SM has a tile, then add the chunks in order
      Span sp(L, 12, s);
      const int tiles = ceil_div(L->E, 128) * ceil_div(L->d, 256);
      const int padded = round_up(tokens, GROUP_ALIGN);
      int splits = std::max(1, std::min(std::min(L->rw_splits, 64), L->sm_count / std::max(1, tiles)));
      const int chunk = round_up(ceil_div(padded, splits), GROUP_ALIGN);
      splits = ceil_div(padded, chunk);
      tc::GemmArgs wg{};
      wg.error_flag = L->error_flag;
      wg.M = L->E; wg.N = L->d; wg.ld0 = L->d;
      tc::Operand Ax{L->last_x, tokens, L->d, 1};
      if (splits > 1) {
        split_meta_kernel<<<1, 128, 0, s>>>(L->rw_meta, splits, chunk, padded); count_launch();
        wg.group_row0 = L->rw_meta; wg.n_groups = splits; wg.out0 = L->rw_scratch;
        wg.group_stride0 = (long long)L->E * L->d; wg.accumulate = 0;
        CK(tc::gemm_rows_tn(RA, Ax, wg, L->sm_count, s));
        RouterWgradArgs rw{};
        rw.grad_w = L->g + L->off_router; rw.scratch = L->rw_scratch; rw.d = L->d; rw.E = L->E; rw.splits = splits;
        rw.accumulate = rep_acc;
        CK(launch_router_wgrad_sum(rw, s));
      } else {
        wg.group_row0 = L->shared_meta; wg.n_groups = 1; wg.out0 = L->g + L->off_router;
        wg.accumulate = rep_acc;
        CK(tc::gemm_rows_tn(RA, Ax, wg, L->sm_count, s));
      }
    } else {
      RouterWgradArgs rw{};
      rw.grad_logits = L->grad_logits; rw.x = L->last_x; rw.grad_w = L->g + L->off_router; rw.scratch = L->rw_scratch;
      rw.tokens = tokens; rw.d = L->d; rw.E = L->E; rw.splits = L->rw_splits; rw.accumulate = rep_acc;
      Span sp(L, 12, s); CK(launch_router_wgrad(rw, L->act, s));
    }
    return MOE_OK;
  };
  // mode 2: only the input-gradient chain stays on the caller's stream; both routed weight gradients
  // go to the side stream and are joined by whichever later call needs their inputs or outputs
  // stage timing brackets launches on the caller's stream; mode 1 keeps every bracketed stage there (only the
  // un-permute moves to the side stream and goes untimed), modes 2 and 3 do not
  const int chosen = overlap_mode() >= 0 ? overlap_mode() : (L->ep_size >= 4 ? 1 : 0);
  const int want = force_mode == 3 && !ep ? 3 : chosen;
  const int mode = L->prof_on && want != 1 ? 0 : want;
  const int first_parts = mode >= 2 ? 1 : 3;
  Groups G{L->meta.pad_off, L->meta.tile_start, L->E, L->rows_cap, L->rows_cap};
  ExpertIO io{};
  io.x = L->x_perm; io.gu = L->gu; io.h = L->h; io.y = L->y_perm; io.dy = L->dy_perm; io.dgu = L->dgu;
  io.dx = L->dx_perm; io.dh = L->dh; io.w_gu = L->off_gu; io.w_d = L->off_d;
  int rc = join_side(L, st);
  if (rc != MOE_OK) return rc;
  if (mode == 3 && (rc = router_backward()) != MOE_OK) return rc;   // needs the gate gradients only
  rc = ep ? ep_backward_experts(L, st, first_parts) : experts_backward(L, G, io, st, true, first_parts);
  if (rc != MOE_OK) return rc;
  if (mode == 2) {
    CK(cudaEventRecord(L->ev_fork, st));
    CK(cudaStreamWaitEvent(L->side_stream, L->ev_fork, 0));
    rc = ep ? ep_backward_experts(L, L->side_stream, 6) : experts_backward(L, G, io, L->side_stream, true, 6);
    if (rc != MOE_OK) return rc;
    CK(cudaEventRecord(L->ev_join, L->side_stream));
    L->side_pending = true;
  }
  if (rc != MOE_OK) return rc;
  if (owner_dots) {
    PullDotsArgs pd{};
    pd.rows = ep_rows(L, 2, L->dy_perm); pd.aux_off = aux_off; pd.slot_pos = L->slot_pos; pd.grad_gates = L->grad_gates;
    pd.slots = tokens * L->k;
    Span sp(L, 5, st); CK(launch_pull_dots(pd, st));
  }

  if (L->shared && tokens > 0) {
    Groups S{L->shared_meta, L->shared_meta + 2, 1, L->shared_rows_cap, tokens};
    ExpertIO sio{};
    sio.x = L->last_x; sio.gu = L->gu_s; sio.h = L->h_s; sio.y = L->y_s; sio.dy = gy; sio.dgu = L->dgu_s;
    sio.dx = L->dx_s; sio.dh = L->dh_s; sio.w_gu = L->off_sgu; sio.w_d = L->off_sd;
    rc = experts_backward(L, S, sio, st, false);
    if (rc != MOE_OK) return rc;
  }

  if (mode != 3 && (rc = router_backward()) != MOE_OK) return rc;
  if (mode == 3) {
    CK(cudaEventRecord(L->ev_fork, st));
    CK(cudaStreamWaitEvent(L->side_stream, L->ev_fork, 0));
    if ((rc = experts_backward(L, G, io, L->side_stream, true, 6)) != MOE_OK) return rc;
    if ((rc = router_weight_gradient(L->side_stream)) != MOE_OK) return rc;
    CK(cudaEventRecord(L->ev_join, L->side_stream));
    L->side_pending = true;
  }

  // Everything the input gradient needs exists now.
  UnpermuteArgs ua{};
  ua.grad_x_perm = ep ? ep_rows(L, 3, L->dx_perm) : local_rows(L->dx_perm); ua.shared = L->shared ? L->dx_s : nullptr;
  ua.extra = L->tc_router ? L->dx_r : nullptr; ua.grad_logits = L->tc_router ? nullptr : L->grad_logits;
  ua.w_router = L->w + L->off_router; ua.expert_of = L->expert_of; ua.slot_pos = L->slot_pos; ua.grad_x = gx;
  ua.tokens = tokens; ua.d = L->d; ua.E = L->E; ua.k = L->k; ua.accumulate = accumulate;
  if (mode == 1) {
    // The gate|up weight gradient goes first so that its persistent CTAs are resident on every SM;
    // the un-permute (HBM / NVLink bound) follows on the side stream with two CTAs per SM, which fit
    // in the registers and shared memory the GEMM leaves free.  The other order lets the un-permute's
    // thousands of small CTAs fill the SMs and the GEMM waits for all of them.
    CK(cudaEventRecord(L->ev_fork, st));
    rc = ep ? ep_backward_experts(L, st, 4) : experts_backward(L, G, io, st, true, 4);
    if (rc != MOE_OK) return rc;
    CK(cudaStreamWaitEvent(L->side_stream, L->ev_fork, 0));
    CK(launch_unpermute(ua, L->act, L->side_stream, 2 * L->sm_count));
    CK(cudaEventRecord(L->ev_join, L->side_stream));
  } else {
    { Span sp(L, 11, st); CK(launch_unpermute(ua, L->act, st)); }
    if (mode < 2) {
      rc = ep ? ep_backward_experts(L, st, 4) : experts_backward(L, G, io, st, true, 4);
      if (rc != MOE_OK) return rc;
    }
  }

  if (mode != 3 && (rc = router_weight_gradient(st)) != MOE_OK) return rc;
  if (ep) {
    Span sp(L, 12, st);
    rc = ep_allreduce_replicated(L, st);
    if (rc != MOE_OK) return rc;
    if (ep_accum) {
      add_inplace_kernel<<<(unsigned)((rep_router + 255) / 256), 256, 0, st>>>(L->g + L->off_router, L->g_rep_save, rep_router); count_launch();
      if (rep_shared > 0) {
        add_inplace_kernel<<<(unsigned)((rep_shared + 255) / 256), 256, 0, st>>>(L->g + L->off_sgu, L->g_rep_save + rep_router, rep_shared); count_launch();
      }
    }
  }
  L->rep_overwrite = false;
  if (mode == 1) CK(cudaStreamWaitEvent(st, L->ev_join, 0));
  CK(cudaGetLastError());
  L->grad_valid = true;
  return MOE_OK;
}

int ensure_host_buffers(moe_layer* L) {
  if (L->own_stream) return MOE_OK;
  const long long n = (long long)L->max_tokens * L->d;
  DA(L->host_stage_f32, n * 4, false);
  DA(L->host_x, n * L->esz, false);
  DA(L->host_y, n * L->esz, false);
  if (L->training) DA(L->host_gx, n * L->esz, false);
  DA(L->host_valid, L->max_tokens, false);
  CK(cudaStreamCreateWithFlags(&L->own_stream, cudaStreamNonBlocking));
  return MOE_OK;
}

}  // namespace

extern "C" {

int32_t moe_config_validate(const moe_config_t* cfg, char* message, int32_t message_len) {
  if (message && message_len > 0) message[0] = 0;
  return validate(cfg, message, message_len);
}

int64_t moe_workspace_bytes(const moe_config_t* cfg) {
  if (validate(cfg, nullptr, 0) != MOE_OK) return -1;
  return workspace_bytes(cfg);
}

int32_t moe_create(const moe_config_t* cfg, moe_layer_t** out) {
  if (!out) return MOE_INVALID_INPUT;
  *out = nullptr;
  char msg[256];
  if (validate(cfg, msg, sizeof(msg)) != MOE_OK) return MOE_INVALID_CONFIG;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0 || cfg->device < 0 || cfg->device >= ndev) {
    cudaGetLastError();
    return MOE_UNSUPPORTED;   // no usable device: fail closed, never a host fallback
  }
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, cfg->device) != cudaSuccess) return MOE_CUDA_ERROR;
  if (prop.major != 10) return MOE_UNSUPPORTED;   // built for sm_100a only
  moe_layer* L = new (std::nothrow) moe_layer;
  if (!L) return MOE_OUT_OF_MEMORY;
  *out = L;   // returned even on failure so the caller can read moe_last_error, then destroy
  L->device = cfg->device;
  L->sm_count = prop.multiProcessorCount;
  CK(cudaSetDevice(cfg->device));

  const Sizes s = sizes_of(cfg);
  L->d = cfg->d_model; L->E = cfg->num_experts; L->k = cfg->experts_per_token; L->F = cfg->d_ff; L->F_pad = s.F_pad;
  L->E_local = s.E_local; L->ep_rank = cfg->ep_rank; L->ep_size = cfg->ep_size; L->e0 = cfg->ep_rank * s.E_local;
  L->shared = cfg->shared_expert != 0; L->training = cfg->training != 0;
  L->aux_w = cfg->aux_loss_weight; L->z_w = cfg->router_z_loss_weight;
  L->precision = cfg->precision; L->act = cfg->precision == MOE_PRECISION_F32 ? PREC_F32 : PREC_BF16;
  L->esz = L->act == PREC_F32 ? 4 : 2;
  L->max_tokens = cfg->max_tokens; L->rows_cap = s.rows_cap; L->shared_rows_cap = s.shared_rows_cap;
  L->off_router = s.off_router; L->off_gu = s.off_gu; L->off_d = s.off_d; L->off_sgu = s.off_sgu; L->off_sd = s.off_sd;
  L->n_params = s.n_params;

  const long long T = L->max_tokens, d = L->d, E = L->E, k = L->k, Fp = L->F_pad;
  L->tc_router = L->precision != MOE_PRECISION_F32 && L->E % 8 == 0;
  if (L->precision == MOE_PRECISION_Q8) {
    DA(L->w, (long long)E * d * 4, true);   // router only
    DA(L->wb, (long long)E * d * 2, true);  // its bf16 copy for the tensor-core logits product
    const long long G = E + 1;   // the shared expert is stored as group E
    DA(L->q_gu, G * 2 * Fp * d, true); DA(L->s_gu, G * 2 * Fp * 4, true);
    DA(L->q_d, G * d * Fp, true); DA(L->s_d, G * d * 4, true);
    // int8 zero in the stored form (sign bit flipped): padding rows and columns stay zero weights
    CK(cudaMemset(L->q_gu, 0x80, (size_t)(G * 2 * Fp * d)));
    CK(cudaMemset(L->q_d, 0x80, (size_t)(G * d * Fp)));
  } else {
    DA(L->w, L->n_params * 4, true);
    L->wc = L->w;
    if (L->training) {
      DA(L->g, L->n_params * 4, true);
      DA(L->m, L->n_params * 4, true);
      DA(L->v, L->n_params * 4, true);
    }
    if (L->act == PREC_BF16) DA(L->wb, L->n_params * 2, true);
  }
  {
    // f32 handle, shapes that fit the tensor-core tiles: forward expert products on tcgen05 (MOE_B200_F32_TC=0: FMA kernels)
    static const bool f32_tc = [] { const char* e = getenv("MOE_B200_F32_TC"); return !(e && *e == '0'); }();
    // (reductions of at most 2048: the tensor core adds into its accumulator with truncation, a bias of about
    // 2^-25 per 16 reduction elements, which stays below the 1e-5 bar up to there)
    if (f32_tc && L->act == PREC_F32 && L->precision == MOE_PRECISION_F32 && d % 32 == 0 && d <= 2048 && Fp <= 2048 &&
        L->ep_size == 1 && L->E_local <= 256) {
      DA(L->w3, 6 * L->n_params * 2, true);
      const long long rows = std::max<long long>(L->rows_cap, L->shared_rows_cap);
      DA(L->xa3, rows * 6 * d * 2, true);
      DA(L->ha3, rows * 6 * Fp * 2, true);
    }
  }
  L->stage_elems = std::max((long long)E * d, 2ll * Fp * d);
  DA(L->stage, L->stage_elems * 4 * 2, false);

  const int nb = ceil_div((int)T, ROUTER_ROWS);
  DA(L->logits, T * E * 4, false); DA(L->probs, T * E * 4, false); DA(L->lse, T * 4, false);
  DA(L->gates, T * k * 4, false); DA(L->expert_of, T * k * 4, false);
  DA(L->partial, (long long)nb * (E + 2) * 4, false); DA(L->hist, (long long)nb * E * 4, false);
  const int halves = L->training && overlap_mode() == 2 ? 2 : 1;   // see moe_layer::parity
  for (int h = 0; h < 2; ++h) {
    if (h < halves) DA(L->meta_block2[h], (4 * (E + 1) + 8) * 4, true);
    else L->meta_block2[h] = L->meta_block2[0];
  }
  DA(L->stats, (E + 2) * 4, true); DA(L->losses, 2 * 4, true);
  DA(L->slot_pos, T * k * 4, false); DA(L->token_of, T * k * 4, false); DA(L->slot_of, T * k * 4, false);
  DA(L->row_token, (long long)L->rows_cap * 4, false); DA(L->row_gate, (long long)L->rows_cap * 4, false);
  DA(L->shared_meta_table, (T + 1) * 16, false); DA(L->error_flag, 4, true); DA(L->route_done, 4, true);
  shared_meta_table_kernel<<<(unsigned)((T + 256) / 256), 256>>>(L->shared_meta_table, (int)T);
  CK(cudaGetLastError());
  L->shared_meta = L->shared_meta_table;

  const bool ep = L->ep_size > 1;
  if (ep) {
    L->ep_capacity = cfg->ep_capacity_factor > 0.f ? cfg->ep_capacity_factor : 1.25f;
    const long long want = (long long)std::ceil((double)L->ep_capacity * (double)T * (double)k) + (long long)L->E_local * (GROUP_ALIGN - 1);
    L->rows_cap_l = (int)std::min<long long>(round_up((int)std::min<long long>(want, 1ll << 30), GROUP_ALIGN),
                                             (long long)round_up((int)(T * k) * L->ep_size + L->E_local * (GROUP_ALIGN - 1), GROUP_ALIGN));
    const int El = L->E_local, N = L->ep_size, words = 2 * (int)E + 2;
    DA(L->ep_pack, words * 4, true); DA(L->ep_gathered, (long long)N * words * 4, true);
    DA(L->ext_stats, (E + 2) * 4, true); DA(L->ext_counts, E * 4, true);
    for (int h = 0; h < 2; ++h) {
      if (h < halves) DA(L->local_meta2[h], 3 * (El + 1) * 4, true);
      else L->local_meta2[h] = L->local_meta2[0];
    }
    DA(L->dest_base, E * 4, true); DA(L->barrier_word, 4, true);
    if (L->training) DA(L->g_rep_save, ((long long)E * d + (L->shared ? L->n_params - L->off_sgu : 0)) * 4, true);
    CK(cudaMallocHost((void**)&L->dest_base_host, (size_t)E * 4));
    if (L->ep_size > MAX_RANKS) return fail(L, MOE_INVALID_CONFIG, "at most %d expert-parallel ranks", MAX_RANKS);
    CK(cudaMallocHost((void**)&L->ep_gathered_host, (size_t)N * words * 4));
    CK(cudaMallocHost((void**)&L->local_meta_host, (size_t)3 * (El + 1) * 4));
    L->cnt_all.assign((size_t)N * E, 0); L->send_off.assign(E + 1, 0); L->recv_row.assign((size_t)N * El, 0);
  }
  const long long rc = L->rows_cap, sc = L->shared_rows_cap, es = (long long)L->esz;
  const long long rl = ep ? L->rows_cap_l : rc;   // rows of the buffers the expert GEMMs work on
  DA(L->x_perm2[0], rc * d * es, true);
  if (halves == 2 && !ep) DA(L->x_perm2[1], rc * d * es, true); else L->x_perm2[1] = L->x_perm2[0];
  DA(L->gu, rl * 2 * Fp * es, true); DA(L->h, rl * Fp * es, true);
  if (ep) {
    DA(L->x_recv2[0], halves * rl * d * es, true);   // one allocation: it is exported to the peers as a whole
    L->x_recv2[1] = (char*)L->x_recv2[0] + (halves - 1) * rl * d * es;
    DA(L->y_recv, rl * d * es, true);
  }
  select_parity(L, 0);
  DA(L->y_perm, rc * d * es, true);
  if (L->shared) { DA(L->gu_s, sc * 2 * Fp * es, true); DA(L->h_s, sc * Fp * es, true); DA(L->y_s, sc * d * es, true); }
  if (L->training) {
    DA(L->dy_perm, rc * d * es, true); DA(L->dgu, rl * 2 * Fp * es, true); DA(L->dx_perm, rc * d * es, true);
    if (L->act == PREC_F32) DA(L->dh, rl * Fp * es, true);
    // behind the gradient rows: the gates pushed with them and the dots computed from them (peer transport)
    if (ep) { DA(L->dy_recv, rl * d * es + rl * 12, true); DA(L->dx_recv, rl * d * es, true); }
    if (L->shared) {
      DA(L->dgu_s, sc * 2 * Fp * es, true); DA(L->dx_s, sc * d * es, true);
      if (L->act == PREC_F32) DA(L->dh_s, sc * Fp * es, true);
    }
    DA(L->grad_gates, T * k * 4, true); DA(L->grad_logits, T * E * 4, true);
    if (L->tc_router) { DA(L->gl_bf16, T * E * 2, true); DA(L->dx_r, sc * d * es, true); }
    if (L->shared && L->act == PREC_BF16) {
      const int tiles = std::min(ceil_div(2 * (int)Fp, tc::BM) * ceil_div((int)d, tc::BN), ceil_div((int)d, tc::BM) * ceil_div((int)Fp, tc::BN));
      if (tiles < L->sm_count) {
        const int splits = std::min(16, std::max(1, L->sm_count / std::max(1, tiles)));
        L->sh_scratch_elems = (long long)splits * 2 * Fp * d;
        DA(L->sh_scratch, L->sh_scratch_elems * 4, false);
        DA(L->sh_meta, 32 * 4, true);
      }
    }
    L->rw_splits = (int)std::min<long long>(64, std::max<long long>(1, T / 256));
    DA(L->rw_scratch, (long long)L->rw_splits * E * d * 4, false);
    DA(L->rw_meta, 130 * 4, true);
  }
  CK(cudaStreamCreateWithFlags(&L->side_stream, cudaStreamNonBlocking));
  CK(cudaEventCreateWithFlags(&L->ev_fork, cudaEventDisableTiming));
  CK(cudaEventCreateWithFlags(&L->ev_join, cudaEventDisableTiming));
  CK(cudaDeviceSynchronize());
  return MOE_OK;
}

void moe_destroy(moe_layer_t* L) {
  if (!L) return;
  cudaSetDevice(L->device);
  cudaDeviceSynchronize();
  if (L->comm) ncclCommDestroy((ncclComm_t)L->comm);
  if (L->ep_gathered_host) cudaFreeHost(L->ep_gathered_host);
  if (L->local_meta_host) cudaFreeHost(L->local_meta_host);
  if (L->dest_base_host) cudaFreeHost(L->dest_base_host);
  if (L->peer_ready)
    for (int b = 0; b < 4; ++b)
      for (int r = 0; r < L->ep_size; ++r)
        if (r != L->ep_rank && L->peer_base[b][r]) cudaIpcCloseMemHandle(L->peer_base[b][r]);
  for (void* p : L->allocations) cudaFree(p);
  for (auto& sp : L->prof_spans) { cudaEventDestroy(sp.begin); cudaEventDestroy(sp.end); }
  for (auto ev : L->prof_pool) cudaEventDestroy(ev);
  if (L->own_stream) cudaStreamDestroy(L->own_stream);
  if (L->side_stream) cudaStreamDestroy(L->side_stream);
  if (L->ev_fork) cudaEventDestroy(L->ev_fork);
  if (L->ev_join) cudaEventDestroy(L->ev_join);
  delete L;
}

const char* moe_last_error(const moe_layer_t* L) { return L ? L->err.c_str() : "null handle"; }

int32_t moe_clear_error(moe_layer_t* L) {
  if (!L) return MOE_INVALID_INPUT;
  L->status = MOE_OK;
  L->err.clear();
  cudaSetDevice(L->device);
  cudaGetLastError();
  if (L->error_flag) cudaMemset(L->error_flag, 0, sizeof(int));
  return MOE_OK;
}

int32_t moe_set_weight_f32(moe_layer_t* L, int32_t which, int32_t expert, const float* src, int32_t rows, int32_t cols) {
  ENTER(L);
  if (L->precision == MOE_PRECISION_Q8 && which != MOE_W_ROUTER) { L->err = "InvalidInput: a quantized layer takes int8 expert weights"; return MOE_INVALID_INPUT; }
  WeightSlot s;
  int rc = slot_of_weight(L, which, expert, &s);
  if (rc != MOE_OK) { L->status = MOE_OK; return rc; }
  if (rows != s.rows || cols != s.cols) { L->err = "InvalidInput: weight shape mismatch"; return MOE_INVALID_INPUT; }
  if (!src) { L->err = "InvalidInput: null weight pointer"; return MOE_INVALID_INPUT; }
  const long long n = (long long)rows * cols;
  const float* dev_src = src;
  // the pack kernel runs on the default stream: wait for passes or optimizer steps still in flight on the
  // caller's (possibly non-blocking) streams before the arenas are rewritten under them
  CK(cudaDeviceSynchronize());
  if (!is_device_pointer(src)) {
    CK(cudaMemcpy(L->stage, src, (size_t)n * 4, cudaMemcpyHostToDevice));
    dev_src = L->stage;
  }
  pack_kernel<<<(unsigned)((n + 255) / 256), 256>>>(dev_src, L->w + s.offset, L->wb ? L->wb + s.offset : nullptr, rows, cols, s.ld, s.kind); count_launch();
  if (L->lora_rank > 0) L->lora_dirty = true;
  L->w3_dirty = true;
  CK(cudaGetLastError());
  CK(cudaDeviceSynchronize());
  return MOE_OK;
}

static int read_arena(moe_layer* L, const float* arena, int which, int expert, float* dst, int rows, int cols, bool zero) {
  WeightSlot s;
  int rc = slot_of_weight(L, which, expert, &s);
  if (rc != MOE_OK) { L->status = MOE_OK; return rc; }
  if (rows != s.rows || cols != s.cols) { L->err = "InvalidInput: weight shape mismatch"; return MOE_INVALID_INPUT; }
  if (!arena) { L->err = "InvalidConfig: the handle holds no such buffer (training = 0 or quantized)"; return MOE_INVALID_CONFIG; }
  const long long n = (long long)rows * cols;
  if (!dst) { L->err = "InvalidInput: null destination pointer"; return MOE_INVALID_INPUT; }
  const bool dev = is_device_pointer(dst);
  float* out = dev ? dst : L->stage;
  if (L->last_stream) WAIT(L, L->last_stream, false);   // a backward pass (with its all-reduce) may still be running
  if (L->side_pending) { CK(cudaStreamSynchronize(L->side_stream)); L->side_pending = false; }   // deferred weight gradients
  CK(cudaDeviceSynchronize());   // the unpack kernel runs on the default stream: see what every stream has written
  unpack_kernel<<<(unsigned)((n + 255) / 256), 256>>>(arena + s.offset, out, rows, cols, s.ld, s.kind, zero ? 1 : 0); count_launch();
  CK(cudaGetLastError());
  if (!dev) CK(cudaMemcpy(dst, L->stage, (size_t)n * 4, cudaMemcpyDeviceToHost));
  else CK(cudaDeviceSynchronize());
  return MOE_OK;
}

int32_t moe_get_weight_f32(moe_layer_t* L, int32_t which, int32_t expert, float* dst, int32_t rows, int32_t cols) {
  ENTER(L);
  if (L->precision == MOE_PRECISION_Q8 && which != MOE_W_ROUTER) { L->err = "InvalidConfig: quantized weights are not readable as f32"; return MOE_INVALID_CONFIG; }
  return read_arena(L, L->w, which, expert, dst, rows, cols, false);
}
int32_t moe_get_grad_f32(moe_layer_t* L, int32_t which, int32_t expert, float* dst, int32_t rows, int32_t cols) {
  ENTER(L);
  return read_arena(L, L->g, which, expert, dst, rows, cols, !L->grad_valid);
}
int32_t moe_get_moments_f32(moe_layer_t* L, int32_t which, int32_t expert, float* m, float* v, int32_t rows, int32_t cols) {
  ENTER(L);
  int rc = read_arena(L, L->m, which, expert, m, rows, cols, false);
  if (rc != MOE_OK) return rc;
  return read_arena(L, L->v, which, expert, v, rows, cols, false);
}
int32_t moe_set_moments_f32(moe_layer_t* L, int32_t which, int32_t expert, const float* m, const float* v, int32_t rows, int32_t cols) {
  ENTER(L);
  if (!L->m) { L->err = "InvalidConfig: the handle holds no optimizer state"; return MOE_INVALID_CONFIG; }
  WeightSlot s;
  int rc = slot_of_weight(L, which, expert, &s);
  if (rc != MOE_OK) { L->status = MOE_OK; return rc; }
  if (rows != s.rows || cols != s.cols) { L->err = "InvalidInput: weight shape mismatch"; return MOE_INVALID_INPUT; }
  if (!m || !v) { L->err = "InvalidInput: null moment pointer"; return MOE_INVALID_INPUT; }
  const long long n = (long long)rows * cols;
  CK(cudaDeviceSynchronize());   // an optimizer step may still be running on a non-blocking stream
  const float* srcs[2] = {m, v};
  float* dsts[2] = {L->m, L->v};
  for (int i = 0; i < 2; ++i) {
    const float* dev_src = srcs[i];
    if (!is_device_pointer(srcs[i])) {
      CK(cudaMemcpy(L->stage, srcs[i], (size_t)n * 4, cudaMemcpyHostToDevice));
      dev_src = L->stage;
    }
    pack_kernel<<<(unsigned)((n + 255) / 256), 256>>>(dev_src, dsts[i] + s.offset, nullptr, rows, cols, s.ld, s.kind); count_launch();
    CK(cudaDeviceSynchronize());
  }
  return MOE_OK;
}

int32_t moe_set_weight_q8(moe_layer_t* L, int32_t which, int32_t expert, const int8_t* q, const float* scale, int32_t rows, int32_t cols) {
  ENTER(L);
  if (L->precision != MOE_PRECISION_Q8) { L->err = "InvalidConfig: int8 weights need a MOE_PRECISION_Q8 handle"; return MOE_INVALID_CONFIG; }
  if (!q || !scale) { L->err = "InvalidInput: null weight pointer"; return MOE_INVALID_INPUT; }
  const int d = L->d, F = L->F, Fp = L->F_pad;
  int group = expert, kind = 0, ld = d;
  bool down = false;
  switch (which) {
    case MOE_W_GATE: kind = 1; break;
    case MOE_W_UP: kind = 2; break;
    case MOE_W_DOWN: down = true; ld = Fp; break;
    case MOE_W_SHARED_GATE: kind = 1; group = L->E; break;
    case MOE_W_SHARED_UP: kind = 2; group = L->E; break;
    case MOE_W_SHARED_DOWN: down = true; ld = Fp; group = L->E; break;
    case MOE_W_ROUTER: {
      // TransformerLm::quantize also quantizes the router (transformer.rs:899-910).  Its product is tiny, so the
      // int8 grid is kept by value: the router's weights become q * scale (quantized.rs:17-24) and run on the
      // ordinary router path; the logits are those of the reference's Quantized::matmul up to summation order.
      if (rows != L->E || cols != L->d) { L->err = "InvalidInput: weight shape mismatch"; return MOE_INVALID_INPUT; }
      std::vector<int8_t> hq((size_t)rows * cols);
      std::vector<float> hs((size_t)rows), hw((size_t)rows * cols);
      CK(cudaMemcpy(hq.data(), q, hq.size(), cudaMemcpyDefault));
      CK(cudaMemcpy(hs.data(), scale, hs.size() * 4, cudaMemcpyDefault));
      for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c) hw[(size_t)r * cols + c] = (float)hq[(size_t)r * cols + c] * hs[r];
      return moe_set_weight_f32(L, MOE_W_ROUTER, 0, hw.data(), rows, cols);
    }
    default: L->err = "InvalidInput: unknown weight id"; return MOE_INVALID_INPUT;
  }
  if (group < 0 || group > L->E || (group == L->E && !L->shared)) { L->err = "InvalidInput: no such expert"; return MOE_INVALID_INPUT; }
  if ((!down && (rows != F || cols != d)) || (down && (rows != d || cols != F))) { L->err = "InvalidInput: weight shape mismatch"; return MOE_INVALID_INPUT; }
  const long long n = (long long)rows * cols;
  int8_t* qs = reinterpret_cast<int8_t*>(L->stage);
  float* ss = L->stage + L->stage_elems;   // second half of the staging buffer
  CK(cudaDeviceSynchronize());   // a decode step may still be reading the weights on a non-blocking stream
  CK(cudaMemcpy(qs, q, (size_t)n, is_device_pointer(q) ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice));
  CK(cudaMemcpy(ss, scale, (size_t)rows * 4, is_device_pointer(scale) ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice));
  int8_t* dst = down ? L->q_d + (long long)group * d * Fp : L->q_gu + (long long)group * 2 * Fp * d;
  float* sdst = down ? L->s_d + (long long)group * d : L->s_gu + (long long)group * 2 * Fp;
  pack_q8_kernel<<<(unsigned)((n + 255) / 256), 256>>>(qs, ss, dst, sdst, rows, cols, ld, kind);
  CK(cudaGetLastError());
  CK(cudaDeviceSynchronize());
  return MOE_OK;
}

int32_t moe_forward(moe_layer_t* L, const void* x, int32_t tokens, int32_t cols, const uint8_t* valid, void* y,
                    int32_t accumulate, int32_t save, void* stream) {
  ENTER(L);
  // the decode pass of a quantized layer is a chain of six short kernels: let each start under its predecessor's tail
  static const bool pdl = [] { const char* e = getenv("MOE_B200_PDL"); return !(e && *e == '0'); }();
  struct Scope { bool on; Scope(bool v) : on(v) { if (on) g_pdl_scope = true; } ~Scope() { if (on) g_pdl_scope = false; } }
      scope(pdl && L->precision == MOE_PRECISION_Q8);
  return forward_impl(L, x, nullptr, tokens, cols, valid, y, accumulate, save, (cudaStream_t)stream);
}

int32_t moe_forward_from_logits(moe_layer_t* L, const void* x, const float* logits, int32_t tokens, int32_t cols,
                                const uint8_t* valid, void* y, int32_t accumulate, int32_t save, void* stream) {
  ENTER(L);
  if (!logits) { L->err = "InvalidInput: null logits"; return MOE_INVALID_INPUT; }
  return forward_impl(L, x, logits, tokens, cols, valid, y, accumulate, save, (cudaStream_t)stream);
}

int32_t moe_backward(moe_layer_t* L, const void* gy, void* gx, int32_t accumulate, void* stream) {
  ENTER(L);
  return backward_impl(L, gy, gx, accumulate, (cudaStream_t)stream);
}

int32_t moe_zero_grad(moe_layer_t* L, void*) {
  ENTER(L);
  L->grad_valid = false;   // a flag, as DeviceParam::zero_grad (gpu_transformer.rs:634-636)
  return MOE_OK;
}

// Param::step over every weight of the layer (param.rs:547-617): kind 0 Adam, 1 Sgd, 2 Lion.  `a` carries the
// hyper-parameters; the pointers are filled here.
static int step_common(moe_layer* L, int kind, AdamArgs a, cudaStream_t st) {
  if (!L->training) { L->err = "InvalidConfig: the handle was created with training = 0"; return MOE_INVALID_CONFIG; }
  { const int jr = join_side(L, st); if (jr != MOE_OK) return jr; }
  if (L->lora_rank > 0) {
    // base weights are frozen (the reference's add_lora): only the adapters move
    const int pr = lora_project_grads(L, st);
    if (pr != MOE_OK) return pr;
    CK(cudaMemsetAsync(L->g, 0, (size_t)L->n_params * 4, st));
    a.w = L->la; a.g = L->lg; a.m = L->lm; a.v = L->lv; a.w_bf16 = nullptr; a.n = L->lora_n;
    L->lora_dirty = true;
  } else {
    if (!L->grad_valid) CK(cudaMemsetAsync(L->g, 0, (size_t)L->n_params * 4, st));
    a.w = L->w; a.g = L->g; a.m = L->m; a.v = L->v; a.w_bf16 = L->wb; a.n = L->n_params;
  }
  { Span sp(L, 15, st); CK(kind == 0 ? launch_adam(a, st) : kind == 1 ? launch_sgd(a, st) : launch_lion(a, st)); }
  L->w3_dirty = true;
  L->grad_valid = false;   // the kernel cleared the gradients
  return MOE_OK;
}

int32_t moe_step_adam(moe_layer_t* L, float lr, float b1, float b2, float eps, float wd, int32_t step, float scale, void* stream) {
  ENTER(L);
  AdamArgs a{};
  a.lr = lr; a.beta1 = b1; a.beta2 = b2; a.eps = eps; a.wd = wd; a.scale = scale;
  a.c1 = 1.0f - powf(b1, (float)step);
  a.c2 = 1.0f - powf(b2, (float)step);
  return step_common(L, 0, a, (cudaStream_t)stream);
}

int32_t moe_step_sgd(moe_layer_t* L, float lr, float scale, void* stream) {
  ENTER(L);
  AdamArgs a{};
  a.lr = lr; a.scale = scale;
  return step_common(L, 1, a, (cudaStream_t)stream);
}

int32_t moe_step_lion(moe_layer_t* L, float lr, float b1, float b2, float wd, float scale, void* stream) {
  ENTER(L);
  AdamArgs a{};
  a.lr = lr; a.beta1 = b1; a.beta2 = b2; a.wd = wd; a.scale = scale;
  return step_common(L, 2, a, (cudaStream_t)stream);
}

int32_t moe_forward_host(moe_layer_t* L, const float* x, int32_t tokens, int32_t cols, const uint8_t* valid, float* y, int32_t save) {
  ENTER(L);
  if (cols != L->d || tokens < 0 || tokens > L->max_tokens || !x || !y) {
    L->err = "InvalidInput: expected " + std::to_string(L->d) + " columns and at most " + std::to_string(L->max_tokens) + " tokens";
    return MOE_INVALID_INPUT;
  }
  int rc = ensure_host_buffers(L);
  if (rc != MOE_OK) return rc;
  cudaStream_t st = L->own_stream;
  const long long n = (long long)tokens * L->d;
  if (tokens > 0) {
    // straight from the caller's buffer: asynchronous when it is pinned, staged by the driver otherwise
    if (L->act == PREC_F32) {
      CK(cudaMemcpyAsync(L->host_x, x, (size_t)n * 4, cudaMemcpyHostToDevice, st));
    } else {
      CK(cudaMemcpyAsync(L->host_stage_f32, x, (size_t)n * 4, cudaMemcpyHostToDevice, st));
      CK(launch_cast_f32_to_bf16(L->host_stage_f32, (bf16*)L->host_x, n, st));
    }
    if (valid) CK(cudaMemcpyAsync(L->host_valid, valid, (size_t)tokens, cudaMemcpyHostToDevice, st));
  }
  rc = forward_impl(L, L->host_x, nullptr, tokens, cols, valid ? L->host_valid : nullptr, L->host_y, 0, save, st);
  if (rc != MOE_OK) return rc;
  if (tokens > 0) {
    if (L->act == PREC_F32) {
      CK(cudaMemcpyAsync(y, L->host_y, (size_t)n * 4, cudaMemcpyDeviceToHost, st));
    } else {
      CK(launch_cast_bf16_to_f32((const bf16*)L->host_y, L->host_stage_f32, n, st));
      CK(cudaMemcpyAsync(y, L->host_stage_f32, (size_t)n * 4, cudaMemcpyDeviceToHost, st));
    }
  }
  WAIT(L, st, false);
  return check_flag(L);
}

int32_t moe_backward_host(moe_layer_t* L, const float* gy, float* gx) {
  ENTER(L);
  if (!gy || !gx) { L->err = "InvalidInput: null gradient pointer"; return MOE_INVALID_INPUT; }
  if (!L->have_cache || L->last_x != L->host_x) { L->err = "InvalidInput: moe_backward_host needs a preceding moe_forward_host with save_for_backward"; return MOE_INVALID_INPUT; }
  cudaStream_t st = L->own_stream;
  const long long n = (long long)L->last_tokens * L->d;
  if (n > 0) {
    // host_y is free once the forward result has been copied out: reuse it for the upstream gradient
    if (L->act == PREC_F32) {
      CK(cudaMemcpyAsync(L->host_y, gy, (size_t)n * 4, cudaMemcpyHostToDevice, st));
    } else {
      CK(cudaMemcpyAsync(L->host_stage_f32, gy, (size_t)n * 4, cudaMemcpyHostToDevice, st));
      CK(launch_cast_f32_to_bf16(L->host_stage_f32, (bf16*)L->host_y, n, st));
    }
  }
  // The weight-gradient GEMMs feed nothing that leaves the device: they run on the side stream while
  // grad_x crosses PCIe, and both are waited for before the call returns.
  static const bool defer = [] { const char* e = getenv("MOE_B200_HOST_DEFER"); return !(e && *e == '0'); }();
  int rc = backward_impl(L, L->host_y, L->host_gx, 0, st, defer ? 3 : -1);
  if (rc != MOE_OK) return rc;
  if (n > 0) {
    if (L->act == PREC_F32) {
      CK(cudaMemcpyAsync(gx, L->host_gx, (size_t)n * 4, cudaMemcpyDeviceToHost, st));
    } else {
      CK(launch_cast_bf16_to_f32((const bf16*)L->host_gx, L->host_stage_f32, n, st));
      CK(cudaMemcpyAsync(gx, L->host_stage_f32, (size_t)n * 4, cudaMemcpyDeviceToHost, st));
    }
  }
  WAIT(L, st, false);
  if (L->side_pending) { CK(cudaStreamSynchronize(L->side_stream)); L->side_pending = false; }
  return check_flag(L);
}

int32_t moe_get_losses(moe_layer_t* L, float* aux, float* z) {
  ENTER(L);
  WAIT(L, L->last_stream, false);
  float v[2] = {0.f, 0.f};
  if (L->last_tokens > 0) CK(cudaMemcpy(v, L->losses, sizeof(v), cudaMemcpyDeviceToHost));
  if (aux) *aux = v[0];
  if (z) *z = v[1];
  return check_flag(L);
}

int32_t moe_get_routing(moe_layer_t* L, int32_t* expert_of, float* gates, int32_t* counts, int32_t* token_of,
                        int32_t* slot_of, int32_t* routed) {
  ENTER(L);
  WAIT(L, L->last_stream, false);
  const long long tk = (long long)L->last_tokens * L->k;
  int total[4] = {0, 0, 0, 0};
  if (L->last_tokens > 0) CK(cudaMemcpy(total, L->meta.total, sizeof(total), cudaMemcpyDeviceToHost));
  if (expert_of && tk > 0) CK(cudaMemcpy(expert_of, L->expert_of, (size_t)tk * 4, cudaMemcpyDeviceToHost));
  if (gates && tk > 0) CK(cudaMemcpy(gates, L->gates, (size_t)tk * 4, cudaMemcpyDeviceToHost));
  if (counts) {
    if (L->last_tokens > 0) CK(cudaMemcpy(counts, L->meta.counts, (size_t)L->E * 4, cudaMemcpyDeviceToHost));
    else memset(counts, 0, (size_t)L->E * 4);
  }
  if (token_of && total[0] > 0) CK(cudaMemcpy(token_of, L->token_of, (size_t)total[0] * 4, cudaMemcpyDeviceToHost));
  if (slot_of && total[0] > 0) CK(cudaMemcpy(slot_of, L->slot_of, (size_t)total[0] * 4, cudaMemcpyDeviceToHost));
  if (routed) *routed = total[0];
  return check_flag(L);
}

int32_t moe_get_router_cache(moe_layer_t* L, float* logits, float* probs, float* lse) {
  ENTER(L);
  WAIT(L, L->last_stream, false);
  const long long te = (long long)L->last_tokens * L->E;
  if (te > 0) {
    if (logits) CK(cudaMemcpy(logits, L->logits, (size_t)te * 4, cudaMemcpyDeviceToHost));
    if (probs) CK(cudaMemcpy(probs, L->probs, (size_t)te * 4, cudaMemcpyDeviceToHost));
    if (lse) CK(cudaMemcpy(lse, L->lse, (size_t)L->last_tokens * 4, cudaMemcpyDeviceToHost));
  }
  return MOE_OK;
}

int32_t moe_debug_profile(moe_layer_t* L, int32_t enable) {
  ENTER(L);
  L->prof_on = enable != 0;
  return MOE_OK;
}

int32_t moe_debug_profile_read(moe_layer_t* L, float* ms, int32_t* stages) {
  ENTER(L);
  CK(cudaDeviceSynchronize());
  for (int i = 0; i < MOE_PROFILE_CATEGORIES; ++i) { if (ms) ms[i] = 0.f; if (stages) stages[i] = 0; }
  for (auto& sp : L->prof_spans) {
    float t = 0.f;
    if (cudaEventElapsedTime(&t, sp.begin, sp.end) == cudaSuccess && sp.cat >= 0 && sp.cat < MOE_PROFILE_CATEGORIES) {
      if (ms) ms[sp.cat] += t;
      if (stages) stages[sp.cat] += 1;
    }
    L->prof_pool.push_back(sp.begin);
    L->prof_pool.push_back(sp.end);
  }
  cudaGetLastError();
  L->prof_spans.clear();
  return MOE_OK;
}

int32_t moe_ep_unique_id(void* out, int32_t len) {
  if (!out || len < (int32_t)sizeof(ncclUniqueId)) return MOE_INVALID_INPUT;
  ncclUniqueId id;
  if (ncclGetUniqueId(&id) != ncclSuccess) return MOE_COMM_ERROR;
  memcpy(out, &id, sizeof(id));
  return MOE_OK;
}

int32_t moe_ep_set_deadline_ms(moe_layer_t* L, int64_t milliseconds) {
  ENTER(L);
  if (milliseconds < 0) { L->err = "InvalidInput: negative deadline"; return MOE_INVALID_INPUT; }
  L->ep_deadline_ms = milliseconds;
  return MOE_OK;
}

int32_t moe_debug_deadline_wait(int32_t ready_after_ms, int32_t deadline_ms, int32_t* gave_up) {
  const auto t0 = std::chrono::steady_clock::now();
  const bool done = poll_until([&]() {
    return std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count() >= ready_after_ms;
  }, deadline_ms);
  if (gave_up) *gave_up = done ? 0 : 1;
  return done ? MOE_OK : MOE_TIMEOUT;
}

int32_t moe_ep_init(moe_layer_t* L, const void* unique_id, int32_t len) {
  ENTER(L);
  if (L->ep_size <= 1) { L->err = "InvalidConfig: the handle was created with ep_size = 1"; return MOE_INVALID_CONFIG; }
  if (!unique_id || len < (int32_t)sizeof(ncclUniqueId)) { L->err = "InvalidInput: bad unique id"; return MOE_INVALID_INPUT; }
  ncclUniqueId id;
  memcpy(&id, unique_id, sizeof(id));
  ncclComm_t comm = nullptr;
  NCK(ncclCommInitRank(&comm, L->ep_size, id, L->ep_rank));
  L->comm = comm;
  L->ep_ready = true;
  return MOE_OK;
}

int32_t moe_ep_export_buffers(moe_layer_t* L, void* out, int32_t len) {
  ENTER(L);
  if (L->ep_size <= 1 || !out || len < (int32_t)(4 * sizeof(cudaIpcMemHandle_t))) { L->err = "InvalidInput: bad export request"; return MOE_INVALID_INPUT; }
  void* bufs[4] = {L->x_recv2[0], L->y_recv, L->training ? L->dy_recv : L->x_recv, L->training ? L->dx_recv : L->y_recv};
  cudaIpcMemHandle_t* h = (cudaIpcMemHandle_t*)out;
  for (int b = 0; b < 4; ++b) CK(cudaIpcGetMemHandle(&h[b], bufs[b]));
  return MOE_OK;
}

int32_t moe_ep_import_buffers(moe_layer_t* L, int32_t rank, const void* handles, int32_t len) {
  ENTER(L);
  if (L->ep_size <= 1 || rank < 0 || rank >= L->ep_size || !handles || len < (int32_t)(4 * sizeof(cudaIpcMemHandle_t))) { L->err = "InvalidInput: bad import request"; return MOE_INVALID_INPUT; }
  if (rank == L->ep_rank) {
    L->peer_base[0][rank] = L->x_recv2[0]; L->peer_base[1][rank] = L->y_recv;
    L->peer_base[2][rank] = L->dy_recv; L->peer_base[3][rank] = L->dx_recv;
  } else {
    const cudaIpcMemHandle_t* h = (const cudaIpcMemHandle_t*)handles;
    for (int b = 0; b < 4; ++b) {
      if (!L->training && b >= 2) { L->peer_base[b][rank] = nullptr; continue; }
      CK(cudaIpcOpenMemHandle(&L->peer_base[b][rank], h[b], cudaIpcMemLazyEnablePeerAccess));
    }
  }
  bool all = true;
  for (int r = 0; r < L->ep_size; ++r) all = all && L->peer_base[0][r] != nullptr;
  L->peer_ready = all;
  return MOE_OK;
}

int32_t moe_ep_plan(const int32_t* counts_all, int32_t ranks, int32_t num_experts, int32_t rank, int32_t* send_off,
                    int32_t* recv_row, int32_t* local_row0, int32_t* local_tiles, int32_t* local_counts) {
  if (!counts_all || ranks <= 0 || num_experts <= 0 || num_experts % ranks != 0 || rank < 0 || rank >= ranks) return -1;
  return ep_plan(counts_all, ranks, num_experts, rank, send_off, recv_row, local_row0, local_tiles, local_counts);
}

static int lora_slot_checked(moe_layer* L, int which, int expert, LoraSlot* out) {
  if (L->lora_rank == 0) { L->err = "InvalidConfig: the layer has no adapters (moe_lora_attach)"; return MOE_INVALID_CONFIG; }
  const int idx = lora_slot_index(L, which, expert);
  if (idx < 0) { L->err = "InvalidInput: no adapter on that matrix (router, foreign or missing expert)"; return MOE_INVALID_INPUT; }
  CK(cudaMemcpy(out, (const LoraSlot*)L->lora_table + idx, sizeof(LoraSlot), cudaMemcpyDeviceToHost));
  return MOE_OK;
}

int32_t moe_lora_attach(moe_layer_t* L, int32_t rank, float alpha) {
  ENTER(L);
  return lora_attach(L, rank, alpha);
}

int32_t moe_lora_set(moe_layer_t* L, int32_t which, int32_t expert, const float* down, const float* up) {
  ENTER(L);
  LoraSlot s;
  int rc = lora_slot_checked(L, which, expert, &s);
  if (rc != MOE_OK) return rc;
  if (!down || !up) { L->err = "InvalidInput: null adapter pointer"; return MOE_INVALID_INPUT; }
  CK(cudaDeviceSynchronize());
  CK(cudaMemcpy(L->la + s.a_off, down, (size_t)L->lora_rank * s.cols * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(L->la + s.a_off + (long long)L->lora_rank * s.cols, up, (size_t)s.rows * L->lora_rank * 4, cudaMemcpyHostToDevice));
  L->lora_dirty = true;
  return MOE_OK;
}

int32_t moe_lora_get(moe_layer_t* L, int32_t which, int32_t expert, float* down, float* up) {
  ENTER(L);
  LoraSlot s;
  int rc = lora_slot_checked(L, which, expert, &s);
  if (rc != MOE_OK) return rc;
  CK(cudaDeviceSynchronize());
  if (down) CK(cudaMemcpy(down, L->la + s.a_off, (size_t)L->lora_rank * s.cols * 4, cudaMemcpyDeviceToHost));
  if (up) CK(cudaMemcpy(up, L->la + s.a_off + (long long)L->lora_rank * s.cols, (size_t)s.rows * L->lora_rank * 4, cudaMemcpyDeviceToHost));
  return MOE_OK;
}

int32_t moe_lora_get_grad(moe_layer_t* L, int32_t which, int32_t expert, float* grad_down, float* grad_up) {
  ENTER(L);
  LoraSlot s;
  int rc = lora_slot_checked(L, which, expert, &s);
  if (rc != MOE_OK) return rc;
  CK(cudaDeviceSynchronize());
  if ((rc = lora_project_grads(L, nullptr)) != MOE_OK) return rc;
  CK(cudaDeviceSynchronize());
  if (grad_down) CK(cudaMemcpy(grad_down, L->lg + s.a_off, (size_t)L->lora_rank * s.cols * 4, cudaMemcpyDeviceToHost));
  if (grad_up) CK(cudaMemcpy(grad_up, L->lg + s.a_off + (long long)L->lora_rank * s.cols, (size_t)s.rows * L->lora_rank * 4, cudaMemcpyDeviceToHost));
  return MOE_OK;
}

int32_t moe_lora_merge(moe_layer_t* L) {
  ENTER(L);
  if (L->lora_rank == 0) { L->err = "InvalidConfig: the layer has no adapters (moe_lora_attach)"; return MOE_INVALID_CONFIG; }
  CK(cudaDeviceSynchronize());
  // W <- W + scale * up * down in the master weights and the bf16 compute copy, then drop the adapters
  lora_fold_kernel<<<dim3(64, L->lora_slots), 256>>>((const LoraSlot*)L->lora_table, L->w, L->la, L->lora_rank, L->lora_scale, L->w, L->wb);
  count_launch();
  CK(cudaGetLastError());
  CK(cudaDeviceSynchronize());
  L->w3_dirty = true;
  L->lora_rank = 0;          // the arenas stay allocated until the handle is destroyed
  L->lora_dirty = false;
  L->wc = L->w;
  return MOE_OK;
}

int32_t moe_synchronize(moe_layer_t* L) {
  ENTER(L);
  if (L->last_stream) WAIT(L, L->last_stream, false);
  WAIT(L, nullptr, true);
  return check_flag(L);
}

}  // extern "C"
