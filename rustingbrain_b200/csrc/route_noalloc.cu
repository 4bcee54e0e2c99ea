// Routing without any allocation (moe_route_noalloc in include/moe_b200.h).
//
// Who needs this: a host runtime that took the whole device for its own arena before
// the first step and runs under a fixed memory budget (the reference checks such a budget
// before it uploads a model, transformer.rs:1265-1277), or a serving loop that must not
// hit the implicit device synchronisation of cudaMalloc between steps.  Such a caller
// cannot let a library allocate on its behalf, so it cannot create a layer handle (which
// owns a workspace).  This entry gives it the routing step alone - softmax, dropless
// top-k, renormalised gates, per-expert counts and the two auxiliary losses from given
// logits - with the caller's own buffers for every input and output.
//
// The step needs scratch memory between its two kernels (per-block partial sums and
// per-block expert histograms).  That scratch is the file-scope array below: a fixed part
// of the library image on every GPU that loads it, held until the process exits.
// Limits: tokens <= 16384 and num_experts <= 64.

#include "../../include/moe_b200.h"
#include "kernels.cuh"

#include <stdio.h>

namespace {

using namespace moe;

constexpr int NA_MAX_TOKENS = MOE_ROUTE_NOALLOC_MAX_TOKENS;
constexpr int NA_MAX_EXPERTS = MOE_ROUTE_NOALLOC_MAX_EXPERTS;
constexpr int NA_BLOCKS = NA_MAX_TOKENS / ROUTER_ROWS;
constexpr int NA_PARTIAL = NA_BLOCKS * (NA_MAX_EXPERTS + 2);   // floats
constexpr int NA_HIST = NA_BLOCKS * NA_MAX_EXPERTS;            // ints
constexpr int NA_META = 4 * (NA_MAX_EXPERTS + 1) + 8;          // offsets, pad_off, tile_start, total
constexpr int NA_STATS = NA_MAX_EXPERTS + 2;
constexpr int NA_WORDS = NA_PARTIAL + NA_HIST + NA_META + NA_STATS;

// ~134 KB per device.  In host code this name is only a handle for the runtime: the
// device address is fetched once per device with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned int g_route_scratch[NA_WORDS];

constexpr int NA_MAX_DEVICES = 64;
unsigned int* g_scratch_addr[NA_MAX_DEVICES] = {};

int na_fail(char* msg, int len, int status, const char* text) {
  if (msg && len > 0) snprintf(msg, len, "%s", text);
  return status;
}

}  // namespace

extern "C" int32_t moe_route_noalloc(const float* logits_dev, const uint8_t* valid_dev, int32_t tokens,
                                     int32_t num_experts, int32_t experts_per_token, float aux_loss_weight,
                                     float router_z_loss_weight, float* probabilities_dev, float* log_sum_exp_dev,
                                     int32_t* expert_of_dev, float* gates_dev, int32_t* counts_dev, float* losses_dev,
                                     void* stream, char* message, int32_t message_len) {
  if (message && message_len > 0) message[0] = 0;
  if (num_experts <= 0 || experts_per_token <= 0 || experts_per_token > num_experts)
    return na_fail(message, message_len, MOE_INVALID_CONFIG, "experts_per_token must be between 1 and num_experts");
  if (tokens < 0 || tokens > NA_MAX_TOKENS || num_experts > NA_MAX_EXPERTS || experts_per_token > MAX_TOPK)
    return na_fail(message, message_len, MOE_INVALID_INPUT,
                   "moe_route_noalloc handles at most 16384 tokens, 64 experts and 16 experts per token; "
                   "larger problems need a layer handle (moe_create), which owns a workspace");
  if (!logits_dev || !probabilities_dev || !log_sum_exp_dev || !expert_of_dev || !gates_dev || !counts_dev || !losses_dev)
    return na_fail(message, message_len, MOE_INVALID_INPUT, "null buffer");

  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NA_MAX_DEVICES)
    return na_fail(message, message_len, MOE_CUDA_ERROR, "no current CUDA device");
  if (!g_scratch_addr[dev]) {
    // first call on this device: resolve the device address of the static scratch array
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_route_scratch);
    if (e != cudaSuccess || !p)
      return na_fail(message, message_len, MOE_CUDA_ERROR, cudaGetErrorString(e));
    g_scratch_addr[dev] = static_cast<unsigned int*>(p);
  }
  unsigned int* base = g_scratch_addr[dev];
  float* partial = reinterpret_cast<float*>(base);
  int* hist = reinterpret_cast<int*>(base + NA_PARTIAL);
  int* meta_words = reinterpret_cast<int*>(base + NA_PARTIAL + NA_HIST);
  float* stats = reinterpret_cast<float*>(base + NA_PARTIAL + NA_HIST + NA_META);

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  RouterArgs ra{};
  ra.logits_in = logits_dev; ra.valid = valid_dev; ra.tokens = tokens; ra.d = 0; ra.E = num_experts;
  ra.k = experts_per_token; ra.probs = probabilities_dev; ra.lse = log_sum_exp_dev; ra.expert_of = expert_of_dev;
  ra.gates = gates_dev; ra.partial = partial; ra.hist = hist;
  RouteMeta meta{};
  meta.counts = counts_dev;
  meta.offsets = meta_words;
  meta.pad_off = meta_words + (NA_MAX_EXPERTS + 1);
  meta.tile_start = meta_words + 2 * (NA_MAX_EXPERTS + 1);
  meta.total = meta_words + 3 * (NA_MAX_EXPERTS + 1);
  cudaError_t e = launch_router(ra, PREC_F32, st);
  if (e == cudaSuccess) e = launch_finalize(ra, meta, aux_loss_weight, router_z_loss_weight, stats, losses_dev, 1, st);
  if (e != cudaSuccess) return na_fail(message, message_len, MOE_CUDA_ERROR, cudaGetErrorString(e));
  return MOE_OK;
}
