// Test hooks (include/moe_b200_debug.h).
#include "../../include/moe_b200_debug.h"
#include "gemm_tc.cuh"

using namespace moe;

namespace moe {
long long g_launch_count = 0;
thread_local bool g_pdl_scope = false;
}

extern "C" {

int32_t moe_debug_tc_gemm(int32_t variant, const void* a, const void* b, void* out0, void* out1, const void* aux,
                          const int32_t* group_row0, const int32_t* tile_start, int32_t n_groups, int32_t rows,
                          int32_t m, int32_t n, int32_t k, int32_t accumulate, int32_t* error_flag, void* stream) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 3;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 3;
  tc::GemmArgs g{};
  g.group_row0 = group_row0; g.tile_start = tile_start; g.n_groups = n_groups; g.error_flag = error_flag;
  g.N = n; g.K = k; g.M = m; g.out0 = out0; g.out1 = out1; g.aux = aux; g.accumulate = accumulate;
  cudaError_t e = cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  switch (variant) {
    case 0: g.ld0 = n; e = tc::gemm_rows_nt({a, rows, k, 1}, {b, n, k, n_groups}, g, tc::EPI_STORE, sms, st); break;
    case 1: g.ld0 = n / 2; g.ld1 = n; e = tc::gemm_rows_nt({a, rows, k, 1}, {b, n, k, n_groups}, g, tc::EPI_SWIGLU, sms, st); break;
    case 2: g.ld0 = n; e = tc::gemm_rows_nn({a, rows, k, 1}, {b, k, n, n_groups}, g, tc::EPI_STORE, sms, st); break;
    case 3: g.ld0 = 2 * n; g.ldaux = 2 * n; e = tc::gemm_rows_nn({a, rows, k, 1}, {b, k, n, n_groups}, g, tc::EPI_SWIGLU_BWD, sms, st); break;
    case 4: g.ld0 = n; g.group_stride0 = (long long)m * n; e = tc::gemm_rows_tn({a, rows, m, 1}, {b, rows, n, 1}, g, sms, st); break;
  }
  return e == cudaSuccess ? 0 : 3;
}

int32_t moe_debug_set_tc_pair(int32_t mode) {
  tc::set_tile_mode(mode);
  return 0;
}

int32_t moe_debug_starve_next_gemm(int64_t wait_limit_cycles) {
  tc::set_starve_next_launch(wait_limit_cycles);
  return 0;
}

int64_t moe_debug_launch_count(void) { return moe::g_launch_count; }

}  // extern "C"
