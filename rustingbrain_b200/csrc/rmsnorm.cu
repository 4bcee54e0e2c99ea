// RMSNorm forward and backward (the ABI of include/rmsnorm_b200.h; reference norm.rs:41-129).
//
// Both directions are bound by HBM: forward reads x and writes y once; backward reads x and grad_y,
// writes grad_x, and leaves one partial weight gradient per tile of 32 rows (the reference's
// ROWS_PER_TILE, norm.rs:14).  A second small kernel adds the tile partials to the gradient: the tiles are
// cut into 32 consecutive runs, each run is summed in tile order, and the run totals are added in run order.
// That order is fixed (scheduling cannot change it, two runs of the same input are bit-equal) but its
// association differs from the reference's single tile-by-tile chain (norm.rs:113-117), so the weight
// gradient matches the reference to f32 rounding, not bit for bit.  Arithmetic is f32 whatever the
// activation type.

#include <cstdio>
#include <cstring>

#include "../../include/moe_b200.h"
#include "../../include/rmsnorm_b200.h"
#include "common.cuh"

namespace moe {
namespace {

constexpr int RN_TILE = 32;       // rows per backward tile (norm.rs:14)
constexpr int RN_THREADS = 256;

template <typename T> __device__ __forceinline__ T rn_cast(float v);
template <> __device__ __forceinline__ float rn_cast<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 rn_cast<bf16>(float v) { return __float2bfloat16_rn(v); }

// 8 consecutive values as f32
template <typename T> __device__ __forceinline__ void load8(const T* p, float* o);
template <> __device__ __forceinline__ void load8<float>(const float* p, float* o) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *(reinterpret_cast<const float4*>(p) + 1);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <> __device__ __forceinline__ void load8<bf16>(const bf16* p, float* o) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o[2 * i] = __uint_as_float(w[i] << 16);
    o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float* v);
template <> __device__ __forceinline__ void store8<float>(float* p, const float* v) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *(reinterpret_cast<float4*>(p) + 1) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8<bf16>(bf16* p, const float* v) {
  uint4 o;
  uint32_t* w = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = o;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per row: the row is read once (kept in registers when it fits 32 values per lane, re-read
// from L1 otherwise), the sum of squares is reduced over the warp, the scaled row is written.
template <typename T>
__global__ void __launch_bounds__(RN_THREADS)
rmsnorm_fwd_kernel(const T* __restrict__ x, const float* __restrict__ weight, T* __restrict__ y, int rows, int d, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * (RN_THREADS / 32) + warp;
  if (row >= rows) return;
  const T* xr = x + (size_t)row * d;
  T* yr = y + (size_t)row * d;
  float ss = 0.f;
  for (int c = lane * 8; c < d; c += 256) {
    float v[8];
    load8<T>(xr + c, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)d + eps);       // norm.rs:124-127
  for (int c = lane * 8; c < d; c += 256) {
    float v[8], w[8];
    load8<T>(xr + c, v);
    load8<float>(weight + c, w);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = v[i] * inv * w[i];     // norm.rs:56
    store8<T>(yr + c, v);
  }
}

// The same with the row held in registers between the two passes (d = 256 NC exactly, bf16): every load
// of the row is issued before the first use, and x is read once.
template <int NC>
__global__ void __launch_bounds__(RN_THREADS, 2)
rmsnorm_fwd_regs_kernel(const bf16* __restrict__ x, const float* __restrict__ weight, bf16* __restrict__ y, int rows, float eps) {
  constexpr int d = 256 * NC;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * (RN_THREADS / 32) + warp;
  if (row >= rows) return;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * d) + lane;
  uint4 raw[NC];
#pragma unroll
  for (int n = 0; n < NC; ++n) raw[n] = xr[32 * n];
  float ss = 0.f;
#pragma unroll
  for (int n = 0; n < NC; ++n) {
    const uint32_t w[4] = {raw[n].x, raw[n].y, raw[n].z, raw[n].w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a = __uint_as_float(w[i] << 16), b = __uint_as_float(w[i] & 0xffff0000u);
      ss = fmaf(a, a, ss);
      ss = fmaf(b, b, ss);
    }
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)d + eps);       // norm.rs:124-127
  bf16* yr = y + (size_t)row * d + lane * 8;
#pragma unroll
  for (int n = 0; n < NC; ++n) {
    const uint32_t w[4] = {raw[n].x, raw[n].y, raw[n].z, raw[n].w};
    float v[8], ww[8];
    load8<float>(weight + lane * 8 + 256 * n, ww);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16) * inv * ww[2 * i];             // norm.rs:56
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u) * inv * ww[2 * i + 1];
    }
    store8<bf16>(yr + 256 * n, v);
  }
}

// One CTA per tile of 32 rows.  Phase A (a warp per row): inverse RMS and the shared term
// projection * inverse_rms^3 / d (norm.rs:88-94).  Phase B (a thread per 8 columns, rows in order):
// grad_x and the tile's partial weight gradient, summed over the rows in row order (norm.rs:96-104).
template <typename T>
__global__ void __launch_bounds__(RN_THREADS)
rmsnorm_bwd_kernel(const T* __restrict__ x, const float* __restrict__ weight, const T* __restrict__ gy,
                   T* __restrict__ gx, float* __restrict__ partial /*[tiles, d] or null*/, int rows, int d, float eps) {
  __shared__ float s_inv[RN_TILE], s_shared[RN_TILE];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * RN_TILE, nrows = min(RN_TILE, rows - row0);
  for (int r = warp; r < nrows; r += RN_THREADS / 32) {
    const T* xr = x + (size_t)(row0 + r) * d;
    const T* gr = gy + (size_t)(row0 + r) * d;
    float ss = 0.f, proj = 0.f;
    for (int c = lane * 8; c < d; c += 256) {
      float v[8], g[8], w[8];
      load8<T>(xr + c, v);
      load8<T>(gr + c, g);
      load8<float>(weight + c, w);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        ss = fmaf(v[i], v[i], ss);
        proj = fmaf(g[i] * w[i], v[i], proj);
      }
    }
    ss = warp_sum(ss);
    proj = warp_sum(proj);
    if (lane == 0) {
      const float inv = 1.0f / sqrtf(ss / (float)d + eps);
      s_inv[r] = inv;
      s_shared[r] = proj * (inv * inv * inv) / (float)d;
    }
  }
  __syncthreads();
  for (int c = threadIdx.x * 8; c < d; c += RN_THREADS * 8) {
    float w[8], acc[8];
    load8<float>(weight + c, w);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int r0 = 0; r0 < nrows; r0 += 4) {     // four rows' loads in flight, then the rows in order
      float v[4][8], g[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = min(r0 + u, nrows - 1);
        load8<T>(x + (size_t)(row0 + r) * d + c, v[u]);
        load8<T>(gy + (size_t)(row0 + r) * d + c, g[u]);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = r0 + u;
        if (r < nrows) {
          const float inv = s_inv[r], sh = s_shared[r];
          float o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            o[i] = __fsub_rn(__fmul_rn(__fmul_rn(g[u][i], w[i]), inv), __fmul_rn(v[u][i], sh));   // norm.rs:97-98
            acc[i] = __fadd_rn(acc[i], __fmul_rn(__fmul_rn(g[u][i], v[u][i]), inv));               // norm.rs:103
          }
          store8<T>(gx + (size_t)(row0 + r) * d + c, o);
        }
      }
    }
    if (partial) store8<float>(partial + (size_t)blockIdx.x * d + c, acc);
  }
}

// The same tile in sub-tiles of 8 rows (d <= 2048 NG): phase A and phase B alternate per sub-tile, so what
// phase B reads again (8 rows of x and grad_y, 128 KB at d 4096 in bf16) is still in L1 / L2 — with whole
// 32-row tiles the CTAs in flight hold more than L2 and the second read came from HBM (1.02 GB read per
// launch against 0.54 GB algorithmic).  The partial weight gradient stays in registers across the
// sub-tiles, rows in order.
template <typename T, int NG>
__global__ void __launch_bounds__(RN_THREADS)
rmsnorm_bwd_sub_kernel(const T* __restrict__ x, const float* __restrict__ weight, const T* __restrict__ gy,
                       T* __restrict__ gx, float* __restrict__ partial /*[tiles, d] or null*/, int rows, int d, float eps) {
  constexpr int SUB = RN_THREADS / 32;   // one row per warp in phase A
  __shared__ float s_inv[SUB], s_shared[SUB];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * RN_TILE, nrows = min(RN_TILE, rows - row0);
  float w[NG][8], acc[NG][8];
#pragma unroll
  for (int n = 0; n < NG; ++n) {
    const int c = threadIdx.x * 8 + n * RN_THREADS * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) { acc[n][i] = 0.f; w[n][i] = 0.f; }
    if (c < d) load8<float>(weight + c, w[n]);
  }
  for (int sub = 0; sub < nrows; sub += SUB) {
    const int nsub = min(SUB, nrows - sub);
    if (warp < nsub) {
      const T* xr = x + (size_t)(row0 + sub + warp) * d;
      const T* gr = gy + (size_t)(row0 + sub + warp) * d;
      float ss = 0.f, proj = 0.f;
      for (int c = lane * 8; c < d; c += 256) {
        float v[8], g[8], ww[8];
        load8<T>(xr + c, v);
        load8<T>(gr + c, g);
        load8<float>(weight + c, ww);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          ss = fmaf(v[i], v[i], ss);
          proj = fmaf(g[i] * ww[i], v[i], proj);
        }
      }
      ss = warp_sum(ss);
      proj = warp_sum(proj);
      if (lane == 0) {
        const float inv = 1.0f / sqrtf(ss / (float)d + eps);
        s_inv[warp] = inv;
        s_shared[warp] = proj * (inv * inv * inv) / (float)d;
      }
    }
    __syncthreads();
#pragma unroll
    for (int n = 0; n < NG; ++n) {
      const int c = threadIdx.x * 8 + n * RN_THREADS * 8;
      if (c >= d) continue;
      for (int r0 = 0; r0 < nsub; r0 += 4) {     // four rows' loads in flight, then the rows in order
        float v[4][8], g[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int r = min(r0 + u, nsub - 1);
          load8<T>(x + (size_t)(row0 + sub + r) * d + c, v[u]);
          load8<T>(gy + (size_t)(row0 + sub + r) * d + c, g[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int r = r0 + u;
          if (r < nsub) {
            const float inv = s_inv[r], sh = s_shared[r];
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              o[i] = __fsub_rn(__fmul_rn(__fmul_rn(g[u][i], w[n][i]), inv), __fmul_rn(v[u][i], sh));   // norm.rs:97-98
              acc[n][i] = __fadd_rn(acc[n][i], __fmul_rn(__fmul_rn(g[u][i], v[u][i]), inv));           // norm.rs:103
            }
            store8<T>(gx + (size_t)(row0 + sub + r) * d + c, o);
          }
        }
      }
    }
    __syncthreads();   // the next sub-tile overwrites s_inv / s_shared
  }
  if (partial) {
#pragma unroll
    for (int n = 0; n < NG; ++n) {
      const int c = threadIdx.x * 8 + n * RN_THREADS * 8;
      if (c < d) store8<float>(partial + (size_t)blockIdx.x * d + c, acc[n]);
    }
  }
}

template <typename T>
void launch_bwd(const T* x, const float* weight, const T* gy, T* gx, float* partial, int rows, int d, float eps, int tiles,
                cudaStream_t st) {
  if (d <= 2048) rmsnorm_bwd_sub_kernel<T, 1><<<tiles, RN_THREADS, 0, st>>>(x, weight, gy, gx, partial, rows, d, eps);
  else if (d <= 4096) rmsnorm_bwd_sub_kernel<T, 2><<<tiles, RN_THREADS, 0, st>>>(x, weight, gy, gx, partial, rows, d, eps);
  else if (d <= 8192) rmsnorm_bwd_sub_kernel<T, 4><<<tiles, RN_THREADS, 0, st>>>(x, weight, gy, gx, partial, rows, d, eps);
  else rmsnorm_bwd_kernel<T><<<tiles, RN_THREADS, 0, st>>>(x, weight, gy, gx, partial, rows, d, eps);
}

// grad_weight[c] += sum over the tiles of partial[t][c] (norm.rs:113-117).  The tiles are cut into 32
// consecutive runs, one warp per run and 32 columns per CTA; a run is summed in tile order and the run
// totals are added in run order, so the result does not depend on how the work was scheduled.
constexpr int RN_RUNS = 32;
__global__ void __launch_bounds__(32 * RN_RUNS)
rmsnorm_wgrad_kernel(const float* __restrict__ partial, float* __restrict__ grad_weight, int tiles, int d) {
  __shared__ float s_run[RN_RUNS][32];
  const int lane = threadIdx.x & 31, run = threadIdx.x >> 5, c = blockIdx.x * 32 + lane;
  const int per = ceil_div(tiles, RN_RUNS), t_lo = run * per, t_hi = min(tiles, t_lo + per);
  float g = 0.f;
  if (c < d) {
    for (int t0 = t_lo; t0 < t_hi; t0 += 8) {     // eight independent loads, then the ordered sum
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = t0 + i < t_hi ? partial[(size_t)(t0 + i) * d + c] : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (t0 + i < t_hi) g = __fadd_rn(g, v[i]);
    }
  }
  s_run[run][lane] = g;
  __syncthreads();
  if (run == 0 && c < d) {
    float total = grad_weight[c];
#pragma unroll
    for (int r = 0; r < RN_RUNS; ++r) total = __fadd_rn(total, s_run[r][lane]);
    grad_weight[c] = total;
  }
}

int rn_fail(char* message, int len, int code, const char* text) {
  if (message && len > 0) snprintf(message, (size_t)len, "%s", text);
  return code;
}

int rn_check(const void* a, const void* b, const void* c, int rows, int d, int precision, char* message, int len) {
  if (!a || !b || !c) return rn_fail(message, len, MOE_INVALID_INPUT, "InvalidInput: null buffer");
  if (rows < 0 || d <= 0) return rn_fail(message, len, MOE_INVALID_INPUT, "InvalidInput: rows and d_model must be positive");
  if (d % 8 != 0) return rn_fail(message, len, MOE_UNSUPPORTED, "Unsupported: d_model must be a multiple of 8");
  if (precision != MOE_PRECISION_F32 && precision != MOE_PRECISION_BF16)
    return rn_fail(message, len, MOE_INVALID_CONFIG, "InvalidConfig: precision is f32 or bf16");
  if ((((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15) != 0)
    return rn_fail(message, len, MOE_INVALID_INPUT, "InvalidInput: buffers must be 16-byte aligned");
  return MOE_OK;
}

}  // namespace
}  // namespace moe

using namespace moe;

extern "C" {

int32_t rmsnorm_forward(const void* x, const float* weight, void* y, int32_t rows, int32_t d, float eps, int32_t precision,
                        void* stream, char* message, int32_t message_len) {
  if (int rc = rn_check(x, weight, y, rows, d, precision, message, message_len)) return rc;
  if (rows == 0) return MOE_OK;
  const int grid = ceil_div(rows, RN_THREADS / 32);
  cudaStream_t st = (cudaStream_t)stream;
  const int nc = d % 256 == 0 ? d / 256 : 0;
  if (precision == MOE_PRECISION_BF16 && (nc == 2 || nc == 4 || nc == 8 || nc == 16)) {
    const bf16* xb = (const bf16*)x;
    bf16* yb = (bf16*)y;
    if (nc == 2) rmsnorm_fwd_regs_kernel<2><<<grid, RN_THREADS, 0, st>>>(xb, weight, yb, rows, eps);
    else if (nc == 4) rmsnorm_fwd_regs_kernel<4><<<grid, RN_THREADS, 0, st>>>(xb, weight, yb, rows, eps);
    else if (nc == 8) rmsnorm_fwd_regs_kernel<8><<<grid, RN_THREADS, 0, st>>>(xb, weight, yb, rows, eps);
    else rmsnorm_fwd_regs_kernel<16><<<grid, RN_THREADS, 0, st>>>(xb, weight, yb, rows, eps);
  } else if (precision == MOE_PRECISION_BF16) rmsnorm_fwd_kernel<bf16><<<grid, RN_THREADS, 0, st>>>((const bf16*)x, weight, (bf16*)y, rows, d, eps);
  else rmsnorm_fwd_kernel<float><<<grid, RN_THREADS, 0, st>>>((const float*)x, weight, (float*)y, rows, d, eps);
  count_launch();
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? MOE_OK : rn_fail(message, message_len, MOE_CUDA_ERROR, cudaGetErrorString(e));
}

int64_t rmsnorm_scratch_bytes(int32_t rows, int32_t d) {
  if (rows <= 0 || d <= 0) return 0;
  return (int64_t)ceil_div(rows, RN_TILE) * d * (int64_t)sizeof(float);
}

int32_t rmsnorm_backward(const void* x, const float* weight, const void* grad_y, void* grad_x, float* grad_weight,
                         void* scratch, int32_t rows, int32_t d, float eps, int32_t precision, void* stream, char* message,
                         int32_t message_len) {
  if (int rc = rn_check(x, weight, grad_y, rows, d, precision, message, message_len)) return rc;
  if (!grad_x || ((uintptr_t)grad_x & 15)) return rn_fail(message, message_len, MOE_INVALID_INPUT, "InvalidInput: grad_x is null or unaligned");
  if (grad_weight && (!scratch || ((uintptr_t)scratch & 15)))
    return rn_fail(message, message_len, MOE_INVALID_INPUT, "InvalidInput: a weight gradient needs 16-byte aligned scratch (rmsnorm_scratch_bytes)");
  if (rows == 0) return MOE_OK;
  const int tiles = ceil_div(rows, RN_TILE);
  cudaStream_t st = (cudaStream_t)stream;
  float* partial = grad_weight ? (float*)scratch : nullptr;
  if (precision == MOE_PRECISION_BF16) launch_bwd<bf16>((const bf16*)x, weight, (const bf16*)grad_y, (bf16*)grad_x, partial, rows, d, eps, tiles, st);
  else launch_bwd<float>((const float*)x, weight, (const float*)grad_y, (float*)grad_x, partial, rows, d, eps, tiles, st);
  count_launch();
  if (grad_weight) {
    rmsnorm_wgrad_kernel<<<ceil_div(d, 32), 32 * RN_RUNS, 0, st>>>(partial, grad_weight, tiles, d);
    count_launch();
  }
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? MOE_OK : rn_fail(message, message_len, MOE_CUDA_ERROR, cudaGetErrorString(e));
}

}  // extern "C"
