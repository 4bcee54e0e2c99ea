// f32 path: grouped GEMMs on the CUDA cores with exact f32 accumulation, plus the
// pointwise SwiGLU kernels and the optimizer / cast helpers.
//
// The f32 configuration has to agree with an f32 host evaluation to 1e-5 relative
// L2, which no bf16 or tf32 tensor-core mode reaches, so these products use FMA
// on the CUDA cores.  They also accept every shape (no alignment rules), which is
// what the small closed-form parity cases need.  Row groups are the same padded
// groups the tensor-core path uses.
//
// Replaces, for the f32 configuration, the per-expert cuBLAS calls of the
// reference (gpu_model.rs:2524-2568, 3595-3656) and swiglu_fwd / swiglu_bwd
// (cuda_training.rs:259-264); Adam follows param.rs:562-589 / cuda_training.rs:66.

#include "kernels.cuh"

namespace moe {

constexpr int ST = 64;   // tile edge
constexpr int SK = 16;   // reduction slice

// MODE 0: C[row,n] = sum_k A[row,k] B_g[n,k]      (rows grouped)
// MODE 1: C[row,n] = sum_k A[row,k] B_g[k,n]      (rows grouped)
// MODE 2: C_g[m,n] (+)= sum_row A[row,m] B[row,n] (rows of group g are the reduction)
template <int MODE>
__global__ void __launch_bounds__(256) simt_gemm_kernel(SimtGemmArgs a) {
  __shared__ float As[SK][ST + 4];
  __shared__ float Bs[SK][ST + 4];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int n0 = blockIdx.x * ST;
  int g = 0, row0 = 0, m0 = 0, kbeg = 0, kend = 0;
  if (MODE == 2) {
    g = blockIdx.z;
    m0 = blockIdx.y * ST;
    kbeg = a.group_row0[g];
    kend = a.group_row0[g + 1];
  } else {
    row0 = blockIdx.y * ST;
    if (row0 >= a.group_row0[a.n_groups]) return;
    int lo = 0, hi = a.n_groups;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (a.group_row0[mid] <= row0) lo = mid; else hi = mid;
    }
    g = lo;
    kbeg = 0;
    kend = a.K;
  }
  const float* B = a.B + (MODE == 2 ? 0 : (long long)g * a.b_group_stride);
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = kbeg; k0 < kend; k0 += SK) {
    for (int i = tid; i < ST * SK; i += 256) {
      float av, bv;
      if (MODE == 2) {
        const int kk = i / ST, c = i - kk * ST;   // contiguous along the output dims
        const int row = k0 + kk;
        av = (row < kend && row < a.a_rows && m0 + c < a.M) ? a.A[(long long)row * a.M + m0 + c] : 0.f;
        bv = (row < kend && row < a.b_rows && n0 + c < a.N) ? a.B[(long long)row * a.N + n0 + c] : 0.f;
        As[kk][c] = av;
        Bs[kk][c] = bv;
      } else {
        const int r = i / SK, kk = i - r * SK;    // contiguous along k
        av = (k0 + kk < kend && row0 + r < a.a_rows) ? a.A[(long long)(row0 + r) * a.K + k0 + kk] : 0.f;
        As[kk][r] = av;
        if (MODE == 0) {
          bv = (n0 + r < a.N && k0 + kk < kend) ? B[(long long)(n0 + r) * a.K + k0 + kk] : 0.f;
          Bs[kk][r] = bv;
        } else {
          const int kk2 = i / ST, c = i - kk2 * ST;
          bv = (k0 + kk2 < kend && n0 + c < a.N) ? B[(long long)(k0 + kk2) * a.N + n0 + c] : 0.f;
          Bs[kk2][c] = bv;
        }
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SK; ++kk) {
      const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      const float ar[4] = {av.x, av.y, av.z, av.w};
      const float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= a.N) continue;
      if (MODE == 2) {
        const int m = m0 + ty * 4 + i;
        if (m >= a.M) continue;
        float* c = a.C + (long long)g * a.c_group_stride + (long long)m * a.N + n;
        *c = a.accumulate ? *c + acc[i][j] : acc[i][j];
      } else {
        a.C[(long long)(row0 + ty * 4 + i) * a.N + n] = acc[i][j];
      }
    }
}

cudaError_t simt_gemm_nt(const SimtGemmArgs& a, cudaStream_t stream) {
  if (a.max_rows <= 0) return cudaSuccess;
  simt_gemm_kernel<0><<<dim3(ceil_div(a.N, ST), ceil_div(a.max_rows, ST)), 256, 0, stream>>>(a); count_launch();
  return cudaGetLastError();
}
cudaError_t simt_gemm_nn(const SimtGemmArgs& a, cudaStream_t stream) {
  if (a.max_rows <= 0) return cudaSuccess;
  simt_gemm_kernel<1><<<dim3(ceil_div(a.N, ST), ceil_div(a.max_rows, ST)), 256, 0, stream>>>(a); count_launch();
  return cudaGetLastError();
}
cudaError_t simt_gemm_tn(const SimtGemmArgs& a, cudaStream_t stream) {
  simt_gemm_kernel<2><<<dim3(ceil_div(a.N, ST), ceil_div(a.M, ST), a.n_groups), 256, 0, stream>>>(a); count_launch();
  return cudaGetLastError();
}

// gu rows are [2*f_pad]: 32 gate values, then the matching 32 up values, repeated.
__global__ void swiglu_fwd_f32_kernel(const float* __restrict__ gu, float* __restrict__ h, long long n, int f_pad) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long row = i / f_pad;
  const int f = (int)(i - row * f_pad);
  const float* r = gu + row * 2 * f_pad;
  h[i] = siluf_(r[gu_row(0, f)]) * r[gu_row(1, f)];
}

__global__ void swiglu_bwd_f32_kernel(const float* __restrict__ dh, const float* __restrict__ gu,
                                      float* __restrict__ dgu, long long n, int f_pad) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long row = i / f_pad;
  const int f = (int)(i - row * f_pad);
  const float* r = gu + row * 2 * f_pad;
  float* o = dgu + row * 2 * f_pad;
  const float g = r[gu_row(0, f)], u = r[gu_row(1, f)], up = dh[i];
  o[gu_row(0, f)] = up * u * silu_grad_(g);
  o[gu_row(1, f)] = up * siluf_(g);
}

// f32 -> three bf16 pieces (value = hi + mid + lo to 24 bits: each piece is the bf16 rounding of what the earlier
// ones left), laid out along the reduction as six segments of `cols` so that ONE bf16 tensor-core product of an
// A-pattern matrix with a B-pattern matrix adds the six significant cross terms with f32 accumulation:
//   A pattern  [hi | hi | mid | mid | hi | lo ]
//   B pattern  [hi | mid| hi  | mid | lo | hi ]      ->  hi*hi + hi*mid + mid*hi + mid*mid + hi*lo + lo*hi
// The dropped terms (mid*lo, lo*mid, lo*lo) are below 2^-24 of the product.
__global__ void expand3_kernel(const float* __restrict__ src, bf16* __restrict__ dst, long long rows, int cols, int b_pattern) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * cols) return;
  const long long r = i / cols;
  const int c = (int)(i - r * cols);
  const float a = src[i];
  const bf16 hi = __float2bfloat16_rn(a);
  const float r1 = a - __bfloat162float(hi);
  const bf16 mid = __float2bfloat16_rn(r1);
  const bf16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
  bf16* d = dst + r * 6 * cols + c;
  if (b_pattern) { d[0] = hi; d[cols] = mid; d[2 * cols] = hi; d[3 * cols] = mid; d[4 * cols] = lo; d[5 * cols] = hi; }
  else { d[0] = hi; d[cols] = hi; d[2 * cols] = mid; d[3 * cols] = mid; d[4 * cols] = hi; d[5 * cols] = lo; }
}
cudaError_t launch_expand3(const float* src, bf16* dst, long long rows, int cols, int b_pattern, cudaStream_t stream) {
  const long long n = rows * cols;
  if (n <= 0) return cudaSuccess;
  expand3_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(src, dst, rows, cols, b_pattern); count_launch();
  return cudaGetLastError();
}

cudaError_t launch_swiglu_fwd_f32(const float* gu, float* h, long long rows, int f_pad, cudaStream_t stream) {
  const long long n = rows * f_pad;
  if (n <= 0) return cudaSuccess;
  swiglu_fwd_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(gu, h, n, f_pad); count_launch();
  return cudaGetLastError();
}
cudaError_t launch_swiglu_bwd_f32(const float* dh, const float* gu, float* dgu, long long rows, int f_pad,
                                  cudaStream_t stream) {
  const long long n = rows * f_pad;
  if (n <= 0) return cudaSuccess;
  swiglu_bwd_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(dh, gu, dgu, n, f_pad); count_launch();
  return cudaGetLastError();
}

// Param::step for Optimizer::Adam (param.rs:562-589), operation for operation, then
// the gradient is cleared and the bf16 compute copy refreshed in the same pass.
__global__ void adam_kernel(AdamArgs a) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += stride) {
    const float g = __fmul_rn(a.g[i], a.scale);
    const float m = __fadd_rn(__fmul_rn(a.beta1, a.m[i]), __fmul_rn(1.0f - a.beta1, g));
    const float v = __fadd_rn(__fmul_rn(a.beta2, a.v[i]), __fmul_rn(__fmul_rn(1.0f - a.beta2, g), g));
    const float m_hat = __fdiv_rn(m, a.c1);
    const float v_hat = __fdiv_rn(v, a.c2);
    float w = a.w[i];
    w = __fsub_rn(w, __fmul_rn(__fmul_rn(a.lr, a.wd), w));
    w = __fsub_rn(w, __fdiv_rn(__fmul_rn(a.lr, m_hat), __fadd_rn(__fsqrt_rn(v_hat), a.eps)));
    a.m[i] = m; a.v[i] = v; a.w[i] = w; a.g[i] = 0.f;
    if (a.w_bf16) a.w_bf16[i] = __float2bfloat16_rn(w);
  }
}

// Param::step for Optimizer::Sgd (param.rs:557-561) and Optimizer::Lion (param.rs:590-613), operation for operation;
// the gradient is cleared and the bf16 compute copy refreshed in the same pass.  sign(0) = 0 (optimizers.rs:50-58).
__global__ void sgd_kernel(AdamArgs a) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += stride) {
    const float w = __fsub_rn(a.w[i], __fmul_rn(__fmul_rn(a.lr, a.g[i]), a.scale));
    a.w[i] = w; a.g[i] = 0.f;
    if (a.w_bf16) a.w_bf16[i] = __float2bfloat16_rn(w);
  }
}
__global__ void lion_kernel(AdamArgs a) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += stride) {
    const float g = __fmul_rn(a.g[i], a.scale);
    const float m = a.m[i];
    const float update = __fadd_rn(__fmul_rn(a.beta1, m), __fmul_rn(1.0f - a.beta1, g));
    a.m[i] = __fadd_rn(__fmul_rn(a.beta2, m), __fmul_rn(1.0f - a.beta2, g));
    const float sg = update > 0.f ? 1.0f : (update < 0.f ? -1.0f : 0.0f);
    float w = a.w[i];
    w = __fsub_rn(w, __fmul_rn(a.lr, __fadd_rn(sg, __fmul_rn(a.wd, w))));
    a.w[i] = w; a.g[i] = 0.f;
    if (a.w_bf16) a.w_bf16[i] = __float2bfloat16_rn(w);
  }
}
static unsigned opt_grid(long long n) { const long long b = (n + 255) / 256; return (unsigned)(b < 148 * 16 ? b : 148 * 16); }
cudaError_t launch_sgd(const AdamArgs& a, cudaStream_t stream) {
  if (a.n <= 0) return cudaSuccess;
  sgd_kernel<<<opt_grid(a.n), 256, 0, stream>>>(a); count_launch();
  return cudaGetLastError();
}
cudaError_t launch_lion(const AdamArgs& a, cudaStream_t stream) {
  if (a.n <= 0) return cudaSuccess;
  lion_kernel<<<opt_grid(a.n), 256, 0, stream>>>(a); count_launch();
  return cudaGetLastError();
}

cudaError_t launch_adam(const AdamArgs& a, cudaStream_t stream) {
  if (a.n <= 0) return cudaSuccess;
  const long long blocks = (a.n + 255) / 256;
  adam_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, stream>>>(a); count_launch();
  return cudaGetLastError();
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ s, bf16* __restrict__ d, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) d[i] = __float2bfloat16_rn(s[i]);
}
__global__ void cast_bf16_f32_kernel(const bf16* __restrict__ s, float* __restrict__ d, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) d[i] = __bfloat162float(s[i]);
}
__global__ void fill_f32_kernel(float* __restrict__ d, float v, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) d[i] = v;
}
static unsigned grid_for(long long n) {
  const long long b = (n + 255) / 256;
  return (unsigned)(b < 148 * 32 ? (b > 0 ? b : 1) : 148 * 32);
}
cudaError_t launch_cast_f32_to_bf16(const float* s, bf16* d, long long n, cudaStream_t stream) {
  if (n > 0) { cast_f32_bf16_kernel<<<grid_for(n), 256, 0, stream>>>(s, d, n); count_launch(); }
  return cudaGetLastError();
}
cudaError_t launch_cast_bf16_to_f32(const bf16* s, float* d, long long n, cudaStream_t stream) {
  if (n > 0) { cast_bf16_f32_kernel<<<grid_for(n), 256, 0, stream>>>(s, d, n); count_launch(); }
  return cudaGetLastError();
}
cudaError_t launch_fill_f32(float* d, float v, long long n, cudaStream_t stream) {
  if (n > 0) { fill_f32_kernel<<<grid_for(n), 256, 0, stream>>>(d, v, n); count_launch(); }
  return cudaGetLastError();
}

}  // namespace moe
