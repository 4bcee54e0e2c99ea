// int8-weight expert projections for decode-sized batches (a few rows per expert).
//
// Replaces Quantized::matmul_rhs_transposed (reference quantized.rs:55-99) on the
// device: y[t, r] = dot(x[t, :], q[r, :]) * scale[r] with int8 weights and one f32
// scale per output row.  The reference cannot move a quantized model to a device at
// all (param.rs:363-369), so this path has no reference GPU counterpart.
//
// With ~8 rows per expert the layer is a weight-streaming problem: every active
// expert's int8 matrix is read once.  One warp owns 8 output columns (for the fused
// gate|up pass: 8 gate rows and the 8 matching up rows of the interleaved matrix) and
// streams their weight rows with 16-byte loads, 16 reduction values per lane per load.
// The int8 values are widened to f16 in registers (exact: |q| <= 127; two instructions per
// pair, see s8x2_to_f16x2) and multiplied with the f16-converted token rows on the tensor
// cores with mma.sync.m16n8k16 (at 16 rows tcgen05 buys nothing); the
// reduction index is permuted consistently for both operands so that each lane's 16
// contiguous weight bytes feed four MMAs.  The f32 accumulators are scaled per output
// row afterwards; SwiGLU is fused into the gate|up pass.

#include <cuda_fp16.h>

#include "kernels.cuh"

namespace moe {

constexpr int Q8_ROWS = 16;     // token rows per CTA (one m16 MMA tile)
constexpr int Q8_WARPS = 8;
constexpr int Q8_CHUNK = 64;    // reduction values per warp-wide 16-byte load round

// Two int8 weights -> two f16 values in two instructions.  `wx` is the weight word with every
// byte's sign bit flipped (v + 128 as an unsigned byte); a byte permute drops two of those bytes
// under the f16 exponent 0x64 (= 1024 + byte, exact), and one packed subtract of 1152 restores v.
// Going through f16 rather than bf16 is what makes this cheap; the products are exact either way
// and the token rows are converted bf16 -> f16 once per CTA when they are staged.
__device__ __forceinline__ uint32_t s8x2_to_f16x2(uint32_t wx, int lo_byte) {
  const uint32_t packed = __byte_perm(wx, 0x64646464u, lo_byte == 0 ? 0x4140 : 0x4342);
  const __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&packed), __half2half2(__ushort_as_half(0x6480)));
  return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ void mma_f16_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t v) {
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&v);
  const __half2 h = __floats2half2_rn(__low2float(b), __high2float(b));
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <bool SWIGLU>
__global__ void __launch_bounds__(Q8_WARPS * 32) q8_rows_kernel(Q8Args a) {
  extern __shared__ __align__(16) unsigned char q8_smem[];
  bf16* xs = reinterpret_cast<bf16*>(q8_smem);
  const int K = a.K, ldx = K + 8;
  const int g = blockIdx.z, m0 = blockIdx.y * Q8_ROWS;
  int rows;
  const bf16* xin;
  bf16* out;
  if (g < a.E) {
    rows = a.counts[g];
    const size_t base = (size_t)a.pad_off[g];
    xin = a.x_rows + base * K;
    out = a.out_rows + base * a.ldo;
  } else {
    rows = a.tokens;
    xin = a.x_shared;
    out = a.out_shared;
  }
  if (m0 >= rows) return;
  const int mrows = min(Q8_ROWS, rows - m0);
  const int tid = threadIdx.x;
  {
    // the token rows of this tile, eight independent 16-byte loads in flight per thread
    constexpr int SU = 8;
    const int cpr = K / 8, total = Q8_ROWS * cpr;
    for (int base = tid; base < total; base += Q8_WARPS * 32 * SU) {
      uint4 v[SU];
#pragma unroll
      for (int u = 0; u < SU; ++u) {
        const int i = base + u * Q8_WARPS * 32;
        v[u] = make_uint4(0, 0, 0, 0);
        if (i < total) {
          const int r = i / cpr, c = i - r * cpr;
          if (r < mrows) v[u] = *reinterpret_cast<const uint4*>(xin + (size_t)(m0 + r) * K + c * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < SU; ++u) {
        const int i = base + u * Q8_WARPS * 32;
        if (i < total) {
          const int r = i / cpr, c = i - r * cpr;
          *reinterpret_cast<uint4*>(xs + r * ldx + c * 8) =
              make_uint4(bf16x2_to_f16x2(v[u].x), bf16x2_to_f16x2(v[u].y), bf16x2_to_f16x2(v[u].z), bf16x2_to_f16x2(v[u].w));
        }
      }
    }
  }
  __syncthreads();

  const int warp = tid >> 5, lane = tid & 31, gq = lane >> 2, q = lane & 3;
  const float* sc = a.scale + (size_t)g * a.s_group_stride;
  const bf16* xa = xs + gq * ldx;
  const bf16* xb = xs + (gq + 8) * ldx;
  // a CTA keeps its token tile and walks over column blocks (64 columns each, 8 per warp)
  for (int nb = blockIdx.x; nb * 8 * Q8_WARPS < a.N; nb += gridDim.x) {
  const int n0 = (nb * Q8_WARPS + warp) * 8;    // first output column of this warp
  if (n0 >= a.N) continue;
  // weight row of the column this lane streams (column n0 + gq)
  const int wrow = SWIGLU ? gu_row(0, n0 + gq) : n0 + gq;
  const int8_t* w0 = a.w + (size_t)g * a.w_group_stride + (size_t)wrow * K;
  const int8_t* w1 = w0 + (size_t)GU_BLOCK * K;          // matching up row (SWIGLU only)
  float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};

  constexpr int UNROLL = SWIGLU ? 4 : 11;  // 16-byte weight loads in flight per lane and matrix (2816 = 4 x 11 x 64)
  for (int c0 = 0; c0 < K; c0 += Q8_CHUNK * UNROLL) {
    uint4 wq[UNROLL], uq[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int kc = c0 + Q8_CHUNK * u;      // warp-uniform: K is a multiple of 64
      const int k = kc + 16 * q;
      wq[u] = make_uint4(0, 0, 0, 0);
      uq[u] = make_uint4(0, 0, 0, 0);
      if (kc < K) {
        wq[u] = __ldg(reinterpret_cast<const uint4*>(w0 + k));
        if (SWIGLU) uq[u] = __ldg(reinterpret_cast<const uint4*>(w1 + k));
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int kc = c0 + Q8_CHUNK * u;
      if (kc >= K) continue;                 // uniform over the warp: every lane joins every MMA
      const int k = kc + 16 * q;
      const uint32_t ww[4] = {wq[u].x ^ 0x80808080u, wq[u].y ^ 0x80808080u, wq[u].z ^ 0x80808080u, wq[u].w ^ 0x80808080u};
      const uint32_t uu[4] = {uq[u].x ^ 0x80808080u, uq[u].y ^ 0x80808080u, uq[u].z ^ 0x80808080u, uq[u].w ^ 0x80808080u};
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        // reduction slots of this MMA: (2q, 2q+1) <- k+4s+{0,1}, (2q+8, 2q+9) <- k+4s+{2,3}
        const uint2 lo = *reinterpret_cast<const uint2*>(xa + k + 4 * s);
        const uint2 hi = *reinterpret_cast<const uint2*>(xb + k + 4 * s);
        mma_f16_16816(acc0, lo.x, hi.x, lo.y, hi.y, s8x2_to_f16x2(ww[s], 0), s8x2_to_f16x2(ww[s], 2));
        if (SWIGLU) mma_f16_16816(acc1, lo.x, hi.x, lo.y, hi.y, s8x2_to_f16x2(uu[s], 0), s8x2_to_f16x2(uu[s], 2));
      }
    }
  }

  // accumulator layout: c[0], c[1] -> row gq, columns 2q, 2q+1; c[2], c[3] -> row gq+8
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int col = n0 + 2 * q + j;
    if (col >= a.N) continue;
    float s0, s1 = 0.f;
    if (SWIGLU) { s0 = sc[gu_row(0, col)]; s1 = sc[gu_row(1, col)]; } else { s0 = sc[col]; }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = gq + 8 * half;
      if (r >= mrows) continue;
      float v = acc0[2 * half + j] * s0;
      if (SWIGLU) v = siluf_(v) * (acc1[2 * half + j] * s1);
      out[(size_t)(m0 + r) * a.ldo + col] = __float2bfloat16_rn(v);
    }
  }
  }   // column blocks
}

cudaError_t launch_q8_rows(const Q8Args& a, bool swiglu, cudaStream_t stream) {
  if (a.tokens <= 0) return cudaSuccess;
  const int groups = a.E + (a.x_shared ? 1 : 0);
  // gate|up: two column blocks per CTA (the token tile is staged once for twice the weight stream);
  // the narrower down projection needs every CTA it can get
  const int nblocks = ceil_div(a.N, 8 * Q8_WARPS);
  const dim3 grid(swiglu ? ceil_div(nblocks, 2) : nblocks, ceil_div(a.tokens, Q8_ROWS), groups);
  const size_t smem = (size_t)Q8_ROWS * (a.K + 8) * sizeof(bf16);
  if (swiglu) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(q8_rows_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    q8_rows_kernel<true><<<grid, Q8_WARPS * 32, smem, stream>>>(a);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(q8_rows_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    q8_rows_kernel<false><<<grid, Q8_WARPS * 32, smem, stream>>>(a);
  }
  count_launch();
  return cudaGetLastError();
}

}  // namespace moe
