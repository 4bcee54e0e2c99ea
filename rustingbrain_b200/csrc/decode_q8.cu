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

// A warp owns two 8-column MMA tiles that share the token fragments: for the fused pass the gate
// rows of 8 hidden columns and the matching up rows, otherwise 16 adjacent output columns.
// U = 16-byte loads per lane and tile in one chunk of 64 U reduction values; K is a multiple of 64 U.
template <bool SWIGLU, int U>
__global__ void __launch_bounds__(Q8_WARPS * 32) q8_rows_kernel(Q8Args a) {
  extern __shared__ __align__(16) unsigned char q8_smem[];
  // Token tile in MMA-fragment order: rows r and r + 8 are interleaved so that one 16-byte unit holds
  // the four A registers of a lane, {x[r][k..k+1], x[r+8][k..k+1], x[r][k+2..k+3], x[r+8][k+2..k+3]} for a
  // group of four reduction values.  Row pair r has K/4 units plus one unit of padding, and units 8..15 of
  // every 16 swap their 2-unit halves: the four quarter-chunks a quarter-warp reads then fall into
  // different banks.
  const int K = a.K;
  const int pitch = (K / 4 + 1) * 16;   // bytes per row pair
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
  const int warp = tid >> 5, lane = tid & 31, gq = lane >> 2, q = lane & 3;

  constexpr int COLS = SWIGLU ? 8 : 16;               // output columns per warp
  constexpr int STEP = Q8_CHUNK * U;                  // reduction values per chunk
  const int chunks = K / STEP;
  const int n_blocks = ceil_div(a.N, COLS * Q8_WARPS);
  const int8_t* wbase = a.w + (size_t)g * a.w_group_stride + 16 * q;
  const size_t tile1 = (size_t)(SWIGLU ? GU_BLOCK : 8) * K;   // second tile's rows relative to the first
  // first weight row of this lane in column block nb (nullptr when the warp has no columns there)
  auto row_ptr0 = [&](int nb) -> const int8_t* {
    const int n0 = (nb * Q8_WARPS + warp) * COLS;
    if (nb >= n_blocks || n0 >= a.N) return nullptr;
    return wbase + (size_t)(SWIGLU ? gu_row(0, n0 + gq) : n0 + gq) * K;
  };
  struct Chunk { uint4 w[U], u[U]; };
  // The weight stream does not depend on the tokens: two register sets alternate so that the loads
  // of the next chunk are in flight while this one is multiplied, and the first chunk is requested
  // before the token tile is staged.
  const int8_t* fp = row_ptr0(blockIdx.x);   // fetch cursor
  int f_nb = blockIdx.x, f_c = 0;
  auto fetch = [&](Chunk& ch) {
    if (fp) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        ch.w[u] = __ldg(reinterpret_cast<const uint4*>(fp + Q8_CHUNK * u));
        ch.u[u] = __ldg(reinterpret_cast<const uint4*>(fp + tile1 + Q8_CHUNK * u));
      }
      fp += STEP;
    }
    if (++f_c == chunks) { f_c = 0; f_nb += gridDim.x; fp = row_ptr0(f_nb); }
  };
  Chunk ca, cb;
  fetch(ca);

  {
    // the token rows of this tile as f16, eight independent 16-byte loads in flight per thread
    constexpr int SU = 8;
    const int cpr = K / 8, total = Q8_ROWS * cpr;
    int r = tid / cpr, c = tid - r * cpr;             // (row, 16-byte column) of this thread's first element
    const int dr = (Q8_WARPS * 32) / cpr, dc = (Q8_WARPS * 32) - dr * cpr;
    for (int base = tid; base < total; base += Q8_WARPS * 32 * SU) {
      uint4 v[SU];
      int rr[SU], cc[SU];
#pragma unroll
      for (int u = 0; u < SU; ++u) {
        rr[u] = r; cc[u] = c;
        v[u] = make_uint4(0, 0, 0, 0);
        if (r < mrows) v[u] = *reinterpret_cast<const uint4*>(xin + (size_t)(m0 + r) * K + c * 8);
        r += dr; c += dc;
        if (c >= cpr) { c -= cpr; ++r; }
      }
#pragma unroll
      for (int u = 0; u < SU; ++u) {
        if (rr[u] < Q8_ROWS) {
          // eight values = two groups of four; row half (r / 8) selects the 4-byte slot inside a unit
          unsigned char* row = q8_smem + (rr[u] & 7) * pitch + (rr[u] >> 3) * 4;
          const int kg = cc[u] * 2;
          unsigned char* u0 = row + (kg ^ ((kg >> 2) & 2)) * 16;
          unsigned char* u1 = row + ((kg + 1) ^ (((kg + 1) >> 2) & 2)) * 16;
          *reinterpret_cast<uint32_t*>(u0) = bf16x2_to_f16x2(v[u].x);
          *reinterpret_cast<uint32_t*>(u0 + 8) = bf16x2_to_f16x2(v[u].y);
          *reinterpret_cast<uint32_t*>(u1) = bf16x2_to_f16x2(v[u].z);
          *reinterpret_cast<uint32_t*>(u1 + 8) = bf16x2_to_f16x2(v[u].w);
        }
      }
    }
  }
  __syncthreads();

  const float* sc = a.scale + (size_t)g * a.s_group_stride;
  // this lane's fragments: unit (k / 4) of row pair gq; for quarter-chunks 2 and 3 the halves are swapped
  const unsigned char* xa0 = q8_smem + gq * pitch + (4 * q) * 16;
  const int sw = (q & 2) ? 32 : 0;
  const unsigned char* xa = xa0;              // compute cursor into the token tile
  int m_nb = blockIdx.x, m_c = 0;
  float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};

  auto multiply = [&](const Chunk& ch) {
    const int n0 = (m_nb * Q8_WARPS + warp) * COLS;
    const bool live = n0 < a.N;              // warp-uniform
    if (live) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t ww[4] = {ch.w[u].x ^ 0x80808080u, ch.w[u].y ^ 0x80808080u, ch.w[u].z ^ 0x80808080u, ch.w[u].w ^ 0x80808080u};
        const uint32_t uu[4] = {ch.u[u].x ^ 0x80808080u, ch.u[u].y ^ 0x80808080u, ch.u[u].z ^ 0x80808080u, ch.u[u].w ^ 0x80808080u};
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          // reduction slots of this MMA: (2q, 2q+1) <- k+4s+{0,1}, (2q+8, 2q+9) <- k+4s+{2,3}
          // the A registers of reduction values k + 4s .. k + 4s + 3, rows gq and gq + 8, in one load
          const uint4 f = *reinterpret_cast<const uint4*>((s < 2 ? xa + sw : xa + (32 - sw)) + u * (Q8_CHUNK * 4) + (s & 1) * 16);
          mma_f16_16816(acc0, f.x, f.y, f.z, f.w, s8x2_to_f16x2(ww[s], 0), s8x2_to_f16x2(ww[s], 2));
          mma_f16_16816(acc1, f.x, f.y, f.z, f.w, s8x2_to_f16x2(uu[s], 0), s8x2_to_f16x2(uu[s], 2));
        }
      }
    }
    xa += STEP * 4;   // 16 bytes per four reduction values
    if (++m_c < chunks) return;
    // last chunk of a column block: scale, activate, store.
    // accumulator layout: c[0], c[1] -> row gq, columns 2q, 2q+1; c[2], c[3] -> row gq+8
    if (live) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int col = n0 + 2 * q + j;
        const float s0 = SWIGLU ? sc[gu_row(0, col)] : sc[col];
        const float s1 = SWIGLU ? sc[gu_row(1, col)] : sc[col + 8];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int r = gq + 8 * half;
          if (r >= mrows) continue;
          bf16* o = out + (size_t)(m0 + r) * a.ldo + col;
          const float v0 = acc0[2 * half + j] * s0, v1 = acc1[2 * half + j] * s1;
          if (SWIGLU) { o[0] = __float2bfloat16_rn(siluf_(v0) * v1); }
          else { o[0] = __float2bfloat16_rn(v0); o[8] = __float2bfloat16_rn(v1); }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) { acc0[i] = 0.f; acc1[i] = 0.f; }
    m_c = 0; m_nb += gridDim.x; xa = xa0;
  };

  const int my_blocks = blockIdx.x < n_blocks ? (n_blocks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int iters = my_blocks * chunks;
  for (int it = 0; it < iters; it += 2) {
    fetch(cb);
    multiply(ca);
    if (it + 1 >= iters) break;
    fetch(ca);
    multiply(cb);
  }
}

template <bool SWIGLU, int U>
static cudaError_t launch_q8_variant(const Q8Args& a, dim3 grid, size_t smem, cudaStream_t stream) {
  if (smem > 48 * 1024) cudaFuncSetAttribute(q8_rows_kernel<SWIGLU, U>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  q8_rows_kernel<SWIGLU, U><<<grid, Q8_WARPS * 32, smem, stream>>>(a);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_q8_rows(const Q8Args& a, bool swiglu, cudaStream_t stream) {
  if (a.tokens <= 0) return cudaSuccess;
  const int groups = a.E + (a.x_shared ? 1 : 0);
  // gate|up: two column blocks (of 64 hidden columns) per CTA, so the token tile is staged once for
  // twice the weight stream; the down projection has 128 output columns per block and few blocks
  const int nblocks = ceil_div(a.N, (swiglu ? 8 : 16) * Q8_WARPS);
  const dim3 grid(swiglu ? ceil_div(nblocks, 2) : nblocks, ceil_div(a.tokens, Q8_ROWS), groups);
  const size_t smem = (size_t)(Q8_ROWS / 2) * (a.K / 4 + 1) * 16;
  const bool deep = a.K % (Q8_CHUNK * 4) == 0;   // K is always a multiple of 64
  if (swiglu) return deep ? launch_q8_variant<true, 4>(a, grid, smem, stream) : launch_q8_variant<true, 1>(a, grid, smem, stream);
  return deep ? launch_q8_variant<false, 4>(a, grid, smem, stream) : launch_q8_variant<false, 1>(a, grid, smem, stream);
}

}  // namespace moe
