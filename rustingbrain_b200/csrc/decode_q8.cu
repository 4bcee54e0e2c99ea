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
// byte's sign bit flipped (v + 128 as an unsigned byte; the library stores the int8 matrices that
// way, see pack_q8_kernel); a byte permute drops two of those bytes
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

// bf16 reaches 3.4e38, f16 ends at 65504: an activation beyond that SATURATES to +-65504 here instead of
// becoming an infinity (a NaN stays a NaN).  A normalised transformer's activations are orders of magnitude
// below the limit, so the clamp changes no result that was finite before; it keeps one outlier from turning
// a whole output row into inf / NaN.
__device__ __forceinline__ float clamp_f16_range(float x) { return fabsf(x) > 65504.f ? copysignf(65504.f, x) : x; }
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t v) {
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&v);
  const __half2 h = __floats2half2_rn(clamp_f16_range(__low2float(b)), clamp_f16_range(__high2float(b)));
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Work list.  An item is one 16-row token tile of one group (an expert, or the shared expert over
// all tokens) times one block of output columns; items are numbered tile-major, so neighbours share
// their token tile.  The grid is two CTAs per SM whatever the routing turned out to be; CTA c takes
// the contiguous item range [c n / grid, (c + 1) n / grid) and stages a token tile only when it changes.
//
// A warp owns two 8-column MMA tiles that share the token fragments: for the fused pass the gate
// rows of 8 hidden columns and the matching up rows, otherwise 16 adjacent output columns.
// U = 16-byte loads per lane and tile in one chunk of 64 U reduction values; K is a multiple of 64 U.
template <bool SWIGLU, int U>
__global__ void __launch_bounds__(Q8_WARPS * 32, 2) q8_rows_kernel(Q8Args a) {
  pdl_enter();
  extern __shared__ __align__(16) unsigned char q8_smem[];
  __shared__ int tile_start[MAX_EXPERTS + 2];   // first token tile of every group
  // Token tile in MMA-fragment order: rows r and r + 8 are interleaved so that one 16-byte unit holds
  // the four A registers of a lane, {x[r][k..k+1], x[r+8][k..k+1], x[r][k+2..k+3], x[r+8][k+2..k+3]} for a
  // group of four reduction values.  Row pair r has K/4 units plus one unit of padding, and units 8..15 of
  // every 16 swap their 2-unit halves: the four quarter-chunks a quarter-warp reads then fall into
  // different banks.
  const int K = a.K;
  const int pitch = (K / 4 + 1) * 16;   // bytes per row pair
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31, gq = lane >> 2, q = lane & 3;
  const int G = a.E + (a.x_shared ? 1 : 0);
  // the counts are read by one thread each (one load latency, not one per group), then scanned in place
  for (int g = tid; g < G; g += Q8_WARPS * 32) tile_start[g + 1] = ceil_div(g < a.E ? a.counts[g] : a.tokens, Q8_ROWS);
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int g = 0; g < G; ++g) {
      const int n = tile_start[g + 1];
      tile_start[g] = run;
      run += n;
    }
    tile_start[G] = run;
  }
  __syncthreads();

  constexpr int COLS = SWIGLU ? 8 : 16;               // output columns per warp
  constexpr int STEP = Q8_CHUNK * U;                  // reduction values per chunk
  const int chunks = K / STEP;
  const int n_blocks = ceil_div(a.N, COLS * Q8_WARPS);
  const long long n_items = (long long)tile_start[G] * n_blocks;
  const int i0 = (int)(n_items * blockIdx.x / gridDim.x), i1 = (int)(n_items * (blockIdx.x + 1) / gridDim.x);
  if (i0 >= i1) return;
  const int n0_warp = warp * COLS;
  const size_t tile1 = (size_t)(SWIGLU ? GU_BLOCK : 8) * K;   // second tile's rows relative to the first

  // A cursor walks the items of this CTA: (token tile, its group, column block).
  struct Cursor { int item, tile, g, nb, c; };
  auto seek = [&](Cursor& cu, int item) {
    cu.item = item;
    cu.c = 0;
    if (item >= i1) return;
    cu.tile = item / n_blocks;
    cu.nb = item - cu.tile * n_blocks;
    while (tile_start[cu.g + 1] <= cu.tile) ++cu.g;   // items only move forward
  };
  // weights are stored in blocks of 8 rows x 64 reduction values (512 contiguous bytes): lane l reads
  // bytes [16 l, 16 l + 16) of a block = row l / 4, reduction values 16 (l % 4) .. + 15
  auto stripe = [&](const Cursor& cu) -> const int8_t* {
    const int n0 = cu.nb * Q8_WARPS * COLS + n0_warp;
    if (cu.item >= i1 || n0 >= a.N) return nullptr;   // warp-uniform
    return a.w + (size_t)cu.g * a.w_group_stride + (size_t)(SWIGLU ? gu_row(0, n0) : n0) * K + 16 * lane;
  };
  struct Chunk { uint4 w[U], u[U]; };
  // The weight stream does not depend on the tokens: two register sets alternate so that the loads
  // of the next chunk are in flight while this one is multiplied, across item boundaries too, and the
  // first chunk is requested before the first token tile is staged.
  Cursor fc{0, 0, 0, 0, 0};
  seek(fc, i0);
  const int8_t* fp = stripe(fc);
  auto fetch = [&](Chunk& ch) {
    if (fp) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        ch.w[u] = __ldg(reinterpret_cast<const uint4*>(fp + 512 * u));
        ch.u[u] = __ldg(reinterpret_cast<const uint4*>(fp + tile1 + 512 * u));
      }
      fp += 512 * U;
    }
    if (++fc.c == chunks) { seek(fc, fc.item + 1); fp = stripe(fc); }
  };
  Chunk ca, cb;
  fetch(ca);

  Cursor mc{0, 0, 0, 0, 0};
  seek(mc, i0);
  int staged_tile = -1, mrows = 0;
  bf16* out = nullptr;
  const float* sc = nullptr;
  // this lane's fragments: unit (k / 4) of row pair gq; for quarter-chunks 2 and 3 the halves are swapped
  const unsigned char* xa0 = q8_smem + gq * pitch + (4 * q) * 16;
  const int sw = (q & 2) ? 32 : 0;
  const unsigned char* xa = xa0;              // compute cursor into the token tile
  float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};

  // Stages the token tile of the compute cursor (all threads; only when the tile changes).
  auto stage_tile = [&]() {
    const int g = mc.g, m0 = (mc.tile - tile_start[g]) * Q8_ROWS;
    int rows;
    const bf16* xin;
    const int* xidx = nullptr;                        // rows gathered through an index (routed rows of the first pass)
    if (g < a.E) {
      rows = a.counts[g];
      const size_t base = (size_t)a.pad_off[g];
      xin = a.x_rows + (base + m0) * K;
      if (a.x_row_index) { xin = a.x_rows; xidx = a.x_row_index + base + m0; }
      out = a.out_rows + (base + m0) * a.ldo;
    } else {
      rows = a.tokens;
      xin = a.x_shared + (size_t)m0 * K;
      out = a.out_shared + (size_t)m0 * a.ldo;
    }
    mrows = min(Q8_ROWS, rows - m0);
    sc = a.scale + (size_t)g * a.s_group_stride;
    __syncthreads();                                  // everyone is done with the previous tile
    // four independent 16-byte loads in flight per thread (both weight register sets are live here),
    // converted bf16 -> f16 on the way in
    constexpr int SU = 4;
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
        if (r < mrows) v[u] = *reinterpret_cast<const uint4*>(xin + (size_t)(xidx ? xidx[r] : r) * K + c * 8);
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
    __syncthreads();
    staged_tile = mc.tile;
  };

  auto multiply = [&](const Chunk& ch) {
    if (mc.c == 0 && mc.tile != staged_tile) stage_tile();   // uniform over the CTA
    const int n0 = mc.nb * Q8_WARPS * COLS + n0_warp;
    const bool live = n0 < a.N;              // warp-uniform
    if (live) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        // stored with the sign bit already flipped (see s8x2_to_f16x2)
        const uint32_t ww[4] = {ch.w[u].x, ch.w[u].y, ch.w[u].z, ch.w[u].w};
        const uint32_t uu[4] = {ch.u[u].x, ch.u[u].y, ch.u[u].z, ch.u[u].w};
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          // the A registers of reduction values k + 4s .. k + 4s + 3, rows gq and gq + 8, in one load
          const uint4 f = *reinterpret_cast<const uint4*>((s < 2 ? xa + sw : xa + (32 - sw)) + u * (Q8_CHUNK * 4) + (s & 1) * 16);
          mma_f16_16816(acc0, f.x, f.y, f.z, f.w, s8x2_to_f16x2(ww[s], 0), s8x2_to_f16x2(ww[s], 2));
          mma_f16_16816(acc1, f.x, f.y, f.z, f.w, s8x2_to_f16x2(uu[s], 0), s8x2_to_f16x2(uu[s], 2));
        }
      }
    }
    xa += STEP * 4;   // 16 bytes per four reduction values
    if (++mc.c < chunks) return;
    // last chunk of an item: scale, activate, store.
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
          bf16* o = out + (size_t)r * a.ldo + col;
          const float v0 = acc0[2 * half + j] * s0, v1 = acc1[2 * half + j] * s1;
          if (SWIGLU) { o[0] = __float2bfloat16_rn(siluf_(v0) * v1); }
          else { o[0] = __float2bfloat16_rn(v0); o[8] = __float2bfloat16_rn(v1); }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) { acc0[i] = 0.f; acc1[i] = 0.f; }
    seek(mc, mc.item + 1);
    xa = xa0;
  };

  const int iters = (i1 - i0) * chunks;
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
  launch_kernel(q8_rows_kernel<SWIGLU, U>, grid, dim3(Q8_WARPS * 32), smem, stream, a);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_q8_rows(const Q8Args& a, bool swiglu, cudaStream_t stream) {
  if (a.tokens <= 0) return cudaSuccess;
  // two CTAs per SM (registers and, for the down projection, shared memory allow no more); the work
  // list is cut on the device, where the routing counts are
  const dim3 grid(2 * a.sm_count);
  const size_t smem = (size_t)(Q8_ROWS / 2) * (a.K / 4 + 1) * 16;
  const bool deep = a.K % (Q8_CHUNK * 4) == 0;   // K is always a multiple of 64
  if (swiglu) return deep ? launch_q8_variant<true, 4>(a, grid, smem, stream) : launch_q8_variant<true, 1>(a, grid, smem, stream);
  return deep ? launch_q8_variant<false, 4>(a, grid, smem, stream) : launch_q8_variant<false, 1>(a, grid, smem, stream);
}

}  // namespace moe
