// int8-weight expert projections for decode-sized batches on the 5th-generation tensor cores.
//
// Same contract as decode_q8.cu (y[t, r] = dot(x[t, :], q[r, :]) * scale[r], reference
// quantized.rs:55-99, SwiGLU fused into the gate|up pass).  That kernel feeds mma.sync and is bound by
// instruction issue: widening 16 int8 weights costs as many instructions as the four small MMAs that
// consume them, on top of fragment loads and address arithmetic.  Here the weights are the 128-row
// operand of tcgen05.mma (A: 128 output columns x 64 reduction values per stage, widened int8 -> f16 by
// eight converter warps and written into shared memory in the canonical 128-byte-swizzled K-major
// layout), the tokens the 16-column operand (B: 16 token rows, brought in once per token tile by TMA
// as bf16 and rewritten in place as f16), the accumulator 128 lanes x 16 columns of tensor memory.  One MMA instruction then covers
// 128 x 16 weights; per 16 weights a converter lane spends 16 widening instructions and two 16-byte
// shared-memory stores and nothing else.
//
// Roles (448 threads): warps 0-3 epilogue (one per TMEM lane quarter), warp 4 control (lane 0 issues the
// token TMA loads and the MMAs; the warp owns the TMEM allocation), warps 5-12 converters, warp 13 weight
// loader (TMA brings the int8 bytes, as stored, into a deep shared-memory ring: up to 96 KiB in flight
// per SM, which is what covers DRAM latency; the converters read that ring, not global memory).
// Work list as in decode_q8.cu: item = (16-row token tile of one group, block of 128 output columns),
// tile-major, one contiguous range per CTA, one CTA per SM.  Every mbarrier wait is bounded.

#include <cuda.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "kernels.cuh"

namespace moe {

namespace {

constexpr int TM = 128;          // output columns per item = MMA M = TMEM lanes
constexpr int TN = 16;           // token rows per tile = MMA N
constexpr int KS = 64;           // reduction values per stage (128 bytes of f16 / bf16 per row)
constexpr int QSTAGES = 2;        // widened (f16) stages between the converters and the MMA
constexpr int RAW_BYTES_TOTAL = 96 * 1024;   // int8 bytes in flight per SM (TMA ring), split into stages
constexpr int MAX_RSTAGES = 12;
constexpr int CONV_WARPS = 8;
constexpr int LOADER_WARP = 5 + CONV_WARPS;
constexpr int Q_THREADS = 32 * (4 + 1 + CONV_WARPS + 1);
constexpr int A_TILE_BYTES = TM * KS * 2;    // 16 KiB
constexpr int B_BOX_BYTES = TN * KS * 2;     // 2 KiB
constexpr int TMEM_COLS_Q = 64;
constexpr long long WAIT_LIMIT = 3000000000LL;   // ~1.5 s

struct __align__(8) QTail {
  unsigned long long full[QSTAGES];
  unsigned long long empty[QSTAGES];
  unsigned long long raw_full[MAX_RSTAGES];
  unsigned long long raw_empty[MAX_RSTAGES];
  unsigned long long tmem_full[2];
  unsigned long long tmem_empty[2];
  unsigned long long b_full;    // token tile landed (TMA, bf16)
  unsigned long long b_ready;   // token tile rewritten as f16 by the epilogue warps
  unsigned long long mma_done;
  uint32_t tmem_base;
  int dead;
  int tile_start[MAX_EXPERTS + 2];
  int rows_of[MAX_EXPERTS + 1];   // token rows of every group
  int row0_of[MAX_EXPERTS + 1];   // first row of every group in its row buffer
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait: false (and `code` in the flag) when the limit passes or another role already failed.
__device__ __noinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* error_flag, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 0xfff) == 0) {
      if (*(volatile int*)error_flag != 0) return false;
      if (clock64() - t0 > WAIT_LIMIT) {
        atomicCAS(error_flag, 0, code);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 16 consecutive fp32 columns: thread i receives lane (quarter base + i), register j = column j.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// K-major operand, 128-byte rows, 128-byte swizzle: 8-row atoms 1024 bytes apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffff) >> 4);
  d |= (uint64_t)(16 >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version for sm_100
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}
// kind::f16, fp32 accumulate, A and B = f16 (an f16 A with a bf16 B is refused by the hardware as an
// illegal instruction, although the descriptor has one format field per operand), both K-major, M 128, N 16.
constexpr uint32_t Q_IDESC = (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);

// Two stored weight bytes (sign bit already flipped, see pack_q8_kernel) -> two f16 values.
__device__ __forceinline__ uint32_t widen2(uint32_t wx, int lo_byte) {
  const uint32_t packed = __byte_perm(wx, 0x64646464u, lo_byte == 0 ? 0x4140 : 0x4342);
  const __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&packed), __half2half2(__ushort_as_half(0x6480)));
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float siluf_tc(float x) { return x / (1.f + __expf(-x)); }

struct ItemInfo { int tile, g, nb, m0, mrows; long long row0; };

template <bool SWIGLU>
__global__ void __launch_bounds__(Q_THREADS, 1)
q8_tc_kernel(const __grid_constant__ CUtensorMap map_rows, const __grid_constant__ CUtensorMap map_shared,
             const __grid_constant__ CUtensorMap map_w, int rstages, Q8Args a) {
  extern __shared__ unsigned char q8tc_smem_raw[];
  constexpr int TILES = SWIGLU ? 2 : 1;
  constexpr int ACC_COLS = 16 * TILES;
  constexpr int RAW_STAGE = TILES * TM * KS;      // int8 bytes of one stage: TILES x 16 stripes of 512 bytes
  const int K = a.K, kstages = K / KS;
  const uint32_t raw = smem_u32(q8tc_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* gbase = q8tc_smem_raw + (base - raw);
  const uint32_t b_base = base;                                   // tokens: kstages boxes of 2 KiB
  const uint32_t ring = b_base + (uint32_t)kstages * B_BOX_BYTES; // QSTAGES x TILES x 16 KiB of f16
  const size_t raw_off = (size_t)kstages * B_BOX_BYTES + (size_t)QSTAGES * TILES * A_TILE_BYTES;
  const uint32_t raw_base = base + (uint32_t)raw_off;             // rstages x RAW_STAGE of int8, as stored
  QTail* st = reinterpret_cast<QTail*>(gbase + raw_off + (size_t)rstages * RAW_STAGE);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = a.E + (a.x_shared ? 1 : 0);

  for (int g = threadIdx.x; g < G; g += Q_THREADS) {
    const int rows = g < a.E ? a.counts[g] : a.tokens;
    st->rows_of[g] = rows;
    st->row0_of[g] = g < a.E ? a.pad_off[g] : 0;
    st->tile_start[g + 1] = ceil_div(rows, TN);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int g = 0; g < G; ++g) {   // counts -> starts, in place
      const int n = st->tile_start[g + 1];
      st->tile_start[g] = run;
      run += n;
    }
    st->tile_start[G] = run;
    for (int s = 0; s < QSTAGES; ++s) {
      mbar_init(smem_u32(&st->full[s]), CONV_WARPS);
      mbar_init(smem_u32(&st->empty[s]), 1);
    }
    for (int s = 0; s < rstages; ++s) {
      mbar_init(smem_u32(&st->raw_full[s]), 1);
      mbar_init(smem_u32(&st->raw_empty[s]), CONV_WARPS);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&st->tmem_full[i]), 1);
      mbar_init(smem_u32(&st->tmem_empty[i]), 4);
    }
    mbar_init(smem_u32(&st->b_full), 1);
    mbar_init(smem_u32(&st->b_ready), 4);
    mbar_init(smem_u32(&st->mma_done), 1);
    st->dead = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 4) tmem_alloc(smem_u32(&st->tmem_base), TMEM_COLS_Q);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = st->tmem_base;

  const int n_blocks = ceil_div(a.N, TM);
  const long long n_items = (long long)st->tile_start[G] * n_blocks;
  const int i0 = (int)(n_items * blockIdx.x / gridDim.x), i1 = (int)(n_items * (blockIdx.x + 1) / gridDim.x);

  // every role walks the same items
  auto locate = [&](int item, int& g_hint) {
    ItemInfo it;
    it.tile = item / n_blocks;
    it.nb = item - it.tile * n_blocks;
    while (st->tile_start[g_hint + 1] <= it.tile) ++g_hint;
    it.g = g_hint;
    it.m0 = (it.tile - st->tile_start[it.g]) * TN;
    it.mrows = min(TN, st->rows_of[it.g] - it.m0);
    it.row0 = (long long)st->row0_of[it.g] + it.m0;
    return it;
  };

  if (warp == LOADER_WARP) {
    if (lane == 0) {
      // ------------------------- weight loads (TMA, int8 as stored) -----------------------
      // The arena is a matrix of 8-row stripes: stripe s = 8 K contiguous bytes, 512 per 64 reduction
      // values.  One box = 512 bytes x (TILES x 16) stripes = the 128 columns (gate and up) of one stage.
      // The loader runs up to `rstages` stages ahead, across items, which is what keeps enough bytes in
      // flight to cover DRAM latency.
      const int stripes_per_group = (int)(a.w_group_stride / (8ll * K));
      uint32_t rs = 0, rphase = 0;
      int g_hint = 0;
      bool ok = true;
      for (int item = i0; item < i1 && ok; ++item) {
        const ItemInfo it = locate(item, g_hint);
        const int n0 = it.nb * TM;
        const int stripe0 = it.g * stripes_per_group + (SWIGLU ? (n0 / GU_BLOCK) * (2 * GU_BLOCK / 8) : n0 / 8);
        for (int kb = 0; kb < kstages; ++kb) {
          if (!mbar_wait(smem_u32(&st->raw_empty[rs]), rphase ^ 1, a.error_flag, 208)) { ok = false; break; }
          const uint32_t bar = smem_u32(&st->raw_full[rs]);
          mbar_expect_tx(bar, RAW_STAGE);
          tma_load_2d(raw_base + rs * RAW_STAGE, &map_w, bar, kb * (512 / 4), stripe0);
          if (++rs == (uint32_t)rstages) { rs = 0; rphase ^= 1; }
        }
      }
      if (!ok) st->dead = 1;
    }
    __syncwarp();
  } else if (warp >= 5) {
    // ------------------------------- converters ---------------------------------
    // Warp cw owns rows 16 cw .. 16 cw + 15 of the 128-row weight tile = two stored blocks of 8 rows x 64
    // reduction values (512 contiguous bytes: lane l holds row l / 4, values 16 (l % 4) .. + 15).
    const int cw = warp - 5, gq = lane >> 2, q = lane & 3;
    // stripe of block j inside the stage's box: gate and up stripes alternate in fours (32 columns)
    int stripe[TILES][2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int c8 = 2 * cw + j;   // 8-column block of the 128
#pragma unroll
      for (int t = 0; t < TILES; ++t) stripe[t][j] = SWIGLU ? (c8 / 4) * 8 + t * 4 + (c8 % 4) : c8;
    }
    uint32_t stage = 0, phase = 0, rs = 0, rphase = 0;
    bool ok = true;
    const long long n_stages = (long long)(i1 - i0) * kstages;
    for (long long sidx = 0; sidx < n_stages; ++sidx) {
      if (!mbar_wait(smem_u32(&st->raw_full[rs]), rphase, a.error_flag, 209)) { ok = false; break; }
      uint4 w[TILES][2];
      const unsigned char* rawp = gbase + raw_off + (size_t)rs * RAW_STAGE + 16 * lane;
#pragma unroll
      for (int t = 0; t < TILES; ++t)
#pragma unroll
        for (int j = 0; j < 2; ++j) w[t][j] = *reinterpret_cast<const uint4*>(rawp + stripe[t][j] * 512);
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&st->raw_empty[rs]));     // the bytes are in registers
      if (++rs == (uint32_t)rstages) { rs = 0; rphase ^= 1; }
      if (!mbar_wait(smem_u32(&st->empty[stage]), phase ^ 1, a.error_flag, 201)) { ok = false; break; }
#pragma unroll
      for (int t = 0; t < TILES; ++t) {
        unsigned char* tile = gbase + (size_t)kstages * B_BOX_BYTES + ((size_t)stage * TILES + t) * A_TILE_BYTES;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int r = 16 * cw + 8 * j + gq;            // row of the tile; r & 7 == gq
          const uint4 v = w[t][j];
          const uint4 lo = make_uint4(widen2(v.x, 0), widen2(v.x, 2), widen2(v.y, 0), widen2(v.y, 2));
          const uint4 hi = make_uint4(widen2(v.z, 0), widen2(v.z, 2), widen2(v.w, 0), widen2(v.w, 2));
          // 16-byte chunks 2q and 2q + 1 of the row, XOR-swizzled with the row inside its 8-row atom
          unsigned char* row = tile + r * 128;
          *reinterpret_cast<uint4*>(row + (((2 * q) ^ gq) << 4)) = lo;
          *reinterpret_cast<uint4*>(row + (((2 * q + 1) ^ gq) << 4)) = hi;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> visible to the MMA
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&st->full[stage]));
      if (++stage == QSTAGES) { stage = 0; phase ^= 1; }
    }
    if (!ok && lane == 0) st->dead = 1;
  } else if (warp == 4) {
    if (lane == 0) {
      // --------------------- token loads (TMA) and MMA issue -----------------------
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0, b_phase = 0, done_phase = 0;
      int g_hint = 0, staged_tile = -1, pending_done = 0;
      bool ok = true;
      for (int item = i0; item < i1 && ok; ++item) {
        const ItemInfo it = locate(item, g_hint);
        if (it.tile != staged_tile) {
          if (pending_done) {   // the MMAs that read the previous token tile have finished
            if (!mbar_wait(smem_u32(&st->mma_done), done_phase, a.error_flag, 202)) { ok = false; break; }
            done_phase ^= 1;
            pending_done = 0;
          }
          const uint32_t bar = smem_u32(&st->b_full);
          mbar_expect_tx(bar, (uint32_t)kstages * B_BOX_BYTES);
          const CUtensorMap* map = it.g < a.E ? &map_rows : &map_shared;
          for (int kb = 0; kb < kstages; ++kb) tma_load_2d(b_base + kb * B_BOX_BYTES, map, bar, kb * KS, (int)it.row0);
          if (!mbar_wait(smem_u32(&st->b_ready), b_phase, a.error_flag, 203)) { ok = false; break; }
          tc_fence_after();
          b_phase ^= 1;
          staged_tile = it.tile;
        }
        if (!mbar_wait(smem_u32(&st->tmem_empty[acc]), acc_phase ^ 1, a.error_flag, 204)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        for (int kb = 0; kb < kstages; ++kb) {
          if (!mbar_wait(smem_u32(&st->full[stage]), phase, a.error_flag, 205)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sb = b_base + kb * B_BOX_BYTES;
#pragma unroll
          for (int t = 0; t < TILES; ++t) {
            const uint32_t sa = ring + (stage * TILES + t) * A_TILE_BYTES;
#pragma unroll
            for (int kk = 0; kk < KS / 16; ++kk)
              umma_f16(d_tmem + t * 16, make_desc(sa + kk * 32), make_desc(sb + kk * 32), Q_IDESC, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&st->empty[stage]));   // frees the stage once these MMAs have read it
          if (++stage == QSTAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(smem_u32(&st->tmem_full[acc]));
        // the next item may bring a new token tile: its load has to wait for these MMAs
        int g2 = g_hint;
        if (item + 1 < i1 && locate(item + 1, g2).tile != it.tile) { umma_commit(smem_u32(&st->mma_done)); pending_done = 1; }
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok) st->dead = 1;
    }
    __syncwarp();
  } else {
    // -------------------------------- epilogue ----------------------------------
    // warp w reads TMEM lanes 32 w .. 32 w + 31 = output columns n0 + 32 w + lane, 16 tokens each
    uint32_t acc = 0, acc_phase = 0, b_phase = 0;
    int g_hint = 0, staged_tile = -1;
    bool ok = true;
    for (int item = i0; item < i1 && ok; ++item) {
      const ItemInfo it = locate(item, g_hint);
      if (it.tile != staged_tile) {
        // The tokens arrive as bf16; both MMA operands have to be f16, so rewrite the tile in place
        // (element by element, which leaves the swizzled layout as it is) and hand it to the issuer.
        if (!mbar_wait(smem_u32(&st->b_full), b_phase, a.error_flag, 207)) { ok = false; break; }
        b_phase ^= 1;
        uint4* bt = reinterpret_cast<uint4*>(gbase);
        for (int i = threadIdx.x; i < kstages * (B_BOX_BYTES / 16); i += 128) {
          uint4 v = bt[i];
          uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[c]));
            // saturate at the end of the f16 range instead of overflowing to infinity (as the mma.sync kernel does)
            f.x = fabsf(f.x) > 65504.f ? copysignf(65504.f, f.x) : f.x;
            f.y = fabsf(f.y) > 65504.f ? copysignf(65504.f, f.y) : f.y;
            const __half2 h = __float22half2_rn(f);
            w[c] = *reinterpret_cast<const uint32_t*>(&h);
          }
          bt[i] = v;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&st->b_ready));
        staged_tile = it.tile;
      }
      if (!mbar_wait(smem_u32(&st->tmem_full[acc]), acc_phase, a.error_flag, 206)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + acc * ACC_COLS;
      float v0[16], v1[16];
      tmem_ld16(taddr, v0);
      if (SWIGLU) tmem_ld16(taddr + 16, v1);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&st->tmem_empty[acc]));   // the values are in registers
      const int col = it.nb * TM + warp * 32 + lane;
      if (col < a.N) {
        const float* sc = a.scale + (size_t)it.g * a.s_group_stride;
        const float s0 = SWIGLU ? sc[gu_row(0, col)] : sc[col];
        const float s1 = SWIGLU ? sc[gu_row(1, col)] : 0.f;
        bf16* out = (it.g < a.E ? a.out_rows : a.out_shared) + it.row0 * a.ldo + col;
#pragma unroll
        for (int t = 0; t < TN; ++t) {
          if (t < it.mrows) {
            float v = v0[t] * s0;
            if (SWIGLU) v = siluf_tc(v) * (v1[t] * s1);
            out[(size_t)t * a.ldo] = __float2bfloat16_rn(v);
          }
        }
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  __syncthreads();
  if (st->dead || *(volatile int*)a.error_flag != 0) {
    // failure path: let copies that may still be in flight land before shared and tensor memory go away
    const long long t0 = clock64();
    while (clock64() - t0 < 4000000LL) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS_Q);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      return (EncodeTiledFn)p;
    return (EncodeTiledFn) nullptr;
  }();
  return fn;
}

// bf16 [rows, K] row-major, boxes of 64 reduction values x 16 rows, 128-byte swizzle, zero fill outside.
bool token_map(CUtensorMap* map, const void* ptr, long long rows, int K) {
  EncodeTiledFn fn = encode_fn();
  if (!fn || !ptr || rows <= 0) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {(cuuint32_t)KS, (cuuint32_t)TN};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// int8 arena as [stripes, 2 K] 32-bit words (a stripe = 8 stored rows = 8 K bytes), boxes of 512 bytes x
// `box_stripes` stripes, no swizzle, zero fill past the last stripe.
bool weight_map(CUtensorMap* map, const void* ptr, long long stripes, int K, int box_stripes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn || !ptr || stripes <= 0) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K * 2, (cuuint64_t)stripes};
  cuuint64_t strides[1] = {(cuuint64_t)K * 8};
  cuuint32_t box[2] = {128, (cuuint32_t)box_stripes};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

constexpr size_t SMEM_BUDGET = 225 * 1024;
size_t fixed_smem(const Q8Args& a, bool swiglu) {
  return (size_t)(a.K / KS) * B_BOX_BYTES + (size_t)QSTAGES * (swiglu ? 2 : 1) * A_TILE_BYTES + 1024 + sizeof(QTail);
}
int raw_stages(const Q8Args& a, bool swiglu) {
  const size_t stage = (size_t)(swiglu ? 2 : 1) * TM * KS, fixed = fixed_smem(a, swiglu);
  if (fixed + 2 * stage > SMEM_BUDGET) return 0;
  const size_t room = std::min((size_t)RAW_BYTES_TOTAL, SMEM_BUDGET - fixed);
  return (int)std::min<size_t>(MAX_RSTAGES, room / stage);
}

template <bool SWIGLU>
cudaError_t launch_variant(const CUtensorMap& mr, const CUtensorMap& ms, const CUtensorMap& mw, const Q8Args& a,
                           cudaStream_t stream) {
  constexpr int TILES = SWIGLU ? 2 : 1;
  const int rstages = raw_stages(a, SWIGLU);
  const size_t smem = fixed_smem(a, SWIGLU) + (size_t)rstages * TILES * TM * KS;
  cudaError_t e = cudaFuncSetAttribute(q8_tc_kernel<SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  q8_tc_kernel<SWIGLU><<<a.sm_count, Q_THREADS, smem, stream>>>(mr, ms, mw, rstages, a);
  count_launch();
  return cudaGetLastError();
}

}  // namespace

// True when the tensor-core variant can take this problem.
bool q8_tc_supported(const Q8Args& a, bool swiglu) {
  const bool aligned = ((uintptr_t)a.x_rows & 15) == 0 && ((uintptr_t)a.x_shared & 15) == 0 && ((uintptr_t)a.w & 15) == 0;
  // whole stripes per group and whole 32-column gate|up blocks per 128-column item
  const bool shaped = a.K % KS == 0 && a.K >= KS && a.N % GU_BLOCK == 0 && a.w_group_stride % (8ll * a.K) == 0;
  return shaped && raw_stages(a, swiglu) >= 2 && a.error_flag != nullptr && a.x_rows_cap > 0 && aligned &&
         (!a.x_shared || a.x_shared_rows > 0);
}

cudaError_t launch_q8_rows_tc(const Q8Args& a, bool swiglu, cudaStream_t stream) {
  if (a.tokens <= 0) return cudaSuccess;
  CUtensorMap mr, ms;
  if (!token_map(&mr, a.x_rows, a.x_rows_cap, a.K)) return cudaErrorInvalidValue;
  if (a.x_shared) {
    if (!token_map(&ms, a.x_shared, a.x_shared_rows, a.K)) return cudaErrorInvalidValue;
  } else {
    ms = mr;
  }
  const int groups = a.E + (a.x_shared ? 1 : 0);
  CUtensorMap mw;
  if (!weight_map(&mw, a.w, (long long)groups * (a.w_group_stride / (8ll * a.K)), a.K, swiglu ? 32 : 16)) return cudaErrorInvalidValue;
  return swiglu ? launch_variant<true>(mr, ms, mw, a, stream) : launch_variant<false>(mr, ms, mw, a, stream);
}

}  // namespace moe
