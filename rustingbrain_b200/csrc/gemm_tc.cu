// Grouped bf16 GEMMs on the Blackwell tensor cores (sm_100a): tcgen05.mma with
// fp32 accumulators in tensor memory, operands staged in shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle), one persistent CTA per SM.
//
// Warp roles inside a CTA of 320 threads:
//   warp 0, one lane : TMA producer (fills a 4-stage ring of A/B tiles)
//   warp 1           : allocates tensor memory; one lane issues tcgen05.mma and
//                      tcgen05.commit
//   warps 2..9       : epilogue; two warps per quarter of the 128 TMEM lanes, each takes
//                      half of the tile's columns: tcgen05.ld, fused pointwise step, stores.
// Two 128x256 fp32 accumulators (all 512 TMEM columns) are double buffered so the
// epilogue of tile i overlaps the MMAs of tile i+1.
//
// The row groups (one per expert) are padded to multiples of 128 rows by the
// dispatch step, so every M tile lies inside one group and the ragged sizes never
// reach the tensor-core loop; only the tile schedule reads them, from device memory.
//
// Every wait on an mbarrier is bounded: after about a second it records an error
// code in GemmArgs::error_flag, the CTA drains and frees its tensor memory, and
// the host reports ST_TIMEOUT.

#include "gemm_tc.cuh"

#include <stdio.h>
#include <stdlib.h>

namespace moe {
namespace tc {

constexpr int STAGES = 4;          // depth of the operand ring (one-SM tiles)
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;           // 16 KiB
constexpr int B_BYTES = BN * BK * 2;           // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES; // 48 KiB
constexpr int BOX_BYTES = 64 * 64 * 2;         // one 64x64 box of an MN-major operand
constexpr int MAX_GROUPS = MAX_EXPERTS + 1;
constexpr int EPI_WARPS = 8;
constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;
constexpr int TMEM_COLS = 512;
constexpr long long WAIT_LIMIT_CYCLES = 3000000000LL;  // ~1.5 s at 2 GHz

struct __align__(8) SharedTail {
  unsigned long long full[STAGES];
  unsigned long long empty[STAGES];
  unsigned long long tmem_full[2];
  unsigned long long tmem_empty[2];
  uint32_t tmem_base;
  int dead;
  int row0[MAX_GROUPS + 1];
  int tstart[MAX_GROUPS + 1];
};

constexpr int STG_TOTAL = 8 * 32 * 80;   // epilogue staging, see STG_* below
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STG_TOTAL + 1024 /*alignment slack*/ + (int)sizeof(SharedTail);

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
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
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(20000u)   // the thread may stay suspended for up to 20 microseconds per try
      : "memory");
  return ok;
}
// Bounded wait.  Returns false (and records `code`) when the limit passes or
// another role of this grid has already reported a failure.
__device__ __noinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* error_flag, int code, long long limit) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 0xff) == 0) {
      if (*(volatile int*)error_flag != 0) return false;
      if (clock64() - t0 > limit) {
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
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], M=128, N=256, K=16, bf16 in, fp32 out.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier gets one arrival once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives row
// (lane quarter base + i), registers j = column (col0 + j).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor (sm_100 format): start address, leading and
// stride byte offsets in 16-byte units, version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffff) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version for sm_100
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16: fp32 accumulate, bf16 A and B, M=128, N=256.
__host__ __device__ constexpr uint32_t make_idesc(bool a_mn, bool b_mn, int n) {
  return (1u << 4)                      // D format: f32
         | (1u << 7)                    // A format: bf16
         | (1u << 10)                   // B format: bf16
         | ((a_mn ? 1u : 0u) << 15)     // A major: 0 = K, 1 = MN
         | ((b_mn ? 1u : 0u) << 16)     // B major
         | ((uint32_t)(n >> 3) << 17)   // N / 8
         | ((uint32_t)(BM >> 4) << 24); // M / 16
}

// ---------------------------------------------------------------------------
// Tile schedule
// ---------------------------------------------------------------------------
struct Tile {
  int group, row0 /*first row of the row-indexed operands*/, m0, n0, k_iters;
  int skip;   // causal products: the tile lies wholly above the diagonal, nobody touches it
};

// rows-as-K causal products: does K-stage ki (64 query rows) reach the tile's keys [m0, m0 + 128)?
template <bool ROWS_ARE_K>
__device__ __forceinline__ bool k_stage_live(const GemmArgs& p, const Tile& tl, int ki) {
  if (!ROWS_ARE_K || p.causal == 0) return true;
  return (ki * BK) % p.causal + BK > tl.m0;
}

template <bool ROWS_ARE_K>
__device__ __forceinline__ int total_tiles(const SharedTail* st, const GemmArgs& p) {
  const int nt = ceil_div(p.N, BN);
  if (ROWS_ARE_K) return p.n_groups * ceil_div(p.M, BM) * nt;
  return st->tstart[p.n_groups] * nt;
}

template <bool ROWS_ARE_K>
__device__ __forceinline__ Tile decode_tile(const SharedTail* st, const GemmArgs& p, int t) {
  Tile tl;
  tl.skip = 0;
  const int nt = ceil_div(p.N, BN);
  if (ROWS_ARE_K) {
    const int mt = ceil_div(p.M, BM);
    const int g = t / (mt * nt);
    const int rem = t - g * mt * nt;
    tl.group = g;
    tl.n0 = (rem / mt) * BN;
    tl.m0 = (rem % mt) * BM;
    tl.row0 = st->row0[g];
    tl.k_iters = (st->row0[g + 1] - st->row0[g]) / BK;
  } else {
    // tiles of group g occupy [tstart[g]*nt, tstart[g+1]*nt); m varies fastest so
    // that neighbouring CTAs share the same weight tile in L2.
    int lo = 0, hi = p.n_groups;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (st->tstart[mid] * nt <= t) lo = mid; else hi = mid;
    }
    const int g = lo;
    const int mt = st->tstart[g + 1] - st->tstart[g];
    const int local = t - st->tstart[g] * nt;
    tl.group = g;
    tl.n0 = (local / mt) * BN;
    tl.m0 = 0;
    tl.row0 = st->row0[g] + (local % mt) * BM;
    tl.k_iters = ceil_div(p.K, BK);
    if (p.causal) {
      // the last query position among the tile's rows (a tile that crosses into the next head sees them all)
      const int s_first = ((local % mt) * BM) % p.causal;
      const int s_last = s_first + BM > p.causal ? p.causal - 1 : s_first + BM - 1;
      if (p.causal_kind == CAUSAL_COLS) tl.skip = tl.n0 > s_last;
      else if (p.causal_kind == CAUSAL_K) tl.k_iters = min(tl.k_iters, s_last / BK + 1);
    }
  }
  return tl;
}

// ---------------------------------------------------------------------------
// Epilogues.  `v` holds 32 consecutive accumulator columns of one row.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void store32_bf16(bf16* dst, const float* v) {
  uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int i = 0; i < 4; ++i)
    d4[i] = make_uint4(pack2(v[8 * i], v[8 * i + 1]), pack2(v[8 * i + 2], v[8 * i + 3]),
                       pack2(v[8 * i + 4], v[8 * i + 5]), pack2(v[8 * i + 6], v[8 * i + 7]));
}
__device__ __forceinline__ void load32_bf16(const bf16* src, float* v) {
  const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 q = s4[i];
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[j]);
      v[8 * i + 2 * j] = __low2float(h);
      v[8 * i + 2 * j + 1] = __high2float(h);
    }
  }
}

// Coalescing through shared memory.  tcgen05.ld hands every lane one ROW (32 columns = 64 bytes
// of bf16); storing that directly makes each warp-wide 16-byte store touch 32 different rows.
// Each epilogue warp therefore owns a 32 x 64-byte staging tile (80-byte row pitch, conflict
// free): lanes drop their row there, and the warp writes it out 8 rows x 64 contiguous bytes per
// instruction (4x fewer L1/L2 request cycles, which the TMA loads share).  Loads of the saved
// g|u rows take the same path in reverse.
constexpr int STG_PITCH = 80;
constexpr int STG_BYTES_PER_WARP = 32 * STG_PITCH;      // 2560
constexpr int STG_BYTES = EPI_WARPS * STG_BYTES_PER_WARP;

__device__ __forceinline__ void store32_bf16_staged(bf16* warp_row0_ptr, long long ld, const float* v, uint8_t* stg,
                                                    int lane) {
  uint4* mine = reinterpret_cast<uint4*>(stg + lane * STG_PITCH);
#pragma unroll
  for (int i = 0; i < 4; ++i)
    mine[i] = make_uint4(pack2(v[8 * i], v[8 * i + 1]), pack2(v[8 * i + 2], v[8 * i + 3]),
                         pack2(v[8 * i + 4], v[8 * i + 5]), pack2(v[8 * i + 6], v[8 * i + 7]));
  __syncwarp();
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int row = it * 8 + (lane >> 2), ch = lane & 3;
    const uint4 q = *reinterpret_cast<const uint4*>(stg + row * STG_PITCH + ch * 16);
    *reinterpret_cast<uint4*>(reinterpret_cast<char*>(warp_row0_ptr + (long long)row * ld) + ch * 16) = q;
  }
  __syncwarp();
}
__device__ __forceinline__ void load32_bf16_staged(const bf16* warp_row0_ptr, long long ld, float* v, uint8_t* stg,
                                                   int lane) {
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int row = it * 8 + (lane >> 2), ch = lane & 3;
    const uint4 q = *reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(warp_row0_ptr + (long long)row * ld) + ch * 16);
    *reinterpret_cast<uint4*>(stg + row * STG_PITCH + ch * 16) = q;
  }
  __syncwarp();
  load32_bf16(reinterpret_cast<const bf16*>(stg + lane * STG_PITCH), v);
  __syncwarp();
}

// 32 columns of 32 rows that a lane already holds as 16 packed bf16 pairs.
__device__ __forceinline__ void store32_packed_staged(bf16* warp_row0_ptr, long long ld, const uint32_t* pk, uint8_t* stg,
                                                      int lane) {
  uint4* mine = reinterpret_cast<uint4*>(stg + lane * STG_PITCH);
#pragma unroll
  for (int i = 0; i < 4; ++i) mine[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
  __syncwarp();
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int row = it * 8 + (lane >> 2), ch = lane & 3;
    const uint4 q = *reinterpret_cast<const uint4*>(stg + row * STG_PITCH + ch * 16);
    *reinterpret_cast<uint4*>(reinterpret_cast<char*>(warp_row0_ptr + (long long)row * ld) + ch * 16) = q;
  }
  __syncwarp();
}

// 32 f32 columns of 32 rows into out_warp (first row m_warp of a matrix with p.M rows), through the warp's staging
// tile, 16 columns (64 bytes per row) at a time: a lane holds one ROW, so direct stores would touch 32 rows per
// instruction, 16 bytes each; staged, an instruction covers 8 rows x 64 contiguous bytes (and the read-modify-write
// of the accumulate mode loads the same way).
__device__ __forceinline__ void store32_f32_staged(const GemmArgs& p, float* out_warp, int m_warp, const float* v, uint8_t* stg,
                                                   int lane) {
#pragma unroll
  for (int hseg = 0; hseg < 2; ++hseg) {
    uint4* mine = reinterpret_cast<uint4*>(stg + lane * STG_PITCH);
#pragma unroll
    for (int i = 0; i < 4; ++i)
      mine[i] = make_uint4(__float_as_uint(v[16 * hseg + 4 * i]), __float_as_uint(v[16 * hseg + 4 * i + 1]),
                           __float_as_uint(v[16 * hseg + 4 * i + 2]), __float_as_uint(v[16 * hseg + 4 * i + 3]));
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int row = it * 8 + (lane >> 2), ch = lane & 3;
      if (m_warp + row < p.M) {
        const uint4 q = *reinterpret_cast<const uint4*>(stg + row * STG_PITCH + ch * 16);
        float4 r = make_float4(__uint_as_float(q.x), __uint_as_float(q.y), __uint_as_float(q.z), __uint_as_float(q.w));
        float4* o = reinterpret_cast<float4*>(out_warp + (long long)row * p.ld0 + 16 * hseg + 4 * ch);
        if (p.accumulate) {
          const float4 old = *o;
          r.x += old.x; r.y += old.y; r.z += old.z; r.w += old.w;
        }
        *o = r;
      }
    }
    __syncwarp();
  }
}

// The tensor-core path rounds its outputs to bf16 (2^-9), so the pointwise step uses
// the fast exponential and reciprocal; the f32 path keeps expf and IEEE division.
__device__ __forceinline__ float fast_sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

template <int EPI>
__device__ __forceinline__ void epilogue_tile(const GemmArgs& p, const Tile& tl, uint32_t taddr, int row_in_tile,
                                              int c_begin, int c_end,
                                              bool have_acc, uint8_t* stg) {
  const int lane = row_in_tile & 31;
  const long long wrow = (long long)tl.row0 + (row_in_tile & ~31);   // first row of this warp
  if (EPI == EPI_STORE) {
    bf16* out = (bf16*)p.out0 + wrow * p.ld0;
#pragma unroll 1
    for (int c = c_begin; c < c_end; c += 32) {
      if (tl.n0 + c >= p.N) break;   // warp-uniform
      float v[32];
      tmem_ld32(taddr + c, v);
      store32_bf16_staged(out + tl.n0 + c, p.ld0, v, stg, lane);
    }
  } else if (EPI == EPI_SWIGLU) {
    bf16* h_out = (bf16*)p.out0 + wrow * p.ld0;
    bf16* gu_out = p.out1 ? (bf16*)p.out1 + wrow * p.ld1 : nullptr;
#pragma unroll 1
    for (int c = c_begin; c < c_end; c += 2 * GU_BLOCK) {
      if (tl.n0 + c >= p.N) break;
      float g[32], u[32];
      tmem_ld32(taddr + c, g);
      tmem_ld32(taddr + c + GU_BLOCK, u);
      if (gu_out) {
        store32_bf16_staged(gu_out + tl.n0 + c, p.ld1, g, stg, lane);
        store32_bf16_staged(gu_out + tl.n0 + c + GU_BLOCK, p.ld1, u, stg, lane);
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) g[i] = g[i] * fast_sigmoid(g[i]) * u[i];
      store32_bf16_staged(h_out + (tl.n0 + c) / 2, p.ld0, g, stg, lane);
    }
  } else if (EPI == EPI_SWIGLU_BWD) {
    // accumulator columns are logical hidden columns f; the saved (g|u) and the
    // output (dg|du) use the interleaved layout: block f/32 -> columns [64b, 64b+64).
    const bf16* gu = (const bf16*)p.aux + wrow * p.ldaux;
    bf16* out = (bf16*)p.out0 + wrow * p.ld0;
#pragma unroll 1
    for (int c = c_begin; c < c_end; c += 32) {
      if (tl.n0 + c >= p.N) break;
      float dh[32], g[32], u[32];
      tmem_ld32(taddr + c, dh);
      const int col = (tl.n0 + c) * 2;
      load32_bf16_staged(gu + col, p.ldaux, g, stg, lane);
      load32_bf16_staged(gu + col + GU_BLOCK, p.ldaux, u, stg, lane);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float s = fast_sigmoid(g[i]);
        const float dg = dh[i] * u[i] * (s * (1.0f + g[i] * (1.0f - s)));
        u[i] = dh[i] * (g[i] * s);
        g[i] = dg;
      }
      store32_bf16_staged(out + col, p.ld0, g, stg, lane);
      store32_bf16_staged(out + col + GU_BLOCK, p.ld0, u, stg, lane);
    }
  } else if (EPI == EPI_STORE_F32) {
    // f32 output with a row limit (p.M) and any column count: the router logits, and the products of the f32
    // configuration (operands split into three bf16 pieces each, see moe_api.cu).
    const long long row = (long long)tl.row0 + row_in_tile;
    float* out = (float*)p.out0 + row * p.ld0;
#pragma unroll 1
    for (int c = c_begin; c < c_end; c += 32) {
      if (tl.n0 + c >= p.N) break;
      float v[32];
      tmem_ld32(taddr + c, v);
      if (tl.n0 + c + 32 <= p.N && (p.ld0 & 3) == 0) {
        // a whole block of 32 columns: through the staging tile, 8 rows x 64 contiguous bytes per store instruction
        const long long row_warp = (long long)tl.row0 + (row_in_tile & ~31);
        float* out_warp = (float*)p.out0 + row_warp * p.ld0 + tl.n0 + c;
#pragma unroll
        for (int hseg = 0; hseg < 2; ++hseg) {
          uint4* mine = reinterpret_cast<uint4*>(stg + lane * STG_PITCH);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            mine[i] = make_uint4(__float_as_uint(v[16 * hseg + 4 * i]), __float_as_uint(v[16 * hseg + 4 * i + 1]),
                                 __float_as_uint(v[16 * hseg + 4 * i + 2]), __float_as_uint(v[16 * hseg + 4 * i + 3]));
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            const int r = it * 8 + (lane >> 2), ch = lane & 3;
            if (row_warp + r < p.M) {
              const uint4 q = *reinterpret_cast<const uint4*>(stg + r * STG_PITCH + ch * 16);
              float4 o4 = make_float4(__uint_as_float(q.x), __uint_as_float(q.y), __uint_as_float(q.z), __uint_as_float(q.w));
              float4* dst = reinterpret_cast<float4*>(out_warp + (long long)r * p.ld0 + 16 * hseg + 4 * ch);
              if (p.accumulate) {   // f32 addition on the CUDA cores, round to nearest
                const float4 old = *dst;
                o4.x += old.x; o4.y += old.y; o4.z += old.z; o4.w += old.w;
              }
              *dst = o4;
            }
          }
          __syncwarp();
        }
      } else if (row < p.M) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (tl.n0 + c + i < p.N) out[tl.n0 + c + i] = p.accumulate ? out[tl.n0 + c + i] + v[i] : v[i];
      }
    }
  } else {  // EPI_ACCUM_F32
#pragma unroll 1
    for (int c = c_begin; c < c_end; c += 32) {
      if (tl.n0 + c >= p.N) break;
      float v[32];
      if (have_acc) {
        tmem_ld32(taddr + c, v);   // every lane of the warp takes part in the load
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.f;
      }
      const int m_warp = tl.m0 + (row_in_tile & ~31);
      float* out_warp = (float*)p.out0 + (long long)tl.group * p.group_stride0 + (long long)m_warp * p.ld0 + tl.n0 + c;
      store32_f32_staged(p, out_warp, m_warp, v, stg, lane);
    }
  }
}

// ---------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------
template <bool A_MN, bool B_MN, bool ROWS_ARE_K, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;   // swizzle atoms need 1024-byte alignment
  uint8_t* stg_all = smem_raw + (tiles_base - raw) + STAGES * STAGE_BYTES;
  SharedTail* st = reinterpret_cast<SharedTail*>(stg_all + STG_TOTAL);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  for (int i = threadIdx.x; i <= p.n_groups; i += NUM_THREADS) {
    st->row0[i] = p.group_row0[i];
    st->tstart[i] = ROWS_ARE_K ? 0 : p.tile_start[i];
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&st->full[s]), 1);
      mbar_init(smem_u32(&st->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&st->tmem_full[a]), 1);
      mbar_init(smem_u32(&st->tmem_empty[a]), EPI_WARPS);
    }
    st->dead = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&st->tmem_base), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = st->tmem_base;

  const int n_tiles = total_tiles<ROWS_ARE_K>(st, p);

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------ TMA producer ------------------------------
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      // p.starve (test hook): the producer loads nothing, so the consumers' bounded waits run out
      for (int t = blockIdx.x; t < n_tiles && ok && !p.starve; t += gridDim.x) {
        const Tile tl = decode_tile<ROWS_ARE_K>(st, p, t);
        if (tl.skip) continue;
        for (int ki = 0; ki < tl.k_iters; ++ki) {
          if (!k_stage_live<ROWS_ARE_K>(p, tl, ki)) continue;
          if (!mbar_wait(smem_u32(&st->empty[stage]), phase ^ 1, p.error_flag, 101, p.wait_limit)) { ok = false; break; }
          const uint32_t bar = smem_u32(&st->full[stage]);
          const uint32_t sa = tiles_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          mbar_expect_tx(bar, STAGE_BYTES);
          if (ROWS_ARE_K) {
            const int krow = tl.row0 + ki * BK;
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * BOX_BYTES, &map_a, bar, tl.m0 + 64 * j, krow);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * BOX_BYTES, &map_b, bar, tl.n0 + 64 * j, krow);
          } else {
            tma_load_2d(sa, &map_a, bar, ki * BK, tl.row0);
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_3d(sb + j * BOX_BYTES, &map_b, bar, tl.n0 + 64 * j, ki * BK, tl.group);
            } else {
              tma_load_3d(sb, &map_b, bar, ki * BK, tl.n0, tl.group);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) st->dead = 1;
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------ MMA issuer --------------------------------
      // K-major tiles: rows of 128 bytes, 8-row swizzle atoms 1024 bytes apart; one
      // MMA (K=16) advances 32 bytes inside the 128-byte row.
      // MN-major tiles: 64x64 boxes of 8 KiB; 64-element chunks of the M/N extent are
      // 8192 bytes apart (leading offset), 8-row groups of K 1024 bytes apart; one MMA
      // (16 rows of K) advances 2048 bytes.
      constexpr uint32_t a_lbo = A_MN ? BOX_BYTES : 16, a_sbo = 1024, a_adv = A_MN ? 2048 : 32;
      constexpr uint32_t b_lbo = B_MN ? BOX_BYTES : 16, b_sbo = 1024, b_adv = B_MN ? 2048 : 32;
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        const Tile tl = decode_tile<ROWS_ARE_K>(st, p, t);
        if (tl.skip) continue;
        if (!mbar_wait(smem_u32(&st->tmem_empty[acc]), acc_phase ^ 1, p.error_flag, 102, p.wait_limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        // the last column tile may be narrower: issue an MMA only as wide as needed (multiple of 16)
        const int n_live = min(BN, ((p.N - tl.n0) + 15) & ~15);
        const uint32_t idesc = make_idesc(A_MN, B_MN, n_live);
        uint32_t accumulate = 0;   // the first MMA of the tile overwrites the accumulator
        for (int ki = 0; ki < tl.k_iters; ++ki) {
          if (!k_stage_live<ROWS_ARE_K>(p, tl, ki)) continue;
          if (!mbar_wait(smem_u32(&st->full[stage]), phase, p.error_flag, 103, p.wait_limit)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = tiles_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t da = make_desc(sa + kk * a_adv, a_lbo, a_sbo);
            const uint64_t db = make_desc(sb + kk * b_adv, b_lbo, b_sbo);
            umma_bf16(d_tmem, da, db, idesc, accumulate);
            accumulate = 1;
          }
          umma_commit(smem_u32(&st->empty[stage]));   // frees the stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (accumulate) umma_commit(smem_u32(&st->tmem_full[acc]));
        else mbar_arrive(smem_u32(&st->tmem_full[acc]));   // empty group: nothing was accumulated
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok) st->dead = 1;
    }
    __syncwarp();
  } else {
    // -------------------------------- epilogue ----------------------------------
    // A warp may only touch TMEM lanes [32*(warp%4), +32); two warps share each lane
    // quarter and split the tile's columns between them.
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int half = (warp - 2) >> 2;
    const int c_begin = half * (BN / 2), c_end = c_begin + BN / 2;
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
      const Tile tl = decode_tile<ROWS_ARE_K>(st, p, t);
      if (tl.skip) continue;
      if (!mbar_wait(smem_u32(&st->tmem_full[acc]), acc_phase, p.error_flag, 104, p.wait_limit)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
      epilogue_tile<EPI>(p, tl, taddr, row_in_tile, c_begin, c_end, tl.k_iters > 0, stg_all + (warp - 2) * STG_BYTES_PER_WARP);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&st->tmem_empty[acc]));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  __syncthreads();
  if (st->dead || *(volatile int*)p.error_flag != 0) {
    // Failure path: give copies that may still be in flight time to land before the
    // shared memory and tensor memory are released.
    const long long t0 = clock64();
    while (clock64() - t0 < 4000000LL) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}


// ---------------------------------------------------------------------------
// Two-SM variant: a cluster of two CTAs computes one 256x256 tile with
// tcgen05.mma.cta_group::2.  Each CTA loads its own 128 rows of A and HALF of the B tile
// (128 of the 256 columns); the tensor cores of both SMs read both halves.  Per SM and
// K-stage that is 32 KiB of shared memory instead of 48, so the ring holds 6 stages
// instead of 4 (longer latency cover for the same 192 KiB) and the L2 -> SM traffic per
// FLOP drops by a third.  CTA 0 of the pair issues the MMAs; both run their epilogue on
// their own 128 TMEM lanes.  Every CTA fetches what it stores; no load is shared across the cluster.
//
//   full[s]      (leader's)  one arrive.expect_tx by the leader for BOTH CTAs' bytes; the
//                            peer's TMA completes its bytes on the leader's barrier
//   empty[s]     (each CTA)  one tcgen05.commit per CTA after the stage's MMAs
//   tmem_full[a] (each CTA)  one tcgen05.commit per CTA after the tile's last MMA
//   tmem_empty[a](leader's)  one arrival per epilogue warp of both CTAs
// ---------------------------------------------------------------------------
constexpr int P_STAGES = 6;
constexpr int P_B_BYTES = (BN / 2) * BK * 2;            // 16 KiB: this CTA's half of B
constexpr int P_STAGE_BYTES = A_BYTES + P_B_BYTES;      // 32 KiB

struct __align__(8) PairTail {
  unsigned long long full[P_STAGES];
  unsigned long long empty[P_STAGES];
  unsigned long long tmem_full[2];
  unsigned long long tmem_empty[2];
  uint32_t tmem_base;
  int dead;
  int row0[MAX_GROUPS + 1];
  int pstart[MAX_GROUPS + 1];   // exclusive prefix of ceil(m-tiles / 2) per group
  int mtiles[MAX_GROUPS + 1];
};
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + STG_TOTAL + 1024 + (int)sizeof(PairTail);

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory object in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_pair_2d(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(leader_bar)
      : "memory");
}
__device__ __forceinline__ void tma_pair_3d(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(leader_bar)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem of both CTAs] (+)= A * B with M = 256 (128 rows per CTA), K = 16.
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
__host__ __device__ constexpr uint32_t make_idesc_pair(bool a_mn, bool b_mn, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
}

struct PairTile {
  int group, row0, m0, n0, k_iters, skip;   // skip: this CTA repeats a neighbour's rows and stores nothing
};

template <bool ROWS_ARE_K>
__device__ __forceinline__ int pair_total(const PairTail* st, const GemmArgs& p) {
  const int nt = ceil_div(p.N, BN);
  if (ROWS_ARE_K) return p.n_groups * ceil_div(ceil_div(p.M, BM), 2) * nt;
  return st->pstart[p.n_groups] * nt;
}

template <bool ROWS_ARE_K>
__device__ __forceinline__ PairTile pair_decode(const PairTail* st, const GemmArgs& p, int t, int rank) {
  PairTile tl;
  const int nt = ceil_div(p.N, BN);
  tl.skip = 0;
  if (ROWS_ARE_K) {
    const int pt = ceil_div(ceil_div(p.M, BM), 2);
    const int g = t / (pt * nt);
    const int rem = t - g * pt * nt;
    tl.group = g;
    tl.n0 = (rem / pt) * BN;
    tl.m0 = ((rem % pt) * 2 + rank) * BM;     // rows past M load zeros and are masked on store
    tl.row0 = st->row0[g];
    tl.k_iters = (st->row0[g + 1] - st->row0[g]) / BK;
  } else {
    int lo = 0, hi = p.n_groups;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (st->pstart[mid] * nt <= t) lo = mid; else hi = mid;
    }
    const int g = lo;
    const int pt = st->pstart[g + 1] - st->pstart[g];
    const int local = t - st->pstart[g] * nt;
    int mtile = (local % pt) * 2 + rank;
    if (mtile >= st->mtiles[g]) { mtile = st->mtiles[g] - 1; tl.skip = 1; }
    tl.group = g;
    tl.n0 = (local / pt) * BN;
    tl.m0 = 0;
    tl.row0 = st->row0[g] + mtile * BM;
    tl.k_iters = ceil_div(p.K, BK);
  }
  return tl;
}

template <bool A_MN, bool B_MN, bool ROWS_ARE_K, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;
  uint8_t* stg_all = smem_raw + (tiles_base - raw) + P_STAGES * P_STAGE_BYTES;
  PairTail* st = reinterpret_cast<PairTail*>(stg_all + STG_TOTAL);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();       // 0 = leader (issues the MMAs)
  const int cluster_id = blockIdx.x >> 1;
  const int n_clusters = gridDim.x >> 1;

  for (int i = threadIdx.x; i <= p.n_groups; i += NUM_THREADS) st->row0[i] = p.group_row0[i];
  if (threadIdx.x == 0) {
    int run = 0;
    for (int g = 0; g < p.n_groups; ++g) {
      const int mt = ROWS_ARE_K ? 0 : p.tile_start[g + 1] - p.tile_start[g];
      st->mtiles[g] = mt;
      st->pstart[g] = run;
      run += (mt + 1) >> 1;
    }
    st->pstart[p.n_groups] = run;
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(smem_u32(&st->full[s]), 1);
      mbar_init(smem_u32(&st->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&st->tmem_full[a]), 1);
      mbar_init(smem_u32(&st->tmem_empty[a]), 2 * EPI_WARPS);
    }
    st->dead = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(smem_u32(&st->tmem_base), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers exist before anything is signalled across the pair
  tc_fence_after();
  const uint32_t tmem_base = st->tmem_base;
  const int n_tiles = pair_total<ROWS_ARE_K>(st, p);

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------ TMA producer (both CTAs) ------------------------------
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int t = cluster_id; t < n_tiles && ok && !p.starve; t += n_clusters) {
        const PairTile tl = pair_decode<ROWS_ARE_K>(st, p, t, (int)rank);
        // this CTA's half of the B tile; a narrower last column tile is split in the middle
        const int n_live = min(BN, ((p.N - tl.n0) + 31) & ~31);
        const int nb0 = tl.n0 + (int)rank * (n_live / 2);
        for (int ki = 0; ki < tl.k_iters; ++ki) {
          if (!mbar_wait(smem_u32(&st->empty[stage]), phase ^ 1, p.error_flag, 201, p.wait_limit)) { ok = false; break; }
          const uint32_t leader_bar = map_to_cta(smem_u32(&st->full[stage]), 0);
          const uint32_t sa = tiles_base + stage * P_STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          if (rank == 0) mbar_expect_tx(smem_u32(&st->full[stage]), 2 * P_STAGE_BYTES);
          if (ROWS_ARE_K) {
            const int krow = tl.row0 + ki * BK;
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_pair_2d(sa + j * BOX_BYTES, &map_a, leader_bar, tl.m0 + 64 * j, krow);
#pragma unroll
            for (int j = 0; j < BN / 128; ++j) tma_pair_2d(sb + j * BOX_BYTES, &map_b, leader_bar, nb0 + 64 * j, krow);
          } else {
            tma_pair_2d(sa, &map_a, leader_bar, ki * BK, tl.row0);
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 128; ++j)
                tma_pair_3d(sb + j * BOX_BYTES, &map_b, leader_bar, nb0 + 64 * j, ki * BK, tl.group);
            } else {
              tma_pair_3d(sb, &map_b, leader_bar, ki * BK, nb0, tl.group);
            }
          }
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) st->dead = 1;
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ------------------------------ MMA issuer (leader CTA only) ------------------------------
      constexpr uint32_t a_lbo = A_MN ? BOX_BYTES : 16, a_sbo = 1024, a_adv = A_MN ? 2048 : 32;
      constexpr uint32_t b_lbo = B_MN ? BOX_BYTES : 16, b_sbo = 1024, b_adv = B_MN ? 2048 : 32;
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int t = cluster_id; t < n_tiles && ok; t += n_clusters) {
        const PairTile tl = pair_decode<ROWS_ARE_K>(st, p, t, 0);
        if (!mbar_wait(smem_u32(&st->tmem_empty[acc]), acc_phase ^ 1, p.error_flag, 202, p.wait_limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int n_live = min(BN, ((p.N - tl.n0) + 31) & ~31);
        const uint32_t idesc = make_idesc_pair(A_MN, B_MN, n_live);
        for (int ki = 0; ki < tl.k_iters; ++ki) {
          if (!mbar_wait(smem_u32(&st->full[stage]), phase, p.error_flag, 203, p.wait_limit)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = tiles_base + stage * P_STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t da = make_desc(sa + kk * a_adv, a_lbo, a_sbo);
            const uint64_t db = make_desc(sb + kk * b_adv, b_lbo, b_sbo);
            umma_bf16_pair(d_tmem, da, db, idesc, (ki | kk) != 0 ? 1u : 0u);
          }
          // the stage is free in BOTH CTAs once these MMAs have read it
          umma_commit_pair(smem_u32(&st->empty[stage]));
          umma_commit_pair(map_to_cta(smem_u32(&st->empty[stage]), 1));
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (tl.k_iters > 0) {
          umma_commit_pair(smem_u32(&st->tmem_full[acc]));
          umma_commit_pair(map_to_cta(smem_u32(&st->tmem_full[acc]), 1));
        } else {
          mbar_arrive(smem_u32(&st->tmem_full[acc]));
          mbar_arrive_cluster(map_to_cta(smem_u32(&st->tmem_full[acc]), 1));
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok) st->dead = 1;
    }
    __syncwarp();
  } else {
    // -------------------------------- epilogue (both CTAs) ----------------------------------
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int half = (warp - 2) >> 2;
    const int c_begin = half * (BN / 2), c_end = c_begin + BN / 2;
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    for (int t = cluster_id; t < n_tiles && ok; t += n_clusters) {
      const PairTile tl = pair_decode<ROWS_ARE_K>(st, p, t, (int)rank);
      if (!mbar_wait(smem_u32(&st->tmem_full[acc]), acc_phase, p.error_flag, 204, p.wait_limit)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
      if (!tl.skip) {
        Tile one;
        one.group = tl.group; one.row0 = tl.row0; one.m0 = tl.m0; one.n0 = tl.n0; one.k_iters = tl.k_iters; one.skip = 0;
        epilogue_tile<EPI>(p, one, taddr, row_in_tile, c_begin, c_end, tl.k_iters > 0, stg_all + (warp - 2) * STG_BYTES_PER_WARP);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&st->tmem_empty[acc]), 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  __syncthreads();
  if (st->dead || *(volatile int*)p.error_flag != 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 4000000LL) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();   // neither CTA leaves while its partner may still signal or read it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// Wide variant: one CTA computes a 256x256 tile as two 128-row sub-tiles that share the B stage.
// A K-stage is 64 KiB (two A sub-tiles of 16 KiB + 32 KiB of B) for 2 x 4 MMAs, so the bytes that enter
// the SM per MMA clock drop from 96 to 64; the ring holds 3 stages.  The two 128x256 fp32 accumulators are all
// 512 tensor-memory columns, so they are not double buffered: the epilogue of a tile does not overlap the
// next tile's MMAs (its loads do: the ring refills meanwhile).  A group with an odd number of 128-row
// tiles ends in a tile with one live sub-tile: nothing is loaded, multiplied or stored for the other.
// Causal skipping is not implemented here (the products are computed in full, which is still correct).
// ---------------------------------------------------------------------------
constexpr int W_STAGES = 3;
constexpr int W_A_BYTES = 2 * A_BYTES;                    // 32 KiB
constexpr int W_STAGE_BYTES = W_A_BYTES + B_BYTES;        // 64 KiB

struct __align__(8) WideTail {
  unsigned long long full[W_STAGES];
  unsigned long long empty[W_STAGES];
  unsigned long long tmem_full;
  unsigned long long tmem_empty;
  uint32_t tmem_base;
  int dead;
  int row0[MAX_GROUPS + 1];
  int pstart[MAX_GROUPS + 1];   // exclusive prefix of ceil(m-tiles / 2) per group
  int mtiles[MAX_GROUPS + 1];
};
constexpr int W_SMEM_BYTES = W_STAGES * W_STAGE_BYTES + STG_TOTAL + 1024 + (int)sizeof(WideTail);
static_assert(W_SMEM_BYTES <= 232448, "wide tiles do not fit the shared memory of one CTA");

struct WideTile {
  int group, row0, m0, n0, k_iters, msub;   // msub: live 128-row sub-tiles (1 or 2)
};

template <bool ROWS_ARE_K>
__device__ __forceinline__ int wide_total(const WideTail* st, const GemmArgs& p) {
  const int nt = ceil_div(p.N, BN);
  if (ROWS_ARE_K) return p.n_groups * ceil_div(ceil_div(p.M, BM), 2) * nt;
  return st->pstart[p.n_groups] * nt;
}

template <bool ROWS_ARE_K>
__device__ __forceinline__ WideTile wide_decode(const WideTail* st, const GemmArgs& p, int t) {
  WideTile tl;
  const int nt = ceil_div(p.N, BN);
  if (ROWS_ARE_K) {
    const int mt = ceil_div(p.M, BM);
    const int pt = ceil_div(mt, 2);
    const int g = t / (pt * nt);
    const int rem = t - g * pt * nt;
    tl.group = g;
    tl.n0 = (rem / pt) * BN;
    tl.m0 = (rem % pt) * 2 * BM;
    tl.msub = min(2, mt - (rem % pt) * 2);
    tl.row0 = st->row0[g];
    tl.k_iters = (st->row0[g + 1] - st->row0[g]) / BK;
  } else {
    int lo = 0, hi = p.n_groups;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (st->pstart[mid] * nt <= t) lo = mid; else hi = mid;
    }
    const int g = lo;
    const int pt = st->pstart[g + 1] - st->pstart[g];
    const int local = t - st->pstart[g] * nt;
    tl.group = g;
    tl.n0 = (local / pt) * BN;
    tl.m0 = 0;
    tl.msub = min(2, st->mtiles[g] - (local % pt) * 2);
    tl.row0 = st->row0[g] + (local % pt) * 2 * BM;
    tl.k_iters = ceil_div(p.K, BK);
  }
  return tl;
}

template <bool A_MN, bool B_MN, bool ROWS_ARE_K, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_wide_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;
  uint8_t* stg_all = smem_raw + (tiles_base - raw) + W_STAGES * W_STAGE_BYTES;
  WideTail* st = reinterpret_cast<WideTail*>(stg_all + STG_TOTAL);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  for (int i = threadIdx.x; i <= p.n_groups; i += NUM_THREADS) st->row0[i] = p.group_row0[i];
  if (threadIdx.x == 0) {
    int run = 0;
    for (int g = 0; g < p.n_groups; ++g) {
      const int mt = ROWS_ARE_K ? 0 : p.tile_start[g + 1] - p.tile_start[g];
      st->mtiles[g] = mt;
      st->pstart[g] = run;
      run += (mt + 1) >> 1;
    }
    st->pstart[p.n_groups] = run;
    for (int s = 0; s < W_STAGES; ++s) {
      mbar_init(smem_u32(&st->full[s]), 1);
      mbar_init(smem_u32(&st->empty[s]), 1);
    }
    mbar_init(smem_u32(&st->tmem_full), 1);
    mbar_init(smem_u32(&st->tmem_empty), EPI_WARPS);
    st->dead = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&st->tmem_base), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = st->tmem_base;
  const int n_tiles = wide_total<ROWS_ARE_K>(st, p);

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------ TMA producer ------------------------------
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok && !p.starve; t += gridDim.x) {
        const WideTile tl = wide_decode<ROWS_ARE_K>(st, p, t);
        for (int ki = 0; ki < tl.k_iters; ++ki) {
          if (!mbar_wait(smem_u32(&st->empty[stage]), phase ^ 1, p.error_flag, 301, p.wait_limit)) { ok = false; break; }
          const uint32_t bar = smem_u32(&st->full[stage]);
          const uint32_t sa = tiles_base + stage * W_STAGE_BYTES;
          const uint32_t sb = sa + W_A_BYTES;
          mbar_expect_tx(bar, tl.msub * A_BYTES + B_BYTES);
          if (ROWS_ARE_K) {
            const int krow = tl.row0 + ki * BK;
            for (int mi = 0; mi < tl.msub; ++mi) {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)
                tma_load_2d(sa + mi * A_BYTES + j * BOX_BYTES, &map_a, bar, tl.m0 + mi * BM + 64 * j, krow);
            }
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * BOX_BYTES, &map_b, bar, tl.n0 + 64 * j, krow);
          } else {
            for (int mi = 0; mi < tl.msub; ++mi) tma_load_2d(sa + mi * A_BYTES, &map_a, bar, ki * BK, tl.row0 + mi * BM);
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_3d(sb + j * BOX_BYTES, &map_b, bar, tl.n0 + 64 * j, ki * BK, tl.group);
            } else {
              tma_load_3d(sb, &map_b, bar, ki * BK, tl.n0, tl.group);
            }
          }
          if (++stage == W_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) st->dead = 1;
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------ MMA issuer --------------------------------
      constexpr uint32_t a_lbo = A_MN ? BOX_BYTES : 16, a_sbo = 1024, a_adv = A_MN ? 2048 : 32;
      constexpr uint32_t b_lbo = B_MN ? BOX_BYTES : 16, b_sbo = 1024, b_adv = B_MN ? 2048 : 32;
      uint32_t stage = 0, phase = 0, acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        const WideTile tl = wide_decode<ROWS_ARE_K>(st, p, t);
        if (!mbar_wait(smem_u32(&st->tmem_empty), acc_phase ^ 1, p.error_flag, 302, p.wait_limit)) { ok = false; break; }
        tc_fence_after();
        const int n_live = min(BN, ((p.N - tl.n0) + 15) & ~15);
        const uint32_t idesc = make_idesc(A_MN, B_MN, n_live);
        uint32_t accumulate = 0;
        for (int ki = 0; ki < tl.k_iters; ++ki) {
          if (!mbar_wait(smem_u32(&st->full[stage]), phase, p.error_flag, 303, p.wait_limit)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = tiles_base + stage * W_STAGE_BYTES;
          const uint32_t sb = sa + W_A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t db = make_desc(sb + kk * b_adv, b_lbo, b_sbo);
            umma_bf16(tmem_base, make_desc(sa + kk * a_adv, a_lbo, a_sbo), db, idesc, accumulate);
            if (tl.msub > 1) umma_bf16(tmem_base + BN, make_desc(sa + A_BYTES + kk * a_adv, a_lbo, a_sbo), db, idesc, accumulate);
            accumulate = 1;
          }
          umma_commit(smem_u32(&st->empty[stage]));
          if (++stage == W_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (accumulate) umma_commit(smem_u32(&st->tmem_full));
        else mbar_arrive(smem_u32(&st->tmem_full));   // empty group: nothing was accumulated
        acc_phase ^= 1;
      }
      if (!ok) st->dead = 1;
    }
    __syncwarp();
  } else {
    // -------------------------------- epilogue ----------------------------------
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int half = (warp - 2) >> 2;
    const int c_begin = half * (BN / 2), c_end = c_begin + BN / 2;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
      const WideTile tl = wide_decode<ROWS_ARE_K>(st, p, t);
      if (!mbar_wait(smem_u32(&st->tmem_full), acc_phase, p.error_flag, 304, p.wait_limit)) { ok = false; break; }
      tc_fence_after();
      // The accumulators are single buffered, so the MMAs of the next tile wait for this epilogue.  For the plain bf16
      // store the warp first moves its whole share of both sub-tiles into registers as packed pairs (2 x 4 pieces of
      // 32 columns = 128 registers), hands tensor memory back, and only then writes the rows out: those stores (about
      // 4000 clocks for a 256x256 tile) run under the next tile's MMAs (+5 % on the two products that use it).  The
      // SwiGLU and f32 epilogues have registers for one sub-tile only; holding that one while the other is written
      // straight from tensor memory was measured 2 - 3 % slower, so they keep the plain order.
      uint8_t* stg = stg_all + (warp - 2) * STG_BYTES_PER_WARP;
      const uint32_t tq = tmem_base + ((uint32_t)(quarter * 32) << 16);
      if (EPI == EPI_STORE) {
        uint32_t pk[2][4][16];
#pragma unroll
        for (int mi = 0; mi < 2; ++mi) {
          if (mi < tl.msub) {
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
              if (tl.n0 + c_begin + 32 * ch < p.N) {   // warp-uniform
                float v[32];
                tmem_ld32(tq + mi * BN + c_begin + 32 * ch, v);
#pragma unroll
                for (int i = 0; i < 16; ++i) pk[mi][ch][i] = pack2(v[2 * i], v[2 * i + 1]);
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&st->tmem_empty));
#pragma unroll
        for (int mi = 0; mi < 2; ++mi) {
          if (mi < tl.msub) {
            bf16* out = (bf16*)p.out0 + ((long long)tl.row0 + mi * BM + quarter * 32) * p.ld0 + tl.n0 + c_begin;
#pragma unroll
            for (int ch = 0; ch < 4; ++ch)
              if (tl.n0 + c_begin + 32 * ch < p.N) store32_packed_staged(out + 32 * ch, p.ld0, pk[mi][ch], stg, lane);
          }
        }
        acc_phase ^= 1;
        continue;
      }
      for (int mi = 0; mi < tl.msub; ++mi) {
        Tile one;
        one.group = tl.group; one.n0 = tl.n0; one.k_iters = tl.k_iters; one.skip = 0;
        one.row0 = ROWS_ARE_K ? tl.row0 : tl.row0 + mi * BM;
        one.m0 = ROWS_ARE_K ? tl.m0 + mi * BM : 0;
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + mi * BN;
        epilogue_tile<EPI>(p, one, taddr, row_in_tile, c_begin, c_end, tl.k_iters > 0, stg_all + (warp - 2) * STG_BYTES_PER_WARP);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&st->tmem_empty));
      acc_phase ^= 1;
    }
  }

  __syncthreads();
  if (st->dead || *(volatile int*)p.error_flag != 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 4000000LL) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// Host side: tensor maps and launches
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// bf16 tensor [groups][rows][cols], cols contiguous; box = {box_cols, box_rows, 1}.
static bool make_map(CUtensorMap* map, const Operand& op, int box_cols, int box_rows, bool three_d) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {(cuuint64_t)op.cols, (cuuint64_t)op.rows, (cuuint64_t)op.groups};
  const cuuint64_t ld = (cuuint64_t)(op.ld > 0 ? op.ld : op.cols);
  cuuint64_t strides[2] = {ld * 2, ld * (cuuint64_t)op.rows * 2};
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, three_d ? 3 : 2, const_cast<void*>(op.ptr), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

static bool operand_ok(const Operand& op) {
  return op.ptr && ((uintptr_t)op.ptr & 15) == 0 && op.cols > 0 && (op.cols % 8) == 0 && op.rows > 0 && op.groups > 0 &&
         (op.ld == 0 || (op.ld >= op.cols && op.ld % 8 == 0));
}

static int g_tile_mode = -1;   // -1: read the environment on first use
void set_tile_mode(int mode) { g_tile_mode = mode >= TILE_ONE_SM && mode <= TILE_AUTO ? mode : TILE_AUTO; }
int tile_mode() {
  if (g_tile_mode < 0) {
    const char* e = getenv("MOE_B200_TC_PAIR");
    const char* w = getenv("MOE_B200_TC_WIDE");
    g_tile_mode = (e && e[0] == '1') ? TILE_PAIR : (w && w[0] == '1') ? TILE_WIDE : (w && w[0] == '0') ? TILE_ONE_SM : TILE_AUTO;
  }
  return g_tile_mode;
}
bool pair_mode() { return tile_mode() == TILE_PAIR; }

// The opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of the kernel:
// one flag per device, so a process that holds layers on several GPUs configures each of them.
constexpr int MAX_DEVICES = 64;
template <typename Kernel>
static cudaError_t opt_in_smem(Kernel kern, bool* configured, int bytes) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < MAX_DEVICES && configured[dev]) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && dev >= 0 && dev < MAX_DEVICES) configured[dev] = true;
  return e;
}

// Test hook: the next launch (one launch only) runs with a producer that loads nothing and with the
// given wait limit, so that the bounded waits of the MMA and epilogue roles give up and the failure path
// (error flag, drain, tensor-memory release) runs.  Nothing is in flight on that path and nothing waits
// for ever.
static long long g_starve_limit = 0;
void set_starve_next_launch(long long wait_limit_cycles) { g_starve_limit = wait_limit_cycles > 0 ? wait_limit_cycles : 0; }

static GemmArgs with_wait_limit(const GemmArgs& in) {
  GemmArgs a = in;
  a.wait_limit = WAIT_LIMIT_CYCLES;
  a.starve = 0;
  if (g_starve_limit > 0) {
    a.wait_limit = g_starve_limit;
    a.starve = 1;
    g_starve_limit = 0;
  }
  return a;
}

template <bool A_MN, bool B_MN, bool ROWS_ARE_K, int EPI>
static cudaError_t launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& args, int sm_count,
                               cudaStream_t stream) {   // args: already through with_wait_limit
  auto kern = grouped_gemm_pair_kernel<A_MN, B_MN, ROWS_ARE_K, EPI>;
  static bool configured[MAX_DEVICES] = {};
  { const cudaError_t e = opt_in_smem(kern, configured, P_SMEM_BYTES); if (e != cudaSuccess) return e; }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)(sm_count & ~1));
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = P_SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ma, mb, args);
  count_launch();
  return e != cudaSuccess ? e : cudaGetLastError();
}

template <bool A_MN, bool B_MN, bool ROWS_ARE_K, int EPI>
static cudaError_t launch_wide(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& args, int sm_count,
                               cudaStream_t stream) {   // args: already through with_wait_limit
  auto kern = grouped_gemm_wide_kernel<A_MN, B_MN, ROWS_ARE_K, EPI>;
  static bool configured[MAX_DEVICES] = {};
  { const cudaError_t e = opt_in_smem(kern, configured, W_SMEM_BYTES); if (e != cudaSuccess) return e; }
  kern<<<sm_count, NUM_THREADS, W_SMEM_BYTES, stream>>>(ma, mb, args); count_launch();
  return cudaGetLastError();
}

// TILE_AUTO: 256x256 tiles where they pay.  They need a third fewer operand bytes per MMA, but their epilogue does not
// overlap the next tile's MMAs and there are half as many tiles to spread over the SMs: so only for products of
// several waves of wide tiles and a reduction long enough to amortise the epilogue (measured: a 256x256 bf16 tile
// leaves the SM in about 4000 clocks, the MMAs of 1024 reduction elements take 16384), not for the SwiGLU-backward epilogue (it reads the saved g|u rows and is the longest),
// not for the f32 store, and not for causal products (only the 128-row tiles skip the masked part).
template <int EPI>
static bool wide_pays(const GemmArgs& a, long long wide_tiles, long long reduction, int sm_count) {
  return a.causal == 0 && EPI != EPI_SWIGLU_BWD && EPI != EPI_STORE_F32 && wide_tiles >= 4ll * sm_count && reduction >= 1024;
}

template <bool A_MN, bool B_MN, bool ROWS_ARE_K, int EPI>
static cudaError_t launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& args_in, long long wide_tiles,
                          long long reduction, int sm_count, cudaStream_t stream) {
  const GemmArgs args = with_wait_limit(args_in);
  const int mode = tile_mode();
  if (mode == TILE_PAIR) return launch_pair<A_MN, B_MN, ROWS_ARE_K, EPI>(ma, mb, args, sm_count, stream);
  if (mode == TILE_WIDE || (mode == TILE_AUTO && wide_pays<EPI>(args, wide_tiles, reduction, sm_count)))
    return launch_wide<A_MN, B_MN, ROWS_ARE_K, EPI>(ma, mb, args, sm_count, stream);
  auto kern = grouped_gemm_kernel<A_MN, B_MN, ROWS_ARE_K, EPI>;
  static bool configured[MAX_DEVICES] = {};
  { const cudaError_t e = opt_in_smem(kern, configured, SMEM_BYTES); if (e != cudaSuccess) return e; }
  kern<<<sm_count, NUM_THREADS, SMEM_BYTES, stream>>>(ma, mb, args); count_launch();
  return cudaGetLastError();
}

cudaError_t gemm_rows_nt(const Operand& A, const Operand& B, const GemmArgs& args, int epilogue, int sm_count,
                         cudaStream_t stream) {
  if (!operand_ok(A) || !operand_ok(B) || A.cols != B.cols || (args.N % 32 != 0 && epilogue != EPI_STORE_F32) ||
      args.n_groups > MAX_GROUPS - 1)
    return cudaErrorInvalidValue;
  CUtensorMap ma, mb;
  if (!make_map(&ma, A, BK, BM, false) || !make_map(&mb, B, BK, pair_mode() ? BN / 2 : BN, true)) return cudaErrorInvalidValue;
  const long long wide_tiles = (A.rows / (2 * BM)) * ceil_div(args.N, BN);   // an estimate: the host does not know the groups
  const long long reduction = A.cols;
  switch (epilogue) {
    case EPI_STORE: return launch<false, false, false, EPI_STORE>(ma, mb, args, wide_tiles, reduction, sm_count, stream);
    case EPI_SWIGLU: return launch<false, false, false, EPI_SWIGLU>(ma, mb, args, wide_tiles, reduction, sm_count, stream);
    case EPI_STORE_F32: return launch<false, false, false, EPI_STORE_F32>(ma, mb, args, wide_tiles, reduction, sm_count, stream);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t gemm_rows_nn(const Operand& A, const Operand& B, const GemmArgs& args, int epilogue, int sm_count,
                         cudaStream_t stream) {
  if (!operand_ok(A) || !operand_ok(B) || A.cols != B.rows || args.N % 32 != 0 || args.n_groups > MAX_GROUPS - 1)
    return cudaErrorInvalidValue;
  CUtensorMap ma, mb;
  if (!make_map(&ma, A, BK, BM, false) || !make_map(&mb, B, 64, 64, true)) return cudaErrorInvalidValue;
  const long long wide_tiles = (A.rows / (2 * BM)) * ceil_div(args.N, BN);
  const long long reduction = A.cols;
  switch (epilogue) {
    case EPI_STORE: return launch<false, true, false, EPI_STORE>(ma, mb, args, wide_tiles, reduction, sm_count, stream);
    case EPI_SWIGLU_BWD: return launch<false, true, false, EPI_SWIGLU_BWD>(ma, mb, args, wide_tiles, reduction, sm_count, stream);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t gemm_rows_tn(const Operand& A, const Operand& B, const GemmArgs& args, int sm_count,
                         cudaStream_t stream) {
  if (!operand_ok(A) || !operand_ok(B) || args.N % 32 != 0 || args.n_groups > MAX_GROUPS - 1)
    return cudaErrorInvalidValue;
  CUtensorMap ma, mb;
  if (!make_map(&ma, A, 64, 64, false) || !make_map(&mb, B, 64, 64, false)) return cudaErrorInvalidValue;
  const long long wide_tiles = (long long)args.n_groups * ceil_div(ceil_div(args.M, BM), 2) * ceil_div(args.N, BN);
  const long long reduction = A.rows / (args.n_groups > 0 ? args.n_groups : 1);   // rows per group on average
  return launch<true, true, true, EPI_ACCUM_F32>(ma, mb, args, wide_tiles, reduction, sm_count, stream);
}

}  // namespace tc
}  // namespace moe
