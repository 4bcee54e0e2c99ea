// Batched KV-cache decode attention (the ABI of include/kv_attention_b200.h).
//
// What MultiHeadAttention::forward_cached does between its projections (reference attention.rs:344-398),
// for many sequences per launch: rotate the new queries and keys (rope.rs:170-225), append keys and values
// to the per-sequence caches (attention.rs:65-78), softmax(q K^T / sqrt(head_dim)) V over the visible
// positions (attention.rs:1100-1160).  A decode step streams every cached key and value once, so the
// kernel is bound by HBM: the cache is [sequence][position][kv_head * head_dim], one CTA takes one
// (sequence, kv head, slice of the positions) and serves every query head of that kv head's group from
// the same loads (grouped-query attention reads the cache once, not once per query head); slices are
// merged by a second small kernel (split softmax: running maximum, denominator and weighted sum).
//
// Launches per step: [rotate + append: scalar path only; the tensor-core kernel does both itself,] partial
// attention, merge (which also advances the lengths).
// Merging inside the attention kernel (the last CTA of a kv head to finish merges its slices) was tried:
// it saves a launch and measured 4 us slower per step than the separate merge kernel.

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <new>
#include <string>
#include <vector>

#include "../../include/kv_attention_b200.h"
#include "../../include/moe_b200.h"
#include "common.cuh"

namespace moe {
namespace {

constexpr int KV_THREADS = 256;
constexpr int KV_WARPS = KV_THREADS / 32;
constexpr int KV_QT = 4;            // queries served per pass over a slice
constexpr int KV_MAX_SPLITS = 64;
constexpr float LOG2E = 1.4426950408889634f;

template <typename T> struct Slice8;
template <> struct Slice8<float> {
  static __device__ __forceinline__ void load(const float* p, float* o) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
  }
  static __device__ __forceinline__ void from_shared(const unsigned char* p, float* o) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *(reinterpret_cast<const float4*>(p) + 1);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
  }
};
template <> struct Slice8<bf16> {
  static __device__ __forceinline__ void load(const bf16* p, float* o) {
    widen(__ldg(reinterpret_cast<const uint4*>(p)), o);
  }
  static __device__ __forceinline__ void from_shared(const unsigned char* p, float* o) {
    widen(*reinterpret_cast<const uint4*>(p), o);
  }
  static __device__ __forceinline__ void widen(const uint4 a, float* o) {
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {   // a bf16 is the upper half of its f32
      o[2 * i] = __uint_as_float(w[i] << 16);
      o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}
// slots of the per-thread copy ring (48 KiB of shared memory per CTA either way)
template <typename T> struct KvRing;
template <> struct KvRing<bf16> { static constexpr int DEPTH = 6; };
template <> struct KvRing<float> { static constexpr int DEPTH = 3; };
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

struct KvShape {
  int H, Hkv, HD, cap, rows;      // rows = new rows per sequence
  int first;                      // first sequence of the range
};

// ---- rotate the new queries and keys, append keys and values (one CTA per new row) ----
template <typename T>
__global__ void kv_append_kernel(T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                 T* __restrict__ keys, T* __restrict__ values, const int* __restrict__ lengths,
                                 const float* __restrict__ cos_t, const float* __restrict__ sin_t, KvShape s, int rope) {
  const int row = blockIdx.x, seq = s.first + row / s.rows, i = row % s.rows;
  if (lengths[seq] + s.rows > s.cap) return;   // no room (reported by the attention kernel): nothing is stored
  const int pos = lengths[seq] + i, half = s.HD / 2;
  const float* ct = cos_t + (size_t)pos * half;
  const float* st = sin_t + (size_t)pos * half;
  T* qr = q + (size_t)row * s.H * s.HD;
  if (rope) {
    for (int idx = threadIdx.x; idx < s.H * half; idx += blockDim.x) {
      const int h = idx / half, c = idx - h * half;
      const float co = ct[c], si = st[c];
      const float lo = to_f32<T>(qr[h * s.HD + c]), hi = to_f32<T>(qr[h * s.HD + half + c]);
      qr[h * s.HD + c] = from_f32<T>(lo * co - hi * si);          // rope.rs:213-218
      qr[h * s.HD + half + c] = from_f32<T>(hi * co + lo * si);
    }
  }
  const int W = s.Hkv * s.HD;
  const T* kr = k + (size_t)row * W;
  const T* vr = v + (size_t)row * W;
  T* kd = keys + ((size_t)seq * s.cap + pos) * W;
  T* vd = values + ((size_t)seq * s.cap + pos) * W;
  for (int idx = threadIdx.x; idx < s.Hkv * half; idx += blockDim.x) {
    const int h = idx / half, c = idx - h * half;
    const float lo = to_f32<T>(kr[h * s.HD + c]), hi = to_f32<T>(kr[h * s.HD + half + c]);
    float a = lo, b = hi;
    if (rope) {
      const float co = ct[c], si = st[c];
      a = lo * co - hi * si;
      b = hi * co + lo * si;
    }
    kd[h * s.HD + c] = from_f32<T>(a);
    kd[h * s.HD + half + c] = from_f32<T>(b);
    vd[h * s.HD + c] = vr[h * s.HD + c];
    vd[h * s.HD + half + c] = vr[h * s.HD + half + c];
  }
}

// ---- partial attention over one slice of one sequence's positions, for one kv head ----
// HD / 8 lanes share a position (each holds 8 channels of its key and of its value), so a warp takes
// 256 / HD positions per step and every load is 16 bytes (bf16) or 32 bytes (f32) per lane, adjacent
// lanes adjacent in memory.  Scores are kept in the base-2 domain (the query is pre-multiplied by
// log2(e) / sqrt(head_dim)); every lane group keeps its own running maximum, denominator and weighted
// value sum per query, merged once at the end through shared memory.
// part: [row][head][split][HD + 2] = weighted sum, maximum, denominator.
template <typename T, int HD>
__global__ void __launch_bounds__(KV_THREADS)
kv_partial_kernel(const T* __restrict__ q, const T* __restrict__ keys, const T* __restrict__ values,
                  const int* __restrict__ lengths, int* __restrict__ full, float* __restrict__ part, KvShape s, int splits,
                  float scale_log2) {
  constexpr int LPK = HD / 8, KPW = 32 / LPK, NG = KV_WARPS * KPW, PW = HD + 2;
  constexpr int SLOT = 8 * (int)sizeof(T), DEPTH = KvRing<T>::DEPTH;
  extern __shared__ __align__(16) float kv_sm[];   // the copy ring, then [KV_QT][NG][PW] for the merge
  const int split = blockIdx.x, kvh = blockIdx.y, sj = blockIdx.z, seq = s.first + sj;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = lane / LPK, ls = lane % LPK;
  const int len0 = lengths[seq], total = len0 + s.rows;
  if (total > s.cap) {   // the cache of this sequence has no room for the step: mark it, touch nothing
    if (threadIdx.x == 0) full[seq] = 1;
    return;
  }
  const int chunk = round_up(ceil_div(total, splits), NG);
  const int k0 = split * chunk, k1 = min(total, k0 + chunk);
  const int group = s.H / s.Hkv, nq = s.rows * group, W = s.Hkv * s.HD;
  const T* kbase = keys + (size_t)seq * s.cap * W + kvh * HD + ls * 8;
  const T* vbase = values + (size_t)seq * s.cap * W + kvh * HD + ls * 8;
  const int grp = warp * KPW + sub;

  for (int q0 = 0; q0 < nq; q0 += KV_QT) {
    float qv[KV_QT][8], acc[KV_QT][8], m[KV_QT], l[KV_QT];
    int vis[KV_QT];
#pragma unroll
    for (int j = 0; j < KV_QT; ++j) {
      const int qi = q0 + j, i = qi / group, g = qi - i * group;
      m[j] = -INFINITY;
      l[j] = 0.f;
      vis[j] = qi < nq ? len0 + i + 1 : 0;        // positions 0 ..= len + i (attention.rs:1116)
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[j][c] = 0.f;
      if (qi < nq) {
        Slice8<T>::load(q + ((size_t)(sj * s.rows + i) * s.H + kvh * group + g) * HD + ls * 8, qv[j]);
#pragma unroll
        for (int c = 0; c < 8; ++c) qv[j][c] *= scale_log2;
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) qv[j][c] = 0.f;
      }
    }
    // a slice ends where the last query of this pass stops seeing
    const int kend = min(k1, vis[KV_QT - 1] > 0 ? vis[KV_QT - 1] : len0 + (nq - 1) / group + 1);
    // Each thread streams its own 8-channel slices of the keys and values through a ring of DEPTH
    // slots in shared memory (cp.async, 16 bytes each): DEPTH - 1 positions per thread are in flight
    // while one is used, which is what covers DRAM latency at two or three CTAs per SM.  A thread reads
    // back only what it copied itself, so waiting on its own copy groups is all the ordering needed.
    // The loop is uniform across the warp (the shuffles below need every lane); a lane group whose
    // position lies past the end copies nothing and updates nothing.
    const int base0 = k0 + warp * KPW + sub;
    const int iters = kend > k0 + warp * KPW ? ceil_div(kend - (k0 + warp * KPW), NG) : 0;
    unsigned char* slot0 = reinterpret_cast<unsigned char*>(kv_sm) + (size_t)threadIdx.x * SLOT;
    auto issue = [&](int it) {
      const int key = base0 + it * NG;
      if (it < iters && key < kend) {
        unsigned char* dk = slot0 + (size_t)(it % DEPTH) * (2 * KV_THREADS * SLOT);
        unsigned char* dv = dk + KV_THREADS * SLOT;
        const unsigned char* gk = reinterpret_cast<const unsigned char*>(kbase + (size_t)key * W);
        const unsigned char* gv = reinterpret_cast<const unsigned char*>(vbase + (size_t)key * W);
#pragma unroll
        for (int b = 0; b < SLOT; b += 16) {
          cp_async16(dk + b, gk + b);
          cp_async16(dv + b, gv + b);
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");   // one group per step, empty or not
    };
    for (int it = 0; it < DEPTH - 1; ++it) issue(it);
    for (int it = 0; it < iters; ++it) {
      issue(it + DEPTH - 1);
      asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 1) : "memory");   // step `it` has landed
      const int key = base0 + it * NG;
      const bool live = key < kend;
      float kf[8], vf[8];
      if (live) {
        const unsigned char* dk = slot0 + (size_t)(it % DEPTH) * (2 * KV_THREADS * SLOT);
        Slice8<T>::from_shared(dk, kf);
        Slice8<T>::from_shared(dk + KV_THREADS * SLOT, vf);
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) kf[c] = vf[c] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < KV_QT; ++j) {
        float sc = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) sc = fmaf(qv[j][c], kf[c], sc);
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, o);
        if (live && key < vis[j]) {
          const float mn = fmaxf(m[j], sc);
          const float corr = exp2f(m[j] - mn), p = exp2f(sc - mn);
          l[j] = fmaf(l[j], corr, p);
#pragma unroll
          for (int c = 0; c < 8; ++c) acc[j][c] = fmaf(acc[j][c], corr, p * vf[c]);
          m[j] = mn;
        }
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // merge the lane groups of the CTA
    __syncthreads();   // every thread is done with its ring slots, and the previous pass with the merge buffer
#pragma unroll
    for (int j = 0; j < KV_QT; ++j) {
      float* dst = kv_sm + ((size_t)j * NG + grp) * PW;
#pragma unroll
      for (int c = 0; c < 8; ++c) dst[ls * 8 + c] = acc[j][c];
      if (ls == 0) { dst[HD] = m[j]; dst[HD + 1] = l[j]; }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < KV_QT * HD; idx += KV_THREADS) {
      const int j = idx / HD, c = idx - j * HD, qi = q0 + j;
      if (qi >= nq) continue;
      const float* src = kv_sm + (size_t)j * NG * PW;
      float mx = -INFINITY;
      for (int g = 0; g < NG; ++g) mx = fmaxf(mx, src[g * PW + HD]);
      float num = 0.f, den = 0.f;
      if (mx > -INFINITY) {
        for (int g = 0; g < NG; ++g) {
          const float w = exp2f(src[g * PW + HD] - mx);   // 0 for a group that saw nothing
          num = fmaf(w, src[g * PW + c], num);
          den = fmaf(w, src[g * PW + HD + 1], den);
        }
      }
      const int i = qi / group, g = qi - i * group;
      float* out = part + (((size_t)(sj * s.rows + i) * s.H + kvh * group + g) * splits + split) * PW;
      out[c] = num;
      if (c == 0) { out[HD] = mx; out[HD + 1] = den; }
    }
    __syncthreads();   // the next pass copies into the memory the merge has just read
  }
}

// ---- the same slice on the tensor cores (bf16 cache, head_dim 64 or 128) ----
// The scalar kernel above spends most of its issue slots on the dot products and on softmax arithmetic
// that every lane of a position repeats.  Here a warp takes blocks of 16 positions: S = Q K^T and
// O += P V are mma.sync m16n8k16 products whose 16 rows are the queries of the group (rows past the
// group are zero), the key and value blocks come through a warp-private cp.async ring in shared memory
// (16-byte chunks XOR-swizzled by row so that ldmatrix is conflict-free), and the softmax touches each
// score once.  Same slice bounds, same result format as the scalar kernel.
constexpr int TC_WARPS = 4, TC_KB = 16, TC_DEPTH = 3;

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16_zfill(uint32_t smem_dst, const void* gmem_src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gmem_src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

template <int HD>
__global__ void __launch_bounds__(TC_WARPS * 32)
kv_partial_tc_kernel(const bf16* __restrict__ q, const bf16* __restrict__ knew, const bf16* __restrict__ vnew,
                     bf16* keys, bf16* values, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                     const int* __restrict__ lengths, int* __restrict__ full, float* __restrict__ part, KvShape s,
                     int splits, float scale_log2, int rope) {
  constexpr int RB = HD * 2, TILE = TC_KB * RB, CPR = HD / 8, PW = HD + 2, KT = HD / 16, NT = HD / 8;
  constexpr int COPIES = TC_KB * CPR / 32;    // 16-byte chunks per lane and tile
  extern __shared__ __align__(128) unsigned char tc_sm[];
  const int split = blockIdx.x, kvh = blockIdx.y, sj = blockIdx.z, seq = s.first + sj;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  const int len0 = lengths[seq], total = len0 + s.rows;
  if (total > s.cap) {   // no room for the step: mark the sequence; nothing is appended, read or advanced
    if (threadIdx.x == 0) full[seq] = 1;
    return;
  }
  const int chunk = round_up(ceil_div(total, splits), TC_WARPS * TC_KB);
  const int k0 = split * chunk, k1 = min(total, k0 + chunk);
  const int group = s.H / s.Hkv, nq = s.rows * group, W = s.Hkv * s.HD;
  bf16* kg = keys + (size_t)seq * s.cap * W + kvh * HD;
  bf16* vg = values + (size_t)seq * s.cap * W + kvh * HD;
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(tc_sm) + warp * (TC_DEPTH * 2 * TILE);
  float* mb = reinterpret_cast<float*>(tc_sm);   // [16][TC_WARPS][PW], after the rings are drained
  constexpr int HALF = HD / 2;

  // Append: the new positions that fall into this slice are rotated (keys) and stored by this CTA, for
  // its kv head, before it reads the slice; every new position lies in exactly one slice, and no CTA reads
  // positions outside its own slice, so no CTA depends on another one's stores.
  {
    const int a0 = max(k0, len0), a1 = min(k0 + chunk, total);
    for (int idx = threadIdx.x; idx < (a1 - a0) * HALF; idx += TC_WARPS * 32) {
      const int r = idx / HALF, c = idx - r * HALF, pos = a0 + r;
      const size_t src = (size_t)(sj * s.rows + pos - len0) * W + kvh * HD;
      const float lo = __bfloat162float(knew[src + c]), hi = __bfloat162float(knew[src + HALF + c]);
      float a = lo, b = hi;
      if (rope) {
        const float co = cos_t[(size_t)pos * HALF + c], si = sin_t[(size_t)pos * HALF + c];
        a = lo * co - hi * si;                                  // rope.rs:213-218
        b = hi * co + lo * si;
      }
      kg[(size_t)pos * W + c] = __float2bfloat16_rn(a);
      kg[(size_t)pos * W + HALF + c] = __float2bfloat16_rn(b);
      vg[(size_t)pos * W + c] = vnew[src + c];
      vg[(size_t)pos * W + HALF + c] = vnew[src + HALF + c];
    }
    __threadfence();
    __syncthreads();
  }

  for (int q0 = 0; q0 < nq; q0 += 16) {
    // query fragments: rows gid and gid + 8 of the pass
    uint32_t qa[KT][4];
    int lim[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int qi = q0 + gid + 8 * h, ok = qi < nq;
      const int i = ok ? qi / group : 0, g = ok ? qi - i * group : 0;
      lim[h] = ok ? min(len0 + i + 1, k1) : 0;     // positions 0 ..= len + i, inside this slice
      const bf16* qr = q + ((size_t)(sj * s.rows + i) * s.H + kvh * group + g) * HD + 2 * tig;
#pragma unroll
      for (int kk = 0; kk < KT; ++kk) {
        qa[kk][h] = ok ? *reinterpret_cast<const uint32_t*>(qr + 16 * kk) : 0u;
        qa[kk][2 + h] = ok ? *reinterpret_cast<const uint32_t*>(qr + 16 * kk + 8) : 0u;
      }
      if (ok && rope) {
        // rotate-half inside the fragments: channel c (k-step kk) pairs with c + HD / 2 (k-step kk + KT / 2),
        // same register slot; rounded to bf16 as a rotated query stored in memory would be
        const float* ct = cos_t + (size_t)(len0 + i) * HALF + 2 * tig;
        const float* st = sin_t + (size_t)(len0 + i) * HALF + 2 * tig;
#pragma unroll
        for (int kk = 0; kk < KT / 2; ++kk)
#pragma unroll
          for (int u = 0; u < 2; ++u) {           // channels 16 kk + 2 tig (+1), then + 8
            const int c = 16 * kk + 8 * u;
            const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qa[kk][2 * u + h]));
            const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qa[kk + KT / 2][2 * u + h]));
            const float c0 = ct[c], c1 = ct[c + 1], s0 = st[c], s1 = st[c + 1];
            qa[kk][2 * u + h] = pack_bf16x2(lo.x * c0 - hi.x * s0, lo.y * c1 - hi.y * s1);
            qa[kk + KT / 2][2 * u + h] = pack_bf16x2(hi.x * c0 + lo.x * s0, hi.y * c1 + lo.y * s1);
          }
      }
    }
    const int last = min(q0 + 15, nq - 1);
    const int kend = min(k1, len0 + last / group + 1);
    const int first_blk = k0 + warp * TC_KB;
    const int nblk = kend > first_blk ? ceil_div(kend - first_blk, TC_WARPS * TC_KB) : 0;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f}, o[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;

    auto issue = [&](int b) {
      if (b < nblk) {
        const int kb = first_blk + b * (TC_WARPS * TC_KB);
        const uint32_t dk = ring + (b % TC_DEPTH) * (2 * TILE), dv = dk + TILE;
#pragma unroll
        for (int i = 0; i < COPIES; ++i) {
          const int idx = lane + 32 * i, row = idx / CPR, ch = idx - row * CPR;
          const int key = kb + row, live = key < kend ? 16 : 0;      // rows past the end are zero-filled
          const size_t src = (size_t)min(key, total - 1) * W + ch * 8;
          const uint32_t off = row * RB + (((ch & ~7) | ((ch ^ row) & 7)) << 4);
          cp_async16_zfill(dk + off, kg + src, live);
          cp_async16_zfill(dv + off, vg + src, live);
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (int b = 0; b < TC_DEPTH - 1; ++b) issue(b);
    for (int b = 0; b < nblk; ++b) {
      issue(b + TC_DEPTH - 1);
      asm volatile("cp.async.wait_group %0;" ::"n"(TC_DEPTH - 1) : "memory");
      __syncwarp();                                  // every lane's copies of block b have landed
      const int kb = first_blk + b * (TC_WARPS * TC_KB);
      const uint32_t tk = ring + (b % TC_DEPTH) * (2 * TILE), tv = tk + TILE;
      // S = Q K^T: two tiles of 8 positions
      float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      {
        const int mi = lane >> 3, r = lane & 7, key = (mi >> 1) * 8 + r;
#pragma unroll
        for (int kk = 0; kk < KT; ++kk) {
          const int ch = 2 * kk + (mi & 1);
          uint32_t bfr[4];
          ldsm_x4(tk + key * RB + (((ch & ~7) | ((ch ^ key) & 7)) << 4), bfr);
          mma_bf16_16816(sc[0], qa[kk], bfr[0], bfr[1]);
          mma_bf16_16816(sc[1], qa[kk], bfr[2], bfr[3]);
        }
      }
      // softmax of the block, base-2 domain; thread holds (row gid | gid + 8) x (positions 8 j + 2 tig, + 1)
      uint32_t pa[4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float v[4];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int key = kb + 8 * j + 2 * tig + e;
            v[2 * j + e] = key < lim[h] ? sc[j][2 * h + e] * scale_log2 : -INFINITY;
          }
        float bm = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
        const float mn = fmaxf(m[h], bm);
        const float ref = mn > -INFINITY ? mn : 0.f;          // nothing visible yet: every weight is 0
        const float corr = exp2f(m[h] - ref);
        float p[4], ps = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) { p[e] = exp2f(v[e] - ref); ps += p[e]; }
        l[h] = fmaf(l[h], corr, ps);                          // this thread's share; summed over the quad at the end
        m[h] = mn;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) { o[nt][2 * h] *= corr; o[nt][2 * h + 1] *= corr; }
        pa[h] = pack_bf16x2(p[0], p[1]);                      // positions 2 tig, + 1
        pa[2 + h] = pack_bf16x2(p[2], p[3]);                  // positions 8 + 2 tig, + 1
      }
      // O += P V: 16 positions x HD channels, two 8-channel tiles per ldmatrix
      {
        const int mi = lane >> 3, r = lane & 7, key = (mi & 1) * 8 + r;
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
          const int ch = 2 * np + (mi >> 1);
          uint32_t bfr[4];
          ldsm_x4_t(tv + key * RB + (((ch & ~7) | ((ch ^ key) & 7)) << 4), bfr);
          mma_bf16_16816(o[2 * np], pa, bfr[0], bfr[1]);
          mma_bf16_16816(o[2 * np + 1], pa, bfr[2], bfr[3]);
        }
      }
      __syncwarp();                                  // the slot may be refilled by the next issue
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
      l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    __syncthreads();   // every warp has drained its ring; the merge buffer takes its place
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float* dst = mb + ((size_t)(gid + 8 * h) * TC_WARPS + warp) * PW;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        dst[8 * nt + 2 * tig] = o[nt][2 * h];
        dst[8 * nt + 2 * tig + 1] = o[nt][2 * h + 1];
      }
      if (tig == 0) { dst[HD] = m[h]; dst[HD + 1] = l[h]; }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 16 * HD; idx += TC_WARPS * 32) {
      const int r = idx / HD, c = idx - r * HD, qi = q0 + r;
      if (qi >= nq) continue;
      const float* src = mb + (size_t)r * TC_WARPS * PW;
      float mx = -INFINITY;
#pragma unroll
      for (int w = 0; w < TC_WARPS; ++w) mx = fmaxf(mx, src[w * PW + HD]);
      float num = 0.f, den = 0.f;
      if (mx > -INFINITY) {
#pragma unroll
        for (int w = 0; w < TC_WARPS; ++w) {
          const float wt = exp2f(src[w * PW + HD] - mx);
          num = fmaf(wt, src[w * PW + c], num);
          den = fmaf(wt, src[w * PW + HD + 1], den);
        }
      }
      const int i = qi / group, g = qi - i * group;
      float* out = part + (((size_t)(sj * s.rows + i) * s.H + kvh * group + g) * splits + split) * PW;
      out[c] = num;
      if (c == 0) { out[HD] = mx; out[HD + 1] = den; }
    }
    __syncthreads();   // the next pass copies into the memory the merge has just read
  }
}

// ---- merge the slices, write the merged heads, advance the cache lengths ----
template <typename T>
__global__ void kv_merge_kernel(const float* __restrict__ part, T* __restrict__ merged, int* __restrict__ lengths,
                                const int* __restrict__ full, KvShape s, int splits) {
  const int PW = s.HD + 2;
  const int rh = blockIdx.x;                      // row * H + head
  if (full[s.first + rh / s.H / s.rows]) {
    // the attention kernel found this sequence's cache full: zeros out, length unchanged; the mark stays
    // until the host reads it (kv_cache_lengths) or the sequence is truncated
    for (int c = threadIdx.x; c < s.HD; c += blockDim.x) merged[(size_t)rh * s.HD + c] = from_f32<T>(0.f);
    return;
  }
  const float* src = part + (size_t)rh * splits * PW;
  float mx = -INFINITY;
  for (int p = 0; p < splits; ++p) mx = fmaxf(mx, src[p * PW + s.HD]);
  for (int c = threadIdx.x; c < s.HD; c += blockDim.x) {
    float num = 0.f, den = 0.f;
    for (int p = 0; p < splits; ++p) {
      const float w = src[p * PW + s.HD] > -INFINITY ? exp2f(src[p * PW + s.HD] - mx) : 0.f;
      num = fmaf(w, src[p * PW + c], num);
      den = fmaf(w, src[p * PW + s.HD + 1], den);
    }
    merged[(size_t)rh * s.HD + c] = from_f32<T>(den > 0.f ? num / den : 0.f);   // activations.rs:65-69
  }
  // one thread per sequence moves its length on (every earlier launch of this step has read it)
  const int row = rh / s.H, head = rh - row * s.H;
  if (head == 0 && row % s.rows == 0 && threadIdx.x == 0) lengths[s.first + row / s.rows] += s.rows;
}

__global__ void kv_set_lengths_kernel(int* lengths, int* full, int first, int count, int value) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) { lengths[first + i] = value; full[first + i] = 0; }
}

template <typename T>
__global__ void kv_to_f32_kernel(const T* __restrict__ src, float* __restrict__ dst, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = to_f32<T>(src[i]);
}

}  // namespace
}  // namespace moe

using namespace moe;

struct kv_cache {
  kv_cache_config_t cfg{};
  void* keys = nullptr;
  void* values = nullptr;
  int* lengths = nullptr;           // device, one per sequence
  int* full = nullptr;              // device, one per sequence: set by a step that found no room (a replayed graph can get there)
  std::vector<int> host_full;
  std::vector<int> host_len;        // mirror: every change goes through this object
  float* cos_t = nullptr;
  float* sin_t = nullptr;
  float* part = nullptr;            // slice results, grown on demand
  size_t part_floats = 0;
  float* read_buf = nullptr;
  size_t read_floats = 0;
  int sm_count = 148;
  std::string err;
};

namespace {

int kv_fail(kv_cache* c, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (c) c->err = buf;
  return code;
}

#define KCK(call)                                                                                          \
  do {                                                                                                     \
    cudaError_t e_ = (call);                                                                               \
    if (e_ != cudaSuccess) return kv_fail(c, MOE_CUDA_ERROR, "%s failed: %s", #call, cudaGetErrorString(e_)); \
  } while (0)

size_t elem_size(const kv_cache* c) { return c->cfg.precision == MOE_PRECISION_BF16 ? 2 : 4; }

bool head_dim_ok(int hd) { return hd == 8 || hd == 16 || hd == 32 || hd == 64 || hd == 128 || hd == 256; }

// KV_B200_SCALAR=1 keeps the bf16 cache on the scalar kernel (for comparison).
bool kv_scalar_only() {
  static const bool on = [] { const char* v = getenv("KV_B200_SCALAR"); return v && atoi(v) != 0; }();
  return on;
}

template <int HD>
cudaError_t launch_partial_tc(const kv_cache* c, const bf16* q, const bf16* k, const bf16* v, KvShape s, int n_seq,
                              int splits, float scale_log2, cudaStream_t st) {
  const size_t smem = std::max((size_t)TC_WARPS * TC_DEPTH * 2 * TC_KB * HD * 2, sizeof(float) * 16 * TC_WARPS * (HD + 2));
  // the opt-in is an attribute of the kernel on the CURRENT device: one flag per device
  static bool configured[64] = {};
  const int dev = c->cfg.device;
  if (smem > 48 * 1024 && !(dev >= 0 && dev < 64 && configured[dev])) {
    cudaError_t e = cudaFuncSetAttribute(kv_partial_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  kv_partial_tc_kernel<HD><<<dim3(splits, s.Hkv, n_seq), TC_WARPS * 32, smem, st>>>(
      q, k, v, (bf16*)c->keys, (bf16*)c->values, c->cos_t, c->sin_t, c->lengths, c->full, c->part, s, splits, scale_log2, c->cfg.rope);
  count_launch();
  return cudaGetLastError();
}

// The tensor-core kernel rotates and appends by itself; the scalar one needs kv_append_kernel first.
template <typename T>
bool takes_tc_path(int head_dim) { return sizeof(T) == 2 && !kv_scalar_only() && (head_dim == 64 || head_dim == 128); }

template <typename T>
cudaError_t launch_partial(const kv_cache* c, const T* q, const T* k, const T* v, KvShape s, int n_seq, int splits,
                           cudaStream_t st) {
  const float scale_log2 = LOG2E / sqrtf((float)s.HD);   // attention.rs:294-296
  if (takes_tc_path<T>(s.HD)) {
    if (s.HD == 64) return launch_partial_tc<64>(c, (const bf16*)q, (const bf16*)k, (const bf16*)v, s, n_seq, splits, scale_log2, st);
    return launch_partial_tc<128>(c, (const bf16*)q, (const bf16*)k, (const bf16*)v, s, n_seq, splits, scale_log2, st);
  }
  const dim3 grid(splits, s.Hkv, n_seq);
#define KV_CASE(HDV)                                                                                         \
  case HDV: {                                                                                                \
    const size_t smem = std::max(sizeof(float) * KV_QT * (KV_WARPS * (32 / (HDV / 8))) * (HDV + 2),          \
                                 (size_t)KvRing<T>::DEPTH * 2 * KV_THREADS * 8 * sizeof(T));                 \
    kv_partial_kernel<T, HDV><<<grid, KV_THREADS, smem, st>>>(q, (const T*)c->keys, (const T*)c->values,     \
                                                               c->lengths, c->full, c->part, s, splits,      \
                                                               scale_log2);                                  \
    break;                                                                                                   \
  }
  switch (s.HD) {
    KV_CASE(8) KV_CASE(16) KV_CASE(32) KV_CASE(64) KV_CASE(128) KV_CASE(256)
    default: return cudaErrorInvalidValue;
  }
#undef KV_CASE
  count_launch();
  return cudaGetLastError();
}

template <typename T>
int forward_t(kv_cache* c, int first, int n_seq, void* q, const void* k, const void* v, int rows, void* merged,
              cudaStream_t st) {
  const kv_cache_config_t& g = c->cfg;
  KvShape s{g.num_heads, g.kv_heads, g.head_dim, g.capacity, rows, first};
  int longest = 0;
  for (int i = 0; i < n_seq; ++i) longest = std::max(longest, c->host_len[first + i] + rows);
  // about eight CTAs per SM (two or three are resident: several waves even out the tail), slices of at least 128 positions
  long long ctas = (long long)n_seq * g.kv_heads;
  int splits = (int)std::min<long long>(KV_MAX_SPLITS, std::max<long long>(1, (8ll * c->sm_count + ctas - 1) / ctas));
  splits = std::max(1, std::min(splits, (longest + 127) / 128));
  if (const char* v = getenv("KV_B200_SPLITS")) splits = std::max(1, std::min(KV_MAX_SPLITS, atoi(v)));   // experiments
  const size_t need = (size_t)n_seq * rows * g.num_heads * splits * (g.head_dim + 2);
  if (need > c->part_floats) {
    // Only a prefill (several rows per sequence) gets here: the buffer made at creation holds a decode step
    // of every sequence at the largest slice count.  Growing allocates, which a capturing stream may not do.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
      return kv_fail(c, MOE_UNSUPPORTED, "Unsupported: this step needs a larger slice buffer (%zu floats); run it once outside stream capture", need);
    if (c->part) { KCK(cudaStreamSynchronize(st)); cudaFree(c->part); c->part = nullptr; c->part_floats = 0; }
    if (cudaMalloc(&c->part, need * sizeof(float)) != cudaSuccess) {
      cudaGetLastError();
      return kv_fail(c, MOE_OUT_OF_MEMORY, "OutOfMemory: %zu bytes for the slice results", need * sizeof(float));
    }
    c->part_floats = need;
  }
  if (!takes_tc_path<T>(g.head_dim)) {
    kv_append_kernel<T><<<n_seq * rows, 128, 0, st>>>((T*)q, (const T*)k, (const T*)v, (T*)c->keys, (T*)c->values,
                                                      c->lengths, c->cos_t, c->sin_t, s, g.rope);
    count_launch();
    KCK(cudaGetLastError());
  }
  KCK(launch_partial<T>(c, (const T*)q, (const T*)k, (const T*)v, s, n_seq, splits, st));
  kv_merge_kernel<T><<<n_seq * rows * g.num_heads, std::min(256, std::max(32, g.head_dim)), 0, st>>>(
      c->part, (T*)merged, c->lengths, c->full, s, splits);
  count_launch();
  KCK(cudaGetLastError());
  for (int i = 0; i < n_seq; ++i) c->host_len[first + i] += rows;
  return MOE_OK;
}

}  // namespace

extern "C" {

int32_t kv_cache_create(const kv_cache_config_t* config, kv_cache_t** out) {
  if (!config || !out) return MOE_INVALID_INPUT;
  *out = nullptr;
  kv_cache* c = new (std::nothrow) kv_cache();
  if (!c) return MOE_OUT_OF_MEMORY;
  *out = c;   // kept on failure so that the message can be read; the caller destroys it
  c->cfg = *config;
  const kv_cache_config_t& g = c->cfg;
  if (g.sequences <= 0 || g.capacity <= 0) return kv_fail(c, MOE_INVALID_CONFIG, "InvalidConfig: sequences and capacity must be positive");
  if (g.num_heads <= 0 || g.kv_heads <= 0) return kv_fail(c, MOE_INVALID_CONFIG, "InvalidConfig: attention needs at least one head");
  if (g.kv_heads > g.num_heads || g.num_heads % g.kv_heads != 0)
    return kv_fail(c, MOE_INVALID_CONFIG, "InvalidConfig: num_heads (%d) must be a multiple of num_kv_heads (%d)", g.num_heads, g.kv_heads);
  if (g.head_dim <= 0 || g.head_dim % 2 != 0)
    return kv_fail(c, MOE_INVALID_CONFIG, "InvalidConfig: rope head_dim must be even and non-zero, got %d", g.head_dim);
  if (!head_dim_ok(g.head_dim)) return kv_fail(c, MOE_UNSUPPORTED, "Unsupported: head_dim %d (8, 16, 32, 64, 128, 256)", g.head_dim);
  if (g.precision != MOE_PRECISION_F32 && g.precision != MOE_PRECISION_BF16)
    return kv_fail(c, MOE_INVALID_CONFIG, "InvalidConfig: precision is f32 or bf16");
  if (g.max_seq_len < g.capacity) return kv_fail(c, MOE_INVALID_CONFIG, "InvalidConfig: capacity %d exceeds max_seq_len %d", g.capacity, g.max_seq_len);
  KCK(cudaSetDevice(g.device));
  cudaDeviceProp prop;
  KCK(cudaGetDeviceProperties(&prop, g.device));
  c->sm_count = prop.multiProcessorCount;
  const size_t bytes = (size_t)g.sequences * g.capacity * g.kv_heads * g.head_dim * elem_size(c);
  if (cudaMalloc(&c->keys, bytes) != cudaSuccess || cudaMalloc(&c->values, bytes) != cudaSuccess) {
    cudaGetLastError();
    return kv_fail(c, MOE_OUT_OF_MEMORY, "OutOfMemory: two cache buffers of %zu bytes", bytes);
  }
  KCK(cudaMalloc(&c->lengths, sizeof(int) * g.sequences));
  KCK(cudaMemset(c->lengths, 0, sizeof(int) * g.sequences));
  KCK(cudaMalloc(&c->full, sizeof(int) * g.sequences));
  KCK(cudaMemset(c->full, 0, sizeof(int) * g.sequences));
  c->host_len.assign(g.sequences, 0);
  c->host_full.assign(g.sequences, 0);
  // slice results of one decode step (one row per sequence) at the largest slice count, so that a serving
  // loop never allocates; a prefill with more rows grows it once
  c->part_floats = (size_t)g.sequences * g.num_heads * KV_MAX_SPLITS * (g.head_dim + 2);
  if (cudaMalloc(&c->part, c->part_floats * sizeof(float)) != cudaSuccess) {
    cudaGetLastError();
    c->part = nullptr; c->part_floats = 0;
    return kv_fail(c, MOE_OUT_OF_MEMORY, "OutOfMemory: slice results");
  }
  // the tables of Rope::new (rope.rs:77-90), in f32 arithmetic like the reference
  const int half = g.head_dim / 2;
  std::vector<float> co((size_t)g.max_seq_len * half), si((size_t)g.max_seq_len * half);
  for (int p = 0; p < g.max_seq_len; ++p)
    for (int ch = 0; ch < half; ++ch) {
      const float frequency = powf(g.rope_base, -2.0f * (float)ch / (float)g.head_dim);
      const float angle = (float)p * frequency;
      co[(size_t)p * half + ch] = cosf(angle);
      si[(size_t)p * half + ch] = sinf(angle);
    }
  KCK(cudaMalloc(&c->cos_t, co.size() * sizeof(float)));
  KCK(cudaMalloc(&c->sin_t, si.size() * sizeof(float)));
  KCK(cudaMemcpy(c->cos_t, co.data(), co.size() * sizeof(float), cudaMemcpyHostToDevice));
  KCK(cudaMemcpy(c->sin_t, si.data(), si.size() * sizeof(float), cudaMemcpyHostToDevice));
  // the largest shared-memory request of the partial kernel is below the default limit for every head_dim
  return MOE_OK;
}

void kv_cache_destroy(kv_cache_t* c) {
  if (!c) return;
  cudaFree(c->keys); cudaFree(c->values); cudaFree(c->lengths); cudaFree(c->full); cudaFree(c->cos_t); cudaFree(c->sin_t);
  cudaFree(c->part); cudaFree(c->read_buf);
  delete c;
}

const char* kv_cache_last_error(const kv_cache_t* c) { return c ? c->err.c_str() : "null cache"; }

int32_t kv_cache_truncate(kv_cache_t* c, int32_t sequence, int32_t length, void* stream) {
  if (!c) return MOE_INVALID_INPUT;
  const int S = c->cfg.sequences;
  if (sequence >= S || length < 0) return kv_fail(c, MOE_INVALID_INPUT, "InvalidInput: sequence %d, length %d", sequence, length);
  const int first = sequence < 0 ? 0 : sequence, count = sequence < 0 ? S : 1;
  for (int i = 0; i < count; ++i)
    if (c->host_len[first + i] < length)
      return kv_fail(c, MOE_INVALID_INPUT, "InvalidInput: sequence %d holds %d positions, cannot keep %d", first + i, c->host_len[first + i], length);
  kv_set_lengths_kernel<<<ceil_div(count, 256), 256, 0, (cudaStream_t)stream>>>(c->lengths, c->full, first, count, length);
  count_launch();
  KCK(cudaGetLastError());
  for (int i = 0; i < count; ++i) c->host_len[first + i] = length;
  return MOE_OK;
}

int32_t kv_cache_clear(kv_cache_t* c, int32_t sequence, void* stream) { return kv_cache_truncate(c, sequence, 0, stream); }

int32_t kv_cache_lengths(kv_cache_t* c, int32_t* lengths_host, void* stream) {
  if (!c || !lengths_host) return MOE_INVALID_INPUT;
  KCK(cudaMemcpyAsync(lengths_host, c->lengths, sizeof(int) * c->cfg.sequences, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  KCK(cudaMemcpyAsync(c->host_full.data(), c->full, sizeof(int) * c->cfg.sequences, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  KCK(cudaStreamSynchronize((cudaStream_t)stream));
  // the device is the truth: a step replayed from a CUDA graph advances it without passing through here
  for (int i = 0; i < c->cfg.sequences; ++i) c->host_len[i] = lengths_host[i];
  // ... and such a step can run into the end of a cache, which only the device sees: the kernels then leave the
  // cache, the lengths and the tables alone and mark the sequence; the mark is reported and cleared here
  for (int i = 0; i < c->cfg.sequences; ++i)
    if (c->host_full[i]) {
      KCK(cudaMemsetAsync(c->full, 0, sizeof(int) * c->cfg.sequences, (cudaStream_t)stream));
      KCK(cudaStreamSynchronize((cudaStream_t)stream));
      return kv_fail(c, MOE_INVALID_INPUT, "SequenceTooLong: a step found the cache of sequence %d full at length %d of %d; the step was skipped for it (output zeros, nothing stored)",
                     i, c->host_len[i], c->cfg.capacity);
    }
  return MOE_OK;
}

int32_t kv_attention_forward_cached(kv_cache_t* c, int32_t first, int32_t n_seq, void* q, const void* k, const void* v,
                                    int32_t rows, void* merged, void* stream) {
  if (!c) return MOE_INVALID_INPUT;
  const kv_cache_config_t& g = c->cfg;
  if (first < 0 || n_seq <= 0 || first + n_seq > g.sequences)
    return kv_fail(c, MOE_INVALID_INPUT, "InvalidInput: sequences %d .. %d of %d", first, first + n_seq - 1, g.sequences);
  if (rows <= 0 || !q || !k || !v || !merged) return kv_fail(c, MOE_INVALID_INPUT, "InvalidInput: empty step or null buffer");
  if ((long long)n_seq * rows * g.num_heads > 0x7fffffffll) return kv_fail(c, MOE_INVALID_INPUT, "InvalidInput: too many rows");
  for (int i = 0; i < n_seq; ++i)
    if (c->host_len[first + i] + rows > g.capacity)
      return kv_fail(c, MOE_INVALID_INPUT, "SequenceTooLong: length %d, max_seq_len %d (sequence %d)", c->host_len[first + i] + rows, g.capacity, first + i);
  KCK(cudaSetDevice(g.device));
  return g.precision == MOE_PRECISION_BF16 ? forward_t<bf16>(c, first, n_seq, q, k, v, rows, merged, (cudaStream_t)stream)
                                           : forward_t<float>(c, first, n_seq, q, k, v, rows, merged, (cudaStream_t)stream);
}

int32_t kv_cache_read(kv_cache_t* c, int32_t sequence, float* keys_host, float* values_host, void* stream) {
  if (!c || sequence < 0 || sequence >= c->cfg.sequences) return MOE_INVALID_INPUT;
  const kv_cache_config_t& g = c->cfg;
  const size_t W = (size_t)g.kv_heads * g.head_dim, n = (size_t)c->host_len[sequence] * W;
  if (n == 0) return MOE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (n > c->read_floats) {
    cudaFree(c->read_buf);
    c->read_buf = nullptr; c->read_floats = 0;
    KCK(cudaMalloc(&c->read_buf, n * sizeof(float)));
    c->read_floats = n;
  }
  for (int which = 0; which < 2; ++which) {
    float* host = which == 0 ? keys_host : values_host;
    if (!host) continue;
    const char* src = (const char*)(which == 0 ? c->keys : c->values) + (size_t)sequence * g.capacity * W * elem_size(c);
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (g.precision == MOE_PRECISION_BF16) kv_to_f32_kernel<bf16><<<blocks, 256, 0, st>>>((const bf16*)src, c->read_buf, (long long)n);
    else kv_to_f32_kernel<float><<<blocks, 256, 0, st>>>((const float*)src, c->read_buf, (long long)n);
    KCK(cudaGetLastError());
    KCK(cudaMemcpyAsync(host, c->read_buf, n * sizeof(float), cudaMemcpyDeviceToHost, st));
    KCK(cudaStreamSynchronize(st));
  }
  return MOE_OK;
}

}  // extern "C"
