// Fused router and device-side dispatch.
//
//   router_kernel   logits = x W_r^T, softmax + log-sum-exp, dropless top-k,
//                   renormalised gates, and per-block partial sums for the Switch
//                   load-balancing loss and the ST-MoE z-loss, plus the per-block
//                   expert histogram the dispatch needs.
//                   Replaces Router::forward + softmax_rows + route + the stats
//                   half of auxiliary_losses (reference moe.rs:262-264, 553-593,
//                   602-639; device kernels softmax_lse / topk_gate / moe_stats,
//                   cuda_training.rs:291-292, 313).
//   finalize_kernel reduces the partials in a fixed order (no float atomics), forms
//                   the two losses, and scans the histogram into per-(block, expert)
//                   write cursors, compact offsets and 128-row padded group offsets.
//                   Replaces the host pass of gpu_model.rs:2474-2507.
//   permute_kernel  stable counting-sort placement of every (token, rank) slot and
//                   the row gather with 16-byte vector copies (moe.rs:266-279,
//                   gather_rows in cuda_training.rs:70).
//
// Selection is done on probabilities with a strict '>' so ties go to the lowest
// expert index, exactly as the reference.  The exponentials follow the host libm's
// own algorithm (expf_libm below) and the row sum is accumulated sequentially in
// expert order, so the probabilities (and therefore the chosen experts) agree bit
// for bit with a host evaluation of the same logits.

#include <algorithm>
#include <cstdlib>

#include "kernels.cuh"

namespace moe {


// Single-precision exp evaluated the way the GNU C library does it (the published
// algorithm of its flt-32 expf: x*32/ln2 split into an integer and a remainder by
// the 1.5*2^52 shift, a 32-entry table of 2^(i/32), a cubic in the remainder, all
// in double, one final rounding to f32).  That routine is not correctly rounded in
// about one case in a thousand; reproducing its arithmetic is what makes the
// device probabilities - and with them the top-k decisions - equal bit for bit to
// a host evaluation with libm, which is what the reference's f32::exp calls.
__device__ const unsigned long long kExp2Tab[32] = {
    0x3ff0000000000000ULL, 0x3fefd9b0d3158574ULL, 0x3fefb5586cf9890fULL, 0x3fef9301d0125b51ULL,
    0x3fef72b83c7d517bULL, 0x3fef54873168b9aaULL, 0x3fef387a6e756238ULL, 0x3fef1e9df51fdee1ULL,
    0x3fef06fe0a31b715ULL, 0x3feef1a7373aa9cbULL, 0x3feedea64c123422ULL, 0x3feece086061892dULL,
    0x3feebfdad5362a27ULL, 0x3feeb42b569d4f82ULL, 0x3feeab07dd485429ULL, 0x3feea47eb03a5585ULL,
    0x3feea09e667f3bcdULL, 0x3fee9f75e8ec5f74ULL, 0x3feea11473eb0187ULL, 0x3feea589994cce13ULL,
    0x3feeace5422aa0dbULL, 0x3feeb737b0cdc5e5ULL, 0x3feec49182a3f090ULL, 0x3feed503b23e255dULL,
    0x3feee89f995ad3adULL, 0x3feeff76f2fb5e47ULL, 0x3fef199bdd85529cULL, 0x3fef3720dcef9069ULL,
    0x3fef5818dcfba487ULL, 0x3fef7c97337b9b5fULL, 0x3fefa4afa2a490daULL, 0x3fefd0765b6e4540ULL};

// `table(i)` returns entry i of kExp2Tab (from memory, or from wherever the caller keeps a copy).
template <typename Table>
__device__ __forceinline__ float expf_libm_with(float x, Table table) {
  if (!(fabsf(x) < 88.0f)) {
    if (x == -INFINITY) return 0.f;
    if (!(fabsf(x) < INFINITY)) return x + x;
    if (x > 0x1.62e42ep6f) return INFINITY;
    if (x < -0x1.9fe368p6f) return 0.f;
    if (x < -0x1.9d1d9ep6f) return 0x1p-149f;
  }
  constexpr double kInvLn2N = 0x1.71547652b82fep+0 * 32.0;
  constexpr double kShift = 0x1.8p52;
  constexpr double c0 = 0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0;
  constexpr double c1 = 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0;
  constexpr double c2 = 0x1.62e42ff0c52d6p-1 / 32.0;
  const double z = __dmul_rn(kInvLn2N, (double)x);
  double kd = __dadd_rn(z, kShift);
  const unsigned long long ki = (unsigned long long)__double_as_longlong(kd);
  kd = __dsub_rn(kd, kShift);
  const double r = __dsub_rn(z, kd);
  const unsigned long long t = table((int)(ki & 31)) + (ki << 47);
  const double s = __longlong_as_double((long long)t);
  const double p = fma(c0, r, c1);
  const double r2 = __dmul_rn(r, r);
  double y = fma(c2, r, 1.0);
  y = fma(p, r2, y);
  y = __dmul_rn(y, s);
  return (float)y;
}
__device__ __forceinline__ float expf_libm(float x) {
  return expf_libm_with(x, [](int i) { return kExp2Tab[i]; });
}

constexpr int RT_THREADS = 256;
constexpr int RT_KC = 32;

// One block.  hist[b][e] becomes the padded-row write cursor of block b for expert e.
constexpr int FIN_THREADS = 1024;
// Plain pointers: the single-block router calls this on what it has just written itself.
__device__ __forceinline__ void finalize_body(const float* partial, int* hist, int nb, int E, int k, float aux_w,
                                              float z_w, RouteMeta meta, float* stats /*[E+2]: sums, lse2, V*/,
                                              float* losses /*[2]*/, int align, int add_base) {
  __shared__ int s_counts[MAX_EXPERTS];
  __shared__ float s_sums[MAX_EXPERTS + 2];
  __shared__ double seg_d[FIN_THREADS + 64];   // [parts][E + 2] partial statistics
  __shared__ int seg_i[FIN_THREADS];           // [parts][E] rows per expert in a run of router blocks
  const int tid = threadIdx.x;
  // The router blocks are cut into `parts` consecutive runs, one thread per (run, column): the
  // statistics are summed per run and then over the runs in order (in double, so the association does
  // not show in the f32 result); the per-expert cursors take one pass for the run totals and a second
  // one that writes the exclusive prefix.
  {
    const int cols = E + 2, parts = max(1, (int)blockDim.x / cols), seg = ceil_div(nb, parts);
    const int part = tid / cols, e = tid - part * cols;
    if (cols > (int)blockDim.x) {                    // more columns than threads: one run, strided columns
      for (int c = tid; c < cols; c += blockDim.x) {
        double sum = 0.0;
        for (int b = 0; b < nb; ++b) sum += (double)partial[(size_t)b * cols + c];
        seg_d[c] = sum;
      }
    } else if (part < parts) {
      double sum = 0.0;
      const int lo = part * seg, hi = min(nb, lo + seg);
      for (int b0 = lo; b0 < hi; b0 += 8) {          // eight independent loads, then the ordered sum
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = b0 + i < hi ? partial[(size_t)(b0 + i) * cols + e] : 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) if (b0 + i < hi) sum += (double)v[i];
      }
      seg_d[part * cols + e] = sum;
    }
    __syncthreads();
    for (int c = tid; c < cols; c += blockDim.x) {
      double t = 0.0;
      for (int p = 0; p < (cols > (int)blockDim.x ? 1 : parts); ++p) t += seg_d[p * cols + c];
      s_sums[c] = (float)t;
      stats[c] = (float)t;
    }
  }
  {
    const int parts = max(1, (int)blockDim.x / E), seg = ceil_div(nb, parts);
    const int part = tid / E, e = tid - part * E;
    const int lo = part * seg, hi = min(nb, lo + seg);
    if (part < parts) {
      int run = 0;
      for (int b0 = lo; b0 < hi; b0 += 8) {
        int h[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = b0 + i < hi ? hist[(size_t)(b0 + i) * E + e] : 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) run += h[i];
      }
      seg_i[part * E + e] = run;
    }
    __syncthreads();
    if (part < parts) {
      int run = 0;
      for (int p = 0; p < part; ++p) run += seg_i[p * E + e];
      for (int b0 = lo; b0 < hi; b0 += 8) {
        int h[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = b0 + i < hi ? hist[(size_t)(b0 + i) * E + e] : 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (b0 + i < hi) hist[(size_t)(b0 + i) * E + e] = run;
          run += h[i];
        }
      }
      if (part == parts - 1) {        // the last run ends at the expert's total
        s_counts[e] = run;
        meta.counts[e] = run;
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    int off = 0, pad = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      meta.offsets[e] = off;
      meta.pad_off[e] = pad;
      meta.tile_start[e] = tiles;
      off += s_counts[e];
      const int padded = round_up(s_counts[e], align);
      pad += padded;
      tiles += ceil_div(padded, GROUP_ALIGN);
    }
    meta.offsets[E] = off;
    meta.pad_off[E] = pad;
    meta.tile_start[E] = tiles;
    const int V = (int)s_sums[E + 1];
    meta.total[0] = off;
    meta.total[1] = pad;
    meta.total[2] = tiles;
    meta.total[3] = V;
    // auxiliary_losses (moe.rs:602-639) over the rows this device saw.
    const float* sums = s_sums;
    const float Vf = (float)V;
    float aux = 0.f, z = 0.f;
    if (Vf > 0.f) {
      const float slots = Vf * (float)k;
      for (int e = 0; e < E; ++e) {
        const float load = (float)s_counts[e] / slots;
        const float mass = sums[e] / Vf;
        aux += load * mass;
      }
      aux *= (float)E * aux_w;
      z = z_w * sums[E] / Vf;
    }
    losses[0] = aux;
    losses[1] = z;
  }
  if (add_base) {   // few blocks: the cursors get their group base here instead of in a second launch
    __syncthreads();
    for (int i = tid; i < nb * E; i += blockDim.x) hist[i] += meta.pad_off[i % E];
  }
}

__global__ void __launch_bounds__(FIN_THREADS)
finalize_kernel(const float* partial, int* hist, int nb, int E, int k, float aux_w, float z_w, RouteMeta meta,
                float* stats, float* losses, int align, int add_base) {
  finalize_body(partial, hist, nb, E, k, aux_w, z_w, meta, stats, losses, align, add_base);
}

template <typename T, int EPT, bool FROM_LOGITS>
__global__ void __launch_bounds__(RT_THREADS)
router_kernel(const T* __restrict__ x, const float* __restrict__ w_router, const float* __restrict__ logits_in,
              const uint8_t* __restrict__ valid, int tokens, int d, int E, int k, float* __restrict__ logits_out,
              float* __restrict__ probs, float* __restrict__ lse, int* __restrict__ expert_of,
              float* __restrict__ gates, float* partial /*[nb, E+2]*/, int* hist /*[nb,E]*/, RouterFinalize fin) {
  pdl_enter();
  extern __shared__ float rt_smem[];
  const int ldl = E + 1;
  float* lg = rt_smem;                          // [64][E+1] logits, then probabilities
  float* xs = lg + ROUTER_ROWS * ldl;           // [64][KC+1]
  float* ws = xs + ROUTER_ROWS * (RT_KC + 1);   // [E][KC+1]
  int* sel = reinterpret_cast<int*>(ws + (size_t)E * (RT_KC + 1));   // [64][k]
  float* row_lse = reinterpret_cast<float*>(sel + ROUTER_ROWS * k);  // [64]
  int* row_valid = reinterpret_cast<int*>(row_lse + ROUTER_ROWS);    // [64]

  const int t0 = blockIdx.x * ROUTER_ROWS;
  const int rows = min(ROUTER_ROWS, tokens - t0);
  const int tid = threadIdx.x;

  if (FROM_LOGITS) {
    for (int i = tid; i < ROUTER_ROWS * E; i += RT_THREADS) {
      const int r = i / E, e = i - r * E;
      lg[r * ldl + e] = r < rows ? logits_in[(size_t)(t0 + r) * E + e] : 0.f;
    }
  } else {
    const int tx = tid & 15, ty = tid >> 4;  // 16 expert lanes x 16 row groups of 4
    float acc[4][EPT];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < EPT; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < d; k0 += RT_KC) {
      for (int i = tid; i < ROUTER_ROWS * RT_KC; i += RT_THREADS) {
        const int r = i / RT_KC, c = i - r * RT_KC;
        xs[r * (RT_KC + 1) + c] = (r < rows && k0 + c < d) ? to_f32<T>(x[(size_t)(t0 + r) * d + k0 + c]) : 0.f;
      }
      for (int i = tid; i < E * RT_KC; i += RT_THREADS) {
        const int e = i / RT_KC, c = i - e * RT_KC;
        ws[e * (RT_KC + 1) + c] = (k0 + c < d) ? w_router[(size_t)e * d + k0 + c] : 0.f;
      }
      __syncthreads();
#pragma unroll 8
      for (int c = 0; c < RT_KC; ++c) {
        float xv[4], wv[EPT];
#pragma unroll
        for (int i = 0; i < 4; ++i) xv[i] = xs[(ty * 4 + i) * (RT_KC + 1) + c];
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
          const int e = tx + 16 * j;
          wv[j] = e < E ? ws[e * (RT_KC + 1) + c] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < EPT; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
      }
      __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < EPT; ++j) {
        const int e = tx + 16 * j;
        if (e < E) lg[(ty * 4 + i) * ldl + e] = acc[i][j];
      }
  }
  __syncthreads();

  // Four adjacent lanes per token row.  Everything that has an order in the reference keeps it: the
  // denominator is summed by one lane in expert order, and the top-k scan (strict `>`, lowest index
  // on ties, moe.rs:549-574) is split into four contiguous index ranges whose winners are merged in
  // range order, which selects the same expert as one scan over all of them.
  {
    const int r = tid >> 2, part = tid & 3;
    const int lane = tid & 31, lead = lane & ~3;
    const unsigned gmask = 0xFu << lead;
    int is_valid = 0;
    if (r < rows) {
      const int t = t0 + r;
      float* row = lg + r * ldl;
      if (logits_out)
        for (int e = part; e < E; e += 4) logits_out[(size_t)t * E + e] = row[e];
      float mx = -INFINITY;
      for (int e = part; e < E; e += 4) mx = fmaxf(mx, row[e]);
      mx = fmaxf(mx, __shfl_xor_sync(gmask, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(gmask, mx, 2));
      for (int e = part; e < E; e += 4) row[e] = expf_libm(__fsub_rn(row[e], mx));
      __syncwarp(gmask);
      float sum = 0.f;
      if (part == 0)
        for (int e = 0; e < E; ++e) sum = __fadd_rn(sum, row[e]);
      sum = __shfl_sync(gmask, sum, lead);
      const float l = mx + logf(sum);
      for (int e = part; e < E; e += 4) {
        const float p = sum > 0.f ? __fdiv_rn(row[e], sum) : row[e];
        row[e] = p;
        probs[(size_t)t * E + e] = p;
      }
      __syncwarp(gmask);
      is_valid = (valid == nullptr || valid[t] != 0) ? 1 : 0;
      int* s = sel + r * k;
      if (part == 0) { lse[t] = l; row_lse[r] = l; }
      if (!is_valid) {
        for (int j = part; j < k; j += 4) {
          s[j] = -1;
          expert_of[(size_t)t * k + j] = -1;
          gates[(size_t)t * k + j] = 0.f;
        }
      } else {
        const int span = (E + 3) / 4;                 // <= 64: one bit per expert of this lane's range
        const int q0 = min(E, part * span), q1 = min(E, q0 + span);
        unsigned long long taken = 0ull;
        float total = 0.f;
        for (int j = 0; j < k; ++j) {
          int best = -1, first = -1;
          float bv = 0.f;
          for (int e = q0; e < q1; ++e) {
            if ((taken >> (e - q0)) & 1ull) continue;
            if (first < 0) first = e;
            const float v = row[e];
            if (v != v) continue;                     // a NaN never compares greater
            if (best < 0 || v > bv) { best = e; bv = v; }
          }
          int gb = -1, gfirst = -1;
          float gv = 0.f;
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            const int b = __shfl_sync(gmask, best, lead + p);
            const float v = __shfl_sync(gmask, bv, lead + p);
            const int f = __shfl_sync(gmask, first, lead + p);
            if (gfirst < 0 && f >= 0) gfirst = f;
            if (b >= 0 && (gb < 0 || v > gv)) { gb = b; gv = v; }
          }
          // the scan starts from the first free expert; if that one is NaN nothing replaces it
          if (gfirst >= 0 && (gb < 0 || row[gfirst] != row[gfirst])) gb = gfirst;
          if (gb >= q0 && gb < q1) taken |= 1ull << (gb - q0);
          if (part == 0) s[j] = gb;
          total = __fadd_rn(total, row[gb]);
        }
        __syncwarp(gmask);
        for (int j = part; j < k; j += 4) {
          const float p = row[s[j]];
          expert_of[(size_t)t * k + j] = s[j];
          gates[(size_t)t * k + j] = total > 0.f ? __fdiv_rn(p, total) : p;
        }
      }
    } else if (part == 0) {
      for (int j = 0; j < k; ++j) sel[r * k + j] = -1;
    }
    if (part == 0) row_valid[r] = is_valid;
  }
  __syncthreads();

  // Per-block partials, rows in order (deterministic): column sums of the
  // probabilities over valid rows, sum of lse^2, valid-row count, expert histogram.
  float* part = partial + (size_t)blockIdx.x * (E + 2);
  for (int e = tid; e < E; e += RT_THREADS) {
    float s = 0.f;
    int h = 0;
    for (int r = 0; r < rows; ++r)
      if (row_valid[r]) s += lg[r * ldl + e];
    for (int i = 0; i < rows * k; ++i) h += (sel[i] == e) ? 1 : 0;
    part[e] = s;
    hist[(size_t)blockIdx.x * E + e] = h;
  }
  if (tid == RT_THREADS - 1) {
    float s = 0.f;
    int v = 0;
    for (int r = 0; r < rows; ++r)
      if (row_valid[r]) { s += row_lse[r] * row_lse[r]; ++v; }
    part[E] = s;
    part[E + 1] = (float)v;
  }
  if (fin.enabled) {   // the only router block of the pass: finalize what it has just written
    __syncthreads();
    finalize_body(partial, hist, 1, E, k, fin.aux_w, fin.z_w, fin.meta, fin.stats, fin.losses, fin.align, 1);
  }
}

// Expert parallelism: every rank contributed {stats[E+2] as floats, counts[E] as ints};
// the statistics of the whole batch are their sums in rank order, and the two losses
// follow from them exactly as on one device (moe.rs:602-639 over the concatenated batch).
__global__ void ep_losses_kernel(const int* __restrict__ gathered, int ranks, int E, int k, float aux_w, float z_w,
                                 float* __restrict__ ext_stats, int* __restrict__ ext_counts, float* __restrict__ losses) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int stride = 2 * E + 2;
  for (int e = 0; e < E + 2; ++e) {
    float s = 0.f;
    for (int r = 0; r < ranks; ++r) s += __int_as_float(gathered[(size_t)r * stride + e]);
    ext_stats[e] = s;
  }
  for (int e = 0; e < E; ++e) {
    int c = 0;
    for (int r = 0; r < ranks; ++r) c += gathered[(size_t)r * stride + E + 2 + e];
    ext_counts[e] = c;
  }
  const float Vf = ext_stats[E + 1];
  float aux = 0.f, z = 0.f;
  if (Vf > 0.f) {
    const float slots = Vf * (float)k;
    for (int e = 0; e < E; ++e) aux += ((float)ext_counts[e] / slots) * (ext_stats[e] / Vf);
    aux *= (float)E * aux_w;
    z = z_w * ext_stats[E] / Vf;
  }
  losses[0] = aux;
  losses[1] = z;
}

// Expert parallelism, peer transport: the exchange plan of this rank, computed on the device from
// the gathered counts so that the pass needs no host round trip.
//   dest_base[e]  row id (owner * cap + row) of this rank's first row of global expert e
//   local_meta    row0[El+1], m-tile prefix[El+1], counts[El+1] of the experts this rank owns
// If any rank would receive more rows than its buffers hold, every rank sees the same counts and
// takes the same decision: nothing is sent (all destinations negative, empty local groups) and
// the error flag is set.
__global__ void ep_plan_kernel(const int* __restrict__ gathered, int ranks, int E, int rank, int cap,
                               int* __restrict__ dest_base, int* __restrict__ local_meta, int* __restrict__ error_flag) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int El = E / ranks, stride = 2 * E + 2;
  bool overflow = false;
  for (int p = 0; p < ranks; ++p) {
    int row = 0, tiles = 0;
    for (int l = 0; l < El; ++l) {
      const int e = p * El + l;
      int total = 0, before_me = 0;
      for (int s = 0; s < ranks; ++s) {
        const int c = gathered[(size_t)s * stride + E + 2 + e];
        if (s < rank) before_me += c;
        total += c;
      }
      dest_base[e] = p * cap + row + before_me;
      if (p == rank) {
        local_meta[l] = row;
        local_meta[(El + 1) + l] = tiles;
        local_meta[2 * (El + 1) + l] = total;
      }
      const int padded = round_up(total, GROUP_ALIGN);
      row += padded;
      tiles += padded / GROUP_ALIGN;
    }
    if (p == rank) {
      local_meta[El] = row;
      local_meta[(El + 1) + El] = tiles;
      local_meta[2 * (El + 1) + El] = 0;
    }
    overflow |= row > cap;
  }
  if (overflow) {
    for (int e = 0; e < E; ++e) dest_base[e] = -(1 << 30);
    for (int i = 0; i < 3 * (El + 1); ++i) local_meta[i] = 0;
    atomicCAS(error_flag, 0, 300);
  }
}

// Packs this rank's contribution to the exchange above: stats as float bits, then counts.
__global__ void ep_pack_stats_kernel(const float* __restrict__ stats, const int* __restrict__ counts, int E,
                                     int* __restrict__ out) {
  for (int i = threadIdx.x; i < 2 * E + 2; i += blockDim.x)
    out[i] = i < E + 2 ? __float_as_int(stats[i]) : counts[i - (E + 2)];
}

// Adds the padded group base to the cursors once pad_off is known.
__global__ void cursor_base_kernel(int* __restrict__ hist, int nb, int E, const int* __restrict__ pad_off) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < nb * E) hist[i] += pad_off[i % E];
}

// The work of block (bx, by) of a grid with `ny` blocks per 64-token group (any whole number of warps, pm_smem of
// (E + 64 k) ints).  COPY = false stops after the placement: slot_pos, row_token, row_gate, token_of, slot_of are
// written and no row is copied (the int8 decode pass gathers its token rows through row_token itself).
// expert_of, gates and cursor carry no __restrict__: the decode routing kernel below reads what other blocks of
// the same launch have written, which a read-only (non-coherent) load must not serve.
template <typename T, int KMAX, bool COPY>
__device__ __forceinline__ void permute_body(const T* __restrict__ x, const int* expert_of, const float* gates,
                                             const int* cursor /*[nb,E]*/, RouteMeta meta, int tokens, int d, int E, int k,
                                             const RowSpace x_perm, const int* __restrict__ dest_base, int* __restrict__ slot_pos /*[T*k]*/,
                                             int* __restrict__ row_token /*[Rp]*/, float* __restrict__ row_gate /*[Rp]*/,
                                             int* __restrict__ token_of /*[R]*/, int* __restrict__ slot_of, int bx, int by, int ny,
                                             int* pm_smem) {
  int* cnt = pm_smem;        // [E] running cursors
  int* spos = cnt + E;       // [64*k] padded row of every slot of this block
  const int t0 = bx * ROUTER_ROWS;
  const int rows = min(ROUTER_ROWS, tokens - t0);
  const int nslots = rows * k;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int e = tid; e < E; e += blockDim.x) cnt[e] = cursor[(size_t)bx * E + e];
  __syncthreads();
  if (warp == 0) {
    // Slots in ascending order, 32 at a time; equal experts inside a chunk are ranked
    // by lane, so the placement is the stable counting sort of the reference.
    for (int base = 0; base < nslots; base += 32) {
      const int i = base + lane;
      const int slot = t0 * k + i;
      const int e = i < nslots ? expert_of[slot] : -1;
      const unsigned peers = __match_any_sync(0xffffffffu, e);
      int pos = -1;
      if (e >= 0) {
        const int rank = __popc(peers & ((1u << lane) - 1u));
        pos = cnt[e] + rank;
      }
      __syncwarp();
      if (e >= 0 && lane == 31 - __clz(peers)) cnt[e] += __popc(peers);
      __syncwarp();
      if (i < nslots) {
        int dest = pos;
        if (pos >= 0 && by != 0) {
          if (dest_base) dest = dest_base[e] + (pos - meta.pad_off[e]);
          if (dest < 0) dest = -1;
        } else if (pos >= 0) {
          const int cpos = meta.offsets[e] + (pos - meta.pad_off[e]);
          token_of[cpos] = slot / k;
          slot_of[cpos] = slot;
          if (dest_base) {
            dest = dest_base[e] + (pos - meta.pad_off[e]);   // a row of the expert's owner
            if (dest < 0) dest = -1;                          // plan refused (a receive buffer would overflow)
          } else {
            row_token[pos] = slot / k;
            row_gate[pos] = gates[slot];
          }
        }
        spos[i] = dest;
        if (by == 0) slot_pos[slot] = dest;
      }
    }
  }
  __syncthreads();
  if (!COPY) return;

  constexpr int VEC = 16 / sizeof(T);
  const bool vec_ok = (d % VEC) == 0;
  const size_t row_bytes = (size_t)d * sizeof(T);
  if (vec_ok) {
    // One warp per token row; the row's destination pointers sit in registers (KMAX is a template
    // parameter, the loops over the slots are unrolled), each lane loads up to sixteen 16-byte chunks of
    // the row and stores them to the token's rows.
    const int cpr = d / VEC;                 // chunks per row
    // small batches: gridDim.y blocks share one 64-token group; each repeats the (cheap) ranking
    // and copies its own slice of the rows, so the copy is not one block's latency chain
    const int slice = ceil_div(rows, ny);
    const int r_begin = min(rows, by * slice), r_end = min(rows, r_begin + slice);
    constexpr int U = 16;   // 16-byte chunks per lane held at once: 8 KB of the row per pass
    for (int r = r_begin + warp; r < r_end; r += blockDim.x / 32) {
      const int* p = spos + r * k;
      if (p[0] < 0) continue;                // padding row: routed nowhere
      uint4* dst[KMAX];
#pragma unroll
      for (int j = 0; j < KMAX; ++j) {
        const int pj = j < k ? p[j] : -1;
        dst[j] = pj >= 0 ? reinterpret_cast<uint4*>(row_ptr(x_perm, pj, row_bytes)) : nullptr;
      }
      const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(t0 + r) * d);
      for (int c0 = lane; c0 < cpr; c0 += 32 * U) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (c0 + 32 * u < cpr) v[u] = src[c0 + 32 * u];
        // destination row by destination row: each row receives its 8 KB back to back, which keeps
        // the writes of one DRAM page together
#pragma unroll
        for (int j = 0; j < KMAX; ++j) {
          if (dst[j]) {
#pragma unroll
            for (int u = 0; u < U; ++u)
              if (c0 + 32 * u < cpr) dst[j][c0 + 32 * u] = v[u];
          }
        }
      }
    }
  } else {
    for (int r = warp + by * (blockDim.x / 32); r < rows; r += (blockDim.x / 32) * ny) {
      const T* src = x + (size_t)(t0 + r) * d;
      const int* p = spos + r * k;
      if (p[0] < 0) continue;
      for (int c = lane; c < d; c += 32) {
        const T v = src[c];
        for (int j = 0; j < k; ++j)
          if (p[j] >= 0) reinterpret_cast<T*>(row_ptr(x_perm, p[j], row_bytes))[c] = v;
      }
    }
  }
}

template <typename T, int KMAX>
__global__ void __launch_bounds__(256)
permute_kernel(const T* __restrict__ x, const int* expert_of, const float* gates, const int* cursor /*[nb,E]*/, RouteMeta meta,
               int tokens, int d, int E, int k, const RowSpace x_perm, const int* __restrict__ dest_base,
               int* __restrict__ slot_pos /*[T*k]*/, int* __restrict__ row_token /*[Rp]*/, float* __restrict__ row_gate /*[Rp]*/,
               int* __restrict__ token_of /*[R]*/, int* __restrict__ slot_of) {
  pdl_enter();
  extern __shared__ int pm_smem[];
  permute_body<T, KMAX, true>(x, expert_of, gates, cursor, meta, tokens, d, E, k, x_perm, dest_base, slot_pos, row_token, row_gate,
                              token_of, slot_of, (int)blockIdx.x, (int)blockIdx.y, (int)gridDim.y, pm_smem);
}

// Zeroes the padding rows at the end of every expert's group (they change place
// every step) so the tensor-core reductions over padded groups stay exact.
template <typename T>
__global__ void pad_rows_kernel(T* __restrict__ buf, int d, RouteMeta meta, int* __restrict__ row_token,
                                float* __restrict__ row_gate) {
  const int e = blockIdx.x;
  const int begin = meta.pad_off[e] + meta.counts[e];
  const int end = meta.pad_off[e + 1];
  constexpr int VEC = 16 / sizeof(T);
  if (d % VEC == 0) {
    const int cpr = d / VEC;
    uint4* base = reinterpret_cast<uint4*>(buf + (size_t)begin * d);   // rows are contiguous
    for (int i = threadIdx.x; i < (end - begin) * cpr; i += blockDim.x) base[i] = make_uint4(0, 0, 0, 0);
  } else {
    for (int r = begin; r < end; ++r)
      for (int c = threadIdx.x; c < d; c += blockDim.x) buf[(size_t)r * d + c] = from_f32<T>(0.f);
  }
  if (row_token)
    for (int r = begin + threadIdx.x; r < end; r += blockDim.x) {
      row_token[r] = -1;
      row_gate[r] = 0.f;
    }
}

// ---------------------------------------------------------------------------
// Host launchers
// ---------------------------------------------------------------------------
static size_t router_smem(int E, int k) {
  return sizeof(float) * ((size_t)ROUTER_ROWS * (E + 1) + (size_t)ROUTER_ROWS * (RT_KC + 1) + (size_t)E * (RT_KC + 1)) +
         sizeof(int) * (size_t)ROUTER_ROWS * k + sizeof(float) * ROUTER_ROWS + sizeof(int) * ROUTER_ROWS;
}

template <typename T, int EPT>
static cudaError_t launch_router_ept(const RouterArgs& a, cudaStream_t stream) {
  const int nb = ceil_div(a.tokens, ROUTER_ROWS);
  const size_t smem = router_smem(a.E, a.k);
  // the kernel also holds the 15 KB of static tables of the finalize step: opt in to more than the default
  // 48 KB as soon as the sum passes it
  RouterFinalize fin = a.fin;
  fin.enabled = (a.fin.enabled && nb == 1) ? 1 : 0;
  if (a.logits_in) {
    auto kern = router_kernel<T, EPT, true>;
    if (smem + 16 * 1024 > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(kern, dim3(nb), dim3(RT_THREADS), smem, stream, (const T*)a.x, a.w_router, a.logits_in, a.valid, a.tokens, a.d,
                  a.E, a.k, a.logits_out, a.probs, a.lse, a.expert_of, a.gates, a.partial, a.hist, fin); count_launch();
  } else {
    auto kern = router_kernel<T, EPT, false>;
    if (smem + 16 * 1024 > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(kern, dim3(nb), dim3(RT_THREADS), smem, stream, (const T*)a.x, a.w_router, a.logits_in, a.valid, a.tokens, a.d,
                  a.E, a.k, a.logits_out, a.probs, a.lse, a.expert_of, a.gates, a.partial, a.hist, fin); count_launch();
  }
  return cudaGetLastError();
}

template <typename T>
static cudaError_t launch_router_t(const RouterArgs& a, cudaStream_t stream) {
  const int ept = ceil_div(a.E, 16);
  if (ept <= 1) return launch_router_ept<T, 1>(a, stream);
  if (ept <= 2) return launch_router_ept<T, 2>(a, stream);
  if (ept <= 4) return launch_router_ept<T, 4>(a, stream);
  if (ept <= 8) return launch_router_ept<T, 8>(a, stream);
  return launch_router_ept<T, 16>(a, stream);
}

cudaError_t launch_router(const RouterArgs& a, int precision, cudaStream_t stream) {
  if (a.tokens <= 0) return cudaSuccess;
  return precision == PREC_BF16 ? launch_router_t<bf16>(a, stream) : launch_router_t<float>(a, stream);
}

cudaError_t launch_ep_plan(const int* gathered, int ranks, int E, int rank, int cap, int* dest_base, int* local_meta,
                           int* error_flag, cudaStream_t stream) {
  ep_plan_kernel<<<1, 32, 0, stream>>>(gathered, ranks, E, rank, cap, dest_base, local_meta, error_flag); count_launch();
  return cudaGetLastError();
}
cudaError_t launch_ep_pack_stats(const float* stats, const int* counts, int E, int* out, cudaStream_t stream) {
  ep_pack_stats_kernel<<<1, 256, 0, stream>>>(stats, counts, E, out); count_launch();
  return cudaGetLastError();
}
cudaError_t launch_ep_losses(const int* gathered, int ranks, int E, int k, float aux_w, float z_w, float* ext_stats,
                             int* ext_counts, float* losses, cudaStream_t stream) {
  ep_losses_kernel<<<1, 32, 0, stream>>>(gathered, ranks, E, k, aux_w, z_w, ext_stats, ext_counts, losses); count_launch();
  return cudaGetLastError();
}

// Router logits for decode-sized batches: logits[t, e] = sum_c x[t, c] * w[e, c], bf16 operands, f32
// sums.  One CTA per token row, a warp per expert (round robin), 16-byte loads; a single 128-row
// tensor-core tile would leave this to one SM and a 16-step dependent pipeline.
// Token row t by four warps (warp = 0..3 of them); out: the row's E logits.  A warp works on EG experts at once,
// 1024 reduction values at a time, and ALL 16-byte loads of such a step (4 of the token row, 4 per expert) are
// issued before the first is used: written as a plain loop the compiler chained every load to its FMAs, and the
// row took 20 L2 round trips (16000 clocks) instead of one or two.
__device__ __forceinline__ void router_logits_row(const bf16* __restrict__ x, const bf16* __restrict__ w, float* out, int d, int E,
                                                  int t, int warp, int lane) {
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)t * d);
  constexpr int EG = 4, NI = 4;
  const int cpr = d / 8;                       // 16-byte chunks per row
  for (int e0 = warp; e0 < E; e0 += 4 * EG) {
    float acc[EG];
#pragma unroll
    for (int j = 0; j < EG; ++j) acc[j] = 0.f;
    for (int c0 = lane; c0 < cpr; c0 += 32 * NI) {
      uint4 a[NI], b[EG][NI];
#pragma unroll
      for (int i = 0; i < NI; ++i) {
        const int c = c0 + 32 * i;
        a[i] = c < cpr ? __ldg(xr + c) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < EG; ++j) {
        const int e = e0 + 4 * j;
        const uint4* wr = reinterpret_cast<const uint4*>(w + (size_t)(e < E ? e : 0) * d);
#pragma unroll
        for (int i = 0; i < NI; ++i) {
          const int c = c0 + 32 * i;
          b[j][i] = (e < E && c < cpr) ? __ldg(wr + c) : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int i = 0; i < NI; ++i) {
        const uint32_t av[4] = {a[i].x, a[i].y, a[i].z, a[i].w};
#pragma unroll
        for (int j = 0; j < EG; ++j) {
          const uint32_t bv[4] = {b[j][i].x, b[j][i].y, b[j][i].z, b[j][i].w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            acc[j] = fmaf(__uint_as_float(av[q] << 16), __uint_as_float(bv[q] << 16), acc[j]);
            acc[j] = fmaf(__uint_as_float(av[q] & 0xffff0000u), __uint_as_float(bv[q] & 0xffff0000u), acc[j]);
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < EG; ++j) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
      const int e = e0 + 4 * j;
      if (lane == 0 && e < E) out[e] = acc[j];
    }
  }
}
__global__ void __launch_bounds__(128)
router_logits_rows_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, float* __restrict__ logits, int d, int E) {
  pdl_enter();
  router_logits_row(x, w, logits + (size_t)blockIdx.x * E, d, E, (int)blockIdx.x, (int)(threadIdx.x >> 5), (int)(threadIdx.x & 31));
}

// Routing of a decode-sized batch (at most 64 token rows, at most 64 experts, one GPU) in ONE launch instead of
// four (logits, softmax / top-k, finalize, permutation): one CTA of four warps per token row computes the row's
// logits (router_logits_row: the sums of router_logits_rows_kernel), then its first warp takes the softmax and the
// top-k with the arithmetic and the order of router_body (exponentials by expf_libm, the denominator summed by one
// lane in expert order, the scan with a strict `>` from the first free expert).  The CTA that finishes last - an
// atomic counter, nothing waits - sums the batch statistics in row order, runs finalize_body and the stable
// placement of permute_body.  No row is copied: the int8 projections fetch their token rows through row_token.
template <int KMAX>
__global__ void __launch_bounds__(128)
decode_route_rows_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w_bf16, RouterArgs ra, PermuteArgs pa, int* done) {
  pdl_enter();
  extern __shared__ float dr_smem[];
  __shared__ float s_row[MAX_EXPERTS];
  __shared__ unsigned long long s_tab[32];   // the exponential's table: fetched while the logits are computed
  __shared__ int s_last;
  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int E = ra.E, k = ra.k;
  if (tid < 32) s_tab[tid] = kExp2Tab[tid];
  float* logits = const_cast<float*>(ra.logits_in);
  router_logits_row(x, w_bf16, s_row, ra.d, E, t, warp, lane);
  __syncthreads();
  if (warp == 0) {
    for (int e = lane; e < E; e += 32) logits[(size_t)t * E + e] = s_row[e];
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, s_row[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    for (int e = lane; e < E; e += 32) s_row[e] = expf_libm_with(__fsub_rn(s_row[e], mx), [&](int i) { return s_tab[i]; });
    __syncwarp();
    float sum = 0.f;
    if (lane == 0)
      for (int e = 0; e < E; ++e) sum = __fadd_rn(sum, s_row[e]);
    sum = __shfl_sync(0xffffffffu, sum, 0);
    for (int e = lane; e < E; e += 32) {
      const float p = sum > 0.f ? __fdiv_rn(s_row[e], sum) : s_row[e];
      s_row[e] = p;
      ra.probs[(size_t)t * E + e] = p;
    }
    __syncwarp();
    if (lane == 0) {
      ra.lse[t] = mx + logf(sum);
      const bool is_valid = ra.valid == nullptr || ra.valid[t] != 0;
      if (!is_valid) {
        for (int j = 0; j < k; ++j) { ra.expert_of[(size_t)t * k + j] = -1; ra.gates[(size_t)t * k + j] = 0.f; }
      } else {
        unsigned long long taken = 0ull;   // E <= 64
        int chosen[KMAX];
        float total = 0.f;
#pragma unroll
        for (int j = 0; j < KMAX; ++j) {
          if (j < k) {
            int best = -1;
            for (int e = 0; e < E; ++e) {
              if ((taken >> e) & 1ull) continue;
              if (best < 0 || s_row[e] > s_row[best]) best = e;   // from the first free expert; a NaN there is never replaced
            }
            taken |= 1ull << best;
            chosen[j] = best;
            total = __fadd_rn(total, s_row[best]);
          }
        }
#pragma unroll
        for (int j = 0; j < KMAX; ++j) {
          if (j < k) {
            const float p = s_row[chosen[j]];
            ra.expert_of[(size_t)t * k + j] = chosen[j];
            ra.gates[(size_t)t * k + j] = total > 0.f ? __fdiv_rn(p, total) : p;
          }
        }
      }
    }
  }
  // the last CTA to get here does the batch-wide part
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    s_last = atomicAdd(done, 1) == (int)gridDim.x - 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (tid == 0) *done = 0;                         // ready for the next launch
  const int T = ra.tokens;
  // What the other CTAs wrote comes into shared memory in one round of loads, and everything after that works on
  // shared memory: a loop that reads global memory pays the L2 latency per step, and with finalize_body and
  // permute_body on global arrays that chain cost more than the launches it replaced.  The sums, the two losses
  // and the tables are those of router_body's tail + finalize_body for a single router block (the double sums
  // of one block are that block's values), the placement is permute_body's stable counting sort.
  float* s_probs = dr_smem;                                   // [T][E]
  float* s_lse = s_probs + (size_t)T * E;                     // [T]
  float* s_gates = s_lse + T;                                 // [T * k]
  int* s_sel = reinterpret_cast<int*>(s_gates + (size_t)T * k);   // [T * k]
  int* s_valid = s_sel + (size_t)T * k;                       // [T]
  __shared__ float s_sums[MAX_EXPERTS + 2];
  __shared__ int s_counts[MAX_EXPERTS], s_pad[MAX_EXPERTS + 1], s_off[MAX_EXPERTS + 1];
  {
    // every load of a thread is issued before its first store (eight at a time for the probabilities)
    const int nk = T * k;
    const int i1 = tid < nk ? __ldcg(ra.expert_of + tid) : -1;
    const float g1 = tid < nk ? __ldcg(ra.gates + tid) : 0.f;
    const float l1 = tid < T ? __ldcg(ra.lse + tid) : 0.f;
    const int v1 = tid < T ? ((ra.valid == nullptr || ra.valid[tid] != 0) ? 1 : 0) : 0;
    for (int base = tid; base < T * E; base += 8 * (int)blockDim.x) {
      float pv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = base + u * (int)blockDim.x;
        pv[u] = i < T * E ? __ldcg(ra.probs + i) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = base + u * (int)blockDim.x;
        if (i < T * E) s_probs[i] = pv[u];
      }
    }
    if (tid < nk) { s_sel[tid] = i1; s_gates[tid] = g1; }
    if (tid < T) { s_lse[tid] = l1; s_valid[tid] = v1; }
    for (int i = tid + (int)blockDim.x; i < nk; i += blockDim.x) { s_sel[i] = __ldcg(ra.expert_of + i); s_gates[i] = __ldcg(ra.gates + i); }
    if (tid < E) s_counts[tid] = 0;
  }
  __syncthreads();
  // rows per expert: integer counting in shared memory (the order does not matter)
  for (int i = tid; i < T * k; i += blockDim.x) {
    const int e = s_sel[i];
    if (e >= 0) atomicAdd(&s_counts[e], 1);
  }
  // column sums over the valid rows, rows in order; an invalid row adds +0, which leaves the sum as it is
  for (int e = tid; e < E; e += blockDim.x) {
    float sm = 0.f;
#pragma unroll 8
    for (int r = 0; r < T; ++r) sm += s_valid[r] ? s_probs[r * E + e] : 0.f;
    s_sums[e] = sm;
  }
  if (tid == blockDim.x - 1) {
    float sm = 0.f;
    int v = 0;
#pragma unroll 8
    for (int r = 0; r < T; ++r) { sm += s_valid[r] ? s_lse[r] * s_lse[r] : 0.f; v += s_valid[r]; }
    s_sums[E] = sm;
    s_sums[E + 1] = (float)v;
  }
  __syncthreads();
  const RouteMeta meta = ra.fin.meta;
  for (int c = tid; c < E + 2; c += blockDim.x) { ra.partial[c] = s_sums[c]; ra.fin.stats[c] = s_sums[c]; }
  for (int e = tid; e < E; e += blockDim.x) meta.counts[e] = s_counts[e];
  if (warp == 1) {
    // offsets, padded offsets and tile numbers: exclusive prefix sums over the experts, by warp scans (E <= 64:
    // two experts per lane, the second half continues from the first half's totals)
    int base_off = 0, base_pad = 0, base_tiles = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      const int c = e < E ? s_counts[e] : 0;
      const int padded = round_up(c, ra.fin.align);
      const int tl = ceil_div(padded, GROUP_ALIGN);
      int so = c, sp = padded, stl = tl;                      // inclusive scans
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int a = __shfl_up_sync(0xffffffffu, so, o), b = __shfl_up_sync(0xffffffffu, sp, o),
                  d2 = __shfl_up_sync(0xffffffffu, stl, o);
        if (lane >= o) { so += a; sp += b; stl += d2; }
      }
      if (e < E) {
        const int off = base_off + so - c, pad = base_pad + sp - padded, tiles = base_tiles + stl - tl;
        s_off[e] = off; s_pad[e] = pad;
        meta.offsets[e] = off;
        meta.pad_off[e] = pad;
        meta.tile_start[e] = tiles;
      }
      base_off += __shfl_sync(0xffffffffu, so, 31);
      base_pad += __shfl_sync(0xffffffffu, sp, 31);
      base_tiles += __shfl_sync(0xffffffffu, stl, 31);
    }
    if (lane == 0) {
      meta.offsets[E] = base_off;
      meta.pad_off[E] = base_pad;
      meta.tile_start[E] = base_tiles;
      meta.total[0] = base_off;
      meta.total[1] = base_pad;
      meta.total[2] = base_tiles;
      meta.total[3] = (int)s_sums[E + 1];
    }
  } else if (warp == 0) {
    // auxiliary_losses (moe.rs:602-639), the arithmetic of finalize_body: the quotients of all experts at once,
    // their products summed by one lane in expert order
    const int V = (int)s_sums[E + 1];
    const float Vf = (float)V;
    float aux = 0.f, z = 0.f;
    if (Vf > 0.f) {
      const float slots = Vf * (float)k;
      float ld[2], ms[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int e = lane + 32 * h;
        ld[h] = e < E ? (float)s_counts[e] / slots : 0.f;
        ms[h] = e < E ? s_sums[e] / Vf : 0.f;
      }
      for (int e = 0; e < E; ++e) {
        const float load = __shfl_sync(0xffffffffu, ld[e >> 5], e & 31);
        const float mass = __shfl_sync(0xffffffffu, ms[e >> 5], e & 31);
        aux += load * mass;
      }
      aux *= (float)E * ra.fin.aux_w;
      z = ra.fin.z_w * s_sums[E] / Vf;
    }
    if (lane == 0) {
      ra.fin.losses[0] = aux;
      ra.fin.losses[1] = z;
    }
  }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) ra.hist[e] = s_pad[e];   // the block's write cursors, as finalize leaves them
  if (warp == 0) {
    // slots in ascending order, 32 at a time; equal experts inside a chunk are ranked by lane (permute_body)
    int* cnt = s_counts;                                     // reused as running cursors
    for (int e = lane; e < E; e += 32) cnt[e] = s_pad[e];
    __syncwarp();
    const int nslots = T * k;
    for (int base = 0; base < nslots; base += 32) {
      const int i = base + lane;
      const int e = i < nslots ? s_sel[i] : -1;
      const unsigned peers = __match_any_sync(0xffffffffu, e);
      int pos = -1;
      if (e >= 0) pos = cnt[e] + __popc(peers & ((1u << lane) - 1u));
      __syncwarp();
      if (e >= 0 && lane == 31 - __clz(peers)) cnt[e] += __popc(peers);
      __syncwarp();
      if (i < nslots) {
        if (pos >= 0) {
          const int cpos = s_off[e] + (pos - s_pad[e]);
          pa.token_of[cpos] = i / k;
          pa.slot_of[cpos] = i;
          pa.row_token[pos] = i / k;
          pa.row_gate[pos] = s_gates[i];
        }
        pa.slot_pos[i] = pos;
      }
    }
  }
}

bool decode_route_supported(const RouterArgs& ra, const PermuteArgs& pa) {
  static const bool on = [] { const char* e = getenv("MOE_B200_DECODE_ROUTE"); return !(e && *e == '0'); }();
  return on && ra.tokens > 0 && ra.tokens <= ROUTER_ROWS && ra.fin.enabled && ra.logits_in && !pa.dest_base && ra.E <= 64 &&
         ra.k <= 8 && ra.k <= ra.E && ra.d % 8 == 0 && ((uintptr_t)ra.x & 15) == 0;
}

cudaError_t launch_decode_route_rows(const RouterArgs& ra, const PermuteArgs& pa, const void* w_bf16, int* done, cudaStream_t stream) {
  const size_t smem = sizeof(float) * (size_t)ROUTER_ROWS * ((size_t)ra.E + 2 + 2 * (size_t)ra.k);
  const bf16* xb = (const bf16*)ra.x;
  const bf16* wb = (const bf16*)w_bf16;
  cudaError_t e;
  if (ra.k <= 1) e = launch_kernel(decode_route_rows_kernel<1>, dim3(ra.tokens), dim3(128), smem, stream, xb, wb, ra, pa, done);
  else if (ra.k <= 2) e = launch_kernel(decode_route_rows_kernel<2>, dim3(ra.tokens), dim3(128), smem, stream, xb, wb, ra, pa, done);
  else if (ra.k <= 4) e = launch_kernel(decode_route_rows_kernel<4>, dim3(ra.tokens), dim3(128), smem, stream, xb, wb, ra, pa, done);
  else e = launch_kernel(decode_route_rows_kernel<8>, dim3(ra.tokens), dim3(128), smem, stream, xb, wb, ra, pa, done);
  count_launch();
  return e != cudaSuccess ? e : cudaGetLastError();
}
cudaError_t launch_router_logits_rows(const void* x, const void* w_bf16, float* logits, int tokens, int d, int E,
                                      cudaStream_t stream) {
  if (tokens <= 0) return cudaSuccess;
  launch_kernel(router_logits_rows_kernel, dim3(tokens), dim3(128), 0, stream, (const bf16*)x, (const bf16*)w_bf16, logits, d, E);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_finalize(const RouterArgs& a, RouteMeta meta, float aux_w, float z_w, float* stats, float* losses,
                            int align, cudaStream_t stream) {
  const int nb = ceil_div(a.tokens, ROUTER_ROWS);
  if (a.fin.enabled && nb == 1) return cudaSuccess;   // done by the router block itself
  const int fold = nb <= 16 ? 1 : 0;
  finalize_kernel<<<1, nb > 32 ? FIN_THREADS : 256, 0, stream>>>(a.partial, a.hist, nb, a.E, a.k, aux_w, z_w, meta, stats, losses, align, fold); count_launch();
  if (nb > 0 && !fold) { cursor_base_kernel<<<ceil_div(nb * a.E, 256), 256, 0, stream>>>(a.hist, nb, a.E, meta.pad_off); count_launch(); }
  return cudaGetLastError();
}

cudaError_t launch_permute(const PermuteArgs& a, int precision, cudaStream_t stream) {
  const int nb = ceil_div(a.tokens, ROUTER_ROWS);
  const size_t smem = sizeof(int) * ((size_t)a.E + (size_t)ROUTER_ROWS * a.k);
  const dim3 pgrid(nb, nb <= 16 ? 8 : 1);
  if (nb > 0) {
#define PERMUTE_LAUNCH(T, KMAX)                                                                                   \
  launch_kernel(permute_kernel<T, KMAX>, pgrid, dim3(256), smem, stream, (const T*)a.x, a.expert_of, a.gates, a.cursor, a.meta,  \
                a.tokens, a.d, a.E, a.k, a.x_perm, a.dest_base, a.slot_pos, a.row_token, a.row_gate, a.token_of, a.slot_of)
#define PERMUTE_BY_K(T)                                                                          \
  do {                                                                                           \
    if (a.k <= 1) PERMUTE_LAUNCH(T, 1);                                                          \
    else if (a.k <= 2) PERMUTE_LAUNCH(T, 2);                                                     \
    else if (a.k <= 4) PERMUTE_LAUNCH(T, 4);                                                     \
    else if (a.k <= 8) PERMUTE_LAUNCH(T, 8);                                                     \
    else PERMUTE_LAUNCH(T, 16);                                                                  \
  } while (0)
    if (precision == PREC_BF16) PERMUTE_BY_K(bf16);
    else PERMUTE_BY_K(float);
#undef PERMUTE_BY_K
#undef PERMUTE_LAUNCH
    count_launch();
  }
  if (a.dest_base || a.skip_pad) return cudaGetLastError();   // remote rows: the owners zero their own padding
  if (precision == PREC_BF16) {
    pad_rows_kernel<bf16><<<a.E, 256, 0, stream>>>((bf16*)a.x_perm.base[0], a.d, a.meta, a.row_token, a.row_gate);
  } else {
    pad_rows_kernel<float><<<a.E, 256, 0, stream>>>((float*)a.x_perm.base[0], a.d, a.meta, a.row_token, a.row_gate);
  }
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_pad_rows(void* buf, int d, RouteMeta meta, int E, int precision, cudaStream_t stream) {
  if (precision == PREC_BF16) { pad_rows_kernel<bf16><<<E, 256, 0, stream>>>((bf16*)buf, d, meta, nullptr, nullptr); count_launch(); }
  else { pad_rows_kernel<float><<<E, 256, 0, stream>>>((float*)buf, d, meta, nullptr, nullptr); count_launch(); }
  return cudaGetLastError();
}

}  // namespace moe
