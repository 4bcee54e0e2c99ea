// Row kernels of the language model around the MoE layer; see lm_kernels.cuh for the layouts.
#include "lm_kernels.cuh"

#include <float.h>

namespace moe {
namespace lm {

namespace {

__device__ __forceinline__ float bf(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ bf16 tb(float v) { return __float2bfloat16_rn(v); }

// ---------------------------------------------------------------------------
// embedding (reference embedding.rs:49-118)
// ---------------------------------------------------------------------------
__global__ void embed_gather_kernel(const uint32_t* __restrict__ ids, const bf16* __restrict__ table, bf16* __restrict__ x,
                                    int d) {
  const int r = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)ids[r] * d);
  uint4* dst = reinterpret_cast<uint4*>(x + (size_t)r * d);
  for (int c = threadIdx.x; c < d / 8; c += blockDim.x) dst[c] = src[c];
}

__global__ void embed_scatter_kernel(const uint32_t* __restrict__ ids, const bf16* __restrict__ grad_x,
                                     float* __restrict__ grad_table, const int* __restrict__ first,
                                     const int* __restrict__ next, int d) {
  const int r = blockIdx.x;
  if (!first[r]) return;
  float* dst = grad_table + (size_t)ids[r] * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float acc = 0.f;
    for (int s = r; s >= 0; s = next[s]) acc += bf(grad_x[(size_t)s * d + c]);   // rows in ascending order
    dst[c] += acc;
  }
}

// ---------------------------------------------------------------------------
// packed QKV -> head-major groups, rotate-half RoPE on queries and keys
// (reference rope.rs:12-18, 171-225; attention.rs:947-978)
// ---------------------------------------------------------------------------
__global__ void rope_pack_kernel(const bf16* __restrict__ qkv, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                 bf16* __restrict__ q_hm, bf16* __restrict__ k_hm, bf16* __restrict__ v_hm, AttnShape a) {
  const int r = blockIdx.x, b = r / a.S, s = r - b * a.S;
  const int half = a.hd / 2, qn = a.H * a.hd, kn = a.Hkv * a.hd;
  const bf16* row = qkv + (size_t)r * (qn + 2 * kn);
  const float* ct = cos_t + (size_t)s * half;
  const float* st = sin_t + (size_t)s * half;
  for (int i = threadIdx.x; i < (a.H + a.Hkv) * half; i += blockDim.x) {
    const int h = i / half, c = i - h * half;
    const float co = ct[c], si = st[c];
    if (h < a.H) {
      const float lo = bf(row[h * a.hd + c]), hi = bf(row[h * a.hd + half + c]);
      const int grp = b * a.Hkv + h / a.g, gi = h % a.g;
      bf16* dst = q_hm + ((size_t)grp * a.GR + (size_t)gi * a.S + s) * a.hd;
      dst[c] = tb(lo * co - hi * si);            // rope.rs:213-218
      dst[half + c] = tb(hi * co + lo * si);
    } else {
      const int kh = h - a.H;
      const float lo = bf(row[qn + kh * a.hd + c]), hi = bf(row[qn + kh * a.hd + half + c]);
      bf16* dst = k_hm + ((size_t)(b * a.Hkv + kh) * a.S_pad + s) * a.hd;
      dst[c] = tb(lo * co - hi * si);
      dst[half + c] = tb(hi * co + lo * si);
    }
  }
  for (int i = threadIdx.x; i < kn; i += blockDim.x) {
    const int kh = i / a.hd, c = i - kh * a.hd;
    v_hm[((size_t)(b * a.Hkv + kh) * a.S_pad + s) * a.hd + c] = row[qn + kn + i];
  }
}

// dL/dq (bf16), dL/dk, dL/dv (f32, summed over the group's query heads by the products) -> packed
// [rows, (H + 2 Hkv) * hd] bf16, with the inverse rotation on the first two (attention.rs:533-540).
__global__ void qkv_grad_unpack_kernel(const bf16* __restrict__ dq_hm, const float* __restrict__ dk_hm,
                                       const float* __restrict__ dv_hm, const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t, bf16* __restrict__ dqkv, AttnShape a) {
  const int r = blockIdx.x, b = r / a.S, s = r - b * a.S;
  const int half = a.hd / 2, qn = a.H * a.hd, kn = a.Hkv * a.hd;
  bf16* row = dqkv + (size_t)r * (qn + 2 * kn);
  const float* ct = cos_t + (size_t)s * half;
  const float* st = sin_t + (size_t)s * half;
  for (int i = threadIdx.x; i < (a.H + a.Hkv) * half; i += blockDim.x) {
    const int h = i / half, c = i - h * half;
    const float co = ct[c], si = -st[c];          // the opposite rotation
    if (h < a.H) {
      const int grp = b * a.Hkv + h / a.g, gi = h % a.g;
      const bf16* src = dq_hm + ((size_t)grp * a.GR + (size_t)gi * a.S + s) * a.hd;
      const float lo = bf(src[c]), hi = bf(src[half + c]);
      row[h * a.hd + c] = tb(lo * co - hi * si);
      row[h * a.hd + half + c] = tb(hi * co + lo * si);
    } else {
      const int kh = h - a.H;
      const float* src = dk_hm + ((size_t)(b * a.Hkv + kh) * a.S_pad + s) * a.hd;
      const float lo = src[c], hi = src[half + c];
      row[qn + kh * a.hd + c] = tb(lo * co - hi * si);
      row[qn + kh * a.hd + half + c] = tb(hi * co + lo * si);
    }
  }
  for (int i = threadIdx.x; i < kn; i += blockDim.x) {
    const int kh = i / a.hd, c = i - kh * a.hd;
    row[qn + kn + i] = tb(dv_hm[((size_t)(b * a.Hkv + kh) * a.S_pad + s) * a.hd + c]);
  }
}

// merged[r, h * hd + c] <-> o_hm[group row, c]
template <bool TO_TOKENS>
__global__ void heads_tokens_kernel(const bf16* __restrict__ src, bf16* __restrict__ dst, AttnShape a) {
  const int r = blockIdx.x, b = r / a.S, s = r - b * a.S;
  const int cph = a.hd / 8;   // 16-byte chunks per head
  for (int i = threadIdx.x; i < a.H * cph; i += blockDim.x) {
    const int h = i / cph, c = i - h * cph;
    const int grp = b * a.Hkv + h / a.g, gi = h % a.g;
    const size_t hm = (((size_t)grp * a.GR + (size_t)gi * a.S + s) * a.hd) / 8 + c;
    const size_t tk = ((size_t)r * a.H * a.hd + (size_t)h * a.hd) / 8 + c;
    if (TO_TOKENS) reinterpret_cast<uint4*>(dst)[tk] = reinterpret_cast<const uint4*>(src)[hm];
    else reinterpret_cast<uint4*>(dst)[hm] = reinterpret_cast<const uint4*>(src)[tk];
  }
}

__global__ void attn_meta_kernel(int* meta, int groups, int group_rows) {
  for (int i = threadIdx.x; i <= groups; i += blockDim.x) {
    meta[i] = i * group_rows;                                   // group_row0
    meta[groups + 1 + i] = i * (group_rows / GROUP_ALIGN);      // tile_start
  }
}

}  // namespace

namespace {

// ---------------------------------------------------------------------------
// softmax over the visible prefix of every score row, and its backward
// (reference attention.rs:1024-1041 and :485-497; the scale 1/sqrt(head_dim) of :294-296 is applied here)
// One warp per row; a row is at most a few KB, so the second and third pass hit L1.
// ---------------------------------------------------------------------------
// 16-byte (8 x bf16) accesses: S_pad is a multiple of 32, so a row is a whole number of them.
__device__ __forceinline__ void unpack8(const uint4& q, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 q;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return q;
}

__global__ void __launch_bounds__(256)
softmax_causal_kernel(const bf16* __restrict__ scores, bf16* __restrict__ probs, AttnShape a, float scale, int causal) {
  const long long row = (long long)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= (long long)a.G * a.GR) return;
  const int within = (int)(row % a.GR);
  const uint4* src = reinterpret_cast<const uint4*>(scores + row * a.S_pad);
  uint4* dst = reinterpret_cast<uint4*>(probs + row * a.S_pad);
  const int chunks = a.S_pad / 8;
  if (within >= a.g * a.S) {                      // padding row of the group
    for (int c = lane; c < chunks; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
    return;
  }
  const int visible = causal ? within % a.S + 1 : a.S;
  const int vchunks = (visible + 7) / 8;
  float mx = -INFINITY;
  for (int c = lane; c < vchunks; c += 32) {
    float f[8];
    unpack8(src[c], f);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (c * 8 + i < visible) mx = fmaxf(mx, f[i] * scale);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int c = lane; c < vchunks; c += 32) {
    float f[8];
    unpack8(src[c], f);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (c * 8 + i < visible) sum += expf(f[i] * scale - mx);
  }
  sum = warp_sum(sum);
  const float inv = sum > 0.f ? 1.0f / sum : 1.0f;   // activations.rs:65-69
  for (int c = lane; c < chunks; c += 32) {
    float f[8];
    if (c < vchunks) {
      unpack8(src[c], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = c * 8 + i < visible ? expf(f[i] * scale - mx) * inv : 0.f;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = 0.f;
    }
    dst[c] = pack8(f);
  }
}

// in place on grad: dL/dscore = p * (dL/dp - sum_j p_j dL/dp_j) * scale.  With `causal` the entries behind the
// visible prefix are not read (the product that made dL/dp skipped them) and are written as zeros, like padding rows.
__global__ void __launch_bounds__(256)
softmax_backward_kernel(const bf16* __restrict__ probs, bf16* __restrict__ grad, AttnShape a, float scale, int causal) {
  const long long row = (long long)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= (long long)a.G * a.GR) return;
  const uint4* p = reinterpret_cast<const uint4*>(probs + row * a.S_pad);
  uint4* g = reinterpret_cast<uint4*>(grad + row * a.S_pad);
  const int chunks = a.S_pad / 8;
  const int within = (int)(row % a.GR);
  if (within >= a.g * a.S) {                      // padding row of the group
    for (int c = lane; c < chunks; c += 32) g[c] = make_uint4(0, 0, 0, 0);
    return;
  }
  const int visible = causal ? within % a.S + 1 : a.S;
  const int vchunks = (visible + 7) / 8;
  float dot = 0.f;
  for (int c = lane; c < vchunks; c += 32) {
    float fp[8], fg[8];
    unpack8(p[c], fp); unpack8(g[c], fg);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (c * 8 + i < visible) dot += fp[i] * fg[i];
  }
  dot = warp_sum(dot);
  for (int c = lane; c < chunks; c += 32) {
    float fp[8], fg[8];
    if (c < vchunks) {
      unpack8(p[c], fp); unpack8(g[c], fg);
#pragma unroll
      for (int i = 0; i < 8; ++i) fg[i] = c * 8 + i < visible ? fp[i] * (fg[i] - dot) * scale : 0.f;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) fg[i] = 0.f;
    }
    g[c] = pack8(fg);
  }
}

// Register-resident variants for rows of at most NC * 256 entries: every lane keeps its NC 16-byte pieces of the row,
// so the scores (and dL/dp) cross the memory system once.  `zero_cols` is how far behind the visible prefix zeros are
// written, rounded up to 128 from the query position: the causal products that read these rows never look further
// (a caller that cannot promise that passes zero_tail_all and the whole tail is written).
template <int NC>
__global__ void __launch_bounds__(256)
softmax_causal_regs_kernel(const bf16* __restrict__ scores, bf16* __restrict__ probs, AttnShape a, float scale, int causal,
                           int zero_tail_all) {
  const long long row = (long long)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= (long long)a.G * a.GR) return;
  const int within = (int)(row % a.GR);
  const uint4* src = reinterpret_cast<const uint4*>(scores + row * a.S_pad);
  uint4* dst = reinterpret_cast<uint4*>(probs + row * a.S_pad);
  const int chunks = a.S_pad / 8;
  if (within >= a.g * a.S) {                      // padding row of the group
    for (int c = lane; c < chunks; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
    return;
  }
  const int visible = causal ? within % a.S + 1 : a.S;
  const int vchunks = (visible + 7) / 8;
  const int zchunks = zero_tail_all ? chunks : min(chunks, ((visible + 127) & ~127) / 8);
  // The row stays in registers as scores, then as exponentials: one exponential per entry (with two the kernel was
  // bound by instruction issue: 80 microseconds for 65536 rows of 1024).  expf, not the hardware exponential: its
  // 2^-21 is enough to flip bf16 roundings of the probabilities, and the parity case with head_dim 32 sits at the
  // 2e-2 bar (one gradient moved from below it to 2.007e-2).
  float e[NC][8];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < NC; ++j) {
    const int c = lane + 32 * j;
    if (c < vchunks) {
      unpack8(src[c], e[j]);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (c * 8 + i >= visible) e[j][i] = -INFINITY;
        mx = fmaxf(mx, e[j][i] * scale);           // scale > 0
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < NC; ++j) {
    const int c = lane + 32 * j;
    if (c < vchunks) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        e[j][i] = expf(fmaf(e[j][i], scale, -mx));     // exp(-inf) = 0 behind the visible prefix
        sum += e[j][i];
      }
    }
  }
  sum = warp_sum(sum);
  const float inv = sum > 0.f ? 1.0f / sum : 1.0f;   // activations.rs:65-69
#pragma unroll
  for (int j = 0; j < NC; ++j) {
    const int c = lane + 32 * j;
    if (c >= zchunks) break;
    float f[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = c < vchunks ? e[j][i] * inv : 0.f;
    dst[c] = pack8(f);
  }
}

template <int NC>
__global__ void __launch_bounds__(256)
softmax_backward_regs_kernel(const bf16* __restrict__ probs, bf16* __restrict__ grad, AttnShape a, float scale, int causal,
                             int zero_tail_all) {
  const long long row = (long long)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= (long long)a.G * a.GR) return;
  const uint4* p = reinterpret_cast<const uint4*>(probs + row * a.S_pad);
  uint4* g = reinterpret_cast<uint4*>(grad + row * a.S_pad);
  const int chunks = a.S_pad / 8;
  const int within = (int)(row % a.GR);
  if (within >= a.g * a.S) {                      // padding row of the group
    for (int c = lane; c < chunks; c += 32) g[c] = make_uint4(0, 0, 0, 0);
    return;
  }
  const int visible = causal ? within % a.S + 1 : a.S;
  const int vchunks = (visible + 7) / 8;
  const int zchunks = zero_tail_all ? chunks : min(chunks, ((visible + 127) & ~127) / 8);
  uint4 vp[NC], vg[NC];
#pragma unroll
  for (int j = 0; j < NC; ++j) {
    const int c = lane + 32 * j;
    vp[j] = c < vchunks ? p[c] : make_uint4(0, 0, 0, 0);
    vg[j] = c < vchunks ? g[c] : make_uint4(0, 0, 0, 0);
  }
  float dot = 0.f;
#pragma unroll
  for (int j = 0; j < NC; ++j) {
    const int c = lane + 32 * j;
    float fp[8], fg[8];
    unpack8(vp[j], fp); unpack8(vg[j], fg);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (c * 8 + i < visible) dot += fp[i] * fg[i];
  }
  dot = warp_sum(dot);
#pragma unroll
  for (int j = 0; j < NC; ++j) {
    const int c = lane + 32 * j;
    if (c >= zchunks) break;
    float fp[8], fg[8];
    unpack8(vp[j], fp); unpack8(vg[j], fg);
#pragma unroll
    for (int i = 0; i < 8; ++i) fg[i] = c * 8 + i < visible ? fp[i] * (fg[i] - dot) * scale : 0.f;
    g[c] = pack8(fg);
  }
}

__global__ void add_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, bf16* __restrict__ out, long long n8) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const uint4 x = reinterpret_cast<const uint4*>(a)[i], y = reinterpret_cast<const uint4*>(b)[i];
  const __nv_bfloat162* xs = reinterpret_cast<const __nv_bfloat162*>(&x);
  const __nv_bfloat162* ys = reinterpret_cast<const __nv_bfloat162*>(&y);
  uint4 r;
  __nv_bfloat162* rs = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 fx = __bfloat1622float2(xs[k]), fy = __bfloat1622float2(ys[k]);
    rs[k] = __floats2bfloat162_rn(fx.x + fy.x, fx.y + fy.y);
  }
  reinterpret_cast<uint4*>(out)[i] = r;
}

__global__ void cast_rows_kernel(const bf16* __restrict__ src, long long ld, float* __restrict__ dst, int rows, int cols) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)rows * cols) return;
  const long long r = i / cols, c = i - r * cols;
  dst[i] = bf(src[r * ld + c]);
}

// ---------------------------------------------------------------------------
// cross-entropy (reference causal_lm_loss.rs:100-150): one block per row
// ---------------------------------------------------------------------------
__device__ __forceinline__ float block_reduce(float v, float* sh, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float w = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, w) : v + w;
  }
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float r = is_max ? -INFINITY : 0.f;
  for (int i = 0; i < nw; ++i) r = is_max ? fmaxf(r, sh[i]) : r + sh[i];   // same order in every thread
  return r;
}

// ld is a multiple of 32, so a row is a whole number of 16-byte vectors; columns past `vocab` are padding.
// Two exponentials per logit make this kernel instruction bound with expf (262 M logits per step of the 55M model),
// so the bulk uses the hardware exponential (relative error about 2^-21 per term, far inside the bf16 logits'
// own rounding); the row's loss, one term, uses expf and logf.
__global__ void __launch_bounds__(256)
cross_entropy_kernel(bf16* __restrict__ logits, const int* __restrict__ targets, float* __restrict__ row_loss, int vocab,
                     int ld, float inv_predicted) {
  __shared__ float sh[8];
  const int r = blockIdx.x, target = targets[r];
  uint4* row = reinterpret_cast<uint4*>(logits + (size_t)r * ld);
  const int chunks = ld / 8;
  if (target < 0) {                               // predicts nothing: zero gradient, no loss
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) row[c] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) row_loss[r] = 0.f;
    return;
  }
  // one pass: running maximum and the sum of exponentials relative to it
  float mx = -INFINITY, sum = 0.f;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    float f[8];
    unpack8(row[c], f);
    float cm = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (c * 8 + i < vocab) cm = fmaxf(cm, f[i]);
    if (cm > mx) { sum *= __expf(mx - cm); mx = cm; }
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (c * 8 + i < vocab) sum += __expf(f[i] - mx);
  }
  const float bm = block_reduce(mx, sh, true);
  sum = block_reduce(mx > -INFINITY ? sum * expf(mx - bm) : 0.f, sh, false);
  const float inv = sum > 0.f ? 1.0f / sum : 1.0f;
  if (threadIdx.x == 0)
    row_loss[r] = -logf(fmaxf(expf(bf(logits[(size_t)r * ld + target]) - bm) * inv, FLT_MIN));
  __syncthreads();                                // the target's logit has been read before it is overwritten
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    float f[8];
    unpack8(row[c], f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int j = c * 8 + i;
      float g = 0.f;
      if (j < vocab) {
        g = __expf(f[i] - bm) * inv * inv_predicted;
        if (j == target) g -= inv_predicted;
      }
      f[i] = g;
    }
    row[c] = pack8(f);
  }
}

__global__ void __launch_bounds__(256) loss_sum_kernel(const float* __restrict__ row_loss, int rows, float inv_predicted,
                                                       float* __restrict__ out) {
  __shared__ float sh[256];
  const int per = (rows + 255) / 256;
  float acc = 0.f;
  for (int i = threadIdx.x * per; i < min(rows, (threadIdx.x + 1) * per); ++i) acc += row_loss[i];   // a contiguous run each
  sh[threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 256; ++i) t += sh[i];     // runs in order: the sum does not depend on scheduling
    out[0] = t * inv_predicted;
  }
}

__global__ void pack_kernel(const float* __restrict__ src, float* __restrict__ dst, bf16* __restrict__ dst_bf16, int rows,
                            int cols, int ld, int row0, int kind) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)rows * cols) return;
  const int r = (int)(i / cols), c = (int)(i - (long long)r * cols);
  const long long o = (long long)(row0 + (kind == 0 ? r : gu_row(kind - 1, r))) * ld + c;
  dst[o] = src[i];
  if (dst_bf16) dst_bf16[o] = tb(src[i]);
}
__global__ void unpack_kernel(const float* __restrict__ src, float* __restrict__ dst, int rows, int cols, int ld, int row0,
                              int kind) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)rows * cols) return;
  const int r = (int)(i / cols), c = (int)(i - (long long)r * cols);
  dst[i] = src[(long long)(row0 + (kind == 0 ? r : gu_row(kind - 1, r))) * ld + c];
}

__global__ void split_qkv_kernel(const bf16* __restrict__ qkv, bf16* __restrict__ q, bf16* __restrict__ k, bf16* __restrict__ v,
                                 int qn, int kn) {
  const int r = blockIdx.x, w = (qn + 2 * kn) / 8;
  const uint4* src = reinterpret_cast<const uint4*>(qkv + (size_t)r * (qn + 2 * kn));
  for (int c = threadIdx.x; c < w; c += blockDim.x) {
    const int col = c * 8;
    uint4* dst = col < qn ? reinterpret_cast<uint4*>(q + (size_t)r * qn + col)
                          : col < qn + kn ? reinterpret_cast<uint4*>(k + (size_t)r * kn + (col - qn))
                                          : reinterpret_cast<uint4*>(v + (size_t)r * kn + (col - qn - kn));
    *dst = src[c];
  }
}

unsigned blocks_for(long long n, int threads) { return (unsigned)((n + threads - 1) / threads); }

}  // namespace

// ---------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------
cudaError_t launch_embed_gather(const uint32_t* ids, const bf16* table, bf16* x, int rows, int d, cudaStream_t st) {
  if (rows <= 0) return cudaSuccess;
  embed_gather_kernel<<<rows, 64, 0, st>>>(ids, table, x, d); count_launch();
  return cudaGetLastError();
}
cudaError_t launch_embed_scatter(const uint32_t* ids, const bf16* grad_x, float* grad_table, const int* first, const int* next,
                                 int rows, int d, cudaStream_t st) {
  if (rows <= 0) return cudaSuccess;
  embed_scatter_kernel<<<rows, 128, 0, st>>>(ids, grad_x, grad_table, first, next, d); count_launch();
  return cudaGetLastError();
}
cudaError_t launch_rope_pack(const bf16* qkv, const float* cos_t, const float* sin_t, bf16* q_hm, bf16* k_hm, bf16* v_hm,
                             AttnShape a, cudaStream_t st) {
  rope_pack_kernel<<<a.B * a.S, 128, 0, st>>>(qkv, cos_t, sin_t, q_hm, k_hm, v_hm, a); count_launch();
  return cudaGetLastError();
}
// The bounded zero tail is only right when a 128-row tile never crosses from one query head into the next.
static int tail_all(const AttnShape& a, int causal, int bounded_tail) { return !(causal && bounded_tail && a.S % 128 == 0); }
cudaError_t launch_softmax_causal(const bf16* scores, bf16* probs, AttnShape a, float scale, int causal, int bounded_tail,
                                  cudaStream_t st) {
  const long long rows = (long long)a.G * a.GR;
  const unsigned grid = blocks_for(rows, 8);
  const int all = tail_all(a, causal, bounded_tail);
  if (a.S_pad <= 256) softmax_causal_regs_kernel<1><<<grid, 256, 0, st>>>(scores, probs, a, scale, causal, all);
  else if (a.S_pad <= 512) softmax_causal_regs_kernel<2><<<grid, 256, 0, st>>>(scores, probs, a, scale, causal, all);
  else if (a.S_pad <= 1024) softmax_causal_regs_kernel<4><<<grid, 256, 0, st>>>(scores, probs, a, scale, causal, all);
  else if (a.S_pad <= 2048) softmax_causal_regs_kernel<8><<<grid, 256, 0, st>>>(scores, probs, a, scale, causal, all);
  else softmax_causal_kernel<<<grid, 256, 0, st>>>(scores, probs, a, scale, causal);
  count_launch();
  return cudaGetLastError();
}
cudaError_t launch_softmax_backward(const bf16* probs, bf16* grad, AttnShape a, float scale, int causal, int bounded_tail,
                                    cudaStream_t st) {
  const long long rows = (long long)a.G * a.GR;
  const unsigned grid = blocks_for(rows, 8);
  const int all = tail_all(a, causal, bounded_tail);
  if (a.S_pad <= 256) softmax_backward_regs_kernel<1><<<grid, 256, 0, st>>>(probs, grad, a, scale, causal, all);
  else if (a.S_pad <= 512) softmax_backward_regs_kernel<2><<<grid, 256, 0, st>>>(probs, grad, a, scale, causal, all);
  else if (a.S_pad <= 1024) softmax_backward_regs_kernel<4><<<grid, 256, 0, st>>>(probs, grad, a, scale, causal, all);
  else if (a.S_pad <= 2048) softmax_backward_regs_kernel<8><<<grid, 256, 0, st>>>(probs, grad, a, scale, causal, all);
  else softmax_backward_kernel<<<grid, 256, 0, st>>>(probs, grad, a, scale, causal);
  count_launch();
  return cudaGetLastError();
}
cudaError_t launch_heads_to_tokens(const bf16* o_hm, bf16* merged, AttnShape a, cudaStream_t st) {
  heads_tokens_kernel<true><<<a.B * a.S, 64, 0, st>>>(o_hm, merged, a); count_launch();
  return cudaGetLastError();
}
cudaError_t launch_tokens_to_heads(const bf16* grad_merged, bf16* do_hm, AttnShape a, cudaStream_t st) {
  heads_tokens_kernel<false><<<a.B * a.S, 64, 0, st>>>(grad_merged, do_hm, a); count_launch();
  return cudaGetLastError();
}
cudaError_t launch_qkv_grad_unpack(const bf16* dq_hm, const float* dk_hm, const float* dv_hm, const float* cos_t,
                                   const float* sin_t, bf16* dqkv, AttnShape a, cudaStream_t st) {
  qkv_grad_unpack_kernel<<<a.B * a.S, 128, 0, st>>>(dq_hm, dk_hm, dv_hm, cos_t, sin_t, dqkv, a); count_launch();
  return cudaGetLastError();
}
cudaError_t launch_attn_meta(int* meta, int groups, int group_rows, cudaStream_t st) {
  attn_meta_kernel<<<1, 256, 0, st>>>(meta, groups, group_rows); count_launch();
  return cudaGetLastError();
}
cudaError_t launch_split_qkv(const bf16* qkv, bf16* q, bf16* k, bf16* v, int rows, int qn, int kn, cudaStream_t st) {
  if (rows <= 0) return cudaSuccess;
  split_qkv_kernel<<<rows, 64, 0, st>>>(qkv, q, k, v, qn, kn); count_launch();
  return cudaGetLastError();
}
cudaError_t launch_add(const bf16* a, const bf16* b, bf16* out, long long n, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  add_kernel<<<blocks_for(n / 8, 256), 256, 0, st>>>(a, b, out, n / 8); count_launch();   // n is a multiple of 8 (d_model is)
  return cudaGetLastError();
}
cudaError_t launch_cast_rows_to_f32(const bf16* src, long long ld, float* dst, int rows, int cols, cudaStream_t st) {
  if (rows <= 0) return cudaSuccess;
  cast_rows_kernel<<<blocks_for((long long)rows * cols, 256), 256, 0, st>>>(src, ld, dst, rows, cols); count_launch();
  return cudaGetLastError();
}
cudaError_t launch_cross_entropy(bf16* logits, const int* targets, float* row_loss, int rows, int vocab, int ld,
                                 float inv_predicted, cudaStream_t st) {
  if (rows <= 0) return cudaSuccess;
  cross_entropy_kernel<<<rows, 256, 0, st>>>(logits, targets, row_loss, vocab, ld, inv_predicted);
  count_launch();
  return cudaGetLastError();
}
cudaError_t launch_loss_sum(const float* row_loss, int rows, float inv_predicted, float* out, cudaStream_t st) {
  loss_sum_kernel<<<1, 256, 0, st>>>(row_loss, rows, inv_predicted, out); count_launch();
  return cudaGetLastError();
}
cudaError_t launch_pack(const float* src, float* dst, bf16* dst_bf16, int rows, int cols, int ld, int row0, int kind,
                        cudaStream_t st) {
  pack_kernel<<<blocks_for((long long)rows * cols, 256), 256, 0, st>>>(src, dst, dst_bf16, rows, cols, ld, row0, kind); count_launch();
  return cudaGetLastError();
}
cudaError_t launch_unpack(const float* src, float* dst, int rows, int cols, int ld, int row0, int kind, cudaStream_t st) {
  unpack_kernel<<<blocks_for((long long)rows * cols, 256), 256, 0, st>>>(src, dst, rows, cols, ld, row0, kind); count_launch();
  return cudaGetLastError();
}

}  // namespace lm
}  // namespace moe
