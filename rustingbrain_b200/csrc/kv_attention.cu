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
// Three launches per step: rotate + append, partial attention, merge (which also advances the lengths).

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
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
};
template <> struct Slice8<bf16> {
  static __device__ __forceinline__ void load(const bf16* p, float* o) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {   // a bf16 is the upper half of its f32
      o[2 * i] = __uint_as_float(w[i] << 16);
      o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};
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
                  const int* __restrict__ lengths, float* __restrict__ part, KvShape s, int splits, float scale_log2) {
  constexpr int LPK = HD / 8, KPW = 32 / LPK, NG = KV_WARPS * KPW, PW = HD + 2;
  extern __shared__ float kv_sm[];   // [KV_QT][NG][PW]
  const int split = blockIdx.x, kvh = blockIdx.y, sj = blockIdx.z, seq = s.first + sj;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = lane / LPK, ls = lane % LPK;
  const int len0 = lengths[seq], total = len0 + s.rows;
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
    // The loop is uniform across the warp (the shuffles below need every lane); a lane group whose
    // position lies past the end loads nothing and updates nothing.
    float kf[8], vf[8], kn[8], vn[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) kf[c] = vf[c] = kn[c] = vn[c] = 0.f;
    const int base0 = k0 + warp * KPW;
    if (base0 + sub < kend) {
      Slice8<T>::load(kbase + (size_t)(base0 + sub) * W, kf);
      Slice8<T>::load(vbase + (size_t)(base0 + sub) * W, vf);
    }
    for (int base = base0; base < kend; base += NG) {
      const int key = base + sub, nxt = key + NG;
      const bool live = key < kend;
      if (nxt < kend) {     // next position's loads are in flight while this one is used
        Slice8<T>::load(kbase + (size_t)nxt * W, kn);
        Slice8<T>::load(vbase + (size_t)nxt * W, vn);
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
#pragma unroll
      for (int c = 0; c < 8; ++c) { kf[c] = kn[c]; vf[c] = vn[c]; }
    }

    // merge the lane groups of the CTA
    __syncthreads();   // the previous pass has finished reading the buffer
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
  }
}

// ---- merge the slices, write the merged heads, advance the cache lengths ----
template <typename T>
__global__ void kv_merge_kernel(const float* __restrict__ part, T* __restrict__ merged, int* __restrict__ lengths,
                                KvShape s, int splits) {
  const int PW = s.HD + 2;
  const int rh = blockIdx.x;                      // row * H + head
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

__global__ void kv_set_lengths_kernel(int* lengths, int first, int count, int value) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) lengths[first + i] = value;
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

template <typename T>
cudaError_t launch_partial(const kv_cache* c, const T* q, KvShape s, int n_seq, int splits, cudaStream_t st) {
  const float scale_log2 = LOG2E / sqrtf((float)s.HD);   // attention.rs:294-296
  const dim3 grid(splits, s.Hkv, n_seq);
#define KV_CASE(HDV)                                                                                         \
  case HDV: {                                                                                                \
    const size_t smem = sizeof(float) * KV_QT * (KV_WARPS * (32 / (HDV / 8))) * (HDV + 2);                   \
    kv_partial_kernel<T, HDV><<<grid, KV_THREADS, smem, st>>>(q, (const T*)c->keys, (const T*)c->values,     \
                                                               c->lengths, c->part, s, splits, scale_log2);  \
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
  // enough CTAs for two per SM, slices of at least 256 positions
  long long ctas = (long long)n_seq * g.kv_heads;
  int splits = (int)std::min<long long>(KV_MAX_SPLITS, std::max<long long>(1, (2ll * c->sm_count + ctas - 1) / ctas));
  splits = std::max(1, std::min(splits, (longest + 255) / 256));
  const size_t need = (size_t)n_seq * rows * g.num_heads * splits * (g.head_dim + 2);
  if (need > c->part_floats) {
    if (c->part) { KCK(cudaStreamSynchronize(st)); cudaFree(c->part); c->part = nullptr; c->part_floats = 0; }
    if (cudaMalloc(&c->part, need * sizeof(float)) != cudaSuccess) {
      cudaGetLastError();
      return kv_fail(c, MOE_OUT_OF_MEMORY, "OutOfMemory: %zu bytes for the slice results", need * sizeof(float));
    }
    c->part_floats = need;
  }
  kv_append_kernel<T><<<n_seq * rows, 128, 0, st>>>((T*)q, (const T*)k, (const T*)v, (T*)c->keys, (T*)c->values,
                                                    c->lengths, c->cos_t, c->sin_t, s, g.rope);
  count_launch();
  KCK(cudaGetLastError());
  KCK(launch_partial<T>(c, (const T*)q, s, n_seq, splits, st));
  kv_merge_kernel<T><<<n_seq * rows * g.num_heads, std::min(256, std::max(32, g.head_dim)), 0, st>>>(
      c->part, (T*)merged, c->lengths, s, splits);
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
  c->host_len.assign(g.sequences, 0);
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
  cudaFree(c->keys); cudaFree(c->values); cudaFree(c->lengths); cudaFree(c->cos_t); cudaFree(c->sin_t);
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
  kv_set_lengths_kernel<<<ceil_div(count, 256), 256, 0, (cudaStream_t)stream>>>(c->lengths, first, count, length);
  count_launch();
  KCK(cudaGetLastError());
  for (int i = 0; i < count; ++i) c->host_len[first + i] = length;
  return MOE_OK;
}

int32_t kv_cache_clear(kv_cache_t* c, int32_t sequence, void* stream) { return kv_cache_truncate(c, sequence, 0, stream); }

int32_t kv_cache_lengths(kv_cache_t* c, int32_t* lengths_host, void* stream) {
  if (!c || !lengths_host) return MOE_INVALID_INPUT;
  KCK(cudaMemcpyAsync(lengths_host, c->lengths, sizeof(int) * c->cfg.sequences, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  KCK(cudaStreamSynchronize((cudaStream_t)stream));
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
