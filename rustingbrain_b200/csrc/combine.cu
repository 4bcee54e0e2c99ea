// Combine (forward) and the HBM-bound halves of the backward pass.
//
//   combine_kernel      y[t] = sum_{slots, ascending expert} gate * y_perm[row] + shared[t]
//                       (reference moe.rs:290-319; replaces the f32-atomic
//                       scatter_add_scaled, cuda_training.rs:294, by a per-token
//                       gather-reduce in a fixed order: deterministic, no atomics).
//   gather_grad_kernel  grad_y_perm[row] = gate * grad_y[token] and
//                       grad_gate[slot] = <grad_y[token], y_perm[row]>
//                       (moe.rs:375-383, 404-415; gather_scale_rows + row_dot_scatter,
//                       cuda_training.rs:293, 300-312, in one pass over grad_y).
//   router_bwd_kernel   top-k renormalisation backward, load-balancing term, softmax
//                       backward and z-loss in one kernel (moe.rs:420-481;
//                       moe_grad_probs + moe_aux_grad + router_grad_logits,
//                       cuda_training.rs:314-316).
//   unpermute_kernel    grad_x[t] = shared + sum_{slots} grad_x_perm[row] + grad_logits[t] W_r
//                       (moe.rs:356-361, 389-399, 483-486; scatter_add_rows + router dgrad).
//   router_wgrad        dW_r = grad_logits^T x, two-stage fixed-order reduction.
//
// One warp handles one token; rows move as 16-byte vectors.

#include <algorithm>

#include "kernels.cuh"

namespace moe {

constexpr int CB_WARPS = 8;

template <typename T> struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  __device__ static void load(const T* p, float* v);
  __device__ static void store(T* p, const float* v);
};
template <> __device__ inline void Vec16<float>::load(const float* p, float* v) {
  const float4 q = *reinterpret_cast<const float4*>(p);
  v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
}
template <> __device__ inline void Vec16<float>::store(float* p, const float* v) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ inline void Vec16<bf16>::load(const bf16* p, float* v) {
  const uint4 q = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
    v[2 * i] = __low2float(h);
    v[2 * i + 1] = __high2float(h);
  }
}
template <> __device__ inline void Vec16<bf16>::store(bf16* p, const float* v) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// Four independent 16-byte row loads in flight per lane before any of them is consumed: the
// rows of one token live in unrelated places, so the loads do not depend on each other.
constexpr int ROW_BATCH = 4;
template <typename T>
__device__ inline void unpack16(const uint4& q, float* v) {
  Vec16<T>::load(reinterpret_cast<const T*>(&q), v);
}

// The slots of one token, held in registers.  KMAX (a power of two >= k) is a template parameter and
// every loop over the slots is fully unrolled, so the arrays are never indexed with a run-time value
// (which would move them to local memory and put a load or store behind every row access).
// Lane j < k reads slot j; the values reach all lanes by shuffles.
constexpr unsigned FULL = 0xffffffffu;

// Slot order (the order of the top-k selection).  pos < 0: the slot moves no row.
template <int KMAX>
__device__ __forceinline__ void slots_in_order(const int* slot_pos, const float* gates, int t, int k, int lane,
                                               int (&pos)[KMAX], float (&gate)[KMAX]) {
  int p = -1;
  float g = 0.f;
  if (lane < k) {
    p = slot_pos[(size_t)t * k + lane];
    g = gates ? gates[(size_t)t * k + lane] : 1.f;
  }
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    pos[j] = __shfl_sync(FULL, p, j);
    gate[j] = __shfl_sync(FULL, g, j);
  }
}

// Ascending expert order (the order in which the reference accumulates a token's contributions,
// moe.rs:290-319): the first n entries are the token's routed rows, the rest have pos = -1.
template <int KMAX>
__device__ __forceinline__ int slots_by_expert(const int* expert_of, const int* slot_pos, const float* gates, int t, int k,
                                               int lane, int (&pos)[KMAX], float (&gate)[KMAX]) {
  int e = -1, p = -1;
  float g = 0.f;
  if (lane < k) {
    e = expert_of[(size_t)t * k + lane];
    p = slot_pos[(size_t)t * k + lane];
    g = gates ? gates[(size_t)t * k + lane] : 1.f;
  }
  const bool valid = e >= 0 && p >= 0;
  int rank = 0;   // routed slots of this token that come before this one
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    const int ej = __shfl_sync(FULL, e, j);
    const int vj = __shfl_sync(FULL, (int)valid, j);
    rank += (vj && (ej < e || (ej == e && j < lane))) ? 1 : 0;
  }
#pragma unroll
  for (int s = 0; s < KMAX; ++s) {
    const unsigned m = __ballot_sync(FULL, valid && rank == s);
    const int src = m ? __ffs(m) - 1 : 0;
    const int ps = __shfl_sync(FULL, p, src);
    gate[s] = __shfl_sync(FULL, g, src);
    pos[s] = m ? ps : -1;
  }
  return __popc(__ballot_sync(FULL, valid));
}

// Launches kernel<T, KMAX> for the smallest KMAX in {1, 2, 4, 8, 16} that holds k.
#define DISPATCH_KMAX(KERNEL, T, k, grid, stream, args)                                         \
  do {                                                                                           \
    if ((k) <= 1) launch_kernel(KERNEL<T, 1>, dim3(grid), dim3(CB_WARPS * 32), 0, stream, args);  \
    else if ((k) <= 2) launch_kernel(KERNEL<T, 2>, dim3(grid), dim3(CB_WARPS * 32), 0, stream, args); \
    else if ((k) <= 4) launch_kernel(KERNEL<T, 4>, dim3(grid), dim3(CB_WARPS * 32), 0, stream, args); \
    else if ((k) <= 8) launch_kernel(KERNEL<T, 8>, dim3(grid), dim3(CB_WARPS * 32), 0, stream, args); \
    else launch_kernel(KERNEL<T, 16>, dim3(grid), dim3(CB_WARPS * 32), 0, stream, args);          \
    count_launch();                                                                              \
  } while (0)

// a.split > 1 (decode-sized batches): `split` warps share a token, each lane owns one 16-byte piece of the row, so
// a token's loads are one round trip instead of one per 512 bytes of a lane's loop.
template <typename T, int KMAX>
__global__ void __launch_bounds__(CB_WARPS * 32) combine_kernel(CombineArgs a) {
  pdl_enter();
  const int item = blockIdx.x * CB_WARPS + (threadIdx.x >> 5);
  const int split = a.split > 1 ? a.split : 1;
  const int t = item / split, part = item - t * split;
  const int lane = threadIdx.x & 31;
  if (t >= a.tokens) return;
  int pos[KMAX];
  float gate[KMAX];
  const int n = slots_by_expert<KMAX>(a.expert_of, a.slot_pos, a.gates, t, a.k, lane, pos, gate);
  const size_t rb = (size_t)a.d * sizeof(T);
  const T* sh = (const T*)a.shared;
  T* y = (T*)a.y + (size_t)t * a.d;
  constexpr int V = Vec16<T>::N;
  constexpr int RB = KMAX < ROW_BATCH ? KMAX : ROW_BATCH;
  const int d = a.d;
  if (d % V == 0) {
    for (int c = (part * 32 + lane) * V; c < d; c += split * 32 * V) {
      float acc[V];
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = 0.f;
      uint4 sh_raw = make_uint4(0, 0, 0, 0);
      if (sh) sh_raw = *reinterpret_cast<const uint4*>(sh + (size_t)t * d + c);   // in flight with the rows
#pragma unroll
      for (int j0 = 0; j0 < KMAX; j0 += RB) {
        if (j0 >= n) break;
        uint4 raw[RB];
#pragma unroll
        for (int b = 0; b < RB; ++b)
          if (j0 + b < n) raw[b] = *reinterpret_cast<const uint4*>((const T*)row_ptr(a.y_perm, pos[j0 + b], rb) + c);
#pragma unroll
        for (int b = 0; b < RB; ++b) {
          if (j0 + b < n) {
            float v[V];
            unpack16<T>(raw[b], v);
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(gate[j0 + b], v[i]));
          }
        }
      }
      if (sh) {
        float v[V];
        unpack16<T>(sh_raw, v);
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = __fadd_rn(acc[i], v[i]);
      }
      if (a.accumulate) {
        float v[V];
        Vec16<T>::load(y + c, v);
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = __fadd_rn(v[i], acc[i]);
      }
      Vec16<T>::store(y + c, acc);
    }
  } else {
    for (int c = part * 32 + lane; c < d; c += split * 32) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < KMAX; ++j)
        if (j < n) acc = __fadd_rn(acc, __fmul_rn(gate[j], to_f32<T>(((const T*)row_ptr(a.y_perm, pos[j], rb))[c])));
      if (sh) acc = __fadd_rn(acc, to_f32<T>(sh[(size_t)t * d + c]));
      if (a.accumulate) acc = __fadd_rn(to_f32<T>(y[c]), acc);
      y[c] = from_f32<T>(acc);
    }
  }
}

cudaError_t launch_combine(const CombineArgs& a_in, int precision, cudaStream_t stream) {
  if (a_in.tokens <= 0) return cudaSuccess;
  CombineArgs a = a_in;
  // decode-sized batches: as many warps per token as the row has 512-byte (32 x 16 B) pieces
  const int pieces = ceil_div(a.d * (precision == PREC_BF16 ? 2 : 4), 512);
  a.split = a.tokens <= 256 ? std::max(1, std::min(pieces, 16)) : 1;
  const int grid = ceil_div(a.tokens * a.split, CB_WARPS);
  if (precision == PREC_BF16) DISPATCH_KMAX(combine_kernel, bf16, a.k, grid, stream, a);
  else DISPATCH_KMAX(combine_kernel, float, a.k, grid, stream, a);
  return cudaGetLastError();
}

template <typename T, int KMAX>
__global__ void __launch_bounds__(CB_WARPS * 32, 2) gather_grad_kernel(GatherGradArgs a) {
  const int t = blockIdx.x * CB_WARPS + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= a.tokens) return;
  const int k = a.k, d = a.d;
  int pos[KMAX];
  float gate[KMAX], dot[KMAX];
  slots_in_order<KMAX>(a.slot_pos, a.gates, t, k, lane, pos, gate);
#pragma unroll
  for (int j = 0; j < KMAX; ++j) dot[j] = 0.f;
  const T* gy = (const T*)a.grad_y + (size_t)t * d;
  const size_t rb = (size_t)d * sizeof(T);
  constexpr int V = Vec16<T>::N;
  constexpr int RB = ROW_BATCH;
  if (d % V == 0) {
    // The lane keeps up to U chunks of grad_y[token] (a 4 KB piece of the row per warp) and walks the
    // token's rows one after the other, so every row is read and written in contiguous pieces instead
    // of 512 bytes at a time interleaved with seven other rows (DRAM pages stay open).
    constexpr int U = 8;
    const int cpr = d / V;
    const uint4* gsrc = reinterpret_cast<const uint4*>(gy);
    for (int c0 = lane; c0 < cpr; c0 += 32 * U) {
      uint4 gq[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (c0 + 32 * u < cpr) gq[u] = gsrc[c0 + 32 * u];
#pragma unroll
      for (int j = 0; j < KMAX; ++j) {
        if (pos[j] >= 0) {
          const uint4* yrow = reinterpret_cast<const uint4*>(row_ptr(a.y_perm, pos[j], rb));
          uint4* drow = reinterpret_cast<uint4*>(row_ptr(a.grad_y_perm, pos[j], rb));
#pragma unroll
          for (int u0 = 0; u0 < U; u0 += RB) {
            uint4 raw[RB];
#pragma unroll
            for (int b = 0; b < RB; ++b)
              if (c0 + 32 * (u0 + b) < cpr) raw[b] = yrow[c0 + 32 * (u0 + b)];
#pragma unroll
            for (int b = 0; b < RB; ++b) {
              if (c0 + 32 * (u0 + b) < cpr) {
                float g[V], o[V], sv[V];
                unpack16<T>(gq[u0 + b], g);
                unpack16<T>(raw[b], o);
#pragma unroll
                for (int i = 0; i < V; ++i) {
                  dot[j] = fmaf(g[i], o[i], dot[j]);
                  sv[i] = gate[j] * g[i];
                }
                Vec16<T>::store(reinterpret_cast<T*>(drow + c0 + 32 * (u0 + b)), sv);
              }
            }
          }
        }
      }
    }
  } else {
    for (int c = lane; c < d; c += 32) {
      const float g = to_f32<T>(gy[c]);
#pragma unroll
      for (int j = 0; j < KMAX; ++j) {
        if (pos[j] >= 0) {
          dot[j] = fmaf(g, to_f32<T>(((const T*)row_ptr(a.y_perm, pos[j], rb))[c]), dot[j]);
          ((T*)row_ptr(a.grad_y_perm, pos[j], rb))[c] = from_f32<T>(gate[j] * g);
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    const float s = warp_sum(dot[j]);
    if (lane == 0 && j < k) a.grad_gates[(size_t)t * k + j] = pos[j] < 0 ? 0.f : s;
  }
}

cudaError_t launch_gather_grad(const GatherGradArgs& a, int precision, cudaStream_t stream) {
  if (a.tokens <= 0) return cudaSuccess;
  const int grid = ceil_div(a.tokens, CB_WARPS);
  if (precision == PREC_BF16) DISPATCH_KMAX(gather_grad_kernel, bf16, a.k, grid, stream, a);
  else DISPATCH_KMAX(gather_grad_kernel, float, a.k, grid, stream, a);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Expert-parallel peer transport: the gate gradient is computed where the expert output lives.
//   push_grad_kernel   (token owner)  stores grad_y[token] unscaled into the expert owner's row and the
//                                      slot's gate beside it: one NVLink crossing per row instead of two
//   scale_dot_kernel   (expert owner) dot[row] = <grad_y row, y row>; grad_y row *= gate (in place);
//                                      zeroes the padding rows of each group
//   pull_dots_kernel   (token owner)  grad_gate[slot] = dot[row] read back from the owner (4 bytes per slot)
// The lane-to-column mapping and the reduction order equal gather_grad_kernel's, so do the results.
// ---------------------------------------------------------------------------
__device__ inline float* aux_ptr(const RowSpace& s, int id, size_t aux_off, int which) {
  const int r = s.n == 1 ? 0 : id / s.cap;
  const int row = id - r * s.cap;
  return reinterpret_cast<float*>((char*)s.base[r] + aux_off) + (size_t)which * s.cap + row;
}

template <typename T, int KMAX>
__global__ void __launch_bounds__(CB_WARPS * 32) push_grad_kernel(PushGradArgs a) {
  const int t = blockIdx.x * CB_WARPS + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= a.tokens) return;
  const int k = a.k, d = a.d;
  int pos[KMAX];
  float gate[KMAX];
  slots_in_order<KMAX>(a.slot_pos, a.gates, t, k, lane, pos, gate);
#pragma unroll
  for (int j = 0; j < KMAX; ++j)
    if (lane == j && pos[j] >= 0) {
      *aux_ptr(a.rows, pos[j], a.aux_off, 0) = gate[j];
      if (a.dedup) *reinterpret_cast<int*>(aux_ptr(a.rows, pos[j], a.aux_off, 2)) = a.stage_base + t;
    }
  const T* gy = (const T*)a.grad_y + (size_t)t * d;
  const size_t rb = (size_t)d * sizeof(T);
  constexpr int V = Vec16<T>::N;
  if (a.dedup) {
    // the destinations become the token's staging rows, one per distinct owner rank (later slots of a rank are dropped)
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {
      const int rj = pos[j] >= 0 ? pos[j] / a.rows.cap : -1;
      bool first = rj >= 0;
#pragma unroll
      for (int i = 0; i < KMAX; ++i)
        if (i < j && pos[i] >= 0 && pos[i] / a.rows.cap == rj) first = false;
      // pos[] now names rows of `stage` (or -1); the gates and indices above are written already
      pos[j] = first ? rj * a.stage.cap + a.stage_base + t : -1;
    }
  }
  const RowSpace& dst_space = a.dedup ? a.stage : a.rows;
  if (d % V == 0) {
    // row by row, 8 KB pieces: the writes of one DRAM page (or one NVLink destination) stay together
    constexpr int U = 16;
    const int cpr = d / V;
    const uint4* gsrc = reinterpret_cast<const uint4*>(gy);
    for (int c0 = lane; c0 < cpr; c0 += 32 * U) {
      uint4 gq[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (c0 + 32 * u < cpr) gq[u] = gsrc[c0 + 32 * u];
#pragma unroll
      for (int j = 0; j < KMAX; ++j) {
        if (pos[j] >= 0) {
          uint4* drow = reinterpret_cast<uint4*>(row_ptr(dst_space, pos[j], rb));
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (c0 + 32 * u < cpr) drow[c0 + 32 * u] = gq[u];
        }
      }
    }
  } else {
    for (int c = lane; c < d; c += 32) {
      const T g = gy[c];
#pragma unroll
      for (int j = 0; j < KMAX; ++j)
        if (pos[j] >= 0) ((T*)row_ptr(dst_space, pos[j], rb))[c] = g;
    }
  }
}

cudaError_t launch_push_grad(const PushGradArgs& a, int precision, cudaStream_t stream) {
  if (a.tokens <= 0) return cudaSuccess;
  const int grid = ceil_div(a.tokens, CB_WARPS);
  if (precision == PREC_BF16) DISPATCH_KMAX(push_grad_kernel, bf16, a.k, grid, stream, a);
  else DISPATCH_KMAX(push_grad_kernel, float, a.k, grid, stream, a);
  return cudaGetLastError();
}

template <typename T>
__global__ void __launch_bounds__(CB_WARPS * 32) scale_dot_kernel(ScaleDotArgs a) {
  const int lane = threadIdx.x & 31;
  const int d = a.d;
  const int total = a.row0[a.groups];
  constexpr int V = Vec16<T>::N;
  for (int row = blockIdx.x * CB_WARPS + (threadIdx.x >> 5); row < total; row += gridDim.x * CB_WARPS) {
    int g = 0;
    while (g + 1 < a.groups && a.row0[g + 1] <= row) ++g;
    const bool live = row - a.row0[g] < a.counts[g];
    T* gy = (T*)a.grad_y + (size_t)row * d;
    const T* y = (const T*)a.y + (size_t)row * d;
    if (!live) {
      if (d % V == 0) for (int c = lane * V; c < d; c += 32 * V) *reinterpret_cast<uint4*>(gy + c) = make_uint4(0, 0, 0, 0);
      else for (int c = lane; c < d; c += 32) gy[c] = from_f32<T>(0.f);
      continue;
    }
    const float gate = a.gate_in[row];
    const T* gin = a.stage ? (const T*)a.stage + (size_t)a.src_index[row] * d : gy;   // the unscaled row
    float dot = 0.f;
    if (d % V == 0) {
      for (int c = lane * V; c < d; c += 32 * V) {
        float gv[V], o[V], s[V];
        Vec16<T>::load(gin + c, gv);
        Vec16<T>::load(y + c, o);
#pragma unroll
        for (int i = 0; i < V; ++i) {
          dot = fmaf(gv[i], o[i], dot);
          s[i] = gate * gv[i];
        }
        Vec16<T>::store(gy + c, s);
      }
    } else {
      for (int c = lane; c < d; c += 32) {
        const float gv = to_f32<T>(gin[c]);
        dot = fmaf(gv, to_f32<T>(y[c]), dot);
        gy[c] = from_f32<T>(gate * gv);
      }
    }
    dot = warp_sum(dot);
    if (lane == 0) a.dot_out[row] = dot;
  }
}

cudaError_t launch_scale_dot(const ScaleDotArgs& a, int precision, int sm_count, cudaStream_t stream) {
  const int grid = sm_count * 8;
  if (precision == PREC_BF16) { scale_dot_kernel<bf16><<<grid, CB_WARPS * 32, 0, stream>>>(a); count_launch(); }
  else { scale_dot_kernel<float><<<grid, CB_WARPS * 32, 0, stream>>>(a); count_launch(); }
  return cudaGetLastError();
}

__global__ void pull_dots_kernel(PullDotsArgs a) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= a.slots) return;
  const int pos = a.slot_pos[i];
  a.grad_gates[i] = pos < 0 ? 0.f : *aux_ptr(a.rows, pos, a.aux_off, 1);
}

cudaError_t launch_pull_dots(const PullDotsArgs& a, cudaStream_t stream) {
  if (a.slots <= 0) return cudaSuccess;
  pull_dots_kernel<<<ceil_div(a.slots, 256), 256, 0, stream>>>(a);
  count_launch();
  return cudaGetLastError();
}

constexpr int RB_ROWS = 64;

__global__ void __launch_bounds__(RB_ROWS) router_bwd_kernel(RouterBwdArgs a) {
  extern __shared__ float rb_smem[];
  const int E = a.E, k = a.k;
  float* gp = rb_smem + (size_t)threadIdx.x * (E + 1);
  const int t = blockIdx.x * RB_ROWS + threadIdx.x;
  if (t >= a.tokens) return;
  float* gl = a.grad_logits + (size_t)t * E;
  const int* sel = a.expert_of + (size_t)t * k;
  bf16* glb = a.grad_logits_bf16 ? a.grad_logits_bf16 + (size_t)t * E : nullptr;
  if (sel[0] < 0) {
    for (int e = 0; e < E; ++e) { gl[e] = 0.f; if (glb) glb[e] = __float2bfloat16_rn(0.f); }
    return;
  }
  const float* p = a.probs + (size_t)t * E;
  const float* gg = a.grad_gates + (size_t)t * k;
  for (int e = 0; e < E; ++e) gp[e] = 0.f;
  float total = 0.f;
  for (int j = 0; j < k; ++j) total = __fadd_rn(total, p[sel[j]]);
  if (total > 0.f) {
    float weighted = 0.f;
    for (int j = 0; j < k; ++j) weighted = __fadd_rn(weighted, __fmul_rn(gg[j], p[sel[j]]));
    for (int j = 0; j < k; ++j)
      gp[sel[j]] = __fadd_rn(gp[sel[j]], __fsub_rn(__fdiv_rn(gg[j], total), __fdiv_rn(weighted, __fmul_rn(total, total))));
  }
  const float Vf = a.ext_stats ? a.ext_stats[E + 1] : (float)a.total[3];
  if (a.aux_w != 0.f && Vf > 0.f) {
    const float scale = __fdiv_rn(__fmul_rn(a.aux_w, (float)E), Vf);
    const float slots = Vf * (float)k;
    for (int e = 0; e < E; ++e) {
      const float load = __fdiv_rn((float)(a.ext_counts ? a.ext_counts[e] : a.counts[e]), slots);
      gp[e] = __fadd_rn(gp[e], __fmul_rn(scale, load));
    }
  }
  float dot = 0.f;
  for (int e = 0; e < E; ++e) dot = __fadd_rn(dot, __fmul_rn(p[e], gp[e]));
  const float factor = a.z_w != 0.f ? __fdiv_rn(__fmul_rn(__fmul_rn(2.0f, a.z_w), a.lse[t]), fmaxf(Vf, 1.f)) : 0.f;
  for (int e = 0; e < E; ++e) {
    float v = __fmul_rn(p[e], __fsub_rn(gp[e], dot));
    if (a.z_w != 0.f) v = __fadd_rn(v, __fmul_rn(factor, p[e]));
    gl[e] = v;
    if (glb) glb[e] = __float2bfloat16_rn(v);
  }
}

cudaError_t launch_router_bwd(const RouterBwdArgs& a, cudaStream_t stream) {
  if (a.tokens <= 0) return cudaSuccess;
  const size_t smem = sizeof(float) * (size_t)RB_ROWS * (a.E + 1);
  if (smem > 48 * 1024) cudaFuncSetAttribute(router_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  router_bwd_kernel<<<ceil_div(a.tokens, RB_ROWS), RB_ROWS, smem, stream>>>(a); count_launch();
  return cudaGetLastError();
}

template <typename T, int KMAX>
__global__ void __launch_bounds__(CB_WARPS * 32) unpermute_kernel(UnpermuteArgs a) {
  const int lane = threadIdx.x & 31;
  // grid-stride over tokens: the launcher may cap the grid so that the kernel fits beside a
  // persistent GEMM on every SM
  for (int t = blockIdx.x * CB_WARPS + (threadIdx.x >> 5); t < a.tokens; t += gridDim.x * CB_WARPS) {
    int pos[KMAX];
    float unused[KMAX];
    const int n = slots_by_expert<KMAX>(a.expert_of, a.slot_pos, nullptr, t, a.k, lane, pos, unused);
    const int d = a.d, E = a.E;
    const size_t rb = (size_t)a.d * sizeof(T);
    const T* sh = (const T*)a.shared;
    const T* ex = (const T*)a.extra;
    const float* gl = a.grad_logits ? a.grad_logits + (size_t)t * E : nullptr;
    T* gx = (T*)a.grad_x + (size_t)t * d;
    constexpr int V = Vec16<T>::N;
    constexpr int RB = KMAX < ROW_BATCH ? KMAX : ROW_BATCH;
    if (d % V == 0 && d % 4 == 0) {
      for (int c = lane * V; c < d; c += 32 * V) {
        float acc[V], r[V];
#pragma unroll
        for (int i = 0; i < V; ++i) { acc[i] = 0.f; r[i] = 0.f; }
        if (sh) Vec16<T>::load(sh + (size_t)t * d + c, acc);
#pragma unroll
        for (int j0 = 0; j0 < KMAX; j0 += RB) {
          if (j0 >= n) break;
          uint4 raw[RB];
#pragma unroll
          for (int b = 0; b < RB; ++b)
            if (j0 + b < n) raw[b] = *reinterpret_cast<const uint4*>((const T*)row_ptr(a.grad_x_perm, pos[j0 + b], rb) + c);
#pragma unroll
          for (int b = 0; b < RB; ++b) {
            if (j0 + b < n) {
              float v[V];
              unpack16<T>(raw[b], v);
#pragma unroll
              for (int i = 0; i < V; ++i) acc[i] = __fadd_rn(acc[i], v[i]);
            }
          }
        }
        if (ex) Vec16<T>::load(ex + (size_t)t * d + c, r);
        for (int e = 0; gl && e < E; ++e) {
          const float g = gl[e];
          const float* w = a.w_router + (size_t)e * d + c;
#pragma unroll
          for (int i = 0; i < V; i += 4) {
            const float4 q = *reinterpret_cast<const float4*>(w + i);
            r[i] = fmaf(g, q.x, r[i]); r[i + 1] = fmaf(g, q.y, r[i + 1]);
            r[i + 2] = fmaf(g, q.z, r[i + 2]); r[i + 3] = fmaf(g, q.w, r[i + 3]);
          }
        }
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = __fadd_rn(acc[i], r[i]);
        if (a.accumulate) {
          float v[V];
          Vec16<T>::load(gx + c, v);
#pragma unroll
          for (int i = 0; i < V; ++i) acc[i] = __fadd_rn(v[i], acc[i]);
        }
        Vec16<T>::store(gx + c, acc);
      }
    } else {
      for (int c = lane; c < d; c += 32) {
        float acc = sh ? to_f32<T>(sh[(size_t)t * d + c]) : 0.f;
#pragma unroll
        for (int j = 0; j < KMAX; ++j)
          if (j < n) acc = __fadd_rn(acc, to_f32<T>(((const T*)row_ptr(a.grad_x_perm, pos[j], rb))[c]));
        float r = ex ? to_f32<T>(ex[(size_t)t * d + c]) : 0.f;
        for (int e = 0; gl && e < E; ++e) r = fmaf(gl[e], a.w_router[(size_t)e * d + c], r);
        acc = __fadd_rn(acc, r);
        if (a.accumulate) acc = __fadd_rn(to_f32<T>(gx[c]), acc);
        gx[c] = from_f32<T>(acc);
      }
    }
  }   // tokens
}

cudaError_t launch_unpermute(const UnpermuteArgs& a, int precision, cudaStream_t stream, int max_blocks) {
  if (a.tokens <= 0) return cudaSuccess;
  int grid = ceil_div(a.tokens, CB_WARPS);
  if (max_blocks > 0) grid = min(grid, max_blocks);
  if (precision == PREC_BF16) DISPATCH_KMAX(unpermute_kernel, bf16, a.k, grid, stream, a);
  else DISPATCH_KMAX(unpermute_kernel, float, a.k, grid, stream, a);
  return cudaGetLastError();
}

// Stage 1: block (col chunk, split) accumulates its tokens; stage 2 adds the splits in order.
constexpr int RW_COLS = 64;
constexpr int RW_TOK = 32;

template <typename T>
__global__ void __launch_bounds__(256) router_wgrad_stage1(RouterWgradArgs a) {
  extern __shared__ float rw_smem[];   // [RW_TOK][E] grad_logits chunk, [RW_TOK][RW_COLS] x chunk
  const int E = a.E, d = a.d;
  float* s_gl = rw_smem;
  float* s_x = rw_smem + (size_t)RW_TOK * E;
  const int c0 = blockIdx.x * RW_COLS;
  const int per = ceil_div(a.tokens, a.splits);
  const int tb = blockIdx.y * per, te = min(a.tokens, tb + per);
  const int col = threadIdx.x % RW_COLS;
  const int eg = threadIdx.x / RW_COLS;           // 4 expert groups
  const int e_per = ceil_div(E, 4);
  float acc[MAX_EXPERTS / 4];
#pragma unroll
  for (int i = 0; i < MAX_EXPERTS / 4; ++i) acc[i] = 0.f;
  const T* x = (const T*)a.x;
  for (int t0 = tb; t0 < te; t0 += RW_TOK) {
    const int nt = min(RW_TOK, te - t0);
    for (int i = threadIdx.x; i < RW_TOK * E; i += 256) {
      const int r = i / E;
      s_gl[i] = r < nt ? a.grad_logits[(size_t)(t0 + r) * E + (i - r * E)] : 0.f;
    }
    for (int i = threadIdx.x; i < RW_TOK * RW_COLS; i += 256) {
      const int r = i / RW_COLS, c = i - r * RW_COLS;
      s_x[i] = (r < nt && c0 + c < d) ? to_f32<T>(x[(size_t)(t0 + r) * d + c0 + c]) : 0.f;
    }
    __syncthreads();
    for (int r = 0; r < nt; ++r) {
      const float xv = s_x[r * RW_COLS + col];
#pragma unroll
      for (int i = 0; i < MAX_EXPERTS / 4; ++i) {
        const int e = eg * e_per + i;
        if (i < e_per && e < E) acc[i] = fmaf(s_gl[r * E + e], xv, acc[i]);
      }
    }
    __syncthreads();
  }
  if (c0 + col < d) {
#pragma unroll
    for (int i = 0; i < MAX_EXPERTS / 4; ++i) {
      const int e = eg * e_per + i;
      if (i < e_per && e < E) a.scratch[((size_t)blockIdx.y * E + e) * d + c0 + col] = acc[i];
    }
  }
}

__global__ void router_wgrad_stage2(RouterWgradArgs a) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long n = (long long)a.E * a.d;
  if (i >= n) return;
  float s = 0.f;
  for (int sp = 0; sp < a.splits; ++sp) s += a.scratch[(size_t)sp * n + i];
  a.grad_w[i] = a.accumulate ? a.grad_w[i] + s : s;
}

cudaError_t launch_router_wgrad(const RouterWgradArgs& a, int precision, cudaStream_t stream) {
  if (a.tokens <= 0) {
    if (!a.accumulate) return cudaMemsetAsync(a.grad_w, 0, sizeof(float) * (size_t)a.E * a.d, stream);
    return cudaSuccess;
  }
  const dim3 grid(ceil_div(a.d, RW_COLS), a.splits);
  const size_t smem = sizeof(float) * ((size_t)RW_TOK * a.E + (size_t)RW_TOK * RW_COLS);
  if (precision == PREC_BF16) { router_wgrad_stage1<bf16><<<grid, 256, smem, stream>>>(a); count_launch(); }
  else { router_wgrad_stage1<float><<<grid, 256, smem, stream>>>(a); count_launch(); }
  const long long n = (long long)a.E * a.d;
  router_wgrad_stage2<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(a); count_launch();
  return cudaGetLastError();
}

// Second stage alone: adds `splits` partial E x d results in order (the tensor-core path writes them).
cudaError_t launch_router_wgrad_sum(const RouterWgradArgs& a, cudaStream_t stream) {
  const long long n = (long long)a.E * a.d;
  router_wgrad_stage2<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(a); count_launch();
  return cudaGetLastError();
}

}  // namespace moe
