// Shared declarations for the sm_100a mixture-of-experts library.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace moe {

typedef __nv_bfloat16 bf16;

constexpr int ROUTER_ROWS = 64;   // token rows handled by one router / permute block
constexpr int GROUP_ALIGN = 128;  // every expert's row group is padded to this many rows
constexpr int GU_BLOCK = 32;      // gate/up interleave: 32 gate rows, then their 32 up rows
constexpr int MAX_EXPERTS = 256;
constexpr int MAX_TOPK = 16;

enum Precision { PREC_F32 = 0, PREC_BF16 = 1 };

// Status codes of the C ABI (mirrors the reference's NetworkError variants that
// this path can raise: network.rs:19-83).
enum Status {
  ST_OK = 0,
  ST_INVALID_CONFIG = 1,  // NetworkError::InvalidConfig
  ST_INVALID_INPUT = 2,   // NetworkError::InvalidInput
  ST_CUDA = 3,            // NetworkError::Cuda
  ST_OOM = 4,             // NetworkError::CudaOutOfMemory
  ST_UNSUPPORTED = 5,     // NetworkError::UnsupportedCuda
  ST_TIMEOUT = 6,         // a bounded device-side wait gave up
  ST_COMM = 7,            // collective layer error
  ST_POISONED = 8,        // an earlier call on this handle failed (gpu_transformer.rs:160-195)
};

// Kernel launches issued by this library in this process (reported by the benchmark).
extern long long g_launch_count;
inline void count_launch(int n = 1) { g_launch_count += n; }

// Programmatic dependent launch.  While `g_pdl_scope` is set (the decode pass of a quantized layer sets it), the
// kernels launched through launch_kernel() may start while their predecessor on the stream is still running: the
// grid's blocks become resident early and wait in pdl_enter() until the predecessor has finished and its
// writes are visible, so the launch latency and the prologue overlap the predecessor's tail.  Outside the scope
// the launch is an ordinary one and pdl_enter() returns at once.
extern thread_local bool g_pdl_scope;
__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // this grid's successor may be scheduled
  asm volatile("griddepcontrol.wait;" ::: "memory");                // everything before this grid is complete
}
template <typename Kernel, typename... Args>
inline cudaError_t launch_kernel(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  if (!g_pdl_scope) {
    kernel<<<grid, block, smem, stream>>>(args...);
    return cudaGetLastError();
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ inline int round_up(int a, int b) { return ceil_div(a, b) * b; }

// Row of the packed gate|up matrix that holds logical row f of `which` (0 gate, 1 up).
__host__ __device__ inline int gu_row(int which, int f) {
  return (f / GU_BLOCK) * 2 * GU_BLOCK + which * GU_BLOCK + (f % GU_BLOCK);
}

template <typename T> __device__ inline float to_f32(T v);
template <> __device__ inline float to_f32<float>(float v) { return v; }
template <> __device__ inline float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ inline T from_f32(float v);
template <> __device__ inline float from_f32<float>(float v) { return v; }
template <> __device__ inline bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ inline float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// silu and its derivative as the reference defines them (ffn.rs:227-238), with
// expf rather than the fast intrinsic (cuda_training.rs:254).
__device__ inline float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ inline float siluf_(float x) { return x * sigmoidf_(x); }
__device__ inline float silu_grad_(float x) {
  const float s = sigmoidf_(x);
  return s * (1.0f + x * (1.0f - s));
}

// Where the expert-major rows live.  On one GPU that is a single local buffer (n = 1 and a
// row id is the row).  In an expert-parallel group every rank exposes its receive buffer to
// its peers (CUDA IPC over NVLink); a row id is then rank * cap + row and the kernels store
// to / load from the owner's memory directly.
constexpr int MAX_RANKS = 8;
struct RowSpace {
  void* base[MAX_RANKS];
  int cap;   // rows per rank
  int n;     // ranks
};
__host__ __device__ inline RowSpace local_rows(void* p) {
  RowSpace s{};
  s.base[0] = p; s.cap = 0x7fffffff; s.n = 1;
  return s;
}
__device__ inline char* row_ptr(const RowSpace& s, int id, size_t row_bytes) {
  if (s.n == 1) return (char*)s.base[0] + (size_t)id * row_bytes;
  const int r = id / s.cap;
  return (char*)s.base[r] + (size_t)(id - r * s.cap) * row_bytes;
}

// Device-resident routing metadata, rebuilt by every forward pass.
struct RouteMeta {
  int* counts;       // [E]   rows routed to each expert
  int* offsets;      // [E+1] compact exclusive prefix of counts
  int* pad_off;      // [E+1] start row of each expert's padded group (multiples of GROUP_ALIGN)
  int* tile_start;   // [E+1] exclusive prefix of padded_rows/GROUP_ALIGN (m-tiles per expert)
  int* total;        // [4]   {R, padded rows, m-tiles, valid tokens}
};

}  // namespace moe
