// Host-side interface of the tcgen05 grouped GEMM family (gemm_tc.cu).
#pragma once
#include "common.cuh"

namespace moe {
namespace tc {

constexpr int BM = 128;   // rows of one output tile (TMEM lanes)
constexpr int BN = 256;   // columns of one output tile (TMEM columns, fp32)
constexpr int BK = 64;    // reduction elements per pipeline stage (128 bytes of bf16)

enum Epilogue {
  EPI_STORE = 0,       // out0[row, col] = bf16(acc)
  EPI_SWIGLU = 1,      // acc holds interleaved gate|up blocks: out0 = silu(g)*u, out1 = (g|u) if non-null
  EPI_SWIGLU_BWD = 2,  // acc = dL/dh; aux = saved (g|u); out0 = (dg|du) in the same interleaved layout
  EPI_ACCUM_F32 = 3,   // out0 (f32) = acc  or  += acc
  EPI_STORE_F32 = 4,   // out0[row, col] = acc in f32, rows < M and cols < N only
};

struct GemmArgs {
  // Schedule.  Row groups come from the dispatch metadata: group g owns rows
  // [group_row0[g], group_row0[g+1]) of the row-indexed operands, a multiple of 128.
  const int* group_row0;  // [n_groups+1], device
  const int* tile_start;  // [n_groups+1], device: exclusive prefix of rows/128 (rows-as-M only)
  int n_groups;
  int N;                  // output columns
  int K;                  // reduction length (rows-as-M); ignored when the rows are the reduction
  int M;                  // output rows per group (rows-as-K only)
  void* out0;
  void* out1;
  const void* aux;
  long long ld0, ld1, ldaux;   // leading dimensions in elements
  long long group_stride0;     // rows-as-K: elements between consecutive groups of out0
  int accumulate;              // EPI_ACCUM_F32: add to out0 instead of overwriting
  int* error_flag;             // device int, set non-zero when a bounded wait gives up
  long long wait_limit = 0;    // filled at launch: clock cycles a barrier wait may take before it gives up
  int starve = 0;              // filled at launch (test hook): the producer loads nothing
  // Causal attention products (0: off).  `causal` is the sequence length S: row r of a group is query position
  // r % S (the g query heads of a group follow one another), key positions are 0 .. S-1, and entries with
  // key > query are known zeros (or never read).  What is skipped depends on where the keys sit:
  //   CAUSAL_COLS  rows-as-M, output columns are keys (Q K^T, dO V^T): tiles wholly above the diagonal are neither
  //                computed nor stored;
  //   CAUSAL_K     rows-as-M, the reduction runs over keys (P V, dS K): it stops after the tile's last visible key;
  //   rows-as-K    (P^T dO, dS^T Q: output rows are keys, the reduction runs over queries): K-stages whose queries
  //                all come before the tile's first key are skipped.  causal_kind is ignored.
  int causal = 0;
  int causal_kind = 0;
};
enum { CAUSAL_COLS = 1, CAUSAL_K = 2 };

// Operand descriptions for tensor-map construction (bf16, row-major).
struct Operand {
  const void* ptr;
  long long rows;      // rows per group (or total rows for row-indexed operands)
  long long cols;      // contiguous dimension
  long long groups;    // 1 for row-indexed operands
  long long ld = 0;    // elements between consecutive rows (0: cols); lets a product read a column range of a wider matrix
};

// Which kernel runs a product: 128x256 tiles on one SM, 256x256 tiles on a pair of SMs (cta_group::2, clusters of two
// CTAs; also MOE_B200_TC_PAIR=1), 256x256 tiles on one SM (forced with MOE_B200_TC_WIDE=1, never with =0), or - the
// default - a choice per launch between the first and the third (see wide_pays in gemm_tc.cu).
enum { TILE_ONE_SM = 0, TILE_PAIR = 1, TILE_WIDE = 2, TILE_AUTO = 3 };
void set_tile_mode(int mode);
int tile_mode();
// Only the 128-row kernel skips the masked part of a causal product; forced to the others, it is computed in full.
inline bool causal_skipping() { return tile_mode() == TILE_ONE_SM || tile_mode() == TILE_AUTO; }
bool pair_mode();
// Test hook: the next launch runs with a producer that loads nothing and this wait limit (clock cycles).
void set_starve_next_launch(long long wait_limit_cycles);

// y[rows, N] = A[rows, K] * B_g[N, K]^T            (forward projections)
cudaError_t gemm_rows_nt(const Operand& A, const Operand& B, const GemmArgs& args, int epilogue, int sm_count,
                         cudaStream_t stream);
// y[rows, N] = A[rows, K] * B_g[K, N]              (input gradients; B is the [out,in] weight itself)
cudaError_t gemm_rows_nn(const Operand& A, const Operand& B, const GemmArgs& args, int epilogue, int sm_count,
                         cudaStream_t stream);
// C_g[M, N] (+)= A[rows_g, M]^T * B[rows_g, N]     (weight gradients; the ragged rows are the reduction)
cudaError_t gemm_rows_tn(const Operand& A, const Operand& B, const GemmArgs& args, int sm_count,
                         cudaStream_t stream);

}  // namespace tc
}  // namespace moe
