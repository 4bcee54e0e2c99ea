// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// CPU restatement of the mixture-of-experts feed-forward layer of the
// `rusting_brain` crate (version 2.0.2), used only as the correctness checker
// for the CUDA library and as the timed CPU baseline of the benchmark.  The
// product library never links, loads or calls anything in this file.
//
// What it follows, by reference file:line (paths inside the crate):
//   src/moe.rs:243-341    MoeLayer::forward_train   -> orc_forward
//   src/moe.rs:348-489    MoeLayer::backward        -> orc_backward
//   src/moe.rs:553-593    MoeLayer::route           -> route_rows / orc_route
//   src/moe.rs:602-639    auxiliary_losses          -> auxiliary_losses
//   src/moe.rs:643-664    softmax_rows, gather_rows -> softmax_rows
//   src/activations.rs:56-70  softmax               -> softmax_inplace
//   src/ffn.rs:56-120,227-238 SwiGlu fwd/bwd, silu  -> swiglu_* / silu
//   src/param.rs:762-825  Linear fwd/bwd ([out,in] weights, y = x W^T)
//   src/param.rs:547-617  Param::step (Sgd, Adam, Lion) -> orc_sgd_step / orc_adam_step / orc_lion_step
//   src/quantized.rs:29-99,154-177 int8 rows + f32 scale, 32-lane dot
//   src/batch.rs:247-268  Layout (padding mask)
//
// Third-party arithmetic that is NOT in the reference tree and is therefore
// restated from its published behaviour rather than reproduced bit for bit:
//   * matrixmultiply 0.3.11 (every CPU sgemm).  Its blocking / FMA summation
//     order cannot be recovered from the crate sources, so the GEMMs here match
//     it to f32 rounding only.  Float parity is "pinned to this restatement plus
//     finite-difference checks"; the summation order is explicitly unpinned.
//   * libm expf/logf (Rust's f32::exp / f32::ln lower to them on Linux/glibc);
//     this file calls the same glibc functions.
// Everything that decides an integer (softmax, top-k selection, stable
// bucketing, counts) follows the reference's sequential f32 order exactly, and is
// pinned by the reference's own closed-form known-answer tests (see
// tests/test_oracle_known_answers.py).
//
// The whole file is compiled with -ffp-contract=off (Rust never contracts a
// multiply and an add); the GEMM micro-kernels use explicit FMA intrinsics.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <immintrin.h>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

constexpr int UNROUTED = -1;  // moe.rs:191 uses usize::MAX; the device path uses -1

// ----------------------------------------------------------------------------
// GEMMs.  Row-major f32, f32 accumulation.
// ----------------------------------------------------------------------------

inline float hsum256(__m256 v) {
  __m128 lo = _mm256_castps256_ps128(v);
  __m128 hi = _mm256_extractf128_ps(v, 1);
  lo = _mm_add_ps(lo, hi);
  __m128 sh = _mm_movehdup_ps(lo);
  __m128 s = _mm_add_ps(lo, sh);
  sh = _mm_movehl_ps(sh, s);
  s = _mm_add_ss(s, sh);
  return _mm_cvtss_f32(s);
}

// C[m, n] = sum_k A[m,k] * B[n,k]   (Matrix::dot_rhs_transposed, matrix.rs:121-173)
// rows [m0, m1) of A only.
void gemm_nt_rows(const float* A, const float* B, float* C, int m0, int m1, int N, int K,
                  int lda, int ldb, int ldc) {
  const int K8 = K & ~7;
  for (int j0 = 0; j0 < N; j0 += 64) {
    const int j1 = std::min(N, j0 + 64);
    int i = m0;
    for (; i + 4 <= m1; i += 4) {
      int j = j0;
      for (; j + 4 <= j1; j += 4) {
        __m256 acc[4][4];
        for (auto& r : acc)
          for (auto& v : r) v = _mm256_setzero_ps();
        for (int k = 0; k < K8; k += 8) {
          __m256 a[4], b[4];
          for (int r = 0; r < 4; ++r) a[r] = _mm256_loadu_ps(A + (size_t)(i + r) * lda + k);
          for (int c = 0; c < 4; ++c) b[c] = _mm256_loadu_ps(B + (size_t)(j + c) * ldb + k);
          for (int r = 0; r < 4; ++r)
            for (int c = 0; c < 4; ++c) acc[r][c] = _mm256_fmadd_ps(a[r], b[c], acc[r][c]);
        }
        for (int r = 0; r < 4; ++r)
          for (int c = 0; c < 4; ++c) {
            float s = hsum256(acc[r][c]);
            for (int k = K8; k < K; ++k)
              s = std::fmaf(A[(size_t)(i + r) * lda + k], B[(size_t)(j + c) * ldb + k], s);
            C[(size_t)(i + r) * ldc + j + c] = s;
          }
      }
      for (; j < j1; ++j)
        for (int r = 0; r < 4; ++r) {
          float s = 0.f;
          for (int k = 0; k < K; ++k)
            s = std::fmaf(A[(size_t)(i + r) * lda + k], B[(size_t)j * ldb + k], s);
          C[(size_t)(i + r) * ldc + j] = s;
        }
    }
    for (; i < m1; ++i)
      for (int j = j0; j < j1; ++j) {
        __m256 acc = _mm256_setzero_ps();
        for (int k = 0; k < K8; k += 8)
          acc = _mm256_fmadd_ps(_mm256_loadu_ps(A + (size_t)i * lda + k),
                                _mm256_loadu_ps(B + (size_t)j * ldb + k), acc);
        float s = hsum256(acc);
        for (int k = K8; k < K; ++k) s = std::fmaf(A[(size_t)i * lda + k], B[(size_t)j * ldb + k], s);
        C[(size_t)i * ldc + j] = s;
      }
  }
}

// C[m, k] = sum_n A[m,n] * B[n,k]   (Matrix::dot, matrix.rs:66-89), rows [m0,m1).
void gemm_nn_rows(const float* A, const float* B, float* C, int m0, int m1, int N, int K,
                  int lda, int ldb, int ldc) {
  const int K16 = K & ~15;
  int i = m0;
  for (; i + 4 <= m1; i += 4) {
    for (int k = 0; k < K16; k += 16) {
      __m256 acc[4][2];
      for (auto& r : acc)
        for (auto& v : r) v = _mm256_setzero_ps();
      for (int n = 0; n < N; ++n) {
        __m256 b0 = _mm256_loadu_ps(B + (size_t)n * ldb + k);
        __m256 b1 = _mm256_loadu_ps(B + (size_t)n * ldb + k + 8);
        for (int r = 0; r < 4; ++r) {
          __m256 a = _mm256_broadcast_ss(A + (size_t)(i + r) * lda + n);
          acc[r][0] = _mm256_fmadd_ps(a, b0, acc[r][0]);
          acc[r][1] = _mm256_fmadd_ps(a, b1, acc[r][1]);
        }
      }
      for (int r = 0; r < 4; ++r) {
        _mm256_storeu_ps(C + (size_t)(i + r) * ldc + k, acc[r][0]);
        _mm256_storeu_ps(C + (size_t)(i + r) * ldc + k + 8, acc[r][1]);
      }
    }
    for (int k = K16; k < K; ++k)
      for (int r = 0; r < 4; ++r) {
        float s = 0.f;
        for (int n = 0; n < N; ++n) s = std::fmaf(A[(size_t)(i + r) * lda + n], B[(size_t)n * ldb + k], s);
        C[(size_t)(i + r) * ldc + k] = s;
      }
  }
  for (; i < m1; ++i)
    for (int k = 0; k < K; ++k) {
      float s = 0.f;
      for (int n = 0; n < N; ++n) s = std::fmaf(A[(size_t)i * lda + n], B[(size_t)n * ldb + k], s);
      C[(size_t)i * ldc + k] = s;
    }
}

// C[n, k] += sum_m A[m,n] * B[m,k]  (Matrix::dot_self_transposed_accumulate,
// matrix.rs:273-296), output rows [n0,n1).
void gemm_tn_acc_rows(const float* A, const float* B, float* C, int M, int n0, int n1, int K,
                      int lda, int ldb, int ldc) {
  const int K16 = K & ~15;
  int i = n0;
  for (; i + 4 <= n1; i += 4) {
    for (int k = 0; k < K16; k += 16) {
      __m256 acc[4][2];
      for (auto& r : acc)
        for (auto& v : r) v = _mm256_setzero_ps();
      for (int m = 0; m < M; ++m) {
        __m256 b0 = _mm256_loadu_ps(B + (size_t)m * ldb + k);
        __m256 b1 = _mm256_loadu_ps(B + (size_t)m * ldb + k + 8);
        for (int r = 0; r < 4; ++r) {
          __m256 a = _mm256_broadcast_ss(A + (size_t)m * lda + i + r);
          acc[r][0] = _mm256_fmadd_ps(a, b0, acc[r][0]);
          acc[r][1] = _mm256_fmadd_ps(a, b1, acc[r][1]);
        }
      }
      for (int r = 0; r < 4; ++r) {
        float* c = C + (size_t)(i + r) * ldc + k;
        _mm256_storeu_ps(c, _mm256_add_ps(_mm256_loadu_ps(c), acc[r][0]));
        _mm256_storeu_ps(c + 8, _mm256_add_ps(_mm256_loadu_ps(c + 8), acc[r][1]));
      }
    }
    for (int k = K16; k < K; ++k)
      for (int r = 0; r < 4; ++r) {
        float s = 0.f;
        for (int m = 0; m < M; ++m) s = std::fmaf(A[(size_t)m * lda + i + r], B[(size_t)m * ldb + k], s);
        C[(size_t)(i + r) * ldc + k] += s;
      }
  }
  for (; i < n1; ++i)
    for (int k = 0; k < K; ++k) {
      float s = 0.f;
      for (int m = 0; m < M; ++m) s = std::fmaf(A[(size_t)m * lda + i], B[(size_t)m * ldb + k], s);
      C[(size_t)i * ldc + k] += s;
    }
}

// ----------------------------------------------------------------------------
// int8 weights (quantized.rs)
// ----------------------------------------------------------------------------

// quantized.rs:29-51  per row: scale = absmax/127; q = round(w/scale) clamped.
void quantize_rows(const float* w, int rows, int cols, int8_t* q, float* scales) {
  for (int r = 0; r < rows; ++r) {
    const float* row = w + (size_t)r * cols;
    float absmax = 0.f;
    for (int c = 0; c < cols; ++c) absmax = std::max(absmax, std::fabs(row[c]));
    const float scale = absmax / 127.0f;
    scales[r] = scale;
    const float inverse = scale > 0.f ? 1.0f / scale : 0.f;
    for (int c = 0; c < cols; ++c) {
      // f32::round is round-half-away-from-zero, as roundf.
      float v = std::round(row[c] * inverse);
      v = std::min(127.f, std::max(-127.f, v));
      q[(size_t)r * cols + c] = (int8_t)v;
    }
  }
}

// quantized.rs:154-177 with LANES = 32 (the AVX2+FMA dispatch of :188-195; Rust
// does not contract x*w + acc, and neither does this file).
float dot_lanes32(const float* x, const int8_t* w, int n) {
  float lanes[32];
  for (float& l : lanes) l = 0.f;
  const int tail = n - n % 32;
  for (int i = 0; i < tail; i += 32)
    for (int lane = 0; lane < 32; ++lane) lanes[lane] += x[i + lane] * (float)w[i + lane];
  float rest = 0.f;
  for (int i = tail; i < n; ++i) rest += x[i] * (float)w[i];
  float s = 0.f;
  for (float l : lanes) s += l;
  return s + rest;
}

struct Weight {
  int rows = 0, cols = 0;        // [out, in]
  std::vector<float> value, grad, m, v;
  std::vector<int8_t> q;         // non-empty => the int8 representation is live
  std::vector<float> scales;
  bool quantized() const { return !q.empty(); }
  void resize(int r, int c) {
    rows = r; cols = c;
    value.assign((size_t)r * c, 0.f);
  }
  // gradient and Adam state are created on first use (a forward-only timing run of a large
  // layer should not hold four copies of every weight)
  void need_grad() { if (grad.size() != value.size()) grad.assign(value.size(), 0.f); }
  void need_moments() {
    if (m.size() != value.size()) { m.assign(value.size(), 0.f); v.assign(value.size(), 0.f); }
  }
};

// Linear::forward (param.rs:762-796) for rows [m0,m1) of `x`.
void linear_forward_rows(const Weight& w, const float* x, float* y, int m0, int m1) {
  if (w.quantized()) {
    // quantized.rs:55-99: y[t,r] = dot(x[t,:], q[r,:]) * scale[r]
    for (int t = m0; t < m1; ++t)
      for (int r = 0; r < w.rows; ++r)
        y[(size_t)t * w.rows + r] =
            dot_lanes32(x + (size_t)t * w.cols, w.q.data() + (size_t)r * w.cols, w.cols) * w.scales[r];
    return;
  }
  gemm_nt_rows(x, w.value.data(), y, m0, m1, w.rows, w.cols, w.cols, w.cols, w.rows);
}

inline float sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }          // ffn.rs:227
inline float silu(float x) { return x * sigmoid(x); }                        // ffn.rs:231
inline float silu_derivative(float x) {                                      // ffn.rs:235
  const float s = sigmoid(x);
  return s * (1.0f + x * (1.0f - s));
}

struct SwiGlu {
  Weight gate, up, down;
};

struct SwiGluCache {
  int rows = 0;
  std::vector<float> input, gate, up, hidden, output;  // output is pre-gate (moe.rs:309)
};

constexpr int ROW_BLOCK = 64;

struct Layer {
  int d = 0, E = 0, k = 0, F = 0;
  bool has_shared = false;
  float aux_w = 0.01f, z_w = 1e-3f;
  Weight router;
  std::vector<SwiGlu> experts;
  SwiGlu shared;

  // MoeCache (moe.rs:131-156)
  int T = 0, valid_tokens = 0;
  std::vector<float> input, logits, probs, lse;
  std::vector<int> expert_of;
  std::vector<float> gates;
  std::vector<uint8_t> valid;
  std::vector<std::vector<int>> expert_tokens, expert_slots;
  std::vector<SwiGluCache> caches;
  SwiGluCache shared_cache;
  float aux = 0.f, z = 0.f;
};

// activations.rs:56-70
void softmax_inplace(float* v, int n) {
  float mx = -INFINITY;
  for (int i = 0; i < n; ++i) mx = std::fmax(mx, v[i]);
  float sum = 0.f;
  for (int i = 0; i < n; ++i) {
    v[i] = expf(v[i] - mx);
    sum += v[i];
  }
  if (sum > 0.f)
    for (int i = 0; i < n; ++i) v[i] /= sum;
}

// moe.rs:643-656
void softmax_rows(const float* logits, int T, int E, float* probs, float* lse) {
  std::memcpy(probs, logits, sizeof(float) * (size_t)T * E);
  for (int r = 0; r < T; ++r) {
    const float* src = logits + (size_t)r * E;
    float mx = -INFINITY;
    for (int i = 0; i < E; ++i) mx = std::fmax(mx, src[i]);
    float sum = 0.f;
    for (int i = 0; i < E; ++i) sum += expf(src[i] - mx);
    lse[r] = mx + logf(sum);
    softmax_inplace(probs + (size_t)r * E, E);
  }
}

// moe.rs:553-593
void route_rows(const float* probs, int T, int E, int k, const uint8_t* valid, int* expert_of,
                float* gates) {
  for (int t = 0; t < T; ++t) {
    int* sel = expert_of + (size_t)t * k;
    float* g = gates + (size_t)t * k;
    if (valid && !valid[t]) {
      for (int r = 0; r < k; ++r) { sel[r] = UNROUTED; g[r] = 0.f; }
      continue;
    }
    const float* row = probs + (size_t)t * E;
    for (int r = 0; r < k; ++r) {
      int best = -1;
      for (int e = 0; e < E; ++e) {
        bool taken = false;
        for (int j = 0; j < r; ++j) taken |= (sel[j] == e);
        if (taken) continue;
        if (best < 0 || row[e] > row[best]) best = e;   // strict > : ties -> lowest index
      }
      sel[r] = best;
      g[r] = row[best];
    }
    float total = 0.f;
    for (int r = 0; r < k; ++r) total += g[r];
    if (total > 0.f)
      for (int r = 0; r < k; ++r) g[r] /= total;
  }
}

// moe.rs:602-639
void auxiliary_losses(Layer& L) {
  L.aux = 0.f; L.z = 0.f;
  if (L.valid_tokens == 0) return;
  const float tokens = (float)L.valid_tokens;
  const float slots = (float)L.valid_tokens * (float)L.k;
  float aux = 0.f;
  for (int e = 0; e < L.E; ++e) {
    const float load = (float)L.expert_tokens[e].size() / slots;
    float sum = 0.f;
    for (int t = 0; t < L.T; ++t)
      if (L.valid.empty() || L.valid[t]) sum += L.probs[(size_t)t * L.E + e];
    const float mass = sum / tokens;
    aux += load * mass;
  }
  aux *= (float)L.E * L.aux_w;
  float zs = 0.f;
  for (int t = 0; t < L.T; ++t)
    if (L.valid.empty() || L.valid[t]) zs += L.lse[t] * L.lse[t];
  L.aux = aux;
  L.z = L.z_w * zs / tokens;
}

struct Task { int expert, m0, m1; };

std::vector<Task> row_tasks(const std::vector<SwiGluCache*>& caches) {
  std::vector<Task> tasks;
  for (int e = 0; e < (int)caches.size(); ++e)
    for (int m0 = 0; m0 < caches[e]->rows; m0 += ROW_BLOCK)
      tasks.push_back({e, m0, std::min(caches[e]->rows, m0 + ROW_BLOCK)});
  return tasks;
}

// SwiGlu::forward_train (ffn.rs:56-85) over a set of independent (expert, rows)
// groups.  The reference forks over experts with rayon (moe.rs:283-288) and lets
// the threaded sgemm split each product; here both levels are flattened into
// (expert, 64-row block) tasks on an OpenMP team.
void swiglu_forward_many(const std::vector<const SwiGlu*>& mods, const std::vector<SwiGluCache*>& caches,
                         int d, int F) {
  for (auto* c : caches) {
    c->gate.assign((size_t)c->rows * F, 0.f);
    c->up.assign((size_t)c->rows * F, 0.f);
    c->hidden.assign((size_t)c->rows * F, 0.f);
    c->output.assign((size_t)c->rows * d, 0.f);
  }
  const std::vector<Task> tasks = row_tasks(caches);
#pragma omp parallel for schedule(dynamic)
  for (int i = 0; i < (int)tasks.size(); ++i) {
    const Task& t = tasks[i];
    SwiGluCache& c = *caches[t.expert];
    const SwiGlu& m = *mods[t.expert];
    linear_forward_rows(m.gate, c.input.data(), c.gate.data(), t.m0, t.m1);
    linear_forward_rows(m.up, c.input.data(), c.up.data(), t.m0, t.m1);
    for (size_t j = (size_t)t.m0 * F; j < (size_t)t.m1 * F; ++j) c.hidden[j] = silu(c.gate[j]) * c.up[j];
    linear_forward_rows(m.down, c.hidden.data(), c.output.data(), t.m0, t.m1);
  }
}

// SwiGlu::backward (ffn.rs:87-120) for many groups: returns dL/dinput per group in
// `grad_inputs` and accumulates the three weight gradients.
void swiglu_backward_many(const std::vector<SwiGlu*>& mods, const std::vector<SwiGluCache*>& caches,
                          const std::vector<std::vector<float>*>& grad_outputs,
                          const std::vector<std::vector<float>*>& grad_inputs, int d, int F) {
  const int G = (int)caches.size();
  std::vector<std::vector<float>> grad_hidden(G), grad_gate(G), grad_up(G);
  for (int e = 0; e < G; ++e) {
    const size_t n = (size_t)caches[e]->rows * F;
    grad_hidden[e].assign(n, 0.f);
    grad_gate[e].assign(n, 0.f);
    grad_up[e].assign(n, 0.f);
    grad_inputs[e]->assign((size_t)caches[e]->rows * d, 0.f);
  }
  const std::vector<Task> tasks = row_tasks(caches);
  // dgrad through down, the pointwise part, and dgrad through gate and up.
#pragma omp parallel for schedule(dynamic)
  for (int i = 0; i < (int)tasks.size(); ++i) {
    const Task& t = tasks[i];
    const int e = t.expert;
    SwiGluCache& c = *caches[e];
    gemm_nn_rows(grad_outputs[e]->data(), mods[e]->down.value.data(), grad_hidden[e].data(), t.m0, t.m1,
                 d, F, d, F, F);
    for (size_t j = (size_t)t.m0 * F; j < (size_t)t.m1 * F; ++j) {
      const float g = c.gate[j];
      grad_gate[e][j] = grad_hidden[e][j] * c.up[j] * silu_derivative(g);
      grad_up[e][j] = grad_hidden[e][j] * silu(g);
    }
    std::vector<float> from_up((size_t)(t.m1 - t.m0) * d);
    gemm_nn_rows(grad_gate[e].data(), mods[e]->gate.value.data(), grad_inputs[e]->data(), t.m0, t.m1, F, d,
                 F, d, d);
    gemm_nn_rows(grad_up[e].data() + (size_t)t.m0 * F, mods[e]->up.value.data(), from_up.data(), 0,
                 t.m1 - t.m0, F, d, F, d, d);
    float* gi = grad_inputs[e]->data() + (size_t)t.m0 * d;
    for (size_t j = 0; j < from_up.size(); ++j) gi[j] += from_up[j];
  }
  // Weight gradients: tasks are (group, which weight, 32-row block of the output).
  struct WTask { int e, which, n0, n1; };
  std::vector<WTask> wt;
  for (int e = 0; e < G; ++e) {
    if (caches[e]->rows == 0) continue;
    for (int n0 = 0; n0 < d; n0 += 32) wt.push_back({e, 0, n0, std::min(d, n0 + 32)});
    for (int n0 = 0; n0 < F; n0 += 32) wt.push_back({e, 1, n0, std::min(F, n0 + 32)});
    for (int n0 = 0; n0 < F; n0 += 32) wt.push_back({e, 2, n0, std::min(F, n0 + 32)});
  }
#pragma omp parallel for schedule(dynamic)
  for (int i = 0; i < (int)wt.size(); ++i) {
    const WTask& t = wt[i];
    SwiGluCache& c = *caches[t.e];
    if (t.which == 0)  // dW_down[d,F] += dy^T h
      gemm_tn_acc_rows(grad_outputs[t.e]->data(), c.hidden.data(), mods[t.e]->down.grad.data(), c.rows, t.n0,
                       t.n1, F, d, F, F);
    else if (t.which == 1)  // dW_gate[F,d] += dg^T x
      gemm_tn_acc_rows(grad_gate[t.e].data(), c.input.data(), mods[t.e]->gate.grad.data(), c.rows, t.n0, t.n1,
                       d, F, d, d);
    else
      gemm_tn_acc_rows(grad_up[t.e].data(), c.input.data(), mods[t.e]->up.grad.data(), c.rows, t.n0, t.n1, d,
                       F, d, d);
  }
}

Weight* pick(Layer& L, int which, int expert) {
  switch (which) {
    case 0: return &L.router;
    case 1: return expert >= 0 && expert < L.E ? &L.experts[expert].gate : nullptr;
    case 2: return expert >= 0 && expert < L.E ? &L.experts[expert].up : nullptr;
    case 3: return expert >= 0 && expert < L.E ? &L.experts[expert].down : nullptr;
    case 4: return L.has_shared ? &L.shared.gate : nullptr;
    case 5: return L.has_shared ? &L.shared.up : nullptr;
    case 6: return L.has_shared ? &L.shared.down : nullptr;
  }
  return nullptr;
}

void for_each_weight(Layer& L, void (*fn)(Weight&, void*), void* ctx) {
  // params_mut order, moe.rs:516-525: router, experts (gate, up, down), shared.
  fn(L.router, ctx);
  for (auto& e : L.experts) { fn(e.gate, ctx); fn(e.up, ctx); fn(e.down, ctx); }
  if (L.has_shared) { fn(L.shared.gate, ctx); fn(L.shared.up, ctx); fn(L.shared.down, ctx); }
}

}  // namespace

extern "C" {

// MoeConfig::validate (moe.rs:68-86): returns nullptr for an invalid config.
void* orc_create(int d_model, int num_experts, int top_k, int d_ff, int shared, float aux_w, float z_w) {
  if (num_experts <= 0 || top_k <= 0 || top_k > num_experts || d_ff <= 0 || d_model <= 0) return nullptr;
  Layer* L = new Layer;
  L->d = d_model; L->E = num_experts; L->k = top_k; L->F = d_ff;
  L->has_shared = shared != 0; L->aux_w = aux_w; L->z_w = z_w;
  L->router.resize(num_experts, d_model);
  L->experts.resize(num_experts);
  for (auto& e : L->experts) {
    e.gate.resize(d_ff, d_model); e.up.resize(d_ff, d_model); e.down.resize(d_model, d_ff);
  }
  if (L->has_shared) {
    L->shared.gate.resize(d_ff, d_model); L->shared.up.resize(d_ff, d_model); L->shared.down.resize(d_model, d_ff);
  }
  return L;
}

void orc_destroy(void* h) { delete (Layer*)h; }

void orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int orc_max_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

int orc_set_weight(void* h, int which, int expert, const float* src, int rows, int cols) {
  Weight* w = pick(*(Layer*)h, which, expert);
  if (!w || w->rows != rows || w->cols != cols) return 1;
  std::memcpy(w->value.data(), src, sizeof(float) * (size_t)rows * cols);
  w->q.clear(); w->scales.clear();
  return 0;
}

int orc_get_weight(void* h, int which, int expert, float* dst) {
  Weight* w = pick(*(Layer*)h, which, expert);
  if (!w) return 1;
  std::memcpy(dst, w->value.data(), sizeof(float) * w->value.size());
  return 0;
}

int orc_get_grad(void* h, int which, int expert, float* dst) {
  Weight* w = pick(*(Layer*)h, which, expert);
  if (!w) return 1;
  w->need_grad();
  std::memcpy(dst, w->grad.data(), sizeof(float) * w->grad.size());
  return 0;
}

int orc_get_moments(void* h, int which, int expert, float* m, float* v) {
  Weight* w = pick(*(Layer*)h, which, expert);
  if (!w) return 1;
  w->need_moments();
  std::memcpy(m, w->m.data(), sizeof(float) * w->m.size());
  std::memcpy(v, w->v.data(), sizeof(float) * w->v.size());
  return 0;
}

// Installs an int8 representation (values + one f32 scale per output row).
int orc_set_weight_q8(void* h, int which, int expert, const int8_t* q, const float* scales, int rows, int cols) {
  Weight* w = pick(*(Layer*)h, which, expert);
  if (!w || w->rows != rows || w->cols != cols) return 1;
  w->q.assign(q, q + (size_t)rows * cols);
  w->scales.assign(scales, scales + rows);
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < cols; ++c) w->value[(size_t)r * cols + c] = (float)q[(size_t)r * cols + c] * scales[r];
  return 0;
}

// TransformerLm::quantize quantizes every Linear including the router
// (transformer.rs:899-910); `include_router` = 0 keeps the router in f32.
void orc_quantize(void* h, int include_router) {
  Layer& L = *(Layer*)h;
  auto qz = [](Weight& w) {
    w.q.resize(w.value.size()); w.scales.resize(w.rows);
    quantize_rows(w.value.data(), w.rows, w.cols, w.q.data(), w.scales.data());
  };
  if (include_router) qz(L.router);
  for (auto& e : L.experts) { qz(e.gate); qz(e.up); qz(e.down); }
  if (L.has_shared) { qz(L.shared.gate); qz(L.shared.up); qz(L.shared.down); }
}

void orc_quantize_rows(const float* w, int rows, int cols, int8_t* q, float* scales) {
  quantize_rows(w, rows, cols, q, scales);
}

void orc_q8_matmul(const float* x, int T, const int8_t* q, const float* scales, int rows, int cols, float* y) {
  for (int t = 0; t < T; ++t)
    for (int r = 0; r < rows; ++r)
      y[(size_t)t * rows + r] = dot_lanes32(x + (size_t)t * cols, q + (size_t)r * cols, cols) * scales[r];
}

void orc_softmax_rows(const float* logits, int T, int E, float* probs, float* lse) {
  softmax_rows(logits, T, E, probs, lse);
}

void orc_route(const float* probs, int T, int E, int k, const uint8_t* valid, int* expert_of, float* gates) {
  route_rows(probs, T, E, k, valid, expert_of, gates);
}

float orc_silu(float x) { return silu(x); }
float orc_silu_derivative(float x) { return silu_derivative(x); }

// MoeLayer::forward_train.  `valid` may be null (every row is a token);
// `logits_override` may be null; when given it replaces the router product so a
// device path's own logits can be fed back for the bit-exact routing checks.
// Returns 0, or 1 for the InvalidInput / InvalidConfig cases of moe.rs:248-259.
int orc_forward(void* h, const float* x, int T, int cols, const uint8_t* valid, int valid_len,
                const float* logits_override, float* y) {
  Layer& L = *(Layer*)h;
  if (cols != L.d) return 1;
  if (valid && valid_len != T) return 1;
  const int d = L.d, E = L.E, k = L.k, F = L.F;
  L.T = T;
  L.input.assign(x, x + (size_t)T * d);
  L.valid.clear();
  if (valid) L.valid.assign(valid, valid + T);
  L.valid_tokens = 0;
  for (int t = 0; t < T; ++t) L.valid_tokens += (!valid || valid[t]) ? 1 : 0;

  L.logits.assign((size_t)T * E, 0.f);
  if (logits_override) {
    std::memcpy(L.logits.data(), logits_override, sizeof(float) * (size_t)T * E);
  } else {
#pragma omp parallel for schedule(static)
    for (int m0 = 0; m0 < T; m0 += ROW_BLOCK)
      linear_forward_rows(L.router, x, L.logits.data(), m0, std::min(T, m0 + ROW_BLOCK));
  }
  L.probs.assign((size_t)T * E, 0.f);
  L.lse.assign(T, 0.f);
  softmax_rows(L.logits.data(), T, E, L.probs.data(), L.lse.data());
  L.expert_of.assign((size_t)T * k, 0);
  L.gates.assign((size_t)T * k, 0.f);
  route_rows(L.probs.data(), T, E, k, valid, L.expert_of.data(), L.gates.data());

  // moe.rs:266-274: stable bucketing of slots by expert.
  L.expert_tokens.assign(E, {});
  L.expert_slots.assign(E, {});
  for (int slot = 0; slot < T * k; ++slot) {
    const int e = L.expert_of[slot];
    if (e == UNROUTED) continue;
    L.expert_tokens[e].push_back(slot / k);
    L.expert_slots[e].push_back(slot);
  }

  // moe.rs:276-288: gather, then the experts.
  L.caches.assign(E, {});
  std::vector<const SwiGlu*> mods(E);
  std::vector<SwiGluCache*> caches(E);
  for (int e = 0; e < E; ++e) {
    SwiGluCache& c = L.caches[e];
    c.rows = (int)L.expert_tokens[e].size();
    c.input.resize((size_t)c.rows * d);
    for (int r = 0; r < c.rows; ++r)
      std::memcpy(c.input.data() + (size_t)r * d, x + (size_t)L.expert_tokens[e][r] * d, sizeof(float) * d);
    mods[e] = &L.experts[e];
    caches[e] = &c;
  }
  swiglu_forward_many(mods, caches, d, F);

  // moe.rs:290-311: combine, experts ascending, rows ascending.
  std::fill(y, y + (size_t)T * d, 0.f);
  for (int e = 0; e < E; ++e)
    for (int r = 0; r < L.caches[e].rows; ++r) {
      const float gate = L.gates[L.expert_slots[e][r]];
      float* dst = y + (size_t)L.expert_tokens[e][r] * d;
      const float* src = L.caches[e].output.data() + (size_t)r * d;
      for (int c = 0; c < d; ++c) dst[c] += gate * src[c];
    }

  // moe.rs:313-319: the shared expert sees every row, padding included.
  if (L.has_shared) {
    L.shared_cache.rows = T;
    L.shared_cache.input.assign(x, x + (size_t)T * d);
    std::vector<const SwiGlu*> sm{&L.shared};
    std::vector<SwiGluCache*> sc{&L.shared_cache};
    swiglu_forward_many(sm, sc, d, F);
    for (size_t i = 0; i < (size_t)T * d; ++i) y[i] += L.shared_cache.output[i];
  }
  auxiliary_losses(L);
  return 0;
}

void orc_get_losses(void* h, float* aux, float* z) {
  Layer& L = *(Layer*)h;
  *aux = L.aux; *z = L.z;
}

// expert_of/gates are [T*k]; counts [E]; token_of/slot_of are the stable
// expert-major permutation, length sum(counts).  Any pointer may be null.
int orc_get_routing(void* h, int* expert_of, float* gates, int* counts, int* token_of, int* slot_of) {
  Layer& L = *(Layer*)h;
  if (expert_of) std::memcpy(expert_of, L.expert_of.data(), sizeof(int) * L.expert_of.size());
  if (gates) std::memcpy(gates, L.gates.data(), sizeof(float) * L.gates.size());
  int n = 0;
  for (int e = 0; e < L.E; ++e) {
    if (counts) counts[e] = (int)L.expert_tokens[e].size();
    for (size_t r = 0; r < L.expert_tokens[e].size(); ++r, ++n) {
      if (token_of) token_of[n] = L.expert_tokens[e][r];
      if (slot_of) slot_of[n] = L.expert_slots[e][r];
    }
  }
  return n;
}

void orc_get_router(void* h, float* logits, float* probs, float* lse) {
  Layer& L = *(Layer*)h;
  if (logits) std::memcpy(logits, L.logits.data(), sizeof(float) * L.logits.size());
  if (probs) std::memcpy(probs, L.probs.data(), sizeof(float) * L.probs.size());
  if (lse) std::memcpy(lse, L.lse.data(), sizeof(float) * L.lse.size());
}

// Expert activations in permuted (expert-major) row order: hidden [R,F] and the
// pre-gate expert outputs [R,d].  Either pointer may be null.
void orc_get_expert_rows(void* h, float* hidden, float* outputs) {
  Layer& L = *(Layer*)h;
  size_t r0 = 0;
  for (int e = 0; e < L.E; ++e) {
    const SwiGluCache& c = L.caches[e];
    if (hidden) std::memcpy(hidden + r0 * L.F, c.hidden.data(), sizeof(float) * c.hidden.size());
    if (outputs) std::memcpy(outputs + r0 * L.d, c.output.data(), sizeof(float) * c.output.size());
    r0 += c.rows;
  }
}

void orc_zero_grad(void* h) {
  for_each_weight(*(Layer*)h, [](Weight& w, void*) { w.need_grad(); std::fill(w.grad.begin(), w.grad.end(), 0.f); }, nullptr);
}

// MoeLayer::backward (moe.rs:348-489).  Weight gradients accumulate.
int orc_backward(void* h, const float* grad_out, float* grad_in) {
  Layer& L = *(Layer*)h;
  const int T = L.T, d = L.d, E = L.E, k = L.k, F = L.F;
  for_each_weight(L, [](Weight& w, void*) { w.need_grad(); }, nullptr);
  std::fill(grad_in, grad_in + (size_t)T * d, 0.f);

  if (L.has_shared) {  // :356-361
    std::vector<float> go(grad_out, grad_out + (size_t)T * d), gi;
    std::vector<SwiGlu*> sm{&L.shared};
    std::vector<SwiGluCache*> sc{&L.shared_cache};
    std::vector<std::vector<float>*> gos{&go}, gis{&gi};
    swiglu_backward_many(sm, sc, gos, gis, d, F);
    for (size_t i = 0; i < gi.size(); ++i) grad_in[i] += gi[i];
  }

  // :366-387 scaled upstream rows per expert, then SwiGlu::backward.
  std::vector<std::vector<float>> scaled(E), contrib(E);
  std::vector<SwiGlu*> mods(E);
  std::vector<SwiGluCache*> caches(E);
  std::vector<std::vector<float>*> gos(E), gis(E);
  for (int e = 0; e < E; ++e) {
    const int rows = L.caches[e].rows;
    scaled[e].resize((size_t)rows * d);
    for (int r = 0; r < rows; ++r) {
      const float gate = L.gates[L.expert_slots[e][r]];
      const float* up = grad_out + (size_t)L.expert_tokens[e][r] * d;
      float* dst = scaled[e].data() + (size_t)r * d;
      for (int c = 0; c < d; ++c) dst[c] = gate * up[c];
    }
    mods[e] = &L.experts[e]; caches[e] = &L.caches[e]; gos[e] = &scaled[e]; gis[e] = &contrib[e];
  }
  swiglu_backward_many(mods, caches, gos, gis, d, F);

  // :389-399 un-permute, experts ascending.
  for (int e = 0; e < E; ++e)
    for (int r = 0; r < L.caches[e].rows; ++r) {
      float* dst = grad_in + (size_t)L.expert_tokens[e][r] * d;
      const float* src = contrib[e].data() + (size_t)r * d;
      for (int c = 0; c < d; ++c) dst[c] += src[c];
    }

  // :404-415 gate gradients.
  std::vector<float> grad_gates((size_t)T * k, 0.f);
  for (int e = 0; e < E; ++e)
    for (int r = 0; r < L.caches[e].rows; ++r) {
      const float* g = grad_out + (size_t)L.expert_tokens[e][r] * d;
      const float* o = L.caches[e].output.data() + (size_t)r * d;
      float s = 0.f;
      for (int c = 0; c < d; ++c) s += g[c] * o[c];
      grad_gates[L.expert_slots[e][r]] = s;
    }

  // :420-443 top-k renormalisation backward.
  std::vector<float> gp((size_t)T * E, 0.f);
  for (int t = 0; t < T; ++t) {
    const int* sel = L.expert_of.data() + (size_t)t * k;
    if (sel[0] == UNROUTED) continue;
    const float* p = L.probs.data() + (size_t)t * E;
    float total = 0.f;
    for (int r = 0; r < k; ++r) total += p[sel[r]];
    if (total <= 0.f) continue;
    float weighted = 0.f;
    for (int r = 0; r < k; ++r) weighted += grad_gates[(size_t)t * k + r] * p[sel[r]];
    for (int r = 0; r < k; ++r)
      gp[(size_t)t * E + sel[r]] += grad_gates[(size_t)t * k + r] / total - weighted / (total * total);
  }

  // :445-457 load-balancing term (counts are constants).
  if (L.aux_w != 0.f && L.valid_tokens > 0) {
    const float scale = L.aux_w * (float)E / (float)L.valid_tokens;
    const float slots = (float)(L.valid_tokens * k);
    for (int e = 0; e < E; ++e) {
      const float load = (float)L.expert_tokens[e].size() / slots;
      for (int t = 0; t < T; ++t) {
        if (L.expert_of[(size_t)t * k] == UNROUTED) continue;
        gp[(size_t)t * E + e] += scale * load;
      }
    }
  }

  // :459-481 softmax backward and the z-loss.
  std::vector<float> gl((size_t)T * E, 0.f);
  for (int t = 0; t < T; ++t) {
    if (L.expert_of[(size_t)t * k] == UNROUTED) continue;
    const float* p = L.probs.data() + (size_t)t * E;
    const float* up = gp.data() + (size_t)t * E;
    float dot = 0.f;
    for (int e = 0; e < E; ++e) dot += p[e] * up[e];
    float* row = gl.data() + (size_t)t * E;
    for (int e = 0; e < E; ++e) row[e] = p[e] * (up[e] - dot);
    if (L.z_w != 0.f) {
      const float factor = 2.0f * L.z_w * L.lse[t] / (float)std::max(L.valid_tokens, 1);
      for (int e = 0; e < E; ++e) row[e] += factor * p[e];
    }
  }

  // :483-486 Router::backward: dW_r += gl^T x ; grad_in += gl W_r.
#pragma omp parallel for schedule(static)
  for (int n0 = 0; n0 < E; n0 += 4)
    gemm_tn_acc_rows(gl.data(), L.input.data(), L.router.grad.data(), T, n0, std::min(E, n0 + 4), d, E, d, d);
  std::vector<float> from_router((size_t)T * d, 0.f);
#pragma omp parallel for schedule(static)
  for (int m0 = 0; m0 < T; m0 += ROW_BLOCK)
    gemm_nn_rows(gl.data(), L.router.value.data(), from_router.data(), m0, std::min(T, m0 + ROW_BLOCK), E, d,
                 E, d, d);
  for (size_t i = 0; i < from_router.size(); ++i) grad_in[i] += from_router[i];
  return 0;
}

// Param::step with Optimizer::Adam (param.rs:562-589), every weight of the
// layer; `step` is the already-incremented global step.  Clears the gradients.
void orc_adam_step(void* h, float lr, float beta1, float beta2, float eps, float wd, int step, float scale) {
  struct Ctx { float lr, b1, b2, eps, wd, c1, c2, scale; } ctx{
      lr, beta1, beta2, eps, wd, 1.0f - std::pow(beta1, (float)step), 1.0f - std::pow(beta2, (float)step), scale};
  for_each_weight(*(Layer*)h, [](Weight& w, void* p) {
    const Ctx& c = *(const Ctx*)p;
    w.need_grad();
    w.need_moments();
    for (size_t i = 0; i < w.value.size(); ++i) {
      const float g = w.grad[i] * c.scale;
      w.m[i] = c.b1 * w.m[i] + (1.0f - c.b1) * g;
      w.v[i] = c.b2 * w.v[i] + (1.0f - c.b2) * g * g;
      const float m_hat = w.m[i] / c.c1;
      const float v_hat = w.v[i] / c.c2;
      w.value[i] -= c.lr * c.wd * w.value[i];
      w.value[i] -= c.lr * m_hat / (std::sqrt(v_hat) + c.eps);
      w.grad[i] = 0.f;
    }
  }, &ctx);
}

// Param::step with Optimizer::Sgd (param.rs:557-561) over one buffer: value -= learning_rate * grad * scale.
// Clears the gradients, as Param::step does at its end.
void orc_sgd_apply(float* value, float* grad, long long n, float lr, float scale) {
  for (long long i = 0; i < n; ++i) {
    value[i] -= lr * grad[i] * scale;
    grad[i] = 0.f;
  }
}

// Param::step with Optimizer::Lion (param.rs:590-613) over one buffer: the step is the sign of
// beta1 * m + (1 - beta1) * g taken from the moment as it was, then m = beta2 * m + (1 - beta2) * g;
// sign(0) = 0 (optimizers.rs:50-58).
void orc_lion_apply(float* value, float* grad, float* m, long long n, float lr, float beta1, float beta2, float wd, float scale) {
  for (long long i = 0; i < n; ++i) {
    const float g = grad[i] * scale;
    const float update = beta1 * m[i] + (1.0f - beta1) * g;
    m[i] = beta2 * m[i] + (1.0f - beta2) * g;
    const float sg = update > 0.f ? 1.0f : (update < 0.f ? -1.0f : 0.0f);
    value[i] -= lr * (sg + wd * value[i]);
    grad[i] = 0.f;
  }
}

void orc_sgd_step(void* h, float lr, float scale) {
  struct Ctx { float lr, scale; } ctx{lr, scale};
  for_each_weight(*(Layer*)h, [](Weight& w, void* p) {
    const Ctx& c = *(const Ctx*)p;
    w.need_grad();
    orc_sgd_apply(w.value.data(), w.grad.data(), (long long)w.value.size(), c.lr, c.scale);
  }, &ctx);
}

void orc_lion_step(void* h, float lr, float beta1, float beta2, float wd, float scale) {
  struct Ctx { float lr, b1, b2, wd, scale; } ctx{lr, beta1, beta2, wd, scale};
  for_each_weight(*(Layer*)h, [](Weight& w, void* p) {
    const Ctx& c = *(const Ctx*)p;
    w.need_grad();
    w.need_moments();
    orc_lion_apply(w.value.data(), w.grad.data(), w.m.data(), (long long)w.value.size(), c.lr, c.b1, c.b2, c.wd, c.scale);
  }, &ctx);
}

}  // extern "C"
