// CPU provider kernels with runtime ISA dispatch (AVX-512F / AVX2+FMA / scalar).
//
// Counterpart of the reference's SIMD helpers (crates/ronn-core/src/simd.rs:10-334:
// feature detection, dot/add/relu) and CPU provider kernels
// (crates/ronn-providers/src/cpu/simd.rs:10-388, whose "AVX2-FMA matmul" is a scalar
// triple loop).  Here the GEMM really is vectorised, and the fused forms the
// reference only names (AddRelu, MatMulAdd: cpu/kernels.rs:20-31) exist.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <immintrin.h>

namespace {

int g_level = -1;  // 0 scalar, 1 avx2+fma, 2 avx512f

int detect() {
  if (g_level >= 0) return g_level;
  int lvl = 0;
  __builtin_cpu_init();
  if (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma")) lvl = 1;
  if (lvl == 1 && __builtin_cpu_supports("avx512f")) lvl = 2;
  g_level = lvl;
  return lvl;
}

int g_forced = -1;
int level() { return g_forced >= 0 ? (g_forced < detect() ? g_forced : detect()) : detect(); }

// ------------------------------------------------------------------ dot
float dot_scalar(const float* a, const float* b, int64_t n) {
  float s = 0.f;
  for (int64_t i = 0; i < n; ++i) s += a[i] * b[i];
  return s;
}
__attribute__((target("avx2,fma"))) float dot_avx2(const float* a, const float* b, int64_t n) {
  __m256 acc0 = _mm256_setzero_ps(), acc1 = _mm256_setzero_ps();
  int64_t i = 0;
  for (; i + 16 <= n; i += 16) {
    acc0 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i), acc0);
    acc1 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i + 8), _mm256_loadu_ps(b + i + 8), acc1);
  }
  acc0 = _mm256_add_ps(acc0, acc1);
  float tmp[8];
  _mm256_storeu_ps(tmp, acc0);
  float s = tmp[0] + tmp[1] + tmp[2] + tmp[3] + tmp[4] + tmp[5] + tmp[6] + tmp[7];
  for (; i < n; ++i) s += a[i] * b[i];
  return s;
}
__attribute__((target("avx512f"))) float dot_avx512(const float* a, const float* b, int64_t n) {
  __m512 acc = _mm512_setzero_ps();
  int64_t i = 0;
  for (; i + 16 <= n; i += 16) acc = _mm512_fmadd_ps(_mm512_loadu_ps(a + i), _mm512_loadu_ps(b + i), acc);
  float s = _mm512_reduce_add_ps(acc);
  for (; i < n; ++i) s += a[i] * b[i];
  return s;
}

// ------------------------------------------------------------------ elementwise
enum BinOp { ADD = 0, MUL = 1, SUB = 2 };

template <int OP>
void binary_scalar(const float* a, const float* b, float* o, int64_t n, bool relu) {
  for (int64_t i = 0; i < n; ++i) {
    float v = OP == ADD ? a[i] + b[i] : (OP == MUL ? a[i] * b[i] : a[i] - b[i]);
    o[i] = relu ? (v > 0.f ? v : 0.f) : v;
  }
}
template <int OP>
__attribute__((target("avx2,fma"))) void binary_avx2(const float* a, const float* b, float* o, int64_t n, bool relu) {
  const __m256 z = _mm256_setzero_ps();
  int64_t i = 0;
  for (; i + 8 <= n; i += 8) {
    __m256 x = _mm256_loadu_ps(a + i), y = _mm256_loadu_ps(b + i);
    __m256 v = OP == ADD ? _mm256_add_ps(x, y) : (OP == MUL ? _mm256_mul_ps(x, y) : _mm256_sub_ps(x, y));
    if (relu) v = _mm256_max_ps(v, z);
    _mm256_storeu_ps(o + i, v);
  }
  binary_scalar<OP>(a + i, b + i, o + i, n - i, relu);
}

void relu_scalar(const float* a, float* o, int64_t n) {
  for (int64_t i = 0; i < n; ++i) o[i] = a[i] > 0.f ? a[i] : 0.f;
}
__attribute__((target("avx2"))) void relu_avx2(const float* a, float* o, int64_t n) {
  const __m256 z = _mm256_setzero_ps();
  int64_t i = 0;
  for (; i + 8 <= n; i += 8) _mm256_storeu_ps(o + i, _mm256_max_ps(_mm256_loadu_ps(a + i), z));
  relu_scalar(a + i, o + i, n - i);
}

// ------------------------------------------------------------------ GEMM: C[M,N] = act(A[M,K] * B[K,N] + bias[N])
void gemm_scalar(const float* A, const float* B, const float* bias, float* C, int64_t M, int64_t N, int64_t K,
                 int act) {
  for (int64_t i = 0; i < M; ++i) {
    float* c = C + i * N;
    for (int64_t j = 0; j < N; ++j) c[j] = bias ? bias[j] : 0.f;
    for (int64_t k = 0; k < K; ++k) {
      float a = A[i * K + k];
      const float* b = B + k * N;
      for (int64_t j = 0; j < N; ++j) c[j] += a * b[j];
    }
    if (act == 1)
      for (int64_t j = 0; j < N; ++j) c[j] = c[j] > 0.f ? c[j] : 0.f;
  }
}

// Register-blocked: 4 rows x 16 columns of C held in 8 ymm accumulators.
__attribute__((target("avx2,fma"))) void gemm_avx2(const float* A, const float* B, const float* bias, float* C,
                                                   int64_t M, int64_t N, int64_t K, int act) {
  const __m256 z = _mm256_setzero_ps();
  int64_t j = 0;
  for (; j + 16 <= N; j += 16) {
    __m256 b0 = bias ? _mm256_loadu_ps(bias + j) : z;
    __m256 b1 = bias ? _mm256_loadu_ps(bias + j + 8) : z;
    int64_t i = 0;
    for (; i + 4 <= M; i += 4) {
      __m256 c00 = b0, c01 = b1, c10 = b0, c11 = b1, c20 = b0, c21 = b1, c30 = b0, c31 = b1;
      const float* a0 = A + i * K;
      for (int64_t k = 0; k < K; ++k) {
        __m256 v0 = _mm256_loadu_ps(B + k * N + j), v1 = _mm256_loadu_ps(B + k * N + j + 8);
        __m256 x0 = _mm256_broadcast_ss(a0 + k), x1 = _mm256_broadcast_ss(a0 + K + k);
        __m256 x2 = _mm256_broadcast_ss(a0 + 2 * K + k), x3 = _mm256_broadcast_ss(a0 + 3 * K + k);
        c00 = _mm256_fmadd_ps(x0, v0, c00); c01 = _mm256_fmadd_ps(x0, v1, c01);
        c10 = _mm256_fmadd_ps(x1, v0, c10); c11 = _mm256_fmadd_ps(x1, v1, c11);
        c20 = _mm256_fmadd_ps(x2, v0, c20); c21 = _mm256_fmadd_ps(x2, v1, c21);
        c30 = _mm256_fmadd_ps(x3, v0, c30); c31 = _mm256_fmadd_ps(x3, v1, c31);
      }
      if (act == 1) {
        c00 = _mm256_max_ps(c00, z); c01 = _mm256_max_ps(c01, z); c10 = _mm256_max_ps(c10, z); c11 = _mm256_max_ps(c11, z);
        c20 = _mm256_max_ps(c20, z); c21 = _mm256_max_ps(c21, z); c30 = _mm256_max_ps(c30, z); c31 = _mm256_max_ps(c31, z);
      }
      _mm256_storeu_ps(C + i * N + j, c00); _mm256_storeu_ps(C + i * N + j + 8, c01);
      _mm256_storeu_ps(C + (i + 1) * N + j, c10); _mm256_storeu_ps(C + (i + 1) * N + j + 8, c11);
      _mm256_storeu_ps(C + (i + 2) * N + j, c20); _mm256_storeu_ps(C + (i + 2) * N + j + 8, c21);
      _mm256_storeu_ps(C + (i + 3) * N + j, c30); _mm256_storeu_ps(C + (i + 3) * N + j + 8, c31);
    }
    for (; i < M; ++i) {
      __m256 c0 = b0, c1 = b1;
      const float* a0 = A + i * K;
      for (int64_t k = 0; k < K; ++k) {
        __m256 x = _mm256_broadcast_ss(a0 + k);
        c0 = _mm256_fmadd_ps(x, _mm256_loadu_ps(B + k * N + j), c0);
        c1 = _mm256_fmadd_ps(x, _mm256_loadu_ps(B + k * N + j + 8), c1);
      }
      if (act == 1) { c0 = _mm256_max_ps(c0, z); c1 = _mm256_max_ps(c1, z); }
      _mm256_storeu_ps(C + i * N + j, c0);
      _mm256_storeu_ps(C + i * N + j + 8, c1);
    }
  }
  if (j < N) {   // column tail
    for (int64_t i = 0; i < M; ++i)
      for (int64_t jj = j; jj < N; ++jj) {
        float s = bias ? bias[jj] : 0.f;
        for (int64_t k = 0; k < K; ++k) s += A[i * K + k] * B[k * N + jj];
        C[i * N + jj] = act == 1 ? (s > 0.f ? s : 0.f) : s;
      }
  }
}

// Batch-1 path: y[j0..N) = act(a[K] * B[K, j0..N) + bias).  k is the outer loop, so B streams through the cache once
// in row order while up to 128 output columns stay in registers.
__attribute__((target("avx2,fma"))) void gemv_avx2(const float* a, const float* B, const float* bias, float* y,
                                                   int64_t j0, int64_t N, int64_t K, int act) {
  const __m256 z = _mm256_setzero_ps();
  int64_t j = j0;
  for (; j + 64 <= N; j += 64) {
    __m256 c[8];
    for (int v = 0; v < 8; ++v) c[v] = bias ? _mm256_loadu_ps(bias + j + 8 * v) : z;
    for (int64_t k = 0; k < K; ++k) {
      const __m256 x = _mm256_broadcast_ss(a + k);
      const float* b = B + k * N + j;
      for (int v = 0; v < 8; ++v) c[v] = _mm256_fmadd_ps(x, _mm256_loadu_ps(b + 8 * v), c[v]);
    }
    for (int v = 0; v < 8; ++v) _mm256_storeu_ps(y + j + 8 * v, act == 1 ? _mm256_max_ps(c[v], z) : c[v]);
  }
  for (; j + 8 <= N; j += 8) {
    __m256 c = bias ? _mm256_loadu_ps(bias + j) : z;
    for (int64_t k = 0; k < K; ++k) c = _mm256_fmadd_ps(_mm256_broadcast_ss(a + k), _mm256_loadu_ps(B + k * N + j), c);
    _mm256_storeu_ps(y + j, act == 1 ? _mm256_max_ps(c, z) : c);
  }
  for (; j < N; ++j) {
    float s = bias ? bias[j] : 0.f;
    for (int64_t k = 0; k < K; ++k) s += a[k] * B[k * N + j];
    y[j] = act == 1 ? (s > 0.f ? s : 0.f) : s;
  }
}

__attribute__((target("avx512f,avx2,fma"))) void gemv_avx512(const float* a, const float* B, const float* bias, float* y,
                                                             int64_t N, int64_t K, int act) {
  const __m512 z = _mm512_setzero_ps();
  int64_t j = 0;
  for (; j + 128 <= N; j += 128) {
    __m512 c[8];
    for (int v = 0; v < 8; ++v) c[v] = bias ? _mm512_loadu_ps(bias + j + 16 * v) : z;
    for (int64_t k = 0; k < K; ++k) {
      const __m512 x = _mm512_set1_ps(a[k]);
      const float* b = B + k * N + j;
      for (int v = 0; v < 8; ++v) c[v] = _mm512_fmadd_ps(x, _mm512_loadu_ps(b + 16 * v), c[v]);
    }
    for (int v = 0; v < 8; ++v) _mm512_storeu_ps(y + j + 16 * v, act == 1 ? _mm512_max_ps(c[v], z) : c[v]);
  }
  if (j < N) gemv_avx2(a, B, bias, y, j, N, K, act);
}

}  // namespace

extern "C" {

// 0 scalar, 1 AVX2+FMA, 2 AVX-512F
int32_t ronn_cpu_simd_level() { return detect(); }
// Cap the ISA level used by the kernels (-1 restores auto-detection).
void ronn_cpu_force_level(int32_t lvl) { g_forced = lvl; }

float ronn_cpu_dot_f32(const float* a, const float* b, int64_t n) {
  int l = level();
  if (l >= 2) return dot_avx512(a, b, n);
  if (l >= 1) return dot_avx2(a, b, n);
  return dot_scalar(a, b, n);
}

// op: 0 add, 1 mul, 2 sub; relu != 0 fuses max(., 0)
void ronn_cpu_binary_f32(const float* a, const float* b, float* o, int64_t n, int32_t op, int32_t relu) {
  bool r = relu != 0;
  if (level() >= 1) {
    if (op == ADD) binary_avx2<ADD>(a, b, o, n, r);
    else if (op == MUL) binary_avx2<MUL>(a, b, o, n, r);
    else binary_avx2<SUB>(a, b, o, n, r);
  } else {
    if (op == ADD) binary_scalar<ADD>(a, b, o, n, r);
    else if (op == MUL) binary_scalar<MUL>(a, b, o, n, r);
    else binary_scalar<SUB>(a, b, o, n, r);
  }
}

void ronn_cpu_relu_f32(const float* a, float* o, int64_t n) {
  if (level() >= 1) relu_avx2(a, o, n);
  else relu_scalar(a, o, n);
}

// act: 0 none, 1 relu.  bias may be null.  Row-major, B is [K,N].
void ronn_cpu_gemm_f32(const float* A, const float* B, const float* bias, float* C, int64_t M, int64_t N, int64_t K,
                       int32_t act) {
  const int l = level();
  if (M == 1 && l >= 2) gemv_avx512(A, B, bias, C, N, K, act);
  else if (M == 1 && l >= 1) gemv_avx2(A, B, bias, C, 0, N, K, act);
  else if (l >= 1) gemm_avx2(A, B, bias, C, M, N, K, act);
  else gemm_scalar(A, B, bias, C, M, N, K, act);
}

// Row-wise max-shifted softmax over the last dimension.
void ronn_cpu_softmax_f32(const float* x, float* o, int64_t rows, int64_t cols) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* xi = x + r * cols;
    float* oi = o + r * cols;
    float m = xi[0];
    for (int64_t j = 1; j < cols; ++j) m = xi[j] > m ? xi[j] : m;
    float s = 0.f;
    for (int64_t j = 0; j < cols; ++j) { oi[j] = std::exp(xi[j] - m); s += oi[j]; }
    float inv = 1.f / s;
    for (int64_t j = 0; j < cols; ++j) oi[j] *= inv;
  }
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------
// Whole-chain execution: a linear sequence of dense layers (+ReLU) and a final softmax runs in one native call,
// ping-ponging between two scratch buffers.  This is what a batch-1 MLP session executes: per-node dispatch in
// the host language costs more than the arithmetic.
//   kinds[i]: 0 = GEMM (+bias, act in acts[i]), 1 = ReLU, 2 = softmax over the last dimension
//   weights[i] / biases[i]: row-major [K_i, N_i] / [N_i] (null for non-GEMM ops); dims[i] = N_i
// x: [M, K0]; out: [M, N_last]; scratch: two buffers of M * max(N_i) floats.
extern "C" void ronn_cpu_run_chain(const float* x, int64_t M, int64_t K0, int32_t n_ops, const int32_t* kinds,
                                   const float* const* weights, const float* const* biases, const int32_t* acts,
                                   const int64_t* dims, float* out, float* scratch0, float* scratch1) {
  const float* cur = x;
  int64_t cols = K0;
  for (int32_t i = 0; i < n_ops; ++i) {
    float* dst = (i == n_ops - 1) ? out : ((i & 1) ? scratch1 : scratch0);
    if (kinds[i] == 0) {
      ronn_cpu_gemm_f32(cur, weights[i], biases[i], dst, M, dims[i], cols, acts[i]);
      cols = dims[i];
    } else if (kinds[i] == 1) {
      ronn_cpu_relu_f32(cur, dst, M * cols);
    } else {
      ronn_cpu_softmax_f32(cur, dst, M, cols);
    }
    cur = dst;
  }
}
