// BitNet host kernels: quantisers, packers and exact integer matmul oracles.
//
// Numeric contracts follow the reference quantiser
// (crates/ronn-providers/src/bitnet/quantization.rs:41-64 binary: bit = x >= 0,
// LSB-first, 8 per byte, scale = mean|x|; :67-109,131-153 ternary: threshold
// 0.7*mean|x|, codes 00=-1 01=0 10=+1, four per byte LSB-first, scale = mean of
// |x| above the threshold) and kernels (bitnet/kernels.rs:74-131 XNOR+popcount,
// :134-178 ternary integer dot).  The b1.58 "absmean" weight quantiser and the
// per-token int8 activation quantiser used by the GPU decode path are added here
// as the CPU oracle of those device kernels.
#include <cmath>
#include <cstdint>
#include <cstring>

extern "C" {

// ---------------------------------------------------------------- binary
// packed must hold ceil(n/8) bytes.  Returns the scale mean|x|.
float ronn_bitnet_quantize_binary(const float* x, int64_t n, uint8_t* packed) {
  double s = 0.0;
  memset(packed, 0, size_t((n + 7) / 8));
  for (int64_t i = 0; i < n; ++i) {
    s += std::fabs(double(x[i]));
    if (x[i] >= 0.f) packed[i >> 3] |= uint8_t(1u << (i & 7));
  }
  return n ? float(s / double(n)) : 0.f;
}

void ronn_bitnet_dequantize_binary(const uint8_t* packed, int64_t n, float scale, float* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = ((packed[i >> 3] >> (i & 7)) & 1) ? scale : -scale;
}

// C[M,N] = scale_a*scale_b * sum_k a_ik*b_kj with a,b in {-1,+1}.
// a_bits: row-major [M, K] bits (row stride ceil(K/8) bytes); bt_bits: B transposed, [N, K] bits.
void ronn_bitnet_binary_matmul(const uint8_t* a_bits, const uint8_t* bt_bits, float* C, int64_t M, int64_t N,
                               int64_t K, float scale_a, float scale_b) {
  int64_t stride = (K + 7) / 8;
  for (int64_t i = 0; i < M; ++i) {
    const uint8_t* a = a_bits + i * stride;
    for (int64_t j = 0; j < N; ++j) {
      const uint8_t* b = bt_bits + j * stride;
      int64_t agree = 0;
      int64_t full = K / 64;
      for (int64_t w = 0; w < full; ++w) {
        uint64_t x, y;
        memcpy(&x, a + w * 8, 8);
        memcpy(&y, b + w * 8, 8);
        agree += __builtin_popcountll(~(x ^ y));
      }
      for (int64_t k = full * 64; k < K; ++k) {
        int xa = (a[k >> 3] >> (k & 7)) & 1, xb = (b[k >> 3] >> (k & 7)) & 1;
        agree += (xa == xb);
      }
      C[i * N + j] = float(2 * agree - K) * scale_a * scale_b;
    }
  }
}

// ---------------------------------------------------------------- ternary
static inline uint8_t tern_code(int v) { return v < 0 ? 0u : (v == 0 ? 1u : 2u); }
static inline int tern_value(uint8_t c) { return c == 0 ? -1 : (c == 2 ? 1 : 0); }

// Reference threshold form.  packed holds ceil(n/4) bytes.  Returns scale; *threshold_out = 0.7*mean|x|.
float ronn_bitnet_quantize_ternary(const float* x, int64_t n, uint8_t* packed, float* threshold_out) {
  double s = 0.0;
  for (int64_t i = 0; i < n; ++i) s += std::fabs(double(x[i]));
  float thr = n ? float(0.7 * s / double(n)) : 0.f;
  memset(packed, 0, size_t((n + 3) / 4));
  double above = 0.0;
  int64_t cnt = 0;
  for (int64_t i = 0; i < n; ++i) {
    float a = std::fabs(x[i]);
    int v = 0;
    if (a > thr) { v = x[i] > 0.f ? 1 : -1; above += a; ++cnt; }
    packed[i >> 2] |= uint8_t(tern_code(v) << (2 * (i & 3)));
  }
  if (threshold_out) *threshold_out = thr;
  return cnt ? float(above / double(cnt)) : 1.f;
}

// b1.58 absmean form: scale = mean|x|, q = clip(round(x/scale), -1, 1).
float ronn_bitnet_quantize_absmean(const float* x, int64_t n, uint8_t* packed) {
  double s = 0.0;
  for (int64_t i = 0; i < n; ++i) s += std::fabs(double(x[i]));
  float scale = n ? float(s / double(n)) : 1.f;
  if (scale < 1e-8f) scale = 1e-8f;
  memset(packed, 0, size_t((n + 3) / 4));
  for (int64_t i = 0; i < n; ++i) {
    float q = std::nearbyint(x[i] / scale);
    int v = q > 1.f ? 1 : (q < -1.f ? -1 : int(q));
    packed[i >> 2] |= uint8_t(tern_code(v) << (2 * (i & 3)));
  }
  return scale;
}

// Pack explicit ternary values (int8 in {-1,0,1}) row by row; each row is padded to a whole byte.
void ronn_bitnet_pack_ternary_rows(const int8_t* v, int64_t rows, int64_t cols, uint8_t* packed) {
  int64_t stride = (cols + 3) / 4;
  memset(packed, 0, size_t(rows * stride));
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c)
      packed[r * stride + (c >> 2)] |= uint8_t(tern_code(v[r * cols + c]) << (2 * (c & 3)));
}

void ronn_bitnet_unpack_ternary(const uint8_t* packed, int64_t n, int8_t* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = int8_t(tern_value((packed[i >> 2] >> (2 * (i & 3))) & 3));
}

void ronn_bitnet_dequantize_ternary(const uint8_t* packed, int64_t n, float scale, float* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = float(tern_value((packed[i >> 2] >> (2 * (i & 3))) & 3)) * scale;
}

// Ternary x ternary: a [M,K] packed rows, bt [N,K] packed rows (B transposed).
void ronn_bitnet_ternary_matmul(const uint8_t* a, const uint8_t* bt, float* C, int64_t M, int64_t N, int64_t K,
                                float scale_a, float scale_b) {
  int64_t stride = (K + 3) / 4;
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      int64_t acc = 0;
      const uint8_t* ra = a + i * stride;
      const uint8_t* rb = bt + j * stride;
      for (int64_t k = 0; k < K; ++k)
        acc += tern_value((ra[k >> 2] >> (2 * (k & 3))) & 3) * tern_value((rb[k >> 2] >> (2 * (k & 3))) & 3);
      C[i * N + j] = float(acc) * scale_a * scale_b;
    }
}

// Per-row (token) absmax int8 quantisation: q = round(x * 127 / max|x|), scale_out = max|x| / 127.
void ronn_bitnet_quantize_act_int8(const float* x, int64_t rows, int64_t cols, int8_t* q, float* scale_out) {
  for (int64_t r = 0; r < rows; ++r) {
    float m = 0.f;
    for (int64_t c = 0; c < cols; ++c) m = std::fmax(m, std::fabs(x[r * cols + c]));
    if (m < 1e-5f) m = 1e-5f;
    float inv = 127.f / m;
    for (int64_t c = 0; c < cols; ++c) {
      float v = std::nearbyint(x[r * cols + c] * inv);
      v = v > 127.f ? 127.f : (v < -127.f ? -127.f : v);
      q[r * cols + c] = int8_t(v);
    }
    scale_out[r] = m / 127.f;
  }
}

// Y[M,N] = (sum_k Xq[m,k] * W[n,k]) * x_scale[m] * w_scale.  W is [N,K] 2-bit packed rows; exact int32 accumulate.
// acc_out (optional) receives the raw integer sums.
void ronn_bitnet_ternary_int8_matmul(const int8_t* xq, const float* x_scale, const uint8_t* w_packed, float w_scale,
                                     float* Y, int32_t* acc_out, int64_t M, int64_t N, int64_t K) {
  int64_t stride = (K + 3) / 4;
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      int32_t acc = 0;
      const uint8_t* w = w_packed + n * stride;
      const int8_t* x = xq + m * K;
      for (int64_t k = 0; k < K; ++k) acc += int32_t(x[k]) * tern_value((w[k >> 2] >> (2 * (k & 3))) & 3);
      if (acc_out) acc_out[m * N + n] = acc;
      Y[m * N + n] = float(acc) * x_scale[m] * w_scale;
    }
}

}  // extern "C"
