// Memory-bound kernels: LayerNorm / RMSNorm (optionally fused with a residual add), row softmax,
// activations, binary elementwise, embedding gather (+ position add), row argmax, casts.
//
// Numeric definitions follow the reference: LayerNorm over the last axis with population variance
// (crates/ronn-core/src/tensor.rs:566-611), max-shifted softmax (crates/ronn-core/src/ops/reduction.rs:432-450),
// tanh-form GELU and x*sigmoid(1.702x) "fast GELU" (crates/ronn-core/src/ops/arithmetic.rs:281-296,
// crates/ronn-providers/src/gpu/cuda_kernels.rs:537-562), embedding = gather on axis 0
// (crates/ronn-onnx/src/ops/tensor_ops.rs:463-489), argmax (crates/ronn-core/src/ops/reduction.rs:282-304).
// All kernels move 16 bytes per thread per access and keep a row in registers between passes.
#include <cstdlib>
#include <mutex>
#include <unordered_set>
#include "common.cuh"
#include "rowwise_stream.h"

namespace ronn {

constexpr int NORM_MAX_CHUNKS = 4;     // a thread keeps up to 4 x 8 values of its row

static int g_pdl = -1;
bool pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("RONN_PDL");
    g_pdl = (e && e[0] == '0') ? 0 : 1;
  }
  return g_pdl != 0;
}

void prefer_max_shared(const void* kern) {
  static std::mutex mu;
  static std::unordered_set<const void*> seen;
  static int enabled = -1;
  std::lock_guard<std::mutex> lock(mu);
  if (enabled < 0) {
    const char* e = getenv("RONN_MAX_SHARED_CARVEOUT");
    enabled = (e && e[0] == '1') ? 1 : 0;
  }
  if (enabled && seen.insert(kern).second) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) !=
        cudaSuccess)
      cudaGetLastError();                    // a preference only: never fail a launch over it
  }
}

// Threads per row of the row-wise kernels: as many 16-byte chunks per thread as the register budget allows when
// there are rows enough to fill the GPU, fewer (more warps per row) when the row count alone would leave most SMs
// with a warp or two, as in decode.
int norm_threads(long rows, int nchunk) {
  int per_thread = NORM_MAX_CHUNKS;
  auto warps_of = [&](int c) { return ((nchunk + c - 1) / c + 31) / 32; };
  while (per_thread > 1 && rows * warps_of(per_thread) < 2048 && warps_of(per_thread / 2) <= 32) per_thread /= 2;
  int threads = warps_of(per_thread) * 32;
  if (threads > 1024) threads = 1024;
  return threads;
}

// y = norm(x [+ res]) * gamma [+ beta];  if sum_out != null the pre-norm sum (x + res) is also written.
// RMS = true: y = v * rsqrt(mean(v^2) + eps) * gamma.
template <class T, bool RMS>
__global__ void norm_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ gamma,
                            const T* __restrict__ beta, T* __restrict__ y, T* __restrict__ sum_out, long rows,
                            int H, long ld_x, long ld_res, long ld_y, float eps) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  // Rows of up to 1024 values run one warp per row, blockDim.y rows per CTA, and reduce with shuffles only.
  const long row = long(blockIdx.x) * blockDim.y + threadIdx.y;
  if (row >= rows) return;                    // whole warps leave: blockDim.y > 1 only with blockDim.x == 32
  const bool one_warp = blockDim.x == 32;
  const T* xr = x + row * ld_x;
  const T* rr = res ? res + row * ld_res : nullptr;
  const int nchunk = H >> 3;
  float v[NORM_MAX_CHUNKS][8];
  Vec8 gp[NORM_MAX_CHUNKS], bp[NORM_MAX_CHUNKS];   // scale and shift, fetched before the reductions need the row
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunk) {
      if (gamma) gp[c] = *reinterpret_cast<const Vec8*>(gamma + ch * 8);
      if (beta) bp[c] = *reinterpret_cast<const Vec8*>(beta + ch * 8);
      unpack8<T>(*reinterpret_cast<const Vec8*>(xr + ch * 8), v[c]);
      if (rr) {
        float r[8];
        unpack8<T>(*reinterpret_cast<const Vec8*>(rr + ch * 8), r);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[c][i] += r[i];
      }
      if (sum_out) *reinterpret_cast<Vec8*>(sum_out + row * ld_y + ch * 8) = pack8<T>(v[c]);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += RMS ? v[c][i] * v[c][i] : v[c][i];
    }
  }
  float mean = 0.f, inv;
  if (RMS) {
    const float ms = (one_warp ? warp_sum(s) : block_sum(s, scratch)) / float(H);
    inv = rsqrtf(ms + eps);
  } else {
    mean = (one_warp ? warp_sum(s) : block_sum(s, scratch)) / float(H);
    float q = 0.f;
#pragma unroll
    for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
      const int ch = threadIdx.x + c * blockDim.x;
      if (ch < nchunk) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float d = v[c][i] - mean;
          q += d * d;
        }
      }
    }
    const float var = (one_warp ? warp_sum(q) : block_sum(q, scratch)) / float(H);
    inv = rsqrtf(var + eps);
  }
#pragma unroll
  for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunk) {
      float g[8], b[8], o[8];
      if (gamma) unpack8<T>(gp[c], g);
      if (beta) unpack8<T>(bp[c], b);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float t = (v[c][i] - mean) * inv;
        if (gamma) t *= g[i];
        if (beta) t += b[i];
        o[i] = t;
      }
      *reinterpret_cast<Vec8*>(y + row * ld_y + ch * 8) = pack8<T>(o);
    }
  }
}

// Split-K finalize: v = sum_s ws[s][row][:] + bias + residual; optional activation; writes v as `sum_out`
// and, when NORM != 0, norm(v) * gamma (+ beta) as `y`.  NORM: 0 none, 1 LayerNorm, 2 RMSNorm.
// ws: [S, rows, N] fp32.  N % 8 == 0, N <= 8 * NORM_MAX_CHUNKS * blockDim.x.
template <class T, int NORM>
__global__ void splitk_finalize_kernel(const float* __restrict__ ws, int S, const T* __restrict__ bias,
                                       const T* __restrict__ residual, T* __restrict__ sum_out,
                                       const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ y,
                                       long rows, int N, float eps, int act) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const long row = blockIdx.x;
  const int nchunk = N >> 3;
  const long slice = rows * long(N);
  float v[NORM_MAX_CHUNKS][8];
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunk) {
      const float* p = ws + row * N + ch * 8;
      float4 a0 = *reinterpret_cast<const float4*>(p), a1 = *reinterpret_cast<const float4*>(p + 4);
      for (int k = 1; k < S; ++k) {
        const float4 b0 = *reinterpret_cast<const float4*>(p + k * slice);
        const float4 b1 = *reinterpret_cast<const float4*>(p + k * slice + 4);
        a0.x += b0.x; a0.y += b0.y; a0.z += b0.z; a0.w += b0.w;
        a1.x += b1.x; a1.y += b1.y; a1.z += b1.z; a1.w += b1.w;
      }
      v[c][0] = a0.x; v[c][1] = a0.y; v[c][2] = a0.z; v[c][3] = a0.w;
      v[c][4] = a1.x; v[c][5] = a1.y; v[c][6] = a1.z; v[c][7] = a1.w;
      if (bias) {
        float b[8];
        unpack8<T>(*reinterpret_cast<const Vec8*>(bias + ch * 8), b);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[c][i] += b[i];
      }
      if (act == 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[c][i] = fmaxf(v[c][i], 0.f);
      } else if (act == 2) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[c][i] = gelu_tanh_f(v[c][i]);
      }
      if (residual) {
        float r[8];
        unpack8<T>(*reinterpret_cast<const Vec8*>(residual + row * N + ch * 8), r);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[c][i] += r[i];
      }
      if (act == 3) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[c][i] = fmaxf(v[c][i], 0.f);
      }
      if (sum_out) {
        const Vec8 pk = pack8<T>(v[c]);
        *reinterpret_cast<Vec8*>(sum_out + row * N + ch * 8) = pk;
        if (NORM != 0) unpack8<T>(pk, v[c]);      // normalise exactly what the residual stream stores
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) s += NORM == 2 ? v[c][i] * v[c][i] : v[c][i];
    }
  }
  if (NORM == 0) return;
  float mean = 0.f, inv;
  if (NORM == 2) {
    inv = rsqrtf(block_sum(s, scratch) / float(N) + eps);
  } else {
    mean = block_sum(s, scratch) / float(N);
    float q = 0.f;
#pragma unroll
    for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
      const int ch = threadIdx.x + c * blockDim.x;
      if (ch < nchunk) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float d = v[c][i] - mean;
          q += d * d;
        }
      }
    }
    inv = rsqrtf(block_sum(q, scratch) / float(N) + eps);
  }
#pragma unroll
  for (int c = 0; c < NORM_MAX_CHUNKS; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunk) {
      float g[8], b[8], o[8];
      if (gamma) unpack8<T>(*reinterpret_cast<const Vec8*>(gamma + ch * 8), g);
      if (beta) unpack8<T>(*reinterpret_cast<const Vec8*>(beta + ch * 8), b);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float t = (v[c][i] - mean) * inv;
        if (gamma) t *= g[i];
        if (beta) t += b[i];
        o[i] = t;
      }
      *reinterpret_cast<Vec8*>(y + row * N + ch * 8) = pack8<T>(o);
    }
  }
}

// Row softmax over the last dimension of [rows, cols]; any cols (scalar accesses when cols % 8 != 0).
template <class T>
__global__ void softmax_kernel(const T* __restrict__ x, T* __restrict__ y, int cols) {
  __shared__ float scratch[32];
  const T* xr = x + long(blockIdx.x) * cols;
  T* yr = y + long(blockIdx.x) * cols;
  float m = -INFINITY;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) m = fmaxf(m, Cvt<T>::to_f(xr[i]));
  m = block_max(m, scratch);
  float s = 0.f;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) s += __expf(Cvt<T>::to_f(xr[i]) - m);
  s = block_sum(s, scratch);
  const float inv = 1.f / s;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) yr[i] = Cvt<T>::from_f(__expf(Cvt<T>::to_f(xr[i]) - m) * inv);
}

// op: 0 relu, 1 gelu(tanh), 2 fast gelu, 3 sigmoid, 4 silu, 5 tanh
__device__ __forceinline__ float act_apply(float x, int op) {
  switch (op) {
    case 0: return fmaxf(x, 0.f);
    case 1: return gelu_tanh_f(x);
    case 2: return x / (1.f + __expf(-1.702f * x));
    case 3: return 1.f / (1.f + __expf(-x));
    case 4: return x / (1.f + __expf(-x));
    default: {
      const float e = __expf(2.f * x);
      return 1.f - 2.f / (e + 1.f);
    }
  }
}

// The element-wise kernels are grid-stride loops over 16-byte chunks, four chunks per thread and turn with the loads
// issued together: one resident wave of CTAs then keeps about 128 KB per SM in flight, which a DRAM stream needs.
template <class T>
__global__ void unary_kernel(const T* __restrict__ x, T* __restrict__ y, long n, int op) {
  const long n8 = n >> 3;
  const long stride = long(gridDim.x) * blockDim.x;
  const Vec8* xv = reinterpret_cast<const Vec8*>(x);
  Vec8* yv = reinterpret_cast<Vec8*>(y);
  long i = blockIdx.x * long(blockDim.x) + threadIdx.x;
  for (; i + 3 * stride < n8; i += 4 * stride) {
    Vec8 in[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) in[u] = xv[i + u * stride];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float f[8];
      unpack8<T>(in[u], f);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] = act_apply(f[k], op);
      yv[i + u * stride] = pack8<T>(f);
    }
  }
  for (; i < n8; i += stride) {
    float f[8];
    unpack8<T>(xv[i], f);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = act_apply(f[k], op);
    yv[i] = pack8<T>(f);
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
    const long j = (n8 << 3) + threadIdx.x;
    y[j] = Cvt<T>::from_f(act_apply(Cvt<T>::to_f(x[j]), op));
  }
}

// op: 0 add, 1 mul, 2 sub, 3 swiglu (silu(a) * b), 4 add+relu
template <class T>
__global__ void binary_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y, long n, int op) {
  const long n8 = n >> 3;
  const long stride = long(gridDim.x) * blockDim.x;
  const Vec8* av = reinterpret_cast<const Vec8*>(a);
  const Vec8* bv = reinterpret_cast<const Vec8*>(b);
  Vec8* yv = reinterpret_cast<Vec8*>(y);
  auto combine = [op](const Vec8& pa, const Vec8& pb) {
    float fa[8], fb[8];
    unpack8<T>(pa, fa);
    unpack8<T>(pb, fb);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float r;
      switch (op) {
        case 0: r = fa[k] + fb[k]; break;
        case 1: r = fa[k] * fb[k]; break;
        case 2: r = fa[k] - fb[k]; break;
        case 3: r = fa[k] / (1.f + __expf(-fa[k])) * fb[k]; break;
        default: r = fmaxf(fa[k] + fb[k], 0.f); break;
      }
      fa[k] = r;
    }
    return pack8<T>(fa);
  };
  long i = blockIdx.x * long(blockDim.x) + threadIdx.x;
  for (; i + 3 * stride < n8; i += 4 * stride) {
    Vec8 pa[4], pb[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      pa[u] = av[i + u * stride];
      pb[u] = bv[i + u * stride];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) yv[i + u * stride] = combine(pa[u], pb[u]);
  }
  for (; i < n8; i += stride) yv[i] = combine(av[i], bv[i]);
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
    const long i = (n8 << 3) + threadIdx.x;
    const float fa = Cvt<T>::to_f(a[i]), fb = Cvt<T>::to_f(b[i]);
    float r = op == 0 ? fa + fb : op == 1 ? fa * fb : op == 2 ? fa - fb
              : op == 3 ? fa / (1.f + __expf(-fa)) * fb : fmaxf(fa + fb, 0.f);
    y[i] = Cvt<T>::from_f(r);
  }
}

// SwiGLU on a fused [rows, 2*F] gate|up projection: y[r, f] = silu(x[r, f]) * x[r, F + f]
template <class T>
__global__ void swiglu_fused_kernel(const T* __restrict__ x, T* __restrict__ y, int F, long rows) {
  pdl_wait();
  pdl_trigger();
  const int f8 = F >> 3;
  const long total = rows * f8;
  const long stride = long(gridDim.x) * blockDim.x;
  auto gate_at = [&](long i) {
    const long r = i / f8;
    return x + r * 2 * F + (i - r * f8) * 8;
  };
  auto apply = [](const Vec8& pg, const Vec8& pu) {
    float g[8], u[8];
    unpack8<T>(pg, g);
    unpack8<T>(pu, u);
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] = g[k] / (1.f + __expf(-g[k])) * u[k];
    return pack8<T>(g);
  };
  long i = blockIdx.x * long(blockDim.x) + threadIdx.x;
  for (; i + 3 * stride < total; i += 4 * stride) {
    Vec8 pg[4], pu[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const T* g = gate_at(i + k * stride);
      pg[k] = *reinterpret_cast<const Vec8*>(g);
      pu[k] = *reinterpret_cast<const Vec8*>(g + F);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) reinterpret_cast<Vec8*>(y)[i + k * stride] = apply(pg[k], pu[k]);
  }
  for (; i < total; i += stride) {
    const T* g = gate_at(i);
    reinterpret_cast<Vec8*>(y)[i] = apply(*reinterpret_cast<const Vec8*>(g), *reinterpret_cast<const Vec8*>(g + F));
  }
}

// out[t, :] = table[ids[t], :] (+ pos_table[pos[t], :]).  H % 8 == 0.  Out-of-range ids produce zeros.
template <class T>
__global__ void embedding_kernel(const int* __restrict__ ids, const int* __restrict__ pos, const T* __restrict__ table,
                                 const T* __restrict__ pos_table, T* __restrict__ out, int H, int vocab, int max_pos,
                                 long ld_out) {
  pdl_wait();
  pdl_trigger();
  const long t = blockIdx.x;
  const int id = ids[t];
  const int p = pos ? pos[t] : 0;
  const bool ok = id >= 0 && id < vocab;
  const bool pok = pos_table && p >= 0 && p < max_pos;
  for (int ch = threadIdx.x; ch < (H >> 3); ch += blockDim.x) {
    float f[8];
    if (ok) unpack8<T>(*reinterpret_cast<const Vec8*>(table + long(id) * H + ch * 8), f);
    else {
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = 0.f;
    }
    if (pok) {
      float g[8];
      unpack8<T>(*reinterpret_cast<const Vec8*>(pos_table + long(p) * H + ch * 8), g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] += g[i];
    }
    *reinterpret_cast<Vec8*>(out + t * ld_out + ch * 8) = pack8<T>(f);
  }
}

// Row argmax with lowest-index tie break.  Writes idx_out[row] (+ col_offset) and optionally max_out[row].
template <class T>
__global__ void argmax_kernel(const T* __restrict__ x, int* __restrict__ idx_out, float* __restrict__ max_out, int cols,
                              long ld, int col_offset) {
  __shared__ float smax[32];
  __shared__ int sidx[32];
  pdl_wait();
  pdl_trigger();
  const T* xr = x + long(blockIdx.x) * ld;
  float m = -INFINITY;
  int mi = 0x7fffffff;
  // a thread visits its elements in increasing index order, so "strictly greater" already keeps the lowest index
  auto take = [&](float v, int i) {
    if (v > m) { m = v; mi = i; }
  };
  // Rows may start at any element (odd vocabulary sizes): scalar accesses up to the first 16-byte boundary, 16-byte
  // loads (two in flight per thread) for the body, scalar accesses for what is left.
  constexpr bool VEC = sizeof(T) == 2;
  int head = VEC ? int(((16u - unsigned(reinterpret_cast<uintptr_t>(xr) & 15u)) & 15u) / sizeof(T)) : 0;
  if (head > cols) head = cols;
  const int nvec = VEC ? (cols - head) >> 3 : 0;
  if (int(threadIdx.x) < head) take(Cvt<T>::to_f(xr[threadIdx.x]), threadIdx.x);
  if constexpr (VEC) {
  const Vec8* xv = reinterpret_cast<const Vec8*>(xr + head);
  int c = threadIdx.x;
  const int bd = int(blockDim.x);
  for (; c + bd < nvec; c += 2 * bd) {
    const Vec8 p0 = xv[c], p1 = xv[c + bd];
    float f0[8], f1[8];
    unpack8<T>(p0, f0);
    unpack8<T>(p1, f1);
#pragma unroll
    for (int k = 0; k < 8; ++k) take(f0[k], head + c * 8 + k);
#pragma unroll
    for (int k = 0; k < 8; ++k) take(f1[k], head + (c + bd) * 8 + k);
  }
  for (; c < nvec; c += blockDim.x) {
    float f[8];
    unpack8<T>(xv[c], f);
#pragma unroll
    for (int k = 0; k < 8; ++k) take(f[k], head + c * 8 + k);
  }
  }
  int done = head + nvec * 8;
  if constexpr (sizeof(T) == 4) {
    // fp32 rows (logits): the same scheme with 16-byte loads of four values
    int head4 = int(((16u - unsigned(reinterpret_cast<uintptr_t>(xr) & 15u)) & 15u) / 4u);
    if (head4 > cols) head4 = cols;
    const int nvec4 = (cols - head4) >> 2;
    if (int(threadIdx.x) < head4) take(xr[threadIdx.x], threadIdx.x);
    const float4* xv4 = reinterpret_cast<const float4*>(xr + head4);
    int c = threadIdx.x;
    for (; c + int(blockDim.x) < nvec4; c += 2 * blockDim.x) {
      const float4 p0 = xv4[c], p1 = xv4[c + blockDim.x];
      const int i0 = head4 + c * 4, i1 = head4 + (c + int(blockDim.x)) * 4;
      take(p0.x, i0); take(p0.y, i0 + 1); take(p0.z, i0 + 2); take(p0.w, i0 + 3);
      take(p1.x, i1); take(p1.y, i1 + 1); take(p1.z, i1 + 2); take(p1.w, i1 + 3);
    }
    for (; c < nvec4; c += blockDim.x) {
      const float4 p0 = xv4[c];
      const int i0 = head4 + c * 4;
      take(p0.x, i0); take(p0.y, i0 + 1); take(p0.z, i0 + 2); take(p0.w, i0 + 3);
    }
    done = head4 + nvec4 * 4;
  }
  for (int i = done + threadIdx.x; i < cols; i += blockDim.x) take(Cvt<T>::to_f(xr[i]), i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
    if (om > m || (om == m && oi < mi)) { m = om; mi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) { smax[warp] = m; sidx[warp] = mi; }
  __syncthreads();
  if (warp == 0) {
    m = lane < nw ? smax[lane] : -INFINITY;
    mi = lane < nw ? sidx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
      if (om > m || (om == m && oi < mi)) { m = om; mi = oi; }
    }
    if (lane == 0) {
      if (mi == 0x7fffffff) mi = 0;                        // nothing compared greater than -inf (a row of -inf or NaN)
      idx_out[blockIdx.x] = mi + col_offset;
      if (max_out) max_out[blockIdx.x] = m;
    }
  }
}

// Combine per-shard (max, idx) pairs: vals/idx are [shards, rows]; picks the largest value, lowest index on ties.
__global__ void argmax_combine_kernel(const float* __restrict__ vals, const int* __restrict__ idx, int* __restrict__ out,
                                      int shards, int rows) {
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float m = -INFINITY;
  int mi = 0x7fffffff;
  for (int s = 0; s < shards; ++s) {
    const float v = vals[s * rows + r];
    const int i = idx[s * rows + r];
    if (v > m || (v == m && i < mi)) { m = v; mi = i; }
  }
  out[r] = mi;
}

template <class TI, class TO>
__global__ void cast_kernel(const TI* __restrict__ x, TO* __restrict__ y, long n) {
  const long stride = long(gridDim.x) * blockDim.x;
  long i = blockIdx.x * long(blockDim.x) + threadIdx.x;
  for (; i + 7 * stride < n; i += 8 * stride) {
    TI in[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) in[u] = x[i + u * stride];
#pragma unroll
    for (int u = 0; u < 8; ++u) y[i + u * stride] = Cvt<TO>::from_f(Cvt<TI>::to_f(in[u]));
  }
  for (; i < n; i += stride) y[i] = Cvt<TO>::from_f(Cvt<TI>::to_f(x[i]));
}

// 16-bit <-> fp32 in 8-element chunks (16-byte access on the 16-bit side, two on the fp32 side), four chunks per
// thread and turn; both pointers 16-byte aligned.  The last n % 8 elements are converted one by one.
template <class T16, bool WIDEN>
__global__ void cast_vec_kernel(const void* __restrict__ xin, void* __restrict__ yout, long n) {
  const long n8 = n >> 3;
  const long stride = long(gridDim.x) * blockDim.x;
  long i = blockIdx.x * long(blockDim.x) + threadIdx.x;
  if (WIDEN) {
    const Vec8* x = static_cast<const Vec8*>(xin);
    float4* y = static_cast<float4*>(yout);
    auto put = [&](long j, const Vec8& p) {
      float f[8];
      unpack8<T16>(p, f);
      y[2 * j] = make_float4(f[0], f[1], f[2], f[3]);
      y[2 * j + 1] = make_float4(f[4], f[5], f[6], f[7]);
    };
    for (; i + 3 * stride < n8; i += 4 * stride) {
      Vec8 in[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) in[u] = x[i + u * stride];
#pragma unroll
      for (int u = 0; u < 4; ++u) put(i + u * stride, in[u]);
    }
    for (; i < n8; i += stride) put(i, x[i]);
    if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
      const long j = (n8 << 3) + threadIdx.x;
      static_cast<float*>(yout)[j] = Cvt<T16>::to_f(static_cast<const T16*>(xin)[j]);
    }
  } else {
    const float4* x = static_cast<const float4*>(xin);
    Vec8* y = static_cast<Vec8*>(yout);
    auto put = [&](long j, const float4& a, const float4& b) {
      const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
      y[j] = pack8<T16>(f);
    };
    for (; i + 3 * stride < n8; i += 4 * stride) {
      float4 a[4], b[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        a[u] = x[2 * (i + u * stride)];
        b[u] = x[2 * (i + u * stride) + 1];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) put(i + u * stride, a[u], b[u]);
    }
    for (; i < n8; i += stride) put(i, x[2 * i], x[2 * i + 1]);
    if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
      const long j = (n8 << 3) + threadIdx.x;
      static_cast<T16*>(yout)[j] = Cvt<T16>::from_f(static_cast<const float*>(xin)[j]);
    }
  }
}

static inline int grid_for(long work, int threads, int cap = 148 * 8) {
  long g = (work + threads - 1) / threads;
  if (g < 1) g = 1;
  return int(g > cap ? cap : g);
}

}  // namespace ronn

using namespace ronn;

#define RONN_BY_DTYPE(dtype, ...)                           \
  do {                                                      \
    if ((dtype) == 0) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else if ((dtype) == 1) { using T = __half; __VA_ARGS__; }   \
    else return -1;                                         \
  } while (0)

static inline int check_launch() { return cudaGetLastError() == cudaSuccess ? 0 : -100; }

// dtype: 0 bf16, 1 fp16.  rms: 0 LayerNorm, 1 RMSNorm.  H % 8 == 0 and H <= 32768.
extern "C" int ronn_norm(const void* x, const void* res, const void* gamma, const void* beta, void* y, void* sum_out,
                         long rows, int H, long ld_x, long ld_res, long ld_y, float eps, int rms, int dtype,
                         cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((H & 7) || H > 1024 * 8 * NORM_MAX_CHUNKS || (ld_x & 7) || (ld_y & 7) || (res && (ld_res & 7))) return -2;
  {
    const int rc = rowwise_stream_try(rms ? 1 : 0, x, res, gamma, beta, y, sum_out, nullptr, rows, H, ld_x, ld_res, ld_y,
                                      eps, dtype, stream);
    if (rc != 0) return rc < 0 ? rc : check_launch();
  }
  const int threads = norm_threads(rows, H >> 3);
  const int rows_per_cta = (threads == 32 && rows >= 4096) ? 4 : 1;
  const dim3 grid(unsigned((rows + rows_per_cta - 1) / rows_per_cta)), block(threads, rows_per_cta);
  RONN_BY_DTYPE(dtype, {
    if (rms) launch(norm_kernel<T, true>, grid, block, 0, stream, (const T*)x, (const T*)res, (const T*)gamma,
                    (const T*)beta, (T*)y, (T*)sum_out, rows, H, ld_x, ld_res, ld_y, eps);
    else launch(norm_kernel<T, false>, grid, block, 0, stream, (const T*)x, (const T*)res, (const T*)gamma,
                (const T*)beta, (T*)y, (T*)sum_out, rows, H, ld_x, ld_res, ld_y, eps);
  });
  return check_launch();
}

// Softmax over an axis that is not the last one, on the tensor as it lies in memory: [outer, n, inner] with the
// reduction over n.  One thread per (outer, inner) column: neighbouring threads read neighbouring addresses at every
// step of the walk over n, so the loads coalesce without a transpose.  Two walks: running maximum and sum (online),
// then the normalised values.
template <class T>
__global__ void softmax_strided_kernel(const T* __restrict__ x, T* __restrict__ y, long outer, int n, long inner) {
  pdl_wait();
  pdl_trigger();
  const long total = outer * inner;
  for (long col = blockIdx.x * long(blockDim.x) + threadIdx.x; col < total; col += long(gridDim.x) * blockDim.x) {
    const long o = col / inner, in = col - o * inner;
    const T* p = x + o * n * inner + in;
    T* q = y + o * n * inner + in;
    float m = -INFINITY, s = 0.f;
    for (int k = 0; k < n; ++k) {
      const float v = Cvt<T>::to_f(p[long(k) * inner]);
      const float nm = fmaxf(m, v);
      s = s * __expf(m - nm) + __expf(v - nm);
      m = nm;
    }
    const float inv = 1.f / s;
    for (int k = 0; k < n; ++k) q[long(k) * inner] = Cvt<T>::from_f(__expf(Cvt<T>::to_f(p[long(k) * inner]) - m) * inv);
  }
}

// x, y: contiguous [outer, n, inner]; softmax over n.  dtype: 0 bf16, 1 fp16, 2 fp32.
extern "C" int ronn_softmax_strided(const void* x, void* y, long outer, int n, long inner, int dtype, cudaStream_t stream) {
  if (outer <= 0 || n <= 0 || inner <= 0) return 0;
  const long total = outer * inner;
  const int grid = int((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
  if (dtype == 2) launch(softmax_strided_kernel<float>, dim3(grid), dim3(256), 0, stream, (const float*)x, (float*)y, outer, n, inner);
  else RONN_BY_DTYPE(dtype, launch(softmax_strided_kernel<T>, dim3(grid), dim3(256), 0, stream, (const T*)x, (T*)y, outer, n, inner));
  return check_launch();
}

// dtype: 0 bf16, 1 fp16, 2 fp32
extern "C" int ronn_softmax(const void* x, void* y, long rows, int cols, int dtype, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  {
    const int rc = rowwise_stream_try(2, x, nullptr, nullptr, nullptr, y, nullptr, nullptr, rows, cols, cols, 0, cols, 0.f,
                                      dtype, stream);
    if (rc != 0) return rc < 0 ? rc : check_launch();
  }
  int threads = cols >= 1024 ? 256 : (cols >= 256 ? 128 : 64);
  if (dtype == 2) softmax_kernel<float><<<unsigned(rows), threads, 0, stream>>>((const float*)x, (float*)y, cols);
  else RONN_BY_DTYPE(dtype, (softmax_kernel<T><<<unsigned(rows), threads, 0, stream>>>((const T*)x, (T*)y, cols)));
  return check_launch();
}

extern "C" int ronn_unary(const void* x, void* y, long n, int op, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) return -2;
  RONN_BY_DTYPE(dtype, (unary_kernel<T><<<grid_for(n >> 3, 256), 256, 0, stream>>>((const T*)x, (T*)y, n, op)));
  return check_launch();
}

extern "C" int ronn_binary(const void* a, const void* b, void* y, long n, int op, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(y)) & 15) return -2;
  RONN_BY_DTYPE(dtype, (binary_kernel<T><<<grid_for(n >> 3, 256), 256, 0, stream>>>((const T*)a, (const T*)b, (T*)y, n, op)));
  return check_launch();
}

extern "C" int ronn_swiglu_fused(const void* x, void* y, long rows, int F, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (F & 7) return -2;
  RONN_BY_DTYPE(dtype, launch(swiglu_fused_kernel<T>, dim3(grid_for(rows * (F >> 3), 256)), dim3(256), 0, stream, (const T*)x, (T*)y, F, rows));
  return check_launch();
}

extern "C" int ronn_embedding(const int* ids, const int* pos, const void* table, const void* pos_table, void* out,
                              long tokens, int H, int vocab, int max_pos, long ld_out, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if ((H & 7) || (ld_out & 7)) return -2;
  int threads = (H >> 3) >= 128 ? 128 : 64;
  RONN_BY_DTYPE(dtype, launch(embedding_kernel<T>, dim3(unsigned(tokens)), dim3(threads), 0, stream, ids, pos, (const T*)table,
                                     (const T*)pos_table, (T*)out, H, vocab, max_pos, ld_out));
  return check_launch();
}

// dtype: 0 bf16, 1 fp16, 2 fp32
extern "C" int ronn_argmax(const void* x, int* idx_out, float* max_out, long rows, int cols, long ld, int col_offset,
                           int dtype, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  const int threads = cols >= 8192 ? 1024 : 256;
  if (dtype == 2) launch(argmax_kernel<float>, dim3(unsigned(rows)), dim3(threads), 0, stream, (const float*)x, idx_out, max_out, cols, ld, col_offset);
  else RONN_BY_DTYPE(dtype, launch(argmax_kernel<T>, dim3(unsigned(rows)), dim3(threads), 0, stream, (const T*)x, idx_out, max_out, cols, ld, col_offset));
  return check_launch();
}

extern "C" int ronn_argmax_combine(const float* vals, const int* idx, int* out, int shards, int rows,
                                   cudaStream_t stream) {
  if (rows <= 0) return 0;
  launch(argmax_combine_kernel, dim3((rows + 127) / 128), dim3(128), 0, stream, vals, idx, out, shards, rows);
  return check_launch();
}

// from/to: 0 bf16, 1 fp16, 2 fp32
extern "C" int ronn_cast(const void* x, void* y, long n, int from, int to, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((from == 2) != (to == 2) && n >= 8 &&
      !((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15)) {
    const int gv = grid_for(n >> 3, 256);
    const int h = from == 2 ? to : from;
    if (h == 0 && to == 2) cast_vec_kernel<__nv_bfloat16, true><<<gv, 256, 0, stream>>>(x, y, n);
    else if (h == 1 && to == 2) cast_vec_kernel<__half, true><<<gv, 256, 0, stream>>>(x, y, n);
    else if (h == 0) cast_vec_kernel<__nv_bfloat16, false><<<gv, 256, 0, stream>>>(x, y, n);
    else cast_vec_kernel<__half, false><<<gv, 256, 0, stream>>>(x, y, n);
    return check_launch();
  }
  const int g = grid_for(n, 256);
#define RONN_CAST(FI, TI, FO, TO) \
  if (from == FI && to == FO) { cast_kernel<TI, TO><<<g, 256, 0, stream>>>((const TI*)x, (TO*)y, n); return check_launch(); }
  RONN_CAST(0, __nv_bfloat16, 2, float)
  RONN_CAST(1, __half, 2, float)
  RONN_CAST(2, float, 0, __nv_bfloat16)
  RONN_CAST(2, float, 1, __half)
  RONN_CAST(0, __nv_bfloat16, 1, __half)
  RONN_CAST(1, __half, 0, __nv_bfloat16)
#undef RONN_CAST
  return -1;
}

// norm: 0 none (sum_out only), 1 LayerNorm, 2 RMSNorm.  act: 0 none, 1 relu, 2 gelu (applied before the residual),
// 3 relu applied after the residual.
extern "C" int ronn_splitk_finalize(const float* ws, int S, const void* bias, const void* residual, void* sum_out,
                                    const void* gamma, const void* beta, void* y, long rows, int N, float eps,
                                    int act, int norm, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((N & 7) || N > 1024 * 8 * NORM_MAX_CHUNKS || S < 1) return -2;
  const int threads = norm_threads(rows, N >> 3);
#define RONN_FIN(NORM_) launch(splitk_finalize_kernel<T, NORM_>, dim3(unsigned(rows)), dim3(threads), 0, stream, ws, S, (const T*)bias, (const T*)residual, (T*)sum_out, (const T*)gamma, (const T*)beta, (T*)y, rows, N, eps, act)
  RONN_BY_DTYPE(dtype, {
    if (norm == 0) RONN_FIN(0);
    else if (norm == 1) RONN_FIN(1);
    else RONN_FIN(2);
  });
#undef RONN_FIN
  return check_launch();
}

// 1 enables, 0 disables programmatic dependent launch for every kernel of the library.
extern "C" void ronn_set_pdl(int on) { ronn::g_pdl = on ? 1 : 0; }
