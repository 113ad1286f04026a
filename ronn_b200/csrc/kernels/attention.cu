// Paged-KV attention.
//
// KV cache layout (per layer, K and V separately):  [num_blocks, kv_heads, BLOCK(=16), head_dim]
// so the 16 tokens of one block for one head are one contiguous 2 KB (d=64) or 4 KB (d=128) run.
// (16-token blocks and the page table come from the KV-cache design
// docs/new/RONN-KV-Cache-Compression-Branch-Prompt.md:125-195; the math is the reference's
// softmax(QK^T/sqrt(d))V, crates/ronn-core/src/tensor.rs:640-709.)
//
//   ronn_kv_append        : split a fused QKV projection, optionally apply rotary embedding to Q (in
//                           place) and K, and scatter K/V of every new token into its cache slot
//   ronn_paged_attention  : one CTA per (query row, head).  A query row carries its own causal length
//                           and page-table row, so the same kernel serves decode (one row per sequence),
//                           chunked / ragged causal prefill (one row per prompt token, length = pos + 1)
//                           and dense encoder attention (every row of a sequence sees the whole sequence).
//                           Scores for the row are kept in shared memory (context <= MAX_CTX); K and V
//                           are streamed once with 16-byte loads, fp32 accumulation, online in two phases.
#include "common.cuh"

namespace ronn {

constexpr int KV_BLOCK = 16;
constexpr int ATTN_MAX_CTX = 4096;
constexpr int ATTN_THREADS = 128;

// qkv: [T, ld] with q at column 0 (heads*D), k at k_off, v at v_off.  positions may be null (no rotary).
template <class T, int D>
__global__ void kv_append_kernel(T* __restrict__ qkv, long ld, int k_off, int v_off, const int* __restrict__ slots,
                                 const int* __restrict__ positions, T* __restrict__ kcache, T* __restrict__ vcache,
                                 int heads, int kv_heads, float rope_base, int use_rope) {
  pdl_wait();
  pdl_trigger();
  const long t = blockIdx.x;
  const int slot = slots[t];
  T* row = qkv + t * ld;
  constexpr int CH = D / 8;           // 16-byte chunks per head
  constexpr int HALF = D / 2;
  const int pos = positions ? positions[t] : 0;
  // ---- rotary on q (in place) and k (registers) : pairs (i, i + D/2)
  if (use_rope) {
    const int total = (heads + kv_heads) * HALF;
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
      const int h = i / HALF, j = i - h * HALF;
      T* base = h < heads ? row + h * D : row + k_off + (h - heads) * D;
      const float inv = __powf(rope_base, -2.f * float(j) / float(D));
      float sn, cs;
      __sincosf(float(pos) * inv, &sn, &cs);
      const float a = Cvt<T>::to_f(base[j]), b = Cvt<T>::to_f(base[j + HALF]);
      base[j] = Cvt<T>::from_f(a * cs - b * sn);
      base[j + HALF] = Cvt<T>::from_f(b * cs + a * sn);
    }
    __syncthreads();
  }
  if (slot < 0) return;
  const int blk = slot / KV_BLOCK, off = slot % KV_BLOCK;
  for (int i = threadIdx.x; i < kv_heads * CH; i += blockDim.x) {
    const int h = i / CH, c = i - h * CH;
    const long dst = ((long(blk) * kv_heads + h) * KV_BLOCK + off) * D + c * 8;
    *reinterpret_cast<Vec8*>(kcache + dst) = *reinterpret_cast<const Vec8*>(row + k_off + h * D + c * 8);
    *reinterpret_cast<Vec8*>(vcache + dst) = *reinterpret_cast<const Vec8*>(row + v_off + h * D + c * 8);
  }
}

// grid = (rows, heads).  q: [rows, ld_q] (head h at column h*D).  out: [rows, ld_o].
// ctx_len[row] : number of cached tokens this row attends to (0 -> zeros).
// bt_row[row]  : which row of block_tables holds its pages (null -> row itself).
template <class T, int D>
__global__ void __launch_bounds__(ATTN_THREADS)
paged_attention_kernel(const T* __restrict__ q, long ld_q, T* __restrict__ kcache, T* __restrict__ vcache,
                       const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ ctx_len,
                       const int* __restrict__ bt_row, T* __restrict__ out, long ld_o, int heads, int kv_heads,
                       float scale, int k_off, int v_off, const int* __restrict__ append_slots,
                       const int* __restrict__ positions, float rope_base) {
  constexpr int LPT = D / 8;                  // lanes cooperating on one token (16-byte chunk each)
  constexpr int TPW = 32 / LPT;               // tokens per warp pass
  constexpr int PASSES = KV_BLOCK / TPW;      // passes per 16-token block
  constexpr int NW = ATTN_THREADS / 32;
  extern __shared__ float smem[];             // scores[ctx rounded to 16] + reductions
  __shared__ float red[32];
  __shared__ float oacc[NW][D];

  pdl_wait();
  pdl_trigger();                 // the successor (a GEMM) may launch now: its set-up and weight prefetch run under this kernel
  const int row = blockIdx.x, head = blockIdx.y;
  const int L = min(ctx_len[row], ATTN_MAX_CTX);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  T* orow = out + long(row) * ld_o + head * D;
  if (L <= 0) {
    for (int i = threadIdx.x; i < D; i += blockDim.x) orow[i] = Cvt<T>::from_f(0.f);
    return;
  }
  const int kvh = head / (heads / kv_heads);
  // Rotary embedding fused into the decode step (rope_base > 0): pairs (j, j + D/2) of the row's q and of its new k are
  // rotated by position x base^(-2j/D), rounded through the storage type as the stand-alone rotation stores them; the
  // q row in memory stays untouched.  `rot8` returns the rotated 16-byte chunk c of the head vector at `base`.
  const bool rope = rope_base > 0.f && positions != nullptr;
  const float pos = rope ? float(positions[row]) : 0.f;
  auto rot8 = [&](const T* base, int c, float (&o)[8]) {
    constexpr int HC = D / 16;                // chunks per half
    float own[8], oth[8];
    unpack8<T>(*reinterpret_cast<const Vec8*>(base + c * 8), own);
    unpack8<T>(*reinterpret_cast<const Vec8*>(base + (c < HC ? c + HC : c - HC) * 8), oth);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int j = (c < HC ? c : c - HC) * 8 + i;          // index inside the half
      const float inv = __powf(rope_base, -2.f * float(j) / float(D));
      float sn, cs;
      __sincosf(pos * inv, &sn, &cs);
      const float r = c < HC ? own[i] * cs - oth[i] * sn : own[i] * cs + oth[i] * sn;
      o[i] = Cvt<T>::to_f(Cvt<T>::from_f(r));
    }
  };
  if (append_slots != nullptr) {
    // decode with fused append: this row's new K/V (columns k_off / v_off of the fused QKV row) go to the row's
    // cache slot first; every CTA of a KV group writes the same bytes, and reads them back only after the barrier
    const int slot = append_slots[row];
    if (slot >= 0 && threadIdx.x < 2 * (D / 8)) {
      const int c = threadIdx.x % (D / 8);
      const bool is_v = threadIdx.x >= D / 8;
      const T* src = q + long(row) * ld_q + (is_v ? v_off : k_off) + kvh * D;
      T* dstc = is_v ? vcache : kcache;
      const long dst = ((long(slot / KV_BLOCK) * kv_heads + kvh) * KV_BLOCK + slot % KV_BLOCK) * D + c * 8;
      if (rope && !is_v) {
        float kr[8];
        rot8(src, c, kr);
        *reinterpret_cast<Vec8*>(dstc + dst) = pack8<T>(kr);
      } else {
        *reinterpret_cast<Vec8*>(dstc + dst) = *reinterpret_cast<const Vec8*>(src + c * 8);
      }
    }
    __syncthreads();
  }
  const int* bt = block_tables + long(bt_row ? bt_row[row] : row) * max_blocks;
  const int nblk = (L + KV_BLOCK - 1) / KV_BLOCK;
  const int sub = lane / LPT, chunk = lane % LPT;

  float qf[8];
  if (rope) rot8(q + long(row) * ld_q + head * D, chunk, qf);
  else unpack8<T>(*reinterpret_cast<const Vec8*>(q + long(row) * ld_q + head * D + chunk * 8), qf);
#pragma unroll
  for (int i = 0; i < 8; ++i) qf[i] *= scale;

  // ---- phase 1: scores
  float lmax = -INFINITY;
  for (int b = warp; b < nblk; b += NW) {
    const int pb = bt[b];
    const T* kb = kcache + (long(pb) * kv_heads + kvh) * (KV_BLOCK * D);
    Vec8 kv[PASSES];
#pragma unroll
    for (int p = 0; p < PASSES; ++p) kv[p] = *reinterpret_cast<const Vec8*>(kb + (p * TPW + sub) * D + chunk * 8);
#pragma unroll
    for (int p = 0; p < PASSES; ++p) {
      float kf[8];
      unpack8<T>(kv[p], kf);
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) s += qf[i] * kf[i];
#pragma unroll
      for (int o = LPT / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      const int tok = b * KV_BLOCK + p * TPW + sub;
      if (tok >= L) s = -INFINITY;
      if (chunk == 0) smem[tok] = s;
      lmax = fmaxf(lmax, s);
    }
  }
  const float m = block_max(lmax, red);
  // ---- phase 2: exponentials + sum
  float lsum = 0.f;
  const int Lpad = nblk * KV_BLOCK;
  for (int i = threadIdx.x; i < Lpad; i += blockDim.x) {
    const float e = i < L ? __expf(smem[i] - m) : 0.f;
    smem[i] = e;
    lsum += e;
  }
  const float denom = block_sum(lsum, red);     // contains the __syncthreads that publishes smem[]
  // ---- phase 3: P.V
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int b = warp; b < nblk; b += NW) {
    const int pb = bt[b];
    const T* vb = vcache + (long(pb) * kv_heads + kvh) * (KV_BLOCK * D);
    Vec8 vv[PASSES];
#pragma unroll
    for (int p = 0; p < PASSES; ++p) vv[p] = *reinterpret_cast<const Vec8*>(vb + (p * TPW + sub) * D + chunk * 8);
#pragma unroll
    for (int p = 0; p < PASSES; ++p) {
      float vf[8];
      unpack8<T>(vv[p], vf);
      const float pr = smem[b * KV_BLOCK + p * TPW + sub];
      if (pr != 0.f) {          // slots past the row's length may hold anything, NaN patterns included
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += pr * vf[i];
      }
    }
  }
  // reduce over the token sub-lanes of the warp, then over warps
#pragma unroll
  for (int o = LPT; o < 32; o <<= 1) {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
  }
  if (sub == 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) oacc[warp][chunk * 8 + i] = acc[i];
  }
  pdl_trigger();               // all K/V traffic of this CTA is done: the successor may start launching
  __syncthreads();
  const float inv = 1.f / denom;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) s += oacc[w][i];
    orow[i] = Cvt<T>::from_f(s * inv);
  }
}

}  // namespace ronn

using namespace ronn;

static inline int check_launch_attn() { return cudaGetLastError() == cudaSuccess ? 0 : -100; }

// dtype 0 bf16, 1 fp16; head_dim 64 or 128.
extern "C" int ronn_kv_append(void* qkv, long ld, int k_off, int v_off, const int* slots, const int* positions,
                              void* kcache, void* vcache, long tokens, int heads, int kv_heads, int head_dim,
                              float rope_base, int use_rope, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if ((ld & 7) || (k_off & 7) || (v_off & 7)) return -2;
#define RONN_KVA(T, D) launch(kv_append_kernel<T, D>, dim3(unsigned(tokens)), dim3(128), 0, stream, (T*)qkv, ld, k_off, v_off, slots, positions, (T*)kcache, (T*)vcache, heads, kv_heads, rope_base, use_rope)
  if (dtype == 0 && head_dim == 64) RONN_KVA(__nv_bfloat16, 64);
  else if (dtype == 0 && head_dim == 128) RONN_KVA(__nv_bfloat16, 128);
  else if (dtype == 1 && head_dim == 64) RONN_KVA(__half, 64);
  else if (dtype == 1 && head_dim == 128) RONN_KVA(__half, 128);
  else return -1;
#undef RONN_KVA
  return check_launch_attn();
}

// max_ctx: upper bound of ctx_len over the rows (sizes the score buffer); must be <= 4096.
// append_slots != null (decode, one row per sequence): the row's new K/V are taken from columns k_off / v_off of its q
// row and written to cache slot append_slots[row] by the same kernel before attending.  positions != null and
// rope_base > 0: rotary embedding of q and of the new k (pairs j, j + head_dim / 2) by the same kernel as well.
extern "C" int ronn_paged_attention(const void* q, long ld_q, void* kcache, void* vcache,
                                    const int* block_tables, int max_blocks, const int* ctx_len, const int* bt_row,
                                    void* out, long ld_o, long rows, int heads, int kv_heads, int head_dim,
                                    int max_ctx, float scale, int dtype, int k_off, int v_off, const int* append_slots,
                                    const int* positions, float rope_base, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (max_ctx <= 0 || max_ctx > ATTN_MAX_CTX || heads % kv_heads || (ld_q & 7)) return -2;
  if (append_slots && ((k_off & 7) || (v_off & 7))) return -2;
  const int padded = (max_ctx + KV_BLOCK - 1) / KV_BLOCK * KV_BLOCK;
  const size_t smem = size_t(padded) * sizeof(float);
  dim3 grid((unsigned)rows, (unsigned)heads);
#define RONN_PA(T, D) launch(paged_attention_kernel<T, D>, grid, dim3(ATTN_THREADS), smem, stream, (const T*)q, ld_q, (T*)kcache, (T*)vcache, block_tables, max_blocks, ctx_len, bt_row, (T*)out, ld_o, heads, kv_heads, scale, k_off, v_off, append_slots, positions, rope_base)
  if (dtype == 0 && head_dim == 64) RONN_PA(__nv_bfloat16, 64);
  else if (dtype == 0 && head_dim == 128) RONN_PA(__nv_bfloat16, 128);
  else if (dtype == 1 && head_dim == 64) RONN_PA(__half, 64);
  else if (dtype == 1 && head_dim == 128) RONN_PA(__half, 128);
  else return -1;
#undef RONN_PA
  return check_launch_attn();
}
