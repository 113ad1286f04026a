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

// grid = (rows, heads, splits).  q: [rows, ld_q] (head h at column h*D).  out: [rows, ld_o].
// ctx_len[row] : number of cached tokens this row attends to (0 -> zeros).
// bt_row[row]  : which row of block_tables holds its pages (null -> row itself).
// splits > 1   : the cache blocks of a (row, head) are divided among `splits` CTAs; each leaves its unnormalised sum,
//                maximum and denominator in `part`, and the one that arrives last (a ticket per (row, head) in
//                `counters`, all zero between launches) combines them.  With few heads per GPU (tensor parallelism)
//                one CTA per (row, head) leaves too few CTAs in flight to hide the latency of their three serial
//                phases, and the longest contexts set the duration (33 us instead of 18 for 256 rows x 4 heads).
// THREADS: 128, or 256 when the grid has few CTAs (few heads per GPU): a warp's blocks are a chain of memory round
// trips, and twice the warps halve the chain of the longest context.
template <class T, int D, int THREADS>
__global__ void __launch_bounds__(THREADS)
paged_attention_kernel(const T* __restrict__ q, long ld_q, T* __restrict__ kcache, T* __restrict__ vcache,
                       const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ ctx_len,
                       const int* __restrict__ bt_row, T* __restrict__ out, long ld_o, int heads, int kv_heads,
                       float scale, int k_off, int v_off, const int* __restrict__ append_slots,
                       const int* __restrict__ positions, float rope_base, int splits, float* __restrict__ part,
                       int* __restrict__ counters) {
  constexpr int LPT = D / 8;                  // lanes cooperating on one token (16-byte chunk each)
  constexpr int TPW = 32 / LPT;               // tokens per warp pass
  constexpr int PASSES = KV_BLOCK / TPW;      // passes per 16-token block
  constexpr int NW = THREADS / 32;
  extern __shared__ float smem[];             // scores[ctx rounded to 16] + reductions
  __shared__ float red[32];
  __shared__ float oacc[NW][D];
  __shared__ int s_bt[ATTN_MAX_CTX / KV_BLOCK];     // this CTA's page-table entries, fetched once

  pdl_wait();
  pdl_trigger();                 // the successor (a GEMM) may launch now: its set-up and weight prefetch run under this kernel
  const int row = blockIdx.x, head = blockIdx.y;
  const int L = min(ctx_len[row], ATTN_MAX_CTX);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  T* orow = out + long(row) * ld_o + head * D;
  if (L <= 0) {                               // every split of the row sees this; none takes a ticket
    if (blockIdx.z == 0)
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
  const int b_lo = splits > 1 ? int(long(nblk) * blockIdx.z / splits) : 0;           // this CTA's blocks [b_lo, b_hi)
  const int b_hi = splits > 1 ? int(long(nblk) * (blockIdx.z + 1) / splits) : nblk;
  const int sub = lane / LPT, chunk = lane % LPT;
  // The page-table entries of the CTA's blocks come in with one coalesced load: read inside the loops, each entry sat
  // in front of its K (and again its V) load as a second dependent memory round trip per block.
  for (int i = threadIdx.x; i < b_hi - b_lo; i += blockDim.x) s_bt[i] = bt[b_lo + i];
  __syncthreads();

  float qf[8];
  if (rope) rot8(q + long(row) * ld_q + head * D, chunk, qf);
  else unpack8<T>(*reinterpret_cast<const Vec8*>(q + long(row) * ld_q + head * D + chunk * 8), qf);
#pragma unroll
  for (int i = 0; i < 8; ++i) qf[i] *= scale;

  // ---- phase 1: scores
  float lmax = -INFINITY;
  // each warp keeps the loads of its next block in flight while it works on the current one (256 rows x 16 heads x
  // 64: 0.89 -> 0.91 of the copy bandwidth; 128 rows x 20 heads x 128 at context 320: 74.5 -> 71.3 us)
  constexpr bool PREFETCH = true;
  auto load_block = [&](const T* cache, int b, Vec8 (&dst)[PASSES]) {
    const T* base = cache + (long(s_bt[b - b_lo]) * kv_heads + kvh) * (KV_BLOCK * D);
#pragma unroll
    for (int p = 0; p < PASSES; ++p) dst[p] = *reinterpret_cast<const Vec8*>(base + (p * TPW + sub) * D + chunk * 8);
  };
  Vec8 kv[PASSES], kn[PREFETCH ? PASSES : 1];
  if (PREFETCH && b_lo + warp < b_hi) load_block(kcache, b_lo + warp, kv);
  for (int b = b_lo + warp; b < b_hi; b += NW) {
    if constexpr (PREFETCH) {
      if (b + NW < b_hi) load_block(kcache, b + NW, kn);
    } else {
      load_block(kcache, b, kv);
    }
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
      if (chunk == 0) smem[tok - b_lo * KV_BLOCK] = s;
      lmax = fmaxf(lmax, s);
    }
    if constexpr (PREFETCH) {
#pragma unroll
      for (int p = 0; p < PASSES; ++p) kv[p] = kn[p];
    }
  }
  const float m = block_max(lmax, red);
  // ---- phase 2: exponentials + sum
  float lsum = 0.f;
  const int Lpad = (b_hi - b_lo) * KV_BLOCK;
  for (int i = threadIdx.x; i < Lpad; i += blockDim.x) {
    const float e = b_lo * KV_BLOCK + i < L ? __expf(smem[i] - m) : 0.f;
    smem[i] = e;
    lsum += e;
  }
  const float denom = block_sum(lsum, red);     // contains the __syncthreads that publishes smem[]
  // ---- phase 3: P.V
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  Vec8 vv[PASSES], vn[PREFETCH ? PASSES : 1];
  if (PREFETCH && b_lo + warp < b_hi) load_block(vcache, b_lo + warp, vv);
  for (int b = b_lo + warp; b < b_hi; b += NW) {
    if constexpr (PREFETCH) {
      if (b + NW < b_hi) load_block(vcache, b + NW, vn);
    } else {
      load_block(vcache, b, vv);
    }
#pragma unroll
    for (int p = 0; p < PASSES; ++p) {
      float vf[8];
      unpack8<T>(vv[p], vf);
      const float pr = smem[(b - b_lo) * KV_BLOCK + p * TPW + sub];
      if (pr != 0.f) {          // slots past the row's length may hold anything, NaN patterns included
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += pr * vf[i];
      }
    }
    if constexpr (PREFETCH) {
#pragma unroll
      for (int p = 0; p < PASSES; ++p) vv[p] = vn[p];
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
  if (splits <= 1) {
    const float inv = 1.f / denom;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) s += oacc[w][i];
      orow[i] = Cvt<T>::from_f(s * inv);
    }
    return;
  }
  // ---- several CTAs per (row, head): leave the partial, take a ticket, the last one combines
  const long item = long(row) * heads + head;
  float* mine = part + (item * splits + blockIdx.z) * (D + 2);
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) s += oacc[w][i];
    mine[i] = s;
  }
  if (threadIdx.x == 0) {
    mine[D] = b_hi > b_lo ? m : -INFINITY;     // an empty split (fewer blocks than splits) weighs nothing
    mine[D + 1] = b_hi > b_lo ? denom : 0.f;
  }
  __threadfence();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(counters + item, 1);
    s_last = ticket == splits - 1;
    if (s_last) counters[item] = 0;            // every split of this item has arrived: ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* all = part + item * splits * (D + 2);
  float gm = -INFINITY;
  for (int z = 0; z < splits; ++z) gm = fmaxf(gm, __ldcg(all + z * (D + 2) + D));
  float gl = 0.f;
  for (int z = 0; z < splits; ++z) {
    const float mz = __ldcg(all + z * (D + 2) + D);
    if (mz > -INFINITY) gl += __ldcg(all + z * (D + 2) + D + 1) * __expf(mz - gm);
  }
  const float ginv = 1.f / gl;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float s = 0.f;
    for (int z = 0; z < splits; ++z) {
      const float mz = __ldcg(all + z * (D + 2) + D);
      if (mz > -INFINITY) s += __ldcg(all + z * (D + 2) + i) * __expf(mz - gm);
    }
    orow[i] = Cvt<T>::from_f(s * ginv);
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
// splits > 1: `splits` CTAs per (row, head); part: fp32 [rows * heads * splits * (head_dim + 2)] scratch, counters:
// int32 [rows * heads], zero before the first launch (the kernel leaves them zero).
extern "C" int ronn_paged_attention(const void* q, long ld_q, void* kcache, void* vcache,
                                    const int* block_tables, int max_blocks, const int* ctx_len, const int* bt_row,
                                    void* out, long ld_o, long rows, int heads, int kv_heads, int head_dim,
                                    int max_ctx, float scale, int dtype, int k_off, int v_off, const int* append_slots,
                                    const int* positions, float rope_base, int splits, float* part, int* counters,
                                    cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (max_ctx <= 0 || max_ctx > ATTN_MAX_CTX || heads % kv_heads || (ld_q & 7)) return -2;
  if (append_slots && ((k_off & 7) || (v_off & 7))) return -2;
  if (splits < 1 || splits > 16 || (splits > 1 && (part == nullptr || counters == nullptr))) return -2;
  const int padded = (max_ctx + KV_BLOCK - 1) / KV_BLOCK * KV_BLOCK;
  const size_t smem = size_t(padded) * sizeof(float);
  dim3 grid((unsigned)rows, (unsigned)heads, (unsigned)splits);
  // 256 threads at 64 registers fit four CTAs per SM: wide CTAs only while the whole grid is resident at that rate
  const bool wide = rows * heads * splits <= 4L * device_sm_count();
#define RONN_PA(T, D)                                                                                              \
  do {                                                                                                               \
    if (wide) RONN_PA_(T, D, 256);                                                                                   \
    else RONN_PA_(T, D, ATTN_THREADS);                                                                               \
  } while (0)
#define RONN_PA_(T, D, TH) launch(paged_attention_kernel<T, D, TH>, grid, dim3(TH), smem, stream, (const T*)q, ld_q, (T*)kcache, (T*)vcache, block_tables, max_blocks, ctx_len, bt_row, (T*)out, ld_o, heads, kv_heads, scale, k_off, v_off, append_slots, positions, rope_base, splits, part, counters)
  if (dtype == 0 && head_dim == 64) RONN_PA(__nv_bfloat16, 64);
  else if (dtype == 0 && head_dim == 128) RONN_PA(__nv_bfloat16, 128);
  else if (dtype == 1 && head_dim == 64) RONN_PA(__half, 64);
  else if (dtype == 1 && head_dim == 128) RONN_PA(__half, 128);
  else return -1;
#undef RONN_PA
#undef RONN_PA_
  return check_launch_attn();
}
