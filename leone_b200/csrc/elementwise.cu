// Row-wise kernels: embedding gather, RMSNorm, SwiGLU, the fused per-head
// q/k RMSNorm + rotary + paged cache write, and sampling.  All take float32 or
// bfloat16 storage; every reduction and every softmax/rotation is in fp32 (the
// sampling sums in fp64, like the reference's host sampler).
#include "common.cuh"

namespace leone {

// ---------------------------------------------------------------------------
// Embedding gather: out[t,:] = table[id_t,:]  (crates/leone/src/cpu.rs:1243-1265;
// CUDA counterpart crates/leone-cuda/cuda/ie_cuda.cu:3569).  Output is the fp32
// residual stream.  An id outside [0, vocab) sets the status word and zeroes the row.
// `scale` multiplies every element (1 for the reference's models, which have no embedding
// multiplier; a product with 1 is exact).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ out, int hidden, int vocab, float scale, int* status) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const int id = ids[row];
  float* dst = out + (size_t)row * hidden;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) set_status(status, kBadTokenId, row, id);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = 0.f;
    return;
  }
  const T* src = table + (size_t)id * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = to_float<T>(src[c]) * scale;
}

// ---------------------------------------------------------------------------
// Logit post-processing for an output head that has one: l <- l * scale, then (cap > 0)
// l <- cap * tanh(l / cap).  The reference's models have neither (no logit scale, soft-cap or
// bias: crates/leone/src/runtime.rs:7442-7452); the head part skips this kernel for them.
// ---------------------------------------------------------------------------
__global__ void logit_post_kernel(float* __restrict__ logits, long long n, float scale, float cap) {
  pdl_trigger();
  pdl_wait();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float v = logits[i] * scale;
    if (cap > 0.f) v = cap * tanhf(v / cap);
    logits[i] = v;
  }
}

// ---------------------------------------------------------------------------
// RMSNorm: y = x * w * rsqrt(mean(x^2) + eps)  (crates/leone/src/cpu.rs:1642-1663;
// crates/leone-cuda/cuda/ie_cuda.cu:2357-2380).  Input rows are fp32 (the residual
// stream); `rows` optionally gathers input rows.  One block per output row.
// ---------------------------------------------------------------------------
template <typename TW, typename TO>
__global__ void rms_norm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                const TW* __restrict__ w, TO* __restrict__ out, int hidden,
                                float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const float* src = x + (size_t)(rows ? rows[r] : r) * hidden;
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float v = src[c];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  TO* dst = out + (size_t)r * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x)
    dst[c] = from_float<TO>(src[c] * to_float<TW>(w[c]) * inv);
}

// The same, for rows of 4*k elements up to 8192: each thread keeps its part of the row in
// registers (float4 loads), so the row is read once.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
  }
};

constexpr int kNormThreads = 256;
constexpr int kNormItems = 8;          // float4 per thread: rows up to 256 * 8 * 4 = 8192 elements

template <typename TW, typename TO>
__global__ void __launch_bounds__(kNormThreads)
rms_norm_vec_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                    const TW* __restrict__ w, TO* __restrict__ out, int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const float* src = x + (size_t)(rows ? rows[r] : r) * hidden;
  const int vecs = hidden >> 2;
  float4 v[kNormItems];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kNormItems; ++i) {
    const int c = threadIdx.x + i * kNormThreads;
    if (c < vecs) {
      v[i] = Vec4<float>::load(src + 4 * c);
      ss = fmaf(v[i].x, v[i].x, ss);
      ss = fmaf(v[i].y, v[i].y, ss);
      ss = fmaf(v[i].z, v[i].z, ss);
      ss = fmaf(v[i].w, v[i].w, ss);
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  TO* dst = out + (size_t)r * hidden;
#pragma unroll
  for (int i = 0; i < kNormItems; ++i) {
    const int c = threadIdx.x + i * kNormThreads;
    if (c < vecs) {
      const float4 g = Vec4<TW>::load(w + 4 * c);
      Vec4<TO>::store(dst + 4 * c, make_float4(v[i].x * g.x * inv, v[i].y * g.y * inv,
                                               v[i].z * g.z * inv, v[i].w * g.w * inv));
    }
  }
}

// ---------------------------------------------------------------------------
// SwiGLU on stacked [gate | up] rows: out = gate / (1 + exp(-gate)) * up
// (crates/leone/src/cpu.rs:903-905; ie_cuda.cu:2864-2874).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int n, int inter) {
  const size_t total = (size_t)n * inter;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / inter, col = i - row * inter;
    const float g = to_float<T>(gate_up[row * 2 * inter + col]);
    const float u = to_float<T>(gate_up[row * 2 * inter + inter + col]);
    out[i] = from_float<T>(g / (1.f + expf(-g)) * u);
  }
}

// ---------------------------------------------------------------------------
// Per-head q/k RMSNorm + rotary + paged cache write, one warp per
// (token, head) of the fused qkv row [q heads | k heads | v heads]
// (crates/leone-cuda/cuda/ie_cuda.cu:2426-2484 does the same three things in one
// launch; formulas crates/leone/src/cpu.rs:802-820 and 1747-1779).  Pair i of a head is
// elements (i, i + rotary_dim/2), or with `adjacent` elements (2i, 2i + 1)
// (crates/leone/src/backend.rs:1216-1222, crates/leone/src/cpu.rs:1767-1770).
//  q heads: normed, rotated, written back in place.
//  k heads: normed, rotated, written back in place and into the key page.
//  v heads: copied into the value page.
// Page of token t: block_table[seq_of_token[t]][pos / page_tokens]; a missing or
// out-of-range page sets the status word and nothing is written.
// Values are rounded to the storage type after the norm and again after the
// rotation only once: the rotation works on fp32 normed values.
// ---------------------------------------------------------------------------
template <typename T, typename TW>
__global__ void qk_norm_rope_write_kernel(
    T* __restrict__ qkv, int n_tokens, int n_q, int n_kv, int d, const TW* __restrict__ q_w,
    const TW* __restrict__ k_w, float eps, const float2* __restrict__ rope, int rotary_dim,
    int max_positions, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ block_table, int table_width, int n_seqs, T* __restrict__ k_pool,
    T* __restrict__ v_pool, int num_pages, int page_tokens, int adjacent, int* status) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = n_q + 2 * n_kv;
  const long long item = (long long)blockIdx.x * warps_per_block + warp;
  if (item >= (long long)n_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item - (long long)t * heads);
  float* buf = smem + warp * d;
  T* row = qkv + ((size_t)t * heads + h) * d;
  const bool is_q = h < n_q, is_k = !is_q && h < n_q + n_kv;
  const int pos = positions[t];

  float ss = 0.f;
  for (int c = lane; c < d; c += 32) {
    const float v = to_float<T>(row[c]);
    buf[c] = v;
    ss = fmaf(v, v, ss);
  }
  const TW* w = is_q ? q_w : (is_k ? k_w : nullptr);
  if (w != nullptr) {
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)d + eps);
    for (int c = lane; c < d; c += 32) buf[c] = buf[c] * to_float<TW>(w[c]) * inv;
  }
  __syncwarp();
  const bool rotate = (is_q || is_k) && rope != nullptr;
  if (rotate && (pos < 0 || pos >= max_positions)) {
    if (lane == 0) set_status(status, kBadPosition, t, pos);
    return;
  }
  // destination in the cache
  T* cache_row = nullptr;
  if (!is_q && k_pool != nullptr) {
    const int s = seq_of_token[t];
    if (s < 0 || s >= n_seqs) {
      if (lane == 0) set_status(status, kBadSequence, t, s);
      return;
    }
    const int blk = pos / page_tokens;
    const int page = (pos >= 0 && blk < table_width) ? block_table[(size_t)s * table_width + blk] : -1;
    if (page < 0 || page >= num_pages) {
      if (lane == 0) set_status(status, kBadPage, t, page, pos);
      return;
    }
    const int kvh = is_k ? h - n_q : h - n_q - n_kv;
    T* pool = is_k ? k_pool : v_pool;
    cache_row = pool + (((size_t)page * n_kv + kvh) * page_tokens + (pos % page_tokens)) * d;
  }
  const int half = rotary_dim >> 1;
  for (int c = lane; c < d; c += 32) {
    float v = buf[c];
    if (rotate && c < rotary_dim) {
      // pair i of the head: elements (i, i + half), or (2i, 2i + 1) with adjacent pairing
      const int pair = adjacent ? c >> 1 : (c < half ? c : c - half);
      const bool first = adjacent ? (c & 1) == 0 : c < half;
      const float2 cs = rope[(size_t)pos * half + pair];
      const float a = buf[adjacent ? 2 * pair : pair], b = buf[adjacent ? 2 * pair + 1 : pair + half];
      v = first ? a * cs.x - b * cs.y : a * cs.y + b * cs.x;
    }
    const T o = from_float<T>(v);
    if (is_q || is_k) row[c] = o;
    if (cache_row != nullptr) cache_row[c] = o;
  }
}

// The same for head sizes 64, 128 and 256 in bfloat16 with a full-width rotary table: a lane
// holds E = head_dim/32 consecutive elements, so the element's rotation partner (half a head
// away) sits in lane ^ 16 at the same place and comes by one shuffle; loads and stores are
// 4- to 16-byte vectors.
template <int E, typename TW>
__global__ void __launch_bounds__(256)
qk_norm_rope_write_vec_kernel(
    __nv_bfloat16* __restrict__ qkv, int n_tokens, int n_q, int n_kv, const TW* __restrict__ q_w,
    const TW* __restrict__ k_w, float eps, const float2* __restrict__ rope, int max_positions,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ block_table, int table_width, int n_seqs,
    __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool, int num_pages,
    int page_tokens, int adjacent, int* status) {
  // One block per token, a warp per head at a time: the token's position, page, rotation row
  // and the norm weights are fetched once per warp and serve all its heads, and the next
  // head's row is requested before the current one is worked on.
  constexpr int d = 32 * E;
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  const int heads = n_q + 2 * n_kv;
  const int t = blockIdx.x;
  const int pos = positions[t];
  const bool rotate = rope != nullptr;
  if (rotate && (pos < 0 || pos >= max_positions)) {
    if (threadIdx.x == 0) set_status(status, kBadPosition, t, pos);
    return;
  }
  long long cache_at = -1;                       // element offset of (page, kv head 0, slot) in the pools
  if (k_pool != nullptr) {
    const int s = seq_of_token[t];
    if (s < 0 || s >= n_seqs) {
      if (threadIdx.x == 0) set_status(status, kBadSequence, t, s);
      return;
    }
    const int blk = pos / page_tokens;
    const int page = (pos >= 0 && blk < table_width) ? block_table[(size_t)s * table_width + blk] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) set_status(status, kBadPage, t, page, pos);
      return;
    }
    cache_at = ((long long)page * n_kv * page_tokens + (pos % page_tokens)) * d;
  }
  const bool upper = lane >= 16;                   // elements of the second half
  const int pair0 = (lane & 15) * E;               // pair index of this lane's first element
  float2 cs[E];                                    // with adjacent pairing: of elements 2j, 2j + 1 in cs[j]
  float wq[E], wk[E];
#pragma unroll
  for (int i = 0; i < E; ++i) {
    const int pair = adjacent ? (lane * E) / 2 + (i >> 1) : pair0 + i;
    cs[i] = rotate ? rope[(size_t)pos * (d / 2) + pair] : make_float2(1.f, 0.f);
    wq[i] = q_w != nullptr ? to_float<TW>(q_w[lane * E + i]) : 1.f;
    wk[i] = k_w != nullptr ? to_float<TW>(k_w[lane * E + i]) : 1.f;
  }
  __nv_bfloat16* tok = qkv + (size_t)t * heads * d + lane * E;
  auto fetch = [&](int h, __nv_bfloat162 (&raw)[E / 2]) {
    if (h < heads) {
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(tok + (size_t)h * d);
#pragma unroll
      for (int i = 0; i < E / 2; ++i) raw[i] = p2[i];
    }
  };
  __nv_bfloat162 nxt[E / 2];
  fetch(warp, nxt);
  for (int h = warp; h < heads; h += n_warps) {
    float v[E];
#pragma unroll
    for (int i = 0; i < E / 2; ++i) {
      v[2 * i] = __low2float(nxt[i]);
      v[2 * i + 1] = __high2float(nxt[i]);
    }
    fetch(h + n_warps, nxt);
    const bool is_q = h < n_q, is_k = !is_q && h < n_q + n_kv;
    if ((is_q && q_w != nullptr) || (is_k && k_w != nullptr)) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < E; ++i) ss = fmaf(v[i], v[i], ss);
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)d + eps);
#pragma unroll
      for (int i = 0; i < E; ++i) v[i] = v[i] * (is_q ? wq[i] : wk[i]) * inv;
    }
    if (rotate && (is_q || is_k)) {
      if (adjacent) {                              // both elements of a pair are this lane's own
#pragma unroll
        for (int i = 0; i < E; i += 2) {
          const float a = v[i], b = v[i + 1];
          v[i] = a * cs[i].x - b * cs[i].y;
          v[i + 1] = a * cs[i].y + b * cs[i].x;
        }
      } else {
#pragma unroll
        for (int i = 0; i < E; ++i) {
          const float other = __shfl_xor_sync(0xffffffffu, v[i], 16);
          v[i] = upper ? other * cs[i].y + v[i] * cs[i].x : v[i] * cs[i].x - other * cs[i].y;
        }
      }
    }
    __nv_bfloat162 o2[E / 2];
#pragma unroll
    for (int i = 0; i < E / 2; ++i) o2[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    if (is_q || is_k) {
      __nv_bfloat162* row = reinterpret_cast<__nv_bfloat162*>(tok + (size_t)h * d);
#pragma unroll
      for (int i = 0; i < E / 2; ++i) row[i] = o2[i];
    }
    if (!is_q && cache_at >= 0) {
      const int kvh = is_k ? h - n_q : h - n_q - n_kv;
      __nv_bfloat16* pool = is_k ? k_pool : v_pool;
      __nv_bfloat162* cache_row =
          reinterpret_cast<__nv_bfloat162*>(pool + cache_at + (long long)kvh * page_tokens * d + lane * E);
#pragma unroll
      for (int i = 0; i < E / 2; ++i) cache_row[i] = o2[i];
    }
  }
}

// ---------------------------------------------------------------------------
// Sampling over fp32 logits [rows, vocab], one block per row.
//  temperature == 0: greedy, highest finite logit, lowest index on a tie
//    (crates/leone/src/sampler.rs:787-799; ie_cuda.cu:4814-4823).
//  temperature > 0: w_i = exp(l_i/t - max_j l_j/t) over finite logits, summed in fp64;
//    u = uniform(seed, position) from the reference's counter-based generator
//    (crates/leone/src/sampler.rs:84-94, 166-171); the token is the first in id order
//    whose cumulative weight exceeds u * total, else the last eligible one (:839-858).
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long splitmix64(unsigned long long v) {
  unsigned long long z = v + 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One block of 1024 threads per row.  Pass 1 (coalesced): highest finite logit and its lowest
// id.  Temperature rows: each of the 32 warps owns one contiguous run of ids and sums its
// weights with coalesced loads; the run that holds u * total is found by a scan over the 32
// warp sums in id order, and that warp walks its run 32 ids at a time with a warp prefix sum,
// so the chosen token is the first in id order whose cumulative weight exceeds the target.
//
// The sampling parameters of a row come either from three arrays indexed by row, or (records !=
// null) from the per-request slot records: row r belongs to slot slot_ids[r], whose record holds
// the position of the token being sampled (field kSlotPosition), the seed (kSlotSeed) and the
// temperature (kSlotTemperature, fp32 bits).
constexpr int kSlotFields = 8;
constexpr int kSlotLength = 0, kSlotPosition = 1, kSlotSeed = 2, kSlotTemperature = 3, kSlotLastToken = 4;

__global__ void __launch_bounds__(1024)
sample_kernel(const float* __restrict__ logits, int vocab,
                              const float* __restrict__ temperature,
                              const long long* __restrict__ seeds,
                              const long long* __restrict__ positions, int* __restrict__ out,
                              const int* __restrict__ slot_ids, const long long* __restrict__ records) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ double s_sum[32];
  __shared__ double s_before;
  __shared__ int s_owner;
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* l = logits + (size_t)row * vocab;
  float best = -INFINITY;
  int best_i = -1;
  for (int i = tid; i < vocab; i += 1024) {      // ids rise within a thread: '>' keeps the lowest
    const float v = l[i];
    if (isfinite(v) && (best_i < 0 || v > best)) { best = v; best_i = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (oi >= 0 && (best_i < 0 || ov > best || (ov == best && oi < best_i))) { best = ov; best_i = oi; }
  }
  if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    best = s_val[lane];
    best_i = s_idx[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (oi >= 0 && (best_i < 0 || ov > best || (ov == best && oi < best_i))) { best = ov; best_i = oi; }
    }
    if (lane == 0) { s_val[0] = best; s_idx[0] = best_i; }
  }
  __syncthreads();
  const float top = s_val[0];
  const int top_i = s_idx[0];
  const long long* record = records ? records + (size_t)slot_ids[row] * kSlotFields : nullptr;
  const float temp = record ? __int_as_float((int)record[kSlotTemperature]) : (temperature ? temperature[row] : 0.f);
  if (!(temp > 0.f) || top_i < 0) {
    if (tid == 0) out[row] = top_i;
    return;
  }
  const double t = (double)temp, hi_scaled = (double)top / t;
  const int run = ((vocab + 31) / 32 + 31) / 32 * 32;          // ids per warp, a multiple of 32
  const int lo = min(warp * run, vocab), hi = min(lo + run, vocab);
  double sum = 0.0;
  for (int i = lo + lane; i < hi; i += 32) {
    const float v = l[i];
    if (isfinite(v)) sum += exp((double)v / t - hi_scaled);
  }
  sum = warp_sum_f64(sum);
  if (lane == 0) s_sum[warp] = sum;
  __syncthreads();
  if (tid == 0) {
    double total = 0.0;
    for (int i = 0; i < 32; ++i) total += s_sum[i];
    const unsigned long long purpose = 0xbf58476d1ce4e5b9ull;
    const unsigned long long seed = (unsigned long long)(record ? record[kSlotSeed] : seeds[row]);
    const unsigned long long position = (unsigned long long)(record ? record[kSlotPosition] : positions[row]);
    const unsigned long long mixed = splitmix64(seed ^ splitmix64(position ^ purpose));
    const double u = (double)(mixed >> 11) * (1.0 / 9007199254740992.0);
    const double target = u * total;
    double c = 0.0;
    int owner = -1;
    for (int i = 0; i < 32; ++i) {
      if (target < c + s_sum[i]) { owner = i; break; }
      c += s_sum[i];
    }
    if (owner < 0) {                     // rounding left the sum just below the target:
      owner = 31;                        // the last run with any weight takes it
      while (owner > 0 && !(s_sum[owner] > 0.0)) --owner;
      c = total - s_sum[owner];
    }
    s_owner = owner;
    s_before = c;
    // the target is recomputed by the owner from the same values
    s_sum[0] = target;
  }
  __syncthreads();
  if (warp != s_owner) return;
  const double target = s_sum[0];
  double c = s_before;
  int chosen = -1, last = -1;
  for (int base = lo; base < hi && chosen < 0; base += 32) {
    const int i = base + lane;
    double wgt = 0.0;
    if (i < hi) {
      const float v = l[i];
      if (isfinite(v)) wgt = exp((double)v / t - hi_scaled);
    }
    double incl = wgt;                   // inclusive prefix over the 32 lanes, in id order
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const double up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    const bool hit = wgt > 0.0 && target < c + incl;
    const unsigned hits = __ballot_sync(0xffffffffu, hit);
    const unsigned live = __ballot_sync(0xffffffffu, wgt > 0.0);
    if (live) last = base + 31 - __clz(live);
    if (hits) chosen = base + __ffs(hits) - 1;
    c += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) out[row] = chosen >= 0 ? chosen : (last >= 0 ? last : top_i);
}

// ---------------------------------------------------------------------------
// Feeds a decode step's sampled tokens back as the next step's inputs without the host:
// token_ids <- sampled, positions/ctx_len/sample positions += 1, and the sampled ids are
// appended to a history the host reads once per quantum.  One block.  The reference keeps
// its decode position in a device word that a kernel increments for graph replay
// (crates/leone-cuda/cuda/ie_cuda.cu:2940); this is the same idea for a whole batch.
// ---------------------------------------------------------------------------
// With slot records (records != null) the request's record is advanced instead of sample_pos:
// its position and length by one, its last token set.
__global__ void decode_advance_kernel(int* token_ids, int* positions, int* ctx_len,
                                      long long* sample_pos, const int* sampled, int* history,
                                      int* step_counter, int n, int max_steps, const int* slot_ids,
                                      long long* records) {
  pdl_trigger();
  pdl_wait();
  const int step = *step_counter;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int tok = sampled[i];
    token_ids[i] = tok;
    positions[i] += 1;
    ctx_len[i] += 1;
    if (records) {
      long long* record = records + (size_t)slot_ids[i] * kSlotFields;
      record[kSlotPosition] += 1;
      record[kSlotLength] += 1;
      record[kSlotLastToken] = tok;
    } else {
      sample_pos[i] += 1;
    }
    if (step < max_steps) history[(size_t)step * n + i] = tok;
  }
  if (threadIdx.x == 0) *step_counter = step + 1;
}

}  // namespace leone

using namespace leone;

extern "C" int leone_decode_advance(int* token_ids, int* positions, int* ctx_len,
                                    long long* sample_pos, const int* sampled, int* history,
                                    int* step_counter, int n, int max_steps, const int* slot_ids,
                                    long long* records, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((records != nullptr) == (sample_pos != nullptr)) return kRefusedSize;    // one of the two
  return launch_kernel(decode_advance_kernel, dim3(1), dim3(n < 1024 ? ((n + 31) / 32) * 32 : 1024), 0,
                       stream, token_ids, positions, ctx_len, sample_pos, sampled, history,
                       step_counter, n, max_steps, slot_ids, records);
}

// Turns programmatic dependent launch on or off for the kernels of this library.
extern "C" void leone_core_set_pdl(int enabled) { pdl_flag() = enabled ? 1 : 0; }

extern "C" int leone_logit_post(float* logits, long long n, float scale, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  const long long want = (n + 255) / 256;
  return launch_kernel(logit_post_kernel, dim3((unsigned)(want < 148 * 8 ? want : 148 * 8)), dim3(256), 0, stream,
                       logits, n, scale, cap);
}

extern "C" int leone_embedding(int dtype, const void* table, const int* ids, float* out, int n,
                               int hidden, int vocab, float scale, int* status, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (hidden <= 0 || vocab <= 0) return kRefusedSize;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == 0)
    return launch_kernel(embedding_kernel<float>, dim3(n), dim3(threads), 0, stream, (const float*)table,
                         ids, out, hidden, vocab, scale, status);
  if (dtype == 1)
    return launch_kernel(embedding_kernel<__nv_bfloat16>, dim3(n), dim3(threads), 0, stream,
                         (const __nv_bfloat16*)table, ids, out, hidden, vocab, scale, status);
  return kRefusedDtype;
}

extern "C" int leone_rms_norm(const float* x, const int* rows, const void* w, int w_dtype, void* out,
                              int out_dtype, int n_out, int hidden, float eps, cudaStream_t stream) {
  if (n_out <= 0) return 0;
  if (hidden <= 0) return kRefusedSize;
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  const bool vec = (hidden % 4) == 0 && hidden >= 512 && hidden <= kNormThreads * kNormItems * 4 &&
                   (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
#define LAUNCH(TW, TO)                                                                           \
  {                                                                                              \
    if (vec)                                                                                     \
      return launch_kernel(rms_norm_vec_kernel<TW, TO>, dim3(n_out), dim3(kNormThreads), 0, stream, x, \
                           rows, (const TW*)w, (TO*)out, hidden, eps);                            \
    return launch_kernel(rms_norm_kernel<TW, TO>, dim3(n_out), dim3(threads), 0, stream, x, rows, \
                         (const TW*)w, (TO*)out, hidden, eps);                                    \
  }
  if (w_dtype == 0 && out_dtype == 0) LAUNCH(float, float);
  if (w_dtype == 0 && out_dtype == 1) LAUNCH(float, __nv_bfloat16);
  if (w_dtype == 1 && out_dtype == 0) LAUNCH(__nv_bfloat16, float);
  if (w_dtype == 1 && out_dtype == 1) LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
  return kRefusedDtype;
}

extern "C" int leone_swiglu(int dtype, const void* gate_up, void* out, int n, int inter,
                            cudaStream_t stream) {
  if (n <= 0) return 0;
  if (inter <= 0) return kRefusedSize;
  const size_t total = (size_t)n * inter;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  if (dtype == 0)
    swiglu_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gate_up, (float*)out, n, inter);
  else if (dtype == 1)
    swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, n, inter);
  else
    return kRefusedDtype;
  return launch_result();
}

extern "C" int leone_qk_norm_rope_write(
    int dtype, void* qkv, int n_tokens, int n_q, int n_kv, int d, const void* q_w, const void* k_w,
    int w_dtype, float eps, const float* rope, int rotary_dim, int max_positions,
    const int* positions, const int* seq_of_token, const int* block_table, int table_width,
    int n_seqs, void* k_pool, void* v_pool, int num_pages, int page_tokens, int adjacent, int* status,
    cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (d <= 0 || d > 1024 || n_q <= 0 || n_kv <= 0) return kRefusedSize;
  if (rope != nullptr && (rotary_dim <= 0 || rotary_dim > d || (rotary_dim & 1))) return kRefusedSize;
  if (k_pool != nullptr && (page_tokens <= 0 || table_width <= 0)) return kRefusedSize;
  const int warps = 4;
  const long long items = (long long)n_tokens * (n_q + 2 * n_kv);
  const int blocks = (int)((items + warps - 1) / warps);
  const size_t smem = (size_t)warps * d * sizeof(float);
  // the vector kernel: a block per token, a warp for up to every eighth head
  const int vec_threads = 32 * (n_q + 2 * n_kv < 8 ? n_q + 2 * n_kv : 8);
  if (dtype == 1 && (d == 64 || d == 128 || d == 256) && (rope == nullptr || rotary_dim == d) &&
      (q_w == nullptr) == (k_w == nullptr)) {
#define LAUNCH_VEC(E, TW)                                                                          \
  return launch_kernel(qk_norm_rope_write_vec_kernel<E, TW>, dim3(n_tokens), dim3(vec_threads), 0, stream, \
                       (__nv_bfloat16*)qkv, n_tokens, n_q, n_kv, (const TW*)q_w, (const TW*)k_w, eps, \
                       (const float2*)rope, max_positions, positions, seq_of_token, block_table,  \
                       table_width, n_seqs, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool,        \
                       num_pages, page_tokens, adjacent, status)
    if (w_dtype == 0) {
      if (d == 64) LAUNCH_VEC(2, float);
      if (d == 128) LAUNCH_VEC(4, float);
      LAUNCH_VEC(8, float);
    } else if (w_dtype == 1) {
      if (d == 64) LAUNCH_VEC(2, __nv_bfloat16);
      if (d == 128) LAUNCH_VEC(4, __nv_bfloat16);
      LAUNCH_VEC(8, __nv_bfloat16);
    }
#undef LAUNCH_VEC
  }
#define LAUNCH(T, TW)                                                                              \
  return launch_kernel(qk_norm_rope_write_kernel<T, TW>, dim3(blocks), dim3(warps * 32), smem, stream, \
                       (T*)qkv, n_tokens, n_q, n_kv, d, (const TW*)q_w, (const TW*)k_w, eps,          \
                       (const float2*)rope, rotary_dim, max_positions, positions, seq_of_token,      \
                       block_table, table_width, n_seqs, (T*)k_pool, (T*)v_pool, num_pages,          \
                       page_tokens, adjacent, status)
  if (dtype == 0 && w_dtype == 0) LAUNCH(float, float);
  if (dtype == 1 && w_dtype == 0) LAUNCH(__nv_bfloat16, float);
  if (dtype == 0 && w_dtype == 1) LAUNCH(float, __nv_bfloat16);
  if (dtype == 1 && w_dtype == 1) LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
  return kRefusedDtype;
}

extern "C" int leone_sample(const float* logits, int rows, int vocab, const float* temperature,
                            const long long* seeds, const long long* positions, int* out,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return kRefusedSize;
  return launch_kernel(sample_kernel, dim3(rows), dim3(1024), 0, stream, logits, vocab, temperature,
                       seeds, positions, out, (const int*)nullptr, (const long long*)nullptr);
}

// The same with every row's parameters taken from its request's slot record.
extern "C" int leone_sample_slots(const float* logits, int rows, int vocab, const int* slot_ids,
                                  const long long* records, int* out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || slot_ids == nullptr || records == nullptr) return kRefusedSize;
  return launch_kernel(sample_kernel, dim3(rows), dim3(1024), 0, stream, logits, vocab, (const float*)nullptr,
                       (const long long*)nullptr, (const long long*)nullptr, out, slot_ids, records);
}
