// Causal grouped-query attention over a paged cache, any sizes, any cut.
//
// One block per (token, query head).  The query at absolute position p reads
// keys lo..p of its own sequence (lo = 0, or p-window+1 for a windowed layer),
// found through the sequence's block table.  kv_head = q_head / (n_q / n_kv);
// score = (q.k) * scale; softmax and the weighted sum run online in fp32 over
// tiles of 128 keys in ascending order (crates/leone/src/cpu.rs:2299-2421; the
// mask is the loop bound, :2372).  Because a row's arithmetic depends only on
// its own sequence, the result is the same however the tokens were cut into
// steps or batched.  This kernel is the attention of the 32-bit path and takes
// every size; the bfloat16 path uses it for sizes its tiled kernels refuse.
#include "common.cuh"

namespace leone {

constexpr int kAttnThreads = 128;
constexpr int kMaxAccPerThread = 8;   // head_dim <= 1024

template <typename T>
__global__ void __launch_bounds__(kAttnThreads)
attention_generic_kernel(const T* __restrict__ qkv, int row_stride, T* __restrict__ out,
                         int out_stride, const T* __restrict__ k_pool,
                         const T* __restrict__ v_pool, const int* __restrict__ block_table,
                         int table_width, const int* __restrict__ seq_of_token,
                         const int* __restrict__ positions, int n_q, int n_kv, int d, float scale,
                         int window, int page_tokens, int num_pages, int n_seqs, int* status) {
  extern __shared__ __align__(16) float smem[];
  long long* off_s = (long long*)smem;                // [128] row index into the pools
  float* p_s = smem + 2 * kAttnThreads;               // [128]
  float* q_s = p_s + kAttnThreads;                    // [d]
  __shared__ float scratch[33];
  __shared__ int bad;

  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int pos = positions[t], s = seq_of_token[t];
  const int kvh = h / (n_q / n_kv);
  T* dst = out + (size_t)t * out_stride + (size_t)h * d;
  if (tid == 0) bad = 0;
  if (s < 0 || s >= n_seqs || pos < 0) {
    if (tid == 0) set_status(status, s < 0 || s >= n_seqs ? kBadSequence : kBadPosition, t, s < 0 || s >= n_seqs ? s : pos);
    for (int c = tid; c < d; c += kAttnThreads) dst[c] = from_float<T>(0.f);
    return;
  }
  const T* q = qkv + (size_t)t * row_stride + (size_t)h * d;
  for (int c = tid; c < d; c += kAttnThreads) q_s[c] = to_float<T>(q[c]);
  __syncthreads();

  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  float m_run = -INFINITY, l_run = 0.f;
  float acc[kMaxAccPerThread];
#pragma unroll
  for (int i = 0; i < kMaxAccPerThread; ++i) acc[i] = 0.f;

  for (int j0 = lo; j0 <= pos; j0 += kAttnThreads) {
    const int j = j0 + tid;
    float score = -INFINITY;
    long long row_index = -1;
    if (j <= pos) {
      const int blk = j / page_tokens;
      const int page = blk < table_width ? block_table[(size_t)s * table_width + blk] : -1;
      if (page < 0 || page >= num_pages) {
        set_status(status, kBadPage, t, page, j);
        bad = 1;
      } else {
        row_index = ((long long)page * n_kv + kvh) * page_tokens + (j % page_tokens);
        const T* krow = k_pool + row_index * d;
        float dot = 0.f;
        for (int c = 0; c < d; ++c) dot = fmaf(q_s[c], to_float<T>(krow[c]), dot);
        score = dot * scale;
      }
    }
    off_s[tid] = row_index;
    const float tile_max = block_max(score, scratch);
    const float m_new = fmaxf(m_run, tile_max);
    const float p = (row_index >= 0) ? expf(score - m_new) : 0.f;
    p_s[tid] = p;
    const float tile_sum = block_sum(p, scratch);   // also orders p_s/off_s writes before reads
    const float alpha = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
    l_run = l_run * alpha + tile_sum;
    m_run = m_new;
    const int count = min(kAttnThreads, pos - j0 + 1);
#pragma unroll
    for (int i = 0; i < kMaxAccPerThread; ++i) {
      const int c = tid + i * kAttnThreads;
      if (c < d) {
        float a = acc[i] * alpha;
        for (int jj = 0; jj < count; ++jj) {
          const long long r = off_s[jj];
          if (r >= 0) a = fmaf(p_s[jj], to_float<T>(v_pool[r * d + c]), a);
        }
        acc[i] = a;
      }
    }
    __syncthreads();
  }
  const float inv = (l_run > 0.f && !bad) ? 1.f / l_run : 0.f;
#pragma unroll
  for (int i = 0; i < kMaxAccPerThread; ++i) {
    const int c = tid + i * kAttnThreads;
    if (c < d) dst[c] = from_float<T>(acc[i] * inv);
  }
}

}  // namespace leone

using namespace leone;

extern "C" int leone_attention_generic(int dtype, const void* qkv, int row_stride, void* out,
                                       int out_stride, const void* k_pool, const void* v_pool,
                                       const int* block_table, int table_width,
                                       const int* seq_of_token, const int* positions, int n_tokens,
                                       int n_q, int n_kv, int d, float scale, int window,
                                       int page_tokens, int num_pages, int n_seqs, int* status,
                                       cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (d <= 0 || d > kAttnThreads * kMaxAccPerThread || n_q <= 0 || n_kv <= 0 || n_q % n_kv != 0 ||
      n_q > 65535 || page_tokens <= 0 || table_width <= 0)
    return kRefusedSize;
  dim3 grid(n_tokens, n_q);
  const size_t smem = (size_t)(d + kAttnThreads) * sizeof(float) + kAttnThreads * sizeof(long long) + 8;
  if (dtype == 0)
    attention_generic_kernel<float><<<grid, kAttnThreads, smem, stream>>>(
        (const float*)qkv, row_stride, (float*)out, out_stride, (const float*)k_pool,
        (const float*)v_pool, block_table, table_width, seq_of_token, positions, n_q, n_kv, d,
        scale, window, page_tokens, num_pages, n_seqs, status);
  else if (dtype == 1)
    attention_generic_kernel<__nv_bfloat16><<<grid, kAttnThreads, smem, stream>>>(
        (const __nv_bfloat16*)qkv, row_stride, (__nv_bfloat16*)out, out_stride,
        (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, block_table, table_width,
        seq_of_token, positions, n_q, n_kv, d, scale, window, page_tokens, num_pages, n_seqs, status);
  else
    return kRefusedDtype;
  return launch_result();
}
