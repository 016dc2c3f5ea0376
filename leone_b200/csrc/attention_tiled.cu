// Causal grouped-query attention over the paged cache in bfloat16 with fp32 softmax:
// a tiled kernel for prompt portions (and mixed batches), and a split-KV kernel
// for decode steps with its merge.
//
// Formulas: kv_head = q_head / (n_q / n_kv); score = (q.k) * scale; online softmax
// with running maximum and sum; output = numerator / sum (crates/leone/src/cpu.rs:2299-2421).
// The reference's decode kernel runs one block per (query head, split), so the keys of
// a KV head are fetched once per query head (crates/leone-cuda/cuda/ie_cuda.cu:4464-4556),
// and its prompt path materialises the score matrix (ie_cuda.cu:5123-5220).  Here the
// query heads of one KV head share each key/value tile, scores never leave registers,
// and pages are gathered through the block table with asynchronous 16-byte copies.
//
// Both kernels keep the products on mma.sync tensor-core tiles (m16n8k16, bf16 in, fp32
// out): the decode step is bound by reading the cache, not by arithmetic.
//
// Sizes: head_dim a multiple of 16 up to 128 (instantiated below); up to 64 query heads
// per KV head; any page size; any window.  Other sizes are refused (the caller falls
// back to the any-size kernel).
#include "common.cuh"

namespace leone {
namespace tiled {

constexpr int kThreads = 128;
constexpr int kKeyTile = 64;
constexpr int kRowsPerBlock = 64;      // query rows (token, head) per block in the prompt kernel
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;     // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
// Transposes an 8x8 matrix of 16-bit values held across the warp (thread t: row t/4, columns
// 2*(t%4) and 2*(t%4)+1 in one register): turns an accumulator's layout into a B operand's.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct PagedArgs {
  const __nv_bfloat16* k_pool;
  const __nv_bfloat16* v_pool;
  const int* block_table;
  int table_width;
  int page_tokens;
  int num_pages;
  int n_kv;
};

// Copies keys/values [tile_start, tile_start+64) of one sequence and KV head into shared
// memory rows of D+8 elements; rows before `k_first` (keys a window has passed, whose pages
// may already be given back) and rows at or past `k_end` are zero-filled.
template <int D>
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* k_s, __nv_bfloat16* v_s,
                                             long long* row_src, const PagedArgs& pa, int seq,
                                             int kvh, int tile_start, int k_first, int k_end,
                                             int* status, int token_row) {
  constexpr int kRow = D + 8;
  constexpr int kChunks = D / 8;
  const int tid = threadIdx.x;
  if (tid < kKeyTile) {
    const int kj = tile_start + tid;
    long long src = -1;
    if (kj < k_end && kj >= k_first) {
      const int blk = kj / pa.page_tokens;
      const int page = blk < pa.table_width ? pa.block_table[(size_t)seq * pa.table_width + blk] : -1;
      if (page < 0 || page >= pa.num_pages) {
        set_status(status, kBadPage, token_row, page, kj);
      } else {
        src = (((long long)page * pa.n_kv + kvh) * pa.page_tokens + (kj % pa.page_tokens)) * D;
      }
    }
    row_src[tid] = src;
  }
  __syncthreads();
  for (int idx = tid; idx < kKeyTile * kChunks; idx += kThreads) {
    const int row = idx / kChunks, ch = idx - row * kChunks;
    const long long src = row_src[row];
    const bool ok = src >= 0;
    const long long off = ok ? src + ch * 8 : 0;
    cp_async16(smem_u32(k_s + row * kRow + ch * 8), pa.k_pool + off, ok);
    cp_async16(smem_u32(v_s + row * kRow + ch * 8), pa.v_pool + off, ok);
  }
}

// ------------------------------------------------------------------------------------
// Prompt portions and mixed batches.  grid = (query tiles, n_kv, sequences).
// A block owns up to 64 rows = (tokens of the tile) x (the g query heads of one KV head),
// 16 rows per warp, and walks the keys in tiles of 64.
// ------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(kThreads)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ qkv, int row_stride,
                         __nv_bfloat16* __restrict__ out, int out_stride, PagedArgs pa,
                         const int* __restrict__ q_start, const int* __restrict__ ctx_len,
                         int n_q, float scale, int window, int* status) {
  constexpr int kRow = D + 8;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [64][kRow]
  __nv_bfloat16* kv_s = q_s + kRowsPerBlock * kRow;                           // [2 stages][K,V][64][kRow]
  long long* row_src = reinterpret_cast<long long*>(kv_s + 4 * kKeyTile * kRow);   // [2][64]

  pdl_trigger();
  pdl_wait();
  const int seq = blockIdx.z, kvh = blockIdx.y, qt = blockIdx.x;
  const int g = n_q / pa.n_kv;
  const int tq = kRowsPerBlock / g;                 // tokens per tile
  const int q0 = q_start[seq], q_len = q_start[seq + 1] - q0;
  const int tok0 = qt * tq;
  if (tok0 >= q_len) return;
  const int ctx = ctx_len[seq], start = ctx - q_len;
  const int tok1 = min(q_len, tok0 + tq);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // gather the tile's query rows
  for (int idx = tid; idx < kRowsPerBlock * (D / 8); idx += kThreads) {
    const int r = idx / (D / 8), ch = idx - r * (D / 8);
    const int tl = r / g, hh = r - tl * g;
    const int token = tok0 + tl;
    const bool ok = tl < tq && token < tok1;
    const __nv_bfloat16* src =
        qkv + (size_t)(q0 + (ok ? token : 0)) * row_stride + (size_t)(kvh * g + hh) * D + ch * 8;
    cp_async16(smem_u32(q_s + r * kRow + ch * 8), src, ok);
  }
  cp_async_commit();

  const int k_hi = start + tok1;                       // one past the last key any row reads
  int k_lo = 0;
  if (window > 0) k_lo = max(0, start + tok0 - window + 1);
  const int tile0 = (k_lo / kKeyTile) * kKeyTile;
  const int n_tiles = (k_hi - tile0 + kKeyTile - 1) / kKeyTile;

  load_kv_tile<D>(kv_s, kv_s + kKeyTile * kRow, row_src, pa, seq, kvh, tile0, k_lo, k_hi, status,
                  q0 + tok0);
  cp_async_commit();

  // this thread's two rows
  int row_pos[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + (lane >> 2) + h * 8;
    const int tl = r / g;
    row_pos[h] = (tl < tq && tok0 + tl < tok1) ? start + tok0 + tl : -1;   // -1: row unused
  }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  uint32_t q_frag[D / 16][4];
  const float sl2 = scale * kLog2e;

  for (int t = 0; t < n_tiles; ++t) {
    const int stage = t & 1;
    __nv_bfloat16* k_s = kv_s + stage * 2 * kKeyTile * kRow;
    __nv_bfloat16* v_s = k_s + kKeyTile * kRow;
    if (t + 1 < n_tiles) {
      __nv_bfloat16* k_n = kv_s + (stage ^ 1) * 2 * kKeyTile * kRow;
      load_kv_tile<D>(k_n, k_n + kKeyTile * kRow, row_src + (stage ^ 1) * kKeyTile, pa, seq, kvh,
                      tile0 + (t + 1) * kKeyTile, k_lo, k_hi, status, q0 + tok0);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (t == 0) {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int mi = lane >> 3;
        const int r = warp * 16 + (mi & 1) * 8 + (lane & 7), c = ks * 16 + (mi >> 1) * 8;
        ldmatrix_x4(smem_u32(q_s + r * kRow + c), q_frag[ks]);
      }
    }
    const int tile_start = tile0 + t * kKeyTile;
    // S = Q K^T for 64 keys: 8 n-tiles of 8 keys
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
      for (int kp = 0; kp < 4; ++kp) {            // 16 keys per ldmatrix.x4
        uint32_t b[4];
        const int mi = lane >> 3;
        const int r = kp * 16 + (mi >> 1) * 8 + (lane & 7), c = ks * 16 + (mi & 1) * 8;
        ldmatrix_x4(smem_u32(k_s + r * kRow + c), b);
        mma_16816(s[kp * 2], q_frag[ks], b[0], b[1]);
        mma_16816(s[kp * 2 + 1], q_frag[ks], b[2], b[3]);
      }
    }
    // mask and online softmax
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int h = j >> 1;
        const int kj = tile_start + nt * 8 + (lane & 3) * 2 + (j & 1);
        const bool keep = row_pos[h] >= 0 && kj <= row_pos[h] &&
                          (window <= 0 || kj > row_pos[h] - window);
        const float v = keep ? s[nt][j] * sl2 : -INFINITY;
        s[nt][j] = v;
        tile_max[h] = fmaxf(tile_max[h], v);
      }
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 1));
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 2));
      const float m_new = fmaxf(m_run[h], tile_max[h]);
      m_use[h] = m_new == -INFINITY ? 0.f : m_new;
      alpha[h] = m_run[h] == -INFINITY ? 0.f : exp2f(m_run[h] - m_use[h]);
      m_run[h] = m_new;
      l_run[h] *= alpha[h];
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o_acc[i][0] *= alpha[0];
      o_acc[i][1] *= alpha[0];
      o_acc[i][2] *= alpha[1];
      o_acc[i][3] *= alpha[1];
    }
    uint32_t p_frag[4][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float p0 = exp2f(s[nt][0] - m_use[0]), p1 = exp2f(s[nt][1] - m_use[0]);
      const float p2 = exp2f(s[nt][2] - m_use[1]), p3 = exp2f(s[nt][3] - m_use[1]);
      l_run[0] += p0 + p1;
      l_run[1] += p2 + p3;
      p_frag[nt >> 1][(nt & 1) * 2] = pack_bf16(p0, p1);
      p_frag[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    // O += P V
#pragma unroll
    for (int kp = 0; kp < 4; ++kp) {
#pragma unroll
      for (int np = 0; np < D / 16; ++np) {
        uint32_t b[4];
        const int mi = lane >> 3;
        const int r = kp * 16 + (mi & 1) * 8 + (lane & 7), c = np * 16 + (mi >> 1) * 8;
        ldmatrix_x4_trans(smem_u32(v_s + r * kRow + c), b);
        mma_16816(o_acc[np * 2], p_frag[kp], b[0], b[1]);
        mma_16816(o_acc[np * 2 + 1], p_frag[kp], b[2], b[3]);
      }
    }
    __syncthreads();      // everyone is done with this stage before it is refilled
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (row_pos[h] < 0) continue;
    const int r = warp * 16 + (lane >> 2) + h * 8;
    const int tl = r / g, hh = r - tl * g;
    const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
    __nv_bfloat16* dst = out + (size_t)(q0 + tok0 + tl) * out_stride + (size_t)(kvh * g + hh) * D;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const uint32_t v = pack_bf16(o_acc[i][h * 2] * inv, o_acc[i][h * 2 + 1] * inv);
      *reinterpret_cast<uint32_t*>(dst + i * 8 + (lane & 3) * 2) = v;
    }
  }
}

// ------------------------------------------------------------------------------------
// Decode: one query token per sequence.  grid = (n_kv * head groups, splits, sequences).
// The (up to 16) query heads of the KV head share every key and value tile.  The block's key
// range is cut into groups of 16 keys dealt round-robin to the four warps; every warp runs a
// private cp.async pipeline (kDecodeStages groups of keys and values in flight) and never
// waits for the others inside the loop; the warps are merged once at the end.  With more than
// one split the block writes (max, sum, unnormalised output) to scratch for the merge kernel.
// ------------------------------------------------------------------------------------
constexpr int kDecodeStages = 3;

// One warp's share of a decode block.  The keys ride the MMA's M side and the block's query
// heads its N side (NT tiles of 8 heads), so a head group of up to 8 costs one MMA per 16 keys
// x 16 dims instead of two, and the scores, the exponentials and the output accumulator are
// held for 8 columns, not 16 padded rows:
//   S^T[16 keys x 8 heads]   = K[16 x D] . Q^T            (A = keys, row-major; B = Q rows)
//   O^T[D x 8 heads]        += V^T[D x 16 keys] . P^T     (A = V through ldmatrix.trans;
//                                                          B = P^T, the transposed S^T tile)
// Thread t holds, of every 16 x 8 accumulator tile, rows t/4 and t/4+8 and columns 2*(t%4),
// 2*(t%4)+1: its two head columns are fixed, so the running maximum and sum are per thread.
template <int D, int NT>
struct DecodeWarp {
  static constexpr int kRow = D + 8;
  uint32_t qb[D / 16][NT][2];
  float m_run[NT][2], l_run[NT][2];
  float o[D / 16][NT][4];

  __device__ __forceinline__ void init() {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      m_run[nt][0] = m_run[nt][1] = -INFINITY;
      l_run[nt][0] = l_run[nt][1] = 0.f;
#pragma unroll
      for (int i = 0; i < D / 16; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][nt][j] = 0.f;
    }
  }

  // q_s: [16 heads][kRow], rows past the block's heads zero.
  __device__ __forceinline__ void load_q(const __nv_bfloat16* q_s, int lane) {
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int mi = (lane >> 3) & 1;
        ldmatrix_x2(smem_u32(q_s + (nt * 8 + (lane & 7)) * kRow + ks * 16 + mi * 8), qb[ks][nt]);
      }
  }

  // One group of 16 keys (rows of k_s / v_s) from absolute position key0; keys at or past
  // k_end are masked.
  __device__ __forceinline__ void group(const __nv_bfloat16* k_s, const __nv_bfloat16* v_s, int key0, int k_end,
                                        float sl2, int lane) {
    const int mi = lane >> 3;
    float st[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) st[nt][j] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a[4];
      ldmatrix_x4(smem_u32(k_s + ((mi & 1) * 8 + (lane & 7)) * kRow + ks * 16 + (mi >> 1) * 8), a);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) mma_16816(st[nt], a, qb[ks][nt][0], qb[ks][nt][1]);
    }
    uint32_t pb[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kj = key0 + (lane >> 2) + (j >> 1) * 8;
        const float v = kj < k_end ? st[nt][j] * sl2 : -INFINITY;
        st[nt][j] = v;
        tile_max[j & 1] = fmaxf(tile_max[j & 1], v);
      }
      float alpha[2], m_use[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 4));
        tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 8));
        tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 16));
        const float m_new = fmaxf(m_run[nt][h], tile_max[h]);
        m_use[h] = m_new == -INFINITY ? 0.f : m_new;
        alpha[h] = m_run[nt][h] == -INFINITY ? 0.f : exp2f(m_run[nt][h] - m_use[h]);
        m_run[nt][h] = m_new;
        l_run[nt][h] *= alpha[h];
      }
#pragma unroll
      for (int i = 0; i < D / 16; ++i) {
        o[i][nt][0] *= alpha[0];
        o[i][nt][1] *= alpha[1];
        o[i][nt][2] *= alpha[0];
        o[i][nt][3] *= alpha[1];
      }
      const float p0 = exp2f(st[nt][0] - m_use[0]), p1 = exp2f(st[nt][1] - m_use[1]);
      const float p2 = exp2f(st[nt][2] - m_use[0]), p3 = exp2f(st[nt][3] - m_use[1]);
      l_run[nt][0] += p0 + p2;
      l_run[nt][1] += p1 + p3;
      pb[nt][0] = movmatrix_trans(pack_bf16(p0, p1));     // keys 0..7 of the group
      pb[nt][1] = movmatrix_trans(pack_bf16(p2, p3));     // keys 8..15
    }
#pragma unroll
    for (int dt = 0; dt < D / 16; ++dt) {
      uint32_t a[4];
      ldmatrix_x4_trans(smem_u32(v_s + ((mi >> 1) * 8 + (lane & 7)) * kRow + dt * 16 + (mi & 1) * 8), a);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) mma_16816(o[dt][nt], a, pb[nt][0], pb[nt][1]);
    }
  }

  // This warp's (max, sum, unnormalised output) per head into mo [4 warps][16 heads][D] and
  // mml [4][16][2]; rows of heads past 8 * NT are not written (and never read).
  __device__ __forceinline__ void stash(float* mo, float* mml, int warp, int lane) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float l = l_run[nt][h];
        l += __shfl_xor_sync(0xffffffffu, l, 4);
        l += __shfl_xor_sync(0xffffffffu, l, 8);
        l += __shfl_xor_sync(0xffffffffu, l, 16);
        const int r = nt * 8 + (lane & 3) * 2 + h;
        if (lane < 4) {
          mml[(warp * 16 + r) * 2] = m_run[nt][h];
          mml[(warp * 16 + r) * 2 + 1] = l;
        }
#pragma unroll
        for (int i = 0; i < D / 16; ++i) {
          float* dst = mo + (size_t)(warp * 16 + r) * D + i * 16 + (lane >> 2);
          dst[0] = o[i][nt][h];
          dst[8] = o[i][nt][2 + h];
        }
      }
  }
};

template <int D, int NT>
__global__ void __launch_bounds__(kThreads)
attention_decode_kernel(const __nv_bfloat16* __restrict__ qkv, int row_stride,
                        __nv_bfloat16* __restrict__ out, int out_stride, PagedArgs pa,
                        const int* __restrict__ q_start, const int* __restrict__ ctx_len, int n_q,
                        float scale, int window, int splits, float* __restrict__ part_o,
                        float* __restrict__ part_ml, int* status) {
  constexpr int kRow = D + 8;
  constexpr int kChunks = D / 8;                        // 16-byte chunks per key row
  constexpr int kGroupElems = 16 * kRow;                // one group of 16 rows
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [16][kRow]
  __nv_bfloat16* kv_s = q_s + kGroupElems;              // [4 warps][stages][K,V][16][kRow]

  pdl_trigger();
  pdl_wait();
  const int g = n_q / pa.n_kv;
  const int groups = (g + 15) / 16;
  const int kvh = blockIdx.x / groups, hg = blockIdx.x - kvh * groups;
  const int head0 = kvh * g + hg * 16, heads = min(16, g - hg * 16);
  const int split = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row_token = q_start[seq];
  const int ctx = ctx_len[seq];
  const int k_lo = window > 0 ? max(0, ctx - window) : 0;
  const int total = ctx - k_lo;
  const int chunk = ((total + splits - 1) / splits + kKeyTile - 1) / kKeyTile * kKeyTile;
  const int k_begin = k_lo + split * chunk, k_end = min(ctx, k_begin + chunk);
  const int n_groups = k_end > k_begin ? (k_end - k_begin + 15) / 16 : 0;

  if (n_groups == 0) {
    if (splits > 1) {
      for (int h = tid; h < heads; h += kThreads) {
        float* ml = part_ml + (((size_t)seq * n_q + head0 + h) * splits + split) * 2;
        ml[0] = -INFINITY;
        ml[1] = 0.f;
      }
    } else {
      for (int idx = tid; idx < heads * D; idx += kThreads)
        out[(size_t)row_token * out_stride + (size_t)head0 * D + idx] = __float2bfloat16_rn(0.f);
    }
    return;
  }

  for (int idx = tid; idx < 16 * kChunks; idx += kThreads) {
    const int r = idx / kChunks, ch = idx - r * kChunks;
    const bool ok = r < heads;
    const __nv_bfloat16* src =
        qkv + (size_t)row_token * row_stride + (size_t)(head0 + (ok ? r : 0)) * D + ch * 8;
    cp_async16(smem_u32(q_s + r * kRow + ch * 8), src, ok);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  DecodeWarp<D, NT> dw;
  dw.init();
  dw.load_q(q_s, lane);

  __nv_bfloat16* my_s = kv_s + (size_t)warp * kDecodeStages * 2 * kGroupElems;
  // Requests keys/values of group `grp` (16 keys from k_begin + 16*grp) into stage `st`.
  auto issue = [&](int grp, int st) {
    if (grp < n_groups) {
      long long src = -1;
      if (lane < 16) {
        const int kj = k_begin + grp * 16 + lane;
        if (kj < k_end) {
          const int blk = kj / pa.page_tokens;
          const int page = blk < pa.table_width ? pa.block_table[(size_t)seq * pa.table_width + blk] : -1;
          if (page < 0 || page >= pa.num_pages) set_status(status, kBadPage, row_token, page, kj);
          else src = (((long long)page * pa.n_kv + kvh) * pa.page_tokens + (kj % pa.page_tokens)) * D;
        }
      }
      __nv_bfloat16* k_dst = my_s + (size_t)st * 2 * kGroupElems;
      __nv_bfloat16* v_dst = k_dst + kGroupElems;
      for (int idx = lane; idx < 16 * kChunks; idx += 32) {
        const int r = idx / kChunks, ch = idx - r * kChunks;
        const long long rs = __shfl_sync(0xffffffffu, src, r);
        const bool ok = rs >= 0;
        const long long off = ok ? rs + ch * 8 : 0;
        cp_async16(smem_u32(k_dst + r * kRow + ch * 8), pa.k_pool + off, ok);
        cp_async16(smem_u32(v_dst + r * kRow + ch * 8), pa.v_pool + off, ok);
      }
    }
    cp_async_commit();          // always: keeps the group count the same in every iteration
  };

  const float sl2 = scale * kLog2e;

#pragma unroll
  for (int s0 = 0; s0 < kDecodeStages - 1; ++s0) issue(warp + 4 * s0, s0);
  int it = 0;
  for (int grp = warp; grp < n_groups; grp += 4, ++it) {
    issue(grp + 4 * (kDecodeStages - 1), (it + kDecodeStages - 1) % kDecodeStages);
    cp_async_wait<kDecodeStages - 1>();
    __syncwarp();
    const __nv_bfloat16* k_s = my_s + (size_t)(it % kDecodeStages) * 2 * kGroupElems;
    const __nv_bfloat16* v_s = k_s + kGroupElems;
    const int key0 = k_begin + grp * 16;
    dw.group(k_s, v_s, key0, k_end, sl2, lane);
    __syncwarp();      // the stage is refilled by the next iteration's request
  }
  cp_async_wait<0>();
  __syncthreads();     // every warp is done with its stages: the space becomes the merge buffer

  float* mo = reinterpret_cast<float*>(kv_s);          // [4 warps][16 rows][D]
  float* mml = mo + 4 * 16 * D;                        // [4][16][2]
  dw.stash(mo, mml, warp, lane);
  __syncthreads();
  for (int idx = tid; idx < heads * D; idx += kThreads) {
    const int r = idx / D, c = idx - r * D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, mml[(w * 16 + r) * 2]);
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = mml[(w * 16 + r) * 2];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - m);
      l += f * mml[(w * 16 + r) * 2 + 1];
      o += f * mo[(size_t)(w * 16 + r) * D + c];
    }
    if (splits > 1) {
      const size_t p = ((size_t)seq * n_q + head0 + r) * splits + split;
      part_o[p * D + c] = o;
      if (c == 0) {
        part_ml[p * 2] = m;
        part_ml[p * 2 + 1] = l;
      }
    } else {
      out[(size_t)row_token * out_stride + (size_t)(head0 + r) * D + c] =
          __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    }
  }
}

// Merge of the split partials: global maximum, rescaled sums, weighted numerators / global
// sum (crates/leone-cuda/cuda/ie_cuda.cu:4769-4812).  grid = (n_q, sequences), D threads... any.
__global__ void attention_merge_kernel(const float* __restrict__ part_o,
                                       const float* __restrict__ part_ml,
                                       __nv_bfloat16* __restrict__ out, int out_stride,
                                       const int* __restrict__ q_start, int n_q, int d, int splits) {
  pdl_trigger();
  pdl_wait();
  const int head = blockIdx.x, seq = blockIdx.y;
  const size_t base = ((size_t)seq * n_q + head) * splits;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[(base + s) * 2]);
  float l = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(base + s) * 2];
    if (ms != -INFINITY) l += exp2f(ms - m) * part_ml[(base + s) * 2 + 1];
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  __nv_bfloat16* dst = out + (size_t)q_start[seq] * out_stride + (size_t)head * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = part_ml[(base + s) * 2];
      if (ms != -INFINITY) o += exp2f(ms - m) * part_o[(base + s) * d + c];
    }
    dst[c] = __float2bfloat16_rn(o * inv);
  }
}

// ------------------------------------------------------------------------------------
// Decode with the splits of one (sequence, KV head group) as a thread-block cluster.
// grid = (n_kv * head groups, splits, sequences), cluster = (1, splits, 1), splits <= 8.
// The loop over the keys is the one above.  Each block then leaves its (max, sum,
// unnormalised output) in its own shared memory; after a cluster barrier the outputs are dealt
// to the blocks, each of which merges its share of all splits in split order through
// distributed shared memory (global maximum, rescaled sums, weighted numerators / global sum,
// crates/leone-cuda/cuda/ie_cuda.cu:4769-4812) and writes it.  No scratch in global memory, no
// merge kernel.
//
// Optionally (DecodeFuse) the step's q/k RMSNorm, rotary and cache write are done here instead
// of in a kernel of their own: the query rows are normed and rotated as they are loaded; the
// block whose key range holds the new position norms and rotates the new key, uses it and the
// new value in place of what the cache holds there, and (one block per KV head) writes both to
// the cache.  The arithmetic is that of qk_norm_rope_write_vec_kernel, operation for operation,
// so a key is the same bits whichever kernel wrote it.
// ------------------------------------------------------------------------------------
struct DecodeFuse {
  int enabled;              // 0: rows of qkv are final and the cache already holds the new token
  const float* q_w;         // [D] norm weights or null
  const float* k_w;
  float eps;
  const float2* rope;       // [max_positions][D / 2] (cos, sin) or null
  int max_positions;
  int write_cache;          // 0 for a layer that only reads another layer's cache
  int adjacent;             // rotation pairs are elements (2i, 2i + 1) instead of (i, i + D/2)
};

// One warp: RMSNorm (if w) and half-split rotary over the whole row (if rope_row) of D bf16
// values at src; the result goes to dst and, if not null, to dst2.  Lane l owns elements
// l*E .. l*E+E-1, E = D / 32.
template <int D>
__device__ __forceinline__ void norm_rope_row(const __nv_bfloat16* src, __nv_bfloat16* dst,
                                              __nv_bfloat16* dst2, const float* w, float eps,
                                              const float2* rope_row, int lane, bool adjacent) {
  constexpr int E = D / 32;
  static_assert(D % 64 == 0, "two elements per lane at least");
  float v[E], wv[E];
  float2 cs[E];
  const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(src + lane * E);
#pragma unroll
  for (int i = 0; i < E / 2; ++i) {
    const __nv_bfloat162 two = p2[i];
    v[2 * i] = __low2float(two);
    v[2 * i + 1] = __high2float(two);
  }
#pragma unroll
  for (int i = 0; i < E; ++i) {
    wv[i] = w != nullptr ? w[lane * E + i] : 1.f;
    const int pair = adjacent ? (lane * E) / 2 + (i >> 1) : (lane & 15) * E + i;
    cs[i] = rope_row != nullptr ? rope_row[pair] : make_float2(1.f, 0.f);
  }
  if (w != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < E; ++i) ss = fmaf(v[i], v[i], ss);
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)D + eps);
#pragma unroll
    for (int i = 0; i < E; ++i) v[i] = v[i] * wv[i] * inv;
  }
  if (rope_row != nullptr && adjacent) {             // both elements of a pair are this lane's own
#pragma unroll
    for (int i = 0; i < E; i += 2) {
      const float a = v[i], b = v[i + 1];
      v[i] = a * cs[i].x - b * cs[i].y;
      v[i + 1] = a * cs[i].y + b * cs[i].x;
    }
  } else if (rope_row != nullptr) {
    const bool upper = lane >= 16;
#pragma unroll
    for (int i = 0; i < E; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, v[i], 16);
      v[i] = upper ? other * cs[i].y + v[i] * cs[i].x : v[i] * cs[i].x - other * cs[i].y;
    }
  }
#pragma unroll
  for (int i = 0; i < E / 2; ++i) {
    const __nv_bfloat162 o2 = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    reinterpret_cast<__nv_bfloat162*>(dst + lane * E)[i] = o2;
    if (dst2 != nullptr) reinterpret_cast<__nv_bfloat162*>(dst2 + lane * E)[i] = o2;
  }
}

// Floats of the inbox's output part of the cluster kernel: up to 8 * NT heads of D outputs, each
// block's range rounded up to a multiple of 4.
template <int D, int NT> struct DecodeInbox { static constexpr int kFloats = 8 * NT * D + 4 * 8; };

template <int D, int NT, bool kFuse>
__global__ void __launch_bounds__(kThreads)
attention_decode_cluster_kernel(const __nv_bfloat16* __restrict__ qkv, int row_stride,
                                __nv_bfloat16* __restrict__ out, int out_stride, PagedArgs pa,
                                const int* __restrict__ q_start, const int* __restrict__ ctx_len,
                                int n_q, float scale, int window, int splits, DecodeFuse fz,
                                int* status) {
  constexpr int kRow = D + 8;
  constexpr int kChunks = D / 8;
  constexpr int kGroupElems = 16 * kRow;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* kv_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [4 warps][stages][K,V][16][kRow]
  __nv_bfloat16* new_s = kv_s + 4 * kDecodeStages * 2 * kGroupElems;  // the new token's key and value: [2][kRow]
  __nv_bfloat16* q_s = new_s + 2 * kRow;                               // [16][kRow]
  // The inbox for the other splits' partial results lies over q_s (dead once every warp holds
  // its query fragments) and runs to the end of the allocation.
  float* inbox_o = reinterpret_cast<float*>(q_s);                      // [splits][per]
  float* inbox_ml = inbox_o + DecodeInbox<D, NT>::kFloats;            // [splits][8 * NT rows][2]

  // What the step's earlier kernels write for this one is the qkv rows (and, unfused, the new
  // token's cache row).  The step's metadata and the cache rows of earlier positions are older
  // than the step, so the fused kernel reads them, and requests its first keys, before it
  // waits for its predecessor.
  pdl_trigger();
  if constexpr (!kFuse) pdl_wait();
  const int g = n_q / pa.n_kv;
  const int groups = (g + 15) / 16;
  const int kvh = blockIdx.x / groups, hg = blockIdx.x - kvh * groups;
  const int head0 = kvh * g + hg * 16, heads = min(16, g - hg * 16);
  const int split = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row_token = q_start[seq];
  const int ctx = ctx_len[seq];
  const int pos = ctx - 1;                              // the query's (and the new key's) position
  const int k_lo = window > 0 ? max(0, ctx - window) : 0;
  const int total = ctx - k_lo;
  const int chunk = ((total + splits - 1) / splits + kKeyTile - 1) / kKeyTile * kKeyTile;
  const int k_begin = k_lo + split * chunk, k_end = min(ctx, k_begin + chunk);
  const int n_groups = k_end > k_begin ? (k_end - k_begin + 15) / 16 : 0;
  // the group of the new token, if this block's range holds it and the cache does not yet
  const bool own_new = kFuse && pos >= k_begin && pos < k_end;
  const int new_grp = own_new ? (pos - k_begin) / 16 : -1;

  DecodeWarp<D, NT> dw;
  dw.init();

  if (n_groups > 0) {
    __nv_bfloat16* my_s = kv_s + (size_t)warp * kDecodeStages * 2 * kGroupElems;
    // Requests keys/values of group `grp` (16 keys from k_begin + 16*grp) into stage `st`.
    auto issue = [&](int grp, int st) {
      if (grp < n_groups) {
        long long src = -1;
        if (lane < 16) {
          const int kj = k_begin + grp * 16 + lane;
          if (kj < k_end && !(kFuse && kj == pos)) {      // the new token's row is filled in below
            const int blk = kj / pa.page_tokens;
            const int page = blk < pa.table_width ? pa.block_table[(size_t)seq * pa.table_width + blk] : -1;
            if (page < 0 || page >= pa.num_pages) set_status(status, kBadPage, row_token, page, kj);
            else src = (((long long)page * pa.n_kv + kvh) * pa.page_tokens + (kj % pa.page_tokens)) * D;
          }
        }
        __nv_bfloat16* k_dst = my_s + (size_t)st * 2 * kGroupElems;
        __nv_bfloat16* v_dst = k_dst + kGroupElems;
        for (int idx = lane; idx < 16 * kChunks; idx += 32) {
          const int r = idx / kChunks, ch = idx - r * kChunks;
          const long long rs = __shfl_sync(0xffffffffu, src, r);
          const bool ok = rs >= 0;
          const long long off = ok ? rs + ch * 8 : 0;
          cp_async16(smem_u32(k_dst + r * kRow + ch * 8), pa.k_pool + off, ok);
          cp_async16(smem_u32(v_dst + r * kRow + ch * 8), pa.v_pool + off, ok);
        }
      }
      cp_async_commit();          // always: keeps the group count the same in every iteration
    };
    // the keys first: nothing of them depends on the query
#pragma unroll
    for (int s0 = 0; s0 < kDecodeStages - 1; ++s0) issue(warp + 4 * s0, s0);
    if constexpr (kFuse) pdl_wait();

    // the query rows (and the new key and value) while those copies are in flight
    const __nv_bfloat16* tok = qkv + (size_t)row_token * row_stride;
    if constexpr (kFuse) {
      const float2* rope_row = nullptr;
      if (fz.rope != nullptr) {
        if (pos < 0 || pos >= fz.max_positions) {
          if (tid == 0) set_status(status, kBadPosition, row_token, pos);
        } else {
          rope_row = fz.rope + (size_t)pos * (D / 2);
        }
      }
      for (int r = warp; r < 16 + (own_new ? 2 : 0); r += 4) {
        if (r < heads) {
          norm_rope_row<D>(tok + (size_t)(head0 + r) * D, q_s + r * kRow, nullptr, fz.q_w, fz.eps, rope_row, lane,
                           fz.adjacent != 0);
        } else if (r < 16) {
          for (int c = lane; c < kRow; c += 32) q_s[r * kRow + c] = __float2bfloat16_rn(0.f);
        } else {
          // r == 16: the new key, normed and rotated; r == 17: the new value as it is
          const bool is_k = r == 16;
          __nv_bfloat16* cache_row = nullptr;
          if (hg == 0 && fz.write_cache) {
            const int blk = pos / pa.page_tokens;
            const int page = blk < pa.table_width ? pa.block_table[(size_t)seq * pa.table_width + blk] : -1;
            if (page < 0 || page >= pa.num_pages) {
              if (lane == 0) set_status(status, kBadPage, row_token, page, pos);
            } else {
              const size_t off = (((size_t)page * pa.n_kv + kvh) * pa.page_tokens + (pos % pa.page_tokens)) * D;
              cache_row = const_cast<__nv_bfloat16*>(is_k ? pa.k_pool : pa.v_pool) + off;
            }
          }
          const __nv_bfloat16* src = tok + (size_t)(n_q + (is_k ? 0 : pa.n_kv) + kvh) * D;
          norm_rope_row<D>(src, new_s + (r - 16) * kRow, cache_row, is_k ? fz.k_w : nullptr, fz.eps,
                           is_k ? rope_row : nullptr, lane, fz.adjacent != 0);
        }
      }
    } else {
      for (int idx = tid; idx < 16 * kChunks; idx += kThreads) {
        const int r = idx / kChunks, ch = idx - r * kChunks;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < heads) v = *reinterpret_cast<const uint4*>(tok + (size_t)(head0 + r) * D + ch * 8);
        *reinterpret_cast<uint4*>(q_s + r * kRow + ch * 8) = v;
      }
    }
    __syncthreads();
    dw.load_q(q_s, lane);
    if (splits > 1) cluster_arrive_release();      // q_s may now receive the other blocks' partials
    const float sl2 = scale * kLog2e;
    int it = 0;
    for (int grp = warp; grp < n_groups; grp += 4, ++it) {
      issue(grp + 4 * (kDecodeStages - 1), (it + kDecodeStages - 1) % kDecodeStages);
      cp_async_wait<kDecodeStages - 1>();
      __syncwarp();
      __nv_bfloat16* k_s = my_s + (size_t)(it % kDecodeStages) * 2 * kGroupElems;
      __nv_bfloat16* v_s = k_s + kGroupElems;
      const int key0 = k_begin + grp * 16;
      if (kFuse && grp == new_grp) {
        // the new token: its key and value come from this step's projections, not from the cache
        const int rp = pos - key0;
        for (int c = lane; c < D / 2; c += 32) {
          reinterpret_cast<uint32_t*>(k_s + rp * kRow)[c] = reinterpret_cast<const uint32_t*>(new_s)[c];
          reinterpret_cast<uint32_t*>(v_s + rp * kRow)[c] = reinterpret_cast<const uint32_t*>(new_s + kRow)[c];
        }
        __syncwarp();
      }
      dw.group(k_s, v_s, key0, k_end, sl2, lane);
      __syncwarp();      // the stage is refilled by the next iteration's request
    }
    cp_async_wait<0>();
  } else {
    if constexpr (kFuse) pdl_wait();
    if (splits > 1) cluster_arrive_release();
  }
  __syncthreads();     // every warp is done with its stages: the space becomes the merge buffer

  // the four warps -> one (max, sum, output) per query row of the block
  float* mo = reinterpret_cast<float*>(kv_s);          // [4 warps][16 rows][D]
  float* mml = mo + 4 * 16 * D;                        // [4][16][2]
  dw.stash(mo, mml, warp, lane);
  __syncthreads();
  // With splits, block `s` finishes outputs [s * per, s * per + per) of the heads * D of this
  // (sequence, head group): every block stores its partial sums of that range, and its (max,
  // sum) per row, into block s's inbox, one cluster barrier follows, and each block finishes
  // its range from its own shared memory.
  const int n_out = heads * D;
  const int per = ((n_out + splits - 1) / splits + 3) / 4 * 4;
  constexpr int kRows = 8 * NT;
  const uint32_t in_o = smem_u32(inbox_o), in_ml = smem_u32(inbox_ml);
  if (splits > 1) cluster_wait_acquire();             // every block of the cluster holds its queries
  for (int idx = tid * 4; idx < n_out; idx += kThreads * 4) {
    const int r = idx / D, c = idx - r * D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, mml[(w * 16 + r) * 2]);
    float l = 0.f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = mml[(w * 16 + r) * 2];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - m);
      const float4 ow = *reinterpret_cast<const float4*>(mo + (size_t)(w * 16 + r) * D + c);
      l += f * mml[(w * 16 + r) * 2 + 1];
      o.x += f * ow.x;
      o.y += f * ow.y;
      o.z += f * ow.z;
      o.w += f * ow.w;
    }
    if (splits > 1) {
      const int owner = idx / per;
      cluster_st_f32x4(cluster_map(in_o + (uint32_t)(split * per + idx - owner * per) * 4, owner), o.x, o.y, o.z, o.w);
      if (c == 0) {
        for (int s2 = 0; s2 < splits; ++s2)
          cluster_st_f32x2(cluster_map(in_ml + (uint32_t)(split * kRows + r) * 8, s2), m, l);
      }
    } else {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(out + (size_t)row_token * out_stride +
                                                              (size_t)(head0 + r) * D + c);
      dst[0] = __floats2bfloat162_rn(o.x * inv, o.y * inv);
      dst[1] = __floats2bfloat162_rn(o.z * inv, o.w * inv);
    }
  }
  if (splits == 1) return;            // grid-uniform: a launch has clusters or it has none

  // Every thread of every block of the cluster comes here.
  cluster_arrive_release();
  cluster_wait_acquire();
  const int mine = min(n_out, split * per + per) - split * per;
  for (int j = tid * 2; j < mine; j += kThreads * 2) {
    const int idx = split * per + j;
    const int r = idx / D;
    float m = -INFINITY;
#pragma unroll
    for (int s2 = 0; s2 < 8; ++s2)
      if (s2 < splits) m = fmaxf(m, inbox_ml[(s2 * kRows + r) * 2]);
    float l = 0.f, o0 = 0.f, o1 = 0.f;
#pragma unroll
    for (int s2 = 0; s2 < 8; ++s2) {
      if (s2 < splits) {
        const float ms = inbox_ml[(s2 * kRows + r) * 2];
        if (ms != -INFINITY) {
          const float f = exp2f(ms - m);
          const float2 os = *reinterpret_cast<const float2*>(inbox_o + s2 * per + j);
          l += f * inbox_ml[(s2 * kRows + r) * 2 + 1];
          o0 += f * os.x;
          o1 += f * os.y;
        }
      }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    *reinterpret_cast<__nv_bfloat162*>(out + (size_t)row_token * out_stride + (size_t)head0 * D + idx) =
        __floats2bfloat162_rn(o0 * inv, o1 * inv);
  }
}

template <int D> constexpr int prefill_smem() {
  return (kRowsPerBlock + 4 * kKeyTile) * (D + 8) * 2 + 2 * kKeyTile * 8;
}
template <int D> constexpr int decode_smem() {
  const int tiles = (16 + 4 * kDecodeStages * 2 * 16) * (D + 8) * 2;
  const int merge = 16 * (D + 8) * 2 + 4 * 16 * D * 4 + 4 * 16 * 2 * 4;
  return tiles > merge ? tiles : merge;
}

template <int D>
int launch_prefill(const __nv_bfloat16* qkv, int row_stride, __nv_bfloat16* out, int out_stride,
                   const PagedArgs& pa, const int* q_start, const int* ctx_len, int n_seqs, int n_q,
                   int max_q_len, float scale, int window, int* status, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, prefill_smem<D>());
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int g = n_q / pa.n_kv;
  const int tq = kRowsPerBlock / g;
  dim3 grid((max_q_len + tq - 1) / tq, pa.n_kv, n_seqs);
  return launch_kernel(attention_prefill_kernel<D>, grid, dim3(kThreads), prefill_smem<D>(), stream, qkv,
                       row_stride, out, out_stride, pa, q_start, ctx_len, n_q, scale, window, status);
}

template <int D, int NT> constexpr int decode_cluster_smem() {
  const int rings = (4 * kDecodeStages * 2 * 16 + 2) * (D + 8) * 2;
  const int q_rows = 16 * (D + 8) * 2;
  const int inbox = (DecodeInbox<D, NT>::kFloats + 8 * 8 * NT * 2) * 4;
  return rings + (q_rows > inbox ? q_rows : inbox);
}

template <int D, int NT, bool kFuse>
int launch_decode_cluster_nt(const __nv_bfloat16* qkv, int row_stride, __nv_bfloat16* out, int out_stride,
                          const PagedArgs& pa, const int* q_start, const int* ctx_len, int n_seqs, int n_q,
                          float scale, int window, int splits, const DecodeFuse& fz, int* status,
                          cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_cluster_kernel<D, NT, kFuse>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, decode_cluster_smem<D, NT>());
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int g = n_q / pa.n_kv;
  dim3 grid(pa.n_kv * ((g + 15) / 16), splits, n_seqs);
  if (splits == 1)
    return launch_kernel(attention_decode_cluster_kernel<D, NT, kFuse>, grid, dim3(kThreads), decode_cluster_smem<D, NT>(),
                         stream, qkv, row_stride, out, out_stride, pa, q_start, ctx_len, n_q, scale, window,
                         splits, fz, status);
  return launch_kernel_cluster(attention_decode_cluster_kernel<D, NT, kFuse>, grid, dim3(kThreads),
                               decode_cluster_smem<D, NT>(), stream, dim3(1, splits, 1), qkv, row_stride, out,
                               out_stride, pa, q_start, ctx_len, n_q, scale, window, splits, fz, status);
}

// Up to 8 query heads per block take one tile of 8 heads (NT = 1), up to 16 take two.
template <int D, bool kFuse>
int launch_decode_cluster(const __nv_bfloat16* qkv, int row_stride, __nv_bfloat16* out, int out_stride,
                          const PagedArgs& pa, const int* q_start, const int* ctx_len, int n_seqs, int n_q,
                          float scale, int window, int splits, const DecodeFuse& fz, int* status,
                          cudaStream_t stream) {
  if (n_q / pa.n_kv <= 8)
    return launch_decode_cluster_nt<D, 1, kFuse>(qkv, row_stride, out, out_stride, pa, q_start, ctx_len, n_seqs,
                                                 n_q, scale, window, splits, fz, status, stream);
  return launch_decode_cluster_nt<D, 2, kFuse>(qkv, row_stride, out, out_stride, pa, q_start, ctx_len, n_seqs,
                                               n_q, scale, window, splits, fz, status, stream);
}

template <int D, int NT>
int launch_decode_nt(const __nv_bfloat16* qkv, int row_stride, __nv_bfloat16* out, int out_stride,
                  const PagedArgs& pa, const int* q_start, const int* ctx_len, int n_seqs, int n_q,
                  float scale, int window, int splits, float* part_o, float* part_ml, int* status,
                  cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<D, NT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, decode_smem<D>());
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int g = n_q / pa.n_kv;
  dim3 grid(pa.n_kv * ((g + 15) / 16), splits, n_seqs);
  int r = launch_kernel(attention_decode_kernel<D, NT>, grid, dim3(kThreads), decode_smem<D>(), stream, qkv,
                        row_stride, out, out_stride, pa, q_start, ctx_len, n_q, scale, window, splits,
                        part_o, part_ml, status);
  if (r != 0 || splits == 1) return r;
  dim3 mgrid(n_q, n_seqs);
  return launch_kernel(attention_merge_kernel, mgrid, dim3(D >= 64 ? 64 : 32), 0, stream,
                       (const float*)part_o, (const float*)part_ml, out, out_stride, q_start, n_q, D,
                       splits);
}

template <int D>
int launch_decode(const __nv_bfloat16* qkv, int row_stride, __nv_bfloat16* out, int out_stride,
                  const PagedArgs& pa, const int* q_start, const int* ctx_len, int n_seqs, int n_q,
                  float scale, int window, int splits, float* part_o, float* part_ml, int* status,
                  cudaStream_t stream) {
  if (n_q / pa.n_kv <= 8)
    return launch_decode_nt<D, 1>(qkv, row_stride, out, out_stride, pa, q_start, ctx_len, n_seqs, n_q, scale,
                                  window, splits, part_o, part_ml, status, stream);
  return launch_decode_nt<D, 2>(qkv, row_stride, out, out_stride, pa, q_start, ctx_len, n_seqs, n_q, scale,
                                window, splits, part_o, part_ml, status, stream);
}

}  // namespace tiled
}  // namespace leone

using namespace leone;
using namespace leone::tiled;

#define LEONE_DISPATCH_D(d, CALL)              \
  switch (d) {                                 \
    case 16: { constexpr int DD = 16; CALL; }  \
    case 32: { constexpr int DD = 32; CALL; }  \
    case 48: { constexpr int DD = 48; CALL; }  \
    case 64: { constexpr int DD = 64; CALL; }  \
    case 80: { constexpr int DD = 80; CALL; }  \
    case 96: { constexpr int DD = 96; CALL; }  \
    case 112: { constexpr int DD = 112; CALL; } \
    case 128: { constexpr int DD = 128; CALL; } \
    default: return kRefusedSize;              \
  }

static int check_common(int d, int n_q, int n_kv, int row_stride, int out_stride, const void* qkv,
                        const void* k_pool, const void* v_pool, int page_tokens, int table_width) {
  if (d <= 0 || d % 16 != 0 || d > 128) return kRefusedSize;
  if (n_q <= 0 || n_kv <= 0 || n_q % n_kv != 0) return kRefusedSize;
  if (page_tokens <= 0 || table_width <= 0) return kRefusedSize;
  if (row_stride % 8 != 0 || out_stride % 2 != 0) return kRefusedAlignment;
  if (((uintptr_t)qkv | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) return kRefusedAlignment;
  return 0;
}

// Prompt portions and mixed batches.  qkv: [tokens, row_stride] bf16 with the query heads first;
// out: [tokens, out_stride] bf16; q_start: [n_seqs+1]; ctx_len: [n_seqs] lengths after this step.
extern "C" int leone_attention_prefill(const void* qkv, int row_stride, void* out, int out_stride,
                                       const void* k_pool, const void* v_pool,
                                       const int* block_table, int table_width, const int* q_start,
                                       const int* ctx_len, int n_seqs, int max_q_len, int n_q,
                                       int n_kv, int d, float scale, int window, int page_tokens,
                                       int num_pages, int* status, cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return 0;
  int r = check_common(d, n_q, n_kv, row_stride, out_stride, qkv, k_pool, v_pool, page_tokens, table_width);
  if (r != 0) return r;
  if (n_q / n_kv > kRowsPerBlock || n_kv > 65535 || n_seqs > 65535) return kRefusedSize;
  PagedArgs pa{(const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, block_table, table_width,
               page_tokens, num_pages, n_kv};
  LEONE_DISPATCH_D(d, return launch_prefill<DD>((const __nv_bfloat16*)qkv, row_stride,
                                                (__nv_bfloat16*)out, out_stride, pa, q_start, ctx_len,
                                                n_seqs, n_q, max_q_len, scale, window, status, stream));
}

// Scratch floats a decode call with `splits` needs: part_o then part_ml, contiguous.
extern "C" long long leone_attention_decode_scratch(int n_seqs, int n_q, int d, int splits) {
  return splits > 1 ? (long long)n_seqs * n_q * splits * (d + 2) : 0;
}

// Decode steps: every sequence has exactly one query token (row q_start[seq]).
extern "C" int leone_attention_decode(const void* qkv, int row_stride, void* out, int out_stride,
                                      const void* k_pool, const void* v_pool, const int* block_table,
                                      int table_width, const int* q_start, const int* ctx_len,
                                      int n_seqs, int n_q, int n_kv, int d, float scale, int window,
                                      int page_tokens, int num_pages, int splits, float* scratch,
                                      int* status, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  int r = check_common(d, n_q, n_kv, row_stride, out_stride, qkv, k_pool, v_pool, page_tokens, table_width);
  if (r != 0) return r;
  if (splits < 1 || splits > 65535 || n_seqs > 65535) return kRefusedSize;
  if (splits > 1 && scratch == nullptr) return kRefusedSize;
  PagedArgs pa{(const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, block_table, table_width,
               page_tokens, num_pages, n_kv};
  float* part_o = scratch;
  float* part_ml = scratch ? scratch + (size_t)n_seqs * n_q * splits * d : nullptr;
  LEONE_DISPATCH_D(d, return launch_decode<DD>((const __nv_bfloat16*)qkv, row_stride,
                                               (__nv_bfloat16*)out, out_stride, pa, q_start, ctx_len,
                                               n_seqs, n_q, scale, window, splits, part_o, part_ml,
                                               status, stream));
}

// The same product with the splits of a (sequence, head group) as a thread-block cluster that
// merges through distributed shared memory: 1 <= splits <= 8, no scratch.  With `fuse` != 0 the
// rows of qkv are raw projections: the kernel applies the per-head RMSNorm (weights q_norm_w /
// k_norm_w, fp32 [d], or null for none) and the rotary table (`rope`: [max_positions][d/2]
// (cos, sin) fp32 over the whole head, or null; pairs (i, i + d/2), or (2i, 2i + 1) with
// `adjacent`) to the queries and to the new key at position
// ctx_len-1, uses the new key and value in place of what the cache holds there and, if
// `write_cache`, stores them into the pools.  fuse needs d of 64 or 128.
extern "C" int leone_attention_decode_cluster(const void* qkv, int row_stride, void* out, int out_stride,
                                              void* k_pool, void* v_pool, const int* block_table,
                                              int table_width, const int* q_start, const int* ctx_len,
                                              int n_seqs, int n_q, int n_kv, int d, float scale, int window,
                                              int page_tokens, int num_pages, int splits, int fuse,
                                              const float* q_norm_w, const float* k_norm_w, float eps,
                                              const float* rope, int max_positions, int write_cache,
                                              int adjacent, int* status, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  int r = check_common(d, n_q, n_kv, row_stride, out_stride, qkv, k_pool, v_pool, page_tokens, table_width);
  if (r != 0) return r;
  if (splits < 1 || splits > 8 || n_seqs > 65535) return kRefusedSize;
  if (fuse && d != 64 && d != 128) return kRefusedSize;
  PagedArgs pa{(const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, block_table, table_width,
               page_tokens, num_pages, n_kv};
  DecodeFuse fz{fuse ? 1 : 0, q_norm_w, k_norm_w, eps, reinterpret_cast<const float2*>(rope), max_positions,
                write_cache, adjacent};
  if (fuse) {
    if (d == 64)
      return launch_decode_cluster<64, true>((const __nv_bfloat16*)qkv, row_stride, (__nv_bfloat16*)out,
                                             out_stride, pa, q_start, ctx_len, n_seqs, n_q, scale, window,
                                             splits, fz, status, stream);
    return launch_decode_cluster<128, true>((const __nv_bfloat16*)qkv, row_stride, (__nv_bfloat16*)out,
                                            out_stride, pa, q_start, ctx_len, n_seqs, n_q, scale, window,
                                            splits, fz, status, stream);
  }
  LEONE_DISPATCH_D(d, return (launch_decode_cluster<DD, false>((const __nv_bfloat16*)qkv, row_stride,
                                                               (__nv_bfloat16*)out, out_stride, pa, q_start,
                                                               ctx_len, n_seqs, n_q, scale, window, splits,
                                                               fz, status, stream)));
}
