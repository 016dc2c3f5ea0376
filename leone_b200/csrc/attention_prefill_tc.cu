// Causal grouped-query attention for prompt portions on the 5th-generation tensor cores.
//
// Same formulas and interface as the mma.sync kernel for prompt portions in attention_tiled.cu
// (kv_head = q_head / (n_q / n_kv); score = (q.k) * scale; online softmax in fp32; output =
// numerator / sum; crates/leone/src/cpu.rs:2299-2421), for head sizes 64 and 128.  The
// reference's prompt path materialises the score matrix (crates/leone-cuda/cuda/ie_cuda.cu:
// 5123-5220); here scores live in tensor memory and never reach global memory.
//
// A block owns 128 query rows = (tokens of its tile) x (the g query heads of one KV head) and
// walks the keys in tiles of 128.  Per tile:
//   S[128 x 128]  = Q . K^T     tcgen05.mma, accumulator in tensor memory (columns 0..127)
//   softmax       four threads per row (one in each of four warps that share the row's lane of
//                 tensor memory), 32 columns each: tcgen05.ld, mask, row maximum (exchanged
//                 through shared memory), P = exp2(S - max) as bf16 into shared memory (an
//                 A operand), running sum
//   PV[128 x D]   = P . V       tcgen05.mma (V is the B operand in MN-major form: it is stored
//                 as it comes from the cache, one key per row), columns 128..128+D-1
//   O            += PV          the row's four threads own D/4 columns each: tcgen05.ld, added
//                 to their fp32 registers, which were rescaled when the maximum moved.
// Operand tiles are rows of 128 bytes with the 128-byte swizzle (16-byte chunk c of row r at
// chunk c ^ (r & 7)); a tile with 128 elements per row is two such halves, 16 KB apart.  Keys
// and values are gathered from the pages with 16-byte asynchronous copies that write this
// layout directly.
//
// The tile loop is software-pipelined so that the tensor core works under the softmax:
// S of tile t+1 is issued (into the second S buffer of tensor memory) before the softmax of
// tile t starts, and P.V of tile t runs while the next iteration loads and reduces S of tile
// t+1; its result is added to the registers in the middle of that iteration, just before P of
// tile t+1 is written.  Keys are copied two tiles ahead, values one tile ahead.  A warp of its
// own issues the MMAs: the softmax warps tell it through mbarriers when an operand tile has
// landed and a tensor-memory buffer is free, so they never wait for one thread's issue loop.
// Every wait is bounded; a wait that runs out sets the status word and the block leaves.
#include "tc_common.cuh"

namespace leone {
namespace tcattn {

using namespace leone::tc;

constexpr int kSplit = 4;         // threads per query row
constexpr int kRows = 128;        // query rows per block
constexpr int kThreads = kRows * kSplit;      // the softmax threads (16 warps); they also copy the tiles
constexpr int kBlockThreads = kThreads + 32;  // + one warp that issues the tensor-core work
constexpr int kKeys = 128;        // keys per tile
constexpr float kLog2e = 1.4426950408889634f;

struct PagedArgs {
  const __nv_bfloat16* k_pool;
  const __nv_bfloat16* v_pool;
  const int* block_table;
  int table_width;
  int page_tokens;
  int num_pages;
  int n_kv;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;     // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// 2^x by the special-function unit (x <= 0 here; -inf gives 0).
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Byte offset of 16-byte chunk `chunk` (8 elements) of row `row` in a tile of rows of
// D elements stored as D/64 swizzled halves of [128 rows x 128 bytes].
__device__ __forceinline__ uint32_t swizzled(int row, int chunk) {
  return (uint32_t)((chunk >> 3) * (128 * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// Descriptor of an MN-major bf16 operand stored as rows of 128 bytes, one row per K index,
// 64 MN elements per row, 128-byte swizzle: 8-row groups (along K) are 1024 bytes apart and
// the next 64 MN elements are `mn_stride` bytes further.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t smem_addr, uint32_t mn_stride) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((mn_stride >> 4) & 0x3FFFu) << 16;   // leading byte offset: between 64-element groups along MN
  d |= (uint64_t)(1024u >> 4) << 32;                   // stride byte offset: between 8-row groups along K
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// bf16 x bf16 -> fp32, A K-major, B MN-major.
__host__ __device__ constexpr uint32_t instr_desc_bf16_b_mn(int m, int n) {
  return instr_desc_bf16(m, n) | (1u << 16);
}

// Where the keys [tile_start, tile_start + 128) of one sequence and KV head lie in the pools,
// in two steps so that the block table's latency can pass under other work: tile_page() reads
// this thread's key's page number (-1: no key here, -2: outside the table), tile_rows() turns
// it into an element offset in row_src[0..127] (-1 for none).  Rows before k_first (keys a
// window has passed, whose pages may already be given back) and rows at or past k_end have
// none.  The caller puts a block barrier between tile_rows and copy_tile.
__device__ __forceinline__ int tile_page(const PagedArgs& pa, int seq, int tile_start, int k_first, int k_end) {
  const int tid = threadIdx.x;
  int page = -1;
  if (tid < kKeys) {
    const int kj = tile_start + tid;
    if (kj < k_end && kj >= k_first) {
      const int blk = kj / pa.page_tokens;
      page = blk < pa.table_width ? pa.block_table[(size_t)seq * pa.table_width + blk] : -2;
      if (page < 0) page = -2;
    }
  }
  return page;
}
template <int D>
__device__ __forceinline__ void tile_rows(long long* row_src, int page, const PagedArgs& pa, int kvh,
                                          int tile_start, int* status, int token_row) {
  const int tid = threadIdx.x;
  if (tid < kKeys) {
    const int kj = tile_start + tid;
    long long src = -1;
    if (page >= pa.num_pages || page == -2) {
      set_status(status, kBadPage, token_row, page, kj);
    } else if (page >= 0) {
      src = (((long long)page * pa.n_kv + kvh) * pa.page_tokens + (kj % pa.page_tokens)) * D;
    }
    row_src[tid] = src;
  }
}

// Copies the 128 rows whose offsets tile_rows gave from `pool` into the swizzled tile at dst
// (rows without a source are zero-filled) and commits the copies as one group.
template <int D>
__device__ __forceinline__ void copy_tile(uint32_t dst, const long long* row_src, const __nv_bfloat16* pool,
                                          bool any) {
  constexpr int kChunks = D / 8;
  constexpr int kStep = kThreads / kChunks;             // rows between a thread's copies
  static_assert(kStep % 8 == 0 && kKeys % kStep == 0, "a thread's rows share their swizzle phase");
  if (any) {
    // a thread copies the same 16-byte chunk of rows r0, r0 + kStep, ..: one address to start from
    const int ch = threadIdx.x % kChunks, r0 = threadIdx.x / kChunks;
    const uint32_t d0 = dst + swizzled(r0, ch);
    const __nv_bfloat16* p0 = pool + ch * 8;
#pragma unroll
    for (int i = 0; i < kKeys / kStep; ++i) {
      const long long src = row_src[r0 + i * kStep];
      const bool ok = src >= 0;
      cp_async16(d0 + i * kStep * 128, ok ? p0 + src : pool, ok);
    }
  }
  cp_async_commit();      // always: the number of groups in flight is the same in every iteration
}

template <int D> constexpr int smem_bytes() {
  // Q, two K and two V tiles, P, row sources [2][128], barriers; 1024 for alignment
  return kRows * D * 2 + 2 * 2 * kKeys * D * 2 + kRows * kKeys * 2 + 2 * kKeys * 8 + 64 + 1024;
}

template <int D>
__global__ void __launch_bounds__(kBlockThreads)
attention_prefill_tc_kernel(const __nv_bfloat16* __restrict__ qkv, int row_stride,
                            __nv_bfloat16* __restrict__ out, int out_stride, PagedArgs pa,
                            const int* __restrict__ q_start, const int* __restrict__ ctx_len, int n_q,
                            float scale, int window, int* status) {
  constexpr int kTileBytes = kKeys * D * 2;             // one K or V tile; the Q tile has the same size
  constexpr int kTmemCols = 512;                        // S: two buffers at columns 0 and 128; PV at 256
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - raw);
  const uint32_t q_t = base;
  const uint32_t k_t = q_t + kTileBytes;                // [2] key tiles
  const uint32_t v_t = k_t + 2 * kTileBytes;            // [2] value tiles
  const uint32_t p_t = v_t + 2 * kTileBytes;
  long long* row_src = reinterpret_cast<long long*>(aligned + 5 * kTileBytes + kRows * kKeys * 2);   // [2][128]
  // bar_s (one per S buffer) and bar_o: the tensor core's results; bar_k and bar_p: the softmax
  // warps' go-ahead for S of a tile and for P.V of a tile (one arrival per warp)
  const uint32_t bar_s = smem_u32(row_src + 2 * kKeys), bar_o = bar_s + 16, bar_k = bar_s + 24, bar_p = bar_s + 32;
  __shared__ uint32_t tmem_holder;
  __shared__ int gave_up;

  __shared__ float max_s[2][kSplit][kRows];             // the row maximum's parts (two tiles' worth), then the row sum's
  const int tid = threadIdx.x, warp = tid >> 5;
  const int row = tid & (kRows - 1), part = tid >> 7;   // this thread: row, and which quarter of the columns
  if (tid == 0) {
    gave_up = 0;
    mbar_init(bar_s, 1);
    mbar_init(bar_s + 8, 1);
    mbar_init(bar_o, 1);
    mbar_init(bar_k, kThreads / 32);
    mbar_init(bar_p, kThreads / 32);
    mbar_fence_init();
  }
  constexpr int kMmaWarp = kThreads / 32;
  if (warp == kMmaWarp) tmem_alloc(smem_u32(&tmem_holder), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_holder;
  volatile int* giveup = &gave_up;
  pdl_trigger();
  pdl_wait();

  // blocks in launch order: the latest query tile (most keys) of every KV head first, so that
  // the long blocks start early and the short ones fill the end
  const int seq = blockIdx.z, kvh = blockIdx.x % pa.n_kv;
  const int qt = gridDim.x / pa.n_kv - 1 - blockIdx.x / pa.n_kv;
  const int g = n_q / pa.n_kv;
  const int tq = kRows / g;                             // tokens per tile
  const int q0 = q_start[seq], q_len = q_start[seq + 1] - q0;
  const int tok0 = qt * tq;
  const bool live = tok0 < q_len;                       // block-uniform
  if (live) {
    const int ctx = ctx_len[seq], start = ctx - q_len;
    const int tok1 = min(q_len, tok0 + tq);
    const int k_hi = start + tok1;                      // one past the last key any row reads
    int k_lo = 0;
    if (window > 0) k_lo = max(0, start + tok0 - window + 1);
    const int tile0 = (k_lo / kKeys) * kKeys;
    const int n_tiles = (k_hi - tile0 + kKeys - 1) / kKeys;
    constexpr uint32_t idesc_s = instr_desc_bf16(kRows, kKeys);
    constexpr uint32_t idesc_o = instr_desc_bf16_b_mn(kRows, D);

    if (warp == kMmaWarp) {
      // ---------------- the warp that issues the tensor-core work ----------------
      // Order of the go-aheads: K(0); then per tile t: K(t+1), P(t).  One thread issues.
      if ((tid & 31) == 0) {
        auto issue_s = [&](int t) {     // S(t) = Q . K(t)^T into S buffer t & 1
          tc_fence_after();
          const uint32_t k_s = k_t + (t & 1) * kTileBytes;
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            // 16 elements further along a 128-byte row: +32 bytes; past 64 elements: the next half
            const uint32_t off = (ks >> 2) * (128 * 128) + (ks & 3) * 32;
            umma_bf16(tmem_base + (t & 1) * kKeys, smem_desc_sw128(q_t + off), smem_desc_sw128(k_s + off),
                      idesc_s, ks > 0 ? 1u : 0u);
          }
          umma_commit(bar_s + 8 * (t & 1));
        };
        bool ok = mbar_wait(bar_k, 0, giveup);
        if (ok) issue_s(0);
        for (int t = 0; t < n_tiles && ok; ++t) {
          if (t + 1 < n_tiles) {
            ok = mbar_wait(bar_k, (t + 1) & 1, giveup);
            if (!ok) break;
            issue_s(t + 1);
          }
          ok = mbar_wait(bar_p, t & 1, giveup);
          if (!ok) break;
          tc_fence_after();
          const uint32_t v_s = v_t + (t & 1) * kTileBytes;
#pragma unroll
          for (int ks = 0; ks < kKeys / 16; ++ks) {
            // A = P: 16 keys further along a row; B = V: 16 keys = 16 rows = 2048 bytes further
            const uint32_t a_off = (ks >> 2) * (128 * 128) + (ks & 3) * 32;
            umma_bf16(tmem_base + 2 * kKeys, smem_desc_sw128(p_t + a_off),
                      smem_desc_mn_sw128(v_s + ks * 2048, 128 * 128), idesc_o, ks > 0 ? 1u : 0u);
          }
          umma_commit(bar_o);
        }
      }
    } else {
      // ---------------- the softmax warps ----------------
      const int lane = tid & 31;
      // the tile's query rows: row r = (token r / g, head r % g)
      for (int idx = tid; idx < kRows * (D / 8); idx += kThreads) {
        const int r = idx / (D / 8), ch = idx - r * (D / 8);
        const int tl = r / g, hh = r - tl * g;
        const int token = tok0 + tl;
        const bool ok = tl < tq && token < tok1;
        const __nv_bfloat16* src =
            qkv + (size_t)(q0 + (ok ? token : 0)) * row_stride + (size_t)(kvh * g + hh) * D + ch * 8;
        cp_async16(q_t + swizzled(r, ch), src, ok);
      }
      auto page_of = [&](int t) {          // this thread's key's page in tile t (read ahead of its use)
        return t < n_tiles ? tile_page(pa, seq, tile0 + t * kKeys, k_lo, k_hi) : -1;
      };
      auto rows_of = [&](int t, int page) {          // row sources of tile t into buffer t & 1
        if (t < n_tiles)
          tile_rows<D>(row_src + (t & 1) * kKeys, page, pa, kvh, tile0 + t * kKeys, status, q0 + tok0);
      };
      auto copy_k = [&](int t) {
        copy_tile<D>(k_t + (t & 1) * kTileBytes, row_src + (t & 1) * kKeys, pa.k_pool, t < n_tiles);
      };
      auto copy_v = [&](int t) {
        copy_tile<D>(v_t + (t & 1) * kTileBytes, row_src + (t & 1) * kKeys, pa.v_pool, t < n_tiles);
      };
      // one arrival per warp at a go-ahead barrier, after the warp's copies and tensor-memory
      // reads are ordered before it
      auto go_ahead = [&](uint32_t bar) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar);
      };
      rows_of(0, page_of(0));
      rows_of(1, page_of(1));
      int page_ahead = page_of(2);          // consumed in the first iteration
      named_barrier_sync(1, kThreads);
      copy_k(0);                           // group: Q and K(0)
      copy_k(1);                           // group: K(1)
      copy_v(0);                           // group: V(0)

      // this thread's row and its share of the columns
      constexpr int kSC = kKeys / kSplit;                 // score columns per thread
      constexpr int kOC = D / kSplit;                     // output columns per thread
      const int my_tl = row / g;
      const int my_pos = (my_tl < tq && tok0 + my_tl < tok1) ? start + tok0 + my_tl : -1;   // -1: row unused
      // the block's rows read keys up to their own position: a tile that ends at or before the
      // first row's position (and lies inside every row's window) needs no masking
      const int first_pos = start + tok0, last_pos = start + tok1 - 1;
      float m_run = -INFINITY, l_run = 0.f;
      float o_acc[kOC];
#pragma unroll
      for (int i = 0; i < kOC; ++i) o_acc[i] = 0.f;
      const float sl2 = scale * kLog2e;
      const uint32_t t_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);   // this warp's lanes
      const int col0 = part * kSC;
      // A wait that runs out leaves ok_all false; the thread still walks the loop (every later
      // wait returns at once), so that the named barriers below keep their counts.
      bool ok_all = true;

      cp_async_wait<2>();                  // Q and K(0) have landed
      go_ahead(bar_k);                     // S(0) may be issued

      for (int t = 0; t < n_tiles; ++t) {
        const int tile_start = tile0 + t * kKeys;
        // (1) S(t) is complete, so K(t)'s tile is free for K(t+2); K(t+1) has landed: S(t+1) may go
        if (ok_all && !mbar_wait(bar_s + 8 * (t & 1), (t >> 1) & 1, giveup)) ok_all = false;
        tc_fence_after();
        rows_of(t + 2, page_ahead);
        page_ahead = page_of(t + 3);
        cp_async_wait<1>();                // groups so far: .. K(t+1), V(t): all but the newest have landed
        if (t + 1 < n_tiles) go_ahead(bar_k);

        // (2) this thread's quarter of its row of S(t)
        float sc[kSC];
#pragma unroll
        for (int c = 0; c < kSC; c += 16) tmem_ld16(t_row + (t & 1) * kKeys + col0 + c, sc + c);
        const bool all_visible = tile_start + kKeys - 1 <= first_pos &&
                                 (window <= 0 || tile_start > last_pos - window) && my_pos >= 0;
        // the maximum of the raw scores; the scale (positive) goes into the exponent's multiply-add
        float tile_max = -INFINITY;
        if (all_visible) {
#pragma unroll
          for (int j = 0; j < kSC; ++j) tile_max = fmaxf(tile_max, sc[j]);
        } else {
#pragma unroll
          for (int j = 0; j < kSC; ++j) {
            const int kj = tile_start + col0 + j;
            const bool keep = my_pos >= 0 && kj <= my_pos && (window <= 0 || kj > my_pos - window);
            sc[j] = keep ? sc[j] : -INFINITY;
            tile_max = fmaxf(tile_max, sc[j]);
          }
        }
        tile_max *= sl2;                   // (-inf stays -inf)
        max_s[t & 1][part][row] = tile_max;
        named_barrier_sync(1, kThreads);   // the row maximum's parts, and the row sources of tile t+2
        copy_k(t + 2);
#pragma unroll
        for (int q = 0; q < kSplit; ++q) tile_max = fmaxf(tile_max, max_s[t & 1][q][row]);
        const float m_new = fmaxf(m_run, tile_max);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        const float alpha = m_run == -INFINITY ? 0.f : ex2(m_run - m_use);
        m_run = m_new;
        l_run *= alpha;

        // (3) P(t-1) . V(t-1) is complete: add it (still at the old maximum's scale), then its
        // value tile is free for V(t+1) and P's tile for P(t)
        if (t > 0) {
          if (ok_all && !mbar_wait(bar_o, (t - 1) & 1, giveup)) ok_all = false;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < kOC; c += 16) {
            float pv[16];
            tmem_ld16(t_row + 2 * kKeys + part * kOC + c, pv);
#pragma unroll
            for (int j = 0; j < 16; ++j) o_acc[c + j] += pv[j];
          }
        }
        copy_v(t + 1);
        if (alpha != 1.f) {
#pragma unroll
          for (int i = 0; i < kOC; ++i) o_acc[i] *= alpha;
        }
#pragma unroll
        for (int c = 0; c < kSC / 8; ++c) {
          uint32_t packed[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float p0 = ex2(fmaf(sc[c * 8 + 2 * j], sl2, -m_use)), p1 = ex2(fmaf(sc[c * 8 + 2 * j + 1], sl2, -m_use));
            l_run += p0 + p1;
            __nv_bfloat162 v2 = __floats2bfloat162_rn(p0, p1);
            packed[j] = *reinterpret_cast<uint32_t*>(&v2);
          }
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(p_t + swizzled(row, col0 / 8 + c)),
                       "r"(packed[0]), "r"(packed[1]), "r"(packed[2]), "r"(packed[3])
                       : "memory");
        }
        // (4) V(t) has landed (groups so far: .. V(t), K(t+2), V(t+1)): P(t) . V(t) may go
        cp_async_wait<2>();
        go_ahead(bar_p);
      }
      // the last tile's P . V
      if (n_tiles > 0) {
        if (ok_all && !mbar_wait(bar_o, (n_tiles - 1) & 1, giveup)) ok_all = false;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < kOC; c += 16) {
          float pv[16];
          tmem_ld16(t_row + 2 * kKeys + part * kOC + c, pv);
#pragma unroll
          for (int j = 0; j < 16; ++j) o_acc[c + j] += pv[j];
        }
      }

      // the row's sum from its four parts, then every thread writes its columns
      named_barrier_sync(1, kThreads);
      max_s[0][part][row] = l_run;
      named_barrier_sync(1, kThreads);
      float l_row = 0.f;
#pragma unroll
      for (int q = 0; q < kSplit; ++q) l_row += max_s[0][q][row];
      if (ok_all && my_pos >= 0) {
        const int hh = row - my_tl * g;
        const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
        __nv_bfloat16* dst = out + (size_t)(q0 + tok0 + my_tl) * out_stride + (size_t)(kvh * g + hh) * D + part * kOC;
#pragma unroll
        for (int c = 0; c < kOC; c += 8) {
          uint32_t packed[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 v2 = __floats2bfloat162_rn(o_acc[c + 2 * j] * inv, o_acc[c + 2 * j + 1] * inv);
            packed[j] = *reinterpret_cast<uint32_t*>(&v2);
          }
          *reinterpret_cast<uint4*>(dst + c) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
      }
      cp_async_wait<0>();
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (gave_up && tid == 0) set_status(status, kWaitTimeout, blockIdx.x, 1);
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int D>
int launch(const __nv_bfloat16* qkv, int row_stride, __nv_bfloat16* out, int out_stride, const PagedArgs& pa,
           const int* q_start, const int* ctx_len, int n_seqs, int n_q, int max_q_len, float scale, int window,
           int* status, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<D>());
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int g = n_q / pa.n_kv;
  const int tq = kRows / g;
  dim3 grid(((max_q_len + tq - 1) / tq) * pa.n_kv, 1, n_seqs);
  return launch_kernel(attention_prefill_tc_kernel<D>, grid, dim3(kBlockThreads), smem_bytes<D>(), stream, qkv,
                       row_stride, out, out_stride, pa, q_start, ctx_len, n_q, scale, window, status);
}

}  // namespace tcattn
}  // namespace leone

using namespace leone;

// Prompt portions and mixed batches on tcgen05; arguments as leone_attention_prefill.  Head size
// 64 or 128, up to 128 query heads per KV head, 16-byte aligned rows.
extern "C" int leone_attention_prefill_tc(const void* qkv, int row_stride, void* out, int out_stride,
                                          const void* k_pool, const void* v_pool, const int* block_table,
                                          int table_width, const int* q_start, const int* ctx_len, int n_seqs,
                                          int max_q_len, int n_q, int n_kv, int d, float scale, int window,
                                          int page_tokens, int num_pages, int* status, cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return 0;
  if (d != 64 && d != 128) return kRefusedSize;
  if (n_q <= 0 || n_kv <= 0 || n_q % n_kv != 0 || n_q / n_kv > tcattn::kRows) return kRefusedSize;
  if (page_tokens <= 0 || table_width <= 0 || n_seqs > 65535) return kRefusedSize;
  if (row_stride % 8 != 0 || out_stride % 8 != 0) return kRefusedAlignment;
  if (((uintptr_t)qkv | (uintptr_t)out | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) return kRefusedAlignment;
  tcattn::PagedArgs pa{(const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, block_table, table_width,
                       page_tokens, num_pages, n_kv};
  if (d == 64)
    return tcattn::launch<64>((const __nv_bfloat16*)qkv, row_stride, (__nv_bfloat16*)out, out_stride, pa, q_start,
                              ctx_len, n_seqs, n_q, max_q_len, scale, window, status, stream);
  return tcattn::launch<128>((const __nv_bfloat16*)qkv, row_stride, (__nv_bfloat16*)out, out_stride, pa, q_start,
                             ctx_len, n_seqs, n_q, max_q_len, scale, window, status, stream);
}
