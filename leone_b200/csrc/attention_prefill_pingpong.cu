// Causal grouped-query attention for prompt portions on the 5th-generation tensor cores:
// two query tiles per block in ping-pong, probabilities kept in tensor memory.
//
// Same formulas and interface as the other prompt kernels (kv_head = q_head / (n_q / n_kv);
// score = (q.k) * scale; online softmax in fp32; output = numerator / sum;
// crates/leone/src/cpu.rs:2299-2421), for head sizes 64 and 128.  The reference's prompt path
// materialises the score matrix (crates/leone-cuda/cuda/ie_cuda.cu:5123-5220); here scores and
// probabilities live in tensor memory and never reach shared or global memory.
//
// A block owns two query tiles of 128 rows each, row = (token, one of the g query heads of the
// block's KV head), and walks the keys in tiles of 128 that both query tiles share.  Per query
// tile j and key tile t:
//   S_j = Q_j . K(t)^T      tcgen05.mma, operands in shared memory, accumulator in tensor memory
//   softmax                 two threads per row, 64 columns each (in two warps that reach the
//                           row's lane of tensor memory): the row maximum over the tile (the
//                           halves meet through shared memory), P = exp2(S * scale - max)
//                           rounded to bf16 and stored back into tensor memory over columns
//                           of S that the same thread has already read
//   O_j += P_j . V(t)       tcgen05.mma with the A operand (P) read from tensor memory, V the
//                           B operand in MN-major form (as the cache stores it: a key per row),
//                           accumulated in tensor memory across all key tiles
// While the eight softmax warps of one query tile work, the tensor core runs the other query
// tile's products: the issue order is PV_0(t), S_0(t+1), PV_1(t), S_1(t+1).  (Letting all
// sixteen warps work on one tile at a time was measured slower: the fixed latencies of a step,
// the loads from tensor memory and the barrier where the maxima meet, then lie end to end
// instead of under the other tile's arithmetic.)  The running
// maximum only moves when the tile's maximum exceeds it by more than 8 (in the exponent of
// two): P then stays below 2^8, the sums stay exact in the same way, and O, which lives in
// tensor memory, has to be rescaled only on those rare moves (by the row's own thread, between
// the completion of PV_j(t-1) and the go-ahead for PV_j(t)).
//
// (Computing part of the exponentials by a polynomial on the FMA pipe instead of the
// special-function unit was measured slower: the softmax is bound by its instruction stream,
// not by that unit.)
//
// Warps: 0-7 softmax of query tile 0, 8-15 of query tile 1, which first gather their own query
// tile into shared memory (a warp reaches the 32 lanes of
// tensor memory given by its number modulo 4; warps w and w + 4 share rows and split the
// columns), 16 issues the tensor-core work, 17-18 gather key tiles, 19-20 gather value tiles
// from the pages with 16-byte asynchronous copies that write the 128-byte-swizzled operand
// layout directly.  Tiles are handed over through mbarriers; the only other barrier in the loop
// is one of the eight warps of a query tile when the halves of the row maximum meet.  Every wait
// is bounded; a wait that runs out sets the status word and the block leaves.  Tensor memory:
// S_0 at column 0, S_1 at 128 (P_j over columns 0-31 and 64-95 of S_j), O_0 at 256, O_1 at 384
// (all 512 columns: one block per SM).
#include "tc_common.cuh"

namespace leone {
namespace pingpong {

using namespace leone::tc;

constexpr int kRows = 128;                 // query rows per query tile
constexpr int kKeys = 128;                 // keys per tile
constexpr int kTileWarps = 8;              // softmax warps per query tile: 4 lane quarters x 2 column halves
constexpr int kTileThreads = kTileWarps * 32;
constexpr int kMmaWarp = 2 * kTileWarps;
constexpr int kLoadWarp0 = kMmaWarp + 1;   // two warps gather keys, the next two values
constexpr int kStreamThreads = 64;         // threads that gather one kind of tile (a thread per two key rows)
constexpr int kLoadThreads = 2 * kStreamThreads;
constexpr int kBlockThreads = (kLoadWarp0 + 4) * 32;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleAt = 8.0f;         // the running maximum moves when a tile's exceeds it by this (log2)

struct PagedArgs {
  const __nv_bfloat16* k_pool;
  const __nv_bfloat16* v_pool;
  const int* block_table;
  int table_width;
  int page_tokens;
  int num_pages;
  int n_kv;
};

// Waits for a phase like tc::mbar_wait, but lets the hardware suspend the warp for up to a few
// microseconds per try: a waiting warp then leaves the issue slots to the warps that compute.
__device__ __forceinline__ bool mbar_wait_long(uint32_t bar, uint32_t parity, volatile int* gave_up) {
  const long long start = clock64();
  while (true) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(4000u)
        : "memory");
    if (ok) return true;
    if (*gave_up) return false;
    if (clock64() - start > kWaitLimitCycles) {
      *gave_up = 1;
      return false;
    }
  }
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

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Byte offset of 16-byte chunk `chunk` (8 elements) of row `row` in a tile of rows of D
// elements stored as D/64 swizzled halves of [128 rows x 128 bytes].
__device__ __forceinline__ uint32_t swizzled(int row, int chunk) {
  return (uint32_t)((chunk >> 3) * (128 * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// Descriptor of an MN-major bf16 operand stored as rows of 128 bytes, one row per K index, 64 MN
// elements per row, 128-byte swizzle: 8-row groups (along K) are 1024 bytes apart and the next
// 64 MN elements are `mn_stride` bytes further.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t smem_addr, uint32_t mn_stride) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((mn_stride >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__host__ __device__ constexpr uint32_t instr_desc_bf16_b_mn(int m, int n) {
  return instr_desc_bf16(m, n) | (1u << 16);
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand is read from tensor memory, where row m is
// lane m and the 32-bit column c holds elements K = 2c (low half) and 2c + 1.
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 16 consecutive 32-bit columns of this thread's lane.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  tmem_st16(taddr, r);
  tmem_st16(taddr + 16, r + 16);
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <int D> constexpr int smem_bytes() {
  // two Q tiles, two K and two V tiles, row sources [2 kinds][2 buffers][128], barriers; 1024 for alignment
  return 2 * kRows * D * 2 + 4 * kKeys * D * 2 + 2 * 2 * kKeys * 8 + 16 * 8 + 1024;
}

template <int D>
__global__ void __launch_bounds__(kBlockThreads)
attention_prefill_pingpong_kernel(const __nv_bfloat16* __restrict__ qkv, int row_stride,
                                  __nv_bfloat16* __restrict__ out, int out_stride, PagedArgs pa,
                                  const int* __restrict__ q_start, const int* __restrict__ ctx_len, int n_q,
                                  float scale, int window, int* status) {
  constexpr int kTileBytes = kKeys * D * 2;             // one K or V tile; a Q tile has the same size
  constexpr int kTmemCols = 512;
  constexpr int kChunks = D / 8;                        // 16-byte chunks per row
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - raw);
  const uint32_t q_t = base;                            // [2] query tiles
  const uint32_t k_t = q_t + 2 * kTileBytes;            // [2] key tiles
  const uint32_t v_t = k_t + 2 * kTileBytes;            // [2] value tiles
  long long* row_src = reinterpret_cast<long long*>(aligned + 6 * kTileBytes);   // [kind][buffer][128]
  const uint32_t bars = smem_u32(row_src + 4 * kKeys);
  // loaders -> tensor core: a tile has landed; tensor core -> loaders: a tile's products are done
  const uint32_t bar_q = bars, bar_k_full = bars + 8, bar_v_full = bars + 24, bar_k_free = bars + 40,
                 bar_v_free = bars + 56;
  // tensor core -> softmax: S_j is complete (and every product issued before it);
  // softmax -> tensor core: P_j is written; tensor core -> softmax: the last O_j is complete
  const uint32_t bar_s = bars + 72, bar_p = bars + 88, bar_o = bars + 104;
  __shared__ uint32_t tmem_holder;
  __shared__ int gave_up;
  __shared__ float halves[2][2][2][kRows];              // [query tile][tile parity][column half][row]: maxima, then sums

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    gave_up = 0;
    mbar_init(bar_q, 2 * kTileWarps);                   // every softmax warp brings its share of its query tile
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_k_full + 8 * b, kStreamThreads / 32);
      mbar_init(bar_v_full + 8 * b, kStreamThreads / 32);
      mbar_init(bar_k_free + 8 * b, 1);
      mbar_init(bar_v_free + 8 * b, 1);
      mbar_init(bar_s + 8 * b, 1);
      mbar_init(bar_p + 8 * b, kTileWarps);
      mbar_init(bar_o + 8 * b, 1);
    }
    mbar_fence_init();
  }
  if (warp == kMmaWarp) tmem_alloc(smem_u32(&tmem_holder), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_holder;
  volatile int* giveup = &gave_up;
  pdl_trigger();
  pdl_wait();

  // blocks in launch order: the latest pair of query tiles (most keys) of every KV head first
  const int seq = blockIdx.z, kvh = blockIdx.x % pa.n_kv;
  const int pair = gridDim.x / pa.n_kv - 1 - blockIdx.x / pa.n_kv;
  const int g = n_q / pa.n_kv;
  const int tq = kRows / g;                             // tokens per query tile
  const int q0 = q_start[seq], q_len = q_start[seq + 1] - q0;
  const int tok0 = pair * 2 * tq;                       // first token of query tile 0
  if (tok0 < q_len) {                                   // block-uniform
    const int ctx = ctx_len[seq], start = ctx - q_len;
    // per query tile: its tokens [lo_j, hi_j), and how many key tiles it reads
    const int lo0 = tok0, hi0 = min(q_len, tok0 + tq);
    const int lo1 = min(q_len, tok0 + tq), hi1 = min(q_len, tok0 + 2 * tq);
    int k_lo = 0;
    if (window > 0) k_lo = max(0, start + tok0 - window + 1);
    const int tile0 = (k_lo / kKeys) * kKeys;
    const int n0 = (start + hi0 - tile0 + kKeys - 1) / kKeys;
    const int n1 = hi1 > lo1 ? (start + hi1 - tile0 + kKeys - 1) / kKeys : 0;
    const int n_tiles = max(n0, n1);
    const int k_hi = start + max(hi0, hi1);             // one past the last key any row reads

    if (warp == kMmaWarp) {
      // ---------------- the warp that issues the tensor-core work ----------------
      if (lane == 0) {
        constexpr uint32_t idesc_s = instr_desc_bf16(kRows, kKeys);
        constexpr uint32_t idesc_o = instr_desc_bf16_b_mn(kRows, D);
        auto issue_s = [&](int j, int t) {     // S_j = Q_j . K(t)^T
          const uint32_t q_s = q_t + j * kTileBytes, k_s = k_t + (t & 1) * kTileBytes;
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            // 16 elements further along a 128-byte row: +32 bytes; past 64 elements: the next half
            const uint32_t off = (ks >> 2) * (128 * 128) + (ks & 3) * 32;
            umma_bf16(tmem_base + j * kKeys, smem_desc_sw128(q_s + off), smem_desc_sw128(k_s + off), idesc_s,
                      ks > 0 ? 1u : 0u);
          }
          umma_commit(bar_s + 8 * j);
        };
        auto issue_pv = [&](int j, int t) {    // O_j (+)= P_j . V(t)
          const uint32_t v_s = v_t + (t & 1) * kTileBytes;
#pragma unroll
          for (int ks = 0; ks < kKeys / 16; ++ks) {
            // A = P_j in tensor memory: 16 keys are 8 columns, the second 64 keys start at column 64;
            // B = V: 16 keys = 16 rows = 2048 bytes further
            umma_bf16_a_tmem(tmem_base + 2 * kKeys + j * kKeys, tmem_base + j * kKeys + (ks >> 2) * 64 + (ks & 3) * 8,
                             smem_desc_mn_sw128(v_s + ks * 2048, 128 * 128), idesc_o, (t > 0 || ks > 0) ? 1u : 0u);
          }
        };
        bool ok = mbar_wait_long(bar_q, 0, giveup) && mbar_wait_long(bar_k_full, 0, giveup);
        if (ok) {
          tc_fence_after();
          if (n0 > 0) issue_s(0, 0);
          if (n1 > 0) issue_s(1, 0);
          umma_commit(bar_k_free);                       // K(0)'s buffer is free once both are done
        }
        for (int t = 0; t < n_tiles && ok; ++t) {
          const bool next = t + 1 < n_tiles;
          ok = mbar_wait_long(bar_v_full + 8 * (t & 1), (t >> 1) & 1, giveup);
          if (ok && next) ok = mbar_wait_long(bar_k_full + 8 * ((t + 1) & 1), ((t + 1) >> 1) & 1, giveup);
          for (int j = 0; j < 2 && ok; ++j) {
            const int nj = j == 0 ? n0 : n1;
            if (t >= nj) continue;
            ok = mbar_wait_long(bar_p + 8 * j, t & 1, giveup);
            if (!ok) break;
            tc_fence_after();
            issue_pv(j, t);
            if (t + 1 < nj) issue_s(j, t + 1);           // its commit also covers PV_j(t)
            else umma_commit(bar_o + 8 * j);
          }
          if (!ok) break;
          umma_commit(bar_v_free + 8 * (t & 1));
          if (next) umma_commit(bar_k_free + 8 * ((t + 1) & 1));
        }
      }
    } else if (warp >= kLoadWarp0) {
      // ---------------- the warps that gather the tiles ----------------
      const int lt = tid - kLoadWarp0 * 32;              // 0..127
      const bool values = lt >= kStreamThreads;
      const int st = lt & (kStreamThreads - 1);
      const __nv_bfloat16* pool = values ? pa.v_pool : pa.k_pool;
      const uint32_t tiles = values ? v_t : k_t;
      const uint32_t bar_full = values ? bar_v_full : bar_k_full, bar_free = values ? bar_v_free : bar_k_free;
      long long* rs = row_src + (values ? 2 * kKeys : 0);
      const int bar_id = values ? 3 : 2;
      // thread st resolves the sources of key rows st and st + 64 of a tile; the page numbers are
      // read a tile ahead (-1: no key here, -2: outside the table)
      auto page_of = [&](int t, int r) {
        int page = -1;
        const int kj = tile0 + t * kKeys + r;
        if (t < n_tiles && kj < k_hi && kj >= k_lo) {
          const int blk = kj / pa.page_tokens;
          page = blk < pa.table_width ? pa.block_table[(size_t)seq * pa.table_width + blk] : -2;
          if (page < 0) page = -2;
        }
        return page;
      };
      auto source_of = [&](int t, int r, int page) {
        const int kj = tile0 + t * kKeys + r;
        long long src = -1;
        if (page >= pa.num_pages || page == -2) set_status(status, kBadPage, q0 + tok0, page, kj);
        else if (page >= 0) src = (((long long)page * pa.n_kv + kvh) * pa.page_tokens + (kj % pa.page_tokens)) * D;
        return src;
      };
      // the first tile's page numbers (the query tiles are gathered by the softmax warps, which have
      // nothing else to do yet, so the first keys are requested at once)
      int page_a = page_of(0, st), page_b = page_of(0, st + kStreamThreads);
      // a thread copies two neighbouring chunks (one 32-byte sector) of rows r0, r0 + step, ..
      constexpr int kPairs = kChunks / 2;
      constexpr int kStep = kStreamThreads / kPairs;     // 8 rows for D = 128, 16 for D = 64: the swizzle phase stays
      const int ch0 = (st % kPairs) * 2, r0 = st / kPairs;
      bool ok_all = true;
      // A tile is announced as soon as it has landed; only then does the thread turn to the next
      // tile, whose buffer it may have to wait for.
      for (int t = 0; t < n_tiles; ++t) {
        long long* rs_t = rs + (t & 1) * kKeys;
        rs_t[st] = source_of(t, st, page_a);
        rs_t[st + kStreamThreads] = source_of(t, st + kStreamThreads, page_b);
        page_a = page_of(t + 1, st);
        page_b = page_of(t + 1, st + kStreamThreads);
        // the buffer's last tile (t - 2) has been consumed
        if (t >= 2 && ok_all && !mbar_wait_long(bar_free + 8 * (t & 1), ((t >> 1) - 1) & 1, giveup)) ok_all = false;
        named_barrier_sync(bar_id, kStreamThreads);      // the row sources of tile t are all written
        const uint32_t dst = tiles + (t & 1) * kTileBytes;
        const uint32_t d0 = dst + swizzled(r0, ch0), d1 = dst + swizzled(r0, ch0 + 1);
#pragma unroll
        for (int i = 0; i < kKeys / kStep; ++i) {
          const long long src = rs_t[r0 + i * kStep];
          const bool ok = src >= 0;
          const __nv_bfloat16* p = ok ? pool + src + ch0 * 8 : pool;
          cp_async16(d0 + i * kStep * 128, p, ok);
          cp_async16(d1 + i * kStep * 128, ok ? p + 8 : pool, ok);
        }
        cp_async_commit();
        cp_async_wait<0>();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_full + 8 * (t & 1));
      }
    } else {
      // ---------------- the softmax warps: two threads per query row ----------------
      const int j = warp / kTileWarps;                   // which query tile
      const int half = (warp >> 2) & 1;                  // which 64 columns of the row
      const int row = (warp & 3) * 32 + lane;
      const int nj = j == 0 ? n0 : n1;
      const int lo = j == 0 ? lo0 : lo1, hi = j == 0 ? hi0 : hi1;
      const int my_tl = row / g;
      const int my_pos = (my_tl < tq && lo + my_tl < hi) ? start + lo + my_tl : -1;   // -1: row unused
      const int first_pos = start + lo, last_pos = start + hi - 1;
      const float sl2 = scale * kLog2e;
      const uint32_t t_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);      // this warp's lanes
      const uint32_t t_s = t_lane + j * kKeys + half * 64;   // this thread's 64 columns of S_j; P_j over their first 32
      const uint32_t t_o = t_lane + 2 * kKeys + j * kKeys + half * (D / 2);          // its half of the row of O_j
      const int bar_id = 4 + j;
      float m_run = -INFINITY, l_run = 0.f;
      bool ok_all = true;
      {
        // this query tile's rows: row r = (token lo + r / g, head r % g), in the swizzled operand
        // layout; the tile's 256 threads take 8 of its 16-byte chunks each
        const int jt = tid - j * kTileThreads;
        for (int idx = jt; idx < kRows * kChunks; idx += kTileThreads) {
          const int r = idx / kChunks, ch = idx - r * kChunks;
          const int tl = r / g, hh = r - tl * g;
          const int token = tok0 + j * tq + tl;
          const bool ok = tl < tq && token < q_len;
          const __nv_bfloat16* src =
              qkv + (size_t)(q0 + (ok ? token : 0)) * row_stride + (size_t)(kvh * g + hh) * D + ch * 8;
          cp_async16(q_t + j * kTileBytes + swizzled(r, ch), src, ok);
        }
        cp_async_commit();
        cp_async_wait<0>();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_q);
      }
      for (int t = 0; t < nj; ++t) {
        const int tile_start = tile0 + t * kKeys + half * 64;     // this thread's first key
        // S_j(t) is complete, and so is PV_j(t - 1): O_j is at rest until this tile's go-ahead
        if (ok_all && !mbar_wait_long(bar_s + 8 * j, t & 1, giveup)) ok_all = false;
        tc_fence_after();
        // A tile that every row of this query tile sees whole needs no masking (the same for all
        // threads, so the branch is uniform; rows that stand for no token compute on zeros and
        // are never stored).
        const bool all_visible = tile0 + (t + 1) * kKeys - 1 <= first_pos &&
                                 (window <= 0 || tile0 + t * kKeys > last_pos - window);
        // keys first .. first + span (relative to this thread's first key) are visible to this row
        const int first = window > 0 ? max(my_pos - window + 1 - tile_start, 0) : 0;
        const unsigned span = my_pos >= 0 && my_pos - tile_start >= first ? (unsigned)(my_pos - tile_start - first) : 0u;
        const bool none = my_pos < 0 || my_pos - tile_start < first;      // no key of this thread's columns is visible
        // pass 1: the maximum over the keys the row may see; four running maxima (the chain of
        // dependent instructions is a quarter as long).  The 64 scores come in two loads of 32
        // that are both in flight at once: a load takes a few hundred cycles to come back.
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
        auto seen = [&](int k) { return !none && (unsigned)(k - first) <= span; };
        {
          uint32_t sc[64];
          tmem_ld32_issue(t_s, sc);
          tmem_ld32_issue(t_s + 32, sc + 32);
          tmem_ld_wait();
          if (all_visible) {
#pragma unroll
            for (int i = 0; i < 64; i += 8) {
              mx0 = fmaxf(fmaxf(mx0, __uint_as_float(sc[i])), __uint_as_float(sc[i + 1]));
              mx1 = fmaxf(fmaxf(mx1, __uint_as_float(sc[i + 2])), __uint_as_float(sc[i + 3]));
              mx2 = fmaxf(fmaxf(mx2, __uint_as_float(sc[i + 4])), __uint_as_float(sc[i + 5]));
              mx3 = fmaxf(fmaxf(mx3, __uint_as_float(sc[i + 6])), __uint_as_float(sc[i + 7]));
            }
          } else {
#pragma unroll
            for (int i = 0; i < 64; i += 4) {
              mx0 = fmaxf(mx0, seen(i) ? __uint_as_float(sc[i]) : -INFINITY);
              mx1 = fmaxf(mx1, seen(i + 1) ? __uint_as_float(sc[i + 1]) : -INFINITY);
              mx2 = fmaxf(mx2, seen(i + 2) ? __uint_as_float(sc[i + 2]) : -INFINITY);
              mx3 = fmaxf(mx3, seen(i + 3) ? __uint_as_float(sc[i + 3]) : -INFINITY);
            }
          }
        }
        float tile_max = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * sl2;    // the scale is positive; -inf stays -inf
        halves[j][t & 1][half][row] = tile_max;
        named_barrier_sync(bar_id, kTileThreads);        // the two halves of every row's maximum
        tile_max = fmaxf(tile_max, halves[j][t & 1][half ^ 1][row]);
        // the running maximum moves only when it must (first key seen) or when the tile's exceeds
        // it by 2^8; both threads of a row decide alike from the same numbers
        float alpha = 1.f;
        if (m_run == -INFINITY) {
          m_run = tile_max;                              // nothing accumulated so far: O_j is zero or not yet written
        } else if (tile_max > m_run + kRescaleAt) {
          alpha = ex2(m_run - tile_max);
          m_run = tile_max;
          l_run *= alpha;
        }
        if (t > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {       // warp-uniform: the loads and stores are collective
#pragma unroll
          for (int c = 0; c < D / 2; c += 16) {
            uint32_t r[16];
            tmem_ld16_issue(t_o + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st16(t_o + c, r);
          }
        }
        const float m_use = m_run == -INFINITY ? 0.f : m_run;
        // pass 2: P = 2^(S * scale - max) as bf16 pairs over the first 32 of this thread's columns.
        // The scores are read again in pieces of 16 columns, the next piece on its way while this
        // one is worked on; a piece goes through the arithmetic stage by stage (all exponents,
        // then all exponentials, then sums and pairs), so that independent instructions follow
        // each other and the pipes' latencies overlap.
        float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
        auto to_p = [&](const uint32_t* r, int c) {
          float x[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) x[i] = fmaf(__uint_as_float(r[i]), sl2, -m_use);
#pragma unroll
          for (int i = 0; i < 16; ++i) x[i] = ex2(x[i]);
          if (!all_visible) {                            // uniform
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = seen(c + i) ? x[i] : 0.f;
          }
          uint32_t packed[8];
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            l0 += x[i];
            l1 += x[i + 1];
            l2 += x[i + 2];
            l3 += x[i + 3];
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            __nv_bfloat162 v2 = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
            packed[i] = *reinterpret_cast<uint32_t*>(&v2);
          }
          tmem_st8(t_s + c / 2, packed);                 // this thread's keys c .. c + 15 are its columns c / 2 .. c / 2 + 7
        };
        {
          uint32_t pa[16], pb[16];
          tmem_ld16_issue(t_s, pa);
          tmem_ld16_issue(t_s + 16, pb);
          tmem_ld_wait();
          to_p(pa, 0);
          tmem_ld16_issue(t_s + 32, pa);
          to_p(pb, 16);
          tmem_ld16_issue(t_s + 48, pb);
          tmem_ld_wait();
          to_p(pa, 32);
          to_p(pb, 48);
        }
        l_run += (l0 + l1) + (l2 + l3);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p + 8 * j);       // PV_j(t) may go
      }
      // the last O_j, divided by the row's sum (its two halves meet like the maxima)
      if (nj > 0) {
        halves[j][nj & 1][half][row] = l_run;
        named_barrier_sync(bar_id, kTileThreads);
        const float l_row = l_run + halves[j][nj & 1][half ^ 1][row];
        if (ok_all && !mbar_wait_long(bar_o + 8 * j, 0, giveup)) ok_all = false;
        tc_fence_after();
        const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
        const bool store = ok_all && my_pos >= 0;
        const int hh = row - my_tl * g;
        __nv_bfloat16* dst = out + (size_t)(q0 + lo + (store ? my_tl : 0)) * out_stride + (size_t)(kvh * g + hh) * D +
                             half * (D / 2);
#pragma unroll
        for (int c = 0; c < D / 2; c += 16) {
          uint32_t r[16];
          tmem_ld16_issue(t_o + c, r);
          tmem_ld_wait();
          if (store) {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              uint32_t pk[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                __nv_bfloat162 v2 = __floats2bfloat162_rn(__uint_as_float(r[q * 8 + 2 * i]) * inv,
                                                          __uint_as_float(r[q * 8 + 2 * i + 1]) * inv);
                pk[i] = *reinterpret_cast<uint32_t*>(&v2);
              }
              *reinterpret_cast<uint4*>(dst + c + q * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
          }
        }
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (gave_up && tid == 0) set_status(status, kWaitTimeout, blockIdx.x, 2);
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
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_pingpong_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<D>());
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int g = n_q / pa.n_kv;
  const int tq = kRows / g;
  dim3 grid(((max_q_len + 2 * tq - 1) / (2 * tq)) * pa.n_kv, 1, n_seqs);
  return launch_kernel(attention_prefill_pingpong_kernel<D>, grid, dim3(kBlockThreads), smem_bytes<D>(), stream,
                       qkv, row_stride, out, out_stride, pa, q_start, ctx_len, n_q, scale, window, status);
}

}  // namespace pingpong
}  // namespace leone

using namespace leone;

// Prompt portions and mixed batches on tcgen05, two query tiles per block; arguments as
// leone_attention_prefill.  Head size 64 or 128, up to 128 query heads per KV head, 16-byte
// aligned rows.
extern "C" int leone_attention_prefill_pingpong(const void* qkv, int row_stride, void* out, int out_stride,
                                                const void* k_pool, const void* v_pool, const int* block_table,
                                                int table_width, const int* q_start, const int* ctx_len, int n_seqs,
                                                int max_q_len, int n_q, int n_kv, int d, float scale, int window,
                                                int page_tokens, int num_pages, int* status, cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return 0;
  if (d != 64 && d != 128) return kRefusedSize;
  if (n_q <= 0 || n_kv <= 0 || n_q % n_kv != 0 || n_q / n_kv > pingpong::kRows) return kRefusedSize;
  if (page_tokens <= 0 || table_width <= 0 || n_seqs > 65535) return kRefusedSize;
  if (row_stride % 8 != 0 || out_stride % 8 != 0) return kRefusedAlignment;
  if (((uintptr_t)qkv | (uintptr_t)out | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) return kRefusedAlignment;
  pingpong::PagedArgs pa{(const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, block_table, table_width,
                         page_tokens, num_pages, n_kv};
  if (d == 64)
    return pingpong::launch<64>((const __nv_bfloat16*)qkv, row_stride, (__nv_bfloat16*)out, out_stride, pa, q_start,
                                ctx_len, n_seqs, n_q, max_q_len, scale, window, status, stream);
  return pingpong::launch<128>((const __nv_bfloat16*)qkv, row_stride, (__nv_bfloat16*)out, out_stride, pa, q_start,
                               ctx_len, n_seqs, n_q, max_q_len, scale, window, status, stream);
}
