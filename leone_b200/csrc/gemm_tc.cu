// out[M,N] = x[M,K] * w[N,K]^T in bfloat16 on the 5th-generation tensor cores.
//
// Orientation.  Both operands are K-major, so either may ride the MMA's M dimension.
// Up to 256 tokens ("swapped"): the weight matrix rides M (128 weight rows per tile, one
// TMEM lane each) and the tokens ride N (BN = 16..256 tokens per tile), so a decode step
// with a handful of tokens is a pure weight stream through 128x16 MMAs.  More tokens
// (prompt portions): 128 tokens ride M and 256 weight rows ride N, so each epilogue
// thread owns one token row and writes 16 consecutive outputs at a time with vector
// stores.  The reference has a GEMV family for decode and a library GEMM for prompts
// (crates/leone-cuda/cuda/ie_cuda.cu:1718, 5069); this kernel replaces both.
//
// Structure (persistent; two blocks per SM for up to 64 tokens, else one; 6 warps):
//   warp 0       TMA producer: weight tile [128 x 64] and token tile [BN x 64] per
//                k-block into a ring of shared-memory stages (128-byte swizzle);
//   warp 1       allocates tensor memory, issues tcgen05.mma (one thread), commits each
//                stage back to the producer and each finished tile to the epilogue;
//   warps 2..5   epilogue: tcgen05.ld of the fp32 accumulator (two buffers, so the next
//                tile's MMAs overlap), then one of
//                  0 store bf16, 1 store fp32, 2 store fp32 = acc + residual,
//                  3 SwiGLU on interleaved gate/up rows -> bf16.
// Split-K (decode shapes with few weight tiles): every split writes its fp32 partial
// tile to a workspace; the split that arrives last at the tile's counter sums the
// partials in split order (deterministic, no atomics on data) and runs the epilogue.
// Every wait is bounded; a wait that runs out sets the status word and the block leaves.
#include "gemm_parts.cuh"

namespace leone {
namespace tc {

static int g_l2_ahead = 8;

// kSwap: weights on the MMA's M side (tile 128), tokens on its N side (tile BN).
// !kSwap: tokens on the M side (tile 128), weights on the N side (tile BN); no split-K.
// kCluster: the `splits` blocks of a tile form a thread-block cluster, one unit per block; every
// block leaves its fp32 partial tile in its own shared memory, then the tile's rows are dealt to
// the blocks, each of which adds its rows' partials in rank order through distributed shared
// memory and runs the epilogue on them.  No workspace, no counters, no round trip through global
// memory.  In the token-major form (rows = tokens) without a folded norm.
template <int BN, bool kSwap, bool kCluster>
__global__ void __launch_bounds__(kGemmThreads, GemmCfg<BN>::kBlocksPerSm)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (tiles_base - raw);
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + kStages * Cfg::kStageBytes);
  // barriers: full[kStages], empty[kStages], acc_full[2], acc_empty[2]
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * kStages;
  const uint32_t acc_full0 = empty0 + 8 * kStages, acc_empty0 = acc_full0 + 16;
  constexpr bool kPush = gemm_pushes<BN, kSwap, kCluster>();
  // the inbox of pushed partial sums: [slot][column][row of the chunk] floats, behind the barriers
  float* inbox = reinterpret_cast<float*>(aligned + kStages * Cfg::kStageBytes + 256);
  __shared__ uint32_t tmem_holder;
  __shared__ int gave_up;
  __shared__ int last_flag;
  __shared__ float rs_s[kSwap ? BN : 1];          // per token: the scale of the norm before this product
  __shared__ float red_s[kSwap ? 4 * BN : 1];

  // Push mode: the residual values and the following norm's weight of the rows this thread
  // finishes (up to four chunks of 32 rows), fetched while the products run.
  constexpr int kPreNC = kPush ? BN / 4 : 1;
  float pre_r[4][kPreNC], pre_gw[4];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) stamp(p, 7);                       // first instruction of the block
  // tiles along the tokens (m) and along the weight rows (n); the token tile index runs
  // fastest so that blocks working at the same time share weight tiles through L2
  constexpr int kTokRows = kSwap ? BN : kTileW, kWRows = kSwap ? kTileW : BN;
  const int n_tiles = (p.N + kWRows - 1) / kWRows;
  const int m_tiles = (p.M + kTokRows - 1) / kTokRows;
  const int k_blocks = (p.K + kTileK - 1) / kTileK;
  const int total = p.full_tiles + (n_tiles * m_tiles - p.full_tiles) * p.splits;

  if (threadIdx.x == 0) {
    gave_up = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 4);
    }
    mbar_init(acc_empty0 + 16, 1);     // token-major cluster mode: the partial sums have landed
    mbar_fence_init();
    tma_prefetch_desc(&map_w);
    tma_prefetch_desc(&map_x);
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_holder), Cfg::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_holder;
  volatile int* giveup = &gave_up;
  pdl_trigger();
  if (threadIdx.x == 0) stamp(p, 0);                       // set-up done
  // pushing blocks write into their cluster peers' shared memory before any full barrier: this
  // arrival (waited for just before the first such write) says that this block is running
  if constexpr (kPush) cluster_arrive_relaxed();
  bool started_seen = false;                               // this thread has waited for that arrival

  if (warp == 0) {
    // ---------------- producer ----------------
    // The weights do not depend on the kernels before this one: the weight halves of the
    // first stages are requested at once, and only then does the producer wait for the
    // predecessor (whose output is the token operand).  Pass 0 issues those early weight
    // loads, pass 1 is the steady loop, which for the first stages adds the token half only.
    if (lane == 0) {
      int early = 0;                       // stages whose weight half was requested in pass 0
      for (int pass = 0; pass < 2; ++pass) {
        int stage = 0, filled = 0;
        uint32_t phase = 0;
        bool stop = false;
        for (int t = blockIdx.x; t < total && !*giveup && !stop; t += gridDim.x) {
          const Unit un = unit_of(t, p);
          const int m_tile = un.tile % m_tiles, n_tile = un.tile / m_tiles;
          const int per = (k_blocks + un.nsplit - 1) / un.nsplit;
          const int kb0 = un.split * per, kb1 = min(k_blocks, kb0 + per);
          for (int kb = kb0; kb < kb1; ++kb, ++filled) {
            if (pass == 0 && filled >= kStages) {
              // further weight tiles cannot land yet (no free stage): the L2 may fetch them
              if (filled >= kStages + p.l2_ahead) { stop = true; break; }
              tma_prefetch_2d(&map_w, kb * kTileK, n_tile * (kSwap ? kTileW : BN));
              continue;
            }
            const bool had_weights = pass == 1 && filled < early;
            if (pass == 1 && !had_weights && !mbar_wait(empty0 + 8 * stage, phase ^ 1, giveup)) {
              stop = true;
              break;
            }
            const uint32_t dst = tiles_base + stage * Cfg::kStageBytes;
            const uint32_t bar = full0 + 8 * stage;
            if (!had_weights) mbar_expect_tx(bar, Cfg::kStageBytes);
            const uint32_t w_dst = kSwap ? dst : dst + kTileW * kTileK * 2;
            const uint32_t x_dst = kSwap ? dst + kTileW * kTileK * 2 : dst;
            if (!had_weights) tma_load_2d(w_dst, &map_w, bar, kb * kTileK, n_tile * (kSwap ? kTileW : BN));
            if (pass == 1) tma_load_2d(x_dst, &map_x, bar, kb * kTileK, m_tile * (kSwap ? BN : kTileW));
            if (++stage == kStages) { stage = 0; phase ^= 1; }
          }
        }
        if (pass == 0) {
          early = min(filled, kStages);
          stamp(p, 1);                                     // early weight requests issued
          pdl_wait();
          stamp(p, 2);                                     // predecessor complete
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_bf16(kTileW, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int t = blockIdx.x; t < total && !*giveup; t += gridDim.x, ++it) {
        const Unit un = unit_of(t, p);
        const int per = (k_blocks + un.nsplit - 1) / un.nsplit;
        const int kb0 = un.split * per, kb1 = min(k_blocks, kb0 + per);
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(acc_empty0 + 8 * buf, acc_phase ^ 1, giveup)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        bool ok = true;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full0 + 8 * stage, phase, giveup)) { ok = false; break; }
          tc_fence_after();
          if (it == 0 && kb == kb0) stamp(p, 3);           // first stage complete in shared memory
          const uint32_t a_addr = tiles_base + stage * Cfg::kStageBytes;
          const uint32_t b_addr = a_addr + kTileW * kTileK * 2;
          const uint64_t a_desc = smem_desc_sw128(a_addr), b_desc = smem_desc_sw128(b_addr);
#pragma unroll
          for (int k = 0; k < kTileK / 16; ++k) {
            // 16 bf16 = 32 bytes further along K inside the swizzled row: +2 in 16-byte units
            umma_bf16(tmem_d, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty0 + 8 * stage);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(acc_full0 + 8 * buf);
        stamp(p, 4);                                       // last MMA of the (latest) unit issued
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;                     // TMEM lanes 32*quarter .. +31
    const int ep_tid = (warp - 2) * 32 + lane;        // 0..127
    int it = 0;
    pdl_wait();      // outputs, residual and the split-K workspace may be in use until here
    if constexpr (kSwap) {
      if (p.norm_in_ss != nullptr) {
        // the scale of every token from the partial sums the product before the norm left:
        // thread t adds parts t, t + 128, ..; then a fixed tree over the warp and the four warps
        // (the loads of a batch of tokens are issued together: one round trip per batch)
        constexpr int kBatch = BN < 32 ? BN : 32;
        for (int mb = 0; mb < p.M && mb < BN; mb += kBatch) {
          float part[kBatch];
#pragma unroll
          for (int j = 0; j < kBatch; ++j) part[j] = 0.f;
          for (int q = ep_tid; q < p.norm_in_parts; q += 128) {
            const float* row = p.norm_in_ss + (size_t)q * p.M + mb;
#pragma unroll
            for (int j = 0; j < kBatch; ++j)
              if (mb + j < p.M) part[j] += row[j];
          }
#pragma unroll
          for (int j = 0; j < kBatch; ++j) {
            float v = part[j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) red_s[(warp - 2) * BN + mb + j] = v;
          }
        }
        named_barrier_sync(1, 128);
        for (int m = ep_tid; m < BN; m += 128) {
          const float ss = red_s[m] + red_s[BN + m] + red_s[2 * BN + m] + red_s[3 * BN + m];
          rs_s[m] = m < p.M ? rsqrtf(ss / (float)p.K + p.norm_eps) : 0.f;
        }
        named_barrier_sync(1, 128);
      }
    }
    if constexpr (kPush) {
      if (blockIdx.x < total) {
        const Unit un = unit_of(blockIdx.x, p);
        const int m_tile = un.tile % m_tiles, n_tile = un.tile / m_tiles;
        const int rank = (int)cluster_ctarank();
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int ch = rank + k * un.nsplit;
          if (ch < kTileW / 32) {
            const int n = n_tile * kTileW + ch * 32 + lane;
            fetch_residual<kPreNC>(p, pre_r[k], n, m_tile * BN, (warp & 3) * kPreNC);
            pre_gw[k] = p.norm_out_x != nullptr && n < p.N ? p.norm_out_w[n] : 0.f;
          }
        }
      }
    }
    for (int t = blockIdx.x; t < total && !*giveup; t += gridDim.x, ++it) {
      const Unit un = unit_of(t, p);
      const int tile = un.tile, split = un.split, nsplit = un.nsplit;
      const int m_tile = tile % m_tiles, n_tile = tile / m_tiles;
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(acc_full0 + 8 * buf, acc_phase, giveup)) break;
      tc_fence_after();
      if (ep_tid == 0) stamp(p, 5);                        // accumulator of the (latest) unit complete
      const int row_local = quarter * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
      if constexpr (kPush) {
        // this thread's row of the partial tile goes straight into the inbox of the block that
        // finishes the row's chunk (chunk = this warp's quarter of the rows; owner = chunk %
        // splits), slot (chunk / splits, this block's rank): one remote store per column, 32
        // lanes side by side.  After the one cluster barrier below nothing remote is touched
        // again, so no second barrier is needed and a finished block just leaves.
        const uint32_t my_rank = cluster_ctarank();
        const uint32_t owner = (uint32_t)quarter % (uint32_t)nsplit;
        const uint32_t slot = smem_u32(inbox) + ((((quarter / nsplit) * nsplit + my_rank) * BN) * 32 + lane) * 4;
        const uint32_t dst = cluster_map(slot, owner);
        cluster_wait();                                  // every block of the cluster is running
        started_seen = true;
        for (int c = 0; c < BN; c += 16) {
          float v[16];
          tmem_ld16(taddr + c, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) cluster_st_f32(dst + (c + j) * 32 * 4, v[j]);
        }
        break;                                           // one unit per block in this mode
      } else if constexpr (kCluster && !kSwap) {
        // Token-major tiles are 128 KB of partial sums: they go through the workspace (L2), which
        // moves several times the bytes per second that distributed shared memory does;
        // [unit][chunk of 32 rows][accumulator column][row of the chunk]: 32 rows side by side
        // in every store, and a chunk of one unit is 32 KB in one piece.
        float* ws = p.workspace + (size_t)t * (BN * kTileW) + (size_t)quarter * (BN * 32) + lane;
        for (int c = 0; c < BN; c += 64) {               // two loads of 32 columns in flight
          uint32_t r[64];
          tmem_ld32_issue(taddr + c, r);
          tmem_ld32_issue(taddr + c + 32, r + 32);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 64; ++j) ws[(c + j) * 32] = __uint_as_float(r[j]);
        }
        __threadfence();
        break;                                           // one unit per block in this mode
      } else if constexpr (kCluster) {
        // this block's partial tile goes to its own shared memory, [accumulator column][row];
        // the stages are free: the accumulator is complete, so every MMA has read its operands
        static_assert(kStages * Cfg::kStageBytes >= BN * kTileW * 4, "partial tile must fit in the stages");
        float* part = reinterpret_cast<float*>(aligned);
        for (int c = 0; c < BN; c += 16) {
          float v[16];
          tmem_ld16(taddr + c, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) part[(c + j) * kTileW + row_local] = v[j];
        }
        break;                                           // one unit per block in this mode
      }
      if (!kSwap) {
        // this thread owns token row m and walks the tile's weight rows 16 at a time
        finish_token_major_row<BN>(p, taddr, m_tile * kTileW + row_local, n_tile * BN, n_tile);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
        continue;
      }
      const int n = n_tile * kTileW + row_local;
      const int m0 = m_tile * BN;
      bool do_epilogue = true;
      const int split_tile = tile - p.full_tiles;        // index among the split tiles
      if (nsplit > 1) {
        float* ws = p.workspace + ((size_t)split_tile * nsplit + split) * (BN * kTileW);
        for (int c = 0; c < BN; c += 16) {
          float v[16];
          tmem_ld16(taddr + c, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) ws[(c + j) * kTileW + row_local] = v[j];
        }
        __threadfence();
        named_barrier_sync(1, 128);
        if (ep_tid == 0) {
          const int old = atomicAdd(&p.counters[split_tile], 1);
          const int last = old == nsplit - 1;
          if (last) p.counters[split_tile] = 0;      // ready for the next launch
          last_flag = last;
        }
        named_barrier_sync(1, 128);
        do_epilogue = last_flag != 0;
        if (do_epilogue) __threadfence();
      }
      // the accumulator buffer is free once its values are in registers or in the workspace
      if (nsplit > 1) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
      }
      if (do_epilogue) {
        const float* ws_tile = nsplit > 1 ? p.workspace + (size_t)split_tile * nsplit * (BN * kTileW) : nullptr;
        for (int c = 0; c < BN; c += 16) {
          float v[16];
          float r[16];
          fetch_residual<16>(p, r, n, m0, c);
          if (nsplit > 1) {
            // Partial sums are added in split order, four splits' loads in flight at a time:
            // one wait per four splits instead of one per split.
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.f;
            for (int s0 = 0; s0 < nsplit; s0 += 4) {
              float t[4][16];
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                if (s0 + u < nsplit) {
                  const float* src = ws_tile + (size_t)(s0 + u) * (BN * kTileW) + c * kTileW + row_local;
#pragma unroll
                  for (int j = 0; j < 16; ++j) t[u][j] = __ldcg(src + j * kTileW);
                }
              }
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                if (s0 + u < nsplit) {
#pragma unroll
                  for (int j = 0; j < 16; ++j) v[j] += t[u][j];
                }
              }
            }
          } else {
            tmem_ld16(taddr + c, v);
          }
          finish_swapped<16>(p, v, r, n, m0, c, lane, rs_s);
        }
      }
      if (nsplit == 1) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
      }
    }
  }

  if constexpr (kCluster) {
    // Every thread of every block of the cluster comes here (all loops above are bounded).
    // The tile's 128 weight rows are four chunks of 32; chunk ch is summed and finished by the
    // block of rank ch % splits, so the sums and the epilogue are spread over the cluster.
    // In a chunk, lane = row and each epilogue warp owns a quarter of the token columns.
    __syncwarp();
    if constexpr (kPush) {
      if (!started_seen) cluster_wait();                 // pairs the arrival at the block's start
    }
    cluster_sync_all();                                  // all partial tiles are in place
    if constexpr (kPush) {
      // The chunks this block owns lie in its own inbox, one slot per rank: sum them in rank
      // order and finish.  Lane = row of the chunk; each epilogue warp owns a quarter of the
      // token columns.
      if (warp >= 2 && blockIdx.x < total) {
        const Unit un = unit_of(blockIdx.x, p);
        const int m_tile = un.tile % m_tiles, n_tile = un.tile / m_tiles;
        const int m0 = m_tile * BN;
        constexpr int NC = BN / 4;
        const int rank = (int)cluster_ctarank();
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int ch = rank + k * un.nsplit;
          if (ch >= kTileW / 32) break;
          const int n = n_tile * kTileW + ch * 32 + lane;
          const float* mine = inbox + (size_t)((ch / un.nsplit) * un.nsplit) * BN * 32 + lane;
          const int c = (warp & 3) * NC;
          float v[NC];
#pragma unroll
          for (int j = 0; j < NC; ++j) v[j] = 0.f;
          for (int s0 = 0; s0 < un.nsplit; ++s0) {       // rank order
#pragma unroll
            for (int j = 0; j < NC; ++j) v[j] += mine[((size_t)s0 * BN + c + j) * 32];
          }
          finish_swapped<NC>(p, v, pre_r[k], n, m0, c, lane, rs_s, &pre_gw[k]);
        }
      }
    } else
    if constexpr (!kSwap) {
      // token-major: the rows are tokens; chunk ch (32 token rows) is finished by the block of
      // rank ch % splits.  The chunk's partial sums of up to four ranks at a time are copied
      // from the workspace into the (now free) stages in pieces of 32 KB, one per rank, by the
      // copy engine; then lane = token row, and each epilogue warp adds, in rank order, a
      // quarter of the tile's weight rows, 32 at a time (a gate/up group for SwiGLU).
      if (warp >= 2 && blockIdx.x < total && !*giveup) {
        const Unit un = unit_of(blockIdx.x, p);
        const int m_tile = un.tile % m_tiles, n_tile = un.tile / m_tiles;
        constexpr int kColsPerWarp = BN / 4;
        constexpr int kGroups = kColsPerWarp / 32;
        constexpr uint32_t kPiece = BN * 32 * 4;         // one rank's partial sums of a chunk
        static_assert(kColsPerWarp % 32 == 0, "a warp's share of the weight rows is whole gate/up groups");
        static_assert(kStages * Cfg::kStageBytes >= 4 * (int)kPiece, "four pieces must fit in the stages");
        const int rank = (int)cluster_ctarank();
        const float* ws_tile = p.workspace + (size_t)(blockIdx.x - rank) * (BN * kTileW);
        const float* box = reinterpret_cast<const float*>(aligned);
        const uint32_t landed = acc_empty0 + 16;
        const int et = (warp - 2) * 32 + lane;
        const uint32_t read0 = acc_empty0;               // (count 4, unused otherwise in this mode)
        uint32_t landed_phase = 0, read_phase = 0;
        bool first = true;
        for (int ch = rank; ch < kTileW / 32; ch += un.nsplit) {
          const int m = m_tile * kTileW + ch * 32 + lane;
          // the sums start from the residual values, which are in flight while the pieces land
          float v[kGroups][32];
#pragma unroll
          for (int g = 0; g < kGroups; ++g)
            fetch_residual32(p, v[g], m, n_tile * BN + (warp & 3) * kColsPerWarp + g * 32);
          bool ok = true;
          for (int sb = 0; sb < un.nsplit; sb += 4) {
            const int nb = min(4, un.nsplit - sb);
            if (et == 0) {
              // the pieces before these have been read by all four warps (every wait is bounded:
              // if this one runs out nothing is requested and the others' waits run out too)
              bool go = true;
              if (!first) {
                go = mbar_wait(read0, read_phase, giveup);
                read_phase ^= 1;
              }
              if (go) {
                fence_proxy_async();
                mbar_expect_tx(landed, (uint32_t)nb * kPiece);
                for (int u = 0; u < nb; ++u)
                  bulk_load(tiles_base + (uint32_t)u * kPiece,
                            ws_tile + (size_t)(sb + u) * (BN * kTileW) + (size_t)ch * (BN * 32), kPiece, landed);
              }
            }
            first = false;
            if (!mbar_wait(landed, landed_phase, giveup)) { ok = false; break; }
            landed_phase ^= 1;
#pragma unroll
            for (int g = 0; g < kGroups; ++g) {
              const float* src = box + (size_t)((warp & 3) * kColsPerWarp + g * 32) * 32 + lane;
              for (int u = 0; u < nb; ++u) {             // rank order
#pragma unroll
                for (int j = 0; j < 32; ++j) v[g][j] += src[(size_t)u * (BN * 32) + j * 32];
              }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(read0);           // this warp has read the pieces
          }
          if (!ok) break;
#pragma unroll
          for (int g = 0; g < kGroups; ++g)
            finish_token_major32(p, v[g], m, n_tile * BN + (warp & 3) * kColsPerWarp + g * 32, true);
        }
      }
    } else
    if (warp >= 2 && blockIdx.x < total) {
      const Unit un = unit_of(blockIdx.x, p);
      const int m_tile = un.tile % m_tiles, n_tile = un.tile / m_tiles;
      const int m0 = m_tile * BN;
      constexpr int kColsPerWarp = BN / 4;
      constexpr int NC = kColsPerWarp < 16 ? kColsPerWarp : 16;
      const int rank = (int)cluster_ctarank();
      for (int ch = rank; ch < kTileW / 32; ch += un.nsplit) {
        const int row_local = ch * 32 + lane;
        const int n = n_tile * kTileW + row_local;
        const uint32_t mine = tiles_base + row_local * 4;
        for (int c = (warp & 3) * kColsPerWarp; c < (warp & 3) * kColsPerWarp + kColsPerWarp; c += NC) {
          float v[NC];
          float r[NC];
          fetch_residual<NC>(p, r, n, m0, c);
#pragma unroll
          for (int j = 0; j < NC; ++j) v[j] = 0.f;
          constexpr int kBatch = NC <= 8 ? 8 : 4;        // ranks whose loads are in flight together
          for (int s0 = 0; s0 < un.nsplit; s0 += kBatch) {
            float t[kBatch][NC];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
              if (s0 + u < un.nsplit) {
                const uint32_t src = cluster_map(mine, s0 + u) + c * kTileW * 4;
#pragma unroll
                for (int j = 0; j < NC; ++j) t[u][j] = cluster_ld_f32(src + j * kTileW * 4);
              }
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {           // rank order
              if (s0 + u < un.nsplit) {
#pragma unroll
                for (int j = 0; j < NC; ++j) v[j] += t[u][j];
              }
            }
          }
          finish_swapped<NC>(p, v, r, n, m0, c, lane, rs_s);
        }
      }
    }
    __syncwarp();
    if constexpr (!kPush && kSwap) cluster_sync_all();   // the partial tiles may go away
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) stamp(p, 6);                       // block done
  if (gave_up) {
    if (threadIdx.x == 0) set_status(p.status, kWaitTimeout, blockIdx.x, 0);
    // let tile copies that are still in flight land before the block's memory goes away
    const long long start = clock64();
    while (clock64() - start < 200000) {}
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BN, bool kSwap, bool kCluster = false>
int launch_gemm(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, int sm_count,
                cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, kSwap, kCluster>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         gemm_smem_bytes<BN, kSwap, kCluster>());
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int w_rows = kSwap ? kTileW : BN, tok_rows = kSwap ? BN : kTileW;
  const int n_tiles = (p.N + w_rows - 1) / w_rows, m_tiles = (p.M + tok_rows - 1) / tok_rows;
  const long long total = p.full_tiles + ((long long)n_tiles * m_tiles - p.full_tiles) * p.splits;
  const long long slots = (long long)sm_count * Cfg::kBlocksPerSm;
  const int grid = (int)(total < slots ? total : slots);
  if constexpr (kCluster) {
    if (total > slots) return kRefusedSize;              // one unit per block, one round
    return launch_kernel_cluster(gemm_tc_kernel<BN, kSwap, true>, dim3((unsigned)total), dim3(kGemmThreads),
                                 gemm_smem_bytes<BN, kSwap, true>(), stream, dim3(p.splits), mw, mx, p);
  }
  return launch_kernel(gemm_tc_kernel<BN, kSwap, kCluster>, dim3(grid), dim3(kGemmThreads),
                       gemm_smem_bytes<BN, kSwap, kCluster>(), stream, mw, mx, p);
}

// How many clusters of `splits` blocks of the swapped kernel for token tile BN can be resident
// at once (0: this cluster size cannot be launched).
template <int BN, bool kSwap = true>
int cluster_capacity(int splits) {
  using Cfg = GemmCfg<BN>;
  cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, kSwap, true>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       gemm_smem_bytes<BN, kSwap, true>());
  if (e != cudaSuccess) { cudaGetLastError(); return 0; }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(splits * 64);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = gemm_smem_bytes<BN, kSwap, true>();
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = splits;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  e = cudaOccupancyMaxActiveClusters(&clusters, gemm_tc_kernel<BN, kSwap, true>, &cfg);
  if (e != cudaSuccess) { cudaGetLastError(); return 0; }
  return clusters;
}

}  // namespace tc
}  // namespace leone

using namespace leone;
using namespace leone::tc;

// Turns programmatic dependent launch on or off for the kernels of this library.
// k-blocks of weights that every block's producer asks the L2 for beyond its early stages, in
// products of up to 16 tokens (measured on the decode step at batch 8: 0 -> 3.64 ms, 4 -> 3.62,
// 8 -> 3.60, 16 -> 3.68; at batch 64 it changes nothing).
extern "C" void leone_gemm_tc_set_l2_ahead(int k_blocks) { g_l2_ahead = k_blocks < 0 ? 0 : k_blocks; }
extern "C" void leone_bf16_set_pdl(int enabled) { pdl_flag() = enabled ? 1 : 0; }

// Phase trace for tuning: while `buffer` is not null every block of a product writes eight
// %globaltimer stamps (ns) at [block * 8 + i]: 0 set-up done, 1 early weight requests issued,
// 2 predecessor complete, 3 first stage landed, 4 last MMA issued, 5 accumulator complete,
// 6 block done, 7 first instruction.  Every launch writes at `buffer` and then moves it on by
// `stride` int64 (0: all launches share one area), so consecutive launches can be told apart.
static long long* g_gemm_trace = nullptr;
static long long g_gemm_trace_stride = 0;
extern "C" void leone_gemm_tc_set_trace(long long* buffer, long long stride) {
  g_gemm_trace = buffer;
  g_gemm_trace_stride = stride;
}

// Token-tile width the kernel will use for M tokens.
extern "C" int leone_gemm_tc_tile(int m) {
  return m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : m <= 128 ? 128 : 256;
}

// Number of (weight tile, token tile) pairs the kernel makes of an [m, n] product.
extern "C" int leone_gemm_tc_tiles(int m, int n) {
  if (m > 256) return ((n + 255) / 256) * ((m + kTileW - 1) / kTileW);
  const int bn = leone_gemm_tc_tile(m);
  return ((n + kTileW - 1) / kTileW) * ((m + bn - 1) / bn);
}

// Tiles of the token-major form (128 tokens x 256 weight rows), which takes any number of tokens.
extern "C" int leone_gemm_tc_tiles_token_major(int m, int n) {
  return ((n + 255) / 256) * ((m + kTileW - 1) / kTileW);
}

static int device_sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  return sms;
}

// Weight rows per tile of the unsplit token-major form above 256 tokens: of 256 and 240 the
// width whose tiles cost the fewer rounds over the SMs times the width (2,048 tokens x 4,096
// outputs: 256 tiles of 256 are two rounds on 148 SMs, the second 73 % full; 288 tiles of 240
// are two full rounds of narrower tiles: 72.6 -> 66.7 us).  gate_up_groups: the rows come in
// gate/up groups of 32 (SwiGLU epilogue), which 240 would cut; 224 was measured no faster there.
extern "C" int leone_gemm_tc_token_major_width(int m, int n, int gate_up_groups) {
  if (m <= 256) return 256;
  const int sms = device_sm_count();
  const long long m_tiles = (m + kTileW - 1) / kTileW;
  int best = 256;
  long long best_cost = -1;
  const int widths[2] = {256, 240};
  for (int w : widths) {
    if (gate_up_groups && (w % 32) != 0) continue;
    const long long tiles = ((n + w - 1) / w) * m_tiles;
    const long long cost = ((tiles + sms - 1) / sms) * w;
    if (best_cost < 0 || cost < best_cost) best = w, best_cost = cost;
  }
  return best;
}

// Parts of the sums of squares a product of m tokens with n outputs leaves for the norm after
// it: one per 32 weight rows up to 256 tokens, one per tile of weight rows above.
extern "C" int leone_gemm_tc_norm_parts(int m, int n) {
  if (m <= 256) return (n + 31) / 32;
  const int w = leone_gemm_tc_token_major_width(m, n, 0);
  return (n + w - 1) / w;
}

// Workspace floats and counters needed when `split_tiles` tiles are split `splits` ways;
// both 0 when splits == 1.
extern "C" void leone_gemm_tc_scratch(int m, int split_tiles, int splits, long long* workspace_floats,
                                      int* counters) {
  const int bn = leone_gemm_tc_tile(m);
  *workspace_floats = splits > 1 ? (long long)split_tiles * splits * bn * kTileW : 0;
  *counters = splits > 1 ? split_tiles : 0;
}

// Clusters of `splits` blocks that can be resident at once for M tokens (0: not launchable).
extern "C" int leone_gemm_tc_cluster_capacity(int m, int splits) {
  if (m > 256 || splits < 2 || splits > 8) return 0;
  switch (leone_gemm_tc_tile(m)) {
    case 16: return cluster_capacity<16>(splits);
    case 32: return cluster_capacity<32>(splits);
    case 64: return cluster_capacity<64>(splits);
    case 128: return cluster_capacity<128>(splits);
    default: return cluster_capacity<256>(splits);
  }
}

// The same for the token-major form (any number of tokens).
extern "C" int leone_gemm_tc_cluster_capacity_token_major(int splits) {
  if (splits < 2 || splits > 8) return 0;
  return cluster_capacity<256, false>(splits);
}

// x: [m, k] bf16 (row stride ldx), w: [n, k] bf16 (row stride ldw), out: [m, n] (row stride ldc).
// epilogue 0: bf16 out; 1: fp32 out; 2: fp32 out = acc + residual (same layout as out);
// 3: w holds interleaved gate/up rows, out is bf16 [m, n/2] = silu(gate) * up.
// The first `full_tiles` tiles (in the kernel's tile order) are computed whole; the others have K
// split `splits` ways.  splits > 1 needs `workspace` (fp32) and zeroed `counters` of the sizes
// leone_gemm_tc_scratch gives for (tiles - full_tiles).  More than 256 tokens are never split.
// A norm between two products without a kernel of its own:
//  norm_out_x != null (epilogue 1 or 2): also write norm_out_x[m][n] = bf16(out[m][n] * norm_out_w[n])
//    (row stride ld_norm_out) and norm_out_ss[part][m] = sum of out[m][n]^2 over the part's weight
//    rows; leone_gemm_tc_norm_parts(m, n) gives the number of parts;
//  norm_in_ss != null: every output of token m is scaled by rsqrt(sum_p norm_in_ss[p][m] / k + norm_eps)
//    (x is then the norm_out_x another product wrote).
// cluster != 0: the splits of a tile form a thread-block cluster and are summed through
// distributed shared memory (needs full_tiles == 0, 2 <= splits <= 8, at most 256 tokens, and
// tiles * splits blocks resident at once: see leone_gemm_tc_cluster_capacity); workspace and
// counters are not used.
// token_major != 0: the token-major form (128 tokens x 256 weight rows per tile) also for 256
// tokens or fewer, where it reads the token operand less often than the swapped form does; the
// norm arguments must then be null.  The token-major form is split along K only with cluster
// != 0 (same conditions as above, for any number of tokens; no norm arguments).
extern "C" int leone_gemm_tc(const void* x, const void* w, void* out, const float* residual, int m,
                             int n, int k, int ldx, int ldw, int ldc, int epilogue, int splits,
                             int full_tiles, float* workspace, int* counters, int* status,
                             int sm_count, int cluster, int token_major, void* norm_out_x, const float* norm_out_w,
                             float* norm_out_ss, int ld_norm_out, const float* norm_in_ss,
                             int norm_in_parts, float norm_eps, cudaStream_t stream) {
  if (m <= 0 || n <= 0) return 0;
  if (k <= 0 || (k % 8) != 0 || (ldx % 8) != 0 || (ldw % 8) != 0) return kRefusedAlignment;
  if (epilogue < 0 || epilogue > 3 || splits < 1 || sm_count < 1) return kRefusedSize;
  if (epilogue == 2 && residual == nullptr) return kRefusedSize;
  if (epilogue == 3 && (n % 32) != 0) return kRefusedSize;
  const int k_blocks = (k + kTileK - 1) / kTileK;
  const bool swap = m <= 256 && !token_major;
  if (!swap && !cluster) splits = 1;
  if (!swap && (m <= 256 || cluster) && (norm_out_x != nullptr || norm_in_ss != nullptr)) return kRefusedSize;
  if (splits > k_blocks) splits = k_blocks;
  // every split must own at least one k-block
  while (splits > 1 && (splits - 1) * ((k_blocks + splits - 1) / splits) >= k_blocks) --splits;
  if (splits == 1) cluster = 0;
  if (norm_out_x != nullptr && ((epilogue != 1 && epilogue != 2) || norm_out_w == nullptr || norm_out_ss == nullptr))
    return kRefusedSize;
  if (norm_in_ss != nullptr && norm_in_parts < 1) return kRefusedSize;
  if (cluster && (full_tiles != 0 || splits > 8)) return kRefusedSize;
  if (splits > 1 && !cluster && (workspace == nullptr || counters == nullptr)) return kRefusedSize;
  if (splits > 1 && cluster && !swap && workspace == nullptr) return kRefusedSize;
  // the token-major tile's width: 256 when split or forced below the prompt sizes
  const int tm_width = (swap || cluster || m <= 256) ? 256 : leone_gemm_tc_token_major_width(m, n, epilogue == 3);
  const int tiles = swap ? leone_gemm_tc_tiles(m, n)
                         : ((n + tm_width - 1) / tm_width) * ((m + kTileW - 1) / kTileW);
  if (splits == 1) full_tiles = tiles;
  if (full_tiles < 0 || full_tiles > tiles) return kRefusedSize;
  const int bn = leone_gemm_tc_tile(m);
  CUtensorMap mw, mx;
  int r = make_tensor_map_2d(&mw, w, (uint64_t)n, (uint64_t)k, (uint64_t)ldw, swap ? kTileW : (uint32_t)tm_width);
  if (r != 0) return r;
  r = make_tensor_map_2d(&mx, x, (uint64_t)m, (uint64_t)k, (uint64_t)ldx, swap ? (uint32_t)bn : kTileW);
  if (r != 0) return r;
  GemmParams p{out, residual, m, n, k, ldc, epilogue, splits, full_tiles, workspace, counters, status,
               g_gemm_trace, (__nv_bfloat16*)norm_out_x, norm_out_w, norm_out_ss, ld_norm_out, norm_in_ss,
               norm_in_parts, norm_eps, (swap && bn <= 16) ? g_l2_ahead : 0};
  if (g_gemm_trace != nullptr) g_gemm_trace += g_gemm_trace_stride;
  if (!swap && cluster) return launch_gemm<256, false, true>(mw, mx, p, sm_count, stream);
  if (!swap && tm_width == 240) return launch_gemm<240, false>(mw, mx, p, sm_count, stream);
  if (!swap) return launch_gemm<256, false>(mw, mx, p, sm_count, stream);
  if (cluster) {
    switch (bn) {
      case 16: return launch_gemm<16, true, true>(mw, mx, p, sm_count, stream);
      case 32: return launch_gemm<32, true, true>(mw, mx, p, sm_count, stream);
      case 64: return launch_gemm<64, true, true>(mw, mx, p, sm_count, stream);
      case 128: return launch_gemm<128, true, true>(mw, mx, p, sm_count, stream);
      default: return launch_gemm<256, true, true>(mw, mx, p, sm_count, stream);
    }
  }
  switch (bn) {
    case 16: return launch_gemm<16, true>(mw, mx, p, sm_count, stream);
    case 32: return launch_gemm<32, true>(mw, mx, p, sm_count, stream);
    case 64: return launch_gemm<64, true>(mw, mx, p, sm_count, stream);
    case 128: return launch_gemm<128, true>(mw, mx, p, sm_count, stream);
    default: return launch_gemm<256, true>(mw, mx, p, sm_count, stream);
  }
}
