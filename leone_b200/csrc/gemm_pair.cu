// out[M,N] = x[M,K] * w[N,K]^T for more than 128 tokens on pairs of SMs (tcgen05 with cta_group::2).
//
// The token-major form of gemm_tc.cu (128 tokens on the MMA's M side, a tile of weight rows on
// its N side) spends 48 KB of operands per k-block and SM.  Here two blocks on neighbouring SMs
// (a cluster of two) work on one tile of 256 tokens x BN weight rows: each block loads its own
// 128 token rows and HALF of the tile's weight rows (at BN = 256: 32 KB per k-block and SM, a
// third less, and seven stages instead of four in the same shared memory), the first block issues one MMA of
// M = 256 per 16 elements of K that reads both blocks' shared memory, and each block's tensor
// memory receives the accumulators of its own 128 token rows, which it finishes exactly as the
// single-block kernel does (same epilogue code: bf16 / fp32 / fp32 + residual / SwiGLU, and the
// RMSNorm folded into the products around it).
//
// BN is a launch argument, any multiple of 16 from 32 to 256 (of 32 with the SwiGLU epilogue): the
// caller picks the width whose tiles cost the fewest rounds over the pairs (the k-loop's time
// follows the bytes a block copies per k-block, so a narrower tile is cheaper by less than its
// width); narrower tiles have smaller stages, so the ring holds more of them (up to ten).
//
// Per block: warp 0 loads (TMA loads into its own shared memory, no multicast; both blocks' loads
// count their bytes on the FIRST block's barrier, which is what the cta_group::2 form of the copy
// is for), warp 1 of the first block issues the MMAs, warps 2..5 run the epilogue.  The MMAs' completion is
// committed to both blocks' barriers (tcgen05.commit with a two-block mask): stage free, and
// accumulator ready.  The second block's epilogue warps release an accumulator by arriving on
// the first block's barrier.  Every wait is bounded; a wait that runs out sets the status word
// and the block goes on to the end, where one cluster barrier keeps either block's shared
// memory and barriers alive until both are done.
#include "gemm_parts.cuh"

namespace leone {
namespace tc {

constexpr int kPairMaxStages = 10;
constexpr int kPairThreads = 192;
constexpr int kPairSmemLimit = 226 * 1024;             // dynamic shared memory of a block (the static part is beside it)

// Shared memory of a pair's block for tiles of bn weight rows: stages of 128 token rows and bn / 2
// weight rows (each operand tile starts on a 1024-byte boundary, as the 128-byte swizzle wants).
struct PairShape {
  int half, stage_bytes, stages, smem_bytes;
};
__host__ __device__ inline PairShape pair_shape(int bn) {
  PairShape c;
  c.half = bn / 2;
  c.stage_bytes = kTileW * kTileK * 2 + ((c.half * kTileK * 2 + 1023) & ~1023);
  c.stages = (kPairSmemLimit - 1024 /*alignment*/ - 256 /*barriers*/) / c.stage_bytes;
  if (c.stages > kPairMaxStages) c.stages = kPairMaxStages;
  c.smem_bytes = c.stages * c.stage_bytes + 1024 + 256;
  return c;
}

__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on the barrier at this offset in both blocks of the pair when every MMA issued so
// far by this thread is done.
__device__ __forceinline__ void umma2_commit_both(uint32_t bar, uint32_t lead) {
  const unsigned short mask = (unsigned short)(3u << lead);      // the pair's two blocks, by rank in the cluster
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(mask)
      : "memory");
}
// Tensor memory of a pair: one warp of each block, the same warp index in both.
__device__ __forceinline__ void tmem_alloc2(uint32_t holder_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder_smem), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// 2-D tile load into this block's shared memory whose bytes are counted on a barrier of the
// pair's first block (bar_cluster: its address from cluster_map).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0,
                                                 int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"((uint64_t)map), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}
// An arrival on a barrier of another block of the cluster (address from cluster_map).
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// The bounded wait of tc_common.cuh for a barrier that another block of the cluster arrives on.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* gave_up) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long start = clock64();
  while (true) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if (*gave_up) return false;
    if (clock64() - start > kWaitLimitCycles) {
      *gave_up = 1;
      return false;
    }
  }
}

// The pair's work: tile t of the launch is token rows [256 * (t % m_pairs), + 256) x weight rows
// [BN * (t / m_pairs), + BN); pair q takes tiles q, q + pairs, ...
//
// With p.splits = S > 1 (clusters of 2 S blocks, one tile per cluster, BN 128 or 256): the S pairs of
// a cluster each take a share of the k-blocks of the same tile.  Every block then leaves its 128
// rows of partial sums in the workspace (L2), [block][chunk of 32 rows][column][row of the chunk];
// after a cluster barrier the tile's eight chunks are dealt to the 2 S blocks, and the block that
// finishes a chunk copies its S pieces into the (now free) stages with the copy engine, adds
// them in split order on top of the residual values and runs the epilogue (no folded norm).
__global__ void __launch_bounds__(kPairThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 const GemmParams p, const int BN) {
  const PairShape cfg = pair_shape(BN);
  const int kStages = cfg.stages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (tiles_base - raw);
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + kStages * cfg.stage_bytes);
  // barriers: full[kStages] (used in the pair's first block), empty[kStages], acc_full[2], acc_empty[2],
  // and for the split mode: the pieces of a chunk have landed, and all four warps have read them
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * kStages;
  const uint32_t acc_full0 = empty0 + 8 * kStages, acc_empty0 = acc_full0 + 16;
  const uint32_t landed = acc_empty0 + 16, pieces_read = landed + 8;
  __shared__ uint32_t tmem_holder;
  __shared__ int gave_up;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t crank = cluster_ctarank();            // 0 .. 2 S - 1
  const uint32_t rank = crank & 1u;                    // within the pair
  const uint32_t lead = crank & ~1u;                   // the pair's first block, by rank in the cluster
  const int S = p.splits, split = (int)(crank >> 1);
  const int n_tiles = (p.N + BN - 1) / BN;
  const int m_tiles = (p.M + kTileW - 1) / kTileW;
  const int m_pairs = (m_tiles + 1) / 2;
  const int total = n_tiles * m_pairs;
  // unsplit: pair q of the grid walks tiles q, q + pairs, ..; split: cluster q has tile q only
  const int pair = blockIdx.x / (2 * S), pairs = S == 1 ? gridDim.x >> 1 : total;
  const int all_k_blocks = (p.K + kTileK - 1) / kTileK;
  const int k_share = (all_k_blocks + S - 1) / S;
  const int kb_lo = split * k_share, kb_hi = min(all_k_blocks, kb_lo + k_share);

  if (threadIdx.x == 0) {
    gave_up = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 8);               // four epilogue warps of each block (used in the first)
    }
    mbar_init(landed, 1);
    mbar_init(pieces_read, 4);
    mbar_fence_init();
    tma_prefetch_desc(&map_w);
    tma_prefetch_desc(&map_x);
  }
  __syncthreads();
  cluster_sync_all();                                  // both blocks' barriers exist before anything arrives on them
  if (warp == 1) tmem_alloc2(smem_u32(&tmem_holder), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_holder;
  volatile int* giveup = &gave_up;
  pdl_trigger();

  if (warp == 0) {
    // ---------------- producer (both blocks) ----------------
    // As in the single-block kernel the weight halves of the first stages are requested before
    // the wait for the kernel before this one, whose output is the token operand.
    if (lane == 0) {
      int early = 0;
      for (int pass = 0; pass < 2; ++pass) {
        int stage = 0, filled = 0;
        uint32_t phase = 0;
        bool stop = false;
        for (int t = pair; t < total && !*giveup && !stop; t += pairs) {
          const int m_tile = (t % m_pairs) * 2 + (int)rank, n_tile = t / m_pairs;
          for (int kb = kb_lo; kb < kb_hi; ++kb, ++filled) {
            if (pass == 0 && filled == kStages) { stop = true; break; }
            const bool had_weights = pass == 1 && filled < early;
            if (pass == 1 && !had_weights && !mbar_wait_cluster(empty0 + 8 * stage, phase ^ 1, giveup)) {
              stop = true;
              break;
            }
            const uint32_t dst = tiles_base + stage * cfg.stage_bytes;
            const uint32_t bar = cluster_map(full0 + 8 * stage, lead);   // the first block's barrier counts both blocks' bytes
            if (!had_weights) {
              if (rank == 0) mbar_expect_tx(full0 + 8 * stage, 2 * (kTileW * kTileK * 2 + cfg.half * kTileK * 2));
              tma_load_2d_pair(dst + kTileW * kTileK * 2, &map_w, bar, kb * kTileK, n_tile * BN + (int)rank * cfg.half);
            }
            if (pass == 1) tma_load_2d_pair(dst, &map_x, bar, kb * kTileK, m_tile * kTileW);
            if (++stage == kStages) { stage = 0; phase ^= 1; }
          }
        }
        if (pass == 0) {
          early = filled;
          pdl_wait();
        }
      }
    }
  } else if (warp == 1 && rank == 1) {
    // the second block's warp 1 has nothing to do between allocating and freeing tensor memory
  } else if (warp == 1) {
    // ---------------- MMA issuer (the first block) ----------------
    if (lane == 0) {
      const uint32_t idesc = instr_desc_bf16(2 * kTileW, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int t = pair; t < total && !*giveup; t += pairs, ++it) {
        const int buf = it & 1;
        if (!mbar_wait_cluster(acc_empty0 + 8 * buf, (((it >> 1) & 1) ^ 1), giveup)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * 256;
        bool ok = true;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait_cluster(full0 + 8 * stage, phase, giveup)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = tiles_base + stage * cfg.stage_bytes;
          const uint32_t b_addr = a_addr + kTileW * kTileK * 2;
          const uint64_t a_desc = smem_desc_sw128(a_addr), b_desc = smem_desc_sw128(b_addr);
#pragma unroll
          for (int k = 0; k < kTileK / 16; ++k)
            umma2_bf16(tmem_d, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > kb_lo || k > 0) ? 1u : 0u);
          umma2_commit_both(empty0 + 8 * stage, lead);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma2_commit_both(acc_full0 + 8 * buf, lead);
      }
    }
  } else {
    // ---------------- epilogue (both blocks) ----------------
    const int quarter = warp & 3;                     // TMEM lanes 32*quarter .. +31
    int it = 0;
    pdl_wait();      // outputs and residual may be in use until here
    for (int t = pair; t < total && !*giveup; t += pairs, ++it) {
      const int m_tile = (t % m_pairs) * 2 + (int)rank, n_tile = t / m_pairs;
      const int buf = it & 1;
      bool ok = mbar_wait_cluster(acc_full0 + 8 * buf, (it >> 1) & 1, giveup);
      ok = __all_sync(0xffffffffu, ok);                // the loads from tensor memory are warp-wide
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * 256;
      if (S > 1) {
        // this block's 128 rows of partial sums go to the workspace; one tile per cluster
        float* ws = p.workspace + (size_t)blockIdx.x * ((size_t)BN * kTileW) + (size_t)quarter * (BN * 32) + lane;
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld32_issue(taddr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) ws[(c + j) * 32] = __uint_as_float(r[j]);
        }
        __threadfence();
        break;
      }
      finish_token_major_row(p, taddr, m_tile * kTileW + quarter * 32 + lane, n_tile * BN, n_tile, BN);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(acc_empty0 + 8 * buf);
        else mbar_arrive_remote(cluster_map(acc_empty0 + 8 * buf, lead));
      }
    }
  }

  if (S > 1) {
    // Every thread of every block of the cluster comes here (all loops above are bounded).
    __syncwarp();
    cluster_sync_all();                                // all partial tiles are in the workspace
    if (warp >= 2 && pair < total && !*giveup) {
      const int m_pair = pair % m_pairs, n_tile = pair / m_pairs;
      const int groups = BN / 128;                     // groups of 32 columns per warp: 1 or 2
      const uint32_t piece = (uint32_t)BN * 32 * 4;    // one block's partial sums of a chunk
      const float* ws_cluster = p.workspace + (size_t)(blockIdx.x - crank) * ((size_t)BN * kTileW);
      const float* box = reinterpret_cast<const float*>(aligned);
      const int et = (warp - 2) * 32 + lane;
      uint32_t landed_phase = 0, read_phase = 0;
      bool first = true;
      for (int ch = (int)crank; ch < 8; ch += 2 * S) { // chunk ch: rows 32 ch .. of the tile's 256
        const int half = ch >> 2, q4 = ch & 3;         // whose rows they are in every pair, and which quarter
        const int m = (m_pair * 2 + half) * kTileW + q4 * 32 + lane;
        const int n0 = n_tile * BN + (warp & 3) * (BN / 4);
        float v[2][32];
#pragma unroll
        for (int g = 0; g < 2; ++g)
          if (g < groups) fetch_residual32(p, v[g], m, n0 + g * 32);
        if (et == 0) {
          // the pieces of the chunk before have been read by all four warps (a wait that runs out
          // requests nothing, and the others' waits run out too)
          bool go = true;
          if (!first) {
            go = mbar_wait(pieces_read, read_phase, giveup);
            read_phase ^= 1;
          }
          if (go) {
            fence_proxy_async();
            mbar_expect_tx(landed, (uint32_t)S * piece);
            for (int u = 0; u < S; ++u)
              bulk_load(tiles_base + (uint32_t)u * piece,
                        ws_cluster + (size_t)(2 * u + half) * ((size_t)BN * kTileW) + (size_t)q4 * (BN * 32), piece, landed);
          }
        }
        first = false;
        if (!mbar_wait(landed, landed_phase, giveup)) break;
        landed_phase ^= 1;
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          if (g < groups) {
            const float* src = box + (size_t)((warp & 3) * (BN / 4) + g * 32) * 32 + lane;
            for (int u = 0; u < S; ++u) {                // split order
#pragma unroll
              for (int j = 0; j < 32; ++j) v[g][j] += src[(size_t)u * (BN * 32) + j * 32];
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(pieces_read);
#pragma unroll
        for (int g = 0; g < 2; ++g)
          if (g < groups) finish_token_major32(p, v[g], m, n0 + g * 32, true);
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (gave_up) {
    if (threadIdx.x == 0) set_status(p.status, kWaitTimeout, blockIdx.x, 5);
    // let tile copies that are still in flight land before the block's memory goes away
    const long long start = clock64();
    while (clock64() - start < 200000) {}
    __syncthreads();
  }
  cluster_sync_all();                                  // neither block's memory goes away under the other
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, 512);
  }
}

static int configure_pair() {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemLimit);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return 0;
}

// Clusters of 2 * splits blocks that can be resident at once for tiles of bn weight rows (0: none).
int pair_cluster_capacity(int bn, int splits) {
  if (configure_pair() != 0) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2u * (unsigned)splits * 64u);
  cfg.blockDim = dim3(kPairThreads);
  cfg.dynamicSmemBytes = (size_t)pair_shape(bn).smem_bytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2u * (unsigned)splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, gemm_pair_kernel, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return clusters;
}

int launch_pair(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, int bn, int sm_count,
                cudaStream_t stream) {
  int r = configure_pair();
  if (r != 0) return r;
  const int n_tiles = (p.N + bn - 1) / bn, m_pairs = ((p.M + kTileW - 1) / kTileW + 1) / 2;
  const long long total = (long long)n_tiles * m_pairs;
  if (p.splits > 1) {
    // one tile per cluster of 2 * splits blocks, all clusters resident at once
    if (total > pair_cluster_capacity(bn, p.splits)) return kRefusedSize;
    return launch_kernel_cluster(gemm_pair_kernel, dim3((unsigned)(total * 2 * p.splits)), dim3(kPairThreads),
                                 (size_t)pair_shape(bn).smem_bytes, stream, dim3(2u * (unsigned)p.splits), mw, mx, p, bn);
  }
  const int pairs = (int)(total < sm_count / 2 ? total : sm_count / 2);
  return launch_kernel_cluster(gemm_pair_kernel, dim3(2u * (unsigned)pairs), dim3(kPairThreads),
                               (size_t)pair_shape(bn).smem_bytes, stream, dim3(2), mw, mx, p, bn);
}

}  // namespace tc
}  // namespace leone

using namespace leone;
using namespace leone::tc;

// The token-major product of gemm_tc.cu for more than 256 tokens on pairs of SMs: the same
// arguments and epilogues (0 bf16, 1 fp32, 2 fp32 += residual, 3 SwiGLU) and the same norm
// arguments; `width`: weight rows per tile, a multiple of 16 from 32 to 256 (of 32 with the SwiGLU
// epilogue); the sums of squares of a folded norm have one part per tile of that width.
// `splits` > 1: the tile's k-blocks are shared among that many pairs (see the kernel).
extern "C" int leone_gemm_pair(const void* x, const void* w, void* out, const float* residual, int m, int n, int k,
                               int ldx, int ldw, int ldc, int epilogue, int width, int splits, float* workspace,
                               int* status, int sm_count, void* norm_out_x, const float* norm_out_w,
                               float* norm_out_ss, int ld_norm_out, const float* norm_in_ss, int norm_in_parts,
                               float norm_eps, cudaStream_t stream) {
  if (m <= 0 || n <= 0) return 0;
  if (k <= 0 || (k % 8) != 0 || (ldx % 8) != 0 || (ldw % 8) != 0) return kRefusedAlignment;
  if (epilogue < 0 || epilogue > 3 || sm_count < 2 || width < 32 || width > 256 || (width % 16) != 0) return kRefusedSize;
  if (epilogue == 2 && residual == nullptr) return kRefusedSize;
  if (epilogue == 3 && ((n % 32) != 0 || (width % 32) != 0)) return kRefusedSize;
  if (norm_out_x != nullptr && ((epilogue != 1 && epilogue != 2) || norm_out_w == nullptr || norm_out_ss == nullptr))
    return kRefusedSize;
  if (norm_in_ss != nullptr && norm_in_parts < 1) return kRefusedSize;
  if (splits != 1) {
    // split along K: 2 or 4 pairs per tile, tiles of 128 or 256 weight rows, every pair with at
    // least four k-blocks, partial sums through the workspace, no folded norm
    if ((splits != 2 && splits != 4) || (width != 128 && width != 256) || workspace == nullptr) return kRefusedSize;
    if (norm_out_x != nullptr || norm_in_ss != nullptr) return kRefusedSize;
    const int k_blocks = (k + kTileK - 1) / kTileK, share = (k_blocks + splits - 1) / splits;
    if (share < 4 || share * (splits - 1) >= k_blocks) return kRefusedSize;
  }
  CUtensorMap mw, mx;
  int r = make_tensor_map_2d(&mw, w, (uint64_t)n, (uint64_t)k, (uint64_t)ldw, (uint32_t)(width / 2));
  if (r != 0) return r;
  r = make_tensor_map_2d(&mx, x, (uint64_t)m, (uint64_t)k, (uint64_t)ldx, kTileW);
  if (r != 0) return r;
  GemmParams p{out, residual, m, n, k, ldc, epilogue, splits, 0, workspace, nullptr, status, nullptr,
               (__nv_bfloat16*)norm_out_x, norm_out_w, norm_out_ss, ld_norm_out, norm_in_ss, norm_in_parts, norm_eps, 0};
  return launch_pair(mw, mx, p, width, sm_count, stream);
}

// Tiles of `width` weight rows whose clusters of 2 * splits blocks can be resident at once, and the
// workspace floats a product split that way needs.
extern "C" int leone_gemm_pair_capacity(int width, int splits) {
  if ((splits != 2 && splits != 4) || (width != 128 && width != 256)) return 0;
  return pair_cluster_capacity(width, splits);
}
extern "C" long long leone_gemm_pair_workspace_floats(int m, int n, int width, int splits) {
  if (splits <= 1) return 0;
  const long long tiles = (long long)((n + width - 1) / width) * (((m + kTileW - 1) / kTileW + 1) / 2);
  return tiles * 2 * splits * width * kTileW;
}
