// out[M,N] = x[M,K] * w[N,K]^T in bfloat16 on the 5th-generation tensor cores.
//
// Orientation.  The weight matrix always rides the MMA's M dimension (128 weight
// rows per tile, one TMEM lane each) and the tokens ride the MMA's N dimension
// (BN = 16..256 tokens per tile).  A decode step with a handful of tokens is
// then a pure weight stream through 128x16 MMAs, and a prompt portion uses
// 128x256 tiles; one kernel serves both.  The reference has a GEMV family for
// decode and a library GEMM for prompts
// (crates/leone-cuda/cuda/ie_cuda.cu:1718, 5069); this kernel replaces both.
//
// Structure (persistent, one block per SM, 6 warps):
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
#include "tc_common.cuh"

namespace leone {
namespace tc {

constexpr int kTileW = 128;     // weight rows per tile = MMA M
constexpr int kTileK = 64;      // one 128-byte swizzle row of bf16
constexpr int kGemmThreads = 192;

template <int BN> struct GemmCfg {
  static constexpr int kStageBytes = kTileW * kTileK * 2 + BN * kTileK * 2;
  static constexpr int kStages = BN <= 16 ? 10 : BN <= 32 ? 9 : BN <= 64 ? 8 : BN <= 128 ? 6 : 4;
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment*/ + 256 /*barriers*/;
};

struct GemmParams {
  void* out;
  const float* residual;
  int M, N, K, ldc;
  int epilogue;
  int splits;
  float* workspace;
  int* counters;
  int* status;
};

template <int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
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
  __shared__ uint32_t tmem_holder;
  __shared__ int gave_up;
  __shared__ int last_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (p.N + kTileW - 1) / kTileW;
  const int m_tiles = (p.M + BN - 1) / BN;
  const int k_blocks = (p.K + kTileK - 1) / kTileK;
  const int kb_per_split = (k_blocks + p.splits - 1) / p.splits;
  const int total = n_tiles * m_tiles * p.splits;

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

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < total && !*giveup; t += gridDim.x) {
        const int split = t % p.splits, tile = t / p.splits;
        const int m_tile = tile % m_tiles, n_tile = tile / m_tiles;
        const int kb0 = split * kb_per_split, kb1 = min(k_blocks, kb0 + kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, giveup)) break;
          const uint32_t dst = tiles_base + stage * Cfg::kStageBytes;
          mbar_expect_tx(full0 + 8 * stage, Cfg::kStageBytes);
          tma_load_2d(dst, &map_w, full0 + 8 * stage, kb * kTileK, n_tile * kTileW);
          tma_load_2d(dst + kTileW * kTileK * 2, &map_x, full0 + 8 * stage, kb * kTileK, m_tile * BN);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
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
        const int split = t % p.splits;
        const int kb0 = split * kb_per_split, kb1 = min(k_blocks, kb0 + kb_per_split);
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(acc_empty0 + 8 * buf, acc_phase ^ 1, giveup)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        bool ok = true;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full0 + 8 * stage, phase, giveup)) { ok = false; break; }
          tc_fence_after();
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
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;                     // TMEM lanes 32*quarter .. +31
    const int ep_tid = (warp - 2) * 32 + lane;        // 0..127
    int it = 0;
    for (int t = blockIdx.x; t < total && !*giveup; t += gridDim.x, ++it) {
      const int split = t % p.splits, tile = t / p.splits;
      const int m_tile = tile % m_tiles, n_tile = tile / m_tiles;
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(acc_full0 + 8 * buf, acc_phase, giveup)) break;
      tc_fence_after();
      const int row_local = quarter * 32 + lane;
      const int n = n_tile * kTileW + row_local;
      const int m0 = m_tile * BN;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
      bool do_epilogue = true;
      if (p.splits > 1) {
        float* ws = p.workspace + ((size_t)tile * p.splits + split) * (BN * kTileW);
        for (int c = 0; c < BN; c += 16) {
          float v[16];
          tmem_ld16(taddr + c, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) ws[(c + j) * kTileW + row_local] = v[j];
        }
        __threadfence();
        named_barrier_sync(1, 128);
        if (ep_tid == 0) {
          const int old = atomicAdd(&p.counters[tile], 1);
          const int last = old == p.splits - 1;
          if (last) p.counters[tile] = 0;      // ready for the next launch
          last_flag = last;
        }
        named_barrier_sync(1, 128);
        do_epilogue = last_flag != 0;
        if (do_epilogue) __threadfence();
      }
      // the accumulator buffer is free once its values are in registers or in the workspace
      if (p.splits > 1) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
      }
      if (do_epilogue) {
        const float* ws_tile = p.splits > 1 ? p.workspace + (size_t)tile * p.splits * (BN * kTileW) : nullptr;
        for (int c = 0; c < BN; c += 16) {
          float v[16];
          if (p.splits > 1) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.f;
            for (int s = 0; s < p.splits; ++s) {
              const float* src = ws_tile + (size_t)s * (BN * kTileW);
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] += __ldcg(src + (c + j) * kTileW + row_local);
            }
          } else {
            tmem_ld16(taddr + c, v);
          }
          if (p.epilogue == 3) {
            // rows come in groups of 32: 16 gate rows then their 16 up rows
            const int col = (n >> 5) * 16 + (lane & 15);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);
              const int m = m0 + c + j;
              if (lane < 16 && n < p.N && m < p.M) {
                const float g = v[j], u = other;
                ((__nv_bfloat16*)p.out)[(size_t)m * p.ldc + col] =
                    __float2bfloat16_rn(g / (1.f + expf(-g)) * u);
              }
            }
          } else if (n < p.N) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int m = m0 + c + j;
              if (m < p.M) {
                const size_t o = (size_t)m * p.ldc + n;
                if (p.epilogue == 0) ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(v[j]);
                else if (p.epilogue == 1) ((float*)p.out)[o] = v[j];
                else ((float*)p.out)[o] = v[j] + p.residual[o];
              }
            }
          }
        }
      }
      if (p.splits == 1) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
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

template <int BN>
int launch_gemm(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, int sm_count,
                cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int n_tiles = (p.N + kTileW - 1) / kTileW, m_tiles = (p.M + BN - 1) / BN;
  const long long total = (long long)n_tiles * m_tiles * p.splits;
  const int grid = (int)(total < sm_count ? total : sm_count);
  gemm_tc_kernel<BN><<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(mw, mx, p);
  return launch_result();
}

}  // namespace tc
}  // namespace leone

using namespace leone;
using namespace leone::tc;

// Token-tile width the kernel will use for M tokens.
extern "C" int leone_gemm_tc_tile(int m) {
  return m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : m <= 128 ? 128 : 256;
}

// Workspace floats and counters needed for (m, n, splits); both 0 when splits == 1.
extern "C" void leone_gemm_tc_scratch(int m, int n, int splits, long long* workspace_floats,
                                      int* counters) {
  const int bn = leone_gemm_tc_tile(m);
  const long long tiles = (long long)((n + kTileW - 1) / kTileW) * ((m + bn - 1) / bn);
  *workspace_floats = splits > 1 ? tiles * splits * bn * kTileW : 0;
  *counters = splits > 1 ? (int)tiles : 0;
}

// x: [m, k] bf16 (row stride ldx), w: [n, k] bf16 (row stride ldw), out: [m, n] (row stride ldc).
// epilogue 0: bf16 out; 1: fp32 out; 2: fp32 out = acc + residual (same layout as out);
// 3: w holds interleaved gate/up rows, out is bf16 [m, n/2] = silu(gate) * up.
// splits > 1 needs `workspace` (fp32) and zeroed `counters` of the sizes leone_gemm_tc_scratch gives.
extern "C" int leone_gemm_tc(const void* x, const void* w, void* out, const float* residual, int m,
                             int n, int k, int ldx, int ldw, int ldc, int epilogue, int splits,
                             float* workspace, int* counters, int* status, int sm_count,
                             cudaStream_t stream) {
  if (m <= 0 || n <= 0) return 0;
  if (k <= 0 || (k % 8) != 0 || (ldx % 8) != 0 || (ldw % 8) != 0) return kRefusedAlignment;
  if (epilogue < 0 || epilogue > 3 || splits < 1 || sm_count < 1) return kRefusedSize;
  if (epilogue == 2 && residual == nullptr) return kRefusedSize;
  if (epilogue == 3 && (n % 32) != 0) return kRefusedSize;
  const int k_blocks = (k + kTileK - 1) / kTileK;
  if (splits > k_blocks) splits = k_blocks;
  // every split must own at least one k-block
  while (splits > 1 && (splits - 1) * ((k_blocks + splits - 1) / splits) >= k_blocks) --splits;
  if (splits > 1 && (workspace == nullptr || counters == nullptr)) return kRefusedSize;
  const int bn = leone_gemm_tc_tile(m);
  CUtensorMap mw, mx;
  int r = make_tensor_map_2d(&mw, w, (uint64_t)n, (uint64_t)k, (uint64_t)ldw, kTileW);
  if (r != 0) return r;
  r = make_tensor_map_2d(&mx, x, (uint64_t)m, (uint64_t)k, (uint64_t)ldx, (uint32_t)bn);
  if (r != 0) return r;
  GemmParams p{out, residual, m, n, k, ldc, epilogue, splits, workspace, counters, status};
  switch (bn) {
    case 16: return launch_gemm<16>(mw, mx, p, sm_count, stream);
    case 32: return launch_gemm<32>(mw, mx, p, sm_count, stream);
    case 64: return launch_gemm<64>(mw, mx, p, sm_count, stream);
    case 128: return launch_gemm<128>(mw, mx, p, sm_count, stream);
    default: return launch_gemm<256>(mw, mx, p, sm_count, stream);
  }
}
