// Shared by the tcgen05 products: tile geometry, the parameters of one product, the work units
// of a launch and the epilogues that finish sums into outputs (all device code is inline).
#pragma once
#include "tc_common.cuh"

namespace leone {
namespace tc {

constexpr int kTileW = 128;     // weight rows per tile = MMA M
constexpr int kTileK = 64;      // one 128-byte swizzle row of bf16
constexpr int kGemmThreads = 192;

// Up to 64 tokens per tile a block keeps about 100 KB of stages, so two blocks (of this kernel
// or of this one and the next) share an SM: while one drains its epilogue the other already
// streams weights.  Larger token tiles take the whole SM.
constexpr int pow2_at_least(int v) {
  int p = 32;
  while (p < v) p *= 2;
  return p;
}
template <int BN> struct GemmCfg {
  static constexpr int kStageBytes = kTileW * kTileK * 2 + BN * kTileK * 2;
  static constexpr int kStages = BN <= 16 ? 5 : BN <= 32 ? 5 : BN <= 64 ? 4 : BN <= 128 ? 6 : 4;
  static constexpr int kBlocksPerSm = BN <= 64 ? 2 : 1;
  static constexpr int kTmemCols = pow2_at_least(2 * BN);      // two accumulators, BN columns apart
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment*/ + 256 /*barriers*/;
};

// Decode-sized token tiles in cluster mode push their partial sums into the shared memory of the
// block that finishes the rows (see the kernel): that block needs an inbox beside its stages, one
// slot of [BN columns][32 rows] floats per (chunk it owns, rank): at most 8 slots.
template <int BN, bool kSwap, bool kCluster> constexpr bool gemm_pushes() { return kCluster && kSwap && BN <= 16; }
template <int BN, bool kSwap, bool kCluster> constexpr int gemm_smem_bytes() {
  return GemmCfg<BN>::kSmemBytes + (gemm_pushes<BN, kSwap, kCluster>() ? 8 * BN * 32 * 4 : 0);
}

struct GemmParams {
  void* out;
  const float* residual;
  int M, N, K, ldc;
  int epilogue;
  int splits;        // K is split this many ways ...
  int full_tiles;    // ... for tiles at or past this index; earlier tiles are not split
  float* workspace;
  int* counters;
  int* status;
  long long* trace;  // optional: 8 nanosecond time stamps per block (see leone_gemm_tc_set_trace)
  // RMSNorm around the product (swapped orientation), so that a norm between two products
  // needs no kernel of its own.  The product before the norm (fp32 output, epilogue 1 or 2)
  // also writes norm_out_x[m][n] = bf16(out[m][n] * norm_out_w[n]) and, per 32 weight rows, the
  // sum of out[m][n]^2 into norm_out_ss[(n / 32)][m]; the product after the norm reads
  // norm_out_x as its token operand and scales every output of token m by
  // rsqrt(sum_p norm_in_ss[p][m] / K + norm_eps), which is W . rmsnorm(out).
  __nv_bfloat16* norm_out_x;
  const float* norm_out_w;
  float* norm_out_ss;
  int ld_norm_out;
  const float* norm_in_ss;
  int norm_in_parts;
  float norm_eps;
  int l2_ahead;      // k-blocks of weights past the early stages that the producer asks the L2 for
};

__device__ __forceinline__ long long global_ns() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)::"memory");
  return t;
}
__device__ __forceinline__ void stamp(const GemmParams& p, int slot) {
  if (p.trace != nullptr) p.trace[(size_t)blockIdx.x * 8 + slot] = global_ns();
}

// Work units in launch order: the unsplit tiles first, then `splits` units per remaining tile.
// Splitting only the tiles of the last, partly filled round keeps every SM busy without
// paying the partial-sum round trip on the others.
struct Unit {
  int tile, split, nsplit;
};
__device__ __forceinline__ Unit unit_of(int u, const GemmParams& p) {
  if (u < p.full_tiles) return Unit{u, 0, 1};
  const int r = u - p.full_tiles;
  return Unit{p.full_tiles + r / p.splits, r % p.splits, p.splits};
}

// SwiGLU of a gate and an up value for a bf16 result: g / (1 + e^-g) * u with the fast exponential
// and division (a few units in the last place of fp32, far below the rounding to bf16; e^-g = inf
// gives g * 0).
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.f + __expf(-g)) * u; }

// Swapped orientation: the thread that owns weight row n finishes NC token columns
// m0 + c .. m0 + c + NC - 1 whose sums are in v (r: the residual values, fetched by the caller
// before anything is stored, because the residual may be the output itself).
// gw_known: the following norm's weight of row n if the caller fetched it already (else null).
template <int NC>
__device__ __forceinline__ void finish_swapped(const GemmParams& p, float (&v)[NC], const float (&r)[NC],
                                               int n, int m0, int c, int lane, const float* rs_s,
                                               const float* gw_known = nullptr) {
  if (p.norm_in_ss != nullptr) {
#pragma unroll
    for (int j = 0; j < NC; ++j) v[j] *= rs_s[c + j];
  }
  if (p.epilogue == 3) {
    // rows come in groups of 32: 16 gate rows (lanes 0-15) then their 16 up rows (lanes 16-31).
    // The halves of the warp swap one value per pair of token columns, so that the lower half
    // finishes the even column and the upper half the odd one (half the arithmetic of letting
    // the lower half finish both, and every store is 32 lanes wide).
    const int col = (n >> 5) * 16 + (lane & 15);
    const bool low = lane < 16;
    static_assert(NC % 2 == 0, "token columns are finished in pairs");
#pragma unroll
    for (int j = 0; j < NC; j += 2) {
      const float x = __shfl_xor_sync(0xffffffffu, low ? v[j + 1] : v[j], 16);
      const float g = low ? v[j] : x, u = low ? x : v[j + 1];
      const int m = m0 + c + j + (low ? 0 : 1);
      if (n < p.N && m < p.M) ((__nv_bfloat16*)p.out)[(size_t)m * p.ldc + col] = __float2bfloat16_rn(silu_mul(g, u));
    }
    return;
  }
  if (n < p.N) {
    if (p.epilogue == 2) {
#pragma unroll
      for (int j = 0; j < NC; ++j) v[j] += r[j];
    }
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      const int m = m0 + c + j;
      if (m < p.M) {
        const size_t o = (size_t)m * p.ldc + n;
        if (p.epilogue == 0) ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(v[j]);
        else ((float*)p.out)[o] = v[j];
      }
    }
  }
  if (p.norm_out_x != nullptr) {
    // the operand of the product after the following norm, and this warp's 32 rows' share of
    // the sums of squares (the lanes of a warp are 32 consecutive weight rows)
    const float gw = gw_known != nullptr ? *gw_known : n < p.N ? p.norm_out_w[n] : 0.f;
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      const int m = m0 + c + j;
      const float val = n < p.N ? v[j] : 0.f;
      if (n < p.N && m < p.M) p.norm_out_x[(size_t)m * p.ld_norm_out + n] = __float2bfloat16_rn(val * gw);
      float sq = val * val;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if (lane == 0 && m < p.M && n < p.N) p.norm_out_ss[(size_t)(n >> 5) * p.M + m] = sq;
    }
  }
}
template <int NC>
__device__ __forceinline__ void fetch_residual(const GemmParams& p, float (&r)[NC], int n, int m0, int c) {
  if (p.epilogue == 2 && n < p.N) {
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      const int m = m0 + c + j;
      r[j] = m < p.M ? p.residual[(size_t)m * p.ldc + n] : 0.f;
    }
  }
}

// The residual values that finish_token_major32 would add to token row m, weight rows n .. n+31
// (zeros where there are none), so that the caller can have them in flight early.
__device__ __forceinline__ void fetch_residual32(const GemmParams& p, float (&r)[32], int m, int n) {
#pragma unroll
  for (int j = 0; j < 32; ++j) r[j] = 0.f;
  if (p.epilogue != 2 || m >= p.M || n >= p.N) return;
  const size_t o = (size_t)m * p.ldc + n;
  if (n + 32 <= p.N && (p.ldc & 3) == 0) {
    const float4* res = reinterpret_cast<const float4*>(p.residual + o);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 q = res[j];
      r[4 * j] = q.x; r[4 * j + 1] = q.y; r[4 * j + 2] = q.z; r[4 * j + 3] = q.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (n + j < p.N) r[j] = p.residual[o + j];
  }
}

// Token-major form, splits summed inside a cluster: 32 finished sums of token row m for the weight
// rows n .. n+31 (n a multiple of 32) go out through the product's epilogue.  No folded norm.
// residual_added: the caller has added the residual already (fetch_residual32).
__device__ __forceinline__ void finish_token_major32(const GemmParams& p, float (&v)[32], int m, int n,
                                                     bool residual_added = false) {
  if (m >= p.M || n >= p.N) return;
  const bool vec_ok = (p.ldc & 7) == 0;
  if (p.epilogue == 3) {                                 // 16 gate columns, then their 16 up columns
    __nv_bfloat16* orow = (__nv_bfloat16*)p.out + (size_t)m * p.ldc;
    const int col = n >> 1;
    uint32_t packed[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = silu_mul(v[2 * j], v[16 + 2 * j]);
      const float b = silu_mul(v[2 * j + 1], v[16 + 2 * j + 1]);
      __nv_bfloat162 v2 = __floats2bfloat162_rn(a, b);
      packed[j] = *reinterpret_cast<uint32_t*>(&v2);
    }
    if (vec_ok) {
      uint4* dst = reinterpret_cast<uint4*>(orow + col);
      dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) *reinterpret_cast<uint32_t*>(orow + col + 2 * j) = packed[j];
    }
    return;
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int nn = n + 16 * h;
    if (nn >= p.N) break;
    float* vv = v + 16 * h;
    const size_t o = (size_t)m * p.ldc + nn;
    const bool full = nn + 16 <= p.N && vec_ok;
    if (p.epilogue == 0) {
      __nv_bfloat16* dst = (__nv_bfloat16*)p.out + o;
      if (full) {
        uint32_t packed[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          __nv_bfloat162 v2 = __floats2bfloat162_rn(vv[2 * j], vv[2 * j + 1]);
          packed[j] = *reinterpret_cast<uint32_t*>(&v2);
        }
        reinterpret_cast<uint4*>(dst)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        reinterpret_cast<uint4*>(dst)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
      } else {
        for (int j = 0; j < 16 && nn + j < p.N; ++j) dst[j] = __float2bfloat16_rn(vv[j]);
      }
    } else {
      float* dst = (float*)p.out + o;
      if (full) {
        if (p.epilogue == 2 && !residual_added) {
          const float4* res = reinterpret_cast<const float4*>(p.residual + o);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float4 r = res[j];
            vv[4 * j] += r.x; vv[4 * j + 1] += r.y; vv[4 * j + 2] += r.z; vv[4 * j + 3] += r.w;
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          reinterpret_cast<float4*>(dst)[j] = make_float4(vv[4 * j], vv[4 * j + 1], vv[4 * j + 2], vv[4 * j + 3]);
      } else {
        for (int j = 0; j < 16 && nn + j < p.N; ++j) {
          if (p.epilogue == 2 && !residual_added) vv[j] += p.residual[o + j];
          dst[j] = vv[j];
        }
      }
    }
  }
}

// Token-major form: the thread that owns token row m finishes the tile's bn weight rows from n0
// on (tile n_tile; bn a multiple of 16, of 32 with the SwiGLU epilogue), 16 at a time, from tensor
// memory at taddr: the norm's factor before, the product's epilogue, and the operand and sum of
// squares of a norm after it.  Warp-wide (the loads from tensor memory are), so every thread of
// the warp calls it, rows past M too.
__device__ __forceinline__ void finish_token_major_row(const GemmParams& p, uint32_t taddr, int m, int n0,
                                                       int n_tile, const int bn) {
  const bool vec_ok = (p.ldc & 7) == 0;
  // the norm before this product: this row's factor from the parts the product before left
  float rs = 1.f;
  if (p.norm_in_ss != nullptr) {
    float ss = 0.f;
    if (m < p.M)
      for (int q = 0; q < p.norm_in_parts; ++q) ss += p.norm_in_ss[(size_t)q * p.M + m];
    rs = rsqrtf(ss / (float)p.K + p.norm_eps);
  }
  // the norm after this product: this row's sum of squares over the tile's columns, and
  // bf16(out * weight) beside the output (token-major: one part per tile of BN columns)
  float ssq = 0.f;
  auto norm_out16 = [&](const float (&val)[16], int n) {      // 16 finished outputs from column n
    if (p.norm_out_x != nullptr && m < p.M && n < p.N) {
      uint32_t packed[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float a = n + 2 * j < p.N ? val[2 * j] : 0.f, b = n + 2 * j + 1 < p.N ? val[2 * j + 1] : 0.f;
        ssq = fmaf(a, a, fmaf(b, b, ssq));
        __nv_bfloat162 v2 = __floats2bfloat162_rn(a * (n + 2 * j < p.N ? p.norm_out_w[n + 2 * j] : 0.f),
                                                  b * (n + 2 * j + 1 < p.N ? p.norm_out_w[n + 2 * j + 1] : 0.f));
        packed[j] = *reinterpret_cast<uint32_t*>(&v2);
      }
      __nv_bfloat16* xrow = p.norm_out_x + (size_t)m * p.ld_norm_out + n;
      if (n + 16 <= p.N && (p.ld_norm_out & 7) == 0) {
        reinterpret_cast<uint4*>(xrow)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        reinterpret_cast<uint4*>(xrow)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
      } else {
        for (int j = 0; j < 16 && n + j < p.N; ++j)
          xrow[j] = __float2bfloat16_rn(val[j] * p.norm_out_w[n + j]);
      }
    }
  };
  if (p.epilogue == 3) {
    __nv_bfloat16* orow = (__nv_bfloat16*)p.out + (size_t)m * p.ldc;
    for (int c = 0; c < bn; c += 32) {             // 16 gate columns, then their 16 up columns
      float g[16], u[16];
      tmem_ld16(taddr + c, g);
      tmem_ld16(taddr + c + 16, u);
      if (p.norm_in_ss != nullptr) {
#pragma unroll
        for (int j = 0; j < 16; ++j) { g[j] *= rs; u[j] *= rs; }
      }
      const int col = (n0 + c) >> 1;
      if (m < p.M && n0 + c < p.N) {
        uint32_t packed[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float a = silu_mul(g[2 * j], u[2 * j]);
          const float b = silu_mul(g[2 * j + 1], u[2 * j + 1]);
          __nv_bfloat162 v2 = __floats2bfloat162_rn(a, b);
          packed[j] = *reinterpret_cast<uint32_t*>(&v2);
        }
        if (vec_ok) {
          uint4* dst = reinterpret_cast<uint4*>(orow + col);
          dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) *reinterpret_cast<uint32_t*>(orow + col + 2 * j) = packed[j];
        }
      }
    }
  } else if (p.epilogue == 2 && vec_ok && n0 + bn <= p.N) {
    // fp32 out = acc + residual for a whole row of the tile: the residual is fetched three
    // chunks ahead of its use, so its latency is paid once per row, not once per chunk
    // (the residual may be the output itself: a chunk is read before it is written, and
    // chunks do not overlap).  The branch is the same for every thread of the block, as
    // the warp-wide tensor-memory loads need; rows past M read row 0 and store nothing.
    constexpr int kAhead = 3;
    const bool row_ok = m < p.M;
    const size_t row_at = (size_t)(row_ok ? m : 0) * p.ldc + n0;
    const float4* res = reinterpret_cast<const float4*>(p.residual + row_at);
    float4* dst = reinterpret_cast<float4*>((float*)p.out + row_at);
    const int chunks = bn / 16;
    float4 rb[kAhead][4];
#pragma unroll
    for (int a = 0; a < kAhead; ++a) {
      if (a < chunks) {
#pragma unroll
        for (int j = 0; j < 4; ++j) rb[a][j] = res[a * 4 + j];
      }
    }
    for (int i0 = 0; i0 < chunks; i0 += kAhead) {
#pragma unroll
      for (int a = 0; a < kAhead; ++a) {        // chunk i0 + a uses and refills slot a
        const int i = i0 + a;
        if (i >= chunks) break;
        float v[16];
        tmem_ld16(taddr + i * 16, v);
        float4 r[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) r[j] = rb[a][j];
        if (i + kAhead < chunks) {
#pragma unroll
          for (int j = 0; j < 4; ++j) rb[a][j] = res[(i + kAhead) * 4 + j];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[4 * j] += r[j].x; v[4 * j + 1] += r[j].y; v[4 * j + 2] += r[j].z; v[4 * j + 3] += r[j].w;
        }
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            dst[i * 4 + j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
        norm_out16(v, n0 + i * 16);
      }
    }
  } else {
    for (int c = 0; c < bn; c += 16) {
      float v[16];
      tmem_ld16(taddr + c, v);
      const int n = n0 + c;
      if (m >= p.M || n >= p.N) continue;
      if (p.norm_in_ss != nullptr) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] *= rs;
      }
      const size_t o = (size_t)m * p.ldc + n;
      const bool full = n + 16 <= p.N && vec_ok;
      if (p.epilogue == 0) {
        __nv_bfloat16* dst = (__nv_bfloat16*)p.out + o;
        if (full) {
          uint32_t packed[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            __nv_bfloat162 v2 = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
            packed[j] = *reinterpret_cast<uint32_t*>(&v2);
          }
          reinterpret_cast<uint4*>(dst)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          reinterpret_cast<uint4*>(dst)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        } else {
          for (int j = 0; j < 16 && n + j < p.N; ++j) dst[j] = __float2bfloat16_rn(v[j]);
        }
      } else {
        float* dst = (float*)p.out + o;
        if (full) {
          if (p.epilogue == 2) {
            const float4* res = reinterpret_cast<const float4*>(p.residual + o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float4 r = res[j];
              v[4 * j] += r.x; v[4 * j + 1] += r.y; v[4 * j + 2] += r.z; v[4 * j + 3] += r.w;
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j)
            reinterpret_cast<float4*>(dst)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
          for (int j = 0; j < 16 && n + j < p.N; ++j) {
            if (p.epilogue == 2) v[j] += p.residual[o + j];
            dst[j] = v[j];
          }
        }
        norm_out16(v, n);
      }
    }
  }
  if (p.norm_out_x != nullptr && m < p.M) p.norm_out_ss[(size_t)n_tile * p.M + m] = ssq;
}
template <int BN>
__device__ __forceinline__ void finish_token_major_row(const GemmParams& p, uint32_t taddr, int m, int n0,
                                                       int n_tile) {
  finish_token_major_row(p, taddr, m, n0, n_tile, BN);
}

}  // namespace tc
}  // namespace leone
