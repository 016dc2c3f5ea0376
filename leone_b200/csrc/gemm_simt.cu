// C[M,N] = A[M,K] * W[N,K]^T on CUDA cores with fp32 FMA accumulation.
//
// This is the matrix product of the true 32-bit path (no tensor cores, no
// reduced-precision mode) and the any-size product of the bfloat16 path for
// shapes the tensor-core kernel refuses.  y[r] = sum_c W[r,c] x[c], weights
// row-major [out][in] (crates/leone/src/cpu.rs:1622-1640).  Each output
// element sums over k in ascending order whatever M is, so a token's result
// does not depend on what else is in the batch.
//
// Epilogues: 0 store in the input type; 1 store fp32; 2 store fp32 = acc + residual
// (residual may alias the output: each element is read then written by one thread).
#include "common.cuh"

namespace leone {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename T, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ W, void* Cv,
                 const float* residual, int M, int N, int K, int lda, int ldw, int ldc) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int ty = tid >> 4, tx = tid & 15;
  const int lr = tid >> 2, lk = (tid & 3) * 4;   // loader: row within tile, first k
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const T* a_row = A + (size_t)(m0 + lr) * lda;
  const T* w_row = W + (size_t)(n0 + lr) * ldw;
  const bool a_ok = m0 + lr < M, w_ok = n0 + lr < N;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      As[lk + i][lr] = (a_ok && k < K) ? to_float<T>(a_row[k]) : 0.f;
      Ws[lk + i][lr] = (w_ok && k < K) ? to_float<T>(w_row[k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      const size_t o = (size_t)m * ldc + n;
      if (EPI == 0) ((T*)Cv)[o] = from_float<T>(acc[i][j]);
      else if (EPI == 1) ((float*)Cv)[o] = acc[i][j];
      else ((float*)Cv)[o] = acc[i][j] + residual[o];
    }
  }
}

}  // namespace leone

using namespace leone;

extern "C" int leone_gemm_simt(int dtype, int epilogue, const void* a, const void* w, void* c,
                               const float* residual, int m, int n, int k, int lda, int ldw,
                               int ldc, cudaStream_t stream) {
  if (m <= 0 || n <= 0) return 0;
  if (k <= 0 || lda < k || ldw < k || ldc < n) return kRefusedSize;
  if (epilogue == 2 && residual == nullptr) return kRefusedSize;
  dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM);
  if (grid.y > 65535) return kRefusedSize;
#define LAUNCH(T, E)                                                                       \
  gemm_simt_kernel<T, E><<<grid, 256, 0, stream>>>((const T*)a, (const T*)w, c, residual, m, \
                                                   n, k, lda, ldw, ldc)
  if (dtype == 0) {
    if (epilogue == 0) LAUNCH(float, 0);
    else if (epilogue == 1) LAUNCH(float, 1);
    else if (epilogue == 2) LAUNCH(float, 2);
    else return kRefusedSize;
  } else if (dtype == 1) {
    if (epilogue == 0) LAUNCH(__nv_bfloat16, 0);
    else if (epilogue == 1) LAUNCH(__nv_bfloat16, 1);
    else if (epilogue == 2) LAUNCH(__nv_bfloat16, 2);
    else return kRefusedSize;
  } else {
    return kRefusedDtype;
  }
#undef LAUNCH
  return launch_result();
}
