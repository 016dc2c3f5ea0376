// Seeded random weights on the device: element i of a tensor is a pure function of
// (key, i), defined in random_draw.h and computed there bit for bit as on the host
// (random_weights_host.cpp).  A model of any size is drawn in place, in its storage dtype,
// without a file and without a host copy.  The reference has no random-weight mode.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "random_draw.h"

namespace {

// out_kind 0: fp32, 1: bfloat16 (round-to-nearest-even of the fp32 value), 2: int32 table
template <int kOut>
__global__ void random_fill_kernel(unsigned long long key, long long start, long long count, double mean,
                                   double std, void* out) {
    long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        uint64_t index = (uint64_t)(start + i);
        if (kOut == 2) {
            static_cast<int32_t*>(out)[i] = leone_rd::table_entry(key, index);
        } else {
            float v = leone_rd::weight(key, index, mean, std);
            if (kOut == 0) static_cast<float*>(out)[i] = v;
            else static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
        }
    }
}

}  // namespace

extern "C" int leone_random_fill_device(unsigned long long key, long long start, long long count, double mean,
                                        double std, int out_kind, void* out, cudaStream_t stream) {
    if (start < 0 || count < 0 || out == nullptr || out_kind < 0 || out_kind > 2) return -1;
    if (count == 0) return 0;
    int threads = 256;
    long long want = (count + threads - 1) / threads;
    int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
    if (out_kind == 0) random_fill_kernel<0><<<blocks, threads, 0, stream>>>(key, start, count, mean, std, out);
    else if (out_kind == 1) random_fill_kernel<1><<<blocks, threads, 0, stream>>>(key, start, count, mean, std, out);
    else random_fill_kernel<2><<<blocks, threads, 0, stream>>>(key, start, count, mean, std, out);
    return (int)cudaGetLastError();
}
