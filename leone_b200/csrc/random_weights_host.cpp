// Seeded random weights on the host: fills a CPU buffer with elements [start, start + count)
// of the tensor keyed `key`, as random_draw.h defines them.  The device side
// (random_weights.cu) computes the same function, so both give the same bits.
// Must be compiled with -ffp-contract=off (no fused multiply-add; see random_draw.h).
#include <algorithm>
#include <cstdint>
#include <thread>
#include <vector>

#include "random_draw.h"

namespace {

template <typename Fn>
void parallel_chunks(long long count, Fn fn) {
  const long long kGrain = 1 << 16;
  unsigned workers = std::max(1u, std::min(std::thread::hardware_concurrency(), 64u));
  if (count <= kGrain || workers == 1) {
    fn(0, count);
    return;
  }
  workers = (unsigned)std::min<long long>(workers, (count + kGrain - 1) / kGrain);
  long long per = (count + workers - 1) / workers;
  std::vector<std::thread> pool;
  for (unsigned w = 0; w < workers; ++w) {
    long long lo = w * per, hi = std::min(count, lo + per);
    if (lo >= hi) break;
    pool.emplace_back([=] { fn(lo, hi); });
  }
  for (auto& t : pool) t.join();
}

}  // namespace

extern "C" {

// kind 0: fp32 normal draws mean + std * z into `out` (float*); kind 1: 15-bit integers
// into `out` (int32_t*).  Returns 0, or -1 for a bad argument.
int leone_random_fill_host(unsigned long long key, long long start, long long count, double mean,
                           double std, int kind, void* out) {
  if (start < 0 || count < 0 || out == nullptr || (kind != 0 && kind != 1)) return -1;
  if (kind == 0) {
    float* dst = static_cast<float*>(out);
    parallel_chunks(count, [=](long long lo, long long hi) {
      for (long long i = lo; i < hi; ++i)
        dst[i] = leone_rd::weight(key, (uint64_t)(start + i), mean, std);
    });
  } else {
    int32_t* dst = static_cast<int32_t*>(out);
    parallel_chunks(count, [=](long long lo, long long hi) {
      for (long long i = lo; i < hi; ++i) dst[i] = leone_rd::table_entry(key, (uint64_t)(start + i));
    });
  }
  return 0;
}

}  // extern "C"
