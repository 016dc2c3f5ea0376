// The sampler's truncation stages on the device, in fp64.
//
// The reference builds a sampling distribution on the host in f64 (crates/leone/src/sampler.rs:
// 451-469): finite logits sorted descending (ties: lower id first), weights exp(l/T - l_max/T)
// normalised (:501-530); the stages that read raw logits (top-n-sigma, min-k) first (:532-553),
// then every other stage in the order given, each seeing the renormalised survivors of the one
// before and never emptying the set (:555-612); the token is then drawn by scanning the whole
// row in id order with u = uniform(seed, position, Select) (:803-857).  The same here:
//
//   sort      one row = P (a power of two >= vocab) pairs (fp64 key, id), bitonic network:
//             tiles of 2,048 pairs in shared memory, larger strides in global memory
//   stages    one block per row walks the stage list over the sorted row with block-wide
//             fp64 sums and scans; "typical" needs a second sort (by |surprise - entropy|),
//             so the stage list is cut there and the host entry launches the pieces in order
//   select    probabilities scattered back to id order, id-order scan against u
//
// Stage types: 0 top-k, 1 top-p, 2 min-p, 3 top-a, 4 tail-free, 5 typical, 6 epsilon, 7 eta,
// 8 min-k, 9 top-n-sigma.
#include <cmath>
#include <climits>
#include "common.cuh"

namespace leone {
namespace samp {

constexpr int kTile = 2048;          // pairs a block sorts in shared memory
constexpr int kThreads = 1024;
constexpr int kMaxStages = 16;

enum Stage { kTopK = 0, kTopP, kMinP, kTopA, kTailFree, kTypical, kEpsilon, kEta, kMinK, kTopNSigma };

struct Stages {
  int n;
  int type[kMaxStages];
  double value[kMaxStages];
};

// Per-row views into the scratch area.
struct Row {
  double* keys;     // [P] sorted raw logits (descending); -inf past the finite ones
  int* order;       // [P] their ids
  double* kept;     // [P] probabilities of the survivors, in the same order
  double* skeys;    // [P] second sort: -score
  int* sidx;        // [P] second sort: slot
  double* aux_f;    // [P]
  int* aux_i;       // [P]
  double* dense;    // [vocab] probabilities in id order
  int* n;           // survivors
};

__host__ __device__ inline size_t row_bytes(int P, int vocab) {
  return (size_t)P * (8 + 4 + 8 + 8 + 4 + 8 + 4) + (size_t)((vocab + 1) / 2 * 2) * 8 + 16;
}
__host__ __device__ inline Row row_of(uint8_t* scratch, int row, int P, int vocab) {
  uint8_t* b = scratch + (size_t)row * row_bytes(P, vocab);
  Row r;
  r.keys = (double*)b; b += (size_t)P * 8;
  r.kept = (double*)b; b += (size_t)P * 8;
  r.skeys = (double*)b; b += (size_t)P * 8;
  r.aux_f = (double*)b; b += (size_t)P * 8;
  r.dense = (double*)b; b += (size_t)((vocab + 1) / 2 * 2) * 8;
  r.order = (int*)b; b += (size_t)P * 4;
  r.sidx = (int*)b; b += (size_t)P * 4;
  r.aux_i = (int*)b; b += (size_t)P * 4;
  r.n = (int*)b;
  return r;
}

// The order of a sorted row: larger key first, equal keys by smaller id.
__device__ __forceinline__ bool precedes(double ka, int ia, double kb, int ib) {
  return ka > kb || (ka == kb && ia < ib);
}

// ---- sort ----------------------------------------------------------------------------------
// row_map (or null): row r of this call works on row row_map[r] of `logits`.
__global__ void sort_init_logits_kernel(const float* __restrict__ logits, const int* __restrict__ row_map,
                                        int vocab, int P, uint8_t* scratch) {
  const int row = blockIdx.y;
  const Row r = row_of(scratch, row, P, vocab);
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) *r.n = 0;
  if (i >= P) return;
  const int src = row_map != nullptr ? row_map[row] : row;
  const float v = i < vocab ? logits[(size_t)src * vocab + i] : NAN;
  const bool ok = i < vocab && isfinite(v);
  r.keys[i] = ok ? (double)v : -INFINITY;
  r.order[i] = ok ? i : vocab + i;            // the excluded ones sort last, in a fixed order
}

__global__ void count_finite_kernel(int vocab, int P, uint8_t* scratch) {
  // after the sort: the finite keys are a prefix
  const int row = blockIdx.y;
  const Row r = row_of(scratch, row, P, vocab);
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  const bool here = r.order[i] < vocab;
  const bool next = i + 1 < P && r.order[i + 1] < vocab;
  if (here && !next) *r.n = i + 1;
}

// All passes with stride below the tile for the levels k_first..k_last, in shared memory.
__global__ void __launch_bounds__(kThreads)
bitonic_tile_kernel(int which, int vocab, int P, int n_sort, uint8_t* scratch, int k_first, int k_last) {
  __shared__ double sk[kTile];
  __shared__ int si[kTile];
  const Row r = row_of(scratch, blockIdx.y, P, vocab);
  double* keys = which ? r.skeys : r.keys;
  int* idx = which ? r.sidx : r.order;
  const int tile = n_sort < kTile ? n_sort : kTile;
  const int base = blockIdx.x * tile;
  for (int t = threadIdx.x; t < tile; t += blockDim.x) {
    sk[t] = keys[base + t];
    si[t] = idx[base + t];
  }
  __syncthreads();
  for (int k = k_first; k <= k_last; k <<= 1) {
    int j = k >> 1;
    if (j > (tile >> 1)) j = tile >> 1;
    for (; j >= 1; j >>= 1) {
      for (int t = threadIdx.x; t < (tile >> 1); t += blockDim.x) {
        const int i = 2 * j * (t / j) + (t % j), l = i + j;
        const bool up = ((base + i) & k) == 0;
        const double ka = sk[i], kb = sk[l];
        const int ia = si[i], ib = si[l];
        const bool swap = up ? precedes(kb, ib, ka, ia) : precedes(ka, ia, kb, ib);
        if (swap) {
          sk[i] = kb; si[i] = ib;
          sk[l] = ka; si[l] = ia;
        }
      }
      __syncthreads();
    }
  }
  for (int t = threadIdx.x; t < tile; t += blockDim.x) {
    keys[base + t] = sk[t];
    idx[base + t] = si[t];
  }
}

// One pass with a stride of at least a tile.
__global__ void bitonic_global_kernel(int which, int vocab, int P, int n_sort, uint8_t* scratch, int k, int j) {
  const Row r = row_of(scratch, blockIdx.y, P, vocab);
  double* keys = which ? r.skeys : r.keys;
  int* idx = which ? r.sidx : r.order;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= (n_sort >> 1)) return;
  const int i = 2 * j * (t / j) + (t % j), l = i + j;
  const bool up = (i & k) == 0;
  const double ka = keys[i], kb = keys[l];
  const int ia = idx[i], ib = idx[l];
  const bool swap = up ? precedes(kb, ib, ka, ia) : precedes(ka, ia, kb, ib);
  if (swap) {
    keys[i] = kb; idx[i] = ib;
    keys[l] = ka; idx[l] = ia;
  }
}

// Sorts the first n_sort (a power of two) pairs of every row's first or second pair of arrays.
// tiles_only: stop when every tile of 2,048 is sorted in itself.
static int sort_rows(int which, int vocab, int P, int n_sort, int rows, uint8_t* scratch, cudaStream_t stream,
                     bool tiles_only = false) {
  const int tile = n_sort < kTile ? n_sort : kTile;
  bitonic_tile_kernel<<<dim3(n_sort / tile, rows), kThreads, 0, stream>>>(which, vocab, P, n_sort, scratch, 2, tile);
  for (int k = 2 * tile; k <= n_sort && !tiles_only; k <<= 1) {
    for (int j = k >> 1; j >= tile; j >>= 1)
      bitonic_global_kernel<<<dim3((n_sort / 2 + 255) / 256, rows), 256, 0, stream>>>(which, vocab, P, n_sort,
                                                                                       scratch, k, j);
    bitonic_tile_kernel<<<dim3(n_sort / tile, rows), kThreads, 0, stream>>>(which, vocab, P, n_sort, scratch, k, k);
  }
  return (int)cudaGetLastError();
}

// After the tiles are sorted in themselves, every tile alternately descending and ascending
// (the network's direction at level kTile): the `take` best pairs of every tile, which hold the
// row's `take` best, go to the front of the second pair of arrays (padded to n_out with pairs
// that sort last).
__global__ void gather_tile_heads_kernel(int vocab, int P, uint8_t* scratch, int take, int n_out) {
  const Row r = row_of(scratch, blockIdx.y, P, vocab);
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_out) return;
  const int tiles = P / kTile;
  const int t = i / take, e = i - t * take;
  if (t < tiles) {
    // tile t is sorted descending ("up") if bit kTile of its base is clear, else ascending
    const int base = t * kTile;
    const int at = (base & kTile) == 0 ? base + e : base + kTile - 1 - e;
    r.skeys[i] = r.keys[at];
    r.sidx[i] = r.order[at];
  } else {
    r.skeys[i] = -INFINITY;
    r.sidx[i] = vocab + P + i;
  }
}

__global__ void take_heads_kernel(int vocab, int P, uint8_t* scratch, int count) {
  const Row r = row_of(scratch, blockIdx.y, P, vocab);
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  // the sorted heads become the row; what follows them is marked as excluded
  r.keys[i] = i < count ? r.skeys[i] : -INFINITY;
  r.order[i] = i < count ? r.sidx[i] : vocab + i;
}

// ---- block-wide fp64 helpers (one block of kThreads per row) ----------------------------------
struct Shared {
  double f[32];
  int i[32];
  double total;
  int result;
};

__device__ __forceinline__ double block_sum(double v, Shared& sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) sh.f[warp] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < kThreads / 32; ++w) t += sh.f[w];
    sh.total = t;
  }
  __syncthreads();
  return sh.total;
}

// Exclusive prefix of v over the threads, in thread order; *total gets the sum.
__device__ __forceinline__ double block_scan(double v, Shared& sh, double* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  double incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const double up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  __syncthreads();
  if (lane == 31) sh.f[warp] = incl;
  __syncthreads();
  if (threadIdx.x == 0) {
    double run = 0.0;
    for (int w = 0; w < kThreads / 32; ++w) {
      const double s = sh.f[w];
      sh.f[w] = run;
      run += s;
    }
    sh.total = run;
  }
  __syncthreads();
  *total = sh.total;
  return sh.f[warp] + incl - v;
}

__device__ __forceinline__ int block_min(int v, Shared& sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if (lane == 0) sh.i[warp] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    int m = INT_MAX;
    for (int w = 0; w < kThreads / 32; ++w) m = min(m, sh.i[w]);
    sh.result = m;
  }
  __syncthreads();
  return sh.result;
}

__device__ __forceinline__ int block_sum_int(int v, Shared& sh) {
  return (int)(block_sum((double)v, sh) + 0.5);
}

// This thread's contiguous share of [0, n).
__device__ __forceinline__ void chunk_of(int n, int* lo, int* hi) {
  const int c = (n + kThreads - 1) / kThreads;
  *lo = min(n, (int)threadIdx.x * c);
  *hi = min(n, *lo + c);
}

__device__ double sum_of(const double* a, int n, Shared& sh) {
  double s = 0.0;
  for (int i = threadIdx.x; i < n; i += kThreads) s += a[i];
  return block_sum(s, sh);
}

__device__ double entropy_of(const double* kept, int n, Shared& sh) {
  double s = 0.0;
  for (int i = threadIdx.x; i < n; i += kThreads) {
    const double p = kept[i];
    if (p > 0.0) s += -p * log(p);
  }
  return block_sum(s, sh);
}

// How many leading entries are at least `floor` (kept is non-increasing, so they are a prefix).
__device__ int threshold_keep(const double* kept, int n, double floor, Shared& sh) {
  int first_below = n;
  for (int i = threadIdx.x; i < n; i += kThreads)
    if (!(kept[i] >= floor)) { first_below = i; break; }
  return block_min(first_below, sh);
}

// First index whose running sum of f(i) satisfies `reached`, scanning [0, count) in order.
template <typename F, typename R>
__device__ int first_where(int count, F f, R reached, Shared& sh) {
  int lo, hi;
  chunk_of(count, &lo, &hi);
  double local = 0.0;
  for (int i = lo; i < hi; ++i) local += f(i);
  double total;
  double run = block_scan(local, sh, &total);
  int found = INT_MAX;
  for (int i = lo; i < hi; ++i) {
    run += f(i);
    if (reached(run)) { found = i; break; }
  }
  return block_min(found, sh);
}

__device__ void renormalize(double* kept, int n, Shared& sh) {
  const double total = sum_of(kept, n, sh);
  for (int i = threadIdx.x; i < n; i += kThreads) kept[i] /= total;
  __syncthreads();
}

// ---- the stages -------------------------------------------------------------------------------
// begin != 0: raw-logit stages, weights, normalisation; then stages [s0, s1) (raw ones skipped).
__global__ void __launch_bounds__(kThreads)
stages_kernel(int vocab, int P, uint8_t* scratch, const double* __restrict__ temperature, Stages st,
              int begin, int s0, int s1) {
  __shared__ Shared sh;
  const Row r = row_of(scratch, blockIdx.x, P, vocab);
  int n = *r.n;
  __syncthreads();
  if (n <= 0) return;
  const double* keys = r.keys;
  double* kept = r.kept;
  if (begin) {
    for (int s = 0; s < st.n; ++s) {
      if (st.type[s] == kTopNSigma && n >= 2) {
        const double mean = sum_of(keys, n, sh) / (double)n;
        double v = 0.0;
        for (int i = threadIdx.x; i < n; i += kThreads) {
          const double d = keys[i] - mean;
          v += d * d;
        }
        const double dev = sqrt(block_sum(v, sh) / (double)n);
        if (isfinite(dev)) {
          const double cut = keys[0] - st.value[s] * dev;
          n = max(1, threshold_keep(keys, n, cut, sh));
        }
      } else if (st.type[s] == kMinK && n >= 2) {
        const double range = keys[0] - keys[n - 1] + 1e-8;
        if (isfinite(range) && range > 0.0) {
          // the rank with the largest (gap / range) / rank; of equal ones the lowest
          double best = -INFINITY;
          int cliff = INT_MAX;
          for (int rank = 1 + threadIdx.x; rank < n; rank += kThreads) {
            const double w = ((keys[rank - 1] - keys[rank]) / range) / (double)rank;
            if (w > best) { best = w; cliff = rank; }
          }
          // block-wide: largest value, then the lowest rank that has it
          double m = best;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) m = fmax(m, __shfl_xor_sync(0xffffffffu, m, o));
          __syncthreads();
          if ((threadIdx.x & 31) == 0) sh.f[threadIdx.x >> 5] = m;
          __syncthreads();
          m = sh.f[0];
          for (int w = 1; w < kThreads / 32; ++w) m = fmax(m, sh.f[w]);
          __syncthreads();
          cliff = block_min(best == m ? cliff : INT_MAX, sh);
          const double fb = floor(st.value[s] / range);
          const int fallback = (isfinite(fb) && fb >= 0.0) ? (int)fmin(fb, (double)n) : n;
          n = min(n, max(1, max(cliff, fallback)));
        }
      }
    }
    const double t = temperature[blockIdx.x];
    const double top = keys[0] / t;
    for (int i = threadIdx.x; i < n; i += kThreads) kept[i] = exp(keys[i] / t - top);
    __syncthreads();
    renormalize(kept, n, sh);
  }
  for (int s = s0; s < s1; ++s) {
    const int type = st.type[s];
    const double value = st.value[s];
    int keep = n;
    if (type == kTopK) {
      keep = (int)fmin(value, (double)n);
    } else if (type == kTopP) {
      const int at = first_where(n, [&](int i) { return kept[i]; }, [&](double c) { return c >= value; }, sh);
      keep = at == INT_MAX ? n : at + 1;
    } else if (type == kMinP) {
      keep = threshold_keep(kept, n, value * kept[0], sh);
    } else if (type == kTopA) {
      keep = threshold_keep(kept, n, value * kept[0] * kept[0], sh);
    } else if (type == kEpsilon) {
      keep = threshold_keep(kept, n, value, sh);
    } else if (type == kEta) {
      const double h = entropy_of(kept, n, sh);
      keep = threshold_keep(kept, n, fmin(value, sqrt(value) * exp(-h)), sh);
    } else if (type == kTailFree) {
      if (n >= 3) {
        auto second = [&](int i) { return fabs(kept[i] - 2.0 * kept[i + 1] + kept[i + 2]); };
        double local = 0.0;
        for (int i = threadIdx.x; i < n - 2; i += kThreads) local += second(i);
        const double total = block_sum(local, sh);
        if (total > 0.0 && isfinite(total)) {
          const int at = first_where(n - 2, [&](int i) { return second(i) / total; },
                                     [&](double c) { return !(c <= value); }, sh);
          keep = 1 + (at == INT_MAX ? n - 2 : at);
        }
      }
    } else {
      continue;                       // raw stages ran at the beginning; typical is the host's cut
    }
    n = max(1, min(n, keep));
    __syncthreads();
    renormalize(kept, n, sh);
  }
  if (threadIdx.x == 0) *r.n = n;
}

// Typical, first half: the keys of the second sort (ascending |surprise - entropy|, then slot).
__global__ void __launch_bounds__(kThreads)
typical_scores_kernel(int vocab, int P, uint8_t* scratch) {
  __shared__ Shared sh;
  const Row r = row_of(scratch, blockIdx.x, P, vocab);
  const int n = *r.n;
  const double h = entropy_of(r.kept, n, sh);
  for (int i = threadIdx.x; i < P; i += kThreads) {
    if (i < n) {
      const double score = fabs(-log(r.kept[i]) - h);
      r.skeys[i] = score == score ? -score : -INFINITY;
      r.sidx[i] = i;
    } else {
      r.skeys[i] = -INFINITY;
      r.sidx[i] = P + i;
    }
  }
}

// Typical, second half: slots in score order until their mass reaches `mass`; the survivors
// keep their descending order.
__global__ void __launch_bounds__(kThreads)
typical_select_kernel(int vocab, int P, uint8_t* scratch, double mass) {
  __shared__ Shared sh;
  const Row r = row_of(scratch, blockIdx.x, P, vocab);
  const int n = *r.n;
  __syncthreads();
  if (n <= 0) return;
  const int at = first_where(n, [&](int i) { return r.kept[r.sidx[i]]; }, [&](double c) { return c >= mass; }, sh);
  const int m = at == INT_MAX ? n : at + 1;
  for (int i = threadIdx.x; i < n; i += kThreads) r.aux_i[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < m; i += kThreads) r.aux_i[r.sidx[i]] = 1;
  __syncthreads();
  // compaction in slot order; the second sort's keys are no longer needed: their place holds
  // the survivors' ids meanwhile
  int* ids = reinterpret_cast<int*>(r.skeys);
  int lo, hi;
  chunk_of(n, &lo, &hi);
  int local = 0;
  for (int i = lo; i < hi; ++i) local += r.aux_i[i];
  double total;
  int pos = (int)(block_scan((double)local, sh, &total) + 0.5);
  for (int i = lo; i < hi; ++i)
    if (r.aux_i[i]) {
      r.aux_f[pos] = r.kept[i];
      ids[pos] = r.order[i];
      ++pos;
    }
  __syncthreads();
  for (int i = threadIdx.x; i < m; i += kThreads) {
    r.kept[i] = r.aux_f[i];
    r.order[i] = ids[i];
  }
  __syncthreads();
  renormalize(r.kept, m, sh);
  if (threadIdx.x == 0) *r.n = m;
}

// Mirostat v2's filter (crates/leone/src/sampler.rs:383-420): of the distribution the stages
// left (the target), the tokens whose surprise -ln p is at most the row's current maximum are
// kept and renormalised (the most probable one if none is); the target's probabilities stay in
// aux_f so that the draw can report the chosen token's.
__global__ void __launch_bounds__(kThreads)
surprise_filter_kernel(int vocab, int P, uint8_t* scratch, const double* __restrict__ maximum_surprise) {
  __shared__ Shared sh;
  const Row r = row_of(scratch, blockIdx.x, P, vocab);
  const int n = *r.n;
  __syncthreads();
  if (n <= 0) return;
  const double mu = maximum_surprise[blockIdx.x];
  int first_out = n;
  for (int i = threadIdx.x; i < n; i += kThreads) r.aux_f[i] = r.kept[i];
  for (int i = threadIdx.x; i < n; i += kThreads)
    if (!(-log(r.kept[i]) <= mu)) { first_out = i; break; }
  const int keep = max(1, block_min(first_out, sh));
  renormalize(r.kept, keep, sh);
  if (threadIdx.x == 0) *r.n = keep;
}

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long v) {
  unsigned long long z = v + 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

// Probabilities back in id order, and the draw: the first id whose running sum exceeds u, else
// the last id with any probability.
__global__ void __launch_bounds__(kThreads)
select_kernel(int vocab, int P, uint8_t* scratch, const long long* __restrict__ seeds,
              const long long* __restrict__ positions, int* __restrict__ out, const int* __restrict__ row_map,
              double* __restrict__ probs, double* __restrict__ chosen_prob) {
  __shared__ Shared sh;
  const int row = blockIdx.x;
  const int dst = row_map != nullptr ? row_map[row] : row;      // where the row's id goes
  const Row r = row_of(scratch, row, P, vocab);
  const int n = *r.n;
  for (int i = threadIdx.x; i < vocab; i += kThreads) r.dense[i] = 0.0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += kThreads) r.dense[r.order[i]] = r.kept[i];
  __syncthreads();
  if (probs != nullptr)
    for (int i = threadIdx.x; i < vocab; i += kThreads) probs[(size_t)row * vocab + i] = r.dense[i];
  if (n <= 0) {
    if (threadIdx.x == 0) out[dst] = -1;
    return;
  }
  const unsigned long long purpose = 0xbf58476d1ce4e5b9ull;
  const unsigned long long mixed =
      splitmix64((unsigned long long)seeds[row] ^ splitmix64((unsigned long long)positions[row] ^ purpose));
  const double u = (double)(mixed >> 11) * (1.0 / 9007199254740992.0);
  const double* dense = r.dense;
  const int at = first_where(vocab, [&](int i) { return dense[i]; }, [&](double c) { return u < c; }, sh);
  int last = -1;
  for (int i = threadIdx.x; i < vocab; i += kThreads)
    if (dense[i] > 0.0) last = i;
  last = -block_min(-last, sh);
  const int token = at == INT_MAX ? last : at;     // a zero entry cannot make the sum pass u
  if (threadIdx.x == 0) out[dst] = token;
  if (chosen_prob != nullptr)                      // the token's probability before the surprise filter
    for (int i = threadIdx.x; i < n; i += kThreads)
      if (r.order[i] == token) chosen_prob[row] = r.aux_f[i];
}

// Penalties from the decode history, before the sampler (crates/leone/src/penalty.rs:163-206).
// The host has walked the history (it owns it) and lists, per (row, token), how often the token
// occurs in the row's window and the largest repeated-suffix (DRY) penalty that reaches it; the
// arithmetic on the logits is done here, in fp64 as there: a seen token's logit is divided by
// the repetition factor if positive, multiplied if not, then loses the presence penalty once
// and the frequency penalty per occurrence, and is rounded to fp32; the DRY penalty is then
// subtracted from that.
__global__ void penalize_kernel(float* __restrict__ logits, int vocab, int n, const int* __restrict__ rows,
                                const int* __restrict__ tokens, const int* __restrict__ counts,
                                const double* __restrict__ dry, const double* __restrict__ repetition,
                                const double* __restrict__ presence, const double* __restrict__ frequency) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  const int row = rows[e], token = tokens[e];
  if (token < 0 || token >= vocab) return;
  float* at = logits + (size_t)row * vocab + token;
  float logit = *at;
  const double rep = repetition[row], pres = presence[row], freq = frequency[row];
  if (counts[e] > 0 && (rep != 1.0 || pres != 0.0 || freq != 0.0)) {
    double value = (double)logit;
    value = value > 0.0 ? value / rep : value * rep;
    value -= pres;
    value -= freq * (double)counts[e];
    logit = (float)value;
  }
  if (dry[e] > 0.0) logit = (float)((double)logit - dry[e]);
  *at = logit;
}

}  // namespace samp
}  // namespace leone

using namespace leone;
using namespace leone::samp;

static int pow2_at_least(int v) {
  int p = 2;
  while (p < v) p <<= 1;
  return p;
}

// Bytes of scratch for `rows` rows of `vocab` logits.
extern "C" long long leone_sample_truncated_scratch(int rows, int vocab) {
  return (long long)rows * (long long)row_bytes(pow2_at_least(vocab), vocab);
}

// logits: fp32 [rows, vocab]; temperature: fp64 [rows] (> 0); seeds, positions: int64 [rows];
// the stage list (types and values, in the order they apply) is the same for all rows; out: int32
// sampled ids; probs: fp64 [rows, vocab] or null, the distribution the draw was made from.
// row_map: int32 [rows] or null: row r of the call reads logits row row_map[r] and writes
// out[row_map[r]] (a subset of a step's rows is sampled in place, without gathering it first).
// maximum_surprise: fp64 [rows] or null: Mirostat v2's filter after the stages; chosen_prob (fp64
// [rows], with it) gets the drawn token's probability before that filter.
extern "C" int leone_sample_truncated(const float* logits, int rows, int vocab, const double* temperature,
                                      const long long* seeds, const long long* positions, int n_stages,
                                      const int* types, const double* values, void* scratch, int* out,
                                      double* probs, const double* maximum_surprise, double* chosen_prob,
                                      const int* row_map, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || n_stages < 0 || n_stages > kMaxStages) return kRefusedSize;
  Stages st;
  st.n = n_stages;
  for (int s = 0; s < n_stages; ++s) {
    if (types[s] < 0 || types[s] > kTopNSigma) return kRefusedSize;
    st.type[s] = types[s];
    st.value[s] = values[s];
  }
  const int P = pow2_at_least(vocab);
  uint8_t* sc = static_cast<uint8_t*>(scratch);
  sort_init_logits_kernel<<<dim3((P + 255) / 256, rows), 256, 0, stream>>>(logits, row_map, vocab, P, sc);
  // A pipeline that starts with a small top-k and has no raw-logit stage needs only the row's k
  // best pairs, which are among the k best of every tile: the tiles are sorted in themselves,
  // their heads gathered and sorted, and the rest of the row is never ordered.
  bool raw = false;
  for (int s = 0; s < n_stages; ++s) raw = raw || st.type[s] == kMinK || st.type[s] == kTopNSigma;
  const int tiles = P / kTile;
  int e;
  if (!raw && n_stages > 0 && st.type[0] == kTopK && P > kTile && st.value[0] * tiles <= 4 * kTile) {
    const int take = (int)st.value[0];
    const int n_out = pow2_at_least(take * tiles);
    e = sort_rows(0, vocab, P, P, rows, sc, stream, true);
    if (e != 0) return e;
    gather_tile_heads_kernel<<<dim3((n_out + 255) / 256, rows), 256, 0, stream>>>(vocab, P, sc, take, n_out);
    e = sort_rows(1, vocab, P, n_out, rows, sc, stream);
    if (e != 0) return e;
    take_heads_kernel<<<dim3((P + 255) / 256, rows), 256, 0, stream>>>(vocab, P, sc, take);
  } else {
    e = sort_rows(0, vocab, P, P, rows, sc, stream);
    if (e != 0) return e;
  }
  count_finite_kernel<<<dim3((P + 255) / 256, rows), 256, 0, stream>>>(vocab, P, sc);
  int done = 0;
  bool begun = false;
  while (true) {
    int cut = done;
    while (cut < n_stages && st.type[cut] != kTypical) ++cut;
    stages_kernel<<<rows, kThreads, 0, stream>>>(vocab, P, sc, temperature, st, begun ? 0 : 1, done, cut);
    begun = true;
    if (cut >= n_stages) break;
    typical_scores_kernel<<<rows, kThreads, 0, stream>>>(vocab, P, sc);
    e = sort_rows(1, vocab, P, P, rows, sc, stream);
    if (e != 0) return e;
    typical_select_kernel<<<rows, kThreads, 0, stream>>>(vocab, P, sc, st.value[cut]);
    done = cut + 1;
  }
  if (maximum_surprise != nullptr) {
    if (chosen_prob == nullptr) return kRefusedSize;
    surprise_filter_kernel<<<rows, kThreads, 0, stream>>>(vocab, P, sc, maximum_surprise);
  }
  select_kernel<<<rows, kThreads, 0, stream>>>(vocab, P, sc, seeds, positions, out, row_map, probs,
                                               maximum_surprise != nullptr ? chosen_prob : nullptr);
  return (int)cudaGetLastError();
}

// logits: fp32 [.., vocab], changed in place at the n listed (row, token) entries (each at most
// once); counts: occurrences in the row's window (0: only the DRY penalty applies); dry: the DRY
// penalty (0: none); repetition, presence, frequency: fp64 per row.
extern "C" int leone_penalize(float* logits, int vocab, int n, const int* rows, const int* tokens,
                              const int* counts, const double* dry, const double* repetition,
                              const double* presence, const double* frequency, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (vocab <= 0) return kRefusedSize;
  penalize_kernel<<<(n + 255) / 256, 256, 0, stream>>>(logits, vocab, n, rows, tokens, counts, dry, repetition,
                                                      presence, frequency);
  return (int)cudaGetLastError();
}
