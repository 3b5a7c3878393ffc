// Seeded index generation for the data pipeline: permutations, weighted sampling
// with replacement, the distributed (per-rank) index slice and batch boundaries.
//
// Behavioural reference: ferrum-data/src/sampler.rs:6-358.  The reference draws from
// an unseeded thread_rng (only RandomSampler::with_seed / DistributedSampler::set_epoch
// are reproducible); here every generator takes a 64-bit seed, and the distributed
// sampler shuffles the padded index list with a seed all ranks share, so that the rank
// slices stay disjoint and cover the dataset.
#include <algorithm>
#include <cstdint>
#include <numeric>
#include <vector>

#define FB_API extern "C" __attribute__((visibility("default")))

namespace {

// PCG-XSH-RR 64/32.
struct Pcg32 {
  uint64_t state;
  uint64_t inc;
  explicit Pcg32(uint64_t seed, uint64_t stream = 0xda3e39cb94b95bdbULL) {
    state = 0;
    inc = (stream << 1u) | 1u;
    next();
    state += seed;
    next();
  }
  uint32_t next() {
    const uint64_t old = state;
    state = old * 6364136223846793005ULL + inc;
    const uint32_t xorshifted = static_cast<uint32_t>(((old >> 18u) ^ old) >> 27u);
    const uint32_t rot = static_cast<uint32_t>(old >> 59u);
    return (xorshifted >> rot) | (xorshifted << ((32 - rot) & 31));
  }
  uint64_t next64() { return (static_cast<uint64_t>(next()) << 32) | next(); }
  // unbiased integer in [0, bound)
  uint64_t below(uint64_t bound) {
    if (bound <= 1) return 0;
    const uint64_t limit = UINT64_MAX - (UINT64_MAX % bound);
    uint64_t r;
    do {
      r = next64();
    } while (r >= limit);
    return r % bound;
  }
  double uniform() { return static_cast<double>(next64() >> 11) * (1.0 / 9007199254740992.0); }
};

void shuffle(long long* v, long long n, Pcg32& rng) {
  for (long long i = n - 1; i > 0; --i) {
    const long long j = static_cast<long long>(rng.below(static_cast<uint64_t>(i) + 1));
    std::swap(v[i], v[j]);
  }
}

}  // namespace

// out[0..n) = a seeded permutation of 0..n-1 (Fisher-Yates).
FB_API void fb_sampler_permutation(long long n, unsigned long long seed, long long* out) {
  for (long long i = 0; i < n; ++i) out[i] = i;
  Pcg32 rng(seed);
  shuffle(out, n, rng);
}

// Shuffles an existing index list in place.
FB_API void fb_sampler_shuffle(long long* idx, long long n, unsigned long long seed) {
  Pcg32 rng(seed);
  shuffle(idx, n, rng);
}

// Sampling with replacement proportional to `weights` (cumulative table + binary search).
FB_API int fb_sampler_weighted(const double* weights, long long nw, long long nsamples, unsigned long long seed,
                               long long* out) {
  if (nw <= 0) return -1;
  std::vector<double> cum(static_cast<size_t>(nw));
  double total = 0.0;
  for (long long i = 0; i < nw; ++i) {
    if (weights[i] < 0.0) return -2;
    total += weights[i];
  }
  if (!(total > 0.0)) return -3;
  double s = 0.0;
  for (long long i = 0; i < nw; ++i) {
    s += weights[i] / total;
    cum[static_cast<size_t>(i)] = s;
  }
  Pcg32 rng(seed);
  for (long long k = 0; k < nsamples; ++k) {
    const double r = rng.uniform();
    auto it = std::upper_bound(cum.begin(), cum.end(), r);
    long long idx = static_cast<long long>(it - cum.begin());
    if (idx >= nw) idx = nw - 1;
    out[k] = idx;
  }
  return 0;
}

// Per-rank indices: pad the list to a multiple of `replicas` by wrapping around,
// optionally shuffle with the shared seed, return the contiguous slice of `rank`.
// Returns the number of indices written (= ceil(len / replicas)) or <0 on error.
FB_API long long fb_sampler_distributed(long long len, int replicas, int rank, int do_shuffle,
                                        unsigned long long seed, long long* out, long long cap) {
  if (len <= 0 || replicas <= 0 || rank < 0 || rank >= replicas) return -1;
  const long long per = (len + replicas - 1) / replicas;
  if (cap < per) return -2;
  const long long padded = per * replicas;
  std::vector<long long> idx(static_cast<size_t>(padded));
  for (long long i = 0; i < padded; ++i) idx[static_cast<size_t>(i)] = i < len ? i : (i % len);
  if (do_shuffle) {
    Pcg32 rng(seed);
    shuffle(idx.data(), padded, rng);
  }
  std::copy(idx.begin() + rank * per, idx.begin() + (rank + 1) * per, out);
  return per;
}

// Number of batches for n indices.
FB_API long long fb_sampler_num_batches(long long n, long long batch, int drop_last) {
  if (batch <= 0) return 0;
  return drop_last ? n / batch : (n + batch - 1) / batch;
}

// Random subset of `src` (a seeded shuffle of the given indices).
FB_API void fb_sampler_subset(const long long* src, long long n, unsigned long long seed, long long* out) {
  for (long long i = 0; i < n; ++i) out[i] = src[i];
  Pcg32 rng(seed);
  shuffle(out, n, rng);
}

// Zipf(s) ids over [0, vocab) by inverse-CDF lookup: the synthetic token stream of the embedding benchmark.
FB_API int fb_sampler_zipf(long long vocab, double s, long long n, unsigned long long seed, long long* out) {
  if (vocab <= 0) return -1;
  std::vector<double> cum(static_cast<size_t>(vocab));
  double total = 0.0;
  for (long long k = 0; k < vocab; ++k) {
    total += 1.0 / __builtin_pow(static_cast<double>(k + 1), s);
    cum[static_cast<size_t>(k)] = total;
  }
  Pcg32 rng(seed);
  for (long long i = 0; i < n; ++i) {
    const double r = rng.uniform() * total;
    auto it = std::upper_bound(cum.begin(), cum.end(), r);
    long long idx = static_cast<long long>(it - cum.begin());
    out[i] = idx >= vocab ? vocab - 1 : idx;
  }
  return 0;
}
