// Layout planner for the data-parallel gradient arena.
//
// The reference stores `bucket_size_mb = 25` and a `GradientBucket` type that nothing
// uses (ferrum-distributed/src/ddp.rs:54,126-198).  Here the plan is real: parameters
// are laid into one flat arena in REVERSE registration order (the order in which their
// gradients become ready during backward), cut into buckets of at most `cap_elems`
// elements (a larger tensor gets a bucket of its own), and every bucket is padded to a
// multiple of `align_elems` so that each rank's shard of a bucket starts on a 16-byte
// boundary and all shards have the same length.
#include <cstdint>

#define FB_API extern "C" __attribute__((visibility("default")))

namespace {
long long round_up(long long v, long long a) { return a <= 1 ? v : ((v + a - 1) / a) * a; }
}  // namespace

// sizes[n]: element counts in registration order.  Outputs (arrays of length n):
// offsets[i] = arena offset of parameter i, bucket_of[i] = its bucket,
// bucket_start / bucket_len for the first *n_buckets entries.  param_align pads every
// parameter slot (elements).  Returns the arena length in elements, or <0 on error.
// kinds (optional, length n): a bucket only holds parameters of ONE kind, so a change of kind between neighbours
// closes the bucket.  The engine uses two kinds: weights that are consumed through their bf16 copies and
// parameters that kernels read in fp32 (biases, normalisation scales); with sharded master weights only buckets
// of the second kind publish fp32 values to the peers.
FB_API long long fb_plan_buckets_kinds(int n, const long long* sizes, const int* kinds, long long cap_elems,
                                       long long align_elems, long long param_align, long long* offsets,
                                       int* bucket_of, long long* bucket_start, long long* bucket_len,
                                       int* n_buckets) {
  if (n < 0 || cap_elems <= 0) return -1;
  long long cursor = 0;
  int nb = 0;
  long long cur_start = 0, cur_fill = 0;
  bool open = false;
  int cur_kind = 0;
  for (int k = n - 1; k >= 0; --k) {
    const long long sz = round_up(sizes[k], param_align);
    const int kind = kinds != nullptr ? kinds[k] : 0;
    if (open && cur_fill > 0 && (cur_fill + sz > cap_elems || kind != cur_kind)) {
      bucket_start[nb] = cur_start;
      bucket_len[nb] = round_up(cur_fill, align_elems);
      cursor = cur_start + bucket_len[nb];
      ++nb;
      open = false;
    }
    if (!open) {
      cur_start = cursor;
      cur_fill = 0;
      open = true;
    }
    cur_kind = kind;
    offsets[k] = cur_start + cur_fill;
    bucket_of[k] = nb;
    cur_fill += sz;
  }
  if (open && cur_fill > 0) {
    bucket_start[nb] = cur_start;
    bucket_len[nb] = round_up(cur_fill, align_elems);
    cursor = cur_start + bucket_len[nb];
    ++nb;
  }
  *n_buckets = nb;
  return cursor;
}

FB_API long long fb_plan_buckets(int n, const long long* sizes, long long cap_elems, long long align_elems,
                                 long long param_align, long long* offsets, int* bucket_of,
                                 long long* bucket_start, long long* bucket_len, int* n_buckets) {
  return fb_plan_buckets_kinds(n, sizes, nullptr, cap_elems, align_elems, param_align, offsets, bucket_of,
                               bucket_start, bucket_len, n_buckets);
}

// Shard [lo, hi) of a bucket of `len` elements owned by `rank` of `world` (len is a multiple of 4*world
// when planned with align_elems = 4*world; otherwise the last shard is shorter).
FB_API void fb_plan_shard(long long len, int world, int rank, long long* lo, long long* hi) {
  long long per = (len + world - 1) / world;
  per = round_up(per, 4);
  long long a = per * rank, b = per * (rank + 1);
  if (a > len) a = len;
  if (b > len) b = len;
  *lo = a;
  *hi = b;
}
