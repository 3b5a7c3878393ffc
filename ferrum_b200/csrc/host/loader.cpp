// Native batch assembler of the DataLoader: worker threads gather the rows a sampler picked from a dataset held
// as stacked host tensors into a ring of staging buffers (pinned host memory when the batches go to a GPU), a few
// batches ahead of the consumer.  The reference fetches one sample at a time on the calling thread
// (ferrum-data/src/dataloader.rs:144-165); here the calling thread only hands over index lists and picks up
// finished slots, so batch assembly overlaps the training step.
//
// Threading model: one mutex guards the job queue and the per-slot counters; a job is a contiguous range of a
// slot's index list, so one batch is split over all workers.  Indices are checked against the dataset length: a
// bad index marks the slot as failed instead of reading outside the source.
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <mutex>
#include <thread>
#if defined(__x86_64__)
#include <immintrin.h>
#endif
#include <vector>

#define FB_API extern "C" __attribute__((visibility("default")))

namespace {

// One row into the staging slot.  The slot is written once and next read by the copy engine, never by this core,
// so rows of a few hundred bytes and more go out with non-temporal stores: no read-for-ownership of the
// destination lines (a third of the gather's memory traffic) and nothing of the batch left in the cache.
inline void copy_row(uint8_t* dst, const uint8_t* src, size_t n) {
#if defined(__x86_64__)
  if (n >= 256 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    size_t i = 0;
    for (; i + 64 <= n; i += 64) {
      const __m128i a = _mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i));
      const __m128i b = _mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i + 16));
      const __m128i c = _mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i + 32));
      const __m128i d = _mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i + 48));
      _mm_stream_si128(reinterpret_cast<__m128i*>(dst + i), a);
      _mm_stream_si128(reinterpret_cast<__m128i*>(dst + i + 16), b);
      _mm_stream_si128(reinterpret_cast<__m128i*>(dst + i + 32), c);
      _mm_stream_si128(reinterpret_cast<__m128i*>(dst + i + 48), d);
    }
    if (i < n) std::memcpy(dst + i, src + i, n - i);
    return;
  }
#endif
  std::memcpy(dst, src, n);
}

struct Field {
  const uint8_t* src;
  long long row_bytes;
};

struct Job {
  int slot;
  long long lo, hi;
};

struct Loader {
  std::vector<Field> fields;
  long long rows = 0;
  int depth = 0;
  std::vector<std::vector<uint8_t*>> slot_ptr;  // [depth][field]
  std::vector<std::vector<long long>> idx;      // [depth]
  std::vector<int> pending;                     // jobs of the slot not finished yet
  std::vector<int> failed;                      // 1: an index of the slot was out of range
  std::deque<Job> jobs;
  std::mutex mu;
  std::condition_variable cv_job, cv_done;
  std::vector<std::thread> workers;
  bool stop = false;

  void run() {
    for (;;) {
      Job j;
      {
        std::unique_lock<std::mutex> lk(mu);
        cv_job.wait(lk, [&] { return stop || !jobs.empty(); });
        if (stop && jobs.empty()) return;
        j = jobs.front();
        jobs.pop_front();
      }
      bool bad = false;
      const long long* ix = idx[j.slot].data();
      for (const Field& f : fields) {
        uint8_t* dst = slot_ptr[j.slot][&f - fields.data()];
        for (long long r = j.lo; r < j.hi; ++r) {
          const long long s = ix[r];
          if (s < 0 || s >= rows) {
            bad = true;
            continue;
          }
          copy_row(dst + r * f.row_bytes, f.src + s * f.row_bytes, static_cast<size_t>(f.row_bytes));
        }
      }
#if defined(__x86_64__)
      _mm_sfence();  // the streamed rows are visible before the slot is reported complete
#endif
      {
        std::lock_guard<std::mutex> lk(mu);
        if (bad) failed[j.slot] = 1;
        if (--pending[j.slot] == 0) cv_done.notify_all();
      }
    }
  }
};

}  // namespace

// nfields source arrays of `rows` rows each (src[f] with row_bytes[f] bytes per row); `depth` staging slots whose
// per-field buffers are slot_ptrs[slot * nfields + f], each large enough for the biggest batch.  Returns a handle.
FB_API void* fb_loader_create(int nfields, const void* const* src, const long long* row_bytes, long long rows,
                              int depth, void* const* slot_ptrs, int threads) {
  if (nfields <= 0 || depth <= 0 || rows < 0 || threads <= 0 || threads > 256) return nullptr;
  Loader* L = new Loader;
  L->rows = rows;
  L->depth = depth;
  for (int f = 0; f < nfields; ++f) {
    if (src[f] == nullptr || row_bytes[f] <= 0) {
      delete L;
      return nullptr;
    }
    L->fields.push_back({static_cast<const uint8_t*>(src[f]), row_bytes[f]});
  }
  L->slot_ptr.resize(depth);
  for (int s = 0; s < depth; ++s)
    for (int f = 0; f < nfields; ++f) L->slot_ptr[s].push_back(static_cast<uint8_t*>(slot_ptrs[s * nfields + f]));
  L->idx.resize(depth);
  L->pending.assign(depth, 0);
  L->failed.assign(depth, 0);
  for (int t = 0; t < threads; ++t) L->workers.emplace_back([L] { L->run(); });
  return L;
}

// Starts filling `slot` with the rows idx[0 .. n).  -1: bad arguments, -3: the slot is still being filled.
FB_API int fb_loader_submit(void* handle, int slot, const long long* idx, long long n) {
  Loader* L = static_cast<Loader*>(handle);
  if (L == nullptr || slot < 0 || slot >= L->depth || n < 0 || (n > 0 && idx == nullptr)) return -1;
  std::lock_guard<std::mutex> lk(L->mu);
  if (L->pending[slot] != 0) return -3;
  L->idx[slot].assign(idx, idx + n);
  L->failed[slot] = 0;
  const long long parts = static_cast<long long>(L->workers.size());
  const long long per = (n + parts - 1) / (parts > 0 ? parts : 1);
  int count = 0;
  for (long long lo = 0; lo < n; lo += (per > 0 ? per : 1)) {
    L->jobs.push_back({slot, lo, lo + per < n ? lo + per : n});
    ++count;
  }
  L->pending[slot] = count;
  if (count > 0) L->cv_job.notify_all();
  return 0;
}

// Blocks until `slot` is complete.  0: ready, -2: an index was out of range (the slot's contents are incomplete).
FB_API int fb_loader_wait(void* handle, int slot) {
  Loader* L = static_cast<Loader*>(handle);
  if (L == nullptr || slot < 0 || slot >= L->depth) return -1;
  std::unique_lock<std::mutex> lk(L->mu);
  L->cv_done.wait(lk, [&] { return L->pending[slot] == 0; });
  return L->failed[slot] ? -2 : 0;
}

FB_API void fb_loader_destroy(void* handle) {
  Loader* L = static_cast<Loader*>(handle);
  if (L == nullptr) return;
  {
    std::lock_guard<std::mutex> lk(L->mu);
    L->stop = true;
    L->jobs.clear();
  }
  L->cv_job.notify_all();
  for (std::thread& t : L->workers) t.join();
  delete L;
}
