// Self-test driver of the host library, meant to be compiled TOGETHER with the host sources under
// -fsanitize=address,undefined (memory errors, undefined behaviour) or -fsanitize=thread (data races between
// concurrent callers) and run on a machine without a GPU.  It exercises every exported entry point with ragged
// and boundary sizes, checks the results it can check cheaply, and exits 0 when nothing was reported.
//
// usage: selftest <scratch directory> [threads]
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

extern "C" {
long long fb_plan_buckets(int n, const long long* sizes, long long cap_elems, long long align_elems,
                          long long param_align, long long* offsets, int* bucket_of, long long* bucket_start,
                          long long* bucket_len, int* n_buckets);
void fb_plan_shard(long long len, int world, int rank, long long* lo, long long* hi);
void fb_ref_matmul(const float* a, const float* b, float* c, int M, int K, int N);
void fb_ref_linear(const float* x, const float* w, const float* b, float* y, int B, int in, int out);
void fb_ref_softmax_rows(const float* x, float* y, int rows, int cols, int log_mode);
void fb_ref_layernorm_rows(const float* x, const float* gamma, const float* beta, float* y, int rows, int cols,
                           float eps);
void fb_ref_adam_step(float* p, const float* g, float* m, float* v, long long n, float lr, float b1, float b2,
                      float eps, float wd, int t);
void fb_ref_sgd_step(float* p, const float* g, float* vel, long long n, float lr, float mu, float wd, int nesterov,
                     int first);
void fb_ref_train_xor(float* w1, float* b1, float* w2, float* b2, int H, float lr, int epochs, int loss_kind,
                      float* losses);
int fb_ser_save(const char* path, int n, const char* const* names, const int* ndims, const long long* dims_flat,
                const int* dtypes, const void* const* data, const unsigned long long* nbytes, char* err, int errlen);
void* fb_ser_open(const char* path, char* err, int errlen);
int fb_ser_count(void* h);
unsigned int fb_ser_version(void* h);
int fb_ser_meta(void* h, int i, char* name_buf, int name_cap, int* ndim, long long* dims, int dims_cap, int* dtype,
                unsigned long long* offset, unsigned long long* size);
int fb_ser_name_len(void* h, int i);
int fb_ser_read(void* h, int i, void* dst);
void fb_ser_close(void* h);
void fb_sampler_permutation(long long n, unsigned long long seed, long long* out);
void fb_sampler_shuffle(long long* idx, long long n, unsigned long long seed);
int fb_sampler_weighted(const double* weights, long long nw, long long nsamples, unsigned long long seed,
                        long long* out);
long long fb_sampler_distributed(long long len, int replicas, int rank, int do_shuffle, unsigned long long seed,
                                 long long* out, long long cap);
long long fb_sampler_num_batches(long long n, long long batch, int drop_last);
void fb_sampler_subset(const long long* src, long long n, unsigned long long seed, long long* out);
int fb_sampler_zipf(long long vocab, double s, long long n, unsigned long long seed, long long* out);
void* fb_loader_create(int nfields, const void* const* src, const long long* row_bytes, long long rows, int depth,
                       void* const* slot_ptrs, int threads);
int fb_loader_submit(void* handle, int slot, const long long* idx, long long n);
int fb_loader_wait(void* handle, int slot);
void fb_loader_destroy(void* handle);
}

namespace {

int g_failures = 0;
#define EXPECT(cond)                                                        \
  do {                                                                      \
    if (!(cond)) {                                                          \
      std::fprintf(stderr, "selftest: %s:%d: %s\n", __FILE__, __LINE__, #cond); \
      __atomic_add_fetch(&g_failures, 1, __ATOMIC_RELAXED);                 \
    }                                                                       \
  } while (0)

void test_planner() {
  const int counts[] = {0, 1, 2, 7, 27};
  const long long caps[] = {1, 5, 64, 6553600};
  for (int n : counts)
    for (long long cap : caps)
      for (int world : {1, 2, 3, 8}) {
        std::vector<long long> sizes(n), offs(n), bstart(n + 1), blen(n + 1);
        std::vector<int> bof(n);
        for (int i = 0; i < n; ++i) sizes[i] = 1 + (i * 37) % 101;
        int nb = -1;
        const long long total = fb_plan_buckets(n, sizes.data(), cap, 4LL * world, 4, offs.data(), bof.data(),
                                                bstart.data(), blen.data(), &nb);
        EXPECT(total >= 0 && nb >= 0 && nb <= n);
        long long covered = 0;
        for (int b = 0; b < nb; ++b) {
          EXPECT(blen[b] % (4LL * world) == 0);
          EXPECT(bstart[b] == covered);
          covered += blen[b];
          long long lo = -1, hi = -1, prev = 0;
          for (int r = 0; r < world; ++r) {
            fb_plan_shard(blen[b], world, r, &lo, &hi);
            EXPECT(lo == prev && hi >= lo && hi <= blen[b]);
            prev = hi;
          }
          EXPECT(prev == blen[b]);
        }
        EXPECT(covered == total);
        for (int i = 0; i < n; ++i) {
          EXPECT(bof[i] >= 0 && bof[i] < nb);
          EXPECT(offs[i] >= bstart[bof[i]] && offs[i] + sizes[i] <= bstart[bof[i]] + blen[bof[i]]);
          EXPECT(offs[i] % 4 == 0);
        }
      }
}

void test_cpu_ref() {
  for (int M : {1, 3, 17})
    for (int K : {1, 5, 33})
      for (int N : {1, 2, 31}) {
        std::vector<float> a(M * K, 0.5f), b(K * N, 2.f), c(M * N, -1.f), bias(N, 1.f), y(M * N), w(N * K, 2.f);
        fb_ref_matmul(a.data(), b.data(), c.data(), M, K, N);
        EXPECT(std::fabs(c[M * N - 1] - static_cast<float>(K)) < 1e-4f);
        fb_ref_linear(a.data(), w.data(), bias.data(), y.data(), M, K, N);
        EXPECT(std::fabs(y[0] - static_cast<float>(K) - 1.f) < 1e-4f);
        fb_ref_linear(a.data(), w.data(), nullptr, y.data(), M, K, N);
      }
  for (int rows : {1, 4})
    for (int cols : {1, 2, 127, 1000}) {
      std::vector<float> x(rows * cols), y(rows * cols), g(cols, 1.f), be(cols, 0.f);
      for (size_t i = 0; i < x.size(); ++i) x[i] = std::sin(0.37f * static_cast<float>(i)) * 30.f;
      fb_ref_softmax_rows(x.data(), y.data(), rows, cols, 0);
      double s = 0;
      for (int c2 = 0; c2 < cols; ++c2) s += y[c2];
      EXPECT(std::fabs(s - 1.0) < 1e-4);
      fb_ref_softmax_rows(x.data(), y.data(), rows, cols, 1);
      EXPECT(y[0] <= 1e-6f);
      fb_ref_layernorm_rows(x.data(), g.data(), be.data(), y.data(), rows, cols, 1e-5f);
      double mean = 0;
      for (int c2 = 0; c2 < cols; ++c2) mean += y[c2];
      EXPECT(std::fabs(mean / cols) < 1e-3);
    }
  for (long long n : {0LL, 1LL, 5LL, 1001LL}) {
    std::vector<float> p(n, 1.f), g(n, 0.1f), m(n, 0.f), v(n, 0.f);
    for (int t = 1; t <= 3; ++t) fb_ref_adam_step(p.data(), g.data(), m.data(), v.data(), n, 1e-3f, .9f, .999f, 1e-8f, 0.01f, t);
    fb_ref_sgd_step(p.data(), g.data(), m.data(), n, 0.1f, 0.9f, 1e-4f, 1, 1);
    fb_ref_sgd_step(p.data(), g.data(), m.data(), n, 0.1f, 0.9f, 1e-4f, 0, 0);
    if (n > 0) EXPECT(p[n - 1] < 1.f);
  }
  const int H = 8, epochs = 50;
  std::vector<float> w1(2 * H), b1(H, 0.f), w2(H), b2(1, 0.f), losses(epochs);
  for (int i = 0; i < 2 * H; ++i) w1[i] = 0.5f * std::sin(1.f + i);
  for (int i = 0; i < H; ++i) w2[i] = 0.5f * std::cos(2.f + i);
  for (int kind : {0, 1}) {
    fb_ref_train_xor(w1.data(), b1.data(), w2.data(), b2.data(), H, 0.5f, epochs, kind, losses.data());
    EXPECT(std::isfinite(losses[epochs - 1]));
  }
}

void test_samplers(unsigned long long salt) {
  for (long long n : {0LL, 1LL, 2LL, 31LL, 1000LL}) {
    std::vector<long long> out(n + 1, -7), seen(n, 0);
    fb_sampler_permutation(n, 11 + salt, out.data());
    for (long long i = 0; i < n; ++i) {
      EXPECT(out[i] >= 0 && out[i] < n);
      if (out[i] >= 0 && out[i] < n) ++seen[out[i]];
    }
    for (long long i = 0; i < n; ++i) EXPECT(seen[i] == 1);
    EXPECT(out[n] == -7);  // nothing written past the end
    fb_sampler_shuffle(out.data(), n, 5 + salt);
    std::vector<long long> sub(n + 1, -7);
    fb_sampler_subset(out.data(), n, 3 + salt, sub.data());
    EXPECT(sub[n] == -7);
  }
  {
    const double w[] = {0.0, 1.0, 3.0, 0.0};
    std::vector<long long> out(257, -7);
    EXPECT(fb_sampler_weighted(w, 4, 256, 9 + salt, out.data()) == 0);
    for (int i = 0; i < 256; ++i) EXPECT(out[i] == 1 || out[i] == 2);
    EXPECT(out[256] == -7);
    EXPECT(fb_sampler_weighted(w, 0, 4, 1, out.data()) != 0);
  }
  for (long long len : {1LL, 10LL, 1001LL})
    for (int replicas : {1, 3, 8}) {
      const long long per = (len + replicas - 1) / replicas;
      std::vector<long long> count(len, 0);
      for (int r = 0; r < replicas; ++r)
        for (int shuf : {0, 1}) {
          std::vector<long long> out(per + 1, -7);
          const long long got = fb_sampler_distributed(len, replicas, r, shuf, 42 + salt, out.data(), per);
          EXPECT(got == per);
          EXPECT(out[per] == -7);
          for (long long i = 0; i < got; ++i) {
            EXPECT(out[i] >= 0 && out[i] < len);
            if (shuf && out[i] >= 0 && out[i] < len) ++count[out[i]];
          }
          // a buffer that is too small is refused, not overrun
          if (per > 1) EXPECT(fb_sampler_distributed(len, replicas, r, shuf, 1, out.data(), per - 1) < 0);
        }
      for (long long i = 0; i < len; ++i) EXPECT(count[i] >= 1);  // every sample is seen by some rank
      EXPECT(fb_sampler_distributed(len, replicas, replicas, 0, 1, nullptr, 0) < 0);
    }
  EXPECT(fb_sampler_num_batches(10, 3, 0) == 4 && fb_sampler_num_batches(10, 3, 1) == 3);
  EXPECT(fb_sampler_num_batches(10, 0, 0) == 0);
  {
    std::vector<long long> out(513, -7);
    EXPECT(fb_sampler_zipf(50000, 1.1, 512, 7 + salt, out.data()) == 0);
    for (int i = 0; i < 512; ++i) EXPECT(out[i] >= 0 && out[i] < 50000);
    EXPECT(out[512] == -7);
    EXPECT(fb_sampler_zipf(0, 1.1, 4, 7, out.data()) != 0);
  }
}

void test_serializer(const std::string& dir, int id) {
  const std::string path = dir + "/selftest_" + std::to_string(id) + ".ferrum";
  char err[256] = {0};
  // one tensor of every dtype code, a scalar, an empty tensor and a long name
  const int kDtypeSize[8] = {4, 8, 2, 2, 4, 8, 1, 1};
  std::vector<std::string> names;
  std::vector<int> ndims, dtypes;
  std::vector<long long> dims;
  std::vector<std::vector<uint8_t>> blobs;
  for (int d = 0; d < 8; ++d) {
    names.push_back("t" + std::to_string(d) + std::string(static_cast<size_t>(d) * 40, 'n'));
    const long long shape[3] = {d % 3 + 1, 5, d == 7 ? 0 : 2};  // the last one has zero elements
    const int nd = d == 0 ? 0 : 3;                              // the first one is a scalar
    ndims.push_back(nd);
    long long numel = 1;
    for (int k = 0; k < nd; ++k) {
      dims.push_back(shape[k]);
      numel *= shape[k];
    }
    dtypes.push_back(d);
    blobs.emplace_back(static_cast<size_t>(numel) * kDtypeSize[d]);
    for (size_t i = 0; i < blobs.back().size(); ++i) blobs.back()[i] = static_cast<uint8_t>(i * 7 + d + id);
  }
  std::vector<const char*> name_ptrs;
  std::vector<const void*> data_ptrs;
  std::vector<unsigned long long> nbytes;
  for (size_t i = 0; i < names.size(); ++i) {
    name_ptrs.push_back(names[i].c_str());
    data_ptrs.push_back(blobs[i].data());
    nbytes.push_back(blobs[i].size());
  }
  EXPECT(fb_ser_save(path.c_str(), 8, name_ptrs.data(), ndims.data(), dims.data(), dtypes.data(), data_ptrs.data(),
                     nbytes.data(), err, sizeof err) == 0);
  void* h = fb_ser_open(path.c_str(), err, sizeof err);
  EXPECT(h != nullptr);
  if (h != nullptr) {
    EXPECT(fb_ser_count(h) == 8 && fb_ser_version(h) == 1);
    for (int i = 0; i < 8; ++i) {
      const int len = fb_ser_name_len(h, i);
      EXPECT(len > 0);
      std::vector<char> name(static_cast<size_t>(len) + 1);
      int nd = -1, dt = -1;
      long long dd[8];
      unsigned long long off = 0, size = 0;
      EXPECT(fb_ser_meta(h, i, name.data(), len + 1, &nd, dd, 8, &dt, &off, &size) == 0);
      EXPECT(dt >= 0 && dt < 8);
      if (dt >= 0 && dt < 8) {
        EXPECT(size == blobs[dt].size());
        std::vector<uint8_t> back(size + 1, 0xEE);
        EXPECT(fb_ser_read(h, i, back.data()) == 0);
        EXPECT(size == 0 || std::memcmp(back.data(), blobs[dt].data(), size) == 0);
        EXPECT(back[size] == 0xEE);
      }
      // buffers that are too small are refused
      char tiny[2];
      EXPECT(fb_ser_meta(h, i, tiny, 2, &nd, dd, 8, &dt, &off, &size) != 0);
    }
    EXPECT(fb_ser_meta(h, 8, nullptr, 0, nullptr, nullptr, 0, nullptr, nullptr, nullptr) != 0);
    EXPECT(fb_ser_read(h, -1, nullptr) != 0);
    fb_ser_close(h);
  }
  // refusals: bad dtype code, size that does not match the shape, missing file, truncated file, bad magic
  int bad_dtype = 9;
  EXPECT(fb_ser_save(path.c_str(), 1, name_ptrs.data(), ndims.data(), dims.data(), &bad_dtype, data_ptrs.data(),
                     nbytes.data(), err, sizeof err) != 0);
  unsigned long long wrong = 3;
  EXPECT(fb_ser_save(path.c_str(), 1, name_ptrs.data(), ndims.data(), dims.data(), dtypes.data(), data_ptrs.data(),
                     &wrong, err, sizeof err) != 0);
  EXPECT(fb_ser_open((dir + "/does_not_exist").c_str(), err, sizeof err) == nullptr);
  for (const char* content : {"FERRUM01", "NOTFERRM\0\0\0\0\0\0\0\0", "FERRUM01\xff\xff\xff\xff\xff\xff\xff\x7f"}) {
    FILE* f = std::fopen(path.c_str(), "wb");
    if (f != nullptr) {
      std::fwrite(content, 1, content[8] == '\0' && content[0] == 'N' ? 16 : std::strlen(content), f);
      std::fclose(f);
      EXPECT(fb_ser_open(path.c_str(), err, sizeof err) == nullptr);
    }
  }
  std::remove(path.c_str());
}

// Batch assembler: two fields, three slots, four workers; ragged batch sizes, a bad index, a busy slot, and a
// destroy while jobs are still queued.
void test_loader() {
  const long long rows = 257, wx = 37, wy = 1;
  std::vector<float> x(rows * wx);
  std::vector<long long> y(rows * wy);
  for (long long r = 0; r < rows; ++r) {
    for (long long c = 0; c < wx; ++c) x[r * wx + c] = static_cast<float>(r * 1000 + c);
    y[r] = r * 7;
  }
  const int depth = 3, cap = 64;
  std::vector<std::vector<float>> sx(depth, std::vector<float>(cap * wx));
  std::vector<std::vector<long long>> sy(depth, std::vector<long long>(cap));
  const void* src[2] = {x.data(), y.data()};
  const long long rb[2] = {wx * 4, wy * 8};
  std::vector<void*> slots;
  for (int s = 0; s < depth; ++s) {
    slots.push_back(sx[s].data());
    slots.push_back(sy[s].data());
  }
  void* h = fb_loader_create(2, src, rb, rows, depth, slots.data(), 4);
  EXPECT(h != nullptr);
  if (h == nullptr) return;
  std::vector<long long> perm(rows);
  fb_sampler_permutation(rows, 99, perm.data());
  const long long sizes[5] = {64, 1, 33, 64, 0};
  long long off = 0;
  for (int b = 0; b < 5; ++b) {
    const int slot = b % depth;
    EXPECT(fb_loader_submit(h, slot, perm.data() + off, sizes[b]) == 0);
    EXPECT(fb_loader_wait(h, slot) == 0);
    for (long long i = 0; i < sizes[b]; ++i) {
      const long long r = perm[off + i];
      EXPECT(sx[slot][i * wx] == static_cast<float>(r * 1000) && sx[slot][i * wx + wx - 1] == x[r * wx + wx - 1]);
      EXPECT(sy[slot][i] == r * 7);
    }
    off += sizes[b];
  }
  const long long bad[3] = {0, rows, 5};
  EXPECT(fb_loader_submit(h, 0, bad, 3) == 0);
  EXPECT(fb_loader_wait(h, 0) == -2);
  EXPECT(fb_loader_submit(h, depth, perm.data(), 1) == -1);
  // all slots in flight, then destroyed without waiting
  for (int s = 0; s < depth; ++s) fb_loader_submit(h, s, perm.data() + s * cap, cap);
  const int busy = fb_loader_submit(h, 0, perm.data(), 1);
  EXPECT(busy == 0 || busy == -3);
  fb_loader_destroy(h);
  EXPECT(fb_loader_create(0, src, rb, rows, depth, slots.data(), 4) == nullptr);
}

}  // namespace

int main(int argc, char** argv) {
  const std::string dir = argc > 1 ? argv[1] : ".";
  const int threads = argc > 2 ? std::atoi(argv[2]) : 1;
  if (threads <= 1) {
    test_planner();
    test_cpu_ref();
    test_samplers(0);
    test_serializer(dir, 0);
    test_loader();
  } else {
    // the library keeps no shared mutable state, so concurrent callers must not race
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t)
      pool.emplace_back([&, t] {
        test_planner();
        test_samplers(static_cast<unsigned long long>(t));
        test_serializer(dir, t + 1);
        test_loader();  // each caller owns its loader; its workers run beside everybody else's
        if (t == 0) test_cpu_ref();
      });
    for (auto& th : pool) th.join();
  }
  if (g_failures != 0) {
    std::fprintf(stderr, "selftest: %d check(s) failed\n", g_failures);
    return 1;
  }
  std::printf("selftest ok\n");
  return 0;
}
