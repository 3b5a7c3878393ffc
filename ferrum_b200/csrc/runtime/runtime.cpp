// Host-side CUDA runtime layer: device queries, a size-bucketed device memory
// pool, RAII-free stream/event handles and the host-mapped status block that
// device code reports errors into.  C ABI (called through ctypes).
//
// Counterparts in the reference, which are host-memory simulations there:
//   ferrum-cuda/src/cuda_device.rs:19-336   DeviceProperties / CudaDevice / manager
//   ferrum-cuda/src/cuda_memory.rs:11-393   CudaBuffer / MemoryPool (21 pow-2 buckets)
//   ferrum-cuda/src/stream.rs:12-429        CudaStream / CudaEvent / StreamPool
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "../common/status.h"

#define FB_API extern "C" __attribute__((visibility("default")))

namespace {

struct DeviceState {
  int32_t* status_host = nullptr;  // pinned + mapped
  int32_t* status_dev = nullptr;
  std::atomic<long long> allocated{0};
  std::atomic<long long> pooled{0};
  std::mutex mu;
  // bucket index -> free blocks
  std::vector<void*> free_blocks[32];
  std::unordered_map<void*, int> live;  // ptr -> bucket
};

constexpr int kMaxDevices = 16;
DeviceState g_dev[kMaxDevices];
std::mutex g_mu;

constexpr size_t kMinBlock = 256;              // bytes, bucket 0
constexpr int kPooledBuckets = 21;             // 256 B ... 256 MiB

int bucket_for(size_t bytes, size_t* rounded) {
  size_t sz = kMinBlock;
  int b = 0;
  while (sz < bytes) {
    sz <<= 1;
    ++b;
  }
  *rounded = sz;
  return b;
}

int current_device() {
  int d = 0;
  cudaGetDevice(&d);
  return d;
}

}  // namespace

// ------------------------------------------------------------------ devices
FB_API int fb_rt_device_count() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}
FB_API int fb_rt_set_device(int d) { return static_cast<int>(cudaSetDevice(d)); }
FB_API int fb_rt_get_device() { return current_device(); }
FB_API int fb_rt_synchronize() { return static_cast<int>(cudaDeviceSynchronize()); }

struct fb_device_props {
  char name[256];
  unsigned long long total_memory;
  int multiprocessor_count;
  int major, minor;
  int max_threads_per_block;
  int max_block_dim[3];
  int max_grid_dim[3];
  int warp_size;
  unsigned long long shared_mem_per_block;
  unsigned long long shared_mem_per_block_optin;
  int unified_addressing;
  int l2_cache_bytes;
  int clock_khz;
  int memory_clock_khz;
  int memory_bus_width;
  int cluster_launch;
  int can_map_host;
};

FB_API int fb_rt_device_props(int dev, fb_device_props* out) {
  cudaDeviceProp p;
  cudaError_t e = cudaGetDeviceProperties(&p, dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  std::memset(out, 0, sizeof(*out));
  std::strncpy(out->name, p.name, sizeof(out->name) - 1);
  out->total_memory = p.totalGlobalMem;
  out->multiprocessor_count = p.multiProcessorCount;
  out->major = p.major;
  out->minor = p.minor;
  out->max_threads_per_block = p.maxThreadsPerBlock;
  for (int i = 0; i < 3; ++i) {
    out->max_block_dim[i] = p.maxThreadsDim[i];
    out->max_grid_dim[i] = p.maxGridSize[i];
  }
  out->warp_size = p.warpSize;
  out->shared_mem_per_block = p.sharedMemPerBlock;
  out->shared_mem_per_block_optin = p.sharedMemPerBlockOptin;
  out->unified_addressing = p.unifiedAddressing;
  out->l2_cache_bytes = p.l2CacheSize;
  int v = 0;
  cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, dev);
  out->clock_khz = v;
  cudaDeviceGetAttribute(&v, cudaDevAttrMemoryClockRate, dev);
  out->memory_clock_khz = v;
  cudaDeviceGetAttribute(&v, cudaDevAttrGlobalMemoryBusWidth, dev);
  out->memory_bus_width = v;
  cudaDeviceGetAttribute(&v, cudaDevAttrClusterLaunch, dev);
  out->cluster_launch = v;
  out->can_map_host = p.canMapHostMemory;
  return 0;
}

FB_API int fb_rt_mem_info(unsigned long long* free_b, unsigned long long* total_b) {
  size_t f = 0, t = 0;
  cudaError_t e = cudaMemGetInfo(&f, &t);
  *free_b = f;
  *total_b = t;
  return static_cast<int>(e);
}

FB_API int fb_rt_can_access_peer(int dev, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return ok;
}

// ------------------------------------------------------------- status block
FB_API int32_t* fb_rt_status_ptr() {
  const int d = current_device();
  DeviceState& s = g_dev[d];
  std::lock_guard<std::mutex> lk(s.mu);
  if (s.status_dev == nullptr) {
    void* h = nullptr;
    if (cudaHostAlloc(&h, fb::kStatusWords * sizeof(int32_t), cudaHostAllocMapped) != cudaSuccess) return nullptr;
    std::memset(h, 0, fb::kStatusWords * sizeof(int32_t));
    void* dptr = nullptr;
    if (cudaHostGetDevicePointer(&dptr, h, 0) != cudaSuccess) return nullptr;
    s.status_host = static_cast<int32_t*>(h);
    s.status_dev = static_cast<int32_t*>(dptr);
  }
  fb::bounds_status_ref() = s.status_dev;  // where kernels without a status argument report in the debug build
  return s.status_dev;
}
// Copies the status words out (after the caller synchronized) and clears them.
FB_API int fb_rt_status_read(int32_t* out4, int clear) {
  const int d = current_device();
  DeviceState& s = g_dev[d];
  if (s.status_host == nullptr) {
    out4[0] = out4[1] = out4[2] = out4[3] = 0;
    return 0;
  }
  volatile int32_t* h = s.status_host;
  for (int i = 0; i < 4; ++i) out4[i] = h[i];
  if (clear)
    for (int i = 0; i < fb::kStatusWords; ++i) h[i] = 0;
  return out4[0];
}

// -------------------------------------------------------------- memory pool
// Power-of-two buckets from 256 B to 256 MiB are cached on free; larger
// requests go straight to cudaMalloc / cudaFree.
FB_API void* fb_rt_pool_alloc(unsigned long long bytes) {
  if (bytes == 0) bytes = 1;
  const int d = current_device();
  DeviceState& s = g_dev[d];
  size_t rounded = 0;
  const int b = bucket_for(bytes, &rounded);
  void* p = nullptr;
  {
    std::lock_guard<std::mutex> lk(s.mu);
    if (b < kPooledBuckets && !s.free_blocks[b].empty()) {
      p = s.free_blocks[b].back();
      s.free_blocks[b].pop_back();
      s.pooled -= static_cast<long long>(rounded);
    }
  }
  if (p == nullptr) {
    const size_t want = (b < kPooledBuckets) ? rounded : static_cast<size_t>(bytes);
    if (cudaMalloc(&p, want) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    if (b >= kPooledBuckets) rounded = want;
  }
  {
    std::lock_guard<std::mutex> lk(s.mu);
    s.live[p] = b;
  }
  s.allocated += static_cast<long long>(b < kPooledBuckets ? (kMinBlock << b) : bytes);
  return p;
}

FB_API int fb_rt_pool_free(void* p, unsigned long long bytes_hint) {
  if (p == nullptr) return 0;
  const int d = current_device();
  DeviceState& s = g_dev[d];
  int b = -1;
  {
    std::lock_guard<std::mutex> lk(s.mu);
    auto it = s.live.find(p);
    if (it == s.live.end()) return -1;
    b = it->second;
    s.live.erase(it);
    if (b < kPooledBuckets) {
      s.free_blocks[b].push_back(p);
      s.pooled += static_cast<long long>(kMinBlock << b);
    }
  }
  s.allocated -= static_cast<long long>(b < kPooledBuckets ? (kMinBlock << b) : bytes_hint);
  if (b >= kPooledBuckets) return static_cast<int>(cudaFree(p));
  return 0;
}

// Returns every cached block to the driver.
FB_API int fb_rt_pool_clear() {
  const int d = current_device();
  DeviceState& s = g_dev[d];
  std::lock_guard<std::mutex> lk(s.mu);
  for (int b = 0; b < kPooledBuckets; ++b) {
    for (void* p : s.free_blocks[b]) cudaFree(p);
    s.free_blocks[b].clear();
  }
  s.pooled = 0;
  return 0;
}
FB_API long long fb_rt_pool_allocated() { return g_dev[current_device()].allocated.load(); }
FB_API long long fb_rt_pool_cached() { return g_dev[current_device()].pooled.load(); }
FB_API unsigned long long fb_rt_pool_round(unsigned long long bytes) {
  size_t r = 0;
  const int b = bucket_for(bytes ? bytes : 1, &r);
  return b < kPooledBuckets ? r : bytes;
}

FB_API int fb_rt_memcpy_h2d(void* dst, const void* src, unsigned long long n, cudaStream_t st) {
  return static_cast<int>(cudaMemcpyAsync(dst, src, n, cudaMemcpyHostToDevice, st));
}
FB_API int fb_rt_memcpy_d2h(void* dst, const void* src, unsigned long long n, cudaStream_t st) {
  return static_cast<int>(cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToHost, st));
}
FB_API int fb_rt_memcpy_d2d(void* dst, const void* src, unsigned long long n, cudaStream_t st) {
  return static_cast<int>(cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToDevice, st));
}
FB_API int fb_rt_memset(void* dst, int v, unsigned long long n, cudaStream_t st) {
  return static_cast<int>(cudaMemsetAsync(dst, v, n, st));
}

// ----------------------------------------------------------- streams/events
FB_API cudaStream_t fb_rt_stream_create(int high_priority) {
  cudaStream_t s = nullptr;
  int lo = 0, hi = 0;
  cudaDeviceGetStreamPriorityRange(&lo, &hi);
  if (cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, high_priority ? hi : lo) != cudaSuccess)
    return nullptr;
  return s;
}
FB_API int fb_rt_stream_destroy(cudaStream_t s) { return static_cast<int>(cudaStreamDestroy(s)); }
FB_API int fb_rt_stream_synchronize(cudaStream_t s) { return static_cast<int>(cudaStreamSynchronize(s)); }
// 1 = all work done, 0 = still running, <0 = error.
FB_API int fb_rt_stream_query(cudaStream_t s) {
  cudaError_t e = cudaStreamQuery(s);
  if (e == cudaSuccess) return 1;
  if (e == cudaErrorNotReady) return 0;
  return -static_cast<int>(e);
}
FB_API cudaEvent_t fb_rt_event_create(int timing) {
  cudaEvent_t e = nullptr;
  if (cudaEventCreateWithFlags(&e, timing ? cudaEventDefault : cudaEventDisableTiming) != cudaSuccess)
    return nullptr;
  return e;
}
FB_API int fb_rt_event_destroy(cudaEvent_t e) { return static_cast<int>(cudaEventDestroy(e)); }
FB_API int fb_rt_event_record(cudaEvent_t e, cudaStream_t s) { return static_cast<int>(cudaEventRecord(e, s)); }
FB_API int fb_rt_stream_wait_event(cudaStream_t s, cudaEvent_t e) {
  return static_cast<int>(cudaStreamWaitEvent(s, e, 0));
}
FB_API int fb_rt_event_synchronize(cudaEvent_t e) { return static_cast<int>(cudaEventSynchronize(e)); }
FB_API int fb_rt_event_query(cudaEvent_t e) {
  cudaError_t r = cudaEventQuery(e);
  if (r == cudaSuccess) return 1;
  if (r == cudaErrorNotReady) return 0;
  return -static_cast<int>(r);
}
FB_API float fb_rt_event_elapsed_ms(cudaEvent_t a, cudaEvent_t b) {
  float ms = -1.f;
  if (cudaEventElapsedTime(&ms, a, b) != cudaSuccess) return -1.f;
  return ms;
}
FB_API const char* fb_rt_error_string(int code) { return cudaGetErrorString(static_cast<cudaError_t>(code)); }
