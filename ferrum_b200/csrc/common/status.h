// Device-side error reporting without traps.
//
// Kernels that wait (on an mbarrier, a peer flag) give up after a deadline,
// write a record into a small host-mapped status block and return; the CUDA
// context stays usable.  The host reads the block after a synchronize and
// turns a non-zero code into an exception.
#pragma once
#include <cstdint>

namespace fb {

enum StatusCode : int32_t {
  kStatusOk = 0,
  kStatusGemmTimeout = 1,     // an mbarrier wait inside the tcgen05 GEMM gave up
  kStatusPeerTimeout = 2,     // a wait on another rank's flag gave up
  kStatusBoundsViolation = 3, // an index check (debug builds) rejected an access
  kStatusBadArgument = 4,
};

// Layout of the status block (int32 words).
enum StatusWord : int {
  kWordCode = 0,   // first non-zero StatusCode recorded
  kWordWhere = 1,  // kernel-specific site id
  kWordInfo0 = 2,  // e.g. peer rank / block index
  kWordInfo1 = 3,  // e.g. epoch / stage
  kStatusWords = 16,
};

#ifdef __CUDACC__
__device__ __forceinline__ void report_status(int32_t* status, int32_t code, int32_t where, int32_t info0,
                                              int32_t info1) {
  if (status == nullptr) return;
  if (atomicCAS(reinterpret_cast<int*>(status + kWordCode), 0, code) == 0) {
    status[kWordWhere] = where;
    status[kWordInfo0] = info0;
    status[kWordInfo1] = info1;
    __threadfence_system();
  }
}

// Index checks of the debug build (-DFERRUM_BOUNDS=1, `FERRUM_BOUNDS=1 python -m ferrum_b200._build`): an index
// outside [0, limit) records {site, index, limit} in the status block and the caller skips the access; nothing
// traps.  In the normal build the macro is the constant `true` and costs nothing.
__device__ __forceinline__ bool check_index(int32_t* status, int32_t site, long long idx, long long limit) {
  if (idx >= 0 && idx < limit) return true;
  report_status(status, kStatusBoundsViolation, site, static_cast<int32_t>(idx), static_cast<int32_t>(limit));
  return false;
}
#ifdef FERRUM_BOUNDS
#define FB_INDEX_OK(status, site, idx, limit) (::fb::check_index((status), (site), (idx), (limit)))
#else
#define FB_INDEX_OK(status, site, idx, limit) (true)
#endif
#endif

// Status block that kernels without a status argument report to in the debug build (set by fb_bounds_set_status).
inline int32_t*& bounds_status_ref() {
  static int32_t* p = nullptr;
  return p;
}

}  // namespace fb
