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
#endif

}  // namespace fb
