// Symmetric arena allocation for the inter-GPU kernels.
//
// One process per GPU allocates an arena with cudaMalloc, exports it as a CUDA IPC
// handle (64 bytes, exchanged by the Python layer over the rendezvous store) and maps
// every peer's arena with cudaIpcOpenMemHandle, which also enables peer access over
// NVLink.  The resulting table of base pointers is what fb_dist_ctx carries.  The
// reference has nothing to mirror here: its ProcessGroup never opens a socket or
// allocates anything (ferrum-distributed/src/process_group.rs:27-45, backend.rs:70-90).
//
// For tests on a single GPU the "peers" are further arenas in the same process
// (fb_symm_alloc called several times); no IPC is involved then.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>

#define FB_API extern "C" __attribute__((visibility("default")))

// Allocates `bytes` of device memory on the current device, zero-filled.  NULL on failure.
FB_API void* fb_symm_alloc(unsigned long long bytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  if (cudaMemset(p, 0, bytes) != cudaSuccess) {
    cudaFree(p);
    cudaGetLastError();
    return nullptr;
  }
  cudaDeviceSynchronize();
  return p;
}

FB_API int fb_symm_free(void* p) { return static_cast<int>(cudaFree(p)); }

FB_API int fb_symm_handle_bytes() { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }

// Writes the IPC handle of an arena obtained from fb_symm_alloc into handle_out (fb_symm_handle_bytes()).
FB_API int fb_symm_export(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return static_cast<int>(e);
  std::memcpy(handle_out, &h, sizeof(h));
  return 0;
}

// Maps a peer process's arena into this process.  NULL on failure (error code in *err).
FB_API void* fb_symm_import(const void* handle, int* err) {
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (err) *err = static_cast<int>(e);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}

FB_API int fb_symm_close(void* peer_ptr) { return static_cast<int>(cudaIpcCloseMemHandle(peer_ptr)); }

// Enables direct access from the current device to `peer_device` (same process, several GPUs).
FB_API int fb_symm_enable_peer(int peer_device) {
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return 0;
  }
  return static_cast<int>(e);
}
