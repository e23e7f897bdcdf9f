// Symmetric peer memory for one-process-per-GPU jobs on an NVSwitch node, and the device-side
// signalling primitives the fused compute+collective kernels share.
//
// Host side: each rank cudaMalloc's a buffer, exports a CUDA IPC handle, opens every peer's handle
// and ends up with a table of W device pointers to "the same" buffer on every GPU.  Kernels then
// read and write peers with plain ld/st/red over NVLink.
//
// Device side (tfb_comm.cuh): flag barriers with release/acquire at system scope.  Every wait is
// bounded; when it runs out the kernel records ST_TIMEOUT_FLAG in the status word and returns, so a
// missing peer shows up as an error code on the host, never as a hung GPU.
//
// Reference counterpart: DistributedContext's mutex/condvar collectives over a shared
// std::vector<float> (src/trainer/distributed.cpp:21-123).
#include "tfb_comm.cuh"
#include "tfb_host.h"

#include <string.h>

TFB_API int tfb_symm_alloc(long long bytes, void** ptr, void* handle64) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, size_t(bytes));
  if (e != cudaSuccess) return int(e);
  e = cudaMemset(p, 0, size_t(bytes));
  if (e != cudaSuccess) return int(e);
  e = cudaDeviceSynchronize();  // the zeros must be in place before any peer can see the handle
  if (e != cudaSuccess) return int(e);
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return int(e);
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  *ptr = p;
  return 0;
}

TFB_API int tfb_symm_open(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return int(e);
  *ptr = p;
  return 0;
}

TFB_API int tfb_symm_close(void* ptr) { return int(cudaIpcCloseMemHandle(ptr)); }
TFB_API int tfb_symm_free(void* ptr) { return int(cudaFree(ptr)); }

namespace tfb {

__global__ void barrier_kernel(CommCtx c) {
  tfb::pdl_sync();
  if (threadIdx.x == 0) {
    const int e = comm_next_epoch(c);
    comm_signal_all(c, e);
    comm_wait_all(c, e);
  }
}

}  // namespace tfb

// Device-side barrier across the ranks of the job: returns once every rank has reached it (or the
// bounded wait ran out and the status word says so).
TFB_API int tfb_comm_barrier(const void* flag_ptrs, int* epoch, int rank, int world, int* status, void* stream) {
  tfb::CommCtx c{static_cast<int* const*>(flag_ptrs), epoch, rank, world, status};
  tfb::launch_k(tfb::barrier_kernel, 1, 32, 0, static_cast<cudaStream_t>(stream), c);
  return int(cudaGetLastError());
}
