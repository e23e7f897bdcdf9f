// Device-side signalling between ranks over symmetric peer memory.
//
// Each rank owns a flag array int[world] in symmetric memory; `flags[r]` is a device pointer to
// rank r's array.  Rank a tells rank b "I have reached epoch e" with a release store of e into
// flags[b][a]; rank b waits with acquire loads of its own array.  Epochs only grow, every rank
// executes the same sequence of communicating kernels, so "value >= e" is the wait condition and a
// fast rank can run ahead safely.  All waits are bounded (TFB_WAIT_NS): on expiry the status word
// gets ST_TIMEOUT_FLAG and the wait returns false.
#pragma once
#include "tfb_ptx.cuh"

namespace tfb {

struct CommCtx {
  int* const* flags;  // device array [world]: flags[r] -> rank r's int[world] flag array
  int* epoch;         // this rank's epoch counter (device memory, touched by one thread at a time)
  int rank, world;
  int* status;
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_volatile(const int* p) {
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// single-thread helpers -------------------------------------------------------------------------
__device__ __forceinline__ int comm_next_epoch(const CommCtx& c) {
  const int e = ld_volatile(c.epoch) + 1;
  *c.epoch = e;
  return e;
}
__device__ __forceinline__ void comm_signal_all(const CommCtx& c, int e) {
  __threadfence_system();
  for (int r = 0; r < c.world; ++r) st_release_sys(c.flags[r] + c.rank, e);
}
__device__ __forceinline__ bool comm_wait_all(const CommCtx& c, int e) {
  const int* mine = c.flags[c.rank];
  const uint64_t t0 = globaltimer_ns();
  for (int r = 0; r < c.world; ++r) {
    uint32_t it = 0;
    while (ld_acquire_sys(mine + r) < e) {
      if ((++it & 255u) == 0u && globaltimer_ns() - t0 > TFB_WAIT_NS) {
        report(c.status, ST_TIMEOUT_FLAG);
        return false;
      }
    }
  }
  return true;
}

// block-level, one thread per peer (blockDim.x >= world): the W release stores, and the W polls, run side by side
// instead of one after the other
__device__ __forceinline__ void comm_signal_all_par(const CommCtx& c, int e) {
  if (threadIdx.x < c.world) {
    __threadfence_system();
    st_release_sys(c.flags[threadIdx.x] + c.rank, e);
  }
}
__device__ __forceinline__ bool comm_wait_all_block_par(const CommCtx& c, int e, int* sh_ok) {
  if (threadIdx.x == 0) *sh_ok = 1;
  __syncthreads();
  if (threadIdx.x < c.world) {
    const int* mine = c.flags[c.rank] + threadIdx.x;
    const uint64_t t0 = globaltimer_ns();
    uint32_t it = 0;
    while (ld_acquire_sys(mine) < e) {
      if ((++it & 255u) == 0u && globaltimer_ns() - t0 > TFB_WAIT_NS) {
        report(c.status, ST_TIMEOUT_FLAG);
        *sh_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  return *sh_ok != 0;
}

// block-level: thread 0 waits, the result is broadcast to the block
__device__ __forceinline__ bool comm_wait_all_block(const CommCtx& c, int e, int* sh_ok) {
  if (threadIdx.x == 0) *sh_ok = comm_wait_all(c, e) ? 1 : 0;
  __syncthreads();
  return *sh_ok != 0;
}

}  // namespace tfb
