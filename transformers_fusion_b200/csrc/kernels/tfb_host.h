// Host-side helpers shared by the kernel translation units: error return convention,
// TMA tensor-map creation (driver entry point looked up at run time, so the library has no
// link-time dependency on libcuda) and a small descriptor cache.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#define TFB_API extern "C" __attribute__((visibility("default")))

// All exported entry points return 0 on success, a negative tfb error or a positive cudaError_t.
enum {
  TFB_OK = 0,
  TFB_ERR_ARG = -1,       // shape / alignment not supported by the kernel
  TFB_ERR_DRIVER = -2,    // driver entry point or tensor-map encode failed
  TFB_ERR_LIMIT = -3,     // size beyond a documented fixed limit
};

namespace tfb {

// 2-D bf16/fp8 tensor map: `inner` contiguous elements per row, `outer` rows, row pitch `ld_bytes`.
// Box = box_inner x box_outer elements, 128-byte swizzle, zero fill outside the tensor.
int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                 uint64_t ld_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle128 = 1);
// 3-D variant (inner, mid, outer) with byte strides for mid and outer.
int make_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t d0, uint64_t d1, uint64_t d2,
                 uint64_t s1_bytes, uint64_t s2_bytes, uint32_t b0, uint32_t b1, uint32_t b2, int swizzle128 = 1);

int sm_count();

// 1 when the environment has TFB_PDL=1 (read once): whether launches allow programmatic stream serialization.  Off by
// default: measured on B200 under CUDA-graph replay it shortens a batch-1 decode step of the 8B shape by 5 % (1.45 -> 1.38
// ms for 8 layers) but lengthens the 64-sequence training step of the 50M model by 3 % (31.1 -> 32.0 ms), where early-placed
// CTAs of the next kernel take shared memory and registers from the tail of the running one.
int pdl_enabled();

// Launch of a kernel of this library: same meaning as kernel<<<grid, block, smem, stream>>>(args...), plus the launch
// attribute that lets the kernel's CTAs be placed while the previous kernel of the stream drains (each kernel starts with
// pdl_sync(), or with its own set-up followed by pdl_sync(), so nothing is read early).  Errors surface through
// cudaGetLastError() as with the <<<>>> form.
template <class... KArgs, class... Args>
inline void launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  (void)cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// One-time set-up per device.  Kernel attributes (cudaFuncSetAttribute) belong to the device that is current when
// they are set, so a process that drives several GPUs has to repeat them on each: `first_use()` is true exactly once
// per device (devices beyond 63 report true on every call, which only repeats an idempotent set-up).
class DeviceOnce {
 public:
  bool first_use() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
    const unsigned long long bit = 1ull << dev;
    const unsigned long long old = __atomic_fetch_or(&done_, bit, __ATOMIC_ACQ_REL);
    return (old & bit) == 0;
  }
  void retry() {   // set-up failed: let the next call on this device try again
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) __atomic_fetch_and(&done_, ~(1ull << dev), __ATOMIC_ACQ_REL);
  }
 private:
  unsigned long long done_ = 0;
};

// Raises a kernel's dynamic shared-memory limit once per device.  Returns 0 or a cudaError_t.
template <class Kern>
inline int ensure_dyn_smem(DeviceOnce& once, Kern kern, int bytes) {
  if (!once.first_use()) return 0;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) { once.retry(); return int(e); }
  return 0;
}

}  // namespace tfb

// ---------------------------------------------------------------------------------------------------------------------
// Bounds-check build (-DTFB_BOUNDS_CHECK, `python -m transformers_fusion_b200.build --bounds-check`, loaded when the
// environment has TFB_BOUNDS_CHECK=1).  Index-driven accesses (token ids, labels, page slots, block tables, expert ids)
// are always kept inside their tables; this build additionally records the first offender of each translation unit:
// {count, site, index, limit}, read and cleared by tfb_bounds_report_<unit>().  A release build compiles the checks out.
// Reference counterpart: the QUANT_CHECK / bounds-checked debug build of the C++ kernels (include/quant/tensor.h).
#ifdef TFB_BOUNDS_CHECK
#define TFB_BOUNDS_DEFINE(unit)                                                                                    \
  static __device__ unsigned long long g_tfb_bounds[4];                                                            \
  TFB_API int tfb_bounds_report_##unit(unsigned long long* out4, int reset) {                                      \
    cudaError_t e = cudaMemcpyFromSymbol(out4, g_tfb_bounds, sizeof(unsigned long long) * 4);                      \
    if (e == cudaSuccess && reset) {                                                                               \
      const unsigned long long z[4] = {0, 0, 0, 0};                                                                \
      e = cudaMemcpyToSymbol(g_tfb_bounds, z, sizeof(z));                                                          \
    }                                                                                                              \
    return int(e);                                                                                                 \
  }
#define TFB_BOUNDS(ok, site, idx, lim)                                                                             \
  do {                                                                                                             \
    if (!(ok) && atomicAdd(&g_tfb_bounds[0], 1ull) == 0ull) {                                                      \
      g_tfb_bounds[1] = (unsigned long long)(site);                                                                \
      g_tfb_bounds[2] = (unsigned long long)(long long)(idx);                                                      \
      g_tfb_bounds[3] = (unsigned long long)(long long)(lim);                                                      \
    }                                                                                                              \
  } while (0)
#else
#define TFB_BOUNDS_DEFINE(unit)
#define TFB_BOUNDS(ok, site, idx, lim) do {} while (0)
#endif

