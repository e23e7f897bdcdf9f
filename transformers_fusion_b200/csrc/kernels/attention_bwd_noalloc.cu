// See attention_bwd_noalloc.h for the contract.  The scratch is a file-scope device array; host code
// may not use its name as an address (on the host the symbol is only a stand-in), so the device
// address is fetched once per device with cudaGetSymbolAddress and handed to the kernels.
#include "attention_bwd_noalloc.h"

#include <mutex>

#include "tfb_host.h"

static __device__ __align__(256) float g_attn_bwd_delta[TFB_ATTN_BWD_NOALLOC_MAX_ROWS];

// the allocating-caller entry point (attention_bwd.cu); same kernels, scratch passed in
extern "C" int tfb_attn_bwd(const void* q, long long ldq, int q_col0, const void* k, long long ldk, int k_col0,
                            const void* v, long long ldv, int v_col0, const void* o, long long ldo, const void* dout,
                            long long lddo, const float* lse, float* delta, void* dq, long long lddq, int dq_col0,
                            void* dk, long long lddk, int dk_col0, void* dv, long long lddv, int dv_col0, int B,
                            int S, int Hq, int Hkv, int D, float scale, int causal, int* status, void* stream);

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {};
std::mutex g_setup_mutex;

// Device address of the scratch array on the current device (looked up on first use per device).
int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return int(e);
  if (dev < 0 || dev >= kMaxDevices) return TFB_ERR_LIMIT;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_addr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_attn_bwd_delta);
    if (e != cudaSuccess) return int(e);
    if (!p) return TFB_ERR_DRIVER;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}
}  // namespace

TFB_API int tfb_attn_bwd_noalloc(const void* q, long long ldq, int q_col0, const void* k, long long ldk, int k_col0,
                                 const void* v, long long ldv, int v_col0, const void* o, long long ldo,
                                 const void* dout, long long lddo, const float* lse, void* dq, long long lddq,
                                 int dq_col0, void* dk, long long lddk, int dk_col0, void* dv, long long lddv,
                                 int dv_col0, int B, int S, int Hq, int Hkv, int D, float scale, int causal,
                                 int* status, void* stream) {
  if (B <= 0 || S <= 0 || Hq <= 0) return TFB_ERR_ARG;
  const long long rows = (long long)B * Hq * S;
  if (rows > TFB_ATTN_BWD_NOALLOC_MAX_ROWS) return TFB_ERR_LIMIT;  // beyond the built-in scratch: refuse
  float* delta = nullptr;
  if (int rc = scratch_for_current_device(&delta)) return rc;
  return tfb_attn_bwd(q, ldq, q_col0, k, ldk, k_col0, v, ldv, v_col0, o, ldo, dout, lddo, lse, delta, dq, lddq,
                      dq_col0, dk, lddk, dk_col0, dv, lddv, dv_col0, B, S, Hq, Hkv, D, scale, causal, status, stream);
}
