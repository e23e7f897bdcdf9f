// Attention backward for callers that are not allowed to allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for users of this
// library only.
//
// tfb_attn_bwd() needs a scratch array (one float per batch x query head x position: the row sums
// of dO * O) and leaves it to the caller to provide that memory.  Some callers cannot: code that
// runs between the begin and end of a stream capture (cudaMalloc is not capturable), a serving or
// training loop that was given a fixed memory budget at start-up and must never grow it, and code
// on a latency-critical path where cudaMalloc's implicit device-wide synchronisation would stall
// every other stream.  For them the scratch lives in a fixed array inside the library.
//
// Contract
//   * Arguments are those of tfb_attn_bwd() without `delta`; inputs and outputs are still the caller's.
//   * B * Hq * S must not exceed TFB_ATTN_BWD_NOALLOC_MAX_ROWS (4 Mi rows = 16 MiB of scratch, held by
//     every GPU that loads the library until the process exits).  Larger problems are refused with
//     TFB_ERR_LIMIT (-3) and nothing is launched.
//   * The first call on a device looks up the device address of the array and raises the kernels'
//     shared-memory limit on that device (no allocation, but both are set-up work that a stream
//     capture does not record): make that first call before any stream capture begins on that device.
//   * The address table covers device indices 0..63; on a device with a higher index the call is
//     refused with TFB_ERR_LIMIT (-3).
//   * All calls share the one array and nothing in it needs to start at zero (every row that is read
//     is written first by the same call).  Two calls that overlap on the GPU - different streams, or
//     two host threads - race on it; serialise them on one stream or use tfb_attn_bwd() with separate
//     scratch for concurrent use.
//   * Calls no cudaMalloc / cudaFree and no allocating library routine.
#pragma once

#define TFB_ATTN_BWD_NOALLOC_MAX_ROWS (4ll * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int tfb_attn_bwd_noalloc(const void* q, long long ldq, int q_col0, const void* k, long long ldk, int k_col0,
                         const void* v, long long ldv, int v_col0, const void* o, long long ldo, const void* dout,
                         long long lddo, const float* lse, void* dq, long long lddq, int dq_col0, void* dk,
                         long long lddk, int dk_col0, void* dv, long long lddv, int dv_col0, int B, int S, int Hq,
                         int Hkv, int D, float scale, int causal, int* status, void* stream);

#ifdef __cplusplus
}
#endif
