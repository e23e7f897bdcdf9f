// Tensor-parallel collectives fused with their GEMMs (Megatron-style TP with sequence parallelism).
//
//   all-gather -> GEMM  : tfb_gemm_bf16_tp mode 1 (gemm_bf16.cu).  The sequence-sharded activation lives in
//       a symmetric [M, K] buffer; each rank's shard is in place, a few CTAs of the GEMM grid pull the peers'
//       shards over NVLink in 128-row blocks while the other CTAs already multiply the local rows, and a
//       tile whose rows come from a peer starts as soon as that block's flag is up.  Every remote row crosses
//       NVLink exactly once and is then read from local memory by TMA.
//   GEMM -> reduce-scatter: tfb_gemm_bf16_tp mode 2.  The epilogue stores every partial tile straight into
//       the staging slot of the rank that owns those rows (peer stores, remote shards first so the transfer
//       overlaps the remaining tiles); tfb_tp_reduce then sums the W slots (+ residual) on the owner.
//
// Reference counterparts: TensorParallelManager::column_parallel_linear (local product then an all-reduce
// where an all-gather was meant, src/trainer/tensor_parallelism.cpp:53-98) and row_parallel_linear
// (:100-142), SequenceParallel scatter / gather (:158-186,514-547).
#include "tfb_comm.cuh"
#include "tfb_host.h"

namespace tfb {

// out[r, :] = sum_s stage[s, r, :] (+ residual[r, :]);  stage is [world, rows, N] bf16
__global__ void tp_reduce_kernel(const __nv_bfloat16* __restrict__ stage, const __nv_bfloat16* __restrict__ residual,
                                 __nv_bfloat16* __restrict__ out, long long rows, int N, int world) {
  tfb::pdl_sync();
  const long long n8 = rows * N / 8;
  const long long slot = rows * (long long)N;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (residual) {
      const uint4 u = reinterpret_cast<const uint4*>(residual)[i];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16(w[j]); acc[2 * j] = f.x; acc[2 * j + 1] = f.y; }
    }
    for (int s = 0; s < world; ++s) {
      const uint4 u = reinterpret_cast<const uint4*>(stage + s * slot)[i];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16(w[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

}  // namespace tfb

TFB_API int tfb_tp_reduce(const void* stage, const void* residual, void* out, long long rows, int N, int world,
                          void* stream) {
  if ((rows * N) % 8) return TFB_ERR_ARG;
  long long blocks = (rows * N / 8 + 255) / 256;
  const long long cap = (long long)tfb::sm_count() * 8;
  if (blocks > cap) blocks = cap;
  tfb::launch_k(tfb::tp_reduce_kernel, unsigned(blocks), 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(stage), static_cast<const __nv_bfloat16*>(residual),
      static_cast<__nv_bfloat16*>(out), rows, N, world);
  return int(cudaGetLastError());
}
