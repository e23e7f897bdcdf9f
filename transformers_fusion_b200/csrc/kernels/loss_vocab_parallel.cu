// Vocabulary-parallel cross entropy: every tensor-parallel rank holds the logits of its own slice of the vocabulary
// ([T, V_local], columns vocab_lo .. vocab_lo + V_local of the full row), so the softmax normaliser needs one small
// exchange between the ranks instead of an all-gather of the logits.
//
//   pass 1  ce_vp_stats : per row, over the local columns: max, sum of exp(z - max), and the label's logit when the
//                         label falls into this slice (0 otherwise)            -> stats[t] = {max, sum, z_label, 0}
//   (host)              : the ranks exchange their stats ([T, 4] floats each) and combine them into the row's
//                         log-sum-exp over the whole vocabulary
//   pass 2  ce_vp_grad  : g = scale * (exp(z - lse) - [column == label]) written over the logits (bf16), zero rows
//                         for ignored labels
// One CTA per row, 16-byte vectors, one read of the row per pass (the second one is served from L2 for rows a CTA
// has just produced when the chunk fits there).
//
// Reference counterparts: cross-entropy forward / backward (src/model/autograd_functions.cpp:363) under the
// vocabulary split of TensorParallelManager::parallelize_model (src/trainer/tensor_parallelism.cpp:334-451).
#include "tfb_host.h"
#include "tfb_ptx.cuh"

TFB_BOUNDS_DEFINE(loss_vocab_parallel)

namespace tfb {

__device__ __forceinline__ float vp_reduce_sum(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  v = (lane < nw) ? sh[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float vp_reduce_max(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  v = (lane < nw) ? sh[lane] : -INFINITY;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__global__ void __launch_bounds__(512) ce_vp_stats_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                                                          float4* __restrict__ stats, int V, long long ld, long long vocab_lo,
                                                          long long vocab_total, long long ignore_index) {
  tfb::pdl_sync();
  __shared__ float sh[32];
  const long long t = blockIdx.x;
  const __nv_bfloat16* row = logits + t * ld;
  const long long label = labels[t];
  if (threadIdx.x == 0) TFB_BOUNDS(label == ignore_index || (label >= 0 && label < vocab_total), 31, label, vocab_total);
  const long long loc = label - vocab_lo;
  const bool vec = ((ld & 7) == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  const int V8 = vec ? (V >> 3) : 0;
  float mx = -INFINITY, sum = 0.f;
  auto upd = [&](float z) {
    if (z > mx) {
      sum = sum * __expf(mx - z) + 1.f;
      mx = z;
    } else {
      sum += __expf(z - mx);
    }
  };
  for (int i = threadIdx.x; i < V8; i += blockDim.x) {
    const uint4 u = reinterpret_cast<const uint4*>(row)[i];
    const uint32_t* p = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_bf16(p[k]);
      upd(f.x);
      upd(f.y);
    }
  }
  for (int i = V8 * 8 + threadIdx.x; i < V; i += blockDim.x) upd(__bfloat162float(row[i]));
  const float gmx = vp_reduce_max(mx, sh);
  const float gsum = vp_reduce_sum(mx == -INFINITY ? 0.f : sum * __expf(mx - gmx), sh);
  if (threadIdx.x == 0) {
    const float zy = (label != ignore_index && loc >= 0 && loc < V) ? __bfloat162float(row[loc]) : 0.f;
    stats[t] = make_float4(gmx, gsum, zy, 0.f);
  }
}

__global__ void __launch_bounds__(512) ce_vp_grad_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                                                         const float* __restrict__ lse, const float* __restrict__ scale_ptr, int V,
                                                         long long ld, long long vocab_lo, long long ignore_index) {
  tfb::pdl_sync();
  const long long t = blockIdx.x;
  __nv_bfloat16* row = logits + t * ld;
  const long long label = labels[t];
  const bool ignored = label == ignore_index;
  const long long loc = ignored ? -1 : label - vocab_lo;
  const float scale = ignored ? 0.f : (scale_ptr ? *scale_ptr : 1.f);
  const float l = lse[t];
  const bool vec = ((ld & 7) == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  const int V8 = vec ? (V >> 3) : 0;
  for (int i = threadIdx.x; i < V8; i += blockDim.x) {
    uint4 u = reinterpret_cast<const uint4*>(row)[i];
    uint32_t* p = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_bf16(p[k]);
      const int c = i * 8 + k * 2;
      float g0 = scale * __expf(f.x - l), g1 = scale * __expf(f.y - l);
      if (c == loc) g0 -= scale;
      if (c + 1 == loc) g1 -= scale;
      p[k] = pack_bf16(g0, g1);
    }
    reinterpret_cast<uint4*>(row)[i] = u;
  }
  for (int i = V8 * 8 + threadIdx.x; i < V; i += blockDim.x) {
    float g = scale * __expf(__bfloat162float(row[i]) - l);
    if (i == loc) g -= scale;
    row[i] = __float2bfloat16(g);
  }
}

}  // namespace tfb

// stats[t] = {max, sum exp(z - max), label logit or 0, 0} over the V local columns of row t (row pitch ld elements).
TFB_API int tfb_ce_vp_stats(const void* logits, const long long* labels, float* stats, int T, int V, long long ld,
                            long long vocab_lo, long long vocab_total, long long ignore_index, void* stream) {
  if (T <= 0 || V <= 0 || (reinterpret_cast<uintptr_t>(stats) & 15)) return TFB_ERR_ARG;
  tfb::launch_k(tfb::ce_vp_stats_kernel, T, 512, 0, static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(logits), labels,
                                                                          reinterpret_cast<float4*>(stats), V, ld, vocab_lo,
                                                                          vocab_total, ignore_index);
  return int(cudaGetLastError());
}

// logits[t, c] <- scale * (exp(z - lse[t]) - [c + vocab_lo == label]) (zero rows for ignored labels); `scale` is a device scalar.
TFB_API int tfb_ce_vp_grad(void* logits, const long long* labels, const float* lse, const float* scale, int T, int V, long long ld,
                           long long vocab_lo, long long ignore_index, void* stream) {
  if (T <= 0 || V <= 0) return TFB_ERR_ARG;
  tfb::launch_k(tfb::ce_vp_grad_kernel, T, 512, 0, static_cast<cudaStream_t>(stream), static_cast<__nv_bfloat16*>(logits), labels, lse, scale, V,
                                                                         ld, vocab_lo, ignore_index);
  return int(cudaGetLastError());
}
