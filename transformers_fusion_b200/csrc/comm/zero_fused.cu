// ZeRO gradient / parameter path as two fused compute+collective kernels over NVLink peer memory.
//
//   zero_reduce_scatter : waits until every rank's backward is complete (flag barrier), then for this
//       rank's contiguous shard of the flat fp32 gradient buffer sums the W copies with 128-bit peer
//       loads, applies 1/W, stores the result into the local shard and accumulates the squared norm of
//       the reduced shard.  The last CTA pushes the partial norm into every peer's slot table and
//       signals "done" (peers may now overwrite their gradient buffers).
//   zero_adamw_allgather: waits for every rank's "done", sums the W partial norms (the global gradient
//       norm, no separate all-reduce), derives the clip factor, applies bias-corrected AdamW with
//       decoupled weight decay to the fp32 master shard, and stores the refreshed bf16 parameters
//       straight into every rank's parameter buffer (the all-gather) with 128-bit peer stores.  It
//       also clears the local gradient buffer for the next step and signals "parameters delivered".
//   zero_wait           : one-thread kernel that waits for all peers' "parameters delivered".
//
// Reference counterparts: allreduce_bucket (src/trainer/ddp.cpp:113-173: pack -> all-reduce ->
// unpack -> /world), FSDP::reduce_scatter_grads implemented as zero-padded all-reduce + slice
// (src/trainer/fsdp.cpp:508-543), ZeroOptimizer::all_gather_params
// (src/trainer/zero_optimizer_core.cpp:252-298), global_grad_norm (src/trainer/ddp.cpp:280-312).
#include "tfb_comm.cuh"
#include "tfb_host.h"

namespace tfb {

constexpr int ZMAX_WORLD = 16;

struct ZeroArgs {
  CommCtx c;
  float* const* grad_ptrs;            // [world] fp32 flat gradient buffer of every rank
  __nv_bfloat16* const* param_ptrs;   // [world] bf16 flat parameter buffer of every rank
  float* const* norm_ptrs;            // [world] each rank's float[world] slot table for partial squared norms
  long long numel;                    // elements in the flat buffers (multiple of world * 8)
  long long shard;                    // numel / world
  float* master; float* m; float* v;  // this rank's shard state (shard elements)
  const float* hyper;                 // device {lr, 1-beta1^t, 1-beta2^t}
  float beta1, beta2, eps, wd, max_norm;
  float* accum;                       // local scratch: [0] squared-norm accumulator
  unsigned int* ticket;               // local scratch: CTA completion counter
  float* grad_norm_out;               // local: global gradient norm of this step (for logging)
};

__device__ __forceinline__ float4 ld_peer_f4(const float* p) {
  float4 v;
  asm volatile("ld.global.relaxed.sys.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

__global__ void __launch_bounds__(512) zero_reduce_scatter_kernel(ZeroArgs a) {
  tfb::pdl_sync();
  __shared__ int sh_ok;
  __shared__ float sh_red[32];
  const CommCtx& c = a.c;
  const int e0 = ld_volatile(c.epoch);
  if (blockIdx.x == 0 && threadIdx.x == 0) comm_signal_all(c, e0 + 1);  // my gradients are complete
  if (!comm_wait_all_block(c, e0 + 1, &sh_ok)) return;

  const int W = c.world;
  const float inv_w = 1.f / float(W);
  const long long lo = a.shard * c.rank;
  const long long n4 = a.shard >> 2;
  float ss = 0.f;
  const float* src[ZMAX_WORLD];
#pragma unroll
  for (int r = 0; r < ZMAX_WORLD; ++r) src[r] = r < W ? a.grad_ptrs[(c.rank + r) % W] + lo : nullptr;  // [0] is local
  float* dst = a.grad_ptrs[c.rank] + lo;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 acc = reinterpret_cast<const float4*>(src[0])[i];
    float4 v[ZMAX_WORLD];
#pragma unroll
    for (int r = 1; r < ZMAX_WORLD; ++r)
      if (r < W) v[r] = ld_peer_f4(src[r] + i * 4);  // all peer loads in flight before the first add
#pragma unroll
    for (int r = 1; r < ZMAX_WORLD; ++r)
      if (r < W) { acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w; }
    acc.x *= inv_w; acc.y *= inv_w; acc.z *= inv_w; acc.w *= inv_w;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    reinterpret_cast<float4*>(dst)[i] = acc;
  }
  // block reduce of the squared norm
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) sh_red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? sh_red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) {
      atomicAdd(a.accum, v);
      __threadfence();
      const unsigned int t = atomicAdd(a.ticket, 1u);
      if (t == gridDim.x - 1) {  // last CTA of this rank
        __threadfence();
        const float total = *reinterpret_cast<volatile float*>(a.accum);
        for (int r = 0; r < W; ++r) a.norm_ptrs[r][c.rank] = total;
        *a.accum = 0.f;
        *a.ticket = 0u;
        comm_signal_all(c, e0 + 2);  // shard reduced, partial norm delivered, peers' buffers no longer read
        *c.epoch = e0 + 2;
      }
    }
  }
}

__global__ void __launch_bounds__(512) zero_adamw_allgather_kernel(ZeroArgs a) {
  tfb::pdl_sync();
  __shared__ int sh_ok;
  const CommCtx& c = a.c;
  const int e0 = ld_volatile(c.epoch);
  if (!comm_wait_all_block(c, e0, &sh_ok)) return;  // every rank finished its reduce-scatter

  const int W = c.world;
  float total = 0.f;
  for (int r = 0; r < W; ++r) total += reinterpret_cast<volatile float*>(a.norm_ptrs[c.rank])[r];
  const float nrm = sqrtf(total);
  float clip = 1.f;
  const bool finite = isfinite(nrm);
  if (a.max_norm > 0.f && nrm > a.max_norm) clip = a.max_norm / (nrm + 1e-6f);
  if (blockIdx.x == 0 && threadIdx.x == 0 && a.grad_norm_out) *a.grad_norm_out = nrm;

  const float lr = a.hyper[0], bc1 = a.hyper[1], bc2 = a.hyper[2];
  const long long lo = a.shard * c.rank;
  const long long n8 = a.shard >> 3;
  float* g = a.grad_ptrs[c.rank] + lo;
  __nv_bfloat16* pdst[ZMAX_WORLD];
#pragma unroll
  for (int r = 0; r < ZMAX_WORLD; ++r) pdst[r] = r < W ? a.param_ptrs[(c.rank + r) % W] + lo : nullptr;
  if (finite) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8;
         i += (long long)gridDim.x * blockDim.x) {
      float p[8], gr[8], mm[8], vv[8];
      *reinterpret_cast<float4*>(p) = reinterpret_cast<const float4*>(a.master)[2 * i];
      *reinterpret_cast<float4*>(p + 4) = reinterpret_cast<const float4*>(a.master)[2 * i + 1];
      *reinterpret_cast<float4*>(gr) = reinterpret_cast<const float4*>(g)[2 * i];
      *reinterpret_cast<float4*>(gr + 4) = reinterpret_cast<const float4*>(g)[2 * i + 1];
      reinterpret_cast<float4*>(g)[2 * i] = make_float4(0.f, 0.f, 0.f, 0.f);  // consumed: ready for the next step
      reinterpret_cast<float4*>(g)[2 * i + 1] = make_float4(0.f, 0.f, 0.f, 0.f);
      *reinterpret_cast<float4*>(mm) = reinterpret_cast<const float4*>(a.m)[2 * i];
      *reinterpret_cast<float4*>(mm + 4) = reinterpret_cast<const float4*>(a.m)[2 * i + 1];
      *reinterpret_cast<float4*>(vv) = reinterpret_cast<const float4*>(a.v)[2 * i];
      *reinterpret_cast<float4*>(vv + 4) = reinterpret_cast<const float4*>(a.v)[2 * i + 1];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float x = gr[k] * clip;
        mm[k] = a.beta1 * mm[k] + (1.f - a.beta1) * x;
        vv[k] = a.beta2 * vv[k] + (1.f - a.beta2) * x * x;
        p[k] -= lr * ((mm[k] / bc1) / (sqrtf(vv[k] / bc2) + a.eps) + a.wd * p[k]);
      }
      reinterpret_cast<float4*>(a.master)[2 * i] = *reinterpret_cast<float4*>(p);
      reinterpret_cast<float4*>(a.master)[2 * i + 1] = *reinterpret_cast<float4*>(p + 4);
      reinterpret_cast<float4*>(a.m)[2 * i] = *reinterpret_cast<float4*>(mm);
      reinterpret_cast<float4*>(a.m)[2 * i + 1] = *reinterpret_cast<float4*>(mm + 4);
      reinterpret_cast<float4*>(a.v)[2 * i] = *reinterpret_cast<float4*>(vv);
      reinterpret_cast<float4*>(a.v)[2 * i + 1] = *reinterpret_cast<float4*>(vv + 4);
      uint4 o;
      o.x = pack_bf16(p[0], p[1]); o.y = pack_bf16(p[2], p[3]);
      o.z = pack_bf16(p[4], p[5]); o.w = pack_bf16(p[6], p[7]);
#pragma unroll
      for (int r = 0; r < ZMAX_WORLD; ++r)
        if (r < W) reinterpret_cast<uint4*>(pdst[r])[i] = o;  // the all-gather
    }
  }
  // clear the rest of the local gradient buffer for the next step (peers finished reading it: barrier
  // above); the owned shard was cleared element by element as it was consumed, unless the step was skipped
  {
    float4* gz = reinterpret_cast<float4*>(a.grad_ptrs[c.rank]);
    const long long t4 = a.numel >> 2, lo4 = lo >> 2, hi4 = (lo + a.shard) >> 2;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < t4; i += (long long)gridDim.x * blockDim.x)
      if (!finite || i < lo4 || i >= hi4) gz[i] = z;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int t = atomicAdd(a.ticket, 1u);
    if (t == gridDim.x - 1) {
      *a.ticket = 0u;
      comm_signal_all(c, e0 + 1);  // my shard of the parameters is in everyone's buffer
      *c.epoch = e0 + 1;
    }
  }
}

__global__ void zero_wait_kernel(CommCtx c) {
  tfb::pdl_sync();
  if (threadIdx.x == 0) comm_wait_all(c, ld_volatile(c.epoch));
}

}  // namespace tfb

using namespace tfb;

struct TfbZeroDesc {
  const void* flag_ptrs; int* epoch; int rank; int world; int* status;
  const void* grad_ptrs; const void* param_ptrs; const void* norm_ptrs;
  long long numel;
  float* master; float* m; float* v;
  const float* hyper;
  float beta1, beta2, eps, wd, max_norm;
  float* accum; unsigned int* ticket; float* grad_norm_out;
};

static int fill(const TfbZeroDesc* d, ZeroArgs& a) {
  if (d->world < 1 || d->world > ZMAX_WORLD || d->numel % (8LL * d->world)) return TFB_ERR_ARG;
  a.c = CommCtx{static_cast<int* const*>(d->flag_ptrs), d->epoch, d->rank, d->world, d->status};
  a.grad_ptrs = static_cast<float* const*>(d->grad_ptrs);
  a.param_ptrs = static_cast<__nv_bfloat16* const*>(d->param_ptrs);
  a.norm_ptrs = static_cast<float* const*>(d->norm_ptrs);
  a.numel = d->numel;
  a.shard = d->numel / d->world;
  a.master = d->master; a.m = d->m; a.v = d->v; a.hyper = d->hyper;
  a.beta1 = d->beta1; a.beta2 = d->beta2; a.eps = d->eps; a.wd = d->wd; a.max_norm = d->max_norm;
  a.accum = d->accum; a.ticket = d->ticket; a.grad_norm_out = d->grad_norm_out;
  return 0;
}

// Phase 1: reduce-scatter of the flat fp32 gradients (+ 1/W, + squared norm of the reduced shard).
TFB_API int tfb_zero_reduce_scatter(const TfbZeroDesc* d, int max_ctas, void* stream) {
  ZeroArgs a;
  if (int rc = fill(d, a)) return rc;
  int grid = sm_count() * 2;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  tfb::launch_k(zero_reduce_scatter_kernel, grid, 512, 0, static_cast<cudaStream_t>(stream), a);
  return int(cudaGetLastError());
}

// Phase 2: clip + AdamW on the shard, all-gather of the refreshed bf16 parameters, gradient clear.
TFB_API int tfb_zero_adamw_allgather(const TfbZeroDesc* d, int max_ctas, void* stream) {
  ZeroArgs a;
  if (int rc = fill(d, a)) return rc;
  int grid = sm_count() * 2;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  tfb::launch_k(zero_adamw_allgather_kernel, grid, 512, 0, static_cast<cudaStream_t>(stream), a);
  return int(cudaGetLastError());
}

// Phase 3: returns once every rank's parameters have arrived in the local buffer.
TFB_API int tfb_zero_wait(const TfbZeroDesc* d, void* stream) {
  CommCtx c{static_cast<int* const*>(d->flag_ptrs), d->epoch, d->rank, d->world, d->status};
  tfb::launch_k(zero_wait_kernel, 1, 32, 0, static_cast<cudaStream_t>(stream), c);
  return int(cudaGetLastError());
}
