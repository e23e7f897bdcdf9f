// ZeRO-3 / FSDP gradient path and sharded embedding lookup over NVLink peer memory.
//
// Every weight matrix of a unit (one transformer layer, the embedding table, the LM head) is sharded by rows over the
// W ranks of the data-parallel group: rank r owns rows [r * per, (r + 1) * per) of the padded matrix.  Backward leaves
// the unit's full fp32 gradient in each rank's own buffer (symmetric memory).
//
//   fsdp_reduce_scatter : one launch per unit, normally on a side stream with a limited grid so that it overlaps the
//       backward of the next unit.  Flag barrier ("this unit's backward is complete on every rank"), then for each
//       weight of the unit: 128-bit peer loads of the W copies of this rank's row shard, sum, 1/W, store into the
//       rank's flat fp32 shard-gradient buffer, and the squared norm of what was stored added to a device accumulator
//       (the global gradient norm needs no separate pass).  The last CTA signals "done reading".
//   fsdp_all_gather : one launch per unit on a side stream, one unit ahead of the compute (prefetch): every weight of
//       the unit is assembled in the local gather buffer from the W row shards with 128-bit peer loads.  No flags: the
//       shards only change in the optimizer step, which ends with a barrier over the group.
//   embedding_fwd_sharded : token-embedding lookup straight from the row shards of the table: the owner of a row is
//       id / per, so each token's row is fetched from whichever rank holds it (the all-gather of the table shrinks to
//       the rows the batch actually uses).  Ids outside [vocab_lo, vocab_lo + vocab_n) give zero rows (vocabulary-
//       parallel tables: another tensor-parallel rank supplies them).
//
// Reference counterparts: FullyShardedDataParallel::reduce_scatter_grads, implemented there as a zero-padded
// all-reduce followed by a slice (src/trainer/fsdp.cpp:508-543), backward hook order (:275-308), and the embedding
// forward (src/model/autograd_functions.cpp:489).
#include "tfb_comm.cuh"
#include "tfb_host.h"

TFB_BOUNDS_DEFINE(fsdp_fused)

namespace tfb {

constexpr int FS_MAX_WORLD = 16;
constexpr int FS_MAX_SEGS = 8;

struct FsdpSeg {
  long long full_off;    // elements: start of this weight's [rows_p, cols] gradient in the full gradient buffer
  long long shard_off;   // elements: start of this rank's shard of the weight in the flat shard buffers
  long long shard_len;   // elements per rank (rows_p / W * cols), a multiple of 4
};

struct FsdpRsArgs {
  CommCtx c;
  float* const* grad_ptrs;   // [world] full fp32 gradient buffer of every rank
  float* gshard;             // local flat fp32 shard-gradient buffer
  float* sumsq;              // local accumulator of the squared norm (cleared by the host at the start of a step)
  unsigned int* ticket;
  float scale;               // 1 / W (times any loss-scale inverse)
  int nseg;
  FsdpSeg seg[FS_MAX_SEGS];
};

__device__ __forceinline__ float4 fs_ld_peer(const float* p) {
  float4 v;
  asm volatile("ld.global.relaxed.sys.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

// MAXW: compile-time bound on the group size (the peer loops unroll over it); UNROLL: 16-byte vectors each thread
// keeps in flight per peer.  The kernel shares the GPU with the backward pass, so its CTAs must fit beside a resident GEMM
// CTA (320 threads x 168 registers = 53,760 of the SM's 65,536 registers, ~225 KB of shared memory): 128 threads x <= 80
// registers and a few bytes of static shared memory fit into what is left, where a larger CTA of this kernel could only
// start once a GEMM CTA had left and would then hold up the persistent GEMM that follows.  One such CTA per SM, so the
// per-thread queues must be deep enough to cover NVLink latency: 148 CTAs x 128 threads x UNROLL x (W - 1) x 16 B in flight.
constexpr int FS_THREADS = 128;
template <int MAXW, int UNROLL>
__global__ void __launch_bounds__(FS_THREADS, 6) fsdp_reduce_scatter_kernel(FsdpRsArgs a) {
  tfb::pdl_sync();
  __shared__ int sh_ok;
  __shared__ float sh_red[32];
  const CommCtx& c = a.c;
  const int e0 = ld_volatile(c.epoch);
  if (blockIdx.x == 0 && threadIdx.x == 0) comm_signal_all(c, e0 + 1);   // this unit's gradients are complete here
  if (!comm_wait_all_block(c, e0 + 1, &sh_ok)) return;
  const int W = c.world;
  float ss = 0.f;
  for (int s = 0; s < a.nseg; ++s) {
    const FsdpSeg sg = a.seg[s];
    const float* src[MAXW];
#pragma unroll
    for (int r = 0; r < MAXW; ++r)
      src[r] = r < W ? a.grad_ptrs[(c.rank + r) % W] + sg.full_off + sg.shard_len * c.rank : nullptr;   // [0] is local
    float* dst = a.gshard + sg.shard_off;
    const long long n4 = sg.shard_len >> 2;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < n4; i0 += stride * UNROLL) {
      float4 acc[UNROLL];
      float4 v[UNROLL][MAXW];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i < n4) {
          acc[u] = reinterpret_cast<const float4*>(src[0])[i];
#pragma unroll
          for (int r = 1; r < MAXW; ++r)
            if (r < W) v[u][r] = fs_ld_peer(src[r] + i * 4);   // all peer loads in flight before the first add
        }
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i < n4) {
          float4 t = acc[u];
#pragma unroll
          for (int r = 1; r < MAXW; ++r)
            if (r < W) { t.x += v[u][r].x; t.y += v[u][r].y; t.z += v[u][r].z; t.w += v[u][r].w; }
          t.x *= a.scale; t.y *= a.scale; t.z *= a.scale; t.w *= a.scale;
          ss += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
          reinterpret_cast<float4*>(dst)[i] = t;
        }
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) sh_red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? sh_red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) {
      atomicAdd(a.sumsq, v);
      __threadfence();
      const unsigned int t = atomicAdd(a.ticket, 1u);
      if (t == gridDim.x - 1) {   // last CTA of this rank: the peers' buffers are no longer read
        *a.ticket = 0u;
        comm_signal_all(c, e0 + 2);
        *c.epoch = e0 + 2;
      }
    }
  }
}

struct FsdpAgSeg {
  const uint4* const* src;   // device array [world]: every rank's shard of this weight
  uint4* dst;                // local gathered matrix: shard r goes to dst + r * shard_vecs
  long long shard_vecs;      // 16-byte vectors per shard
};
struct FsdpAgArgs {
  int rank, world, nseg;
  FsdpAgSeg seg[FS_MAX_SEGS];
};

// Like the reduce-scatter above, sized to sit beside a resident GEMM CTA: 128 threads, <= 80 registers, no shared memory.
// Every thread has one 16-byte load in flight to each rank at a time (UNROLL of them per rank): all W - 1 peers are read
// at once, which spreads the traffic over every NVLink port instead of draining one peer after the other.
template <int MAXW, int UNROLL>
__global__ void __launch_bounds__(FS_THREADS, 6) fsdp_all_gather_kernel(FsdpAgArgs a) {
  tfb::pdl_sync();
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long t0 = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const int W = a.world;
  for (int s = 0; s < a.nseg; ++s) {
    const FsdpAgSeg sg = a.seg[s];
    const uint4* src[MAXW];
#pragma unroll
    for (int rr = 0; rr < MAXW; ++rr) src[rr] = rr < W ? sg.src[(a.rank + rr) % W] : nullptr;   // [0] is the local shard
    for (long long i0 = t0; i0 < sg.shard_vecs; i0 += stride * UNROLL) {
      uint4 v[UNROLL][MAXW];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i < sg.shard_vecs) {
#pragma unroll
          for (int rr = 0; rr < MAXW; ++rr)
            if (rr < W)
              asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(v[u][rr].x), "=r"(v[u][rr].y), "=r"(v[u][rr].z), "=r"(v[u][rr].w) : "l"(src[rr] + i) : "memory");
        }
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i < sg.shard_vecs) {
#pragma unroll
          for (int rr = 0; rr < MAXW; ++rr)
            if (rr < W) sg.dst[(long long)((a.rank + rr) % W) * sg.shard_vecs + i] = v[u][rr];
        }
      }
    }
  }
}

__global__ void embedding_fwd_sharded_kernel(const long long* __restrict__ ids, const __nv_bfloat16* const* __restrict__ shard_ptrs,
                                             __nv_bfloat16* __restrict__ out, int T, int H, long long per_rows, int world,
                                             long long vocab_lo, long long vocab_n) {
  tfb::pdl_sync();
  const int vec = H >> 3;
  const long long total = (long long)T * vec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = int(i / vec), col = int(i % vec) * 8;
    const long long id = ids[t] - vocab_lo;
    uint4 u = make_uint4(0u, 0u, 0u, 0u);
    if (id >= 0 && id < vocab_n) {
      const int owner = int(id / per_rows);
      TFB_BOUNDS(owner < world, 21, id, per_rows * world);
      if (owner < world) {
        const __nv_bfloat16* src = shard_ptrs[owner] + (id - (long long)owner * per_rows) * H + col;
        asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(src) : "memory");
      }
    }
    *reinterpret_cast<uint4*>(out + (long long)t * H + col) = u;
  }
}

}  // namespace tfb

using namespace tfb;

struct TfbFsdpSeg { long long full_off, shard_off, shard_len; };

struct TfbFsdpRsDesc {
  const void* flag_ptrs; int* epoch; int rank; int world; int* status;
  const void* grad_ptrs;      // device array [world] of full fp32 gradient buffers
  float* gshard; float* sumsq; unsigned int* ticket;
  float scale;
  int nseg;
  TfbFsdpSeg seg[FS_MAX_SEGS];
};

// Reduce-scatter of one unit's gradients into this rank's flat shard-gradient buffer (see the top of the file).
// `max_ctas` bounds the grid so that the kernel can share the GPU with the backward pass of the next unit.
TFB_API int tfb_fsdp_reduce_scatter(const TfbFsdpRsDesc* d, int max_ctas, void* stream) {
  if (!d || d->world < 1 || d->world > FS_MAX_WORLD || d->nseg < 1 || d->nseg > FS_MAX_SEGS) return TFB_ERR_ARG;
  FsdpRsArgs a;
  a.c = CommCtx{static_cast<int* const*>(d->flag_ptrs), d->epoch, d->rank, d->world, d->status};
  a.grad_ptrs = static_cast<float* const*>(d->grad_ptrs);
  a.gshard = d->gshard; a.sumsq = d->sumsq; a.ticket = d->ticket; a.scale = d->scale; a.nseg = d->nseg;
  for (int s = 0; s < d->nseg; ++s) {
    if (d->seg[s].shard_len % 4 || d->seg[s].full_off % 4 || d->seg[s].shard_off % 4) return TFB_ERR_ARG;
    a.seg[s] = FsdpSeg{d->seg[s].full_off, d->seg[s].shard_off, d->seg[s].shard_len};
  }
  int grid = sm_count() * 4;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (d->world <= 2) tfb::launch_k(fsdp_reduce_scatter_kernel<2, 5>, grid, FS_THREADS, 0, st, a);
  else if (d->world <= 4) tfb::launch_k(fsdp_reduce_scatter_kernel<4, 2>, grid, FS_THREADS, 0, st, a);
  else if (d->world <= 8) tfb::launch_k(fsdp_reduce_scatter_kernel<8, 1>, grid, FS_THREADS, 0, st, a);
  else tfb::launch_k(fsdp_reduce_scatter_kernel<FS_MAX_WORLD, 1>, grid, FS_THREADS, 0, st, a);
  return int(cudaGetLastError());
}

struct TfbFsdpAgSeg { const void* src_ptrs; void* dst; long long shard_bytes; };
struct TfbFsdpAgDesc {
  int rank, world, nseg, pad;
  TfbFsdpAgSeg seg[FS_MAX_SEGS];
};

// All-gather of one unit's weights from the row shards of the W ranks into this rank's gather buffer (see the top of the
// file).  Every segment: src_ptrs = device array [world] of shard addresses, dst = local [world * shard_bytes] matrix,
// shard_bytes a multiple of 16.  `max_ctas` bounds the grid (0: four CTAs per SM; beside a resident GEMM CTA one fits
// per SM and the others follow as slots free up).
TFB_API int tfb_fsdp_all_gather(const TfbFsdpAgDesc* d, int max_ctas, void* stream) {
  if (!d || d->world < 1 || d->world > FS_MAX_WORLD || d->nseg < 1 || d->nseg > FS_MAX_SEGS || d->rank < 0 || d->rank >= d->world)
    return TFB_ERR_ARG;
  FsdpAgArgs a;
  a.rank = d->rank; a.world = d->world; a.nseg = d->nseg;
  for (int s = 0; s < d->nseg; ++s) {
    const TfbFsdpAgSeg& g = d->seg[s];
    if (!g.src_ptrs || !g.dst || g.shard_bytes <= 0 || g.shard_bytes % 16 || (reinterpret_cast<uintptr_t>(g.dst) & 15)) return TFB_ERR_ARG;
    a.seg[s] = FsdpAgSeg{static_cast<const uint4* const*>(g.src_ptrs), static_cast<uint4*>(g.dst), g.shard_bytes / 16};
  }
  int grid = sm_count() * 4;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (d->world <= 2) tfb::launch_k(fsdp_all_gather_kernel<2, 4>, grid, FS_THREADS, 0, st, a);
  else if (d->world <= 4) tfb::launch_k(fsdp_all_gather_kernel<4, 2>, grid, FS_THREADS, 0, st, a);
  else if (d->world <= 8) tfb::launch_k(fsdp_all_gather_kernel<8, 1>, grid, FS_THREADS, 0, st, a);
  else tfb::launch_k(fsdp_all_gather_kernel<FS_MAX_WORLD, 1>, grid, FS_THREADS, 0, st, a);
  return int(cudaGetLastError());
}

// out[t, :] = table row ids[t] fetched from the rank that owns it (zero when the id is outside this vocabulary slice).
TFB_API int tfb_embedding_fwd_sharded(const long long* ids, const void* shard_ptrs, void* out, int T, int H, long long per_rows,
                                      int world, long long vocab_lo, long long vocab_n, void* stream) {
  if (H % 8 || per_rows < 1 || world < 1) return TFB_ERR_ARG;
  const long long work = (long long)T * (H / 8);
  long long g = (work + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  tfb::launch_k(embedding_fwd_sharded_kernel, int(g < 1 ? 1 : g), 256, 0, static_cast<cudaStream_t>(stream), 
      ids, static_cast<const __nv_bfloat16* const*>(shard_ptrs), static_cast<__nv_bfloat16*>(out), T, H, per_rows, world,
      vocab_lo, vocab_n);
  return int(cudaGetLastError());
}
