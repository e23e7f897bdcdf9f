// Collectives over symmetric peer memory for messages where launch latency, not bandwidth, decides: the activations
// of tensor-parallel decode, gradient-norm scalars, small buckets.  One kernel per collective; every rank launches
// the same kernel on its own GPU, they meet at a flag barrier, move data with 128-bit peer loads / stores over
// NVLink and meet again before anyone may reuse the buffers.  No ring: through NVSwitch every peer is one hop away.
//
//   mode 0  all-reduce, one shot : every rank reads all W copies and reduces them in rank order (bit-identical
//                                  results everywhere); W x the traffic, one phase.  Output to a local buffer.
//   mode 1  all-reduce, two shot : rank r reduces slice r from all peers, then stores the result into slice r of
//                                  every peer (in place).  2 (W-1)/W of the data crosses NVLink per rank.
//   mode 2  reduce-scatter       : the first half of mode 1, result to a local buffer.
//   mode 3  all-gather           : every rank stores its slice into slice `rank` of every peer.
//   mode 4  broadcast            : the root stores its buffer into every peer's.
// ops: 0 sum, 1 average, 2 max, 3 min.  dtype: 0 bf16 (fp32 accumulation), 1 fp32.
//
// Reference counterparts: DistributedContext::all_reduce / broadcast / all_gather (src/trainer/distributed.cpp:43-123),
// RingAllReduce allreduce / reduce_scatter / allgather and its SUM/AVG/MAX/MIN ops (:288-519).
#include "tfb_comm.cuh"
#include "tfb_host.h"

namespace tfb {

constexpr int AR_MAX_WORLD = 16;

struct ArArgs {
  CommCtx c;
  void* const* bufs;       // [world] symmetric buffers
  void* local;             // local output (modes 0, 2) or local input slice (mode 3); may alias nothing symmetric
  long long n;             // elements in the whole buffer
  int dtype, op, mode, root;
  unsigned int* ticket;
};

__device__ __forceinline__ uint4 ld_peer_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_peer_u4(void* p, uint4 v) {
  asm volatile("st.global.relaxed.sys.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ float ar_op(float a, float b, int op) {
  return op <= 1 ? a + b : (op == 2 ? fmaxf(a, b) : fminf(a, b));
}

// reduce W 16-byte vectors (in rank order) -> one vector
__device__ __forceinline__ uint4 ar_reduce(const uint4* v, int W, int dtype, int op) {
  if (dtype == 1) {
    float4 acc = *reinterpret_cast<const float4*>(&v[0]);
    for (int r = 1; r < W; ++r) {
      const float4 x = *reinterpret_cast<const float4*>(&v[r]);
      acc.x = ar_op(acc.x, x.x, op); acc.y = ar_op(acc.y, x.y, op); acc.z = ar_op(acc.z, x.z, op); acc.w = ar_op(acc.w, x.w, op);
    }
    if (op == 1) { const float s = 1.f / float(W); acc.x *= s; acc.y *= s; acc.z *= s; acc.w *= s; }
    return *reinterpret_cast<uint4*>(&acc);
  }
  float acc[8];
  {
    const uint32_t w[4] = {v[0].x, v[0].y, v[0].z, v[0].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16(w[j]); acc[2 * j] = f.x; acc[2 * j + 1] = f.y; }
  }
  for (int r = 1; r < W; ++r) {
    const uint32_t w[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16(w[j]);
      acc[2 * j] = ar_op(acc[2 * j], f.x, op);
      acc[2 * j + 1] = ar_op(acc[2 * j + 1], f.y, op);
    }
  }
  const float s = op == 1 ? 1.f / float(W) : 1.f;
  uint4 o;
  o.x = pack_bf16(acc[0] * s, acc[1] * s); o.y = pack_bf16(acc[2] * s, acc[3] * s);
  o.z = pack_bf16(acc[4] * s, acc[5] * s); o.w = pack_bf16(acc[6] * s, acc[7] * s);
  return o;
}

__global__ void __launch_bounds__(512) collective_kernel(ArArgs a) {
  tfb::pdl_sync();
  __shared__ int sh_ok;
  const CommCtx& c = a.c;
  const int W = c.world, rank = c.rank;
  const int e0 = ld_volatile(c.epoch);
  if (blockIdx.x == 0 && threadIdx.x == 0) comm_signal_all(c, e0 + 1);   // my input is in place / my buffer may be written
  if (!comm_wait_all_block(c, e0 + 1, &sh_ok)) return;

  const int esz = a.dtype == 1 ? 4 : 2;
  const long long nvec = a.n * esz / 16;          // 16-byte vectors in the whole buffer
  const long long svec = nvec / W;                // vectors per slice
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x, nth = (long long)gridDim.x * blockDim.x;
  const uint4* src[AR_MAX_WORLD];
  uint4* dst[AR_MAX_WORLD];
#pragma unroll
  for (int r = 0; r < AR_MAX_WORLD; ++r) {
    src[r] = r < W ? static_cast<const uint4*>(a.bufs[r]) : nullptr;
    dst[r] = r < W ? static_cast<uint4*>(a.bufs[(rank + r) % W]) : nullptr;   // stores start at the local copy, then fan out
  }
  if (a.mode == 0) {
    uint4* out = static_cast<uint4*>(a.local);
    for (long long i = tid; i < nvec; i += nth) {
      uint4 v[AR_MAX_WORLD];
#pragma unroll
      for (int r = 0; r < AR_MAX_WORLD; ++r)
        if (r < W) v[r] = r == rank ? src[r][i] : ld_peer_u4(src[r] + i);
      out[i] = ar_reduce(v, W, a.dtype, a.op);
    }
  } else if (a.mode == 1 || a.mode == 2) {
    const long long lo = svec * rank;
    uint4* out = static_cast<uint4*>(a.local);
    for (long long i = tid; i < svec; i += nth) {
      uint4 v[AR_MAX_WORLD];
#pragma unroll
      for (int r = 0; r < AR_MAX_WORLD; ++r)
        if (r < W) v[r] = r == rank ? src[r][lo + i] : ld_peer_u4(src[r] + lo + i);
      const uint4 o = ar_reduce(v, W, a.dtype, a.op);
      if (a.mode == 2) out[i] = o;
      else {
#pragma unroll
        for (int r = 0; r < AR_MAX_WORLD; ++r)
          if (r < W) { if (r == 0) dst[0][lo + i] = o; else st_peer_u4(dst[r] + lo + i, o); }
      }
    }
  } else if (a.mode == 3) {
    const long long lo = svec * rank;
    const uint4* in = static_cast<const uint4*>(a.local);
    for (long long i = tid; i < svec; i += nth) {
      const uint4 o = in[i];
#pragma unroll
      for (int r = 0; r < AR_MAX_WORLD; ++r)
        if (r < W) { if (r == 0) dst[0][lo + i] = o; else st_peer_u4(dst[r] + lo + i, o); }
    }
  } else if (a.mode == 4 && rank == a.root) {
    for (long long i = tid; i < nvec; i += nth) {
      const uint4 o = src[rank][i];
#pragma unroll
      for (int r = 1; r < AR_MAX_WORLD; ++r)
        if (r < W) st_peer_u4(dst[r] + i, o);
    }
  }
  // the last CTA to finish tells the peers and waits for theirs: afterwards nobody reads or writes this rank's buffer
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int t = atomicAdd(a.ticket, 1u);
    if (t == gridDim.x - 1) {
      *a.ticket = 0u;
      comm_signal_all(c, e0 + 2);
      comm_wait_all(c, e0 + 2);
      *c.epoch = e0 + 2;
    }
  }
}

}  // namespace tfb

// bufs: device table of the W symmetric buffer addresses (n elements each, n * elem_size a multiple of 16 * world).
// local: modes 0 / 2 output, mode 3 input slice, else unused.  ticket: one zero-initialised unsigned int in local memory.
// max_ctas: 0 = sized from n (small messages get one CTA so that the barrier cost is paid once).
TFB_API int tfb_collective(const void* bufs, void* local, long long n, int dtype, int op, int mode, int root,
                           const void* flag_ptrs, int* epoch, int rank, int world, int* status, void* ticket, int max_ctas,
                           void* stream) {
  using namespace tfb;
  if (world < 1 || world > AR_MAX_WORLD || n <= 0 || mode < 0 || mode > 4 || op < 0 || op > 3 || root < 0 || root >= world) return TFB_ERR_ARG;
  const int esz = dtype == 1 ? 4 : 2;
  if ((n * esz) % (16 * world)) return TFB_ERR_ARG;
  if ((mode == 0 || mode == 2 || mode == 3) && !local) return TFB_ERR_ARG;
  ArArgs a;
  a.c = CommCtx{static_cast<int* const*>(flag_ptrs), epoch, rank, world, status};
  a.bufs = static_cast<void* const*>(bufs);
  a.local = local;
  a.n = n; a.dtype = dtype; a.op = op; a.mode = mode; a.root = root;
  a.ticket = static_cast<unsigned int*>(ticket);
  const long long work = (mode == 0 || mode == 4) ? n * esz / 16 : n * esz / 16 / world;
  long long ctas = (work + 512 * 4 - 1) / (512 * 4);
  const long long cap = max_ctas > 0 ? max_ctas : sm_count();   // one CTA per SM at most: every CTA must be resident to poll
  if (ctas > cap) ctas = cap;
  if (ctas < 1) ctas = 1;
  tfb::launch_k(collective_kernel, unsigned(ctas), 512, 0, static_cast<cudaStream_t>(stream), a);
  return int(cudaGetLastError());
}
