// Collectives over symmetric peer memory for messages where launch latency, not bandwidth, decides: the activations
// of tensor-parallel decode, gradient-norm scalars, small buckets.  One kernel per collective; every rank launches
// the same kernel on its own GPU, they meet at a flag barrier, move data with 128-bit peer loads / stores over
// NVLink and meet again before anyone may reuse the buffers.  No ring: through NVSwitch every peer is one hop away.
//
//   mode 0  all-reduce, one shot : every rank reads all W copies and reduces them in rank order (bit-identical
//                                  results everywhere); W x the traffic, one phase.  Output to a local buffer, with an
//                                  optional local addend (the residual stream of a decoder block) summed in fp32
//                                  before the one rounding.
//   mode 1  all-reduce, two shot : rank r reduces slice r from all peers, then stores the result into slice r of
//                                  every peer (in place).  2 (W-1)/W of the data crosses NVLink per rank.
//   mode 2  reduce-scatter       : the first half of mode 1, result to a local buffer.
//   mode 3  all-gather           : every rank stores its slice into slice `rank` of every peer.
//   mode 4  broadcast            : the root stores its buffer into every peer's.
// ops: 0 sum, 1 average, 2 max, 3 min.  dtype: 0 bf16 (fp32 accumulation), 1 fp32.
//
// Closing barrier.  It exists so that nobody overwrites a staging buffer that a slower peer still reads.  A caller
// that alternates between two staging buffers can drop it for the one-shot all-reduce (flags bit 0): a rank passes the
// opening barrier of collective n+1 only after every peer has finished collective n, so when it refills the buffer of
// collective n (for n+2) no peer reads it any more.  That halves the synchronisation cost of the decode all-reduce.
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
  const void* extra;       // mode 0, op sum: local addend of n elements or null
  int flags;               // bit 0: no closing barrier (see the top of the file)
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
__device__ __forceinline__ uint4 ar_reduce(const uint4* v, int W, int dtype, int op, const uint4* extra = nullptr) {
  if (dtype == 1) {
    float4 acc = *reinterpret_cast<const float4*>(&v[0]);
    for (int r = 1; r < W; ++r) {
      const float4 x = *reinterpret_cast<const float4*>(&v[r]);
      acc.x = ar_op(acc.x, x.x, op); acc.y = ar_op(acc.y, x.y, op); acc.z = ar_op(acc.z, x.z, op); acc.w = ar_op(acc.w, x.w, op);
    }
    if (op == 1) { const float s = 1.f / float(W); acc.x *= s; acc.y *= s; acc.z *= s; acc.w *= s; }
    if (extra) {
      const float4 x = *reinterpret_cast<const float4*>(extra);
      acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
    }
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
  if (extra) {
    const uint32_t w[4] = {extra->x, extra->y, extra->z, extra->w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16(w[j]);
      acc[2 * j] = acc[2 * j] * s + f.x;
      acc[2 * j + 1] = acc[2 * j + 1] * s + f.y;
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    return o;
  }
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
  if (blockIdx.x == 0) comm_signal_all_par(c, e0 + 1);   // my input is in place / my buffer may be written
  if (!comm_wait_all_block_par(c, e0 + 1, &sh_ok)) return;

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
    const uint4* extra = static_cast<const uint4*>(a.extra);
    for (long long i = tid; i < nvec; i += nth) {
      uint4 v[AR_MAX_WORLD];
#pragma unroll
      for (int r = 0; r < AR_MAX_WORLD; ++r)
        if (r < W) v[r] = r == rank ? src[r][i] : ld_peer_u4(src[r] + i);
      uint4 x;
      if (extra) x = extra[i];
      out[i] = ar_reduce(v, W, a.dtype, a.op, extra ? &x : nullptr);
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
      if (a.flags & 1) {
        *c.epoch = e0 + 1;
      } else {
        comm_signal_all(c, e0 + 2);
        comm_wait_all(c, e0 + 2);
        *c.epoch = e0 + 2;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Flag-in-data all-reduce for decode-sized messages: no barrier at all.  Every rank pushes its input into a receive area
// of every peer as 8-byte {data word, sequence number} pairs (two pairs per 16-byte store; an 8-byte aligned store is
// not torn on NVLink, so a pair whose sequence number matches carries valid data), then reads the W - 1 areas peers
// fill in its own memory, spinning on the sequence number of each pair, reduces in rank order and writes the result
// (plus an optional local addend) to a local buffer.  One NVLink store latency end to end instead of a flag barrier, a
// round of peer loads and a second barrier.
//
// Receive areas are double-buffered on the parity of the sequence number.  That is enough: a rank starts collective
// s + 2 only after it finished s + 1, for which it needed every peer's s + 1 data, which a peer pushes only after its
// own collective s is complete - so nobody still reads the area of collective s when it is overwritten.  The sequence
// number lives in device memory (one counter per rank, advanced by the last CTA), so captured graphs replay correctly.
// Layout of a rank's area: [2 parities][W senders][cap_vec] x 32 bytes.
struct LlArgs {
  uint4* const* recv;      // [world] receive areas
  const uint4* in;         // local input, n elements
  const uint4* extra;      // optional local addend
  uint4* out;              // local output
  long long nvec, cap_vec; // 16-byte vectors in the message / per sender slot
  int* seq;                // local sequence counter
  unsigned int* ticket;
  int* status;
  int rank, world, dtype, op;
};

__device__ __forceinline__ void ll_accumulate(float* acc, uint4 x, int dtype, int op, bool first) {
  float f[8];
  int n = 8;
  if (dtype == 1) {
    f[0] = __uint_as_float(x.x); f[1] = __uint_as_float(x.y); f[2] = __uint_as_float(x.z); f[3] = __uint_as_float(x.w);
    f[4] = f[5] = f[6] = f[7] = 0.f;
    n = 4;
  } else {
    const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 t = unpack_bf16(w[j]); f[2 * j] = t.x; f[2 * j + 1] = t.y; }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j)
    if (j < n) acc[j] = first ? f[j] : ar_op(acc[j], f[j], op);
}
__device__ __forceinline__ uint4 ll_finish(const float* acc, int W, int dtype, int op, const uint4* extra) {
  const float s = op == 1 ? 1.f / float(W) : 1.f;
  if (dtype == 1) {
    float4 o = make_float4(acc[0] * s, acc[1] * s, acc[2] * s, acc[3] * s);
    if (extra) {
      const float4 x = *reinterpret_cast<const float4*>(extra);
      o.x += x.x; o.y += x.y; o.z += x.z; o.w += x.w;
    }
    return *reinterpret_cast<uint4*>(&o);
  }
  float r[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) r[j] = acc[j] * s;
  if (extra) {
    const uint32_t w[4] = {extra->x, extra->y, extra->z, extra->w};
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 t = unpack_bf16(w[j]); r[2 * j] += t.x; r[2 * j + 1] += t.y; }
  }
  uint4 o;
  o.x = pack_bf16(r[0], r[1]); o.y = pack_bf16(r[2], r[3]); o.z = pack_bf16(r[4], r[5]); o.w = pack_bf16(r[6], r[7]);
  return o;
}

__global__ void __launch_bounds__(512) allreduce_ll_kernel(LlArgs a) {
  tfb::pdl_sync();
  const int W = a.world, rank = a.rank;
  const int seq = ld_volatile(a.seq) + 1;
  const uint32_t tag = uint32_t(seq);
  const long long par = seq & 1;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x, nth = (long long)gridDim.x * blockDim.x;
  const uint64_t t0 = globaltimer_ns();
  bool ok = true;
  for (long long i = tid; i < a.nvec; i += nth) {
    const uint4 v = a.in[i];
    const uint4 p0 = make_uint4(v.x, tag, v.y, tag), p1 = make_uint4(v.z, tag, v.w, tag);
#pragma unroll
    for (int rr = 1; rr < AR_MAX_WORLD; ++rr) {
      if (rr < W) {
        const int r = (rank + rr) % W;
        uint4* dst = a.recv[r] + ((par * W + rank) * a.cap_vec + i) * 2;
        st_peer_u4(dst, p0);
        st_peer_u4(dst + 1, p1);
      }
    }
    float acc[8];
    for (int r = 0; r < W; ++r) {       // rank order: every rank adds the same numbers in the same order
      uint4 val = v;
      if (r != rank) {
        const uint4* src = a.recv[rank] + ((par * W + r) * a.cap_vec + i) * 2;
        uint4 x = ld_peer_u4(src), y = ld_peer_u4(src + 1);
        uint32_t it = 0;
        while (ok && !(x.y == tag && x.w == tag && y.y == tag && y.w == tag)) {
          if ((++it & 255u) == 0u && globaltimer_ns() - t0 > TFB_WAIT_NS) {
            report(a.status, ST_TIMEOUT_FLAG);
            ok = false;
          }
          x = ld_peer_u4(src);
          y = ld_peer_u4(src + 1);
        }
        val = make_uint4(x.x, x.z, y.x, y.z);
      }
      ll_accumulate(acc, val, a.dtype, a.op, r == 0);
    }
    uint4 e;
    if (a.extra) e = a.extra[i];
    if (ok) a.out[i] = ll_finish(acc, W, a.dtype, a.op, a.extra ? &e : nullptr);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(a.ticket, 1u);
    if (t == gridDim.x - 1) {
      *a.ticket = 0u;
      *a.seq = seq;
    }
  }
}

}  // namespace tfb

// Flag-in-data all-reduce (see allreduce_ll_kernel).  recv: device table of the W receive areas, each
// 2 * world * cap_bytes * 2 bytes, zero-initialised; n elements with n * elem_size a multiple of 16 and <= cap_bytes;
// in / out / extra local (16-byte aligned; out may alias in); seq: one zero-initialised int in local memory per
// communicator; ticket: one zero-initialised unsigned int.  op: 0 sum, 1 average, 2 max, 3 min (extra with sum only).
TFB_API int tfb_allreduce_ll(const void* recv, const void* in, const void* extra, void* out, long long n, long long cap_bytes,
                             int dtype, int op, int rank, int world, int* seq, void* ticket, int* status, int max_ctas,
                             void* stream) {
  using namespace tfb;
  const int esz = dtype == 1 ? 4 : 2;
  if (world < 1 || world > AR_MAX_WORLD || rank < 0 || rank >= world || n <= 0 || op < 0 || op > 3 || !recv || !in || !out || !seq || !ticket)
    return TFB_ERR_ARG;
  if ((n * esz) % 16 || n * esz > cap_bytes || cap_bytes % 16) return TFB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(extra)) & 15) return TFB_ERR_ARG;
  if (extra && op != 0) return TFB_ERR_ARG;
  LlArgs a;
  a.recv = static_cast<uint4* const*>(recv);
  a.in = static_cast<const uint4*>(in);
  a.extra = static_cast<const uint4*>(extra);
  a.out = static_cast<uint4*>(out);
  a.nvec = n * esz / 16;
  a.cap_vec = cap_bytes / 16;
  a.seq = seq;
  a.ticket = static_cast<unsigned int*>(ticket);
  a.status = status;
  a.rank = rank; a.world = world; a.dtype = dtype; a.op = op;
  long long ctas = (a.nvec + 511) / 512;
  const long long cap = max_ctas > 0 ? max_ctas : 64;
  if (ctas > cap) ctas = cap;
  tfb::launch_k(allreduce_ll_kernel, unsigned(ctas), 512, 0, static_cast<cudaStream_t>(stream), a);
  return int(cudaGetLastError());
}

// bufs: device table of the W symmetric buffer addresses (n elements each, n * elem_size a multiple of 16 * world).
// local: modes 0 / 2 output, mode 3 input slice, else unused.  ticket: one zero-initialised unsigned int in local memory.
// max_ctas: 0 = sized from n (small messages get one CTA so that the barrier cost is paid once).
// extra: mode 0 with op sum only: local addend (n elements, 16-byte aligned) or null.  flags bit 0: mode 0 only, no closing
// barrier; the caller alternates between two staging buffers.
TFB_API int tfb_collective(const void* bufs, void* local, long long n, int dtype, int op, int mode, int root,
                           const void* flag_ptrs, int* epoch, int rank, int world, int* status, void* ticket, int max_ctas,
                           const void* extra, int flags, void* stream) {
  using namespace tfb;
  if (world < 1 || world > AR_MAX_WORLD || n <= 0 || mode < 0 || mode > 4 || op < 0 || op > 3 || root < 0 || root >= world) return TFB_ERR_ARG;
  const int esz = dtype == 1 ? 4 : 2;
  if ((n * esz) % (16 * world)) return TFB_ERR_ARG;
  if ((mode == 0 || mode == 2 || mode == 3) && !local) return TFB_ERR_ARG;
  if ((extra || (flags & 1)) && mode != 0) return TFB_ERR_ARG;
  if (extra && (op != 0 || (reinterpret_cast<uintptr_t>(extra) & 15))) return TFB_ERR_ARG;
  ArArgs a;
  a.c = CommCtx{static_cast<int* const*>(flag_ptrs), epoch, rank, world, status};
  a.bufs = static_cast<void* const*>(bufs);
  a.local = local;
  a.n = n; a.dtype = dtype; a.op = op; a.mode = mode; a.root = root;
  a.ticket = static_cast<unsigned int*>(ticket);
  a.extra = extra;
  a.flags = flags;
  const long long work = (mode == 0 || mode == 4) ? n * esz / 16 : n * esz / 16 / world;
  long long ctas = (work + 512 * 4 - 1) / (512 * 4);
  const long long cap = max_ctas > 0 ? max_ctas : sm_count();   // one CTA per SM at most: every CTA must be resident to poll
  if (ctas > cap) ctas = cap;
  if (ctas < 1) ctas = 1;
  tfb::launch_k(collective_kernel, unsigned(ctas), 512, 0, static_cast<cudaStream_t>(stream), a);
  return int(cudaGetLastError());
}
