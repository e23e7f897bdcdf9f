// Expert parallelism over NVLink peer memory: the dispatch and combine all-to-alls of a mixture-of-experts
// layer, each fused with the data movement it would otherwise need.
//
//   ep_plan      every rank holds the W x E matrix of routed-token counts (each rank pushed its row to all
//                peers).  From it every rank derives, identically, the layout of every expert's input
//                segment on its owner (segments padded to 128 rows, sources in rank order), hence the first
//                row `base[e]` that THIS rank's tokens for expert e occupy there, and for its own experts the
//                tile -> expert table of the grouped GEMM.
//   ep_dispatch  permutation fused with the all-to-all: one warp per (token, k) claims the next row of its
//                expert's segment and stores the token row straight into the owner's input buffer (16-byte
//                peer stores).
//   ep_combine   all-to-all fused with the top-k weighting: y[t] = sum_k w[t,k] * (row read from the owner's
//                output buffer with 16-byte peer loads).
//   ep_combine_bwd / ep_dispatch_bwd   the transposes (gradient rows pushed to / pulled from the owners).
// Barriers between the phases are tfb_comm_barrier launches (bounded waits, status word).
//
// Reference counterparts: ExpertParallel::forward_with_parallel (every rank routes all tokens, runs its
// experts, all-reduces [T, D]; src/model/moe_model.cpp:550-665), ExpertDispatcher::plan_all_to_all /
// dispatch_tokens / gather_results (plan only, src/model/expert_parallel.cpp:451-555).
#include "tfb_comm.cuh"
#include "tfb_host.h"

TFB_BOUNDS_DEFINE(ep_fused)

namespace tfb {

constexpr int EP_MAX_E = 256;
constexpr int EP_MAX_W = 16;

// counts_all: [W, E] int32 (local copy).  Outputs (all local):
//   base[E]            first row of this rank's tokens inside the owner's segment of expert e
//   seg_start[El + 1]  padded segment starts of this rank's own experts; expert_of_tile[max_tiles]; total_rows
//   cursor[E]          zeroed claim counters
__global__ void ep_plan_kernel(const int* __restrict__ counts_all, int W, int E, int rank, int* __restrict__ base,
                               int* __restrict__ seg_start, int* __restrict__ expert_of_tile, int max_tiles,
                               int* __restrict__ total_rows, int* __restrict__ cursor) {
  tfb::pdl_sync();
  if (threadIdx.x != 0) return;
  const int El = E / W;
  for (int owner = 0; owner < W; ++owner) {
    int off = 0;
    for (int j = 0; j < El; ++j) {
      const int e = owner * El + j;
      int tot = 0, before = 0;
      for (int s = 0; s < W; ++s) {
        if (s < rank) before += counts_all[s * E + e];
        tot += counts_all[s * E + e];
      }
      base[e] = off + before;
      cursor[e] = 0;
      if (owner == rank) {
        seg_start[j] = off;
        const int n = (tot + 127) / 128;
        for (int i = 0; i < n; ++i) {
          const int tile = off / 128 + i;
          if (tile < max_tiles) expert_of_tile[tile] = j;
        }
      }
      off += (tot + 127) / 128 * 128;
    }
    if (owner == rank) {
      seg_start[El] = off;
      *total_rows = off;
      for (int tile = off / 128; tile < max_tiles; ++tile) expert_of_tile[tile] = -1;
    }
  }
}

// every rank pushes its E counts into row `rank` of every peer's counts_all
__global__ void ep_push_counts_kernel(const int* __restrict__ counts, int* const* __restrict__ peer_counts_all, int W,
                                      int E, int rank) {
  tfb::pdl_sync();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= W * E) return;
  const int peer = i / E, e = i % E;
  peer_counts_all[peer][rank * E + e] = counts[e];
}

__global__ void ep_dispatch_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ topk_idx,
                                   const int* __restrict__ base, int* __restrict__ cursor, int* __restrict__ row_of,
                                   __nv_bfloat16* const* __restrict__ peer_xp, int T, int K, int H, int El,
                                   int max_rows) {
  tfb::pdl_sync();
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (w >= (long long)T * K) return;
  const int t = int(w / K);
  const int e = topk_idx[w];
  int row = 0;
  if (lane == 0) {
    row = base[e] + atomicAdd(cursor + e, 1);
    TFB_BOUNDS(row >= 0 && row < max_rows, 41, row, max_rows);
    if (row >= max_rows || row < 0) row = -1;  // beyond the buffer: dropped (cannot happen with worst-case sizing)
    row_of[w] = row;
  }
  row = __shfl_sync(0xffffffffu, row, 0);
  if (row < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (long long)t * H);
  uint4* dst = reinterpret_cast<uint4*>(peer_xp[e / El] + (long long)row * H);
  for (int i = lane; i < H / 8; i += 32) dst[i] = src[i];
}

__global__ void ep_combine_kernel(__nv_bfloat16* const* __restrict__ peer_yp, const int* __restrict__ topk_idx,
                                  const int* __restrict__ row_of, const float* __restrict__ topk_w,
                                  __nv_bfloat16* __restrict__ y, int T, int K, int H, int El) {
  tfb::pdl_sync();
  const int lane = threadIdx.x & 31;
  const long long t = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (t >= T) return;
  for (int i = lane; i < H / 8; i += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = 0; k < K; ++k) {
      const int row = row_of[t * K + k];
      if (row < 0) continue;
      const float wk = topk_w[t * K + k];
      const uint4 u = reinterpret_cast<const uint4*>(peer_yp[topk_idx[t * K + k] / El] + (long long)row * H)[i];
      const uint32_t ww[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16(ww[j]);
        acc[2 * j] = fmaf(wk, f.x, acc[2 * j]);
        acc[2 * j + 1] = fmaf(wk, f.y, acc[2 * j + 1]);
      }
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    reinterpret_cast<uint4*>(y + t * H)[i] = o;
  }
}

// dyp_owner[row] = w * dy[t] (peer store);  dw[t,k] = <dy[t], yp_owner[row]> (peer load)
__global__ void ep_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* const* __restrict__ peer_yp,
                                      __nv_bfloat16* const* __restrict__ peer_dyp, const int* __restrict__ topk_idx,
                                      const int* __restrict__ row_of, const float* __restrict__ topk_w,
                                      float* __restrict__ dw, int T, int K, int H, int El) {
  tfb::pdl_sync();
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (w >= (long long)T * K) return;
  const long long t = w / K;
  const int row = row_of[w];
  if (row < 0) { if (lane == 0) dw[w] = 0.f; return; }
  const int owner = topk_idx[w] / El;
  const float wk = topk_w[w];
  float dot = 0.f;
  for (int i = lane; i < H / 8; i += 32) {
    const uint4 g = reinterpret_cast<const uint4*>(dy + t * H)[i];
    const uint4 yv = reinterpret_cast<const uint4*>(peer_yp[owner] + (long long)row * H)[i];
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, yw[4] = {yv.x, yv.y, yv.z, yv.w};
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16(gw[j]), b = unpack_bf16(yw[j]);
      dot += a.x * b.x + a.y * b.y;
      op[j] = pack_bf16(wk * a.x, wk * a.y);
    }
    reinterpret_cast<uint4*>(peer_dyp[owner] + (long long)row * H)[i] = o;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  if (lane == 0) dw[w] = dot;
}

// dx[t] = sum_k dxp_owner[row]
__global__ void ep_dispatch_bwd_kernel(__nv_bfloat16* const* __restrict__ peer_dxp, const int* __restrict__ topk_idx,
                                       const int* __restrict__ row_of, __nv_bfloat16* __restrict__ dx, int T, int K,
                                       int H, int El) {
  tfb::pdl_sync();
  const int lane = threadIdx.x & 31;
  const long long t = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (t >= T) return;
  for (int i = lane; i < H / 8; i += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = 0; k < K; ++k) {
      const int row = row_of[t * K + k];
      if (row < 0) continue;
      const uint4 u = reinterpret_cast<const uint4*>(peer_dxp[topk_idx[t * K + k] / El] + (long long)row * H)[i];
      const uint32_t ww[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16(ww[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    reinterpret_cast<uint4*>(dx + t * H)[i] = o;
  }
}

}  // namespace tfb

using namespace tfb;
static inline unsigned ep_blocks(long long warps) { return unsigned((warps * 32 + 255) / 256); }

TFB_API int tfb_ep_push_counts(const int* counts, const void* peer_counts_all, int W, int E, int rank, void* stream) {
  if (W > EP_MAX_W || E > EP_MAX_E || E % W) return TFB_ERR_LIMIT;
  tfb::launch_k(ep_push_counts_kernel, (W * E + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream), 
      counts, static_cast<int* const*>(peer_counts_all), W, E, rank);
  return int(cudaGetLastError());
}
TFB_API int tfb_ep_plan(const int* counts_all, int W, int E, int rank, int* base, int* seg_start, int* expert_of_tile,
                        int max_tiles, int* total_rows, int* cursor, void* stream) {
  if (W > EP_MAX_W || E > EP_MAX_E || E % W) return TFB_ERR_LIMIT;
  tfb::launch_k(ep_plan_kernel, 1, 32, 0, static_cast<cudaStream_t>(stream), counts_all, W, E, rank, base, seg_start,
                                                                 expert_of_tile, max_tiles, total_rows, cursor);
  return int(cudaGetLastError());
}
TFB_API int tfb_ep_dispatch(const void* x, const int* topk_idx, const int* base, int* cursor, int* row_of,
                            const void* peer_xp, int T, int K, int H, int El, int max_rows, void* stream) {
  if (H % 8) return TFB_ERR_ARG;
  tfb::launch_k(ep_dispatch_kernel, ep_blocks((long long)T * K), 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(x), topk_idx, base, cursor, row_of,
      static_cast<__nv_bfloat16* const*>(peer_xp), T, K, H, El, max_rows);
  return int(cudaGetLastError());
}
TFB_API int tfb_ep_combine(const void* peer_yp, const int* topk_idx, const int* row_of, const float* topk_w, void* y,
                           int T, int K, int H, int El, void* stream) {
  if (H % 8) return TFB_ERR_ARG;
  tfb::launch_k(ep_combine_kernel, ep_blocks(T), 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<__nv_bfloat16* const*>(peer_yp), topk_idx, row_of, topk_w, static_cast<__nv_bfloat16*>(y), T, K, H, El);
  return int(cudaGetLastError());
}
TFB_API int tfb_ep_combine_bwd(const void* dy, const void* peer_yp, const void* peer_dyp, const int* topk_idx,
                               const int* row_of, const float* topk_w, float* dw, int T, int K, int H, int El,
                               void* stream) {
  if (H % 8) return TFB_ERR_ARG;
  tfb::launch_k(ep_combine_bwd_kernel, ep_blocks((long long)T * K), 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16* const*>(peer_yp),
      static_cast<__nv_bfloat16* const*>(peer_dyp), topk_idx, row_of, topk_w, dw, T, K, H, El);
  return int(cudaGetLastError());
}
TFB_API int tfb_ep_dispatch_bwd(const void* peer_dxp, const int* topk_idx, const int* row_of, void* dx, int T, int K,
                                int H, int El, void* stream) {
  if (H % 8) return TFB_ERR_ARG;
  tfb::launch_k(ep_dispatch_bwd_kernel, ep_blocks(T), 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<__nv_bfloat16* const*>(peer_dxp), topk_idx, row_of, static_cast<__nv_bfloat16*>(dx), T, K, H, El);
  return int(cudaGetLastError());
}
