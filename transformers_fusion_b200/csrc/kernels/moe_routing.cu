// Mixture-of-experts routing on the device.
//
//   router_topk     : softmax over E experts + top-k selection per token (weights optionally
//                     renormalised over the selected k), per-expert token counts and probability sums
//                     (the two factors of the load-balance loss E * sum_e f_e * P_e), log-sum-exp for z-loss.
//   moe_plan        : exclusive scan of the counts into expert segments padded to 128 rows, plus the
//                     expert index of every 128-row tile (what the grouped GEMMs consume).
//   moe_permute     : scatter token rows into their expert segments (row of every (token, k) recorded).
//   moe_combine     : y[t] = sum_k w[t,k] * expert_out[row[t,k]]   (the top-k weighting of the combine step).
//   moe_permute_bwd / moe_combine_bwd : the transposes of the two data movements.
//
// Reference counterparts: softmax_with_topk (src/model/moe_core.cpp:98-149), load-balance loss
// (:155-188), moe_gather_kernel / moe_scatter_kernel (src/backend/gpu_compute_cuda.cpp:539,578),
// ExpertDispatcher::route_tokens (src/model/expert_parallel.cpp:354-418, renormalised top-k).
#include <algorithm>
#include "tfb_host.h"
#include "tfb_ptx.cuh"

TFB_BOUNDS_DEFINE(moe_routing)

namespace tfb {

constexpr int MAX_E = 256;
constexpr int MAX_K = 8;

// one warp per token, grid-stride; expert counts, probability sums and the sum of lse^2 are aggregated per block in shared
// memory and reach global memory with one atomic per expert per block (a global atomic per (token, k) on E addresses
// serialises: 65k assignments on 16 experts took 53 us)
__global__ void __launch_bounds__(256) router_topk_kernel(const __nv_bfloat16* __restrict__ logits_bf16, const float* __restrict__ logits_f32,
                                                          int T, int E, int K, int renorm, int* __restrict__ topk_idx,
                                                          float* __restrict__ topk_w, float* __restrict__ probs_out,
                                                          int* __restrict__ counts, float* __restrict__ prob_sums,
                                                          float* __restrict__ lse_out, float* __restrict__ lse_sq_sum) {
  tfb::pdl_sync();
  __shared__ int s_cnt[MAX_E];
  __shared__ float s_ps[MAX_E];
  __shared__ float s_lsq;
  for (int e = threadIdx.x; e < E; e += blockDim.x) { s_cnt[e] = 0; s_ps[e] = 0.f; }
  if (threadIdx.x == 0) s_lsq = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (gridDim.x * (long long)blockDim.x) >> 5;
  constexpr int PER = MAX_E / 32;
  for (long long t = warp0; t < T; t += nwarps) {
    float v[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + i * 32;
      v[i] = -INFINITY;
      if (e < E) v[i] = logits_f32 ? logits_f32[t * E + e] : __bfloat162float(logits_bf16[t * E + e]);
      mx = fmaxf(mx, v[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      v[i] = (lane + i * 32 < E) ? __expf(v[i] - mx) : 0.f;
      sum += v[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.f / sum;
    if (lane == 0) {
      const float lse = mx + logf(sum);
      if (lse_out) lse_out[t] = lse;
      if (lse_sq_sum) atomicAdd(&s_lsq, lse * lse);
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      v[i] *= inv;
      const int e = lane + i * 32;
      if (e < E) {
        if (probs_out) probs_out[t * E + e] = v[i];
        if (prob_sums) atomicAdd(&s_ps[e], v[i]);
      }
    }
    // iterative arg-max, ties to the lower expert index
    float sel_w[MAX_K];
    int sel_i[MAX_K];
    float wsum = 0.f;
    for (int k = 0; k < K; ++k) {
      float best = -1.f;
      int bi = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int e = lane + i * 32;
        if (e < E && (v[i] > best || (v[i] == best && e < bi))) { best = v[i]; bi = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      sel_w[k] = best;
      sel_i[k] = bi;
      wsum += best;
      if ((bi & 31) == lane) v[bi >> 5] = -1.f;  // remove from the next round
    }
    if (lane == 0) {
      for (int k = 0; k < K; ++k) {
        topk_idx[t * K + k] = sel_i[k];
        topk_w[t * K + k] = renorm ? sel_w[k] / wsum : sel_w[k];
        if (counts) atomicAdd(&s_cnt[sel_i[k]], 1);
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    if (counts && s_cnt[e]) atomicAdd(counts + e, s_cnt[e]);
    if (prob_sums && s_ps[e] != 0.f) atomicAdd(prob_sums + e, s_ps[e]);
  }
  if (threadIdx.x == 0 && lse_sq_sum) atomicAdd(lse_sq_sum, s_lsq);
}

// single block: seg_start[e] (padded to 128), expert_of_tile, total padded rows; cursor[e] = seg_start[e]
__global__ void moe_plan_kernel(const int* __restrict__ counts, int E, int* __restrict__ seg_start,
                                int* __restrict__ cursor, int* __restrict__ expert_of_tile, int max_tiles,
                                int* __restrict__ total_rows) {
  tfb::pdl_sync();
  if (threadIdx.x == 0) {
    int off = 0, tile = 0;
    for (int e = 0; e < E; ++e) {
      seg_start[e] = off;
      cursor[e] = off;
      const int n = (counts[e] + 127) / 128;
      for (int i = 0; i < n && tile < max_tiles; ++i) expert_of_tile[tile++] = e;
      off += n * 128;
    }
    seg_start[E] = off;
    *total_rows = off;
    for (; tile < max_tiles; ++tile) expert_of_tile[tile] = -1;
  }
}

// A block takes PERM_ROWS consecutive (token, k) assignments: it counts them per expert in shared memory, claims one
// contiguous range per expert with a single global atomic, and then its warps copy the rows.  (One global atomic per
// assignment on E cursors serialised: 83 us for 65k rows.)
constexpr int PERM_ROWS = 64;
__global__ void __launch_bounds__(256) moe_permute_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ topk_idx,
                                                          int* __restrict__ cursor, int* __restrict__ row_of, int* __restrict__ token_of_row,
                                                          __nv_bfloat16* __restrict__ xp, int T, int K, int H, int E) {
  tfb::pdl_sync();
  __shared__ int s_cnt[MAX_E];
  __shared__ int s_base[MAX_E];
  __shared__ int s_rank[PERM_ROWS];
  __shared__ int s_exp[PERM_ROWS];
  const long long total = (long long)T * K;
  const long long w0 = blockIdx.x * (long long)PERM_ROWS;
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_cnt[e] = 0;
  __syncthreads();
  if (threadIdx.x < PERM_ROWS && w0 + threadIdx.x < total) {
    int e = topk_idx[w0 + threadIdx.x];
    TFB_BOUNDS(e >= 0 && e < E, 5, e, E);
    e = min(max(e, 0), E - 1);
    s_exp[threadIdx.x] = e;
    s_rank[threadIdx.x] = atomicAdd(&s_cnt[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_base[e] = s_cnt[e] ? atomicAdd(cursor + e, s_cnt[e]) : 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = warp; i < PERM_ROWS && w0 + i < total; i += 8) {
    const long long w = w0 + i;
    const int t = int(w / K);
    const int row = s_base[s_exp[i]] + s_rank[i];
    if (lane == 0) {
      row_of[w] = row;
      token_of_row[row] = t;
    }
    const uint4* src = reinterpret_cast<const uint4*>(x + (long long)t * H);
    uint4* dst = reinterpret_cast<uint4*>(xp + (long long)row * H);
    for (int j = lane; j < H / 8; j += 32) dst[j] = src[j];
  }
}

// Zeroes the rows of a [max_rows, H] expert buffer that hold no assignment: the padding behind every expert's segment
// (with `counts`) and everything from `total` on.  Without `counts` only the tail is cleared (outputs of the grouped GEMM,
// whose padding rows are products of zero rows already).
__global__ void __launch_bounds__(256) moe_zero_pads_kernel(__nv_bfloat16* __restrict__ buf, int H, const int* __restrict__ seg_start,
                                                            const int* __restrict__ counts, int E, const int* __restrict__ total,
                                                            int max_rows) {
  tfb::pdl_sync();
  const int seg = blockIdx.x;                       // 0..E-1: expert padding, E: tail
  int r0, r1;
  if (seg < E) {
    if (!counts) return;
    r0 = seg_start[seg] + counts[seg];
    r1 = seg_start[seg + 1];
  } else {
    r0 = *total;
    r1 = max_rows;
  }
  // grid.y is sized for a tail of many thousand rows (an expert-parallel buffer is provisioned for the worst-case
  // imbalance); blocks beyond the range leave at once
  const long long n8 = (long long)(r1 - r0) * H / 8;
  if (blockIdx.y * (long long)blockDim.x >= n8) return;
  uint4* p = reinterpret_cast<uint4*>(buf + (long long)r0 * H);
  for (long long i = blockIdx.y * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.y * blockDim.x)
    p[i] = make_uint4(0, 0, 0, 0);
}

// y[t] = sum_k w[t,k] * yp[row_of[t,k]]; one warp per token
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ yp, const int* __restrict__ row_of,
                                   const float* __restrict__ topk_w, __nv_bfloat16* __restrict__ y,
                                   const __nv_bfloat16* __restrict__ residual, int T, int K, int H) {
  tfb::pdl_sync();
  const int lane = threadIdx.x & 31;
  const long long t = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (t >= T) return;
  for (int i = lane; i < H / 8; i += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (residual) {
      const uint4 u = reinterpret_cast<const uint4*>(residual + t * H)[i];
      const uint32_t ww[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16(ww[j]);
        acc[2 * j] = f.x;
        acc[2 * j + 1] = f.y;
      }
    }
    for (int k = 0; k < K; ++k) {
      const float wk = topk_w[t * K + k];
      const uint4 u = reinterpret_cast<const uint4*>(yp + (long long)row_of[t * K + k] * H)[i];
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

// backward of combine: dyp[row_of[t,k]] = w[t,k] * dy[t];  dw[t,k] = <dy[t], yp[row_of[t,k]]>; one warp per (token, k)
__global__ void moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ yp,
                                       const int* __restrict__ row_of, const float* __restrict__ topk_w,
                                       __nv_bfloat16* __restrict__ dyp, float* __restrict__ dw, int T, int K, int H) {
  tfb::pdl_sync();
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (w >= (long long)T * K) return;
  const long long t = w / K;
  const long long row = row_of[w];
  const float wk = topk_w[w];
  float dot = 0.f;
  for (int i = lane; i < H / 8; i += 32) {
    const uint4 g = reinterpret_cast<const uint4*>(dy + t * H)[i];
    const uint4 yv = reinterpret_cast<const uint4*>(yp + row * H)[i];
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, yw[4] = {yv.x, yv.y, yv.z, yv.w};
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16(gw[j]), b = unpack_bf16(yw[j]);
      dot += a.x * b.x + a.y * b.y;
      op[j] = pack_bf16(wk * a.x, wk * a.y);
    }
    reinterpret_cast<uint4*>(dyp + row * H)[i] = o;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  if (lane == 0 && dw) dw[w] = dot;
}

// backward of permute: dx[t] = sum_k dxp[row_of[t,k]]; one warp per token
__global__ void moe_permute_bwd_kernel(const __nv_bfloat16* __restrict__ dxp, const int* __restrict__ row_of,
                                       __nv_bfloat16* __restrict__ dx, int T, int K, int H) {
  tfb::pdl_sync();
  const int lane = threadIdx.x & 31;
  const long long t = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (t >= T) return;
  for (int i = lane; i < H / 8; i += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = 0; k < K; ++k) {
      const uint4 u = reinterpret_cast<const uint4*>(dxp + (long long)row_of[t * K + k] * H)[i];
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

static inline unsigned warps_to_blocks(long long warps) { return unsigned((warps * 32 + 255) / 256); }

TFB_API int tfb_router_topk2(const void* logits, int logits_f32, int T, int E, int K, int renorm, int* topk_idx, float* topk_w,
                             float* probs, int* counts, float* prob_sums, float* lse, float* lse_sq_sum, void* stream);
TFB_API int tfb_moe_permute2(const void* x, const int* topk_idx, int* cursor, int* row_of, int* token_of_row, void* xp, int T, int K,
                             int H, int E, void* stream);
TFB_API int tfb_router_topk(const void* logits, int logits_f32, int T, int E, int K, int renorm, int* topk_idx,
                            float* topk_w, float* probs, int* counts, float* prob_sums, float* lse, void* stream) {
  return tfb_router_topk2(logits, logits_f32, T, E, K, renorm, topk_idx, topk_w, probs, counts, prob_sums, lse, nullptr, stream);
}
// As tfb_router_topk, plus lse_sq_sum: one float that receives sum_t lse_t^2 (zero it first).
TFB_API int tfb_router_topk2(const void* logits, int logits_f32, int T, int E, int K, int renorm, int* topk_idx, float* topk_w,
                             float* probs, int* counts, float* prob_sums, float* lse, float* lse_sq_sum, void* stream) {
  if (E > MAX_E || K > MAX_K || K < 1 || K > E) return TFB_ERR_LIMIT;
  const int blocks = int(std::min<long long>(warps_to_blocks(T), 148 * 8));
  tfb::launch_k(router_topk_kernel, blocks, 256, 0, static_cast<cudaStream_t>(stream), 
      logits_f32 ? nullptr : static_cast<const __nv_bfloat16*>(logits),
      logits_f32 ? static_cast<const float*>(logits) : nullptr, T, E, K, renorm, topk_idx, topk_w, probs, counts,
      prob_sums, lse, lse_sq_sum);
  return int(cudaGetLastError());
}
TFB_API int tfb_moe_plan(const int* counts, int E, int* seg_start, int* cursor, int* expert_of_tile, int max_tiles,
                         int* total_rows, void* stream) {
  tfb::launch_k(moe_plan_kernel, 1, 32, 0, static_cast<cudaStream_t>(stream), counts, E, seg_start, cursor, expert_of_tile,
                                                                  max_tiles, total_rows);
  return int(cudaGetLastError());
}
TFB_API int tfb_moe_permute(const void* x, const int* topk_idx, int* cursor, int* row_of, int* token_of_row, void* xp,
                            int T, int K, int H, void* stream) {
  return tfb_moe_permute2(x, topk_idx, cursor, row_of, token_of_row, xp, T, K, H, MAX_E, stream);
}
TFB_API int tfb_moe_permute2(const void* x, const int* topk_idx, int* cursor, int* row_of, int* token_of_row, void* xp, int T, int K,
                             int H, int E, void* stream) {
  if (H % 8 || E < 1 || E > MAX_E) return TFB_ERR_ARG;
  const long long rows = (long long)T * K;
  tfb::launch_k(moe_permute_kernel, int((rows + PERM_ROWS - 1) / PERM_ROWS), 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(x), topk_idx, cursor, row_of, token_of_row, static_cast<__nv_bfloat16*>(xp), T, K, H, E);
  return int(cudaGetLastError());
}
// buf [max_rows, H] bf16: zero the padding rows of every expert segment (counts != null) and the rows from *total on.
TFB_API int tfb_moe_zero_pads(void* buf, int H, const int* seg_start, const int* counts, int E, const int* total, int max_rows,
                              void* stream) {
  if (H % 8) return TFB_ERR_ARG;
  tfb::launch_k(moe_zero_pads_kernel, dim3(E + 1, 296), 256, 0, static_cast<cudaStream_t>(stream), static_cast<__nv_bfloat16*>(buf), H, seg_start,
                                                                                      counts, E, total, max_rows);
  return int(cudaGetLastError());
}
TFB_API int tfb_moe_combine(const void* yp, const int* row_of, const float* topk_w, void* y, const void* residual,
                            int T, int K, int H, void* stream) {
  if (H % 8) return TFB_ERR_ARG;
  tfb::launch_k(moe_combine_kernel, warps_to_blocks(T), 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(yp), row_of, topk_w, static_cast<__nv_bfloat16*>(y),
      static_cast<const __nv_bfloat16*>(residual), T, K, H);
  return int(cudaGetLastError());
}
TFB_API int tfb_moe_combine_bwd(const void* dy, const void* yp, const int* row_of, const float* topk_w, void* dyp,
                                float* dw, int T, int K, int H, void* stream) {
  if (H % 8) return TFB_ERR_ARG;
  tfb::launch_k(moe_combine_bwd_kernel, warps_to_blocks((long long)T * K), 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(yp), row_of, topk_w,
      static_cast<__nv_bfloat16*>(dyp), dw, T, K, H);
  return int(cudaGetLastError());
}
TFB_API int tfb_moe_permute_bwd(const void* dxp, const int* row_of, void* dx, int T, int K, int H, void* stream) {
  if (H % 8) return TFB_ERR_ARG;
  tfb::launch_k(moe_permute_bwd_kernel, warps_to_blocks(T), 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(dxp), row_of, static_cast<__nv_bfloat16*>(dx), T, K, H);
  return int(cudaGetLastError());
}
