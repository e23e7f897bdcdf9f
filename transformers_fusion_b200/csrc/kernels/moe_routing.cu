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
#include "tfb_host.h"
#include "tfb_ptx.cuh"

namespace tfb {

constexpr int MAX_E = 256;
constexpr int MAX_K = 8;

// one warp per token
__global__ void router_topk_kernel(const __nv_bfloat16* __restrict__ logits_bf16, const float* __restrict__ logits_f32,
                                   int T, int E, int K, int renorm, int* __restrict__ topk_idx,
                                   float* __restrict__ topk_w, float* __restrict__ probs_out,
                                   int* __restrict__ counts, float* __restrict__ prob_sums, float* __restrict__ lse_out) {
  const int lane = threadIdx.x & 31;
  const long long t = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (t >= T) return;
  constexpr int PER = MAX_E / 32;
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
  if (lane == 0 && lse_out) lse_out[t] = mx + logf(sum);
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    v[i] *= inv;
    const int e = lane + i * 32;
    if (e < E) {
      if (probs_out) probs_out[t * E + e] = v[i];
      if (prob_sums) atomicAdd(prob_sums + e, v[i]);
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
      if (counts) atomicAdd(counts + sel_i[k], 1);
    }
  }
}

// single block: seg_start[e] (padded to 128), expert_of_tile, total padded rows; cursor[e] = seg_start[e]
__global__ void moe_plan_kernel(const int* __restrict__ counts, int E, int* __restrict__ seg_start,
                                int* __restrict__ cursor, int* __restrict__ expert_of_tile, int max_tiles,
                                int* __restrict__ total_rows) {
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

// one warp per (token, k): claims a row in its expert's segment, copies the token row there
__global__ void moe_permute_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ topk_idx,
                                   int* __restrict__ cursor, int* __restrict__ row_of, int* __restrict__ token_of_row,
                                   __nv_bfloat16* __restrict__ xp, int T, int K, int H) {
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (w >= (long long)T * K) return;
  const int t = int(w / K);
  int row = 0;
  if (lane == 0) {
    row = atomicAdd(cursor + topk_idx[w], 1);
    row_of[w] = row;
    token_of_row[row] = t;
  }
  row = __shfl_sync(0xffffffffu, row, 0);
  const uint4* src = reinterpret_cast<const uint4*>(x + (long long)t * H);
  uint4* dst = reinterpret_cast<uint4*>(xp + (long long)row * H);
  for (int i = lane; i < H / 8; i += 32) dst[i] = src[i];
}

// y[t] = sum_k w[t,k] * yp[row_of[t,k]]; one warp per token
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ yp, const int* __restrict__ row_of,
                                   const float* __restrict__ topk_w, __nv_bfloat16* __restrict__ y,
                                   const __nv_bfloat16* __restrict__ residual, int T, int K, int H) {
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

TFB_API int tfb_router_topk(const void* logits, int logits_f32, int T, int E, int K, int renorm, int* topk_idx,
                            float* topk_w, float* probs, int* counts, float* prob_sums, float* lse, void* stream) {
  if (E > MAX_E || K > MAX_K || K < 1 || K > E) return TFB_ERR_LIMIT;
  router_topk_kernel<<<warps_to_blocks(T), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      logits_f32 ? nullptr : static_cast<const __nv_bfloat16*>(logits),
      logits_f32 ? static_cast<const float*>(logits) : nullptr, T, E, K, renorm, topk_idx, topk_w, probs, counts,
      prob_sums, lse);
  return int(cudaGetLastError());
}
TFB_API int tfb_moe_plan(const int* counts, int E, int* seg_start, int* cursor, int* expert_of_tile, int max_tiles,
                         int* total_rows, void* stream) {
  moe_plan_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(counts, E, seg_start, cursor, expert_of_tile,
                                                                  max_tiles, total_rows);
  return int(cudaGetLastError());
}
TFB_API int tfb_moe_permute(const void* x, const int* topk_idx, int* cursor, int* row_of, int* token_of_row, void* xp,
                            int T, int K, int H, void* stream) {
  if (H % 8) return TFB_ERR_ARG;
  moe_permute_kernel<<<warps_to_blocks((long long)T * K), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), topk_idx, cursor, row_of, token_of_row, static_cast<__nv_bfloat16*>(xp), T,
      K, H);
  return int(cudaGetLastError());
}
TFB_API int tfb_moe_combine(const void* yp, const int* row_of, const float* topk_w, void* y, const void* residual,
                            int T, int K, int H, void* stream) {
  if (H % 8) return TFB_ERR_ARG;
  moe_combine_kernel<<<warps_to_blocks(T), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(yp), row_of, topk_w, static_cast<__nv_bfloat16*>(y),
      static_cast<const __nv_bfloat16*>(residual), T, K, H);
  return int(cudaGetLastError());
}
TFB_API int tfb_moe_combine_bwd(const void* dy, const void* yp, const int* row_of, const float* topk_w, void* dyp,
                                float* dw, int T, int K, int H, void* stream) {
  if (H % 8) return TFB_ERR_ARG;
  moe_combine_bwd_kernel<<<warps_to_blocks((long long)T * K), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(yp), row_of, topk_w,
      static_cast<__nv_bfloat16*>(dyp), dw, T, K, H);
  return int(cudaGetLastError());
}
TFB_API int tfb_moe_permute_bwd(const void* dxp, const int* row_of, void* dx, int T, int K, int H, void* stream) {
  if (H % 8) return TFB_ERR_ARG;
  moe_permute_bwd_kernel<<<warps_to_blocks(T), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dxp), row_of, static_cast<__nv_bfloat16*>(dx), T, K, H);
  return int(cudaGetLastError());
}
