// Multi-tensor Adafactor over flat fp32 state: every matrix of the model in five launches per step, whatever the number
// of tensors (a device table describes them).  Second moments are factored for matrices (row vector r, column vector c);
// a vector [n] is handled as a 1 x n matrix, for which the factored estimate r_0 c_j / mean(r) reduces to the plain
// running average c_j.
//
//   1 rows     warp per row:   r_i <- b2 r_i + (1 - b2) (mean_j g_ij^2 + eps1)
//   2 cols     thread per column over 64-row chunks: column sums of g^2 accumulated into a scratch vector
//   3 finish   CTA per tensor: c_j <- b2 c_j + (1 - b2) (colsum_j / d0 + eps1), scratch cleared, rmean = mean_i r_i
//   4 usq      warp per row:   sum of u^2 with u = g / sqrt(r_i c_j / rmean)            (for the update clipping)
//   5 apply    warp per row:   u <- u / max(1, rms(u) / clip), optional momentum, decoupled weight decay, p -= lr u,
//                              bf16 copy of p refreshed, gradient cleared
// The gradient is read four times and the parameters once: ~22 bytes per element per step.
//
// Reference counterpart: Adafactor::step (src/trainer/optimizer.cpp:338-416): factored row / column statistics, clipped
// update, momentum on the update, decoupled decay.
#include "tfb_host.h"
#include "tfb_ptx.cuh"

namespace tfb {

struct AfTensor {
  long long off;      // first element in the flat gradient / master / low-precision buffers
  long long r_off;    // first element of r in the flat row-statistics buffer
  long long c_off;    // first element of c (and of the column scratch) in the flat column-statistics buffers
  int d0, d1;
  int row0;           // index of the tensor's first row among all rows of all tensors
  float wd_scale;     // 1 for matrices, 0 for vectors (no decay on norms and biases)
};

struct AfArgs {
  const AfTensor* t;
  int nt, total_rows;
  const float* g_ro;
  float* g;
  float* p;
  __nv_bfloat16* p_lp;
  float* m;           // momentum (null when beta1 == 0)
  float* r; float* c; float* csum;
  float* rmean; float* usq;      // [nt]
  const float* gscale;           // device scalar multiplied into every gradient (gradient-norm clip factor) or null
  float b2, eps1, clip, lr, wd, beta1;
};

__device__ __forceinline__ int af_find(const AfTensor* t, int nt, int row) {
  int lo = 0, hi = nt - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (t[mid].row0 <= row) lo = mid; else hi = mid - 1;
  }
  return lo;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(256) af_rows_kernel(AfArgs a) {
  tfb::pdl_sync();
  const int lane = threadIdx.x & 31;
  const int nwarp = (gridDim.x * blockDim.x) >> 5;
  const float gs = a.gscale ? *a.gscale : 1.f;
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < a.total_rows; row += nwarp) {
    const int ti = af_find(a.t, a.nt, row);
    const AfTensor t = a.t[ti];
    const int i = row - t.row0;
    const float* g = a.g_ro + t.off + (long long)i * t.d1;
    float s = 0.f;
    for (int j = lane; j < t.d1; j += 32) { const float x = g[j] * gs; s += x * x; }
    s = warp_sum(s);
    if (lane == 0) a.r[t.r_off + i] = a.b2 * a.r[t.r_off + i] + (1.f - a.b2) * (s / float(t.d1) + a.eps1);
  }
}

// grid.x = column blocks of 256 over the widest tensor, grid.y = 64-row chunks over all rows
__global__ void __launch_bounds__(256) af_cols_kernel(AfArgs a) {
  tfb::pdl_sync();
  const float gs = a.gscale ? *a.gscale : 1.f;
  for (int chunk = blockIdx.y; chunk * 64 < a.total_rows; chunk += gridDim.y) {
    int row = chunk * 64;
    const int row_end = min(a.total_rows, row + 64);
    while (row < row_end) {            // a chunk may straddle tensors
      const int ti = af_find(a.t, a.nt, row);
      const AfTensor t = a.t[ti];
      const int i0 = row - t.row0, i1 = min(t.d0, i0 + (row_end - row));
      for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < t.d1; j += gridDim.x * blockDim.x) {
        float s = 0.f;
        for (int i = i0; i < i1; ++i) { const float x = a.g_ro[t.off + (long long)i * t.d1 + j] * gs; s += x * x; }
        atomicAdd(a.csum + t.c_off + j, s);
      }
      row += i1 - i0;
    }
  }
}

__global__ void __launch_bounds__(256) af_finish_kernel(AfArgs a) {
  tfb::pdl_sync();
  __shared__ float sh[8];
  for (int ti = blockIdx.x; ti < a.nt; ti += gridDim.x) {
    const AfTensor t = a.t[ti];
    for (int j = threadIdx.x; j < t.d1; j += blockDim.x) {
      const float cs = a.csum[t.c_off + j];
      a.csum[t.c_off + j] = 0.f;
      a.c[t.c_off + j] = a.b2 * a.c[t.c_off + j] + (1.f - a.b2) * (cs / float(t.d0) + a.eps1);
    }
    float s = 0.f;
    for (int i = threadIdx.x; i < t.d0; i += blockDim.x) s += a.r[t.r_off + i];
    s = warp_sum(s);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
      float tot = 0.f;
      for (int w = 0; w < (blockDim.x >> 5); ++w) tot += sh[w];
      a.rmean[ti] = tot / float(t.d0);
      a.usq[ti] = 0.f;
    }
    __syncthreads();
  }
}

template <bool APPLY>
__global__ void __launch_bounds__(256) af_update_kernel(AfArgs a) {
  tfb::pdl_sync();
  const int lane = threadIdx.x & 31;
  const int nwarp = (gridDim.x * blockDim.x) >> 5;
  const float gs = a.gscale ? *a.gscale : 1.f;
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < a.total_rows; row += nwarp) {
    const int ti = af_find(a.t, a.nt, row);
    const AfTensor t = a.t[ti];
    const int i = row - t.row0;
    const long long base = t.off + (long long)i * t.d1;
    const float rm = a.rmean[ti];
    const float rfac = rm > 0.f ? a.r[t.r_off + i] / rm : 0.f;
    if (!APPLY) {
      float s = 0.f;
      for (int j = lane; j < t.d1; j += 32) {
        const float v = rfac * a.c[t.c_off + j];
        const float u = v > 0.f ? a.g_ro[base + j] * gs * rsqrtf(v) : 0.f;
        s += u * u;
      }
      s = warp_sum(s);
      if (lane == 0) atomicAdd(a.usq + ti, s);
    } else {
      const float n = float(t.d0) * float(t.d1);
      const float rms = sqrtf(a.usq[ti] / n);
      const float scale = 1.f / fmaxf(1.f, rms / a.clip);
      const float decay = 1.f - a.lr * a.wd * t.wd_scale;
      const bool usable = rm > 0.f && isfinite(rm) && isfinite(rms);   // no usable gradient: only the decay is applied
      for (int j = lane; j < t.d1; j += 32) {
        const float v = rfac * a.c[t.c_off + j];
        float u = (usable && v > 0.f) ? a.g[base + j] * gs * rsqrtf(v) * scale : 0.f;
        if (a.m) {
          const float mm = a.beta1 * a.m[base + j] + (1.f - a.beta1) * u;
          a.m[base + j] = mm;
          u = mm;
        }
        const float pn = a.p[base + j] * decay - a.lr * u;
        a.p[base + j] = pn;
        if (a.p_lp) a.p_lp[base + j] = __float2bfloat16(pn);
        a.g[base + j] = 0.f;
      }
    }
  }
}

}  // namespace tfb

// One Adafactor step over `nt` tensors described by the device table `tensors` (struct AfTensor; see the top of the
// file).  g / p / p_lp / m are the flat gradient, fp32 parameter, bf16 parameter (may be null) and momentum (null when
// beta1 == 0) buffers; r / c / csum the flat row / column statistics and a zeroed column scratch; rmean / usq float[nt].
// `gscale`: optional device scalar applied to every gradient.  max_d1: widest tensor (sizes the column pass).
TFB_API int tfb_adafactor(const void* tensors, int nt, int total_rows, int max_d1, float* g, float* p, void* p_lp, float* m, float* r,
                          float* c, float* csum, float* rmean, float* usq, const float* gscale, float b2, float eps1, float clip,
                          float lr, float wd, float beta1, void* stream) {
  using namespace tfb;
  if (nt < 1 || total_rows < 1 || max_d1 < 1) return TFB_ERR_ARG;
  AfArgs a{static_cast<const AfTensor*>(tensors), nt, total_rows, g, g, p, static_cast<__nv_bfloat16*>(p_lp), m, r, c, csum, rmean, usq,
           gscale, b2, eps1, clip, lr, wd, beta1};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int sms = sm_count();
  const int row_grid = min((total_rows + 7) / 8, sms * 8);
  tfb::launch_k(af_rows_kernel, row_grid, 256, 0, st, a);
  dim3 cg(min((max_d1 + 255) / 256, 64), min((total_rows + 63) / 64, sms * 4));
  tfb::launch_k(af_cols_kernel, cg, 256, 0, st, a);
  tfb::launch_k(af_finish_kernel, min(nt, sms), 256, 0, st, a);
  tfb::launch_k(af_update_kernel<false>, row_grid, 256, 0, st, a);
  tfb::launch_k(af_update_kernel<true>, row_grid, 256, 0, st, a);
  return int(cudaGetLastError());
}
