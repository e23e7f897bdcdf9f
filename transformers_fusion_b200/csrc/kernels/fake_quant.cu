// Quantisation-aware-training kernels: block-wise fake quantisation (quantise -> dequantise in one pass,
// the straight-through estimator's forward), and LSQ (learned step size) forward / backward.
//
//   fake_quant_block: every `block` consecutive elements share one scale (symmetric: absmax / qmax) or a
//                     scale and zero point (asymmetric: (max - min) / (2^bits - 1)).  One warp per block,
//                     128-bit loads, values held in registers between the reduction and the rounding pass,
//                     so the tensor is read once and written once.
//   lsq_fwd / lsq_bwd: y = clamp(round(x / s), qn, qp) * s;  dx = dy inside the clamp range, 0 outside;
//                     ds = sum dy * (round(x/s) - x/s inside | qn | qp) * grad_scale.
//
// Reference counterparts: fake_quantize / lsq_fake_quantize (src/codec/qat.cpp), STE quantizer
// (src/codec/ste_quantizer.cpp).
#include "tfb_host.h"
#include "tfb_ptx.cuh"
#include <algorithm>

namespace tfb {

template <typename T> __device__ __forceinline__ float ld_f(const T* p);
template <> __device__ __forceinline__ float ld_f<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_f<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void st_f(T* p, float v);
template <> __device__ __forceinline__ void st_f<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void st_f<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

constexpr int FQ_MAX_PER_LANE = 32;   // block <= 1024 elements

template <typename T>
__global__ void fake_quant_block_kernel(const T* __restrict__ x, T* __restrict__ y, float* __restrict__ scale_out,
                                        long long n, int block, int bits, int symmetric) {
  tfb::pdl_sync();
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long nblocks = (n + block - 1) / block;
  const float qmax = float((1 << (bits - 1)) - 1), levels = float((1 << bits) - 1);
  for (long long b = warp; b < nblocks; b += nwarps) {
    const long long base = b * block;
    const int cnt = int(min((long long)block, n - base));
    float v[FQ_MAX_PER_LANE];
    float lo = INFINITY, hi = -INFINITY;
#pragma unroll
    for (int i = 0; i < FQ_MAX_PER_LANE; ++i) {
      const int e = i * 32 + lane;
      if (e < cnt) {
        v[i] = ld_f(x + base + e);
        lo = fminf(lo, v[i]);
        hi = fmaxf(hi, v[i]);
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
      hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    float s, zp = 0.f;
    if (symmetric) {
      const float amax = fmaxf(fabsf(lo), fabsf(hi));
      s = amax > 0.f ? amax / qmax : 1.f;
    } else {
      s = hi > lo ? (hi - lo) / levels : 1.f;
      zp = lo;
    }
    const float inv = 1.f / s;
#pragma unroll
    for (int i = 0; i < FQ_MAX_PER_LANE; ++i) {
      const int e = i * 32 + lane;
      if (e < cnt) {
        float q;
        if (symmetric) q = fminf(fmaxf(rintf(v[i] * inv), -qmax), qmax) * s;
        else q = fminf(fmaxf(rintf((v[i] - zp) * inv), 0.f), levels) * s + zp;
        st_f(y + base + e, q);
      }
    }
    if (scale_out && lane == 0) scale_out[b] = s;
  }
}

template <typename T>
__global__ void lsq_fwd_kernel(const T* __restrict__ x, const float* __restrict__ step, T* __restrict__ y, long long n,
                               float qn, float qp) {
  tfb::pdl_sync();
  const float s = fmaxf(*step, 1e-12f), inv = 1.f / s;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    st_f(y + i, fminf(fmaxf(rintf(ld_f(x + i) * inv), qn), qp) * s);
}

template <typename T>
__global__ void lsq_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy, const float* __restrict__ step,
                               T* __restrict__ dx, float* __restrict__ dstep, long long n, float qn, float qp,
                               float grad_scale) {
  tfb::pdl_sync();
  const float s = fmaxf(*step, 1e-12f), inv = 1.f / s;
  float acc = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float r = ld_f(x + i) * inv, g = ld_f(dy + i);
    float ds;
    if (r <= qn) { ds = qn; st_f(dx + i, 0.f); }
    else if (r >= qp) { ds = qp; st_f(dx + i, 0.f); }
    else { ds = rintf(r) - r; st_f(dx + i, g); }
    acc += g * ds;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ float part[32];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) atomicAdd(dstep, t * grad_scale);
  }
}

static int fq_grid(long long warps) { return int(std::min<long long>((warps * 32 + 255) / 256, (long long)sm_count() * 8)); }

}  // namespace tfb

using namespace tfb;

// dtype: 0 bf16, 1 fp32.  scale_out (optional) receives one scale per block.
TFB_API int tfb_fake_quant_block(const void* x, void* y, void* scale_out, long long n, int block, int bits, int symmetric,
                                 int dtype, void* stream) {
  if (n <= 0 || block <= 0 || block > 32 * FQ_MAX_PER_LANE || bits < 2 || bits > 16) return TFB_ERR_ARG;
  const long long nb = (n + block - 1) / block;
  auto st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    tfb::launch_k(fake_quant_block_kernel<__nv_bfloat16>, fq_grid(nb), 256, 0, st, static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y),
                                                                          static_cast<float*>(scale_out), n, block, bits, symmetric);
  else
    tfb::launch_k(fake_quant_block_kernel<float>, fq_grid(nb), 256, 0, st, static_cast<const float*>(x), static_cast<float*>(y),
                                                                static_cast<float*>(scale_out), n, block, bits, symmetric);
  return int(cudaGetLastError());
}

TFB_API int tfb_lsq_fwd(const void* x, const void* step, void* y, long long n, float qn, float qp, int dtype, void* stream) {
  if (n <= 0) return TFB_ERR_ARG;
  auto st = static_cast<cudaStream_t>(stream);
  const int grid = int(std::min<long long>((n + 255) / 256, (long long)sm_count() * 8));
  if (dtype == 0)
    tfb::launch_k(lsq_fwd_kernel<__nv_bfloat16>, grid, 256, 0, st, static_cast<const __nv_bfloat16*>(x), static_cast<const float*>(step),
                                                        static_cast<__nv_bfloat16*>(y), n, qn, qp);
  else
    tfb::launch_k(lsq_fwd_kernel<float>, grid, 256, 0, st, static_cast<const float*>(x), static_cast<const float*>(step), static_cast<float*>(y), n, qn, qp);
  return int(cudaGetLastError());
}

// dstep (one fp32) is accumulated into; the caller zeroes it.
TFB_API int tfb_lsq_bwd(const void* x, const void* dy, const void* step, void* dx, void* dstep, long long n, float qn, float qp,
                        float grad_scale, int dtype, void* stream) {
  if (n <= 0) return TFB_ERR_ARG;
  auto st = static_cast<cudaStream_t>(stream);
  const int grid = int(std::min<long long>((n + 255) / 256, (long long)sm_count() * 8));
  if (dtype == 0)
    tfb::launch_k(lsq_bwd_kernel<__nv_bfloat16>, grid, 256, 0, st, static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy),
                                                        static_cast<const float*>(step), static_cast<__nv_bfloat16*>(dx),
                                                        static_cast<float*>(dstep), n, qn, qp, grad_scale);
  else
    tfb::launch_k(lsq_bwd_kernel<float>, grid, 256, 0, st, static_cast<const float*>(x), static_cast<const float*>(dy), static_cast<const float*>(step),
                                                static_cast<float*>(dx), static_cast<float*>(dstep), n, qn, qp, grad_scale);
  return int(cudaGetLastError());
}
