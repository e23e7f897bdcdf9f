// RMSNorm / LayerNorm forward and backward, fused with the residual add.
//
// One warp per row, 128-bit loads, the row held in registers between the statistics pass and
// the scale pass (one read of the activations per kernel).  The backward accumulates the weight
// gradient in registers over all rows a warp visits and flushes it once with fp32 atomics into
// the fp32 gradient buffer.
//
// Replaces the reference's one-thread-per-row kernels (src/backend/gpu_compute_cuda.cpp:219
// rmsnorm_kernel, :617 layernorm_kernel) and its CPU fused residual+norm
// (src/backend/gpu_compute_vulkan.cpp:1749-1761 vk_rms_norm_add).
#include "tfb_host.h"
#include "tfb_ptx.cuh"

namespace tfb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack_bf16(w[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16(f[0], f[1]);
  u.y = pack_bf16(f[2], f[3]);
  u.z = pack_bf16(f[4], f[5]);
  u.w = pack_bf16(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// y = norm(x + res) * w (+ b);  h_out = x + res (optional);  stats: rstd (and mean for LayerNorm).
template <int NCHUNK, bool LAYERNORM>
__global__ void __launch_bounds__(256) norm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                       const __nv_bfloat16* __restrict__ res,
                                                       const __nv_bfloat16* __restrict__ w,
                                                       const __nv_bfloat16* __restrict__ b,
                                                       __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h_out,
                                                       float* __restrict__ rstd_out, float* __restrict__ mean_out,
                                                       int rows, int H, float eps) {
  tfb::pdl_sync();
  const int lane = threadIdx.x & 31;
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int row = warp_global; row < rows; row += nwarps) {
    const long long off = (long long)row * H;
    float v[NCHUNK][8];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < H) {
        load8(x + off + col, v[c]);
        if (res) {
          float r[8];
          load8(res + off + col, r);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[c][i] += r[i];
        }
        if (h_out) {
          store8(h_out + off + col, v[c]);
          // statistics are taken on the bf16-rounded residual stream so forward and backward agree
#pragma unroll
          for (int i = 0; i < 8; ++i) v[c][i] = __bfloat162float(__float2bfloat16(v[c][i]));
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          s += v[c][i];
          ss += v[c][i] * v[c][i];
        }
      }
    }
    s = warp_sum(s);
    ss = warp_sum(ss);
    float mean = 0.f, rstd;
    if (LAYERNORM) {
      mean = s / H;
      rstd = rsqrtf(fmaxf(ss / H - mean * mean, 0.f) + eps);
    } else {
      rstd = rsqrtf(ss / H + eps);
    }
    if (lane == 0) {
      if (rstd_out) rstd_out[row] = rstd;
      if (LAYERNORM && mean_out) mean_out[row] = mean;
    }
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < H) {
        float wv[8], o[8];
        load8(w + col, wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (v[c][i] - mean) * rstd * wv[i];
        if (LAYERNORM && b) {
          float bv[8];
          load8(b + col, bv);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += bv[i];
        }
        store8(y + off + col, o);
      }
    }
  }
}

// dx = rstd * (g - xhat * mean(g * xhat) [- mean(g)])  with g = dy * w, xhat = (h - mean) * rstd,
// plus the incoming residual-stream gradient `dres`.  With FUSE_DW the warp also accumulates
// dw += sum_rows dy * xhat (db += sum_rows dy) in registers and flushes once per block; for wide
// rows the weight gradient is a separate column reduction (norm_dw_kernel) to bound registers.
__device__ __forceinline__ void cvt8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack_bf16(w[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

template <int NCHUNK, bool LAYERNORM, bool FUSE_DW>
__global__ void __launch_bounds__(256) norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                       const __nv_bfloat16* __restrict__ h,
                                                       const __nv_bfloat16* __restrict__ w,
                                                       const float* __restrict__ rstd_in,
                                                       const float* __restrict__ mean_in,
                                                       const __nv_bfloat16* __restrict__ dres,
                                                       __nv_bfloat16* __restrict__ dx, float* __restrict__ dw,
                                                       float* __restrict__ db, int rows, int H) {
  tfb::pdl_sync();
  const int lane = threadIdx.x & 31;
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  constexpr int NACC = FUSE_DW ? NCHUNK : 1;
  float dw_acc[NACC][8], db_acc[NACC][8];
#pragma unroll
  for (int c = 0; c < NACC; ++c)
#pragma unroll
    for (int i = 0; i < 8; ++i) dw_acc[c][i] = 0.f, db_acc[c][i] = 0.f;

  for (int row = warp_global; row < rows; row += nwarps) {
    const long long off = (long long)row * H;
    const float rstd = rstd_in[row];
    const float mean = LAYERNORM ? mean_in[row] : 0.f;
    uint4 dyr[NCHUNK], hr[NCHUNK];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < H) {
        dyr[c] = *reinterpret_cast<const uint4*>(dy + off + col);
        hr[c] = *reinterpret_cast<const uint4*>(h + off + col);
        float d[8], xh[8], wv[8];
        cvt8(dyr[c], d);
        cvt8(hr[c], xh);
        load8(w + col, wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[i] = (xh[i] - mean) * rstd;
          if (FUSE_DW) {
            dw_acc[c % NACC][i] += d[i] * xh[i];
            if (LAYERNORM) db_acc[c % NACC][i] += d[i];
          }
          const float g = d[i] * wv[i];
          s1 += g * xh[i];
          s2 += g;
        }
      }
    }
    s1 = warp_sum(s1) / H;
    s2 = LAYERNORM ? warp_sum(s2) / H : 0.f;
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < H) {
        float d[8], xh[8], wv[8], o[8];
        cvt8(dyr[c], d);
        cvt8(hr[c], xh);
        load8(w + col, wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xn = (xh[i] - mean) * rstd;
          o[i] = rstd * (d[i] * wv[i] - xn * s1 - s2);
        }
        if (dres) {
          float r[8];
          load8(dres + off + col, r);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += r[i];
        }
        store8(dx + off + col, o);
      }
    }
  }
  if (FUSE_DW) {
    // block-level reduction of the weight gradient through shared memory, then one atomic per column
    extern __shared__ float red[];  // [H]
    for (int pass = 0; pass < (LAYERNORM && db ? 2 : 1); ++pass) {
      for (int i = threadIdx.x; i < H; i += blockDim.x) red[i] = 0.f;
      __syncthreads();
#pragma unroll
      for (int c = 0; c < NACC; ++c) {
        const int col = (c * 32 + lane) * 8;
        if (col < H) {
#pragma unroll
          for (int i = 0; i < 8; ++i) atomicAdd(&red[col + i], pass == 0 ? dw_acc[c][i] : db_acc[c][i]);
        }
      }
      __syncthreads();
      float* dst = pass == 0 ? dw : db;
      for (int i = threadIdx.x; i < H; i += blockDim.x) atomicAdd(dst + i, red[i]);
      __syncthreads();
    }
  }
}

// Column reduction for wide rows: block (x) owns 256 columns, blocks along y split the rows.
template <bool LAYERNORM>
__global__ void __launch_bounds__(256) norm_dw_kernel(const __nv_bfloat16* __restrict__ dy,
                                                      const __nv_bfloat16* __restrict__ h,
                                                      const float* __restrict__ rstd_in,
                                                      const float* __restrict__ mean_in, float* __restrict__ dw,
                                                      float* __restrict__ db, int rows, int H) {
  tfb::pdl_sync();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = (blockIdx.x * 32 + lane) * 8;
  float aw[8] = {0, 0, 0, 0, 0, 0, 0, 0}, ab[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col < H) {
    for (int row = blockIdx.y * 8 + warp; row < rows; row += gridDim.y * 8) {
      float d[8], xh[8];
      load8(dy + (long long)row * H + col, d);
      load8(h + (long long)row * H + col, xh);
      const float rstd = rstd_in[row], mean = LAYERNORM ? mean_in[row] : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        aw[i] += d[i] * (xh[i] - mean) * rstd;
        if (LAYERNORM) ab[i] += d[i];
      }
    }
  }
  __shared__ float red[2][256];
  for (int i = threadIdx.x; i < 512; i += 256) (&red[0][0])[i] = 0.f;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    atomicAdd(&red[0][lane * 8 + i], aw[i]);
    if (LAYERNORM) atomicAdd(&red[1][lane * 8 + i], ab[i]);
  }
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < H) {
    atomicAdd(dw + c, red[0][threadIdx.x]);
    if (LAYERNORM && db) atomicAdd(db + c, red[1][threadIdx.x]);
  }
}

// Few rows (decode batches): one CTA per row, so that a 4096-wide row is two 16-byte loads per thread instead of sixteen
// dependent round trips in one warp; the warp-per-row kernel above relies on many resident rows to hide that latency.
template <int NCH, bool LAYERNORM>
__global__ void __launch_bounds__(256) norm_fwd_rowblock_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                                                const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                                                                __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h_out,
                                                                float* __restrict__ rstd_out, float* __restrict__ mean_out, int rows, int H,
                                                                float eps) {
  tfb::pdl_sync();
  __shared__ float red[2][8];
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long off = (long long)row * H;
  float v[NCH][8], wv[NCH][8];
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (c * 256 + threadIdx.x) * 8;
    if (col < H) {
      load8(x + off + col, v[c]);
      load8(w + col, wv[c]);
    }
  }
  if (res) {
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = (c * 256 + threadIdx.x) * 8;
      if (col < H) {
        float r[8];
        load8(res + off + col, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[c][i] += r[i];
      }
    }
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (c * 256 + threadIdx.x) * 8;
    if (col < H) {
      if (h_out) {
        store8(h_out + off + col, v[c]);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[c][i] = __bfloat162float(__float2bfloat16(v[c][i]));
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        s += v[c][i];
        ss += v[c][i] * v[c][i];
      }
    }
  }
  s = warp_sum(s);
  ss = warp_sum(ss);
  if (lane == 0) {
    red[0][warp] = s;
    red[1][warp] = ss;
  }
  __syncthreads();
  s = ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    s += red[0][i];
    ss += red[1][i];
  }
  float mean = 0.f, rstd;
  if (LAYERNORM) {
    mean = s / H;
    rstd = rsqrtf(fmaxf(ss / H - mean * mean, 0.f) + eps);
  } else {
    rstd = rsqrtf(ss / H + eps);
  }
  if (threadIdx.x == 0) {
    if (rstd_out) rstd_out[row] = rstd;
    if (LAYERNORM && mean_out) mean_out[row] = mean;
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = (c * 256 + threadIdx.x) * 8;
    if (col < H) {
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = (v[c][i] - mean) * rstd * wv[c][i];
      if (LAYERNORM && b) {
        float bv[8];
        load8(b + col, bv);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] += bv[i];
      }
      store8(y + off + col, o);
    }
  }
}

template <bool LN>
static int launch_fwd(const void* x, const void* res, const void* w, const void* b, void* y, void* h_out, float* rstd,
                      float* mean, int rows, int H, float eps, cudaStream_t st) {
  if (H % 8 || H > 8192) return TFB_ERR_ARG;
  const int blocks = min((rows + 7) / 8, sm_count() * 8);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto R = static_cast<const __nv_bfloat16*>(res);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto B = static_cast<const __nv_bfloat16*>(b);
  auto Y = static_cast<__nv_bfloat16*>(y);
  auto Ho = static_cast<__nv_bfloat16*>(h_out);
  if (H >= 2048 && rows <= 4 * sm_count()) {
    if (H <= 4096) tfb::launch_k(norm_fwd_rowblock_kernel<2, LN>, rows, 256, 0, st, X, R, W, B, Y, Ho, rstd, mean, rows, H, eps);
    else tfb::launch_k(norm_fwd_rowblock_kernel<4, LN>, rows, 256, 0, st, X, R, W, B, Y, Ho, rstd, mean, rows, H, eps);
    return int(cudaGetLastError());
  }
#define TFB_GO(NC) tfb::launch_k(norm_fwd_kernel<NC, LN>, blocks, 256, 0, st, X, R, W, B, Y, Ho, rstd, mean, rows, H, eps)
  if (H <= 512) TFB_GO(2);
  else if (H <= 1024) TFB_GO(4);
  else if (H <= 2048) TFB_GO(8);
  else if (H <= 4096) TFB_GO(16);
  else TFB_GO(32);
#undef TFB_GO
  return int(cudaGetLastError());
}

template <bool LN>
static int launch_bwd(const void* dy, const void* h, const void* w, const float* rstd, const float* mean,
                      const void* dres, void* dx, float* dw, float* db, int rows, int H, cudaStream_t st) {
  if (H % 8 || H > 8192) return TFB_ERR_ARG;
  auto DY = static_cast<const __nv_bfloat16*>(dy);
  auto Hh = static_cast<const __nv_bfloat16*>(h);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto DR = static_cast<const __nv_bfloat16*>(dres);
  auto DX = static_cast<__nv_bfloat16*>(dx);
  const size_t sm = size_t(H) * 4;
  if (H <= 1024) {
    // 64 registers per thread: four resident blocks per SM; fewer leaves the loads of a row unhidden (94 -> 70 us at
    // 65536 x 512), more only adds atomics on dw
    const int blocks = min((rows + 7) / 8, sm_count() * 4);
    if (H <= 512) tfb::launch_k(norm_bwd_kernel<2, LN, true>, blocks, 256, sm, st, DY, Hh, W, rstd, mean, DR, DX, dw, db, rows, H);
    else tfb::launch_k(norm_bwd_kernel<4, LN, true>, blocks, 256, sm, st, DY, Hh, W, rstd, mean, DR, DX, dw, db, rows, H);
  } else {
    const int blocks = min((rows + 7) / 8, sm_count() * 8);
    if (H <= 2048) tfb::launch_k(norm_bwd_kernel<8, LN, false>, blocks, 256, 0, st, DY, Hh, W, rstd, mean, DR, DX, dw, db, rows, H);
    else if (H <= 4096) tfb::launch_k(norm_bwd_kernel<16, LN, false>, blocks, 256, 0, st, DY, Hh, W, rstd, mean, DR, DX, dw, db, rows, H);
    else tfb::launch_k(norm_bwd_kernel<32, LN, false>, blocks, 256, 0, st, DY, Hh, W, rstd, mean, DR, DX, dw, db, rows, H);
    dim3 g((H + 255) / 256, min(64, (rows + 7) / 8));
    tfb::launch_k(norm_dw_kernel<LN>, g, 256, 0, st, DY, Hh, rstd, mean, dw, db, rows, H);
  }
  return int(cudaGetLastError());
}

}  // namespace tfb

// y = rmsnorm(x + res) * w; h_out (optional) receives x + res; rstd [rows] fp32 is saved for backward.
TFB_API int tfb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd, int rows,
                            int H, float eps, void* stream) {
  return tfb::launch_fwd<false>(x, res, w, nullptr, y, h_out, rstd, nullptr, rows, H, eps,
                                static_cast<cudaStream_t>(stream));
}
// dx = d rmsnorm / d h (+ dres); dw (fp32) accumulates.
TFB_API int tfb_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd, const void* dres, void* dx,
                            float* dw, int rows, int H, void* stream) {
  return tfb::launch_bwd<false>(dy, h, w, rstd, nullptr, dres, dx, dw, nullptr, rows, H,
                                static_cast<cudaStream_t>(stream));
}
TFB_API int tfb_layernorm_fwd(const void* x, const void* res, const void* w, const void* b, void* y, void* h_out,
                              float* rstd, float* mean, int rows, int H, float eps, void* stream) {
  return tfb::launch_fwd<true>(x, res, w, b, y, h_out, rstd, mean, rows, H, eps, static_cast<cudaStream_t>(stream));
}
TFB_API int tfb_layernorm_bwd(const void* dy, const void* h, const void* w, const float* rstd, const float* mean,
                              const void* dres, void* dx, float* dw, float* db, int rows, int H, void* stream) {
  return tfb::launch_bwd<true>(dy, h, w, rstd, mean, dres, dx, dw, db, rows, H, static_cast<cudaStream_t>(stream));
}
