// Cross-entropy (forward + in-place logit gradient), global gradient norm / clip factor, and the
// fused multi-tensor optimizers over flat fp32 state (AdamW, Lion, SGD-momentum; Adafactor's
// factored second moment is the multi-tensor kernel set of adafactor.cu).
//
// Reference counterparts: cross-entropy forward/backward (src/model/autograd_functions.cpp:363,
// src/backend/gpu_compute_vulkan.cpp:1675-1721 vk_cross_entropy(+grad)); AdamW::step
// (src/trainer/optimizer.cpp:91-121: clip -> schedule -> bias-corrected update -> decoupled decay);
// reduce_sum_kernel (src/backend/gpu_compute_cuda.cpp:419); Trainer::clip_gradients
// (src/trainer/trainer_core.cpp:841).
#include "tfb_host.h"
#include "tfb_ptx.cuh"

TFB_BOUNDS_DEFINE(loss_optim)

namespace tfb {

__device__ __forceinline__ float block_reduce_sum(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  v = (lane < nw) ? sh[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float block_reduce_max(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  v = (lane < nw) ? sh[lane] : -INFINITY;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Register-resident variant for rows of at most 512 * 8 * NV elements (vocabularies up to 32768 with NV = 8): every
// thread keeps its NV 16-byte vectors in registers, so the row is read from memory exactly once and the gradient is
// written exactly once.  Same contract as cross_entropy_kernel below.
template <int NV>
__global__ void __launch_bounds__(512, 2) cross_entropy_regs_kernel(const __nv_bfloat16* logits, const long long* __restrict__ labels,
                                                                 float* __restrict__ loss, float* __restrict__ lse_out,
                                                                 __nv_bfloat16* dlogits, const float* __restrict__ scale_ptr, int V,
                                                                 long long ld, long long ignore_index, float eps, float zw) {
  tfb::pdl_sync();
  __shared__ float sh[32];
  const long long t = blockIdx.x;
  const uint4* row = reinterpret_cast<const uint4*>(logits + t * ld);
  const long long label = labels[t];
  const bool ignored = (label == ignore_index);
  if (threadIdx.x == 0) TFB_BOUNDS(ignored || (label >= 0 && label < V), 3, label, V);
  const int V8 = V >> 3;
  uint4 u[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = threadIdx.x + j * 512;
    if (i < V8) u[j] = row[i];
  }
  float mx = -INFINITY, tot = 0.f, zy = 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = threadIdx.x + j * 512;
    if (i < V8) {
      const uint32_t* p = reinterpret_cast<const uint32_t*>(&u[j]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = unpack_bf16(p[k]);
        mx = fmaxf(mx, fmaxf(f.x, f.y));
        tot += f.x + f.y;
        const int c = i * 8 + k * 2;
        if (c == label) zy = f.x;
        if (c + 1 == label) zy = f.y;
      }
    }
  }
  const float gmx = block_reduce_max(mx, sh);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = threadIdx.x + j * 512;
    if (i < V8) {
      const uint32_t* p = reinterpret_cast<const uint32_t*>(&u[j]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = unpack_bf16(p[k]);
        sum += __expf(f.x - gmx) + __expf(f.y - gmx);
      }
    }
  }
  const float gsum = block_reduce_sum(sum, sh);
  const float gtot = block_reduce_sum(tot, sh);
  const float gzy = block_reduce_sum(zy, sh);     // exactly one thread holds the label's logit
  const float lse = gmx + logf(gsum);
  if (threadIdx.x == 0) {
    loss[t] = ignored ? 0.f : (1.f - eps) * (lse - gzy) + eps * (lse - gtot / V) + zw * lse * lse;
    if (lse_out) lse_out[t] = lse;
  }
  if (!dlogits) return;
  uint4* drow = reinterpret_cast<uint4*>(dlogits + t * ld);
  const float scale = ignored ? 0.f : (scale_ptr ? *scale_ptr : 1.f);
  const float pm = scale * (1.f + 2.f * zw * lse);
  const float sm = scale * eps / V;
  const float hot = scale * (1.f - eps);
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = threadIdx.x + j * 512;
    if (i < V8) {
      uint32_t* p = reinterpret_cast<uint32_t*>(&u[j]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = unpack_bf16(p[k]);
        const int c = i * 8 + k * 2;
        float g0 = pm * __expf(f.x - lse) - sm, g1 = pm * __expf(f.y - lse) - sm;
        if (c == label) g0 -= hot;
        if (c + 1 == label) g1 -= hot;
        p[k] = pack_bf16(g0, g1);
      }
      drow[i] = u[j];
    }
  }
}

// One CTA per token row.  loss[t] = (1-eps) * (lse - z_y) + eps * (lse - mean z) + zw * lse^2, 0 when the
// label equals ignore_index.  When `dlogits` is non-null it receives
// scale * (softmax * (1 + 2 zw lse) - (1-eps) onehot - eps / V); it may alias `logits`.
__global__ void __launch_bounds__(512) cross_entropy_kernel(const __nv_bfloat16* logits,
                                                            const long long* __restrict__ labels,
                                                            float* __restrict__ loss, float* __restrict__ lse_out,
                                                            __nv_bfloat16* dlogits, const float* __restrict__ scale_ptr,
                                                            int V, long long ld, long long ignore_index, float eps,
                                                            float zw, int vocab_start, int vocab_total) {
  tfb::pdl_sync();
  __shared__ float sh[32];
  const long long t = blockIdx.x;
  const __nv_bfloat16* row = logits + t * ld;
  const long long label = labels[t];
  const bool ignored = (label == ignore_index);
  if (threadIdx.x == 0) TFB_BOUNDS(ignored || (label >= 0 && label < V), 3, label, V);
  // read before any thread starts overwriting the row with gradients (dlogits may alias logits)
  const float zy = (!ignored && label >= 0 && label < V) ? __bfloat162float(row[label]) : 0.f;
  const bool vec = ((ld & 7) == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  const int V8 = vec ? (V >> 3) : 0;

  float mx = -INFINITY, sum = 0.f, tot = 0.f;
  auto upd = [&](float z) {
    tot += z;
    if (z > mx) {
      sum = sum * __expf(mx - z) + 1.f;
      mx = z;
    } else {
      sum += __expf(z - mx);
    }
  };
  for (int i = threadIdx.x; i < V8; i += blockDim.x) {
    const uint4 u = reinterpret_cast<const uint4*>(row)[i];
    const uint32_t* p = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_bf16(p[k]);
      upd(f.x);
      upd(f.y);
    }
  }
  for (int i = V8 * 8 + threadIdx.x; i < V; i += blockDim.x) upd(__bfloat162float(row[i]));
  const float gmx = block_reduce_max(mx, sh);
  const float gsum = block_reduce_sum(mx == -INFINITY ? 0.f : sum * __expf(mx - gmx), sh);
  const float gtot = block_reduce_sum(tot, sh);
  const float lse = gmx + logf(gsum);
  (void)vocab_start;
  (void)vocab_total;
  if (threadIdx.x == 0) {
    float l = 0.f;
    if (!ignored) {
      l = (1.f - eps) * (lse - zy) + eps * (lse - gtot / V) + zw * lse * lse;
    }
    loss[t] = l;
    if (lse_out) lse_out[t] = lse;
  }
  if (!dlogits) return;
  __nv_bfloat16* drow = dlogits + t * ld;
  const float scale = ignored ? 0.f : (scale_ptr ? *scale_ptr : 1.f);
  const float pm = scale * (1.f + 2.f * zw * lse);
  const float sm = scale * eps / V;
  const float hot = scale * (1.f - eps);
  for (int i = threadIdx.x; i < V8; i += blockDim.x) {
    uint4 u = reinterpret_cast<const uint4*>(row)[i];
    uint32_t* p = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_bf16(p[k]);
      const int c = i * 8 + k * 2;
      float g0 = pm * __expf(f.x - lse) - sm, g1 = pm * __expf(f.y - lse) - sm;
      if (c == label) g0 -= hot;
      if (c + 1 == label) g1 -= hot;
      p[k] = pack_bf16(g0, g1);
    }
    reinterpret_cast<uint4*>(drow)[i] = u;
  }
  for (int i = V8 * 8 + threadIdx.x; i < V; i += blockDim.x) {
    float g = pm * __expf(__bfloat162float(row[i]) - lse) - sm;
    if (i == label) g -= hot;
    drow[i] = __float2bfloat16(g);
  }
}

// Three-pass form for large vocabularies with in-place gradients (row in 16-byte vectors):
//   1  max of the row                                   (reads logits from HBM)
//   2  p = 2^((z - max) * log2 e), sum p, store p over the row   (reads L2, one exponential per element)
//   3  g = p * (pm / sum) - sm, label fix, store g               (reads L2, no exponential)
// One exponential per element instead of the two of the online form, and about half its instructions; the row a CTA
// works on (64 KB at 32k vocabulary) stays in L2 between passes, so HBM sees one read and one write.  p is rounded to
// bf16 before the final scaling, which adds one bf16 rounding to a gradient that is stored in bf16 anyway.
__global__ void __launch_bounds__(512) cross_entropy_3pass_kernel(const __nv_bfloat16* logits, const long long* __restrict__ labels,
                                                                  float* __restrict__ loss, float* __restrict__ lse_out,
                                                                  __nv_bfloat16* dlogits, const float* __restrict__ scale_ptr, int V,
                                                                  long long ld, long long ignore_index, float eps, float zw) {
  tfb::pdl_sync();
  __shared__ float sh[32];
  constexpr float L2E = 1.4426950408889634f;
  const long long t = blockIdx.x;
  const uint4* row = reinterpret_cast<const uint4*>(logits + t * ld);
  uint4* drow = reinterpret_cast<uint4*>(dlogits + t * ld);
  const long long label = labels[t];
  const bool ignored = (label == ignore_index);
  if (threadIdx.x == 0) TFB_BOUNDS(ignored || (label >= 0 && label < V), 3, label, V);
  const bool has_label = !ignored && label >= 0 && label < V;
  const float zy = has_label ? __bfloat162float(logits[t * ld + label]) : 0.f;   // read before the row is overwritten
  const int V8 = V >> 3;
  float mx = -INFINITY, tot = 0.f;
  for (int i = threadIdx.x; i < V8; i += 512) {
    const uint4 u = row[i];
    const uint32_t* p = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_bf16(p[k]);
      mx = fmaxf(mx, fmaxf(f.x, f.y));
      if (eps != 0.f) tot += f.x + f.y;
    }
  }
  const float gmx = block_reduce_max(mx, sh);
  const float gtot = eps != 0.f ? block_reduce_sum(tot, sh) : 0.f;
  const float off = -gmx * L2E;
  float sum = 0.f;
  for (int i = threadIdx.x; i < V8; i += 512) {
    uint4 u = row[i];
    uint32_t* p = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_bf16(p[k]);
      const float e0 = exp2f(fmaf(f.x, L2E, off)), e1 = exp2f(fmaf(f.y, L2E, off));
      sum += e0 + e1;
      p[k] = pack_bf16(e0, e1);
    }
    drow[i] = u;
  }
  const float gsum = block_reduce_sum(sum, sh);           // also orders pass 2's stores before pass 3's loads (bar.sync)
  const float lse = gmx + logf(gsum);
  if (threadIdx.x == 0) {
    loss[t] = ignored ? 0.f : (1.f - eps) * (lse - zy) + eps * (lse - gtot / V) + zw * lse * lse;
    if (lse_out) lse_out[t] = lse;
  }
  const float scale = ignored ? 0.f : (scale_ptr ? *scale_ptr : 1.f);
  const float pm = scale * (1.f + 2.f * zw * lse) / gsum;
  const float sm = scale * eps / V;
  const float hot = scale * (1.f - eps);
  const int lab_vec = has_label ? int(label >> 3) : -1, lab_k = int(label & 7);
  for (int i = threadIdx.x; i < V8; i += 512) {            // thread i revisits exactly the vectors it wrote in pass 2
    uint4 u = drow[i];
    uint32_t* p = reinterpret_cast<uint32_t*>(&u);
    float g[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_bf16(p[k]);
      g[2 * k] = fmaf(f.x, pm, -sm);
      g[2 * k + 1] = fmaf(f.y, pm, -sm);
    }
    if (i == lab_vec) {
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (k == lab_k) g[k] -= hot;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) p[k] = pack_bf16(g[2 * k], g[2 * k + 1]);
    drow[i] = u;
  }
}

// sum over n of x^2, accumulated into *out (fp32).  x is fp32.
__global__ void __launch_bounds__(512) sumsq_kernel(const float* __restrict__ x, long long n, float* __restrict__ out) {
  tfb::pdl_sync();
  __shared__ float sh[32];
  float acc = 0.f;
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  for (long long i = n4 * 4 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    acc += x[i] * x[i];
  acc = block_reduce_sum(acc, sh);
  if (threadIdx.x == 0) atomicAdd(out, acc);
}

// norm_out = sqrt(sumsq * inv_scale^2); clip_out = inv_scale * min(1, max_norm / (norm + 1e-6)).
// A non-finite norm yields clip 0 and sets *found_inf (dynamic loss scaling skips that step).
__global__ void clip_factor_kernel(const float* __restrict__ sumsq, float inv_scale, float max_norm,
                                   float* __restrict__ norm_out, float* __restrict__ clip_out, int* found_inf) {
  tfb::pdl_sync();
  const float nrm = sqrtf(*sumsq) * inv_scale;
  float c = inv_scale;
  if (!isfinite(nrm)) {
    c = 0.f;
    if (found_inf) *found_inf = 1;
  } else if (max_norm > 0.f && nrm > max_norm) {
    c *= max_norm / (nrm + 1e-6f);
  }
  *norm_out = nrm;
  *clip_out = c;
}

struct AdamArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2;
};

// p (fp32 master), m, v updated in place; p_lp (bf16 compute copy) refreshed; g optionally zeroed.
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m,
                                                    float* __restrict__ v, __nv_bfloat16* __restrict__ p_lp,
                                                    long long n, AdamArgs a, const float* __restrict__ gscale_ptr,
                                                    int zero_grad, const float* __restrict__ hyper) {
  tfb::pdl_sync();
  // hyper (optional, device): {lr, 1 - beta1^t, 1 - beta2^t}; lets a captured CUDA graph see per-step values
  if (hyper) { a.lr = hyper[0]; a.bc1 = hyper[1]; a.bc2 = hyper[2]; }
  const float gs = gscale_ptr ? *gscale_ptr : 1.f;
  if (gs == 0.f && gscale_ptr) {  // skipped step (overflow): only clear the gradients
    if (zero_grad)
      for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        g[i] = 0.f;
    return;
  }
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 pp = reinterpret_cast<float4*>(p)[i];
    float4 gg = reinterpret_cast<float4*>(g)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float* P = reinterpret_cast<float*>(&pp);
    float* G = reinterpret_cast<float*>(&gg);
    float* Mv = reinterpret_cast<float*>(&mm);
    float* Vv = reinterpret_cast<float*>(&vv);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gr = G[k] * gs;
      Mv[k] = a.beta1 * Mv[k] + (1.f - a.beta1) * gr;
      Vv[k] = a.beta2 * Vv[k] + (1.f - a.beta2) * gr * gr;
      const float mh = Mv[k] / a.bc1, vh = Vv[k] / a.bc2;
      P[k] = P[k] - a.lr * (mh / (sqrtf(vh) + a.eps) + a.wd * P[k]);
    }
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (zero_grad) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (p_lp) {
      uint2 o;
      o.x = pack_bf16(P[0], P[1]);
      o.y = pack_bf16(P[2], P[3]);
      reinterpret_cast<uint2*>(p_lp)[i] = o;
    }
  }
  for (long long i = n4 * 4 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float gr = g[i] * gs;
    const float mn = a.beta1 * m[i] + (1.f - a.beta1) * gr;
    const float vn = a.beta2 * v[i] + (1.f - a.beta2) * gr * gr;
    const float pn = p[i] - a.lr * ((mn / a.bc1) / (sqrtf(vn / a.bc2) + a.eps) + a.wd * p[i]);
    m[i] = mn; v[i] = vn; p[i] = pn;
    if (zero_grad) g[i] = 0.f;
    if (p_lp) p_lp[i] = __float2bfloat16(pn);
  }
}

// Lion: u = sign(b1 m + (1-b1) g); p -= lr (u + wd p); m = b2 m + (1-b2) g.   SGD: m = mu m + g; p -= lr (m + wd p).
__global__ void __launch_bounds__(256) lion_sgd_kernel(float* __restrict__ p, float* __restrict__ g,
                                                       float* __restrict__ m, __nv_bfloat16* __restrict__ p_lp,
                                                       long long n, float lr, float b1, float b2, float wd, int mode,
                                                       const float* __restrict__ gscale_ptr, int zero_grad) {
  tfb::pdl_sync();
  const float gs = gscale_ptr ? *gscale_ptr : 1.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float gr = g[i] * gs;
    float pn = p[i], mn = m ? m[i] : 0.f;
    if (mode == 0) {  // Lion
      const float u = b1 * mn + (1.f - b1) * gr;
      pn -= lr * ((u > 0.f ? 1.f : (u < 0.f ? -1.f : 0.f)) + wd * pn);
      mn = b2 * mn + (1.f - b2) * gr;
    } else {  // SGD with momentum b1
      mn = b1 * mn + gr;
      pn -= lr * (mn + wd * pn);
    }
    p[i] = pn;
    if (m) m[i] = mn;
    if (zero_grad) g[i] = 0.f;
    if (p_lp) p_lp[i] = __float2bfloat16(pn);
  }
}

// dst(bf16) = src(fp32) and dst(fp32) = src(bf16)
__global__ void cast_f32_bf16_kernel(const float* __restrict__ s, __nv_bfloat16* __restrict__ d, long long n) {
  tfb::pdl_sync();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    d[i] = __float2bfloat16(s[i]);
}
__global__ void cast_bf16_f32_kernel(const __nv_bfloat16* __restrict__ s, float* __restrict__ d, long long n) {
  tfb::pdl_sync();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    d[i] = __bfloat162float(s[i]);
}

static inline int grid_cap(long long work, int threads, int per_sm) {
  long long b = (work + threads - 1) / threads;
  const long long cap = (long long)sm_count() * per_sm;
  return int(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace tfb

using namespace tfb;

TFB_API int tfb_cross_entropy(const void* logits, const long long* labels, float* loss, float* lse, void* dlogits,
                              const float* scale_ptr, int T, int V, long long ld, long long ignore_index,
                              float label_smoothing, float z_weight, void* stream) {
  if (T <= 0 || V <= 0) return TFB_ERR_ARG;
  const bool vec = (V % 8 == 0) && (ld % 8 == 0) && (reinterpret_cast<uintptr_t>(logits) & 15) == 0 &&
                   (!dlogits || (reinterpret_cast<uintptr_t>(dlogits) & 15) == 0);
  // Small vocabularies fit in two vectors per thread at full occupancy; for larger ones the streaming kernel, which
  // keeps four CTAs per SM in flight, measured faster than holding the row in registers (fewer resident warps).
  if (vec && V <= 512 * 8 * 2) {
    tfb::launch_k(cross_entropy_regs_kernel<2>, T, 512, 0, static_cast<cudaStream_t>(stream), 
        static_cast<const __nv_bfloat16*>(logits), labels, loss, lse, static_cast<__nv_bfloat16*>(dlogits), scale_ptr, V, ld,
        ignore_index, label_smoothing, z_weight);
    return int(cudaGetLastError());
  }
  if (vec && dlogits == logits) {
    tfb::launch_k(cross_entropy_3pass_kernel, T, 512, 0, static_cast<cudaStream_t>(stream), 
        static_cast<const __nv_bfloat16*>(logits), labels, loss, lse, static_cast<__nv_bfloat16*>(dlogits), scale_ptr, V, ld,
        ignore_index, label_smoothing, z_weight);
    return int(cudaGetLastError());
  }
  tfb::launch_k(cross_entropy_kernel, T, 512, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(logits), labels, loss, lse, static_cast<__nv_bfloat16*>(dlogits), scale_ptr, V,
      ld, ignore_index, label_smoothing, z_weight, 0, V);
  return int(cudaGetLastError());
}

TFB_API int tfb_sumsq_f32(const float* x, long long n, float* out, void* stream) {
  tfb::launch_k(sumsq_kernel, grid_cap(n / 4 + 1, 512, 2), 512, 0, static_cast<cudaStream_t>(stream), x, n, out);
  return int(cudaGetLastError());
}

TFB_API int tfb_clip_factor(const float* sumsq, float inv_scale, float max_norm, float* norm_out, float* clip_out,
                            int* found_inf, void* stream) {
  tfb::launch_k(clip_factor_kernel, 1, 1, 0, static_cast<cudaStream_t>(stream), sumsq, inv_scale, max_norm, norm_out, clip_out,
                                                                    found_inf);
  return int(cudaGetLastError());
}

TFB_API int tfb_adamw(float* p, float* g, float* m, float* v, void* p_lp, long long n, float lr, float beta1,
                      float beta2, float eps, float wd, int step, const float* gscale_ptr, int zero_grad,
                      const float* hyper, void* stream) {
  if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
       reinterpret_cast<uintptr_t>(v)) & 15)
    return TFB_ERR_ARG;
  if (p_lp && (reinterpret_cast<uintptr_t>(p_lp) & 7)) return TFB_ERR_ARG;
  AdamArgs a{lr, beta1, beta2, eps, wd, 1.f - powf(beta1, float(step)), 1.f - powf(beta2, float(step))};
  tfb::launch_k(adamw_kernel, grid_cap(n / 4 + 1, 256, 8), 256, 0, static_cast<cudaStream_t>(stream), 
      p, g, m, v, static_cast<__nv_bfloat16*>(p_lp), n, a, gscale_ptr, zero_grad, hyper);
  return int(cudaGetLastError());
}

TFB_API int tfb_lion_sgd(float* p, float* g, float* m, void* p_lp, long long n, float lr, float b1, float b2, float wd,
                         int mode, const float* gscale_ptr, int zero_grad, void* stream) {
  tfb::launch_k(lion_sgd_kernel, grid_cap(n, 256, 8), 256, 0, static_cast<cudaStream_t>(stream), 
      p, g, m, static_cast<__nv_bfloat16*>(p_lp), n, lr, b1, b2, wd, mode, gscale_ptr, zero_grad);
  return int(cudaGetLastError());
}

TFB_API int tfb_cast_f32_bf16(const float* s, void* d, long long n, void* stream) {
  tfb::launch_k(cast_f32_bf16_kernel, grid_cap(n, 256, 8), 256, 0, static_cast<cudaStream_t>(stream), 
      s, static_cast<__nv_bfloat16*>(d), n);
  return int(cudaGetLastError());
}
TFB_API int tfb_cast_bf16_f32(const void* s, float* d, long long n, void* stream) {
  tfb::launch_k(cast_bf16_f32_kernel, grid_cap(n, 256, 8), 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(s), d, n);
  return int(cudaGetLastError());
}
