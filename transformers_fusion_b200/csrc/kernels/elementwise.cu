// Memory-bound fused ops: rotary embedding, gated activations (SwiGLU / GeGLU) and plain
// activations with their backward, embedding gather / scatter-add, bf16<->fp32 casts and adds.
// All use 128-bit accesses; each kernel makes exactly one pass over its operands.
//
// Reference counterparts: rope_kernel / silu_kernel / gelu_kernel / relu_kernel / add_kernel /
// mul_kernel / scale_kernel (src/backend/gpu_compute_cuda.cpp:112-296), rotate-half RoPE
// (src/model/transformer.cpp:213-270), SwiGLU / GeGLU FFN (src/model/transformer.cpp:534-595),
// embedding forward/backward (src/model/autograd_functions.cpp:489).
#include "tfb_host.h"
#include "tfb_ptx.cuh"

TFB_BOUNDS_DEFINE(elementwise)

namespace tfb {

// ------------------------------------------------------------------------------------------------
// RoPE (rotate-half) applied in place to the q and k heads of a fused [T, (Hq + 2*Hkv) * D] buffer
// (or any buffer with `n_heads` rotary heads of width D at the start of each row of pitch `ld`).
// cos/sin tables are [max_pos, D/2] fp32, which is where Linear / NTK / YARN scaling lives.
// sign = +1 forward, -1 backward (the transpose of a rotation is the inverse rotation).
// ------------------------------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, const int* __restrict__ positions, int T, int S,
                            int pos_offset, int n_heads, int D, long long ld, float sign) {
  tfb::pdl_sync();
  const int half = D >> 1;
  const int vec_per_head = half >> 3;  // 8 pairs per thread
  const long long total = (long long)T * n_heads * vec_per_head;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int v = int(i % vec_per_head);
    const long long th = i / vec_per_head;
    const int hd = int(th % n_heads);
    const int t = int(th / n_heads);
    const int pos = positions ? positions[t] : (t % S) + pos_offset;
    __nv_bfloat16* p = x + (long long)t * ld + (long long)hd * D + v * 8;
    const float* c = cos_t + (long long)pos * half + v * 8;
    const float* s = sin_t + (long long)pos * half + v * 8;
    uint4 u1 = *reinterpret_cast<uint4*>(p);
    uint4 u2 = *reinterpret_cast<uint4*>(p + half);
    uint32_t* a = reinterpret_cast<uint32_t*>(&u1);
    uint32_t* b = reinterpret_cast<uint32_t*>(&u2);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 x1 = unpack_bf16(a[k]), x2 = unpack_bf16(b[k]);
      const float c0 = c[2 * k], c1 = c[2 * k + 1];
      const float s0 = sign * s[2 * k], s1 = sign * s[2 * k + 1];
      a[k] = pack_bf16(x1.x * c0 - x2.x * s0, x1.y * c1 - x2.y * s1);
      b[k] = pack_bf16(x2.x * c0 + x1.x * s0, x2.y * c1 + x1.y * s1);
    }
    *reinterpret_cast<uint4*>(p) = u1;
    *reinterpret_cast<uint4*>(p + half) = u2;
  }
}

// ------------------------------------------------------------------------------------------------
// Gated activation: in [M, 2F] = [gate | up]  ->  out [M, F] = act(gate) * up.   act: 3 silu, 2 gelu
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float act_fwd(float g, int act) {
  switch (act) {
    case 1: return fmaxf(g, 0.f);
    case 2: return gelu_tanh(g);
    case 3: return silu(g);
    default: return g;
  }
}
__device__ __forceinline__ float act_grad(float g, int act) {
  switch (act) {
    case 1: return g > 0.f ? 1.f : 0.f;
    case 2: {
      const float k = 0.7978845608028654f;
      const float u = k * (g + 0.044715f * g * g * g);
      const float t = tanhf(u);
      return 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * k * (1.f + 3.f * 0.044715f * g * g);
    }
    case 3: {
      const float s = 1.f / (1.f + __expf(-g));
      return s * (1.f + g * (1.f - s));
    }
    default: return 1.f;
  }
}

// `rows_dev` (optional): a device-side row count below M, e.g. the routed rows of an expert buffer provisioned for more.
__global__ void glu_fwd_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, long long M,
                               int F, int act, const int* __restrict__ rows_dev) {
  tfb::pdl_sync();
  const int vec = F >> 3;
  if (rows_dev) M = min(M, (long long)max(*rows_dev, 0));
  const long long total = M * vec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec;
    const int c = int(i % vec) * 8;
    const uint4 ug = *reinterpret_cast<const uint4*>(in + r * 2 * F + c);
    const uint4 uu = *reinterpret_cast<const uint4*>(in + r * 2 * F + F + c);
    const uint32_t* g = reinterpret_cast<const uint32_t*>(&ug);
    const uint32_t* u = reinterpret_cast<const uint32_t*>(&uu);
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 gv = unpack_bf16(g[k]), uv = unpack_bf16(u[k]);
      op[k] = pack_bf16(act_fwd(gv.x, act) * uv.x, act_fwd(gv.y, act) * uv.y);
    }
    *reinterpret_cast<uint4*>(out + r * F + c) = o;
  }
}

// din [M, 2F] = [dout * up * act'(gate) | dout * act(gate)]
__global__ void glu_bwd_kernel(const __nv_bfloat16* __restrict__ in, const __nv_bfloat16* __restrict__ dout,
                               __nv_bfloat16* __restrict__ din, long long M, int F, int act,
                               const int* __restrict__ rows_dev) {
  tfb::pdl_sync();
  const int vec = F >> 3;
  if (rows_dev) M = min(M, (long long)max(*rows_dev, 0));
  const long long total = M * vec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec;
    const int c = int(i % vec) * 8;
    const uint4 ug = *reinterpret_cast<const uint4*>(in + r * 2 * F + c);
    const uint4 uu = *reinterpret_cast<const uint4*>(in + r * 2 * F + F + c);
    const uint4 ud = *reinterpret_cast<const uint4*>(dout + r * F + c);
    const uint32_t* g = reinterpret_cast<const uint32_t*>(&ug);
    const uint32_t* u = reinterpret_cast<const uint32_t*>(&uu);
    const uint32_t* d = reinterpret_cast<const uint32_t*>(&ud);
    uint4 og, ou;
    uint32_t* pg = reinterpret_cast<uint32_t*>(&og);
    uint32_t* pu = reinterpret_cast<uint32_t*>(&ou);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 gv = unpack_bf16(g[k]), uv = unpack_bf16(u[k]), dv = unpack_bf16(d[k]);
      pg[k] = pack_bf16(dv.x * uv.x * act_grad(gv.x, act), dv.y * uv.y * act_grad(gv.y, act));
      pu[k] = pack_bf16(dv.x * act_fwd(gv.x, act), dv.y * act_fwd(gv.y, act));
    }
    *reinterpret_cast<uint4*>(din + r * 2 * F + c) = og;
    *reinterpret_cast<uint4*>(din + r * 2 * F + F + c) = ou;
  }
}

// Plain activation y = act(x) and dx = dy * act'(x) over n elements (n % 8 == 0).
__global__ void act_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n8,
                               int act) {
  tfb::pdl_sync();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    uint4 u = reinterpret_cast<const uint4*>(x)[i];
    uint32_t* p = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 v = unpack_bf16(p[k]);
      p[k] = pack_bf16(act_fwd(v.x, act), act_fwd(v.y, act));
    }
    reinterpret_cast<uint4*>(y)[i] = u;
  }
}
__global__ void act_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                               __nv_bfloat16* __restrict__ dx, long long n8, int act) {
  tfb::pdl_sync();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    const uint4 u = reinterpret_cast<const uint4*>(x)[i];
    uint4 d = reinterpret_cast<const uint4*>(dy)[i];
    const uint32_t* p = reinterpret_cast<const uint32_t*>(&u);
    uint32_t* q = reinterpret_cast<uint32_t*>(&d);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 v = unpack_bf16(p[k]), g = unpack_bf16(q[k]);
      q[k] = pack_bf16(g.x * act_grad(v.x, act), g.y * act_grad(v.y, act));
    }
    reinterpret_cast<uint4*>(dx)[i] = d;
  }
}

// ------------------------------------------------------------------------------------------------
// Embedding: out[t, :] = W[ids[t], :] (+ P[pos[t], :] for learned positions);
// backward: dW[ids[t], :] += dout[t, :] (fp32 atomics straight into the fp32 gradient buffer).
// ------------------------------------------------------------------------------------------------
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ W,
                                     const __nv_bfloat16* __restrict__ P, __nv_bfloat16* __restrict__ out, int T,
                                     int S, int H, int V) {
  tfb::pdl_sync();
  const int vec = H >> 3;
  const long long total = (long long)T * vec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = int(i / vec), c = int(i % vec) * 8;
    long long id = ids[t];
    TFB_BOUNDS(id >= 0 && id < V, 1, id, V);
    if (id < 0 || id >= V) id = 0;
    uint4 u = *reinterpret_cast<const uint4*>(W + id * H + c);
    if (P) {
      const uint4 pu = *reinterpret_cast<const uint4*>(P + (long long)(t % S) * H + c);
      uint32_t* a = reinterpret_cast<uint32_t*>(&u);
      const uint32_t* b = reinterpret_cast<const uint32_t*>(&pu);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 x = unpack_bf16(a[k]), y = unpack_bf16(b[k]);
        a[k] = pack_bf16(x.x + y.x, x.y + y.y);
      }
    }
    *reinterpret_cast<uint4*>(out + (long long)t * H + c) = u;
  }
}

__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ dW, float* __restrict__ dP, int T, int S, int H, int V) {
  tfb::pdl_sync();
  const int vec = H >> 2;
  const long long total = (long long)T * vec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = int(i / vec), c = int(i % vec) * 4;
    const long long id = ids[t];
    TFB_BOUNDS(id >= 0 && id < V, 2, id, V);
    if (id < 0 || id >= V) continue;
    const uint2 u = *reinterpret_cast<const uint2*>(dout + (long long)t * H + c);
    const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
    float* dst = dW + id * H + c;
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y)
                 : "memory");
    if (dP) {
      float* dp = dP + (long long)(t % S) * H + c;
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dp), "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y)
                   : "memory");
    }
  }
}

// out = a + b (bf16), n % 8 == 0
__global__ void add_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                           __nv_bfloat16* __restrict__ out, long long n8) {
  tfb::pdl_sync();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    uint4 u = reinterpret_cast<const uint4*>(a)[i];
    const uint4 v = reinterpret_cast<const uint4*>(b)[i];
    uint32_t* p = reinterpret_cast<uint32_t*>(&u);
    const uint32_t* q = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 x = unpack_bf16(p[k]), y = unpack_bf16(q[k]);
      p[k] = pack_bf16(x.x + y.x, x.y + y.y);
    }
    reinterpret_cast<uint4*>(out)[i] = u;
  }
}

static inline int grid_for(long long work, int threads = 256) {
  long long b = (work + threads - 1) / threads;
  const long long cap = (long long)sm_count() * 16;
  return int(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace tfb

using namespace tfb;

TFB_API int tfb_rope(void* x, const float* cos_t, const float* sin_t, const int* positions, int T, int S,
                     int pos_offset, int n_heads, int D, long long ld, int backward, void* stream) {
  if (D % 16 || ld % 8 || (reinterpret_cast<uintptr_t>(x) & 15)) return TFB_ERR_ARG;
  const long long work = (long long)T * n_heads * (D / 16);
  tfb::launch_k(rope_kernel, grid_for(work), 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<__nv_bfloat16*>(x), cos_t, sin_t, positions, T, S, pos_offset, n_heads, D, ld, backward ? -1.f : 1.f);
  return int(cudaGetLastError());
}

TFB_API int tfb_glu_fwd_rows(const void* in, void* out, long long M, int F, int act, const int* rows_dev, void* stream) {
  if (F % 8) return TFB_ERR_ARG;
  tfb::launch_k(glu_fwd_kernel, grid_for(M * (F / 8)), 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out), M, F, act, rows_dev);
  return int(cudaGetLastError());
}
TFB_API int tfb_glu_fwd(const void* in, void* out, long long M, int F, int act, void* stream) {
  return tfb_glu_fwd_rows(in, out, M, F, act, nullptr, stream);
}
TFB_API int tfb_glu_bwd_rows(const void* in, const void* dout, void* din, long long M, int F, int act, const int* rows_dev,
                             void* stream) {
  if (F % 8) return TFB_ERR_ARG;
  tfb::launch_k(glu_bwd_kernel, grid_for(M * (F / 8)), 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(in), static_cast<const __nv_bfloat16*>(dout), static_cast<__nv_bfloat16*>(din),
      M, F, act, rows_dev);
  return int(cudaGetLastError());
}
TFB_API int tfb_glu_bwd(const void* in, const void* dout, void* din, long long M, int F, int act, void* stream) {
  return tfb_glu_bwd_rows(in, dout, din, M, F, act, nullptr, stream);
}
TFB_API int tfb_act_fwd(const void* x, void* y, long long n, int act, void* stream) {
  if (n % 8) return TFB_ERR_ARG;
  tfb::launch_k(act_fwd_kernel, grid_for(n / 8), 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n / 8, act);
  return int(cudaGetLastError());
}
TFB_API int tfb_act_bwd(const void* x, const void* dy, void* dx, long long n, int act, void* stream) {
  if (n % 8) return TFB_ERR_ARG;
  tfb::launch_k(act_bwd_kernel, grid_for(n / 8), 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dx),
      n / 8, act);
  return int(cudaGetLastError());
}
TFB_API int tfb_embedding_fwd(const long long* ids, const void* W, const void* P, void* out, int T, int S, int H, int V,
                              void* stream) {
  if (H % 8) return TFB_ERR_ARG;
  tfb::launch_k(embedding_fwd_kernel, grid_for((long long)T * (H / 8)), 256, 0, static_cast<cudaStream_t>(stream), 
      ids, static_cast<const __nv_bfloat16*>(W), static_cast<const __nv_bfloat16*>(P), static_cast<__nv_bfloat16*>(out),
      T, S, H, V);
  return int(cudaGetLastError());
}
TFB_API int tfb_embedding_bwd(const long long* ids, const void* dout, float* dW, float* dP, int T, int S, int H, int V,
                              void* stream) {
  if (H % 4) return TFB_ERR_ARG;
  tfb::launch_k(embedding_bwd_kernel, grid_for((long long)T * (H / 4)), 256, 0, static_cast<cudaStream_t>(stream), 
      ids, static_cast<const __nv_bfloat16*>(dout), dW, dP, T, S, H, V);
  return int(cudaGetLastError());
}
TFB_API int tfb_add_bf16(const void* a, const void* b, void* out, long long n, void* stream) {
  if (n % 8) return TFB_ERR_ARG;
  tfb::launch_k(add_kernel, grid_for(n / 8), 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), static_cast<__nv_bfloat16*>(out),
      n / 8);
  return int(cudaGetLastError());
}
