// Token sampling on the device: repetition penalty, temperature, top-k, top-p (nucleus), greedy.
//
// One CTA per sequence.  The filtered set is never sorted: the top-k cut and the top-p cut are found
// by bisection on a logit threshold (count / probability mass above the threshold are block
// reductions), then one uniform random number (counter-based hash of seed, row and step) picks a
// token by walking the cumulative mass of the surviving logits in vocabulary order.
//
// Reference counterpart: Sampler::sample (src/inference/sampler.cpp:166-180: repetition penalty ->
// top-p if p < 1 else top-k; nth_element / sort on the host).
#include "tfb_host.h"
#include "tfb_ptx.cuh"

namespace tfb {

constexpr int SAMP_THREADS = 1024;

__device__ __forceinline__ float blk_sum(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  v = (threadIdx.x & 31) < (blockDim.x >> 5) ? sh[threadIdx.x & 31] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float blk_max(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  v = (threadIdx.x & 31) < (blockDim.x >> 5) ? sh[threadIdx.x & 31] : -INFINITY;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ uint32_t hash_u32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
  return x;
}

struct SampleArgs {
  const void* logits; int logits_bf16; long long ld;  // [B, V]
  float* work;                                         // [B, V] fp32 scratch (processed logits)
  const int* history; int hist_len;                    // [B, hist_len] token ids (-1 = empty) for repetition penalty
  const float* temperature; const int* top_k; const float* top_p; const float* rep_penalty;  // per row (may be null)
  long long* out_ids; float* out_logprob;
  int V; unsigned long long seed; int step;
};

__global__ void __launch_bounds__(SAMP_THREADS) sample_kernel(SampleArgs a) {
  tfb::pdl_sync();
  __shared__ float sh[32];
  __shared__ float s_thr;
  __shared__ int s_pick;
  const int b = blockIdx.x, tid = threadIdx.x;
  const int V = a.V;
  float* w = a.work + (long long)b * V;
  const float T = a.temperature ? a.temperature[b] : 1.f;
  const int K = a.top_k ? a.top_k[b] : 0;
  const float P = a.top_p ? a.top_p[b] : 1.f;
  const float rp = a.rep_penalty ? a.rep_penalty[b] : 1.f;
  const float invT = T > 0.f ? 1.f / T : 1.f;

  // ---- load (+ temperature) ----
  for (int i = tid; i < V; i += SAMP_THREADS) {
    float x = a.logits_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.logits)[(long long)b * a.ld + i])
                            : static_cast<const float*>(a.logits)[(long long)b * a.ld + i];
    w[i] = x;
  }
  __syncthreads();
  // ---- repetition penalty on the raw logits (each history token once) ----
  if (rp != 1.f && a.history) {
    const int* h = a.history + (long long)b * a.hist_len;
    for (int j = tid; j < a.hist_len; j += SAMP_THREADS) {
      const int tok = h[j];
      if (tok < 0 || tok >= V) continue;
      bool first = true;  // apply once per distinct token: only the first occurrence acts
      for (int k = 0; k < j; ++k)
        if (h[k] == tok) { first = false; break; }
      if (first) {
        const float x = w[tok];
        w[tok] = x > 0.f ? x / rp : x * rp;
      }
    }
    __syncthreads();
  }
  float mx = -INFINITY;
  int arg = 0;
  for (int i = tid; i < V; i += SAMP_THREADS) {
    const float x = w[i] * invT;
    w[i] = x;
    if (x > mx) { mx = x; arg = i; }
  }
  const float gmx = blk_max(mx, sh);
  // ---- greedy ----
  if (T <= 0.f || K == 1) {
    // lowest index among the maxima
    int cand = (mx == gmx) ? arg : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __shared__ int shi[32];
    __syncthreads();
    if ((tid & 31) == 0) shi[tid >> 5] = cand;
    __syncthreads();
    if (tid == 0) {
      int best = 0x7fffffff;
      for (int i = 0; i < SAMP_THREADS / 32; ++i) best = min(best, shi[i]);
      s_pick = best;
    }
    __syncthreads();
    float z = 0.f;
    for (int i = tid; i < V; i += SAMP_THREADS) z += __expf(w[i] - gmx);
    z = blk_sum(z, sh);
    if (tid == 0) {
      a.out_ids[b] = s_pick;
      if (a.out_logprob) a.out_logprob[b] = w[s_pick] - gmx - logf(z);
    }
    return;
  }
  float gmn = INFINITY;
  for (int i = tid; i < V; i += SAMP_THREADS) gmn = fminf(gmn, w[i]);
  gmn = -blk_max(-gmn, sh);
  float z_all = 0.f;
  for (int i = tid; i < V; i += SAMP_THREADS) z_all += __expf(w[i] - gmx);
  z_all = blk_sum(z_all, sh);

  float thr = gmn;  // keep everything >= thr
  // ---- top-k: largest threshold with count(x >= thr) >= K ----
  if (K > 0 && K < V) {
    float lo = gmn, hi = gmx;
    for (int it = 0; it < 30; ++it) {
      const float mid = 0.5f * (lo + hi);
      float c = 0.f;
      for (int i = tid; i < V; i += SAMP_THREADS) c += (w[i] >= mid) ? 1.f : 0.f;
      c = blk_sum(c, sh);
      if (c >= float(K)) lo = mid; else hi = mid;
    }
    thr = lo;
  }
  // ---- top-p: largest threshold whose kept mass (within the top-k set) reaches P ----
  if (P < 1.f) {
    float zk = 0.f;
    for (int i = tid; i < V; i += SAMP_THREADS) zk += (w[i] >= thr) ? __expf(w[i] - gmx) : 0.f;
    zk = blk_sum(zk, sh);
    float lo = thr, hi = gmx;
    for (int it = 0; it < 30; ++it) {
      const float mid = 0.5f * (lo + hi);
      float mass = 0.f;
      for (int i = tid; i < V; i += SAMP_THREADS) mass += (w[i] >= mid) ? __expf(w[i] - gmx) : 0.f;
      mass = blk_sum(mass, sh);
      if (mass >= P * zk) lo = mid; else hi = mid;
    }
    thr = lo;
  }
  if (tid == 0) s_thr = thr;
  __syncthreads();
  thr = s_thr;
  // ---- draw: contiguous chunk per thread so that the walk follows vocabulary order ----
  const int per = (V + SAMP_THREADS - 1) / SAMP_THREADS;
  const int i0 = tid * per, i1 = min(V, i0 + per);
  float part = 0.f;
  for (int i = i0; i < i1; ++i) part += (w[i] >= thr) ? __expf(w[i] - gmx) : 0.f;
  __shared__ float s_part[SAMP_THREADS];
  s_part[tid] = part;
  const float zkeep = blk_sum(part, sh);
  __syncthreads();
  if (tid == 0) {
    const uint32_t h1 = hash_u32(uint32_t(a.seed) ^ hash_u32(uint32_t(a.seed >> 32) + 0x9e3779b9u * uint32_t(b + 1)) ^
                                 hash_u32(0x85ebca6bu * uint32_t(a.step + 1)));
    const float u = (float(h1 >> 8) + 0.5f) * (1.f / 16777216.f) * zkeep;
    float cum = 0.f;
    int chunk = SAMP_THREADS - 1;
    for (int t = 0; t < SAMP_THREADS; ++t) {
      if (cum + s_part[t] >= u && s_part[t] > 0.f) { chunk = t; break; }
      cum += s_part[t];
    }
    int pick = -1;
    const int c0 = chunk * per, c1 = min(V, c0 + per);
    for (int i = c0; i < c1; ++i) {
      if (w[i] >= thr) {
        cum += __expf(w[i] - gmx);
        pick = i;
        if (cum >= u) break;
      }
    }
    if (pick < 0) pick = 0;
    a.out_ids[b] = pick;
    if (a.out_logprob) a.out_logprob[b] = w[pick] - gmx - logf(z_all);
  }
}

}  // namespace tfb

struct TfbSampleDesc {
  const void* logits; int logits_bf16; long long ld;
  float* work;
  const int* history; int hist_len;
  const float* temperature; const int* top_k; const float* top_p; const float* rep_penalty;
  long long* out_ids; float* out_logprob;
  int V; unsigned long long seed; int step;
};

TFB_API int tfb_sample(const TfbSampleDesc* d, int B, void* stream) {
  static_assert(sizeof(TfbSampleDesc) == sizeof(tfb::SampleArgs), "layout");
  if (B <= 0 || d->V <= 0) return TFB_ERR_ARG;
  tfb::SampleArgs a;
  memcpy(&a, d, sizeof(a));
  tfb::launch_k(tfb::sample_kernel, B, tfb::SAMP_THREADS, 0, static_cast<cudaStream_t>(stream), a);
  return int(cudaGetLastError());
}
