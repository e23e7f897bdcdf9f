// Paged KV cache (16-token pages) with bf16 / fp8-e4m3 / 4-bit storage, and decode attention that
// dequantises K and V on the fly.
//
// Storage per layer, per K or V ("pool"):
//   KV_BF16 : [pages, 16, Hkv, D] bf16
//   KV_FP8  : [pages, 16, Hkv, D] e4m3 bytes + scale fp32 [pages, 16, Hkv]       (amax / 448 per head row)
//   KV_Q4   : [pages, 16, Hkv, D/2] bytes (low nibble = even element) + scale fp16 [pages, 16, Hkv, D/32]
//             value = (nibble - 8) * scale, scale = amax / 7 per 32-element block
//
// kv_append   : quantise and scatter the K/V rows of new tokens into their page slots
// paged_decode: one CTA per (sequence, kv head, split of the context).  The G = Hq / Hkv query heads
//               that share the kv head are processed together.  Per 128-token tile: each thread scores
//               one token against all G queries (K row dequantised in registers, queries in shared
//               memory), the block updates the running max / sum, then each thread owns output
//               dimensions and accumulates p * V over the tile with coalesced V reads.
// paged_combine: merges the per-split partial results.
//
// Reference counterparts: PagedAttention::forward (src/inference/inference_paging.cpp:24-117, no length
// mask), Q4KVCache 4-bit blocks (src/model/kv_cache_quant4.cpp:207-362), flash_decoding
// (src/inference/inference_kv.cpp:141-205).
#include <algorithm>
#include <cuda_fp16.h>

#include "tfb_host.h"
#include "tfb_ptx.cuh"

TFB_BOUNDS_DEFINE(paged_attention)

namespace tfb {

enum { KV_BF16 = 0, KV_FP8 = 1, KV_Q4 = 2 };
constexpr int PAGE = 16;

__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
  __half2_raw h2;
  asm("{\n\t.reg .b16 t;\n\tmov.b16 t, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, t;\n\t}" : "=r"(*reinterpret_cast<uint32_t*>(&h2)) : "h"(uint16_t(b)));
  return __half2float(__half(__half_raw{h2.x}));
}
__device__ __forceinline__ uint8_t f32_to_e4m3_sat(float x) {
  uint16_t r;
  asm("{\n\t.reg .b16 t;\n\tcvt.rn.satfinite.e4m3x2.f32 t, %1, %2;\n\tmov.b16 %0, t;\n\t}" : "=h"(r) : "f"(0.f), "f"(x));
  return uint8_t(r & 0xff);
}

struct KvPool {
  void* data;     // packed values
  void* scale;    // fp32 (fp8) or fp16 (q4) scales, null for bf16
  long long rows; // token slots in the pool (pages x PAGE); 0 = not given.  Read by the bounds-check build only.
};

// ------------------------------------------------------------------------------------------------
// append: src rows are [T, ld] bf16 with K head h at column k_col0 + h*D, V at v_col0 + h*D
// one warp per (token, kv head); slot_mapping[t] = page * 16 + slot (negative = skip)
// ------------------------------------------------------------------------------------------------
template <int MODE>
__device__ __forceinline__ void store_row(KvPool pool, long long slot, int h, int Hkv, int D, const float* v, int n,
                                          int lane) {
  // each lane holds n = D/32 consecutive elements starting at lane * n
  const long long row = slot * Hkv + h;
  if (MODE == KV_BF16) {
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(pool.data) + row * D + lane * n;
    for (int i = 0; i < n; ++i) dst[i] = __float2bfloat16(v[i]);
  } else if (MODE == KV_FP8) {
    float amax = 0.f;
    for (int i = 0; i < n; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = amax > 0.f ? amax / 448.f : 1.f;
    if (lane == 0) static_cast<float*>(pool.scale)[row] = s;
    uint8_t* dst = static_cast<uint8_t*>(pool.data) + row * D + lane * n;
    for (int i = 0; i < n; ++i) dst[i] = f32_to_e4m3_sat(v[i] / s);
  } else {
    // 32-element blocks: the lanes that share a block are 32 / n consecutive lanes
    const int lanes_per_block = 32 / n;
    float amax = 0.f;
    for (int i = 0; i < n; ++i) amax = fmaxf(amax, fabsf(v[i]));
    for (int o = lanes_per_block >> 1; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = amax > 0.f ? amax / 7.f : 1.f;
    const float sh = __half2float(__float2half(s));  // the decoder sees the fp16-rounded scale
    if ((lane % lanes_per_block) == 0)
      static_cast<__half*>(pool.scale)[row * (D / 32) + (lane * n) / 32] = __float2half(s);
    uint8_t* dst = static_cast<uint8_t*>(pool.data) + row * (D / 2) + (lane * n) / 2;
    for (int i = 0; i < n; i += 2) {
      int a = __float2int_rn(v[i] / sh) + 8, b = __float2int_rn(v[i + 1] / sh) + 8;
      a = min(max(a, 0), 15);
      b = min(max(b, 0), 15);
      dst[i / 2] = uint8_t(a | (b << 4));
    }
  }
}

template <int MODE>
__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ src, long long ld, int k_col0, int v_col0,
                                 const long long* __restrict__ slot_mapping, KvPool kpool, KvPool vpool, int T,
                                 int Hkv, int D) {
  tfb::pdl_sync();
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (w >= (long long)T * Hkv) return;
  const int h = int(w % Hkv);
  const long long t = w / Hkv;
  const long long slot = slot_mapping[t];
  if (slot < 0) return;
  TFB_BOUNDS(kpool.rows == 0 || slot < kpool.rows, 51, slot, kpool.rows);
#ifdef TFB_BOUNDS_CHECK
  if (kpool.rows != 0 && slot >= kpool.rows) return;
#endif
  const int n = D / 32;  // 2 (D=64) or 4 (D=128)
  float kv[4], vv[4];
  const __nv_bfloat16* kp = src + t * ld + k_col0 + h * D + lane * n;
  const __nv_bfloat16* vp = src + t * ld + v_col0 + h * D + lane * n;
  for (int i = 0; i < n; ++i) {
    kv[i] = __bfloat162float(kp[i]);
    vv[i] = __bfloat162float(vp[i]);
  }
  store_row<MODE>(kpool, slot, h, Hkv, D, kv, n, lane);
  store_row<MODE>(vpool, slot, h, Hkv, D, vv, n, lane);
}

// ------------------------------------------------------------------------------------------------
// decode
// ------------------------------------------------------------------------------------------------
template <int MODE, int D>
__device__ __forceinline__ void load_row(const KvPool& pool, long long row, float* out) {
  // whole row (D values) into registers of one thread
  if (MODE == KV_BF16) {
    const uint4* p = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(pool.data) + row * D);
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const uint4 u = p[i];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16(w[j]);
        out[i * 8 + 2 * j] = f.x;
        out[i * 8 + 2 * j + 1] = f.y;
      }
    }
  } else if (MODE == KV_FP8) {
    const float s = static_cast<const float*>(pool.scale)[row];
    const uint4* p = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(pool.data) + row * D);
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
      const uint4 u = p[i];
      const uint8_t* b = reinterpret_cast<const uint8_t*>(&u);
#pragma unroll
      for (int j = 0; j < 16; ++j) out[i * 16 + j] = e4m3_to_f32(b[j]) * s;
    }
  } else {
    const __half* sp = static_cast<const __half*>(pool.scale) + row * (D / 32);
    const uint4* p = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(pool.data) + row * (D / 2));
#pragma unroll
    for (int i = 0; i < D / 32; ++i) {
      const float s = __half2float(sp[i]);
      const uint4 u = p[i];
      const uint8_t* b = reinterpret_cast<const uint8_t*>(&u);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        out[i * 32 + 2 * j] = float(int(b[j] & 15) - 8) * s;
        out[i * 32 + 2 * j + 1] = float(int(b[j] >> 4) - 8) * s;
      }
    }
  }
}

template <int MODE, int D>
__device__ __forceinline__ float load_elem(const KvPool& pool, long long row, int d) {
  if (MODE == KV_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(pool.data)[row * D + d]);
  if (MODE == KV_FP8)
    return e4m3_to_f32(static_cast<const uint8_t*>(pool.data)[row * D + d]) * static_cast<const float*>(pool.scale)[row];
  const uint8_t b = static_cast<const uint8_t*>(pool.data)[row * (D / 2) + d / 2];
  const float s = __half2float(static_cast<const __half*>(pool.scale)[row * (D / 32) + d / 32]);
  return float(int((d & 1) ? (b >> 4) : (b & 15)) - 8) * s;
}

constexpr int DEC_THREADS = 128;
constexpr int DEC_TILE = 128;
constexpr int MAX_G = 8;

// partial outputs: acc [B, Hq, splits, D] fp32 (unnormalised), ml [B, Hq, splits, 2] (max, sum)
template <int MODE, int D, int G>
__global__ void __launch_bounds__(DEC_THREADS) paged_decode_kernel(
    const __nv_bfloat16* __restrict__ q, long long ldq, KvPool kpool, KvPool vpool,
    const int* __restrict__ block_table, int max_pages, const int* __restrict__ seq_lens, float* __restrict__ acc_out,
    float* __restrict__ ml_out, int Hq, int Hkv, int splits, float scale) {
  tfb::pdl_sync();
  __shared__ float sq[G][D];
  __shared__ float sp[G][DEC_TILE];
  __shared__ float red[G][DEC_THREADS / 32];
  const int b = blockIdx.x, hk = blockIdx.y, sp_idx = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int len = seq_lens[b];
  const int per = ((len + splits - 1) / splits + PAGE - 1) / PAGE * PAGE;
  const int t_begin = sp_idx * per, t_end = min(len, t_begin + per);
  for (int i = tid; i < G * D; i += DEC_THREADS) {
    const int g = i / D, d = i % D;
    sq[g][d] = __bfloat162float(q[(long long)b * ldq + (hk * G + g) * D + d]) * scale;
  }
  __syncthreads();
  float m[G], l[G];
  // P.V: warp w takes the tokens w, w + 4, ... of a tile, lane l the DL consecutive output dims starting at l * DL; the
  // four partial sums meet in shared memory after the last tile
  constexpr int DL = D / 32;
  constexpr int NW = DEC_THREADS / 32;
  float acc[G][DL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < DL; ++j) acc[g][j] = 0.f;
  }
  const int* bt = block_table + (long long)b * max_pages;
  for (int t0 = t_begin; t0 < t_end; t0 += DEC_TILE) {
    // ---- scores: thread tid <-> token t0 + tid ----
    const int t = t0 + tid;
    float s[G];
    if (t < t_end) {
      long long page = bt[t / PAGE];
      TFB_BOUNDS(kpool.rows == 0 || (page >= 0 && (page + 1) * PAGE <= kpool.rows), 52, page, kpool.rows / PAGE);
#ifdef TFB_BOUNDS_CHECK
      if (kpool.rows != 0 && (page < 0 || (page + 1) * PAGE > kpool.rows)) page = 0;
#endif
      const long long row = (page * PAGE + (t % PAGE)) * Hkv + hk;
      float kr[D];
      load_row<MODE, D>(kpool, row, kr);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float a = 0.f;
#pragma unroll
        for (int d = 0; d < D; ++d) a = fmaf(kr[d], sq[g][d], a);
        s[g] = a;
      }
    } else {
#pragma unroll
      for (int g = 0; g < G; ++g) s[g] = -INFINITY;
    }
    // ---- block max per head ----
    float tile_m[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float v = s[g];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
      if (lane == 0) red[g][warp] = v;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float v = red[g][0];
#pragma unroll
      for (int w2 = 1; w2 < DEC_THREADS / 32; ++w2) v = fmaxf(v, red[g][w2]);
      tile_m[g] = fmaxf(m[g], v);
    }
    __syncthreads();
    float alpha[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float p = (t < t_end) ? __expf(s[g] - tile_m[g]) : 0.f;
      sp[g][tid] = p;
      alpha[g] = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - tile_m[g]);
      float v = p;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) red[g][warp] = v;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float v = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < DEC_THREADS / 32; ++w2) v += red[g][w2];
      l[g] = l[g] * alpha[g] + v;
      m[g] = tile_m[g];
#pragma unroll
      for (int j = 0; j < DL; ++j) acc[g][j] *= alpha[g];
    }
    // ---- P.V: thread tid <-> output dims tid + j * DEC_THREADS ----
    const int nt = min(DEC_TILE, t_end - t0);
    __syncthreads();                                   // sp[][] of this tile is complete
    // four tokens of this warp per step: their V loads are independent and in flight together
    constexpr int VU = 4;
    for (int tt0 = warp; tt0 < nt; tt0 += NW * VU) {
      float vv[VU][DL];
#pragma unroll
      for (int u = 0; u < VU; ++u) {
        const int tt = min(tt0 + u * NW, nt - 1);
        const int tk = t0 + tt;
        long long page = bt[tk / PAGE];
#ifdef TFB_BOUNDS_CHECK
        if (vpool.rows != 0 && (page < 0 || (page + 1) * PAGE > vpool.rows)) page = 0;   // reported by the score pass above
#endif
        const long long row = (page * PAGE + (tk % PAGE)) * Hkv + hk;
        if (MODE == KV_BF16) {
          const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(vpool.data) + row * D + lane * DL;
          if (DL == 4) {
            const uint2 w2 = *reinterpret_cast<const uint2*>(src);
            const float2 a = unpack_bf16(w2.x), c = unpack_bf16(w2.y);
            vv[u][0] = a.x; vv[u][1] = a.y; vv[u][DL - 2] = c.x; vv[u][DL - 1] = c.y;
          } else {
            const float2 a = unpack_bf16(*reinterpret_cast<const uint32_t*>(src));
            vv[u][0] = a.x; vv[u][DL - 1] = a.y;
          }
        } else {
#pragma unroll
          for (int j = 0; j < DL; ++j) vv[u][j] = load_elem<MODE, D>(vpool, row, lane * DL + j);
        }
      }
#pragma unroll
      for (int u = 0; u < VU; ++u) {
        const int tt = tt0 + u * NW;
        if (tt < nt) {
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float pw = sp[g][tt];
#pragma unroll
            for (int j = 0; j < DL; ++j) acc[g][j] = fmaf(pw, vv[u][j], acc[g][j]);
          }
        }
      }
    }
    __syncthreads();
  }
  // cross-warp sum of the partial outputs
  __shared__ float part[NW][G][D];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int j = 0; j < DL; ++j) part[warp][g][lane * DL + j] = acc[g][j];
  __syncthreads();
  for (int i = tid; i < G * D; i += DEC_THREADS) {
    const int g = i / D, d = i % D;
    float v = 0.f;
#pragma unroll
    for (int w2 = 0; w2 < NW; ++w2) v += part[w2][g][d];
    const long long base = (((long long)b * Hq + hk * G + g) * splits + sp_idx);
    acc_out[base * D + d] = v;
  }
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (tid == g) {
      const long long base = (((long long)b * Hq + hk * G + g) * splits + sp_idx);
      ml_out[base * 2] = m[g];
      ml_out[base * 2 + 1] = l[g];
    }
  }
}

// o[b, h, :] = sum_s acc_s * exp(m_s - M) / sum_s l_s * exp(m_s - M)
__global__ void paged_combine_kernel(const float* __restrict__ acc, const float* __restrict__ ml,
                                     __nv_bfloat16* __restrict__ o, long long ldo, int Hq, int D, int splits) {
  tfb::pdl_sync();
  const int b = blockIdx.x, h = blockIdx.y;
  const long long base = ((long long)b * Hq + h) * splits;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, ml[(base + s) * 2]);
  float L = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = ml[(base + s) * 2];
    if (ms != -INFINITY) L += ml[(base + s) * 2 + 1] * __expf(ms - M);
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = ml[(base + s) * 2];
      if (ms != -INFINITY) v += acc[(base + s) * D + d] * __expf(ms - M);
    }
    o[(long long)b * ldo + h * D + d] = __float2bfloat16(L > 0.f ? v / L : 0.f);
  }
}

template <int MODE, int D>
static int launch_decode_g(int G, dim3 grid, cudaStream_t st, const __nv_bfloat16* q, long long ldq, KvPool k, KvPool v,
                           const int* bt, int max_pages, const int* lens, float* acc, float* ml, int Hq, int Hkv,
                           int splits, float scale) {
#define TFB_CASE(GG)                                                                                              \
  case GG:                                                                                                        \
    tfb::launch_k(paged_decode_kernel<MODE, D, GG>, grid, DEC_THREADS, 0, st, q, ldq, k, v, bt, max_pages, lens, acc, ml, Hq, \
                                                                   Hkv, splits, scale);                           \
    break;
  switch (G) {
    TFB_CASE(1) TFB_CASE(2) TFB_CASE(4) TFB_CASE(8)
    default: return TFB_ERR_ARG;
  }
#undef TFB_CASE
  return int(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------------
// gather: the first n cached tokens of one sequence -> contiguous bf16 rows [n, Hkv * D] for K and V (dequantised), so
// that a prompt suffix behind a cached prefix can run through the tensor-core attention kernel instead of one
// decode-style query per token.  One thread per (token, kv head, 32-element chunk).
// ------------------------------------------------------------------------------------------------
template <int MODE, int D>
__device__ __forceinline__ void load_chunk32(const KvPool& pool, long long row, int c, float* out) {
  if (MODE == KV_BF16) {
    const uint4* p = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(pool.data) + row * D + c * 32);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 u = p[i];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16(w[j]);
        out[i * 8 + 2 * j] = f.x;
        out[i * 8 + 2 * j + 1] = f.y;
      }
    }
  } else if (MODE == KV_FP8) {
    const float s = static_cast<const float*>(pool.scale)[row];
    const uint4* p = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(pool.data) + row * D + c * 32);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint4 u = p[i];
      const uint8_t* b = reinterpret_cast<const uint8_t*>(&u);
#pragma unroll
      for (int j = 0; j < 16; ++j) out[i * 16 + j] = e4m3_to_f32(b[j]) * s;
    }
  } else {
    const float s = __half2float(static_cast<const __half*>(pool.scale)[row * (D / 32) + c]);
    const uint4 u = *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(pool.data) + row * (D / 2) + c * 16);
    const uint8_t* b = reinterpret_cast<const uint8_t*>(&u);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      out[2 * j] = float(int(b[j] & 15) - 8) * s;
      out[2 * j + 1] = float(int(b[j] >> 4) - 8) * s;
    }
  }
}

template <int MODE, int D>
__global__ void __launch_bounds__(256) kv_gather_kernel(KvPool kpool, KvPool vpool, const int* __restrict__ block_table, int n,
                                                        __nv_bfloat16* __restrict__ out_k, __nv_bfloat16* __restrict__ out_v,
                                                        long long ld, int Hkv) {
  tfb::pdl_sync();
  constexpr int C = D / 32;
  const long long total = (long long)n * Hkv * C;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = int(i % C);
    const int h = int((i / C) % Hkv);
    const int t = int(i / ((long long)C * Hkv));
    long long page = block_table[t / PAGE];
    TFB_BOUNDS(kpool.rows == 0 || (page >= 0 && (page + 1) * PAGE <= kpool.rows), 53, page, kpool.rows / PAGE);
#ifdef TFB_BOUNDS_CHECK
    if (kpool.rows != 0 && (page < 0 || (page + 1) * PAGE > kpool.rows)) page = 0;
#endif
    const long long row = (page * PAGE + (t % PAGE)) * Hkv + h;
    float f[32];
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      load_chunk32<MODE, D>(which ? vpool : kpool, row, c, f);
      uint4* dst = reinterpret_cast<uint4*>((which ? out_v : out_k) + (long long)t * ld + h * D + c * 32);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 u;
        u.x = pack_bf16(f[q * 8], f[q * 8 + 1]); u.y = pack_bf16(f[q * 8 + 2], f[q * 8 + 3]);
        u.z = pack_bf16(f[q * 8 + 4], f[q * 8 + 5]); u.w = pack_bf16(f[q * 8 + 6], f[q * 8 + 7]);
        dst[q] = u;
      }
    }
  }
}

}  // namespace tfb

using namespace tfb;

// The first n cached tokens of one sequence (block_table: its page list) as contiguous bf16 rows: out_k / out_v
// [n, ld] with kv head h at column h * D (ld a multiple of 8, buffers 16-byte aligned).
TFB_API int tfb_kv_gather(void* k_data, void* k_scale, void* v_data, void* v_scale, const int* block_table, int n, void* out_k,
                          void* out_v, long long ld, int Hkv, int D, int mode, long long pool_rows, void* stream) {
  if ((D != 64 && D != 128) || Hkv <= 0 || n <= 0 || (ld & 7) || ld < (long long)Hkv * D) return TFB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(out_k) | reinterpret_cast<uintptr_t>(out_v)) & 15) return TFB_ERR_ARG;
  KvPool kp{k_data, k_scale, pool_rows}, vp{v_data, v_scale, pool_rows};
  const long long total = (long long)n * Hkv * (D / 32);
  const int grid = int(std::min<long long>((total + 255) / 256, 148 * 8));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto ok = static_cast<__nv_bfloat16*>(out_k);
  auto ov = static_cast<__nv_bfloat16*>(out_v);
#define TFB_GATHER(MODE)                                                                                            \
  do {                                                                                                              \
    if (D == 64) tfb::launch_k(kv_gather_kernel<MODE, 64>, grid, 256, 0, st, kp, vp, block_table, n, ok, ov, ld, Hkv);   \
    else tfb::launch_k(kv_gather_kernel<MODE, 128>, grid, 256, 0, st, kp, vp, block_table, n, ok, ov, ld, Hkv);          \
  } while (0)
  if (mode == KV_BF16) TFB_GATHER(KV_BF16);
  else if (mode == KV_FP8) TFB_GATHER(KV_FP8);
  else if (mode == KV_Q4) TFB_GATHER(KV_Q4);
  else return TFB_ERR_ARG;
#undef TFB_GATHER
  return int(cudaGetLastError());
}

// pool_rows: token slots in each pool (pages x 16), checked by the bounds-check build; 0 = not given.
TFB_API int tfb_kv_append(const void* src, long long ld, int k_col0, int v_col0, const long long* slot_mapping,
                          void* k_data, void* k_scale, void* v_data, void* v_scale, int T, int Hkv, int D, int mode,
                          long long pool_rows, void* stream) {
  if (D != 64 && D != 128) return TFB_ERR_ARG;
  KvPool kp{k_data, k_scale, pool_rows}, vp{v_data, v_scale, pool_rows};
  const long long warps = (long long)T * Hkv;
  const unsigned blocks = unsigned((warps * 32 + 255) / 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto s = static_cast<const __nv_bfloat16*>(src);
  if (mode == KV_BF16) tfb::launch_k(kv_append_kernel<KV_BF16>, blocks, 256, 0, st, s, ld, k_col0, v_col0, slot_mapping, kp, vp, T, Hkv, D);
  else if (mode == KV_FP8) tfb::launch_k(kv_append_kernel<KV_FP8>, blocks, 256, 0, st, s, ld, k_col0, v_col0, slot_mapping, kp, vp, T, Hkv, D);
  else if (mode == KV_Q4) tfb::launch_k(kv_append_kernel<KV_Q4>, blocks, 256, 0, st, s, ld, k_col0, v_col0, slot_mapping, kp, vp, T, Hkv, D);
  else return TFB_ERR_ARG;
  return int(cudaGetLastError());
}

// q: [B, ldq] bf16 (query head h at column h*D).  acc_ws: fp32 [B*Hq*splits*D], ml_ws: fp32 [B*Hq*splits*2].
TFB_API int tfb_paged_decode(const void* q, long long ldq, void* k_data, void* k_scale, void* v_data, void* v_scale,
                             const int* block_table, int max_pages, const int* seq_lens, void* o, long long ldo,
                             float* acc_ws, float* ml_ws, int B, int Hq, int Hkv, int D, int splits, int mode,
                             float scale, long long pool_rows, void* stream) {
  if ((D != 64 && D != 128) || Hkv <= 0 || Hq % Hkv || splits < 1) return TFB_ERR_ARG;
  const int G = Hq / Hkv;
  KvPool kp{k_data, k_scale, pool_rows}, vp{v_data, v_scale, pool_rows};
  dim3 grid(B, Hkv, splits);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto Q = static_cast<const __nv_bfloat16*>(q);
  int rc;
#define TFB_GO(MODE)                                                                                                  \
  rc = (D == 64) ? launch_decode_g<MODE, 64>(G, grid, st, Q, ldq, kp, vp, block_table, max_pages, seq_lens, acc_ws,   \
                                             ml_ws, Hq, Hkv, splits, scale)                                           \
                 : launch_decode_g<MODE, 128>(G, grid, st, Q, ldq, kp, vp, block_table, max_pages, seq_lens, acc_ws,  \
                                              ml_ws, Hq, Hkv, splits, scale)
  if (mode == KV_BF16) { TFB_GO(KV_BF16); }
  else if (mode == KV_FP8) { TFB_GO(KV_FP8); }
  else if (mode == KV_Q4) { TFB_GO(KV_Q4); }
  else return TFB_ERR_ARG;
#undef TFB_GO
  if (rc) return rc;
  tfb::launch_k(paged_combine_kernel, dim3(B, Hq), 128, 0, st, acc_ws, ml_ws, static_cast<__nv_bfloat16*>(o), ldo, Hq, D, splits);
  return int(cudaGetLastError());
}
