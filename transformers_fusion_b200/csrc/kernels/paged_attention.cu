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
#include <cstdlib>
#include <cstring>
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
        } else if (MODE == KV_FP8) {
          // the lane's DL consecutive values in one load (4 or 2 bytes) + the row's scale
          const float sc = static_cast<const float*>(vpool.scale)[row];
          const uint8_t* src = static_cast<const uint8_t*>(vpool.data) + row * D + lane * DL;
          uint32_t w;
          if (DL == 4) w = *reinterpret_cast<const uint32_t*>(src);
          else w = *reinterpret_cast<const uint16_t*>(src);
#pragma unroll
          for (int j = 0; j < DL; ++j) vv[u][j] = e4m3_to_f32(uint8_t(w >> (8 * j))) * sc;
        } else {
          // 4-bit: DL values = DL / 2 bytes, all inside one 32-element scale group
          const float sc = __half2float(static_cast<const __half*>(vpool.scale)[row * (D / 32) + (lane * DL) / 32]);
          const uint8_t* src = static_cast<const uint8_t*>(vpool.data) + row * (D / 2) + (lane * DL) / 2;
          uint32_t w;
          if (DL == 4) w = *reinterpret_cast<const uint16_t*>(src);
          else w = *src;
#pragma unroll
          for (int j = 0; j < DL; ++j) vv[u][j] = float(int((w >> (4 * j)) & 15u) - 8) * sc;
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

// ------------------------------------------------------------------------------------------------
// decode on the tensor cores
//
// The kernel above spends ~1500 thread instructions per cached token and kv head (one K row per thread: 128 loads from
// shared memory and 512 FMAs for four query heads, then a warp walks the V rows) and ends up issue- and latency-bound at
// 0.3 of the copy bandwidth.  Here the G query heads of a kv head are the (zero-padded) 16 rows of an mma.sync
// m16n8k16 tile: S = Q K^T and O += P V cost 64 tensor instructions per 32 cached tokens, and what is left is moving
// the rows.  Each of the four warps of a CTA owns every fourth 32-token chunk of the split's range: it brings the
// chunk's K and V rows into its private shared-memory tile (cp.async for bf16 pools; load, dequantise, store for the
// fp8 / 4-bit pools), runs the two products with ldmatrix-fed fragments, and keeps its own running max / sum / output;
// the four partial results are merged once at the end.  Nothing is shared between the warps while they stream, so
// there is no CTA barrier in the loop; several CTAs per SM keep enough loads in flight.
// (mma.sync rather than tcgen05: with at most 8 query rows per kv head a 128-row UMMA tile would be 94 % padding.)
// ------------------------------------------------------------------------------------------------
constexpr int TC_THREADS = 128;
constexpr int TC_CHUNK = 32;

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void st_shared_u4(uint32_t dst, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// byte offset of 16-byte chunk c of row r in a [rows][D] bf16 tile with rows padded by 16 bytes: a row is one contiguous
// piece (the target of one bulk copy), and eight consecutive rows at one chunk index fall into eight different bank groups
// (row pitch = 17 or 9 chunks), which is what ldmatrix reads
template <int D>
__device__ __forceinline__ uint32_t tc_off(int r, int c) {
  return uint32_t(r * (D * 2 + 16) + (c << 4));
}

// rows t0 .. t0 + 31 (t0 a multiple of 16: two pages) of one sequence's cache, kv head hk -> the warp's [32][D] bf16 tile;
// rows from `nvalid` on are zero.  bf16 pools: lane r sends row r as one bulk copy that completes on the warp's mbarrier
// (the caller has armed it with the byte count); fp8 / 4-bit pools: 16-byte loads, conversion in registers, 16-byte stores.
template <int MODE, int D>
__device__ __forceinline__ void tc_stage(const KvPool& pool, const int* __restrict__ bt, int t0, int nvalid, int hk, int Hkv,
                                         uint32_t tile, int lane, uint32_t bar) {
  auto page_of = [&](int which) -> long long {
    long long page = bt[t0 / PAGE + which];
    TFB_BOUNDS(pool.rows == 0 || (page >= 0 && (page + 1) * PAGE <= pool.rows), 52, page, pool.rows / PAGE);
#ifdef TFB_BOUNDS_CHECK
    if (pool.rows != 0 && (page < 0 || (page + 1) * PAGE > pool.rows)) page = 0;
#endif
    return page;
  };
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  if (MODE == KV_BF16) {
    const int r = lane;
    if (r < nvalid) {
      const long long row = (page_of(r >> 4) * PAGE + (r & 15)) * Hkv + hk;
      bulk_load(tile + tc_off<D>(r, 0), static_cast<const __nv_bfloat16*>(pool.data) + row * D, D * 2, bar);
    } else {
#pragma unroll
      for (int c = 0; c < D / 8; ++c) st_shared_u4(tile + tc_off<D>(r, c), zero);
    }
    return;
  }
  const long long pg0 = page_of(0), pg1 = nvalid > PAGE ? page_of(1) : 0;
  auto row_of = [&](int r) -> long long { return ((r < PAGE ? pg0 : pg1) * PAGE + (r & 15)) * Hkv + hk; };
  if (MODE == KV_FP8) {
    constexpr int UPR = D / 16;                 // 16-byte loads (16 values) per row
    constexpr int N = TC_CHUNK * UPR / 32;      // loads per lane
    uint4 raw[N];
    float sc[N];
#pragma unroll
    for (int j = 0; j < N; ++j) {
      const int id = lane + 32 * j, r = id / UPR, u = id % UPR;
      raw[j] = zero;
      sc[j] = 0.f;
      if (r < nvalid) {
        const long long row = row_of(r);
        raw[j] = *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(pool.data) + row * D + u * 16);
        sc[j] = static_cast<const float*>(pool.scale)[row];
      }
    }
#pragma unroll
    for (int j = 0; j < N; ++j) {
      const int id = lane + 32 * j, r = id / UPR, u = id % UPR;
      const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw[j]);
      uint32_t w[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) w[q] = pack_bf16(e4m3_to_f32(b[2 * q]) * sc[j], e4m3_to_f32(b[2 * q + 1]) * sc[j]);
      st_shared_u4(tile + tc_off<D>(r, 2 * u), make_uint4(w[0], w[1], w[2], w[3]));
      st_shared_u4(tile + tc_off<D>(r, 2 * u + 1), make_uint4(w[4], w[5], w[6], w[7]));
    }
  } else {
    constexpr int UPR = D / 32;                 // 16-byte loads (32 values, one scale group) per row
    constexpr int N = TC_CHUNK * UPR / 32;
    uint4 raw[N];
    float sc[N];
#pragma unroll
    for (int j = 0; j < N; ++j) {
      const int id = lane + 32 * j, r = id / UPR, u = id % UPR;
      raw[j] = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);   // code 8 = value 0
      sc[j] = 0.f;
      if (r < nvalid) {
        const long long row = row_of(r);
        raw[j] = *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(pool.data) + row * (D / 2) + u * 16);
        sc[j] = __half2float(static_cast<const __half*>(pool.scale)[row * (D / 32) + u]);
      }
    }
#pragma unroll
    for (int j = 0; j < N; ++j) {
      const int id = lane + 32 * j, r = id / UPR, u = id % UPR;
      const uint32_t words[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
#pragma unroll
      for (int c = 0; c < 4; ++c) {             // one 32-bit word = eight codes = one output chunk
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          // code -> float without an integer conversion: 2^23 + code as bits, minus (2^23 + 8)
          const float lo = __uint_as_float(0x4B000000u | ((words[c] >> (8 * q)) & 15u)) - 8388616.f;
          const float hi = __uint_as_float(0x4B000000u | ((words[c] >> (8 * q + 4)) & 15u)) - 8388616.f;
          w[q] = pack_bf16(lo * sc[j], hi * sc[j]);
        }
        st_shared_u4(tile + tc_off<D>(r, 4 * u + c), make_uint4(w[0], w[1], w[2], w[3]));
      }
    }
  }
}

template <int MODE, int D>
__global__ void __launch_bounds__(TC_THREADS) paged_decode_mma_kernel(
    const __nv_bfloat16* __restrict__ q, long long ldq, KvPool kpool, KvPool vpool, const int* __restrict__ block_table,
    int max_pages, const int* __restrict__ seq_lens, float* __restrict__ acc_out, float* __restrict__ ml_out, int Hq, int Hkv,
    int G, int splits, float scale, int* status) {
  tfb::pdl_sync();
  extern __shared__ __align__(128) uint8_t tc_smem[];
  constexpr int ROWB = D * 2 + 16;                 // padded row pitch (see tc_off)
  constexpr int TILEB = TC_CHUNK * ROWB;
  constexpr int CPR = D / 8;
  constexpr int KS = D / 16;       // k steps of S = Q K^T
  constexpr int NBD = D / 8;       // n blocks of O
  const int b = blockIdx.x, hk = blockIdx.y, sp_idx = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t sQ = smem_u32(tc_smem);
  const uint32_t sK = sQ + 16 * ROWB + warp * 2 * TILEB, sV = sK + TILEB;
  // bf16 pools: two mbarriers per warp (K tile, V tile)
  const uint32_t bar_k = sQ + 16 * ROWB + (TC_THREADS / 32) * 2 * TILEB + warp * 16, bar_v = bar_k + 8;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tc_smem + 16 * ROWB + (TC_THREADS / 32) * 2 * TILEB + 64);
  if (MODE == KV_BF16 && lane == 0) {
    mbar_init(bar_k, 1);
    mbar_init(bar_v, 1);
    if (warp == 0) *abort_flag = 0;
    mbar_fence_init();
  }
  const int len = seq_lens[b];
  const int per = ((len + splits - 1) / splits + PAGE - 1) / PAGE * PAGE;
  const int t_begin = sp_idx * per, t_end = min(len, t_begin + per);
  const int* bt = block_table + (long long)b * max_pages;

  // the G query heads of this kv head as rows 0 .. G-1 of a 16-row tile
  for (int i = tid; i < 16 * CPR; i += TC_THREADS) {
    const int r = i / CPR, c = i % CPR;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < G) v = *reinterpret_cast<const uint4*>(q + (long long)b * ldq + (hk * G + r) * D + c * 8);
    st_shared_u4(sQ + tc_off<D>(r, c), v);
  }
  __syncthreads();
  uint32_t qa[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const int r = (lane & 7) + ((lane >> 3) & 1) * 8, c = 2 * ks + (lane >> 4);
    ldsm_x4(sQ + tc_off<D>(r, c), qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
  }
  float o[NBD][4];
#pragma unroll
  for (int n = 0; n < NBD; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;          // of row lane / 4 (log2 units), l summed over this thread's columns
  const float sl2 = scale * 1.4426950408889634f;

  // bf16 pools: lane r sends row r of a chunk as one bulk copy (`page`: the lane's page of that chunk), rows past the end
  // are zeroed.  The K tile is refilled as soon as S is computed and the V tile as soon as O is updated, so the next
  // chunk's rows travel while this chunk's softmax / products run, and the page indices are fetched one chunk ahead.
  auto issue_rows = [&](const KvPool& pool, long long page, int nv, uint32_t tile, uint32_t bar) {
    if (lane == 0) mbar_expect_tx(bar, uint32_t(nv) * D * 2);
    __syncwarp();
    if (lane < nv) {
      const long long row = (page * PAGE + (lane & 15)) * Hkv + hk;
      bulk_load(tile + tc_off<D>(lane, 0), static_cast<const __nv_bfloat16*>(pool.data) + row * D, D * 2, bar);
    } else {
      const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int c = 0; c < D / 8; ++c) st_shared_u4(tile + tc_off<D>(lane, c), zero);
    }
  };
  auto page_for = [&](int t0c, int nv) -> long long {
    long long page = lane < nv ? bt[t0c / PAGE + (lane >> 4)] : 0;
    TFB_BOUNDS(kpool.rows == 0 || (page >= 0 && (page + 1) * PAGE <= kpool.rows), 52, page, kpool.rows / PAGE);
#ifdef TFB_BOUNDS_CHECK
    if (kpool.rows != 0 && (page < 0 || (page + 1) * PAGE > kpool.rows)) page = 0;
#endif
    return page;
  };
  // after a wait that ran out: give the copies still in flight a bounded time to land before shared memory is reused
  auto drain = [&](uint32_t ph) {
    const uint64_t t0 = globaltimer_ns();
    while (!(mbar_try_wait(bar_k, ph) && mbar_try_wait(bar_v, ph))) {
      if (globaltimer_ns() - t0 > 2000000ull) { report(status, ST_TIMEOUT_DRAIN); break; }
    }
  };
  constexpr int STEP = (TC_THREADS / 32) * TC_CHUNK;
  uint32_t phase = 0;
  const int t_first = t_begin + warp * TC_CHUNK;
  if (MODE == KV_BF16 && t_first < t_end) {
    const int nv = min(TC_CHUNK, t_end - t_first);
    const long long pg = page_for(t_first, nv);
    issue_rows(kpool, pg, nv, sK, bar_k);
    issue_rows(vpool, pg, nv, sV, bar_v);
  }
  for (int t0 = t_first; t0 < t_end; t0 += STEP) {
    const int nvalid = min(TC_CHUNK, t_end - t0);
    const int nv_next = min(TC_CHUNK, t_end - (t0 + STEP));         // <= 0: this is the warp's last chunk
    long long pg_next = 0;
    if (MODE == KV_BF16) {
      if (nv_next > 0) pg_next = page_for(t0 + STEP, nv_next);
      // bounded: a copy that never lands sets the status word and the warp leaves the loop (its partial result is wrong,
      // the host raises from the status word)
      if (!mbar_wait_warp(bar_k, phase, abort_flag, status, ST_TIMEOUT_FULL)) { drain(phase); break; }
    } else {
      tc_stage<MODE, D>(kpool, bt, t0, nvalid, hk, Hkv, sK, lane, 0u);
      tc_stage<MODE, D>(vpool, bt, t0, nvalid, hk, Hkv, sV, lane, 0u);
    }
    __syncwarp();
    // ---- S = Q K^T: four blocks of eight tokens; the four accumulators are independent, so they are interleaved ----
    float sc[TC_CHUNK / 8][4];
#pragma unroll
    for (int nb = 0; nb < TC_CHUNK / 8; ++nb) sc[nb][0] = sc[nb][1] = sc[nb][2] = sc[nb][3] = 0.f;
#pragma unroll
    for (int k2 = 0; k2 < KS / 2; ++k2) {
#pragma unroll
      for (int nb = 0; nb < TC_CHUNK / 8; ++nb) {
        uint32_t k0, k1, k2r, k3;
        ldsm_x4(sK + tc_off<D>(nb * 8 + (lane & 7), k2 * 4 + (lane >> 3)), k0, k1, k2r, k3);
        mma_bf16_16816(sc[nb], qa[2 * k2], k0, k1);
        mma_bf16_16816(sc[nb], qa[2 * k2 + 1], k2r, k3);
      }
    }
    if (MODE == KV_BF16 && nv_next > 0) {      // the K tile is free: fetch the next chunk's keys
      __syncwarp();
      fence_proxy_async_smem();
      issue_rows(kpool, pg_next, nv_next, sK, bar_k);
    }
    // ---- online softmax of row lane / 4 (this thread: columns nb * 8 + (lane & 3) * 2 + {0, 1}) ----
    float mx = m_run;
#pragma unroll
    for (int nb = 0; nb < TC_CHUNK / 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int tok = nb * 8 + (lane & 3) * 2 + e;
        const float v = tok < nvalid ? sc[nb][e] * sl2 : -INFINITY;
        sc[nb][e] = v;
        mx = fmaxf(mx, v);
      }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - mx);
    m_run = mx;
    l_run *= alpha;
    uint32_t pa[TC_CHUNK / 16][4];
#pragma unroll
    for (int nb = 0; nb < TC_CHUNK / 8; ++nb) {
      const float p0 = exp2f(sc[nb][0] - mx), p1 = exp2f(sc[nb][1] - mx);
      l_run += p0 + p1;
      pa[nb >> 1][(nb & 1) * 2] = pack_bf16(p0, p1);     // rows 0-7 of the A tile; rows 8-15 (padding) stay zero
      pa[nb >> 1][(nb & 1) * 2 + 1] = 0u;
    }
#pragma unroll
    for (int n = 0; n < NBD; ++n) { o[n][0] *= alpha; o[n][1] *= alpha; }
    // ---- O += P V ----
    if (MODE == KV_BF16) {
      if (!mbar_wait_warp(bar_v, phase, abort_flag, status, ST_TIMEOUT_FULL)) { drain(phase); break; }
      phase ^= 1u;
    }
#pragma unroll
    for (int kk = 0; kk < TC_CHUNK / 16; ++kk) {
#pragma unroll
      for (int n2 = 0; n2 < NBD / 2; ++n2) {
        uint32_t v0, v1, v2, v3;
        ldsm_x4_t(sV + tc_off<D>(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * n2 + (lane >> 4)), v0, v1, v2, v3);
        mma_bf16_16816(o[2 * n2], pa[kk], v0, v1);
        mma_bf16_16816(o[2 * n2 + 1], pa[kk], v2, v3);
      }
    }
    __syncwarp();      // every lane is done with the tiles before they are refilled
    if (MODE == KV_BF16 && nv_next > 0) {            // ... by bulk copies, which write through the async proxy
      fence_proxy_async_smem();
      issue_rows(vpool, pg_next, nv_next, sV, bar_v);
    }
  }
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  // ---- merge the four warps (the staging area is free now) ----
  __syncthreads();
  float* red_m = reinterpret_cast<float*>(tc_smem);          // [4][8]
  float* red_l = red_m + 32;                                 // [4][8]
  float* red_o = red_l + 32;                                 // [4][8][D]
  const int row = lane >> 2;
  if ((lane & 3) == 0) {
    red_m[warp * 8 + row] = m_run;
    red_l[warp * 8 + row] = l_run;
  }
#pragma unroll
  for (int n = 0; n < NBD; ++n) {
    float* dst = red_o + (warp * 8 + row) * D + n * 8 + (lane & 3) * 2;
    dst[0] = o[n][0];
    dst[1] = o[n][1];
  }
  __syncthreads();
  for (int i = tid; i < G * D; i += TC_THREADS) {
    const int g = i / D, d = i % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, red_m[w * 8 + g]);
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = red_m[w * 8 + g];
      if (mw != -INFINITY) v += red_o[(w * 8 + g) * D + d] * exp2f(mw - M);
    }
    const long long base = (((long long)b * Hq + hk * G + g) * splits + sp_idx);
    acc_out[base * D + d] = v;
  }
  if (tid < G) {
    const int g = tid;
    float M = -INFINITY, L = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, red_m[w * 8 + g]);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = red_m[w * 8 + g];
      if (mw != -INFINITY) L += red_l[w * 8 + g] * exp2f(mw - M);
    }
    const long long base = (((long long)b * Hq + hk * G + g) * splits + sp_idx);
    ml_out[base * 2] = M * 0.6931471805599453f;      // back to natural-log units for the combine kernel
    ml_out[base * 2 + 1] = L;
  }
}

template <int MODE, int D>
static int launch_decode_mma(dim3 grid, cudaStream_t st, const __nv_bfloat16* q, long long ldq, KvPool k, KvPool v, const int* bt,
                             int max_pages, const int* lens, float* acc, float* ml, int Hq, int Hkv, int G, int splits, float scale,
                             int* status) {
  constexpr int SMEM = (16 + (TC_THREADS / 32) * 2 * TC_CHUNK) * (D * 2 + 16) + 128;   // Q tile, four K/V tile pairs, barriers
  static_assert(SMEM >= int(sizeof(float)) * (64 + 4 * 8 * D), "the merge buffers reuse the staging area");
  static DeviceOnce once;
  auto kern = paged_decode_mma_kernel<MODE, D>;
  if (int e = ensure_dyn_smem(once, kern, SMEM)) return e;
  tfb::launch_k(kern, grid, TC_THREADS, SMEM, st, q, ldq, k, v, bt, max_pages, lens, acc, ml, Hq, Hkv, G, splits, scale, status);
  return int(cudaGetLastError());
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
// status: the device status word (a bulk copy that does not land within the wait bound is reported there).
TFB_API int tfb_paged_decode(const void* q, long long ldq, void* k_data, void* k_scale, void* v_data, void* v_scale,
                             const int* block_table, int max_pages, const int* seq_lens, void* o, long long ldo,
                             float* acc_ws, float* ml_ws, int B, int Hq, int Hkv, int D, int splits, int mode,
                             float scale, long long pool_rows, int* status, void* stream) {
  if ((D != 64 && D != 128) || Hkv <= 0 || Hq % Hkv || splits < 1) return TFB_ERR_ARG;
  const int G = Hq / Hkv;
  KvPool kp{k_data, k_scale, pool_rows}, vp{v_data, v_scale, pool_rows};
  dim3 grid(B, Hkv, splits);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto Q = static_cast<const __nv_bfloat16*>(q);
  int rc;
  // tensor-core kernel by default (up to 8 query heads per kv head, q rows 16-byte aligned); TFB_PAGED_DECODE=simt
  // selects the CUDA-core kernel
  static const bool simt = [] { const char* e = getenv("TFB_PAGED_DECODE"); return e && !strcmp(e, "simt"); }();
  const bool mma_ok = !simt && G <= 8 && (ldq % 8) == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0;
#define TFB_GO(MODE)                                                                                                  \
  rc = mma_ok ? ((D == 64) ? launch_decode_mma<MODE, 64>(grid, st, Q, ldq, kp, vp, block_table, max_pages, seq_lens, acc_ws, ml_ws, \
                                                         Hq, Hkv, G, splits, scale, status)                           \
                           : launch_decode_mma<MODE, 128>(grid, st, Q, ldq, kp, vp, block_table, max_pages, seq_lens, acc_ws,       \
                                                          ml_ws, Hq, Hkv, G, splits, scale, status))                  \
     : (D == 64) ? launch_decode_g<MODE, 64>(G, grid, st, Q, ldq, kp, vp, block_table, max_pages, seq_lens, acc_ws,   \
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
