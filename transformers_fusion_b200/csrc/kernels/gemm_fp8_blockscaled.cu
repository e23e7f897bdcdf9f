// Block-scaled FP8 (E4M3) GEMM for sm_100a with DeepSeek-style scaling granularity:
//   A [M,K] e4m3, one fp32 scale per row per 128 K-elements   (sa [M, K/128])
//   B [N,K] e4m3, one fp32 scale per 128 x 128 block           (sb [N/128, K/128])
//   C [M,N] bf16 = sum_kb  sa[m,kb] * sb[n/128,kb] * (A_kb . B_kb^T)
// optionally grouped: rows of A belong to experts (row ranges padded to 128, offsets on the device),
// B / sb carry a leading expert dimension.
//
// tcgen05.mma kind::f8f6f4 has no notion of these scales, so the product of every 128-wide K block is
// left un-accumulated in a TMEM partial buffer (two buffers alternate) and the epilogue warps promote
// it into fp32 register accumulators with the two scales while the tensor core works on the next
// block.  Tiles are 128 x 128 x 128; operands arrive by TMA with the 128-byte swizzle (128 fp8 = one
// swizzle row).
//
// The reference has no block-scaled FP8 GEMM: its fp8 path is elementwise quantise + fp32 accumulate
// (src/math/simd_math.cpp fp8_gemm) and a block-fp8 importer (src/adapters/include/adapters/safetensors_bridge.h:28-45).
#include "tfb_host.h"
#include "tfb_ptx.cuh"

namespace tfb {

constexpr int F8_BM = 128, F8_BN = 128, F8_BK = 128;
constexpr int F8_STAGES = 6;
constexpr int F8_THREADS = 192;
constexpr int F8_TILE = 128 * 128;  // bytes per operand tile

struct F8Params {
  int M, N, K;
  __nv_bfloat16* C;
  long long ldc;
  const float* sa;   // [M, kblocks]
  const float* sb;   // [experts, N/128 (ceil), kblocks]
  int tiles_m, tiles_n, kblocks;
  const int* expert_of_mtile;  // grouped mode: expert index of every 128-row tile (null = dense)
  int* status;
};

struct F8Smem {
  static constexpr int STAGE = 2 * F8_TILE;
  static constexpr int BAR_OFF = F8_STAGES * STAGE;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap ta, const __grid_constant__ CUtensorMap tb, const F8Params p) {
  tfb::pdl_sync();
  using L = F8Smem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + F8_STAGES * 8;
  const uint32_t bar_pfull = bar_empty + F8_STAGES * 8;  // [2] partial product ready
  const uint32_t bar_pempty = bar_pfull + 16;            // [2] partial product consumed (128 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * F8_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < F8_STAGES; ++s) {
      mbar_init(bar_full + s * 8, 1);
      mbar_init(bar_empty + s * 8, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_pfull + b * 8, 1);
      mbar_init(bar_pempty + b * 8, 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int mt = t / p.tiles_n, nt = t % p.tiles_n;
        const int e = p.expert_of_mtile ? p.expert_of_mtile[mt] : 0;
        if (e < 0) continue;  // padding tile of the grouped layout
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait(bar_empty + stage * 8, phase ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          const uint32_t fb = bar_full + stage * 8;
          mbar_expect_tx(fb, L::STAGE);
          const uint32_t sa = sbase + stage * L::STAGE;
          tma_load_2d(sa, &ta, fb, kb * F8_BK, mt * F8_BM);
          tma_load_3d(sa + F8_TILE, &tb, fb, kb * F8_BK, nt * F8_BN, e);
          if (++stage == F8_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(FMT_E4M3, FMT_E4M3, false, false, F8_BM, F8_BN);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t pcount = 0;  // running count of partial products, selects buffer and parity
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int mt = t / p.tiles_n;
        if (p.expert_of_mtile && p.expert_of_mtile[mt] < 0) continue;
        for (int kb = 0; kb < p.kblocks; ++kb, ++pcount) {
          const int pb = pcount & 1;
          if (!mbar_wait(bar_pempty + pb * 8, ((pcount >> 1) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
          if (!mbar_wait(bar_full + stage * 8, phase, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = sbase + stage * L::STAGE, sb = sa + F8_TILE;
#pragma unroll
          for (int k = 0; k < F8_BK / 32; ++k)
            umma_f8f6f4_ss(tmem_base + pb * 128, umma_smem_desc(sa + k * 32, 16, 1024),
                           umma_smem_desc(sb + k * 32, 16, 1024), idesc, k > 0);
          umma_commit(bar_empty + stage * 8);
          umma_commit(bar_pfull + pb * 8);
          if (++stage == F8_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else {
    const int quad = warp & 3;
    const uint32_t lane_off = uint32_t(quad * 32) << 16;
    uint32_t pcount = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const int mt = t / p.tiles_n, nt = t % p.tiles_n;
      const int e = p.expert_of_mtile ? p.expert_of_mtile[mt] : 0;
      if (e < 0) continue;
      const int row = mt * F8_BM + quad * 32 + lane;
      const bool row_ok = row < p.M;
      const float* sa_row = p.sa + (long long)(row_ok ? row : 0) * p.kblocks;
      const float* sb_row = p.sb + ((long long)e * ((p.N + 127) / 128) + nt) * p.kblocks;
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.f;
      bool ok = true;
      for (int kb = 0; kb < p.kblocks; ++kb, ++pcount) {
        const int pb = pcount & 1;
        if (!mbar_wait_warp(bar_pfull + pb * 8, (pcount >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const float s = sa_row[kb] * sb_row[kb];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + pb * 128 + lane_off + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c * 32 + i] = fmaf(__uint_as_float(v[i]), s, acc[c * 32 + i]);
        }
        tc_fence_before();
        mbar_arrive(bar_pempty + pb * 8);
      }
      if (!ok) break;
      if (row_ok) {
        __nv_bfloat16* cp = p.C + (long long)row * p.ldc + nt * F8_BN;
        const int ncols = min(F8_BN, p.N - nt * F8_BN);
        if (ncols == F8_BN && (p.ldc & 7) == 0) {
#pragma unroll
          for (int q = 0; q < 16; ++q) {
            uint4 u;
            u.x = pack_bf16(acc[q * 8 + 0], acc[q * 8 + 1]);
            u.y = pack_bf16(acc[q * 8 + 2], acc[q * 8 + 3]);
            u.z = pack_bf16(acc[q * 8 + 4], acc[q * 8 + 5]);
            u.w = pack_bf16(acc[q * 8 + 6], acc[q * 8 + 7]);
            *reinterpret_cast<uint4*>(cp + q * 8) = u;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (i < ncols) cp[i] = __float2bfloat16(acc[i]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// ------------------------------------------------------------------------------------------------
// quantisers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint8_t f32_to_e4m3(float x) {
  // saturating round-to-nearest-even conversion (max finite 448, no infinities)
  uint16_t r;
  asm("{\n\t.reg .b16 t;\n\tcvt.rn.satfinite.e4m3x2.f32 t, %1, %2;\n\tmov.b16 %0, t;\n\t}" : "=h"(r) : "f"(0.f), "f"(x));
  return uint8_t(r & 0xff);
}

// x [rows, K] bf16 -> q [rows, K] e4m3 + scale [rows, K/128] fp32 (amax / 448 per 1x128 block); one warp per block
__global__ void quant_fp8_1x128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                       float* __restrict__ scale, long long rows, int K) {
  tfb::pdl_sync();
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int kblocks = (K + 127) / 128;
  if (w >= rows * kblocks) return;
  const long long r = w / kblocks;
  const int kb = int(w % kblocks);
  const int c = kb * 128 + lane * 4;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (c + 3 < K) {
    const uint2 u = *reinterpret_cast<const uint2*>(x + r * K + c);
    const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  } else {
    for (int i = 0; i < 4; ++i)
      if (c + i < K) v[i] = __bfloat162float(x[r * K + c + i]);
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float s = amax > 0.f ? amax / 448.f : 1.f;
  const float inv = 1.f / s;
  if (lane == 0) scale[r * kblocks + kb] = s;
  uint32_t packed = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) packed |= uint32_t(f32_to_e4m3(v[i] / s)) << (8 * i);
  if (c + 3 < K) *reinterpret_cast<uint32_t*>(q + r * K + c) = packed;
  else
    for (int i = 0; i < 4; ++i)
      if (c + i < K) q[r * K + c + i] = uint8_t(packed >> (8 * i));
}

// w [N, K] bf16 -> q e4m3 + scale [ceil(N/128), ceil(K/128)] fp32 (amax / 448 per 128x128 block); one CTA per block
__global__ void __launch_bounds__(256) quant_fp8_128x128_kernel(const __nv_bfloat16* __restrict__ w,
                                                                uint8_t* __restrict__ q, float* __restrict__ scale,
                                                                int N, int K) {
  tfb::pdl_sync();
  __shared__ float red[8];
  const int kb = blockIdx.x, nb = blockIdx.y;
  const int kblocks = gridDim.x;
  float amax = 0.f;
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int n = nb * 128 + i / 128, k = kb * 128 + i % 128;
    if (n < N && k < K) amax = fmaxf(amax, fabsf(__bfloat162float(w[(long long)n * K + k])));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float s = amax > 0.f ? amax / 448.f : 1.f;
  const float inv = 1.f / s;
  if (threadIdx.x == 0) scale[(long long)nb * kblocks + kb] = s;
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int n = nb * 128 + i / 128, k = kb * 128 + i % 128;
    if (n < N && k < K) q[(long long)n * K + k] = f32_to_e4m3(__bfloat162float(w[(long long)n * K + k]) / s);
  }
}

}  // namespace tfb

using namespace tfb;

// C[M,N] bf16 = blockscaled(A e4m3 [M,K], sa [M,K/128]) x blockscaled(B e4m3 [E,N,K], sb [E,N/128,K/128])^T.
// Dense: experts = 1, expert_of_mtile = null.  Grouped: A rows are expert segments padded to multiples of
// 128 rows; expert_of_mtile[i] (device int32, M/128 entries) names the expert of row tile i (-1 = skip).
TFB_API int tfb_gemm_fp8_blockscaled(const void* A, const float* sa, const void* B, const float* sb, void* C,
                                     long long ldc, int M, int N, int K, int experts, const int* expert_of_mtile,
                                     int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (K & 15) || experts < 1) return TFB_ERR_ARG;
  CUtensorMap ta, tb;
  int rc;
  if ((rc = make_tmap_2d(&ta, A, 1, K, M, K, F8_BK, F8_BM))) return rc;
  if ((rc = make_tmap_3d(&tb, B, 1, K, N, experts, K, (unsigned long long)K * N, F8_BK, F8_BN, 1))) return rc;
  F8Params p;
  p.M = M; p.N = N; p.K = K;
  p.C = static_cast<__nv_bfloat16*>(C); p.ldc = ldc; p.sa = sa; p.sb = sb;
  p.tiles_m = (M + F8_BM - 1) / F8_BM; p.tiles_n = (N + F8_BN - 1) / F8_BN; p.kblocks = (K + F8_BK - 1) / F8_BK;
  p.expert_of_mtile = expert_of_mtile; p.status = status;
  static DeviceOnce once;
  if (int e = ensure_dyn_smem(once, gemm_fp8_kernel, F8Smem::TOTAL)) return e;
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  tfb::launch_k(gemm_fp8_kernel, grid, F8_THREADS, F8Smem::TOTAL, static_cast<cudaStream_t>(stream), ta, tb, p);
  return int(cudaGetLastError());
}

TFB_API int tfb_quant_fp8_1x128(const void* x, void* q, float* scale, long long rows, int K, void* stream) {
  if (K % 4) return TFB_ERR_ARG;
  const long long warps = rows * ((K + 127) / 128);
  const long long blocks = (warps * 32 + 255) / 256;
  tfb::launch_k(quant_fp8_1x128_kernel, (unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), scale, rows, K);
  return int(cudaGetLastError());
}

TFB_API int tfb_quant_fp8_128x128(const void* w, void* q, float* scale, int N, int K, void* stream) {
  dim3 g((K + 127) / 128, (N + 127) / 128);
  tfb::launch_k(quant_fp8_128x128_kernel, g, 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const __nv_bfloat16*>(w), static_cast<uint8_t*>(q), scale, N, K);
  return int(cudaGetLastError());
}
