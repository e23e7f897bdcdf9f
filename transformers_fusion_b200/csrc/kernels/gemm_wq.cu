// GEMM with quantised weights dequantised inside the kernel: C[M, N] = A[M, K] (bf16) * dequant(Wq)[N, K]^T.
// The weights stay at 8, 4 or 2 bits per element in HBM; the bf16 image of a weight tile exists only in shared memory.
//
// Weight formats (all with one scale per `group` = 32 or 64 consecutive k of a row, scales stored as bf16):
//   0 int8 symmetric         value = s8 * scale
//   1 int4 symmetric         value = (u4 - 8) * scale            two codes per byte, low nibble first
//   2 fp8 e4m3               value = e4m3 * scale                 (MXFP8 when the scales are powers of two and group = 32)
//   3 fp4 e2m1               value = e2m1 * scale                 (MXFP4 / NVFP4-style), two codes per byte
//   4 ternary                value = (u2 - 1) * scale             four codes per byte: {-1, 0, +1}
// Device layout ("tile-major", produced by quant/wq.py at load time): tiles of 128 weight rows x 64 k; tile (nb, kb) at
// ((nb * KB + kb) * 128 rows) * row_bytes, row r of the tile contiguous after row r - 1, so that the 128 dequantising
// threads (one weight row each) read one contiguous span per k-block.  Scales: [(nb * KB + kb) * 128 + r][64 / group].
//
// One persistent CTA per SM, 320 threads:
//   warp 0      TMA producer of the activation tiles (128 rows x 64 k, zero-filled past M)
//   warp 1      MMA issuer (tcgen05.mma 128 x 128 x 16, accumulator in TMEM, double-buffered)
//   warps 2-5   dequantisers: packed codes -> bf16 -> the B tile in shared memory, in the 128-byte-swizzled K-major
//               layout the MMA descriptor expects, then fence.proxy.async + mbarrier arrive
//   warps 6-9   epilogue: TMEM -> registers -> bf16 store (+ bias), or fp32 atomic accumulation for split-K
// Small-M (decode) problems are weight-bandwidth bound; split-K spreads the few N tiles over all SMs.
//
// Reference counterparts: the CPU quantised matmul kernels (src/kernel/kernel_quant8.cpp, kernel_quant4.cpp, kernel_tl.cpp
// ternary lookup, kernel_q3 / q6 / q12 / q24), INT8Inference / FP8Inference (src/inference/inference_lowprec.cpp).
#include "tfb_host.h"
#include "tfb_ptx.cuh"

namespace tfb {

constexpr int WQ_BM = 128, WQ_BN = 128, WQ_BK = 64, WQ_STAGES = 4, WQ_THREADS = 320;
constexpr int WQ_A_BYTES = WQ_BM * WQ_BK * 2, WQ_B_BYTES = WQ_BN * WQ_BK * 2, WQ_STAGE = WQ_A_BYTES + WQ_B_BYTES;
constexpr int WQ_BAR_OFF = WQ_STAGES * WQ_STAGE;
constexpr int WQ_SMEM = WQ_BAR_OFF + 256 + 1024;

struct WqParams {
  int M, N, K;
  const uint8_t* wq;                 // tile-major packed codes
  const __nv_bfloat16* scales;       // tile-major scales
  int fmt, group;
  void* C;                           // bf16 [M, ldc] (splits == 1) or fp32 [M, ldc] accumulated into (splits > 1)
  long long ldc;
  const __nv_bfloat16* bias;
  int tiles_m, tiles_n, splits, kb_per_split;
  int* status;
};

__device__ __forceinline__ int wq_row_bytes(int fmt) { return fmt == 0 || fmt == 2 ? 64 : (fmt == 4 ? 16 : 32); }

__device__ __forceinline__ float e4m3_to_f(uint32_t v) {
  // e4m3 -> half bits: sign | (exp + 8) << 10 | mant << 7 for normals; the half conversion below handles subnormals of
  // e4m3 (exp == 0) through the fp16 subnormal range scaled by 2^-6 * 2^... : use the exact arithmetic form instead
  const uint32_t s = v >> 7, e = (v >> 3) & 15, m = v & 7;
  const float mag = e == 0 ? float(m) * 0.001953125f : __uint_as_float(((e + 120u) << 23) | (m << 20));   // 2^-9 * m | 2^(e-7) * (1 + m/8)
  return s ? -mag : mag;
}
__device__ __forceinline__ float e2m1_to_f(uint32_t v) {
  // 0, 0.5, 1, 1.5, 2, 3, 4, 6 with a sign bit
  const uint32_t s = v >> 3, e = (v >> 1) & 3, m = v & 1;
  const float mag = e == 0 ? 0.5f * float(m) : __uint_as_float(((e + 126u) << 23) | (m << 22));
  return s ? -mag : mag;
}

// Decodes the 64 k-values of one weight row of one k-block and stores them as bf16 into the swizzled B tile.
__device__ __forceinline__ void wq_dequant_row(const uint8_t* __restrict__ src, const __nv_bfloat16* __restrict__ sc, int fmt,
                                               int group, uint32_t row_smem, uint32_t xr) {
  float s[2];
  s[0] = __bfloat162float(sc[0]);
  s[1] = group == 32 ? __bfloat162float(sc[1]) : s[0];
  if (fmt == 0 || fmt == 2) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {                       // 16 bytes = 16 values = two 16-byte chunks of bf16
      const uint4 u = *reinterpret_cast<const uint4*>(src + q * 16);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
      float f[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const uint32_t b = (w[j >> 2] >> ((j & 3) * 8)) & 255u;
        f[j] = (fmt == 0 ? float(int(int8_t(b))) : e4m3_to_f(b)) * s[q >> 1];
      }
#pragma unroll
      for (int h = 0; h < 2; ++h)
        st_shared_v4(row_smem + ((uint32_t(q * 2 + h) ^ xr) << 4), pack_bf16(f[h * 8 + 0], f[h * 8 + 1]), pack_bf16(f[h * 8 + 2], f[h * 8 + 3]),
                     pack_bf16(f[h * 8 + 4], f[h * 8 + 5]), pack_bf16(f[h * 8 + 6], f[h * 8 + 7]));
    }
  } else if (fmt == 1 || fmt == 3) {
#pragma unroll
    for (int q = 0; q < 2; ++q) {                       // 16 bytes = 32 values = four chunks
      const uint4 u = *reinterpret_cast<const uint4*>(src + q * 16);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t nib = (w[h] >> (j * 4)) & 15u;
          f[j] = (fmt == 1 ? float(int(nib) - 8) : e2m1_to_f(nib)) * s[q];
        }
        st_shared_v4(row_smem + ((uint32_t(q * 4 + h) ^ xr) << 4), pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]),
                     pack_bf16(f[6], f[7]));
      }
    }
  } else {
    const uint4 u = *reinterpret_cast<const uint4*>(src);   // 16 bytes = 64 two-bit codes
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int i = c * 8 + j;
        const uint32_t code = (w[i >> 4] >> ((i & 15) * 2)) & 3u;
        f[j] = float(int(code) - 1) * s[c >> 2];
      }
      st_shared_v4(row_smem + ((uint32_t(c) ^ xr) << 4), pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
    }
  }
}

__global__ void __launch_bounds__(WQ_THREADS, 1) gemm_wq_kernel(const __grid_constant__ CUtensorMap tma_a, const WqParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + WQ_BAR_OFF);
  const uint32_t bar_full = smem_u32(bars);                 // [S] 1 TMA arrive (+tx) + 128 dequant arrivals
  const uint32_t bar_empty = bar_full + WQ_STAGES * 8;      // [S]
  const uint32_t bar_tfull = bar_empty + WQ_STAGES * 8;     // [2]
  const uint32_t bar_tempty = bar_tfull + 16;               // [2] 128 arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * WQ_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < WQ_STAGES; ++s) {
      mbar_init(bar_full + s * 8, 129);
      mbar_init(bar_empty + s * 8, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + b * 8, 1);
      mbar_init(bar_tempty + b * 8, 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tma_a);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 2 * WQ_BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int KB = (p.K + WQ_BK - 1) / WQ_BK;
  const int num_work = p.tiles_m * p.tiles_n * p.splits;
  const int nctas = gridDim.x, cta = blockIdx.x;
  auto decode = [&](int w, int& m0, int& nb, int& kb0, int& kb1) {
    const int tile = w / p.splits, split = w - tile * p.splits;
    m0 = (tile % p.tiles_m) * WQ_BM;
    nb = tile / p.tiles_m;
    kb0 = split * p.kb_per_split;
    kb1 = min(KB, kb0 + p.kb_per_split);
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = cta; w < num_work && ok; w += nctas) {
        int m0, nb, kb0, kb1;
        decode(w, m0, nb, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(bar_empty + stage * 8, phase ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          const uint32_t fb = bar_full + stage * 8;
          mbar_expect_tx(fb, WQ_A_BYTES);
          tma_load_2d(smem_base + stage * WQ_STAGE, &tma_a, fb, kb * WQ_BK, m0);
          if (++stage == WQ_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(FMT_BF16, FMT_BF16, false, false, WQ_BM, WQ_BN);
      int stage = 0, abuf = 0;
      uint32_t phase = 0, aphase = 0;
      bool ok = true;
      for (int w = cta; w < num_work && ok; w += nctas) {
        int m0, nb, kb0, kb1;
        decode(w, m0, nb, kb0, kb1);
        if (kb1 <= kb0) continue;
        if (!mbar_wait(bar_tempty + abuf * 8, aphase ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + abuf * WQ_BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(bar_full + stage * 8, phase, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * WQ_STAGE, sb = sa + WQ_A_BYTES;
#pragma unroll
          for (int k = 0; k < WQ_BK / 16; ++k)
            umma_f16_ss(tmem_d, umma_smem_desc(sa + k * 32, 16, 1024), umma_smem_desc(sb + k * 32, 16, 1024), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          umma_commit(bar_empty + stage * 8);
          if (++stage == WQ_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(bar_tfull + abuf * 8);
        abuf ^= 1;
        if (abuf == 0) aphase ^= 1;
      }
    }
  } else if (warp < 6) {
    // ------------------------------ dequantisers: one weight row of the tile per thread ------------------------------
    const int r = (warp - 2) * 32 + lane;
    const int rb = wq_row_bytes(p.fmt), spr = WQ_BK / p.group;   // scales per row per k-block
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int w = cta; w < num_work && ok; w += nctas) {
      int m0, nb, kb0, kb1;
      decode(w, m0, nb, kb0, kb1);
      for (int kb = kb0; kb < kb1; ++kb) {
        const long long tile = (long long)nb * KB + kb;
        const uint8_t* src = p.wq + (tile * WQ_BN + r) * rb;
        const __nv_bfloat16* sc = p.scales + (tile * WQ_BN + r) * spr;
        // prefetch the codes before waiting for the stage: the wait is the long part
        if (!mbar_wait_warp(bar_empty + stage * 8, phase ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
        const uint32_t row_smem = smem_base + stage * WQ_STAGE + WQ_A_BYTES + r * 128;
        wq_dequant_row(src, sc, p.fmt, p.group, row_smem, uint32_t(r & 7));
        fence_proxy_async_smem();
        mbar_arrive(bar_full + stage * 8);
        if (++stage == WQ_STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int quad = warp & 3;
    int abuf = 0;
    uint32_t aphase = 0;
    for (int w = cta; w < num_work; w += nctas) {
      int m0, nb, kb0, kb1;
      decode(w, m0, nb, kb0, kb1);
      if (kb1 <= kb0) continue;
      if (!mbar_wait_warp(bar_tfull + abuf * 8, aphase, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const int row = m0 + quad * 32 + lane;
      const uint32_t taddr0 = tmem_base + abuf * WQ_BN + (uint32_t(quad * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < WQ_BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(taddr0 + c * 32, v);
        tmem_ld_wait();
        const int col0 = nb * WQ_BN + c * 32;
        if (row >= p.M || col0 >= p.N) continue;
        if (p.splits > 1) {
          float* cp = static_cast<float*>(p.C) + (long long)row * p.ldc + col0;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) atomicAdd(cp + j, __uint_as_float(v[j]) + ((p.bias && kb0 == 0) ? __bfloat162float(p.bias[col0 + j]) : 0.f));
        } else {
          __nv_bfloat16* cp = static_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) cp[j] = __float2bfloat16(__uint_as_float(v[j]) + (p.bias ? __bfloat162float(p.bias[col0 + j]) : 0.f));
        }
      }
      tc_fence_before();
      mbar_arrive(bar_tempty + abuf * 8);
      abuf ^= 1;
      if (abuf == 0) aphase ^= 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * WQ_BN);
  }
}

}  // namespace tfb

// A [M, lda] bf16 (K % 64 == 0, N % 128 == 0: the packer pads).  wq / scales in the tile-major layout described at the top.
// splits == 1: C bf16 [M, ldc]; splits > 1: C fp32 [M, ldc], accumulated into (zero it first).  splits == 0 picks a value
// that fills the SMs.  Returns the number of splits used (>= 1) or a negative error.
TFB_API int tfb_gemm_wq(const void* A, long long lda, const void* wq, const void* scales, int fmt, int group, void* C, long long ldc,
                        int M, int N, int K, const void* bias, int splits, int c_is_fp32, int* status, void* stream) {
  using namespace tfb;
  if (M <= 0 || N <= 0 || K <= 0 || K % WQ_BK || N % WQ_BN || fmt < 0 || fmt > 4 || (group != 32 && group != 64)) return TFB_ERR_ARG;
  CUtensorMap ta;
  if (int rc = make_tmap_2d(&ta, A, 2, K, M, lda * 2, WQ_BK, WQ_BM)) return rc;
  WqParams p;
  p.M = M; p.N = N; p.K = K;
  p.wq = static_cast<const uint8_t*>(wq);
  p.scales = static_cast<const __nv_bfloat16*>(scales);
  p.fmt = fmt; p.group = group;
  p.C = C; p.ldc = ldc;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.tiles_m = (M + WQ_BM - 1) / WQ_BM;
  p.tiles_n = N / WQ_BN;
  p.status = status;
  const int KB = K / WQ_BK, tiles = p.tiles_m * p.tiles_n, sms = sm_count();
  if (splits <= 0) {
    splits = c_is_fp32 ? std::max(1, std::min(sms / std::max(1, tiles), KB / 4)) : 1;
  }
  if (splits > 1 && !c_is_fp32) return TFB_ERR_ARG;
  if (splits == 1 && c_is_fp32) return TFB_ERR_ARG;
  p.kb_per_split = (KB + splits - 1) / splits;
  p.splits = (KB + p.kb_per_split - 1) / p.kb_per_split;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_wq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, WQ_SMEM);
    if (e != cudaSuccess) return int(e);
    configured = true;
  }
  const long long work = (long long)tiles * p.splits;
  const int grid = int(work < sms ? work : sms);
  gemm_wq_kernel<<<grid, WQ_THREADS, WQ_SMEM, static_cast<cudaStream_t>(stream)>>>(ta, p);
  const int rc = int(cudaGetLastError());
  return rc ? -1000 - rc : p.splits;
}
