// GEMM with quantised weights dequantised inside the kernel: C[M, N] = A[M, K] (bf16) * dequant(Wq)[N, K]^T.
// The weights stay at 8, 4 or 2 bits per element in HBM; the bf16 image of a weight tile exists only in shared memory.
//
// Weight formats (all with one scale per `group` = 32 or 64 consecutive k of a row, scales stored as bf16):
//   0 int8 symmetric         value = s8 * scale
//   1 int4 symmetric         value = (u4 - 8) * scale            two codes per byte, low nibble first
//   2 fp8 e4m3               value = e4m3 * scale                 (MXFP8 when the scales are powers of two and group = 32)
//   3 fp4 e2m1               value = e2m1 * scale                 (MXFP4 / NVFP4-style), two codes per byte
//   4 ternary                value = (u2 - 1) * scale             four codes per byte: {-1, 0, +1}
// Device layout ("tile-major", produced by quant/wq.py at load time): tiles of 128 weight rows x 64 k.  Tile (nb, kb) is one
// contiguous blob of 128 * row_bytes bytes at (nb * KB + kb) * 128 * row_bytes; inside it the rows are cut into units of
// U = min(16, row_bytes / 2) bytes and stored unit-major: unit u of row r at ((u * 128) + r) * U, so that the 32 lanes of a
// warp (32 consecutive rows) read consecutive addresses of shared memory.  Scales: [(nb * KB + kb) * 128 + r][64 / group].
//
// One persistent CTA per SM, 480 threads:
//   warp 0       TMA producer of the activation tiles (128 rows x 64 k, zero-filled past M), 3-stage ring with the B tiles
//   warp 1       MMA issuer (tcgen05.mma 128 x 128 x 16, accumulator in TMEM, double-buffered)
//   warps 2-9    dequantisers: thread (row r, half h) turns 32 codes of one weight row into bf16 and stores them into the
//                B tile in the 128-byte-swizzled K-major layout the MMA descriptor expects, then fence.proxy.async + arrive
//   warps 10-13  epilogue: TMEM -> registers -> bf16 store (+ bias), or fp32 atomic accumulation for split-K
//   warp 14      bulk-copy producer of the packed codes and scales (one contiguous blob per tile), 8-stage ring: the
//                weight stream stays ~68 KB per SM deep in flight, independent of the pace of the dequantisers
// Small-M (decode) problems are weight-bandwidth bound; split-K spreads the few N tiles over all SMs.
//
// Reference counterparts: the CPU quantised matmul kernels (src/kernel/kernel_quant8.cpp, kernel_quant4.cpp, kernel_tl.cpp
// ternary lookup, kernel_q3 / q6 / q12 / q24), INT8Inference / FP8Inference (src/inference/inference_lowprec.cpp).
#include "tfb_host.h"
#include "tfb_ptx.cuh"

namespace tfb {

constexpr int WQ_BM = 128, WQ_BN = 128, WQ_BK = 64, WQ_STAGES = 3, WQ_RAW_STAGES = 8, WQ_THREADS = 480, WQ_DQ_THREADS = 256;
constexpr int WQ_A_BYTES = WQ_BM * WQ_BK * 2, WQ_B_BYTES = WQ_BN * WQ_BK * 2, WQ_STAGE = WQ_A_BYTES + WQ_B_BYTES;
constexpr int WQ_RAW_CODES = 128 * 64, WQ_RAW_STAGE = WQ_RAW_CODES + 128 * 2 * 2;     // codes (<= 8 KB) + scales (<= 512 B)
constexpr int WQ_RAW_OFF = WQ_STAGES * WQ_STAGE;
constexpr int WQ_BAR_OFF = WQ_RAW_OFF + WQ_RAW_STAGES * WQ_RAW_STAGE;
constexpr int WQ_SMEM = WQ_BAR_OFF + 512 + 1024;

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

__host__ __device__ constexpr int wq_row_bytes(int fmt) { return fmt == 0 || fmt == 2 ? 64 : (fmt == 4 ? 16 : 32); }

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 ld_shared_v2(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t ld_shared_u16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
// two e4m3 bytes (low 16 bits of v) -> two floats, through the hardware e4m3x2 -> f16x2 conversion
__device__ __forceinline__ float2 e4m3x2_to_f2(uint32_t v) {
  uint32_t h2;
  const uint16_t lo = uint16_t(v);
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(lo));
  return __half22float2(*reinterpret_cast<const __half2*>(&h2));
}

// Loads the codes of 32 consecutive k of one weight row (half h of row r) from the staged blob into registers.
template <int FMT>
__device__ __forceinline__ void wq_load_codes(uint32_t raw, int r, int h, uint32_t (&w)[8]) {
  if (FMT == 0 || FMT == 2) {                      // 64-byte rows, 4 units of 16 bytes: units 2h, 2h + 1
    const uint4 a = ld_shared_v4(raw + ((2 * h) * 128 + r) * 16), b = ld_shared_v4(raw + ((2 * h + 1) * 128 + r) * 16);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
  } else if (FMT == 1 || FMT == 3) {               // 32-byte rows, 2 units of 16 bytes: unit h
    const uint4 a = ld_shared_v4(raw + (h * 128 + r) * 16);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
  } else {                                         // 16-byte rows, 2 units of 8 bytes: unit h
    const uint2 a = ld_shared_v2(raw + (h * 128 + r) * 8);
    w[0] = a.x; w[1] = a.y;
  }
}

// Decodes the 32 codes held in w, scales them and packs them as 16 bf16x2 words in k order.  `sbits` is the bf16 scale.
// Every path yields exactly round_to_bf16(code_value * scale), the value the fp32 oracle computes:
//   int8     the byte (biased by 128) is placed in byte 1 of 0x47000000, which reads as the float 2^15 + u; one FMA with
//            the scale and the constant -(2^15 + 128) * scale (exact: 257 * 128 times an 8-bit mantissa) gives b * scale
//   int4 / ternary   the code is OR-ed into the bf16 128.0 (0x4300 | u = 128 + u exactly), a packed bf16 subtract removes
//            128 + zero_point and a packed bf16 multiply applies the scale: two values per instruction, no final pack
template <int FMT>
__device__ __forceinline__ void wq_convert(const uint32_t (&w)[8], uint32_t sbits, uint32_t (&o)[16]) {
  const float s = __uint_as_float(sbits << 16);
  const uint32_t s2u = sbits | (sbits << 16);
  const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162*>(&s2u);
  auto bf2 = [&](uint32_t magic_or_codes, uint32_t offset_bits) -> uint32_t {
    const __nv_bfloat162 v = __hmul2(__hsub2(*reinterpret_cast<const __nv_bfloat162*>(&magic_or_codes),
                                             *reinterpret_cast<const __nv_bfloat162*>(&offset_bits)), s2);
    return *reinterpret_cast<const uint32_t*>(&v);
  };
  if (FMT == 0) {
    const float c = -32896.f * s;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t x = w[i] ^ 0x80808080u;
      const float f0 = fmaf(__uint_as_float(__byte_perm(x, 0x47000000u, 0x7504)), s, c);
      const float f1 = fmaf(__uint_as_float(__byte_perm(x, 0x47000000u, 0x7514)), s, c);
      const float f2 = fmaf(__uint_as_float(__byte_perm(x, 0x47000000u, 0x7524)), s, c);
      const float f3 = fmaf(__uint_as_float(__byte_perm(x, 0x47000000u, 0x7534)), s, c);
      o[2 * i] = pack_bf16(f0, f1);
      o[2 * i + 1] = pack_bf16(f2, f3);
    }
  } else if (FMT == 1) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t lo = w[i] & 0x0F0F0F0Fu, hi = (w[i] >> 4) & 0x0F0F0F0Fu;   // even / odd k, one code per byte
      o[4 * i + 0] = bf2((__byte_perm(lo, hi, 0x0400) & 0x00FF00FFu) | 0x43004300u, 0x43084308u);
      o[4 * i + 1] = bf2((__byte_perm(lo, hi, 0x0501) & 0x00FF00FFu) | 0x43004300u, 0x43084308u);
      o[4 * i + 2] = bf2((__byte_perm(lo, hi, 0x0602) & 0x00FF00FFu) | 0x43004300u, 0x43084308u);
      o[4 * i + 3] = bf2((__byte_perm(lo, hi, 0x0703) & 0x00FF00FFu) | 0x43004300u, 0x43084308u);
    }
  } else if (FMT == 2) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float2 a = e4m3x2_to_f2(w[i]), b = e4m3x2_to_f2(w[i] >> 16);
      o[2 * i] = pack_bf16(a.x * s, a.y * s);
      o[2 * i + 1] = pack_bf16(b.x * s, b.y * s);
    }
  } else if (FMT == 3) {
    // e2m1 nibble s|ee|m placed as an fp16 with exponent field ee and top mantissa bit m is the value / 2^14
    // (zero, the subnormal 0.5 and the normals alike), so one multiply by 2^14 * scale finishes the job
    const float s14 = s * 16384.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t t = w[i] >> (8 * j);
        const uint32_t y = (t & 0xFu) | ((t & 0xF0u) << 12);                     // nibbles at bits 0-3 and 16-19
        const uint32_t h2 = ((y & 0x00070007u) << 9) | ((y & 0x00080008u) << 12);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
        o[4 * i + j] = pack_bf16(f.x * s14, f.y * s14);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      // stream m holds the codes k = 4 * byte + m, one per byte
      const uint32_t c0 = w[i] & 0x03030303u, c1 = (w[i] >> 2) & 0x03030303u, c2 = (w[i] >> 4) & 0x03030303u, c3 = (w[i] >> 6) & 0x03030303u;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t sel = uint32_t(((4 + j) << 8) | j);
        o[8 * i + 2 * j] = bf2((__byte_perm(c0, c1, sel) & 0x00FF00FFu) | 0x43004300u, 0x43014301u);
        o[8 * i + 2 * j + 1] = bf2((__byte_perm(c2, c3, sel) & 0x00FF00FFu) | 0x43004300u, 0x43014301u);
      }
    }
  }
}

template <int FMT>
__global__ void __launch_bounds__(WQ_THREADS, 1) gemm_wq_kernel(const __grid_constant__ CUtensorMap tma_a, const WqParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + WQ_BAR_OFF);
  const uint32_t bar_full = smem_u32(bars);                     // [S]  1 TMA arrive (+tx) + 256 dequant arrivals
  const uint32_t bar_empty = bar_full + WQ_STAGES * 8;          // [S]  MMA commit
  const uint32_t bar_rfull = bar_empty + WQ_STAGES * 8;         // [R]  bulk copies of codes + scales (tx)
  const uint32_t bar_rempty = bar_rfull + WQ_RAW_STAGES * 8;    // [R]  256 dequant arrivals (codes are in registers)
  const uint32_t bar_tfull = bar_rempty + WQ_RAW_STAGES * 8;    // [2]
  const uint32_t bar_tempty = bar_tfull + 16;                   // [2]  128 arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * WQ_STAGES + 2 * WQ_RAW_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int RB = wq_row_bytes(FMT);
  const int spr = WQ_BK / p.group;                              // scales per row per k-block
  const uint32_t code_bytes = 128 * RB, scale_bytes = 128 * spr * 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < WQ_STAGES; ++s) {
      mbar_init(bar_full + s * 8, 1 + WQ_DQ_THREADS / 32);
      mbar_init(bar_empty + s * 8, 1);
    }
    for (int s = 0; s < WQ_RAW_STAGES; ++s) {
      mbar_init(bar_rfull + s * 8, 1);
      mbar_init(bar_rempty + s * 8, WQ_DQ_THREADS / 32);
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
  // after a timed-out wait the issuing thread lets its copies in flight land before the CTA exits
  auto drain = [&]() {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {}
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
      if (!ok) drain();
    }
  } else if (warp == 14) {
    if (lane == 0) {
      int rs = 0;
      uint32_t rphase = 0;
      bool ok = true;
      for (int w = cta; w < num_work && ok; w += nctas) {
        int m0, nb, kb0, kb1;
        decode(w, m0, nb, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(bar_rempty + rs * 8, rphase ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          const long long tile = (long long)nb * KB + kb;
          const uint32_t rb_ = bar_rfull + rs * 8, dst = smem_base + WQ_RAW_OFF + rs * WQ_RAW_STAGE;
          mbar_expect_tx(rb_, code_bytes + scale_bytes);
          bulk_load_1d(dst, p.wq + tile * code_bytes, code_bytes, rb_);
          bulk_load_1d(dst + WQ_RAW_CODES, p.scales + tile * (128 * spr), scale_bytes, rb_);
          if (++rs == WQ_RAW_STAGES) { rs = 0; rphase ^= 1; }
        }
      }
      if (!ok) drain();
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
  } else if (warp < 10) {
    // ------------------------------ dequantisers: 32 k of one weight row per thread ------------------------------
    const int t = threadIdx.x - 64, r = t & 127, h = t >> 7;
    const uint32_t scale_off = WQ_RAW_CODES + (p.group == 32 ? (r * 2 + h) * 2 : r * 2);
    const uint32_t xr = uint32_t(r & 7);
    int stage = 0, rs = 0;
    uint32_t phase = 0, rphase = 0;
    bool ok = true;
    for (int w = cta; w < num_work && ok; w += nctas) {
      int m0, nb, kb0, kb1;
      decode(w, m0, nb, kb0, kb1);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait_warp(bar_rfull + rs * 8, rphase, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
        const uint32_t raw = smem_base + WQ_RAW_OFF + rs * WQ_RAW_STAGE;
        uint32_t wd[8];
        wq_load_codes<FMT>(raw, r, h, wd);
        const uint32_t sbits = ld_shared_u16(raw + scale_off);
        __syncwarp();                                        // every lane holds its codes: one arrival per warp
        if (lane == 0) mbar_arrive(bar_rempty + rs * 8);
        if (++rs == WQ_RAW_STAGES) { rs = 0; rphase ^= 1; }
        uint32_t o[16];
        wq_convert<FMT>(wd, sbits, o);
        if (!mbar_wait_warp(bar_empty + stage * 8, phase ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
        const uint32_t row_smem = smem_base + stage * WQ_STAGE + WQ_A_BYTES + r * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c)
          st_shared_v4(row_smem + ((uint32_t(4 * h + c) ^ xr) << 4), o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_full + stage * 8);
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
      // rows past M hold zeros: a warp whose 32 rows are all past M only releases the accumulator
      if (m0 + quad * 32 < p.M) {
#pragma unroll 1
        for (int c = 0; c < WQ_BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(taddr0 + c * 32, v);
          tmem_ld_wait();
          const int col0 = nb * WQ_BN + c * 32;
          if (row >= p.M || col0 >= p.N) continue;
          // N is a multiple of 128 and ldc of 8 (the packer pads), so every 32-column run is whole and 16-byte aligned
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
          if (p.bias && kb0 == 0) {
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] += __bfloat162float(p.bias[col0 + j]);
          }
          if (p.splits > 1) {
            float4* cp = reinterpret_cast<float4*>(static_cast<float*>(p.C) + (long long)row * p.ldc + col0);
#pragma unroll
            for (int j = 0; j < 8; ++j) atomicAdd(cp + j, make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]));
          } else {
            uint4* cp = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              cp[j] = make_uint4(pack_bf16(f[8 * j], f[8 * j + 1]), pack_bf16(f[8 * j + 2], f[8 * j + 3]), pack_bf16(f[8 * j + 4], f[8 * j + 5]),
                                 pack_bf16(f[8 * j + 6], f[8 * j + 7]));
          }
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
  if (M <= 0 || N <= 0 || K <= 0 || K % WQ_BK || N % WQ_BN || ldc % 8 || fmt < 0 || fmt > 4 || (group != 32 && group != 64)) return TFB_ERR_ARG;
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
  using Kern = void (*)(const CUtensorMap, const WqParams);
  static const Kern kerns[5] = {gemm_wq_kernel<0>, gemm_wq_kernel<1>, gemm_wq_kernel<2>, gemm_wq_kernel<3>, gemm_wq_kernel<4>};
  static bool configured = false;
  if (!configured) {
    for (Kern k : kerns) {
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, WQ_SMEM);
      if (e != cudaSuccess) return int(e);
    }
    configured = true;
  }
  const long long work = (long long)tiles * p.splits;
  const int grid = int(work < sms ? work : sms);
  kerns[fmt]<<<grid, WQ_THREADS, WQ_SMEM, static_cast<cudaStream_t>(stream)>>>(ta, p);
  const int rc = int(cudaGetLastError());
  return rc ? -1000 - rc : p.splits;
}
