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
// One persistent CTA per SM, 768 threads:
//   warp 0       TMA producer of the activation tiles (128 rows x 64 k, zero-filled past M), 4-stage ring with the B tiles
//   warp 1       MMA issuer (tcgen05.mma 128 x 128 x 16, accumulator in TMEM, double-buffered)
//   warp 2       bulk-copy producer of the packed codes and scales (one contiguous blob per tile), 8-stage ring: the
//                weight stream stays ~68 KB per SM deep in flight, independent of the pace of the dequantisers
//   warps 4-7    epilogue: TMEM -> registers -> bf16 store (+ bias), or fp32 vector atomics for split-K
//   Every role but the MMA issuer waits with mbar_wait_sleep: a polling warp takes issue slots from the warps that share
//   its scheduler, and the converters need those slots (they are the instruction-issue bound of this kernel).
//   warps 8-23   dequantisers in two groups of eight warps; group g takes the k-blocks with (index & 1) == g, so two
//                k-blocks are decoded at once and the latency of one (shared-memory round trips, proxy fence, barrier)
//                hides behind the other.  Thread (row r, half h) of a group turns 32 codes of one weight row into bf16
//                and stores them into the B tile in the 128-byte-swizzled K-major layout the MMA descriptor expects.
// Inside a 32-bit word of 4-bit codes, nibble j holds element 2j and nibble j + 4 element 2j + 1 (j < 4), so that
// (word >> 4j) & 0x000F000F is the bf16x2-aligned pair (2j, 2j + 1); 2-bit codes likewise: field j = element 2j, field
// j + 8 = element 2j + 1 (j < 8).
// Small-M (decode) problems are weight-bandwidth bound; split-K spreads the few N tiles over all SMs.
//
// Reference counterparts: the CPU quantised matmul kernels (src/kernel/kernel_quant8.cpp, kernel_quant4.cpp, kernel_tl.cpp
// ternary lookup, kernel_q3 / q6 / q12 / q24), INT8Inference / FP8Inference (src/inference/inference_lowprec.cpp).
#include <algorithm>
#include "tfb_host.h"
#include "tfb_ptx.cuh"

namespace tfb {

constexpr int WQ_BM = 128, WQ_BN = 128, WQ_BK = 64, WQ_RAW_STAGES = 8, WQ_THREADS = 768, WQ_DQ_THREADS = 256;
constexpr int WQ_B_BYTES = WQ_BN * WQ_BK * 2;
constexpr int WQ_RAW_CODES = 128 * 64, WQ_RAW_STAGE = WQ_RAW_CODES + 128 * 2 * 2;     // codes (<= 8 KB) + scales (<= 512 B)
// Shared-memory plan for an activation tile of AROWS real rows.  With AROWS = 16 (decode batches) the activation tile is two
// 8-row swizzle groups (2 KB) and the product is issued with swapped operands (weights on the M side, batch on the N = 16
// side).  The small tile doubles the ring depth, which covers the commit -> refill round trip when the MMAs are short.
template <int AROWS>
struct WqPlan {
  static constexpr int STAGES = AROWS == 16 ? 8 : 4;
  static constexpr int A_BYTES = AROWS * WQ_BK * 2;
  static constexpr int STAGE = A_BYTES + WQ_B_BYTES;
  static constexpr int RAW_OFF = STAGES * STAGE;
  static constexpr int BAR_OFF = RAW_OFF + WQ_RAW_STAGES * WQ_RAW_STAGE;
  static constexpr int SMEM = BAR_OFF + 512 + 1024;
};

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
#pragma unroll
      for (int j = 0; j < 4; ++j) o[4 * i + j] = bf2(((w[i] >> (4 * j)) & 0x000F000Fu) | 0x43004300u, 0x43084308u);
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
        const uint32_t y = (w[i] >> (4 * j)) & 0x000F000Fu;
        const uint32_t h2 = ((y & 0x00070007u) << 9) | ((y & 0x00080008u) << 12);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
        o[4 * i + j] = pack_bf16(f.x * s14, f.y * s14);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[8 * i + j] = bf2(((w[i] >> (2 * j)) & 0x00030003u) | 0x43004300u, 0x43014301u);
    }
  }
}

template <int FMT, int AROWS>
__global__ void __launch_bounds__(WQ_THREADS, 1) gemm_wq_kernel(const __grid_constant__ CUtensorMap tma_a, const WqParams p) {
  tfb::pdl_sync();
  using PL = WqPlan<AROWS>;
  constexpr int WQ_STAGES = PL::STAGES, WQ_A_BYTES = PL::A_BYTES, WQ_STAGE = PL::STAGE, WQ_RAW_OFF = PL::RAW_OFF, WQ_BAR_OFF = PL::BAR_OFF;
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
          if (!mbar_wait_sleep(bar_empty + stage * 8, phase ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY, 32)) { ok = false; break; }
          const uint32_t fb = bar_full + stage * 8;
          mbar_expect_tx(fb, WQ_A_BYTES);
          tma_load_2d(smem_base + stage * WQ_STAGE, &tma_a, fb, kb * WQ_BK, m0);
          if (++stage == WQ_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) drain();
    }
  } else if (warp == 2) {
    if (lane == 0) {
      int rs = 0;
      uint32_t rphase = 0;
      bool ok = true;
      for (int w = cta; w < num_work && ok; w += nctas) {
        int m0, nb, kb0, kb1;
        decode(w, m0, nb, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_sleep(bar_rempty + rs * 8, rphase ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY, 32)) { ok = false; break; }
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
      // AROWS == 16 (decode): operands swapped, D^T[n, m] = W[n, :] . X[m, :]: the 128 weight rows of the tile are the M side
      // of the instruction and the batch its N = 16 side, so an MMA costs an eighth of the 128 x 128 form and the k-block is
      // no longer bounded below by tensor time
      constexpr bool SWAP = AROWS == 16;
      constexpr uint32_t idesc = umma_idesc(FMT_BF16, FMT_BF16, false, false, WQ_BM, SWAP ? 16 : WQ_BN);
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
            umma_f16_ss(tmem_d, umma_smem_desc((SWAP ? sb : sa) + k * 32, 16, 1024), umma_smem_desc((SWAP ? sa : sb) + k * 32, 16, 1024), idesc,
                        (kb > kb0 || k > 0) ? 1u : 0u);
          umma_commit(bar_empty + stage * 8);
          if (++stage == WQ_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(bar_tfull + abuf * 8);
        abuf ^= 1;
        if (abuf == 0) aphase ^= 1;
      }
    }
  } else if (warp >= 8) {
    // ------------------------------ dequantisers: 32 k of one weight row per thread, two groups on alternate k-blocks ------
    const int t = threadIdx.x - 256, g = t >> 8, r = t & 127, h = (t >> 7) & 1;
    const uint32_t scale_off = WQ_RAW_CODES + (p.group == 32 ? (r * 2 + h) * 2 : r * 2);
    const uint32_t xr = uint32_t(r & 7);
    int it = 0;
    bool ok = true;
    for (int w = cta; w < num_work && ok; w += nctas) {
      int m0, nb, kb0, kb1;
      decode(w, m0, nb, kb0, kb1);
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        if ((it & 1) != g) continue;
        const int rs = it & (WQ_RAW_STAGES - 1), stage = it & (WQ_STAGES - 1);
        const uint32_t rphase = (it / WQ_RAW_STAGES) & 1, phase = (it / WQ_STAGES) & 1;
        if (!mbar_wait_sleep_warp(bar_rfull + rs * 8, rphase, abort_flag, p.status, ST_TIMEOUT_FULL, 40)) { ok = false; break; }
        const uint32_t raw = smem_base + WQ_RAW_OFF + rs * WQ_RAW_STAGE;
        uint32_t wd[8];
        wq_load_codes<FMT>(raw, r, h, wd);
        const uint32_t sbits = ld_shared_u16(raw + scale_off);
        __syncwarp();                                        // every lane holds its codes: one arrival per warp
        if (lane == 0) mbar_arrive(bar_rempty + rs * 8);
        uint32_t o[16];
        wq_convert<FMT>(wd, sbits, o);
        if (!mbar_wait_sleep_warp(bar_empty + stage * 8, phase ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY, 40)) { ok = false; break; }
        const uint32_t row_smem = smem_base + stage * WQ_STAGE + WQ_A_BYTES + r * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c)
          st_shared_v4(row_smem + ((uint32_t(4 * h + c) ^ xr) << 4), o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_full + stage * 8);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ epilogue ------------------------------
    const int quad = warp & 3;
    int abuf = 0;
    uint32_t aphase = 0;
    for (int w = cta; w < num_work; w += nctas) {
      int m0, nb, kb0, kb1;
      decode(w, m0, nb, kb0, kb1);
      if (kb1 <= kb0) continue;
      if (!mbar_wait_sleep_warp(bar_tfull + abuf * 8, aphase, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL, 400)) break;
      tc_fence_after();
      const int row = m0 + quad * 32 + lane;
      const uint32_t taddr0 = tmem_base + abuf * WQ_BN + (uint32_t(quad * 32) << 16);
      if (AROWS == 16) {
        // swapped operands: lane = weight row n of the tile, the 16 accumulator columns = batch rows m
        uint32_t v[16];
        tmem_ld_32x16(taddr0, v);
        tmem_ld_wait();
        const int n = nb * WQ_BN + quad * 32 + lane;
        const float bv = (p.bias && kb0 == 0) ? __bfloat162float(p.bias[n]) : 0.f;
#pragma unroll
        for (int m = 0; m < 16; ++m) {
          if (m < p.M) {
            const float f = __uint_as_float(v[m]) + bv;
            if (p.splits > 1) atomicAdd(static_cast<float*>(p.C) + (long long)m * p.ldc + n, f);
            else static_cast<__nv_bfloat16*>(p.C)[(long long)m * p.ldc + n] = __float2bfloat16(f);
          }
        }
      } else if (m0 + quad * 32 < p.M) {
#pragma unroll 1
        for (int c = 0; c < WQ_BN / 16; ++c) {
          uint32_t v[16];
          tmem_ld_32x16(taddr0 + c * 16, v);
          tmem_ld_wait();
          const int col0 = nb * WQ_BN + c * 16;
          if (row >= p.M) continue;
          // N is a multiple of 128 and ldc of 8 (the packer pads), so every 16-column run is whole and 16-byte aligned
          float f[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) f[j] = __uint_as_float(v[j]);
          if (p.bias && kb0 == 0) {
#pragma unroll
            for (int j = 0; j < 16; ++j) f[j] += __bfloat162float(p.bias[col0 + j]);
          }
          if (p.splits > 1) {
            float4* cp = reinterpret_cast<float4*>(static_cast<float*>(p.C) + (long long)row * p.ldc + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) atomicAdd(cp + j, make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]));
          } else {
            uint4* cp = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0);
#pragma unroll
            for (int j = 0; j < 2; ++j)
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

// Whole-matrix dequantisation to row-major bf16 (large-M products run as a plain bf16 GEMM on this image; the image lives in
// a scratch buffer the caller reuses, so the weights stay packed in HBM between calls).  One CTA per tile, thread (r, h).
template <int FMT>
__global__ void __launch_bounds__(256) wq_dequant_kernel(const uint8_t* __restrict__ wq, const __nv_bfloat16* __restrict__ scales, int group,
                                                          __nv_bfloat16* __restrict__ out, long long ld, int KB) {
  tfb::pdl_sync();
  constexpr int RB = wq_row_bytes(FMT);
  const int kb = blockIdx.x, nb = blockIdx.y, r = threadIdx.x & 127, h = threadIdx.x >> 7;
  const long long tile = (long long)nb * KB + kb;
  const uint8_t* raw = wq + tile * (128 * RB);
  uint32_t w[8];
  if (FMT == 0 || FMT == 2) {
    const uint4 a = *reinterpret_cast<const uint4*>(raw + ((2 * h) * 128 + r) * 16), b = *reinterpret_cast<const uint4*>(raw + ((2 * h + 1) * 128 + r) * 16);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
  } else if (FMT == 1 || FMT == 3) {
    const uint4 a = *reinterpret_cast<const uint4*>(raw + (h * 128 + r) * 16);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
  } else {
    const uint2 a = *reinterpret_cast<const uint2*>(raw + (h * 128 + r) * 8);
    w[0] = a.x; w[1] = a.y;
  }
  const int spr = WQ_BK / group;
  const uint16_t sb = reinterpret_cast<const uint16_t*>(scales)[(tile * 128 + r) * spr + (group == 32 ? h : 0)];
  uint32_t o[16];
  wq_convert<FMT>(w, uint32_t(sb), o);
  uint4* dst = reinterpret_cast<uint4*>(out + (long long)(nb * 128 + r) * ld + kb * 64 + h * 32);
#pragma unroll
  for (int c = 0; c < 4; ++c) dst[c] = make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
}

}  // namespace tfb

// out [N, ld] bf16 row-major (ld % 8 == 0) = dequant(wq); N % 128 == 0, K % 64 == 0.
TFB_API int tfb_wq_dequant(const void* wq, const void* scales, int fmt, int group, void* out, long long ld, int N, int K, void* stream) {
  using namespace tfb;
  if (N <= 0 || K <= 0 || K % WQ_BK || N % WQ_BN || fmt < 0 || fmt > 4 || (group != 32 && group != 64) || ld % 8) return TFB_ERR_ARG;
  const dim3 grid(K / WQ_BK, N / WQ_BN);
  const auto* c = static_cast<const uint8_t*>(wq);
  const auto* sc = static_cast<const __nv_bfloat16*>(scales);
  auto* o = static_cast<__nv_bfloat16*>(out);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (fmt) {
    case 0: tfb::launch_k(wq_dequant_kernel<0>, grid, 256, 0, st, c, sc, group, o, ld, K / WQ_BK); break;
    case 1: tfb::launch_k(wq_dequant_kernel<1>, grid, 256, 0, st, c, sc, group, o, ld, K / WQ_BK); break;
    case 2: tfb::launch_k(wq_dequant_kernel<2>, grid, 256, 0, st, c, sc, group, o, ld, K / WQ_BK); break;
    case 3: tfb::launch_k(wq_dequant_kernel<3>, grid, 256, 0, st, c, sc, group, o, ld, K / WQ_BK); break;
    default: tfb::launch_k(wq_dequant_kernel<4>, grid, 256, 0, st, c, sc, group, o, ld, K / WQ_BK); break;
  }
  const int rc = int(cudaGetLastError());
  return rc ? -1000 - rc : 0;
}

namespace tfb {
// fp32 split-K sums -> bf16 output, and the workspace goes back to zero for its next use (one launch instead of a memset
// before the product and a cast after it)
__global__ void __launch_bounds__(256) wq_finalize_kernel(float* __restrict__ ws, long long ldw, __nv_bfloat16* __restrict__ C,
                                                          long long ldc, int M, int N, int W4) {
  tfb::pdl_sync();
  const long long total = (long long)M * W4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = int(i / W4), c = int(i % W4) * 4;
    float4* src = reinterpret_cast<float4*>(ws + (long long)r * ldw + c);
    const float4 v = *src;
    *src = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < N) {
      uint2 o;
      o.x = pack_bf16(v.x, v.y);
      o.y = pack_bf16(v.z, v.w);
      *reinterpret_cast<uint2*>(C + (long long)r * ldc + c) = o;
    }
  }
}
}  // namespace tfb

// C [M, ldc] bf16 <- ws [M, ldw] fp32 for the first N columns, and ws <- 0 over its first `width` columns (the padded
// width the product accumulated into).  N, width, ldw, ldc multiples of 4; N <= width <= ldw.
TFB_API int tfb_wq_finalize(float* ws, long long ldw, void* C, long long ldc, int M, int N, int width, void* stream) {
  if (M <= 0 || N <= 0 || (N & 3) || (width & 3) || width < N || width > ldw || (ldw & 3) || (ldc & 3) ||
      (reinterpret_cast<uintptr_t>(ws) & 15) || (reinterpret_cast<uintptr_t>(C) & 7))
    return TFB_ERR_ARG;
  const long long total = (long long)M * (width / 4);
  const int grid = int(std::min<long long>((total + 255) / 256, 148 * 8));
  tfb::launch_k(tfb::wq_finalize_kernel, grid, 256, 0, static_cast<cudaStream_t>(stream), ws, ldw, static_cast<__nv_bfloat16*>(C), ldc, M,
                N, width / 4);
  return int(cudaGetLastError());
}

// A [M, lda] bf16 (K % 64 == 0, N % 128 == 0: the packer pads).  wq / scales in the tile-major layout described at the top.
// splits == 1: C bf16 [M, ldc]; splits > 1: C fp32 [M, ldc], accumulated into (zero it first).  splits == 0 picks a value
// that fills the SMs.  Returns the number of splits used (>= 1) or a negative error.
TFB_API int tfb_gemm_wq(const void* A, long long lda, const void* wq, const void* scales, int fmt, int group, void* C, long long ldc,
                        int M, int N, int K, const void* bias, int splits, int c_is_fp32, int* status, void* stream) {
  using namespace tfb;
  if (M <= 0 || N <= 0 || K <= 0 || K % WQ_BK || N % WQ_BN || ldc % 8 || fmt < 0 || fmt > 4 || (group != 32 && group != 64)) return TFB_ERR_ARG;
  CUtensorMap ta;
  const int arows = M <= 16 ? 16 : 128;
  if (int rc = make_tmap_2d(&ta, A, 2, K, M, lda * 2, WQ_BK, arows)) return rc;
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
  static const Kern kerns[2][5] = {
      {gemm_wq_kernel<0, 16>, gemm_wq_kernel<1, 16>, gemm_wq_kernel<2, 16>, gemm_wq_kernel<3, 16>, gemm_wq_kernel<4, 16>},
      {gemm_wq_kernel<0, 128>, gemm_wq_kernel<1, 128>, gemm_wq_kernel<2, 128>, gemm_wq_kernel<3, 128>, gemm_wq_kernel<4, 128>}};
  static const int smem_of[2] = {WqPlan<16>::SMEM, WqPlan<128>::SMEM};
  static DeviceOnce once;
  if (once.first_use()) {
    for (int a = 0; a < 2; ++a)
      for (Kern k : kerns[a]) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_of[a]);
        if (e != cudaSuccess) { once.retry(); return int(e); }
      }
  }
  const long long work = (long long)tiles * p.splits;
  const int grid = int(work < sms ? work : sms);
  const int ai = arows == 16 ? 0 : 1;
  tfb::launch_k(kerns[ai][fmt], grid, WQ_THREADS, smem_of[ai], static_cast<cudaStream_t>(stream), ta, p);
  const int rc = int(cudaGetLastError());
  return rc ? -1000 - rc : p.splits;
}
