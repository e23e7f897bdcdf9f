// Flash attention backward for sm_100a: exact gradients, probabilities recomputed from the saved
// log-sum-exp (nothing of size S x S is ever stored).  Two tcgen05 kernels, no atomics:
//
//   attn_bwd_dkdv : one CTA per (batch, kv head, 128-key block); loops over the query heads of the
//                   group and the query blocks that see these keys.  Per step
//                     S^T = K Q^T, dP^T = V dO^T            (shared-memory operands)
//                     P^T = exp(S^T - lse), dS^T = P^T * (dP^T - delta) * scale   (one key row per thread)
//                     dV += P^T dO, dK += dS^T Q            (A operand from TMEM, B MN-major), accumulated in TMEM
//   attn_bwd_dq   : one CTA per (batch, query head, 128-query block); loops over key blocks:
//                     S = Q K^T, dP = dO V^T, dS = P * (dP - delta) * scale, dQ += dS K
//   attn_delta    : delta[b,h,s] = sum_d dO * O
//
// The reference's memory-efficient attention backward is approximate
// (src/trainer/zero_optimizer_mem.cpp:496-574); its autograd attention op (src/model/autograd_functions.cpp:17-226)
// materialises the S x S matrix.  This computes the exact gradient without either.
#include "tfb_host.h"
#include "tfb_ptx.cuh"

namespace tfb {

constexpr int AB_THREADS = 192;
constexpr int AB_BOX = 128 * 64 * 2;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float bwd_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct AttnBwdParams {
  int B, S, Hq, Hkv;
  float scale;
  int causal;
  int q_col0, k_col0, v_col0;       // head-0 column of q / k / v in their source rows
  const float* lse;                 // [B, Hq, S]
  const float* delta;               // [B, Hq, S]
  __nv_bfloat16* dq; long long lddq; int dq_col0;
  __nv_bfloat16* dk; long long lddk; int dk_col0;
  __nv_bfloat16* dv; long long lddv; int dv_col0;
  int* status;
};

template <int D>
struct BwdSmem {
  static constexpr int NB = D / 64;
  static constexpr int TILE = NB * AB_BOX;
  static constexpr int RES_OFF = 0;              // two resident tiles
  static constexpr int RING_OFF = 2 * TILE;      // 2 stages x 2 tiles
  static constexpr int STAT_OFF = RING_OFF + 4 * TILE;  // [2][2][128] floats
  static constexpr int BAR_OFF = STAT_OFF + 2 * 2 * 128 * 4;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};


// ------------------------------------------------------------------------------------------------
// dK / dV
// ------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(AB_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                     const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                     const AttnBwdParams p) {
  using L = BwdSmem<D>;
  constexpr int NB = L::NB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sK = sbase, sV = sbase + L::TILE;
  float* stats = reinterpret_cast<float*>(smem + L::STAT_OFF);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  const uint32_t bar_kv = smem_u32(bars);
  const uint32_t bar_full = bar_kv + 8;        // [2]
  const uint32_t bar_empty = bar_full + 16;    // [2]
  const uint32_t bar_s = bar_empty + 16;       // S^T ready
  const uint32_t bar_dp = bar_s + 8;           // dP^T ready
  const uint32_t bar_p = bar_dp + 8;           // P^T written (128 arrivals)
  const uint32_t bar_ds = bar_p + 8;           // dS^T written (128 arrivals)
  const uint32_t bar_acc = bar_ds + 8;         // all accumulation done
  const uint32_t bar_stat = bar_acc + 8;       // per-step lse / delta staged in shared memory (128 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.S + 127) / 128;
  const int nkb = nqb;
  const int jb = int(blockIdx.x) % nkb;
  const int rem = int(blockIdx.x) / nkb;
  const int hk = rem % p.Hkv, b = rem / p.Hkv;
  const int G = p.Hq / p.Hkv;
  const int i0 = p.causal ? jb : 0;
  const int n_i = nqb - i0;
  const int n_it = G * n_i;

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_full + s * 8, 1);
      mbar_init(bar_empty + s * 8, 1);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_dp, 1);
    mbar_init(bar_p, 128);
    mbar_init(bar_ds, 128);
    mbar_init(bar_acc, 1);
    mbar_init(bar_stat, 128);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 128, tDV = tmem_base + 256, tDK = tmem_base + 256 + D;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar_kv, 2 * L::TILE);
#pragma unroll
      for (int c = 0; c < NB; ++c) {
        tma_load_3d(sK + c * AB_BOX, &tk, bar_kv, p.k_col0 + hk * D + c * 64, jb * 128, b);
        tma_load_3d(sV + c * AB_BOX, &tv, bar_kv, p.v_col0 + hk * D + c * 64, jb * 128, b);
      }
      for (int it = 0; it < n_it; ++it) {
        const int st = it & 1;
        const int h = hk * G + it / n_i, i = i0 + it % n_i;
        if (!mbar_wait(bar_empty + st * 8, ((it >> 1) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) break;
        const uint32_t fb = bar_full + st * 8;
        mbar_expect_tx(fb, 2 * L::TILE);
        const uint32_t sQ = sbase + L::RING_OFF + st * 2 * L::TILE, sDO = sQ + L::TILE;
#pragma unroll
        for (int c = 0; c < NB; ++c) {
          tma_load_3d(sQ + c * AB_BOX, &tq, fb, p.q_col0 + h * D + c * 64, i * 128, b);
          tma_load_3d(sDO + c * AB_BOX, &tdo, fb, h * D + c * 64, i * 128, b);
        }
      }
      if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc(FMT_BF16, FMT_BF16, false, false, 128, 128);
      constexpr uint32_t idesc_acc = umma_idesc(FMT_BF16, FMT_BF16, false, true, 128, D);
      bool ok = mbar_wait(bar_kv, 0, abort_flag, p.status, ST_TIMEOUT_FULL);
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it & 1;
        const uint32_t ph = it & 1;  // single-buffered barriers flip every iteration
        if (!mbar_wait(bar_full + st * 8, (it >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_FULL)) break;
        tc_fence_after();
        const uint32_t sQ = sbase + L::RING_OFF + st * 2 * L::TILE, sDO = sQ + L::TILE;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * AB_BOX + (k & 3) * 32;
          umma_f16_ss(tS, umma_smem_desc(sK + off, 16, 1024), umma_smem_desc(sQ + off, 16, 1024), idesc_s, k > 0);
        }
        umma_commit(bar_s);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * AB_BOX + (k & 3) * 32;
          umma_f16_ss(tDP, umma_smem_desc(sV + off, 16, 1024), umma_smem_desc(sDO + off, 16, 1024), idesc_s, k > 0);
        }
        umma_commit(bar_dp);
        if (!mbar_wait(bar_p, ph, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16_ts(tDV, tS + k * 8, umma_smem_desc(sDO + k * 2048, AB_BOX, 1024), idesc_acc, (it > 0 || k > 0));
        if (!mbar_wait(bar_ds, ph, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16_ts(tDK, tDP + k * 8, umma_smem_desc(sQ + k * 2048, AB_BOX, 1024), idesc_acc, (it > 0 || k > 0));
        umma_commit(bar_empty + st * 8);
      }
      umma_commit(bar_acc);
    }
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int key_idx = jb * 128 + r;
    const uint32_t lane_off = uint32_t(quad * 32) << 16;
    const float sl2 = p.scale * LOG2E;
    bool ok = true;
    // per-query statistics of iteration `it` (pre-scaled log-sum-exp and delta); loaded one iteration ahead so that
    // the global-memory latency hides behind the previous block's arithmetic
    auto load_stats = [&](int it, float& l2, float& dl) {
      const int h = hk * G + it / n_i, i = i0 + it % n_i;
      const int qi = i * 128 + r;
      const long long o = ((long long)b * p.Hq + h) * p.S + qi;
      l2 = qi < p.S ? p.lse[o] * LOG2E : INFINITY;  // +inf => probability 0 for padded queries
      dl = qi < p.S ? p.delta[o] : 0.f;
    };
    float nxt_l2 = 0.f, nxt_dl = 0.f;
    if (n_it > 0) load_stats(0, nxt_l2, nxt_dl);
    for (int it = 0; it < n_it; ++it) {
      const int i = i0 + it % n_i;
      const uint32_t ph = it & 1;
      float* s_lse = stats + (it & 1) * 256;
      float* s_dl = s_lse + 128;
      s_lse[r] = nxt_l2;
      s_dl[r] = nxt_dl;
      mbar_arrive(bar_stat);
      if (it + 1 < n_it) load_stats(it + 1, nxt_l2, nxt_dl);
      if (!mbar_wait_warp(bar_stat, ph, abort_flag, p.status, ST_TIMEOUT_FLAG)) { ok = false; break; }
      if (!mbar_wait_warp(bar_s, ph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const bool diag = p.causal && (i == jb);
      uint32_t pk[64];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tS + lane_off + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int e4 = 0; e4 < 8; ++e4) {
          const float4 l4 = *reinterpret_cast<const float4*>(s_lse + c * 32 + e4 * 4);   // same address in every lane: broadcast
          const int q0 = c * 32 + e4 * 4;
          float p0 = bwd_exp2(fmaf(__uint_as_float(v[e4 * 4 + 0]), sl2, -l4.x));
          float p1 = bwd_exp2(fmaf(__uint_as_float(v[e4 * 4 + 1]), sl2, -l4.y));
          float p2 = bwd_exp2(fmaf(__uint_as_float(v[e4 * 4 + 2]), sl2, -l4.z));
          float p3 = bwd_exp2(fmaf(__uint_as_float(v[e4 * 4 + 3]), sl2, -l4.w));
          if (diag) {
            if (q0 < r) p0 = 0.f;
            if (q0 + 1 < r) p1 = 0.f;
            if (q0 + 2 < r) p2 = 0.f;
            if (q0 + 3 < r) p3 = 0.f;
          }
          pk[c * 16 + e4 * 2] = pack_bf16(p0, p1);
          pk[c * 16 + e4 * 2 + 1] = pack_bf16(p2, p3);
        }
        uint32_t (&chunk)[16] = *reinterpret_cast<uint32_t (*)[16]>(&pk[c * 16]);
        tmem_st_32x16(tS + lane_off + c * 16, chunk);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar_p);
      if (!mbar_wait_warp(bar_dp, ph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tDP + lane_off + c * 32, v);
        tmem_ld_wait();
        uint32_t ds[16];
#pragma unroll
        for (int e4 = 0; e4 < 8; ++e4) {
          const float4 d4 = *reinterpret_cast<const float4*>(s_dl + c * 32 + e4 * 4);
          const float2 pa = unpack_bf16(pk[c * 16 + e4 * 2]), pb = unpack_bf16(pk[c * 16 + e4 * 2 + 1]);
          // the softmax scale is applied once to dK when it is written out
          ds[e4 * 2] = pack_bf16(pa.x * (__uint_as_float(v[e4 * 4 + 0]) - d4.x), pa.y * (__uint_as_float(v[e4 * 4 + 1]) - d4.y));
          ds[e4 * 2 + 1] = pack_bf16(pb.x * (__uint_as_float(v[e4 * 4 + 2]) - d4.z), pb.y * (__uint_as_float(v[e4 * 4 + 3]) - d4.w));
        }
        tmem_st_32x16(tDP + lane_off + c * 16, ds);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar_ds);
    }
    if (ok && mbar_wait_warp(bar_acc, 0, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      const bool valid = key_idx < p.S;
      const long long row = (long long)b * p.S + (valid ? key_idx : 0);
      __nv_bfloat16* dvp = p.dv + row * p.lddv + p.dv_col0 + hk * D;
      __nv_bfloat16* dkp = p.dk + row * p.lddk + p.dk_col0 + hk * D;
      // the tensor-memory loads are warp-collective: every lane executes them, only the stores are predicated
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32], u2[32];
        tmem_ld_32x32(tDV + lane_off + c * 32, v);
        tmem_ld_32x32(tDK + lane_off + c * 32, u2);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u;
            u.x = pack_bf16(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
            u.y = pack_bf16(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
            u.z = pack_bf16(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
            u.w = pack_bf16(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
            *reinterpret_cast<uint4*>(dvp + c * 32 + q * 8) = u;
            const float sc = p.scale;
            u.x = pack_bf16(__uint_as_float(u2[q * 8 + 0]) * sc, __uint_as_float(u2[q * 8 + 1]) * sc);
            u.y = pack_bf16(__uint_as_float(u2[q * 8 + 2]) * sc, __uint_as_float(u2[q * 8 + 3]) * sc);
            u.z = pack_bf16(__uint_as_float(u2[q * 8 + 4]) * sc, __uint_as_float(u2[q * 8 + 5]) * sc);
            u.w = pack_bf16(__uint_as_float(u2[q * 8 + 6]) * sc, __uint_as_float(u2[q * 8 + 7]) * sc);
            *reinterpret_cast<uint4*>(dkp + c * 32 + q * 8) = u;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// dS = P * (dP - delta) for one query row (128 keys): reads S and dP from tensor memory, writes dS (bf16 pairs) over
// the dP columns.  The softmax scale is folded into the final dQ store.
template <bool MASK>
__device__ __forceinline__ void dq_block(uint32_t tS, uint32_t tDP, float sl2, float lse2, float dl, int k0, int k_lim) {
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    uint32_t s[32], dp[32];
    tmem_ld_32x32(tS + c * 32, s);
    tmem_ld_32x32(tDP + c * 32, dp);
    tmem_ld_wait();
    uint32_t ds[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      float p0 = bwd_exp2(fmaf(__uint_as_float(s[2 * e]), sl2, -lse2));
      float p1 = bwd_exp2(fmaf(__uint_as_float(s[2 * e + 1]), sl2, -lse2));
      if (MASK) {
        if (k0 + c * 32 + 2 * e > k_lim) p0 = 0.f;
        if (k0 + c * 32 + 2 * e + 1 > k_lim) p1 = 0.f;
      }
      ds[e] = pack_bf16(p0 * (__uint_as_float(dp[2 * e]) - dl), p1 * (__uint_as_float(dp[2 * e + 1]) - dl));
    }
    tmem_st_32x16(tDP + c * 16, ds);
  }
}

// ------------------------------------------------------------------------------------------------
// dQ
// ------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(AB_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                   const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                   const AttnBwdParams p) {
  using L = BwdSmem<D>;
  constexpr int NB = L::NB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sQ = sbase, sDO = sbase + L::TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  const uint32_t bar_q = smem_u32(bars);
  const uint32_t bar_full = bar_q + 8;
  const uint32_t bar_empty = bar_full + 16;
  const uint32_t bar_s = bar_empty + 16;  // S and dP ready
  const uint32_t bar_ds = bar_s + 8;      // dS written (128 arrivals)
  const uint32_t bar_acc = bar_ds + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.S + 127) / 128;
  const int bh = p.B * p.Hq;
  const int qb = nqb - 1 - int(blockIdx.x) / bh;
  const int rem = int(blockIdx.x) % bh;
  const int b = rem / p.Hq, h = rem % p.Hq;
  const int hk = h / (p.Hq / p.Hkv);
  const int n_kv = p.causal ? qb + 1 : nqb;

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_full + s * 8, 1);
      mbar_init(bar_empty + s * 8, 1);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_ds, 128);
    mbar_init(bar_acc, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 128, tDQ = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar_q, 2 * L::TILE);
#pragma unroll
      for (int c = 0; c < NB; ++c) {
        tma_load_3d(sQ + c * AB_BOX, &tq, bar_q, p.q_col0 + h * D + c * 64, qb * 128, b);
        tma_load_3d(sDO + c * AB_BOX, &tdo, bar_q, h * D + c * 64, qb * 128, b);
      }
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        if (!mbar_wait(bar_empty + st * 8, ((j >> 1) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) break;
        const uint32_t fb = bar_full + st * 8;
        mbar_expect_tx(fb, 2 * L::TILE);
        const uint32_t sK = sbase + L::RING_OFF + st * 2 * L::TILE, sV = sK + L::TILE;
#pragma unroll
        for (int c = 0; c < NB; ++c) {
          tma_load_3d(sK + c * AB_BOX, &tk, fb, p.k_col0 + hk * D + c * 64, j * 128, b);
          tma_load_3d(sV + c * AB_BOX, &tv, fb, p.v_col0 + hk * D + c * 64, j * 128, b);
        }
      }
      if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc(FMT_BF16, FMT_BF16, false, false, 128, 128);
      constexpr uint32_t idesc_acc = umma_idesc(FMT_BF16, FMT_BF16, false, true, 128, D);
      bool ok = mbar_wait(bar_q, 0, abort_flag, p.status, ST_TIMEOUT_FULL);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1;
        if (!mbar_wait(bar_full + st * 8, (j >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_FULL)) break;
        tc_fence_after();
        const uint32_t sK = sbase + L::RING_OFF + st * 2 * L::TILE, sV = sK + L::TILE;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * AB_BOX + (k & 3) * 32;
          umma_f16_ss(tS, umma_smem_desc(sQ + off, 16, 1024), umma_smem_desc(sK + off, 16, 1024), idesc_s, k > 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * AB_BOX + (k & 3) * 32;
          umma_f16_ss(tDP, umma_smem_desc(sDO + off, 16, 1024), umma_smem_desc(sV + off, 16, 1024), idesc_s, k > 0);
        }
        umma_commit(bar_s);
        if (!mbar_wait(bar_ds, j & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16_ts(tDQ, tDP + k * 8, umma_smem_desc(sK + k * 2048, AB_BOX, 1024), idesc_acc, (j > 0 || k > 0));
        umma_commit(bar_empty + st * 8);
      }
      umma_commit(bar_acc);
    }
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int q_idx = qb * 128 + r;
    const uint32_t lane_off = uint32_t(quad * 32) << 16;
    const float sl2 = p.scale * LOG2E;
    const long long so = ((long long)b * p.Hq + h) * p.S + q_idx;
    const float lse2 = q_idx < p.S ? p.lse[so] * LOG2E : INFINITY;
    const float dl = q_idx < p.S ? p.delta[so] : 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait_warp(bar_s, j & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int k0 = j * 128;
      const bool need_mask = (p.causal && j == qb) || (k0 + 128 > p.S);
      const int k_lim = p.causal ? min(q_idx, p.S - 1) : p.S - 1;
      if (need_mask) dq_block<true>(tS + lane_off, tDP + lane_off, sl2, lse2, dl, k0, k_lim);
      else dq_block<false>(tS + lane_off, tDP + lane_off, sl2, lse2, dl, k0, k_lim);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar_ds);
    }
    if (ok && mbar_wait_warp(bar_acc, 0, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      __nv_bfloat16* dqp = p.dq + ((long long)b * p.S + q_idx) * p.lddq + p.dq_col0 + h * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tDQ + lane_off + c * 32, v);
        tmem_ld_wait();
        if (q_idx < p.S) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u;
            const float sc = p.scale;
            u.x = pack_bf16(__uint_as_float(v[q * 8 + 0]) * sc, __uint_as_float(v[q * 8 + 1]) * sc);
            u.y = pack_bf16(__uint_as_float(v[q * 8 + 2]) * sc, __uint_as_float(v[q * 8 + 3]) * sc);
            u.z = pack_bf16(__uint_as_float(v[q * 8 + 4]) * sc, __uint_as_float(v[q * 8 + 5]) * sc);
            u.w = pack_bf16(__uint_as_float(v[q * 8 + 6]) * sc, __uint_as_float(v[q * 8 + 7]) * sc);
            *reinterpret_cast<uint4*>(dqp + c * 32 + q * 8) = u;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b,h,s] = sum_d dO[t, h*D + d] * O[t, h*D + d]; one warp per (token, head)
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, long long ldo,
                                  const __nv_bfloat16* __restrict__ dout, long long lddo, float* __restrict__ delta,
                                  int B, int S, int Hq, int D) {
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long total = (long long)B * S * Hq;
  if (w >= total) return;
  const int h = int(w % Hq);
  const long long t = w / Hq;
  float acc = 0.f;
  for (int d = lane * 2; d < D; d += 64) {
    const float2 a = unpack_bf16(*reinterpret_cast<const uint32_t*>(o + t * ldo + h * D + d));
    const float2 g = unpack_bf16(*reinterpret_cast<const uint32_t*>(dout + t * lddo + h * D + d));
    acc += a.x * g.x + a.y * g.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    const long long bb = t / S, s = t % S;
    delta[(bb * Hq + h) * S + s] = acc;
  }
}

template <int D>
static int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                      const AttnBwdParams& p, cudaStream_t st) {
  using L = BwdSmem<D>;
  static bool configured = false;
  auto k1 = attn_bwd_dkdv_kernel<D>;
  auto k2 = attn_bwd_dq_kernel<D>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return int(e);
    e = cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return int(e);
    configured = true;
  }
  const int nqb = (p.S + 127) / 128;
  k1<<<nqb * p.Hkv * p.B, AB_THREADS, L::TOTAL, st>>>(tq, tk, tv, tdo, p);
  k2<<<nqb * p.Hq * p.B, AB_THREADS, L::TOTAL, st>>>(tq, tk, tv, tdo, p);
  return int(cudaGetLastError());
}

}  // namespace tfb

// Gradients of tfb_attn_fwd.  q/k/v as in the forward; o and dout are [B*S, ld] with head h at column
// h*D; lse from the forward; delta is [B,Hq,S] fp32 scratch filled here.  dq/dk/dv are written (not
// accumulated) at column offsets d*_col0 + head*D of rows with pitches ldd* - they may all point into
// one fused [T, (Hq + 2 Hkv) D] gradient buffer.
TFB_API int tfb_attn_bwd(const void* q, long long ldq, int q_col0, const void* k, long long ldk, int k_col0,
                         const void* v, long long ldv, int v_col0, const void* o, long long ldo, const void* dout,
                         long long lddo, const float* lse, float* delta, void* dq, long long lddq, int dq_col0,
                         void* dk, long long lddk, int dk_col0, void* dv, long long lddv, int dv_col0, int B, int S,
                         int Hq, int Hkv, int D, float scale, int causal, int* status, void* stream) {
  using namespace tfb;
  if ((D != 64 && D != 128) || Hkv <= 0 || Hq % Hkv || B <= 0 || S <= 0) return TFB_ERR_ARG;
  if ((q_col0 | k_col0 | v_col0 | dq_col0 | dk_col0 | dv_col0) & 7) return TFB_ERR_ARG;
  if ((lddq | lddk | lddv) & 7) return TFB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) | reinterpret_cast<uintptr_t>(dv)) & 15)
    return TFB_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  {
    const long long warps = (long long)B * S * Hq;
    const int blocks = int((warps * 32 + 255) / 256);
    attn_delta_kernel<<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(o), ldo,
                                              static_cast<const __nv_bfloat16*>(dout), lddo, delta, B, S, Hq, D);
  }
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_tmap_3d(&tq, q, 2, ldq, S, B, ldq * 2, ldq * 2 * S, 64, 128, 1))) return rc;
  if ((rc = make_tmap_3d(&tk, k, 2, ldk, S, B, ldk * 2, ldk * 2 * S, 64, 128, 1))) return rc;
  if ((rc = make_tmap_3d(&tv, v, 2, ldv, S, B, ldv * 2, ldv * 2 * S, 64, 128, 1))) return rc;
  if ((rc = make_tmap_3d(&tdo, dout, 2, lddo, S, B, lddo * 2, lddo * 2 * S, 64, 128, 1))) return rc;
  AttnBwdParams p;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.scale = scale; p.causal = causal;
  p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0;
  p.lse = lse; p.delta = delta;
  p.dq = static_cast<__nv_bfloat16*>(dq); p.lddq = lddq; p.dq_col0 = dq_col0;
  p.dk = static_cast<__nv_bfloat16*>(dk); p.lddk = lddk; p.dk_col0 = dk_col0;
  p.dv = static_cast<__nv_bfloat16*>(dv); p.lddv = lddv; p.dv_col0 = dv_col0;
  p.status = status;
  return D == 64 ? launch_bwd<64>(tq, tk, tv, tdo, p, st) : launch_bwd<128>(tq, tk, tv, tdo, p, st);
}
