// Flash attention backward for sm_100a: exact gradients, probabilities recomputed from the saved
// log-sum-exp (nothing of size S x S is ever stored).  Two tcgen05 kernels, no atomics; each runs two compute
// warpgroups that work on the two halves of a 128 x 128 score block, so that the tensor core computes one half while
// the other half's exponentials and products are in flight, and every scheduler has two compute warps to issue from.
//
//   attn_bwd_dkdv : one CTA per (batch, kv head, 128-key block); loops over the query heads of the group and the
//                   query blocks that see these keys.  Per step and per half w (64 queries):
//                     S^T_w = K Q_w^T, dP^T_w = V dO_w^T                       (shared-memory operands, 128 x 64)
//                     P^T_w = exp(S^T_w - lse), dS^T_w = P^T_w * (dP^T_w - delta)    (one key row per thread)
//                     dV += P^T_w dO_w, dK += dS^T_w Q_w     (A operand from TMEM, B MN-major), accumulated in TMEM
//   attn_bwd_dq   : one CTA per (batch, query head, 128-query block); loops over key blocks, half w = 64 keys:
//                     S_w = Q K_w^T, dP_w = dO V_w^T, dS_w = P_w * (dP_w - delta), dQ += dS_w K_w
//   attn_delta    : delta[b,h,s] = sum_d dO * O
// The softmax scale multiplies dK and dQ once, when they are written out.
// Tensor memory: half w owns columns [128 w, 128 w + 64) for S / P and [128 w + 64, 128 w + 128) for dP / dS; the
// accumulators start at column 256.
//
// The reference's memory-efficient attention backward is approximate
// (src/trainer/zero_optimizer_mem.cpp:496-574); its autograd attention op (src/model/autograd_functions.cpp:17-226)
// materialises the S x S matrix.  This computes the exact gradient without either.
#include "tfb_host.h"
#include "tfb_ptx.cuh"

namespace tfb {

constexpr int AB_THREADS = 320;   // warp 0 TMA, warp 1 MMA, warps 2-5 half 0, warps 6-9 half 1
constexpr int AB_BOX = 128 * 64 * 2;
constexpr int AB_HALF = 64 * 128;  // byte offset of row 64 inside a 128-row, 128-byte-pitch box
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
  static constexpr int STAT_OFF = RING_OFF + 4 * TILE;  // [2 stages][2 halves][64 lse | 64 delta] floats
  static constexpr int BAR_OFF = STAT_OFF + 2 * 2 * 128 * 4;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

// 16 output rows x 128 bf16 columns of an accumulator, written by one thread (its row)
__device__ __forceinline__ void store_row32(__nv_bfloat16* dst, const uint32_t (&v)[32], float sc) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint4 u;
    u.x = pack_bf16(__uint_as_float(v[q * 8 + 0]) * sc, __uint_as_float(v[q * 8 + 1]) * sc);
    u.y = pack_bf16(__uint_as_float(v[q * 8 + 2]) * sc, __uint_as_float(v[q * 8 + 3]) * sc);
    u.z = pack_bf16(__uint_as_float(v[q * 8 + 4]) * sc, __uint_as_float(v[q * 8 + 5]) * sc);
    u.w = pack_bf16(__uint_as_float(v[q * 8 + 6]) * sc, __uint_as_float(v[q * 8 + 7]) * sc);
    *reinterpret_cast<uint4*>(dst + q * 8) = u;
  }
}

// ------------------------------------------------------------------------------------------------
// dK / dV
// ------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(AB_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                     const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                     const AttnBwdParams p) {
  tfb::pdl_sync();
  using L = BwdSmem<D>;
  constexpr int NB = L::NB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sK = sbase, sV = sbase + L::TILE;
  float* stats = reinterpret_cast<float*>(smem + L::STAT_OFF);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  const uint32_t bar_kv = smem_u32(bars);
  const uint32_t bar_full = bar_kv + 8;        // [2] Q / dO stage loaded
  const uint32_t bar_empty = bar_full + 16;    // [2] stage consumed
  const uint32_t bar_s = bar_empty + 16;       // [2] S^T_w and dP^T_w ready
  const uint32_t bar_pds = bar_s + 16;         // [2] P^T_w and dS^T_w written (128 arrivals)
  const uint32_t bar_stat = bar_pds + 16;      // [2] per-step statistics of half w staged (128 arrivals)
  const uint32_t bar_acc = bar_stat + 16;      // all accumulation done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
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
      mbar_init(bar_s + s * 8, 1);
      mbar_init(bar_pds + s * 8, 128);
      mbar_init(bar_stat + s * 8, 128);
    }
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
  const uint32_t tDV = tmem_base + 256, tDK = tmem_base + 256 + D;

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
      constexpr uint32_t idesc_s = umma_idesc(FMT_BF16, FMT_BF16, false, false, 128, 64);
      constexpr uint32_t idesc_acc = umma_idesc(FMT_BF16, FMT_BF16, false, true, 128, D);
      // scores of half w for the step whose Q / dO tiles sit in stage st
      auto issue_scores = [&](int w, int st) {
        const uint32_t sQ = sbase + L::RING_OFF + st * 2 * L::TILE + w * AB_HALF, sDO = sQ + L::TILE;
        const uint32_t tS = tmem_base + w * 128, tDP = tS + 64;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * AB_BOX + (k & 3) * 32;
          umma_f16_ss(tS, umma_smem_desc(sK + off, 16, 1024), umma_smem_desc(sQ + off, 16, 1024), idesc_s, k > 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * AB_BOX + (k & 3) * 32;
          umma_f16_ss(tDP, umma_smem_desc(sV + off, 16, 1024), umma_smem_desc(sDO + off, 16, 1024), idesc_s, k > 0);
        }
        umma_commit(bar_s + w * 8);
      };
      bool ok = mbar_wait(bar_kv, 0, abort_flag, p.status, ST_TIMEOUT_FULL) &&
                (n_it == 0 || mbar_wait(bar_full, 0, abort_flag, p.status, ST_TIMEOUT_FULL));
      if (ok && n_it > 0) {
        tc_fence_after();
        issue_scores(0, 0);
        issue_scores(1, 0);
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it & 1;
        if (it + 1 < n_it) {
          if (!mbar_wait(bar_full + ((it + 1) & 1) * 8, ((it + 1) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_FULL)) break;
          tc_fence_after();
        }
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          if (!ok) continue;
          if (!mbar_wait(bar_pds + w * 8, it & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; continue; }
          tc_fence_after();
          const uint32_t sQ = sbase + L::RING_OFF + st * 2 * L::TILE + w * AB_HALF, sDO = sQ + L::TILE;
          const uint32_t tS = tmem_base + w * 128, tDP = tS + 64;
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ts(tDV, tS + k * 8, umma_smem_desc(sDO + k * 2048, AB_BOX, 1024), idesc_acc, (it > 0 || w > 0 || k > 0));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ts(tDK, tDP + k * 8, umma_smem_desc(sQ + k * 2048, AB_BOX, 1024), idesc_acc, (it > 0 || w > 0 || k > 0));
          if (it + 1 < n_it) issue_scores(w, (it + 1) & 1);
        }
        if (ok) umma_commit(bar_empty + st * 8);
      }
      umma_commit(bar_acc);
    }
  } else {
    const int w = (warp - 2) >> 2;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int key_idx = jb * 128 + r;
    const uint32_t lane_off = uint32_t(quad * 32) << 16;
    const uint32_t tS = tmem_base + w * 128 + lane_off, tDP = tS + 64;
    const float sl2 = p.scale * LOG2E;
    bool ok = true;
    // thread r stages one statistic of this half's 64 queries: r < 64 the pre-scaled log-sum-exp of query r, else the
    // delta of query r - 64.  Loaded one step ahead so that the global-memory latency hides behind the arithmetic.
    auto load_stat = [&](int it) -> float {
      const int h = hk * G + it / n_i, i = i0 + it % n_i;
      const int qi = i * 128 + w * 64 + (r & 63);
      const long long o = ((long long)b * p.Hq + h) * p.S + qi;
      if (r < 64) return qi < p.S ? p.lse[o] * LOG2E : INFINITY;   // +inf => probability 0 for padded queries
      return qi < p.S ? p.delta[o] : 0.f;
    };
    float nxt = n_it > 0 ? load_stat(0) : 0.f;
    for (int it = 0; it < n_it; ++it) {
      const int i = i0 + it % n_i;
      const uint32_t ph = it & 1;
      float* s_lse = stats + ((it & 1) * 2 + w) * 128;
      float* s_dl = s_lse + 64;
      s_lse[r] = nxt;
      mbar_arrive(bar_stat + w * 8);
      if (it + 1 < n_it) nxt = load_stat(it + 1);
      if (!mbar_wait_warp(bar_stat + w * 8, ph, abort_flag, p.status, ST_TIMEOUT_FLAG)) { ok = false; break; }
      if (!mbar_wait_warp(bar_s + w * 8, ph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const bool diag = p.causal && (i == jb);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(tS + c * 32, sv);
        tmem_ld_32x32(tDP + c * 32, dv);
        tmem_ld_wait();
        uint32_t pk[16], ds[16];
#pragma unroll
        for (int e4 = 0; e4 < 8; ++e4) {
          const float4 l4 = *reinterpret_cast<const float4*>(s_lse + c * 32 + e4 * 4);   // same address in every lane: broadcast
          const float4 d4 = *reinterpret_cast<const float4*>(s_dl + c * 32 + e4 * 4);
          const int q0 = w * 64 + c * 32 + e4 * 4;      // query index inside the 128-query block
          float p0 = bwd_exp2(fmaf(__uint_as_float(sv[e4 * 4 + 0]), sl2, -l4.x));
          float p1 = bwd_exp2(fmaf(__uint_as_float(sv[e4 * 4 + 1]), sl2, -l4.y));
          float p2 = bwd_exp2(fmaf(__uint_as_float(sv[e4 * 4 + 2]), sl2, -l4.z));
          float p3 = bwd_exp2(fmaf(__uint_as_float(sv[e4 * 4 + 3]), sl2, -l4.w));
          if (diag) {
            if (q0 < r) p0 = 0.f;
            if (q0 + 1 < r) p1 = 0.f;
            if (q0 + 2 < r) p2 = 0.f;
            if (q0 + 3 < r) p3 = 0.f;
          }
          pk[e4 * 2] = pack_bf16(p0, p1);
          pk[e4 * 2 + 1] = pack_bf16(p2, p3);
          ds[e4 * 2] = pack_bf16(p0 * (__uint_as_float(dv[e4 * 4 + 0]) - d4.x), p1 * (__uint_as_float(dv[e4 * 4 + 1]) - d4.y));
          ds[e4 * 2 + 1] = pack_bf16(p2 * (__uint_as_float(dv[e4 * 4 + 2]) - d4.z), p3 * (__uint_as_float(dv[e4 * 4 + 3]) - d4.w));
        }
        tmem_st_32x16(tS + c * 16, pk);
        tmem_st_32x16(tDP + c * 16, ds);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar_pds + w * 8);
    }
    if (ok && mbar_wait_warp(bar_acc, 0, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      const bool valid = key_idx < p.S;
      const long long row = (long long)b * p.S + (valid ? key_idx : 0);
      // half 0 writes dV, half 1 writes dK (scaled).  The tensor-memory loads are warp-collective: every lane executes
      // them, only the stores are predicated.
      __nv_bfloat16* dst = w == 0 ? p.dv + row * p.lddv + p.dv_col0 + hk * D : p.dk + row * p.lddk + p.dk_col0 + hk * D;
      const uint32_t tA = (w == 0 ? tDV : tDK) + lane_off;
      const float sc = w == 0 ? 1.f : p.scale;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tA + c * 32, v);
        tmem_ld_wait();
        if (valid) store_row32(dst + c * 32, v, sc);
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

// ------------------------------------------------------------------------------------------------
// dQ
// ------------------------------------------------------------------------------------------------
// dS = P * (dP - delta) for one query row and one half block (64 keys): reads S and dP from tensor memory, writes dS
// (bf16 pairs) over the dP columns.
template <bool MASK>
__device__ __forceinline__ void dq_half_block(uint32_t tS, uint32_t tDP, float sl2, float lse2, float dl, int k0, int k_lim) {
#pragma unroll
  for (int c = 0; c < 2; ++c) {
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

template <int D>
__global__ void __launch_bounds__(AB_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                   const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                   const AttnBwdParams p) {
  tfb::pdl_sync();
  using L = BwdSmem<D>;
  constexpr int NB = L::NB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sQ = sbase, sDO = sbase + L::TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  const uint32_t bar_q = smem_u32(bars);
  const uint32_t bar_full = bar_q + 8;     // [2]
  const uint32_t bar_empty = bar_full + 16;
  const uint32_t bar_s = bar_empty + 16;   // [2] S_w and dP_w ready
  const uint32_t bar_ds = bar_s + 16;      // [2] dS_w written (128 arrivals)
  const uint32_t bar_acc = bar_ds + 16;
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
      mbar_init(bar_s + s * 8, 1);
      mbar_init(bar_ds + s * 8, 128);
    }
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
  const uint32_t tDQ = tmem_base + 256;

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
      constexpr uint32_t idesc_s = umma_idesc(FMT_BF16, FMT_BF16, false, false, 128, 64);
      constexpr uint32_t idesc_acc = umma_idesc(FMT_BF16, FMT_BF16, false, true, 128, D);
      auto issue_scores = [&](int w, int st) {
        const uint32_t sK = sbase + L::RING_OFF + st * 2 * L::TILE + w * AB_HALF, sV = sK + L::TILE;
        const uint32_t tS = tmem_base + w * 128, tDP = tS + 64;
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
        umma_commit(bar_s + w * 8);
      };
      bool ok = mbar_wait(bar_q, 0, abort_flag, p.status, ST_TIMEOUT_FULL) &&
                (n_kv == 0 || mbar_wait(bar_full, 0, abort_flag, p.status, ST_TIMEOUT_FULL));
      if (ok && n_kv > 0) {
        tc_fence_after();
        issue_scores(0, 0);
        issue_scores(1, 0);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1;
        if (j + 1 < n_kv) {
          if (!mbar_wait(bar_full + ((j + 1) & 1) * 8, ((j + 1) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_FULL)) break;
          tc_fence_after();
        }
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          if (!ok) continue;
          if (!mbar_wait(bar_ds + w * 8, j & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; continue; }
          tc_fence_after();
          const uint32_t sK = sbase + L::RING_OFF + st * 2 * L::TILE + w * AB_HALF;
          const uint32_t tDP = tmem_base + w * 128 + 64;
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ts(tDQ, tDP + k * 8, umma_smem_desc(sK + k * 2048, AB_BOX, 1024), idesc_acc, (j > 0 || w > 0 || k > 0));
          if (j + 1 < n_kv) issue_scores(w, (j + 1) & 1);
        }
        if (ok) umma_commit(bar_empty + st * 8);
      }
      umma_commit(bar_acc);
    }
  } else {
    const int w = (warp - 2) >> 2;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int q_idx = qb * 128 + r;
    const uint32_t lane_off = uint32_t(quad * 32) << 16;
    const uint32_t tS = tmem_base + w * 128 + lane_off, tDP = tS + 64;
    const float sl2 = p.scale * LOG2E;
    const long long so = ((long long)b * p.Hq + h) * p.S + q_idx;
    const float lse2 = q_idx < p.S ? p.lse[so] * LOG2E : INFINITY;
    const float dl = q_idx < p.S ? p.delta[so] : 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait_warp(bar_s + w * 8, j & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int k0 = j * 128 + w * 64;
      const bool need_mask = (p.causal && j == qb) || (k0 + 64 > p.S);
      const int k_lim = p.causal ? min(q_idx, p.S - 1) : p.S - 1;
      if (need_mask) dq_half_block<true>(tS, tDP, sl2, lse2, dl, k0, k_lim);
      else dq_half_block<false>(tS, tDP, sl2, lse2, dl, k0, k_lim);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar_ds + w * 8);
    }
    if (ok && mbar_wait_warp(bar_acc, 0, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      // each half writes D / 2 columns of the row
      __nv_bfloat16* dqp = p.dq + ((long long)b * p.S + q_idx) * p.lddq + p.dq_col0 + h * D + w * (D / 2);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tDQ + lane_off + w * (D / 2) + c * 32, v);
        tmem_ld_wait();
        if (q_idx < p.S) store_row32(dqp + c * 32, v, p.scale);
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

// delta[b,h,s] = sum_d dO[t, h*D + d] * O[t, h*D + d].  One thread per 8 consecutive elements of a token row (16-byte
// loads, consecutive lanes on consecutive addresses); the D / 8 lanes of a head reduce with shuffles.
__global__ void __launch_bounds__(256) attn_delta_kernel(const __nv_bfloat16* __restrict__ o, long long ldo,
                                                         const __nv_bfloat16* __restrict__ dout, long long lddo,
                                                         float* __restrict__ delta, int B, int S, int Hq, int D) {
  tfb::pdl_sync();
  const int per_row = Hq * D / 8;                       // threads per token row
  const long long total = (long long)B * S * per_row;
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const bool live = i < total;
  const long long t = live ? i / per_row : 0;
  const int c = live ? int(i - t * per_row) * 8 : 0;    // first column of this thread
  float acc = 0.f;
  if (live) {
    const uint4 a = *reinterpret_cast<const uint4*>(o + t * ldo + c);
    const uint4 g = *reinterpret_cast<const uint4*>(dout + t * lddo + c);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = unpack_bf16(aw[j]), y = unpack_bf16(gw[j]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
  const int group = D / 8;                              // 8 or 16 lanes per head, aligned inside the warp
  for (int off = group >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (live && (threadIdx.x & (group - 1)) == 0) {
    const int h = c / D;
    const long long bb = t / S, s_ = t % S;
    delta[(bb * Hq + h) * S + s_] = acc;
  }
}

template <int D>
static int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                      const AttnBwdParams& p, cudaStream_t st) {
  using L = BwdSmem<D>;
  static DeviceOnce once1, once2;   // kernel attributes are per device: set on the first launch on each one
  auto k1 = attn_bwd_dkdv_kernel<D>;
  auto k2 = attn_bwd_dq_kernel<D>;
  if (int e = ensure_dyn_smem(once1, k1, L::TOTAL)) return e;
  if (int e = ensure_dyn_smem(once2, k2, L::TOTAL)) return e;
  const int nqb = (p.S + 127) / 128;
  tfb::launch_k(k1, nqb * p.Hkv * p.B, AB_THREADS, L::TOTAL, st, tq, tk, tv, tdo, p);
  tfb::launch_k(k2, nqb * p.Hq * p.B, AB_THREADS, L::TOTAL, st, tq, tk, tv, tdo, p);
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
  if (((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(dout)) & 15) || (ldo & 7) || (lddo & 7)) return TFB_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  {
    const long long threads = (long long)B * S * Hq * D / 8;
    const int blocks = int((threads + 255) / 256);
    tfb::launch_k(attn_delta_kernel, blocks, 256, 0, st, static_cast<const __nv_bfloat16*>(o), ldo,
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
