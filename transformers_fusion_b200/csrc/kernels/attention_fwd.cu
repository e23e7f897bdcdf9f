// Flash attention forward for sm_100a (causal or full, grouped-query heads, head_dim 64 or 128).
//
// One CTA per (batch, query head, 256-query block), handled as two 128-query tiles that share every K / V tile;
// 320 threads:
//   warp 0        TMA producer: both Q tiles once, then K_j / V_j tiles (128 keys) through a shared-memory ring
//   warp 1        MMA issuer:   S_t = Q_t K_j^T  (tcgen05.mma, both operands in shared memory, fp32 in TMEM)
//                               O_t = P_t V_j    (A operand = bf16 probabilities read from TMEM, B = V_j MN-major)
//   warps 2..5    softmax of tile 0, warps 6..9 softmax of tile 1: one query row per thread - tcgen05.ld the score
//                 row, online max / sum, exp2, write P (bf16 pairs) back over the score columns with tcgen05.st,
//                 accumulate O in registers with the running rescale
// The two tiles ping-pong: while one softmax group works, the tensor core computes the other tile's scores, and each
// scheduler always has two softmax warps to issue from.  Tensor memory: S/P of tile t at columns [128 t, 128 t + 128),
// O of tile t at 256 + t * D.  P overwrites S, so S_t(j+1) is issued after P_t(j) V_j (the tensor core runs them in
// issue order); the commit that announces S_t(j+1) therefore also covers O_t(j), which the softmax warps fold into
// their registers before they release P_t(j+1).  Nothing but Q, K, V is read and nothing but O and the log-sum-exp
// row is written.
//
// Reference counterparts: attention_kernel (src/backend/gpu_compute_cuda.cpp:296, one thread per
// query, three passes, non-causal), CPU flash attention (src/kernel/flash_attention.cpp:38-225).
#include "tfb_host.h"
#include "tfb_ptx.cuh"

namespace tfb {

constexpr int ATT_THREADS = 320;
constexpr int ATT_BM = 128;   // queries per tile (two tiles per CTA)
constexpr int ATT_BN = 128;   // keys per step
constexpr int BOX_BYTES = 128 * 64 * 2;

struct AttnFwdParams {
  int B, S, Hq, Hkv;
  int Skv, q_off;  // keys per sequence; causal: query i sees keys <= i + q_off (q_off = Skv - S: the queries are the last S positions)
  float scale;
  int causal;
  int q_col0, k_col0, v_col0;
  __nv_bfloat16* O;
  long long ldo;
  float* lse;  // [B, Hq, S]
  int* status;
};

template <int D>
struct AttnSmem {
  static constexpr int NB = D / 64;  // 64-column boxes per tile
  static constexpr int TILE = NB * BOX_BYTES;
  static constexpr int STAGES = (D == 64) ? 4 : 2;
  static constexpr int Q_OFF = 0;
  static constexpr int KV_OFF = 2 * TILE;
  static constexpr int BAR_OFF = KV_OFF + STAGES * 2 * TILE;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Row maximum of 128 scores held in tensor memory (one row per thread).  MASK: keys after k_lim do not count.
// Four independent chains of three-input max keep the dependent-issue latency off the critical path.
template <bool MASK>
__device__ __forceinline__ float row_max(uint32_t tS, float m, int k0, int k_lim) {
  float mx0 = m, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    uint32_t v[32];
    tmem_ld_32x32(tS + c * 32, v);
    tmem_ld_wait();
    if (MASK) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (k0 + c * 32 + i > k_lim) v[i] = 0xff800000u;  // -inf
    }
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      mx0 = fmax3(mx0, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
      mx1 = fmax3(mx1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
      mx2 = fmax3(mx2, __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
      mx3 = fmax3(mx3, __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
    }
  }
  return fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
}

// p = 2^(s * sl2 - mb) for the 128 scores of this thread's row, written back over the score columns as bf16 pairs;
// returns the row sum (fp32, four partial sums).
template <bool MASK>
__device__ __forceinline__ float row_probs(uint32_t tS, float sl2, float mb, int k0, int k_lim) {
  float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    uint32_t v[32];
    tmem_ld_32x32(tS + c * 32, v);
    tmem_ld_wait();
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      float p0 = fast_exp2(fmaf(__uint_as_float(v[2 * i]), sl2, -mb));
      float p1 = fast_exp2(fmaf(__uint_as_float(v[2 * i + 1]), sl2, -mb));
      float p2 = fast_exp2(fmaf(__uint_as_float(v[2 * i + 2]), sl2, -mb));
      float p3 = fast_exp2(fmaf(__uint_as_float(v[2 * i + 3]), sl2, -mb));
      if (MASK) {
        if (k0 + c * 32 + 2 * i > k_lim) p0 = 0.f;
        if (k0 + c * 32 + 2 * i + 1 > k_lim) p1 = 0.f;
        if (k0 + c * 32 + 2 * i + 2 > k_lim) p2 = 0.f;
        if (k0 + c * 32 + 2 * i + 3 > k_lim) p3 = 0.f;
      }
      rs0 += p0;
      rs1 += p1;
      rs2 += p2;
      rs3 += p3;
      pk[i] = pack_bf16(p0, p1);
      pk[i + 1] = pack_bf16(p2, p3);
    }
    tmem_st_32x16(tS + c * 16, pk);
  }
  return (rs0 + rs1) + (rs2 + rs3);
}

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, const AttnFwdParams p) {
  using L = AttnSmem<D>;
  constexpr int NB = L::NB;
  constexpr int ST = L::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sQ = sbase + L::Q_OFF;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  const uint32_t bar_q = smem_u32(bars);
  const uint32_t bar_kv_full = bar_q + 8;
  const uint32_t bar_kv_empty = bar_kv_full + ST * 8;
  const uint32_t bar_s_full = bar_kv_empty + ST * 8;
  const uint32_t bar_p_ready = bar_s_full + 16;
  const uint32_t bar_o_full = bar_p_ready + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1 + 2 * ST + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int npair = (p.S + 2 * ATT_BM - 1) / (2 * ATT_BM);
  const int nkb = (p.Skv + ATT_BN - 1) / ATT_BN;
  const int bh = p.B * p.Hq;
  const int pair = npair - 1 - int(blockIdx.x) / bh;  // longest (latest) query blocks are scheduled first
  const int rem = int(blockIdx.x) % bh;
  const int b = rem / p.Hq, h = rem % p.Hq;
  const int hk = h / (p.Hq / p.Hkv);
  // number of key blocks each tile visits (0: the tile lies past the end of the sequence)
  int n_t[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int qb = pair * 2 + t;
    const int q_last = min(qb * ATT_BM + ATT_BM - 1, p.S - 1);   // last query row of the tile
    n_t[t] = qb * ATT_BM >= p.S ? 0 : (p.causal ? min((q_last + p.q_off) / ATT_BN + 1, nkb) : nkb);
  }
  const int n_kv = max(n_t[0], n_t[1]);

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < ST; ++s) {
      mbar_init(bar_kv_full + s * 8, 1);
      mbar_init(bar_kv_empty + s * 8, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_s_full + i * 8, 1);
      mbar_init(bar_p_ready + i * 8, 128);
      mbar_init(bar_o_full + i * 8, 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tq);
    tma_prefetch_desc(&tk);
    tma_prefetch_desc(&tv);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  tfb::pdl_sync();   // set-up above touches no global memory; operands written by the previous kernel are read below
  const uint32_t tS0 = tmem_base, tO0 = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar_q, 2 * L::TILE);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int i = 0; i < NB; ++i)
          tma_load_3d(sQ + t * L::TILE + i * BOX_BYTES, &tq, bar_q, p.q_col0 + h * D + i * 64, (pair * 2 + t) * ATT_BM, b);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j % ST;
        if (!mbar_wait(bar_kv_empty + st * 8, ((j / ST) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) break;
        const uint32_t fb = bar_kv_full + st * 8;
        mbar_expect_tx(fb, 2 * L::TILE);
        const uint32_t sK = sbase + L::KV_OFF + st * 2 * L::TILE, sV = sK + L::TILE;
#pragma unroll
        for (int i = 0; i < NB; ++i) {
          tma_load_3d(sK + i * BOX_BYTES, &tk, fb, p.k_col0 + hk * D + i * 64, j * ATT_BN, b);
          tma_load_3d(sV + i * BOX_BYTES, &tv, fb, p.v_col0 + hk * D + i * 64, j * ATT_BN, b);
        }
      }
      if (*abort_flag) {  // unwinding: bounded wait for copies already issued
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc(FMT_BF16, FMT_BF16, false, false, ATT_BM, ATT_BN);
      constexpr uint32_t idesc_o = umma_idesc(FMT_BF16, FMT_BF16, false, true, ATT_BM, D);
      auto issue_s = [&](int t, int j) {
        const uint32_t sK = sbase + L::KV_OFF + (j % ST) * 2 * L::TILE;
        const uint32_t sQt = sQ + t * L::TILE;
        const uint32_t tS = tS0 + t * 128;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * BOX_BYTES + (k & 3) * 32;
          umma_f16_ss(tS, umma_smem_desc(sQt + off, 16, 1024), umma_smem_desc(sK + off, 16, 1024), idesc_s, k > 0);
        }
        umma_commit(bar_s_full + t * 8);
      };
      bool ok = mbar_wait(bar_q, 0, abort_flag, p.status, ST_TIMEOUT_FULL) &&
                (n_kv == 0 || mbar_wait(bar_kv_full, 0, abort_flag, p.status, ST_TIMEOUT_FULL));
      if (ok && n_kv > 0) {
        tc_fence_after();
#pragma unroll
        for (int t = 0; t < 2; ++t)
          if (n_t[t] > 0) issue_s(t, 0);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          const int st1 = (j + 1) % ST;
          if (!mbar_wait(bar_kv_full + st1 * 8, ((j + 1) / ST) & 1, abort_flag, p.status, ST_TIMEOUT_FULL)) break;
          tc_fence_after();
        }
        const int st = j % ST;
        const uint32_t sV = sbase + L::KV_OFF + st * 2 * L::TILE + L::TILE;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (!ok || j >= n_t[t]) continue;
          if (!mbar_wait(bar_p_ready + t * 8, j & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) {
            ok = false;
            continue;
          }
          tc_fence_after();
          const uint32_t tP = tS0 + t * 128;
          const uint32_t tO = tO0 + t * D;
#pragma unroll
          for (int k = 0; k < ATT_BN / 16; ++k) {
            // V_j tile is [key rows][64-col boxes]: MN-major B; 16 keys = 2048 B further, next 64 columns one box on
            umma_f16_ts(tO, tP + k * 8, umma_smem_desc(sV + k * 2048, BOX_BYTES, 1024), idesc_o, k > 0);
          }
          if (j + 1 < n_t[t]) issue_s(t, j + 1);              // its commit also covers the P V product above
          else umma_commit(bar_o_full + t * 8);
        }
        if (ok) umma_commit(bar_kv_empty + st * 8);
      }
    }
  } else {
    const int t = (warp - 2) >> 2;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int qb = pair * 2 + t;
    const int q_idx = qb * ATT_BM + r;
    const int n_mine = t ? n_t[1] : n_t[0];
    const uint32_t lane_off = uint32_t(quad * 32) << 16;
    const uint32_t tS = tS0 + t * 128 + lane_off;
    const uint32_t tO = tO0 + t * D + lane_off;
    const float sl2 = p.scale * 1.4426950408889634f;
    float m = -INFINITY, l = 0.f, alpha_prev = 1.f;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < n_mine; ++j) {
      if (!mbar_wait_warp(bar_s_full + t * 8, j & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int k0 = j * ATT_BN;
      const bool need_mask = (p.causal && k0 + ATT_BN - 1 > qb * ATT_BM + p.q_off) || (k0 + ATT_BN > p.Skv);
      const int k_lim = p.causal ? min(q_idx + p.q_off, p.Skv - 1) : (p.Skv - 1);  // last visible key index for this row
      const float mx = need_mask ? row_max<true>(tS, m, k0, k_lim) : row_max<false>(tS, m, k0, k_lim);
      if (j > 0) {  // O_t(j-1) is complete: the commit behind S_t(j) was issued after it
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tO + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], alpha_prev, __uint_as_float(v[i]));
        }
      }
      const float m_new = mx;
      const float mb = (m_new == -INFINITY) ? 0.f : m_new * sl2;
      const float alpha = (m == -INFINITY) ? 0.f : fast_exp2(m * sl2 - mb);
      const float rs = need_mask ? row_probs<true>(tS, sl2, mb, k0, k_lim) : row_probs<false>(tS, sl2, mb, k0, k_lim);
      l = fmaf(l, alpha, rs);
      m = m_new;
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar_p_ready + t * 8);
      alpha_prev = alpha;
    }
    if (ok && n_mine > 0) {
      if (mbar_wait_warp(bar_o_full + t * 8, 0, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tO + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], alpha_prev, __uint_as_float(v[i]));
        }
        if (q_idx < p.S) {
          const float inv = l > 0.f ? 1.f / l : 0.f;
          __nv_bfloat16* op = p.O + ((long long)b * p.S + q_idx) * p.ldo + h * D;
#pragma unroll
          for (int c = 0; c < D / 8; ++c) {
            uint4 u;
            u.x = pack_bf16(o[c * 8 + 0] * inv, o[c * 8 + 1] * inv);
            u.y = pack_bf16(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv);
            u.z = pack_bf16(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv);
            u.w = pack_bf16(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv);
            *reinterpret_cast<uint4*>(op + c * 8) = u;
          }
          if (p.lse) p.lse[((long long)b * p.Hq + h) * p.S + q_idx] = m * p.scale + logf(l);
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

template <int D>
static int launch_attn_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnFwdParams& p,
                           cudaStream_t st) {
  using L = AttnSmem<D>;
  static DeviceOnce once;
  auto kern = attn_fwd_kernel<D>;
  if (int e = ensure_dyn_smem(once, kern, L::TOTAL)) return e;
  const int npair = (p.S + 2 * ATT_BM - 1) / (2 * ATT_BM);
  tfb::launch_k(kern, npair * p.B * p.Hq, ATT_THREADS, L::TOTAL, st, tq, tk, tv, p);
  return int(cudaGetLastError());
}

}  // namespace tfb

// q, k, v: bf16 buffers whose rows are tokens (b * S + s) with pitches ldq / ldk / ldv (elements);
// head h of q starts at column q_col0 + h * D of its row (likewise k, v with the kv head index), so
// the three pointers may be the same fused [T, (Hq + 2 Hkv) D] projection output.
// o: [B*S, ldo] bf16, head h at column h * D.  lse: [B, Hq, S] fp32 (may be null).
//
// tfb_attn_fwd_kv: the keys / values have Skv >= S rows per sequence (k, v rows are b * Skv + s) and the S queries are the
// last S positions: with `causal`, query i sees keys 0 .. i + (Skv - S).  This is the prefill of a prompt suffix behind a
// cached prefix (the prefix keys come out of the paged cache, see tfb_kv_gather).
TFB_API int tfb_attn_fwd_kv(const void* q, long long ldq, int q_col0, const void* k, long long ldk, int k_col0,
                            const void* v, long long ldv, int v_col0, void* o, long long ldo, float* lse, int B, int S,
                            int Skv, int Hq, int Hkv, int D, float scale, int causal, int* status, void* stream);

TFB_API int tfb_attn_fwd(const void* q, long long ldq, int q_col0, const void* k, long long ldk, int k_col0,
                         const void* v, long long ldv, int v_col0, void* o, long long ldo, float* lse, int B, int S,
                         int Hq, int Hkv, int D, float scale, int causal, int* status, void* stream) {
  return tfb_attn_fwd_kv(q, ldq, q_col0, k, ldk, k_col0, v, ldv, v_col0, o, ldo, lse, B, S, S, Hq, Hkv, D, scale, causal, status,
                         stream);
}

TFB_API int tfb_attn_fwd_kv(const void* q, long long ldq, int q_col0, const void* k, long long ldk, int k_col0,
                            const void* v, long long ldv, int v_col0, void* o, long long ldo, float* lse, int B, int S,
                            int Skv, int Hq, int Hkv, int D, float scale, int causal, int* status, void* stream) {
  using namespace tfb;
  if ((D != 64 && D != 128) || Hkv <= 0 || Hq % Hkv || B <= 0 || S <= 0 || Skv < S) return TFB_ERR_ARG;
  if ((q_col0 | k_col0 | v_col0) & 7 || (ldo & 7) || (reinterpret_cast<uintptr_t>(o) & 15)) return TFB_ERR_ARG;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_tmap_3d(&tq, q, 2, ldq, S, B, ldq * 2, ldq * 2 * S, 64, 128, 1))) return rc;
  if ((rc = make_tmap_3d(&tk, k, 2, ldk, Skv, B, ldk * 2, ldk * 2 * Skv, 64, 128, 1))) return rc;
  if ((rc = make_tmap_3d(&tv, v, 2, ldv, Skv, B, ldv * 2, ldv * 2 * Skv, 64, 128, 1))) return rc;
  AttnFwdParams p;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.Skv = Skv; p.q_off = Skv - S;
  p.scale = scale; p.causal = causal;
  p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0;
  p.O = static_cast<__nv_bfloat16*>(o); p.ldo = ldo; p.lse = lse; p.status = status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return D == 64 ? launch_attn_fwd<64>(tq, tk, tv, p, st) : launch_attn_fwd<128>(tq, tk, tv, p, st);
}
