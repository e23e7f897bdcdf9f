// bf16 GEMM for sm_100a: C[M,N] = epilogue(A * B), fp32 accumulation in tensor memory.
//
// Design (one persistent CTA per SM, 320 threads, warp-specialised):
//   warp 0      TMA producer  : cp.async.bulk.tensor tiles of A and B into a 4-stage shared-memory ring
//   warp 1      MMA issuer    : one thread issues tcgen05.mma (128 x BN x 16) per 32 bytes of K and
//                               commits stage-release / accumulator-ready mbarriers
//   warps 2..9  epilogue      : tcgen05.ld the 128 x BN fp32 accumulator (one row per thread, two warps per TMEM lane
//                               quadrant, each taking half of the columns),
//                               apply alpha / bias / activation / residual, stage 32-row x 128-byte slabs in
//                               shared memory (128-byte swizzle, conflict-free) and hand them to TMA: a tiled
//                               store for bf16 / fp32 outputs, a tiled fp32 reduce-add for accumulating outputs
//                               (weight gradients, split-K).  Ragged edges are clipped by the tensor map.
// The accumulator is double-buffered in TMEM (2 x BN columns), so the epilogue of tile i overlaps
// the main loop of tile i+1.  Either operand may be K-major (reduction dim contiguous) or MN-major
// (output dim contiguous): the forward, data-gradient and weight-gradient GEMMs of a linear layer
// all run without a transpose copy.  Small-output / long-K problems (weight gradients) are split
// along K across CTAs and summed into the fp32 gradient buffer by TMA reduce-add from the staged epilogue.
//
// This replaces the reference's scalar one-thread-per-output kernels
// (src/backend/gpu_compute_cuda.cpp:68 gemm_kernel; src/kernel/kernel_gemm.cpp:26 scalar_gemm_bt).
#include <string.h>

#include <mutex>
#include "tfb_host.h"
#include "tfb_ptx.cuh"

TFB_BOUNDS_DEFINE(gemm_bf16)

namespace tfb {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int STAGES = 4;
constexpr int EPI_WARPS = 8;   // two warps per TMEM lane quadrant, each draining half of the tile's columns
constexpr int GEMM_THREADS = 64 + 32 * EPI_WARPS;

enum : int { TP_AG = 1, TP_RS = 2, TP_WG = 4 };

// Rows of one operand that live as row shards on `world` ranks and are copied into a local buffer in 128-row blocks.
struct GatherSpec {
  int rank, world, rows_per_shard, row_len, epoch, rows;  // rows: rows of the operand that the product touches
  int src_is_full;   // 1: src[r] is rank r's whole gathered buffer (block b at b * 128 * ld); 0: rank r's shard only
  int skip_local;    // 1: this rank's rows are already in place in dst
  int* ready;        // local int[padded rows / 128]: ready[b] >= epoch once block b has landed in dst
  const __nv_bfloat16* const* src;   // [world] base pointers (peer memory)
  __nv_bfloat16* dst;
  long long ld;
};

// C tensor maps of the reduce-scatter form: one per destination rank's staging buffer (peer memory).
constexpr int RS_TMA_MAX_WORLD = 8;
struct PeerMaps {
  CUtensorMap m[RS_TMA_MAX_WORLD];
};

struct GemmParams {
  int M, N, K;
  void* C;
  long long ldc;
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, ldr] or null (bf16 output mode only)
  long long ldr;
  float alpha;
  int act;       // 0 none, 1 relu, 2 gelu(tanh), 3 silu
  int out_mode;  // 0 bf16 store, 1 fp32 store, 2 fp32 atomic accumulate
  int splits, kb_per_split, tiles_m, tiles_n;
  int raster_gn;   // tile order: groups of raster_gn tile columns; inside a group n runs fastest, then m
  // grouped (mixture-of-experts) modes; expert segments are padded to multiples of 128 rows
  //   1: rows of A / C grouped by expert, B = [E, ...] picked per 128-row tile (forward, data gradient)
  //   2: reduction dimension grouped by expert, C = [E, M, N] (weight gradient of every expert in one launch)
  int group_mode, num_experts;
  const int* expert_of_mtile;   // mode 1: expert of every 128-row tile (-1 = padding, skipped)
  const int* seg_start;         // mode 2: [E + 1] first row of every expert segment
  long long c_expert_stride;    // mode 2: elements between the C matrices of consecutive experts
  // fusion with the collective that precedes / follows the GEMM (see tp_fused.cu); tp_mode is a set of bits:
  //   TP_AG (1): all-gather -> GEMM.  A is the gathered [M, K] buffer in symmetric memory; this rank's rows are in
  //      place, the first `copy_ctas` CTAs of the grid pull the other ranks' rows over NVLink in 128-row blocks
  //      and raise ready[block] = epoch; the TMA producer waits for a block's flag before loading from it.
  //   TP_RS (2): GEMM -> reduce-scatter.  Output rows of shard d are stored straight into rank d's staging buffer
  //      [world, rows_per_shard, N] at slot `rank` (peer stores from the epilogue); remote shards first.
  //   TP_WG (4): weight all-gather -> GEMM (ZeRO-3 / FSDP).  Every rank of the data-parallel group keeps one row
  //      shard of B (128-row blocks) in symmetric memory; the copy CTAs pull all shards (the local one first) into the
  //      local gather buffer B and the TMA producer waits for the flag of every block a B tile touches.  Tiles
  //      (K-major B) or k-blocks (MN-major B) that use the local shard come first.
  //   TP_AG and TP_WG may be combined (column-parallel product of a sharded weight), and so may TP_RS and TP_WG.
  int tp_mode, tp_copy_ctas;
  GatherSpec ag, wg;
  int wg_n_shift, wg_k_shift;   // TP_WG: first n tile / k block of the local shard
  int rs_rank, rs_world, rs_rows_per_shard;
  __nv_bfloat16* const* rs_peer_c;
  int c_tma;     // 1: the epilogue goes through shared memory and the C tensor map (aligned, dense C)
  int* status;
};

// Decodes work item w into tile coordinates / k-block range / expert.  Returns false when there is nothing to do.
struct WorkItem {
  int m0, n0, kb0, kb1, expert;  // n0 is the tile index along N (the kernel scales it by its BN)
};
__device__ __forceinline__ bool decode_work(const GemmParams& p, int w, int total_kb, WorkItem& it) {
  if (p.group_mode == 2) {
    const int tiles = p.tiles_m * p.tiles_n;
    it.expert = w / tiles;
    const int tile = w - it.expert * tiles;
    it.m0 = (tile / p.tiles_n) * BM;
    it.kb0 = p.seg_start[it.expert] / BK;
    it.kb1 = p.seg_start[it.expert + 1] / BK;
    it.n0 = tile % p.tiles_n;
    return it.kb1 > it.kb0;
  }
  const int tile = w / p.splits, split = w - tile * p.splits;
  // Grouped raster.  A wave of 148 tiles in plain row-major order spans every tile column, i.e. reads all of B once per
  // wave; with a wide N (B larger than L2) that is one DRAM pass over B per wave.  In groups of raster_gn columns a wave
  // covers a roughly square patch, the group's slice of B stays in L2 for the whole sweep over M, and A is streamed once
  // per group.  raster_gn == tiles_n is the plain row-major order, raster_gn == 1 column-major.
  const int per_group = p.raster_gn * p.tiles_m;
  const int grp = tile / per_group, within = tile - grp * per_group;
  const int gn = min(p.raster_gn, p.tiles_n - grp * p.raster_gn);
  const int m_idx = within / gn, n_idx = grp * p.raster_gn + (within - m_idx * gn);
  it.m0 = m_idx * BM;
  it.n0 = n_idx;
  it.kb0 = split * p.kb_per_split;
  it.kb1 = min(total_kb, it.kb0 + p.kb_per_split);
  it.expert = 0;
  if (p.group_mode == 1) {
    it.expert = p.expert_of_mtile[m_idx];
    if (it.expert < 0) return false;
    TFB_BOUNDS(it.expert < p.num_experts, 12, it.expert, p.num_experts);
    if (it.expert >= p.num_experts) return false;
  }
  if ((p.tp_mode & TP_WG) && p.wg_n_shift >= 0) {
    // K-major gathered B: the column groups are visited starting at the local shard's columns, in the order in which
    // the copy CTAs deliver the peers' rows
    it.n0 = (n_idx + p.wg_n_shift) % p.tiles_n;
  }
  if (p.tp_mode & TP_AG) {
    // rotate the row-block order: start with the local shard (already in place)
    it.m0 = ((it.m0 / BM + p.ag.rank * (p.ag.rows_per_shard / BM)) % p.tiles_m) * BM;
  } else if (p.tp_mode & TP_RS) {
    // ... and for the reduce-scatter end with it: remote shards are stored first
    it.m0 = ((it.m0 / BM + (p.rs_rank + 1) * (p.rs_rows_per_shard / BM)) % p.tiles_m) * BM;
  }
  return true;
}

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Copy role of the gather -> GEMM fusions: pulls 128-row blocks of the ranks' shards into the local gathered buffer
// and publishes each block with a release store.  Contiguous blocks (row pitch == row length) travel as untiled bulk
// copies through a shared-memory ring driven by one thread: 16 KB chunks in the CTA's operand-stage memory (8 slots for
// the 128-wide tile configuration, 12 for the 256-wide one), all but two slots' worth of loads in flight, so that about
// a dozen CTAs keep more than a megabyte in flight, which is what a ~2 us NVLink round trip needs to run near link
// bandwidth.  Strided rows fall back to per-thread 16-byte copies.
constexpr int COPY_CHUNK = 16384;
constexpr int COPY_MAX_SLOTS = 12;

__device__ __forceinline__ bool copy_block_bulk(const __nv_bfloat16* src, __nv_bfloat16* dst, long long bytes, uint32_t ring,
                                                uint32_t bars, uint32_t& seq, volatile int* abort_flag, int* status,
                                                const uint32_t COPY_SLOTS) {
  const int nt = int((bytes + COPY_CHUNK - 1) / COPY_CHUNK);
  const char* s8 = reinterpret_cast<const char*>(src);
  char* d8 = reinterpret_cast<char*>(dst);
  int nl = 0, ns = 0;
  const uint32_t seq0 = seq;
  while (ns < nt) {
    while (nl < nt && nl - ns < int(COPY_SLOTS) - 2) {
      tma_store_wait_read<2>();   // at most two stores still reading: the one that last used this slot is not among them
      const uint32_t q = seq0 + nl, slot = q % COPY_SLOTS;
      const uint32_t sz = uint32_t(min((long long)COPY_CHUNK, bytes - (long long)nl * COPY_CHUNK));
      mbar_expect_tx(bars + slot * 8, sz);
      bulk_load(ring + slot * COPY_CHUNK, s8 + (long long)nl * COPY_CHUNK, sz, bars + slot * 8);
      ++nl;
    }
    const uint32_t q = seq0 + ns, slot = q % COPY_SLOTS, parity = (q / COPY_SLOTS) & 1u;
    if (!mbar_wait(bars + slot * 8, parity, abort_flag, status, ST_TIMEOUT_FULL)) {
      // give the loads already issued a bounded time to land before shared memory goes away
      const uint64_t t0 = globaltimer_ns();
      for (int j = ns; j < nl; ++j) {
        const uint32_t qq = seq0 + j;
        while (!mbar_try_wait(bars + (qq % COPY_SLOTS) * 8, (qq / COPY_SLOTS) & 1u)) {
          if (globaltimer_ns() - t0 > 2000000ull) { report(status, ST_TIMEOUT_DRAIN); break; }
        }
      }
      tma_store_wait<0>();
      return false;
    }
    fence_proxy_async_smem();
    const uint32_t sz = uint32_t(min((long long)COPY_CHUNK, bytes - (long long)ns * COPY_CHUNK));
    bulk_store(d8 + (long long)ns * COPY_CHUNK, ring + slot * COPY_CHUNK, sz);
    tma_store_commit();
    ++ns;
  }
  seq = seq0 + nt;
  tma_store_wait<0>();       // the block is in the gathered buffer
  fence_proxy_async_all();   // bulk-copy writes before the flag that publishes them
  return true;
}

__device__ __forceinline__ void copy_block_threads(const __nv_bfloat16* src, __nv_bfloat16* dst, long long ld, long long row_chunks,
                                                   int rows) {
  const long long total = (long long)rows * row_chunks;
  for (long long c = threadIdx.x; c < total; c += 4 * blockDim.x) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long cc = c + (long long)u * blockDim.x;
      if (cc < total) {
        const long long r = cc / row_chunks, k = cc % row_chunks;
        v[u] = *reinterpret_cast<const uint4*>(src + r * ld + k * 8);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long cc = c + (long long)u * blockDim.x;
      if (cc < total) {
        const long long r = cc / row_chunks, k = cc % row_chunks;
        *reinterpret_cast<uint4*>(dst + r * ld + k * 8) = v[u];
      }
    }
  }
}

__device__ __forceinline__ void tp_copy_role(const GemmParams& p, int cta, int ncopy, uint32_t ring, uint32_t bars,
                                             volatile int* abort_flag, const uint32_t slots) {
  if (threadIdx.x == 0) {
    for (uint32_t i = 0; i < slots; ++i) mbar_init(bars + i * 8, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  const int nA = (p.tp_mode & TP_AG) ? (p.ag.world - 1) * (p.ag.rows_per_shard / BM) : 0;
  const int nB = (p.tp_mode & TP_WG) ? (p.wg.world - (p.wg.skip_local ? 1 : 0)) * (p.wg.rows_per_shard / BM) : 0;
  uint32_t seq = 0;
  for (int idx = cta; idx < nA + nB; idx += ncopy) {
    const GatherSpec& g = idx < nA ? p.ag : p.wg;
    const int j = idx < nA ? idx : idx - nA;
    const int bps = g.rows_per_shard / BM;
    const int peer = (g.rank + (g.skip_local ? 1 : 0) + j / bps) % g.world;
    const int b = j % bps, blk = peer * bps + b;  // block inside the shard / inside the gathered operand
    if (blk * BM >= g.rows) continue;             // padding rows: nothing reads them
    TFB_BOUNDS(peer >= 0 && peer < g.world && blk >= 0, 11, blk, g.world * bps);
    const __nv_bfloat16* src = g.src[peer] + (long long)(g.src_is_full ? blk : b) * BM * g.ld;
    __nv_bfloat16* dst = g.dst + (long long)blk * BM * g.ld;
    if (g.ld == g.row_len) {
      // after a copy that ran out of time nothing more is published: the consumers' own bounded waits end the kernel
      if (threadIdx.x == 0 && !*abort_flag &&
          copy_block_bulk(src, dst, (long long)BM * g.row_len * 2, ring, bars, seq, abort_flag, p.status, slots)) {
        __threadfence();
        asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(g.ready + blk), "r"(g.epoch) : "memory");
      }
    } else {
      copy_block_threads(src, dst, g.ld, (long long)g.row_len / 8, BM);
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence();
        asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(g.ready + blk), "r"(g.epoch) : "memory");
      }
    }
  }
}

template <int BN>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STG_OFF = STAGES * STAGE_BYTES;   // epilogue staging slabs follow the operand stages
  // epilogue staging: one 32-row x 128-byte slab per epilogue warp, double-buffered where shared memory allows (the
  // 256-wide tile leaves room for one slab per warp next to its four operand stages)
  static constexpr int STG_BUFS = (BN == 256) ? 1 : 2;
  static constexpr int STG_BYTES = EPI_WARPS * STG_BUFS * 4096;
  static constexpr int BAR_OFF = STG_OFF + STG_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;  // + barriers + alignment slack
};

__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case 1: return fmaxf(v, 0.f);
    case 2: return gelu_tanh(v);
    case 3: return silu(v);
    default: return v;
  }
}

template <bool A_MN, bool B_MN, int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ CUtensorMap tma_c, const __grid_constant__ PeerMaps tma_peers, const GemmParams p) {
  using L = SmemLayout<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + STAGES * 8;
  const uint32_t bar_tfull = bar_empty + STAGES * 8;
  const uint32_t bar_tempty = bar_tfull + 2 * 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  // copy CTAs take the lowest block indices so that they are scheduled first: a GEMM CTA may wait for a copy
  // CTA, never the other way round
  const int ncopy = (p.tp_mode & (TP_AG | TP_WG)) ? p.tp_copy_ctas : 0;
  const int nctas = int(gridDim.x) - ncopy;  // CTAs that run GEMM tiles
  const int cta = int(blockIdx.x) - ncopy;
  if (cta < 0) {
    tfb::pdl_sync();
    constexpr uint32_t kSlots = (STAGES * L::STAGE_BYTES / COPY_CHUNK) < COPY_MAX_SLOTS ? (STAGES * L::STAGE_BYTES / COPY_CHUNK)
                                                                                          : COPY_MAX_SLOTS;
    tp_copy_role(p, int(blockIdx.x), ncopy, smem_base, bar_full, abort_flag, kSlots);
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + s * 8, 1);
      mbar_init(bar_empty + s * 8, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + b * 8, 1);
      mbar_init(bar_tempty + b * 8, 32 * EPI_WARPS);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    if (p.c_tma) tma_prefetch_desc(&tma_c);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  tfb::pdl_sync();   // set-up above touches no global memory; operands written by the previous kernel are read below

  const int total_kb = (p.K + BK - 1) / BK;
  const int num_work = p.tiles_m * p.tiles_n * (p.group_mode == 2 ? p.num_experts : p.splits);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = cta; w < num_work && ok; w += nctas) {
        WorkItem it;
        if (!decode_work(p, w, total_kb, it)) continue;
        const int m0 = it.m0, n0 = it.n0 * BN, kb0 = it.kb0, kb1 = it.kb1;
        const int bz = p.group_mode == 1 ? it.expert : 0;
        auto wait_block = [&](const GatherSpec& g, int blk) -> bool {   // block `blk` of a gathered operand has landed locally
          if (g.skip_local && blk / (g.rows_per_shard / BM) == g.rank) return true;
          const uint64_t t0 = globaltimer_ns();
          uint32_t spins = 0;
          while (ld_acquire_gpu(g.ready + blk) < g.epoch) {
            if ((++spins & 255u) == 0u && (*abort_flag || globaltimer_ns() - t0 > TFB_WAIT_NS)) {
              report(p.status, ST_TIMEOUT_FLAG);
              *abort_flag = 1;
              return false;
            }
          }
          asm volatile("fence.proxy.async;" ::: "memory");  // the copy CTAs' writes -> visible to the TMA reads below
          return true;
        };
        if (p.tp_mode & TP_AG) {
          if (!wait_block(p.ag, m0 / BM)) { ok = false; break; }
        }
        if ((p.tp_mode & TP_WG) && !B_MN) {
          for (int r0 = n0; r0 < n0 + BN && r0 < p.N && ok; r0 += BM) ok = wait_block(p.wg, r0 / BM);
          if (!ok) break;
        }
        int last_blk = -1;
        for (int kb = kb0; kb < kb1; ++kb) {
          const int kbr = ((p.tp_mode & TP_WG) && B_MN) ? (kb + p.wg_k_shift) % total_kb : kb;   // local shard's rows first
          if ((p.tp_mode & TP_WG) && B_MN) {
            const int blk = kbr * BK / BM;
            if (blk != last_blk) {
              if (!wait_block(p.wg, blk)) { ok = false; break; }
              last_blk = blk;
            }
          }
          if (!mbar_wait(bar_empty + stage * 8, phase ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t fb = bar_full + stage * 8;
          mbar_expect_tx(fb, L::STAGE_BYTES);
          const uint32_t sa = smem_base + stage * L::STAGE_BYTES;
          const uint32_t sb = sa + L::A_BYTES;
          const int k0 = kbr * BK;
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tma_a, fb, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * 8192, &tma_a, fb, m0 + j * 64, k0);
          }
          if constexpr (!B_MN) {
            tma_load_3d(sb, &tma_b, fb, k0, n0, bz);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_3d(sb + j * 8192, &tma_b, fb, n0 + j * 64, k0, bz);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Unwinding: give copies already issued a bounded time to land before shared memory goes away.
        const uint64_t t0 = globaltimer_ns();
        for (int s = 0; s < STAGES; ++s) {
          const uint32_t par = (s < stage) ? phase : (phase ^ 1);
          while (!mbar_try_wait(bar_full + s * 8, par)) {
            if (globaltimer_ns() - t0 > 2000000ull) { report(p.status, ST_TIMEOUT_DRAIN); break; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(FMT_BF16, FMT_BF16, A_MN, B_MN, BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int abuf = 0;
      uint32_t aphase = 0;
      bool ok = true;
      for (int w = cta; w < num_work && ok; w += nctas) {
        WorkItem it;
        if (!decode_work(p, w, total_kb, it)) continue;
        const int kb0 = it.kb0, kb1 = it.kb1;
        if (!mbar_wait(bar_tempty + abuf * 8, aphase ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + abuf * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(bar_full + stage * 8, phase, abort_flag, p.status, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * L::STAGE_BYTES;
          const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? umma_smem_desc(sa + k * 2048, 8192, 1024)
                                        : umma_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_smem_desc(sb + k * 2048, 8192, 1024)
                                        : umma_smem_desc(sb + k * 32, 16, 1024);
            umma_f16_ss(tmem_d, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(bar_empty + stage * 8);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(bar_tfull + abuf * 8);
        abuf ^= 1;
        if (abuf == 0) aphase ^= 1;
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    int abuf = 0;
    uint32_t aphase = 0;
    const bool vec_ok_bf16 = ((p.ldc & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    const bool vec_ok_f32 = ((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    const bool vec_ok_res =
        p.residual && ((p.ldr & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0);
    const int ew = warp - 2;           // epilogue warp 0..7
    const int half = ew >> 2;          // which half of the tile's columns this warp drains
    const uint32_t stg_u32 = smem_base + L::STG_OFF + ew * (L::STG_BUFS * 4096);
    int sbuf = 0;
    for (int w = cta; w < num_work; w += nctas) {
      WorkItem it;
      if (!decode_work(p, w, total_kb, it)) continue;
      const int m0 = it.m0, n0 = it.n0 * BN;
      const long long c_off = p.group_mode == 2 ? (long long)it.expert * p.c_expert_stride : 0;
      if (!mbar_wait_warp(bar_tfull + abuf * 8, aphase, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const int row = m0 + quad * 32 + lane;
      const uint32_t taddr0 = tmem_base + abuf * BN + (uint32_t(quad * 32) << 16);
      if (p.c_tma) {
        // ---- staged epilogue: registers -> swizzled shared-memory slab -> TMA store / reduce-add ----
        const int slab_row0 = m0 + quad * 32;
        const bool slab_live = slab_row0 < p.M;            // warp-uniform
        const uint32_t xr = uint32_t(lane & 7);
        if (p.out_mode == 0) {
#pragma unroll 1
          for (int c = half * (BN / 128); c < (half + 1) * (BN / 128); ++c) {
            const int col0 = n0 + c * 64;
            if (col0 >= p.N) break;
            uint32_t r0[32], r1[32];
            tmem_ld_32x32(taddr0 + c * 64, r0);
            tmem_ld_32x32(taddr0 + c * 64 + 32, r1);
            tmem_ld_wait();
            if (!slab_live) continue;
            float v[64];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              v[j] = __uint_as_float(r0[j]) * p.alpha;
              v[32 + j] = __uint_as_float(r1[j]) * p.alpha;
            }
            if (p.bias) {
#pragma unroll
              for (int j = 0; j < 64; ++j)
                if (col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
            }
            if (p.act) {
#pragma unroll
              for (int j = 0; j < 64; ++j) v[j] = apply_act(v[j], p.act);
            }
            if (p.residual && row < p.M) {
              const __nv_bfloat16* rp = p.residual + (long long)row * p.ldr + col0;
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                if (vec_ok_res && col0 + q * 8 + 8 <= p.N) {
                  const uint4 u = *reinterpret_cast<const uint4*>(rp + q * 8);
                  const uint32_t uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                  for (int h = 0; h < 4; ++h) {
                    const float2 f = unpack_bf16(uu[h]);
                    v[q * 8 + h * 2] += f.x;
                    v[q * 8 + h * 2 + 1] += f.y;
                  }
                } else {
#pragma unroll
                  for (int j = 0; j < 8; ++j)
                    if (col0 + q * 8 + j < p.N) v[q * 8 + j] += __bfloat162float(rp[q * 8 + j]);
                }
              }
            }
            if (lane == 0) tma_store_wait_read<L::STG_BUFS - 1>();   // the slab about to be rewritten has been read by its copy
            __syncwarp();
            const uint32_t slab = stg_u32 + sbuf * 4096 + lane * 128;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              st_shared_v4(slab + ((uint32_t(q) ^ xr) << 4), pack_bf16(v[q * 8 + 0], v[q * 8 + 1]), pack_bf16(v[q * 8 + 2], v[q * 8 + 3]),
                           pack_bf16(v[q * 8 + 4], v[q * 8 + 5]), pack_bf16(v[q * 8 + 6], v[q * 8 + 7]));
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (p.tp_mode & TP_RS) {
                // rows of shard d go to rank d's staging buffer, slot `rank`: one 32-row x 128-byte slab per copy, so the
                // bytes cross NVLink in whole lines (tile rows never straddle two shards: shards are multiples of 128 rows)
                const int d = slab_row0 / p.rs_rows_per_shard;
                tma_store_3d(&tma_peers.m[d], stg_u32 + sbuf * 4096, col0,
                             p.rs_rank * p.rs_rows_per_shard + (slab_row0 - d * p.rs_rows_per_shard), 0);
              } else {
                tma_store_3d(&tma_c, stg_u32 + sbuf * 4096, col0, slab_row0, 0);
              }
              tma_store_commit();
            }
            sbuf ^= (L::STG_BUFS - 1);
          }
        } else {
          const int cz = p.group_mode == 2 ? it.expert : 0;
#pragma unroll 1
          for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
            const int col0 = n0 + c * 32;
            if (col0 >= p.N) break;
            uint32_t r[32];
            tmem_ld_32x32(taddr0 + c * 32, r);
            tmem_ld_wait();
            if (!slab_live) continue;
            if (lane == 0) tma_store_wait_read<L::STG_BUFS - 1>();
            __syncwarp();
            const uint32_t slab = stg_u32 + sbuf * 4096 + lane * 128;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              st_shared_v4(slab + ((uint32_t(q) ^ xr) << 4), __float_as_uint(__uint_as_float(r[q * 4]) * p.alpha),
                           __float_as_uint(__uint_as_float(r[q * 4 + 1]) * p.alpha), __float_as_uint(__uint_as_float(r[q * 4 + 2]) * p.alpha),
                           __float_as_uint(__uint_as_float(r[q * 4 + 3]) * p.alpha));
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (p.out_mode == 2) tma_reduce_add_3d(&tma_c, stg_u32 + sbuf * 4096, col0, slab_row0, cz);
              else tma_store_3d(&tma_c, stg_u32 + sbuf * 4096, col0, slab_row0, cz);
              tma_store_commit();
            }
            sbuf ^= (L::STG_BUFS - 1);
          }
        }
        tc_fence_before();
        mbar_arrive(bar_tempty + abuf * 8);
        abuf ^= 1;
        if (abuf == 0) aphase ^= 1;
        continue;
      }
#pragma unroll 1
      for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr0 + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row >= p.M || col0 >= p.N) continue;
        const bool full = col0 + 32 <= p.N;
        if (p.out_mode == 0) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
          if (p.bias) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (full || col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
          }
          if (p.act) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], p.act);
          }
          if (p.residual) {
            const __nv_bfloat16* rp = p.residual + (long long)row * p.ldr + col0;
            if (full && vec_ok_res) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 u = *reinterpret_cast<const uint4*>(rp + q * 8);
                const uint32_t uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                  const float2 f = unpack_bf16(uu[h]);
                  v[q * 8 + h * 2] += f.x;
                  v[q * 8 + h * 2 + 1] += f.y;
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) v[j] += __bfloat162float(rp[j]);
            }
          }
          __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
          if (p.tp_mode & TP_RS) {  // row belongs to shard d: store into rank d's staging slot for this rank
            const int d = row / p.rs_rows_per_shard;
            cp = p.rs_peer_c[d] + ((long long)p.rs_rank * p.rs_rows_per_shard + (row - d * p.rs_rows_per_shard)) * p.ldc + col0;
          }
          if (full && vec_ok_bf16) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 u;
              u.x = pack_bf16(v[q * 8 + 0], v[q * 8 + 1]);
              u.y = pack_bf16(v[q * 8 + 2], v[q * 8 + 3]);
              u.z = pack_bf16(v[q * 8 + 4], v[q * 8 + 5]);
              u.w = pack_bf16(v[q * 8 + 6], v[q * 8 + 7]);
              *reinterpret_cast<uint4*>(cp + q * 8) = u;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) cp[j] = __float2bfloat16(v[j]);
          }
        } else {
          float* cp = reinterpret_cast<float*>(p.C) + c_off + (long long)row * p.ldc + col0;
          if (p.out_mode == 1) {
            if (full && vec_ok_f32) {
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                float4 f = make_float4(__uint_as_float(r[q * 4]) * p.alpha, __uint_as_float(r[q * 4 + 1]) * p.alpha,
                                       __uint_as_float(r[q * 4 + 2]) * p.alpha, __uint_as_float(r[q * 4 + 3]) * p.alpha);
                *reinterpret_cast<float4*>(cp + q * 4) = f;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) cp[j] = __uint_as_float(r[j]) * p.alpha;
            }
          } else {
            if (full && vec_ok_f32) {
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(cp + q * 4),
                             "f"(__uint_as_float(r[q * 4]) * p.alpha), "f"(__uint_as_float(r[q * 4 + 1]) * p.alpha),
                             "f"(__uint_as_float(r[q * 4 + 2]) * p.alpha), "f"(__uint_as_float(r[q * 4 + 3]) * p.alpha)
                             : "memory");
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) atomicAdd(cp + j, __uint_as_float(r[j]) * p.alpha);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(bar_tempty + abuf * 8);
      abuf ^= 1;
      if (abuf == 0) aphase ^= 1;
    }
    if (p.c_tma && lane == 0) tma_store_wait<0>();   // staged slabs must be out of shared memory before the CTA ends
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// -------------------------------------------------------------------------------------------------
// host launcher
// -------------------------------------------------------------------------------------------------
template <bool A_MN, bool B_MN, int BN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const PeerMaps& tpeers, const GemmParams& p,
                  int grid, cudaStream_t st) {
  using L = SmemLayout<BN>;
  static DeviceOnce once;
  auto kern = gemm_bf16_kernel<A_MN, B_MN, BN>;
  if (int e = ensure_dyn_smem(once, kern, L::TOTAL)) return e;
  tfb::launch_k(kern, grid, GEMM_THREADS, L::TOTAL, st, ta, tb, tc, tpeers, p);
  return int(cudaGetLastError());
}

}  // namespace tfb

struct TfbGemmGroup {
  int mode;                    // 0 dense, 1 rows grouped (B has a leading expert dim), 2 reduction grouped (C has one)
  int num_experts;
  const int* expert_of_mtile;  // mode 1 (device)
  const int* seg_start;        // mode 2 (device, [E + 1])
  long long b_expert_stride;   // mode 1: elements between consecutive experts' B matrices
  long long c_expert_stride;   // mode 2: elements between consecutive experts' C matrices
};

struct TfbGemmTp {
  int mode;               // bits: 1 all-gather -> GEMM, 2 GEMM -> reduce-scatter, 4 weight gather -> GEMM
  int rank, world;        // tensor-parallel group (bits 1, 2)
  int copy_ctas;          // bits 1, 4: CTAs that move data instead of multiplying
  int epoch;              // bit 1: value of a ready flag once its block has landed
  int* ready;             // bit 1: local int[M / 128]
  const void* peer_a;     // bit 1: device array [world] of gathered-A base pointers
  const void* peer_c;     // bit 2: device array [world] of staging-buffer base pointers
  const void* const* peer_c_host;   // bit 2, optional: the same addresses in host memory; with them (and world <= 8) the
                                    // partial tiles leave through TMA stores instead of per-thread stores
  // bit 4: B is the local gather buffer of a weight whose row shards ([wg_rows / wg_world, ldb] each, 128-row blocks)
  // live on the wg_world ranks of the data-parallel group
  int wg_rank, wg_world, wg_epoch, wg_rows;   // wg_rows: padded row count, a multiple of 128 * wg_world
  int* wg_ready;          // local int[wg_rows / 128]
  const void* wg_src;     // device array [wg_world] of shard base pointers
  int wg_skip_local;      // 1: the caller has already copied this rank's shard into B (the copy CTAs then move remote rows only)
};

// ---------------------------------------------------------------------------------------------------------------------
// Small-M path (decode batches): a product with few output tiles cannot fill the machine, and split-K needs an fp32
// accumulation target.  The partial products go into a per-device fp32 workspace with TMA reduce-add, and a finalize
// kernel applies bias / activation / residual and writes the requested type.  The workspace is allocated once
// (256 MB: up to 256 rows x 262144 columns); a shape that needs more takes the single-wave path instead.
constexpr long long SPLITK_WS_ELEMS = 64ll << 20;

// One workspace per device, allocated at the first small-M product outside a stream capture (an allocation inside a
// capture would invalidate it: a product that arrives first during capture takes the ordinary single-wave path).
// Products of one device are expected to be issued from one stream at a time, as the inference engine does; two streams
// running small-M products concurrently on the same device would share the buffer.
static float* splitk_workspace(cudaStream_t stream) {
  static float* ws[64] = {};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!ws[dev]) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) {
      (void)cudaGetLastError();
      return nullptr;
    }
    void* q = nullptr;
    if (cudaMalloc(&q, SPLITK_WS_ELEMS * sizeof(float)) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    // The workspace is all zero between products: cleared once here, and the finalize kernel clears what it has read.
    if (cudaMemset(q, 0, SPLITK_WS_ELEMS * sizeof(float)) != cudaSuccess) {
      (void)cudaGetLastError();
      (void)cudaFree(q);
      return nullptr;
    }
    ws[dev] = static_cast<float*>(q);
  }
  return ws[dev];
}

__global__ void __launch_bounds__(256) splitk_finalize_kernel(float* __restrict__ ws, long long ldw, void* __restrict__ C, long long ldc,
                                                              const __nv_bfloat16* __restrict__ bias,
                                                              const __nv_bfloat16* __restrict__ residual, long long ldr, int M, int N,
                                                              int act, int out_fp32) {
  tfb::pdl_sync();
  const long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4;      // 4 consecutive columns
  if (i >= (long long)M * ldw) return;
  const int m = int(i / ldw), n = int(i % ldw);
  if (n >= N) return;
  const float4 a = *reinterpret_cast<const float4*>(ws + i);
  *reinterpret_cast<float4*>(ws + i) = make_float4(0.f, 0.f, 0.f, 0.f);     // leave the workspace clear for the next product
  float v[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (n + j < N) {
      if (bias) v[j] += __bfloat162float(bias[n + j]);
      v[j] = tfb::apply_act(v[j], act);
      if (residual) v[j] += __bfloat162float(residual[(long long)m * ldr + n + j]);
      if (out_fp32) static_cast<float*>(C)[(long long)m * ldc + n + j] = v[j];
      else static_cast<__nv_bfloat16*>(C)[(long long)m * ldc + n + j] = __float2bfloat16(v[j]);
    }
  }
}

static int gemm_impl(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn, void* C,
                     long long ldc, int M, int N, int K, const void* bias, const void* residual, long long ldr,
                     float alpha, int act, int out_mode, int max_ctas, const TfbGemmGroup* grp, int* status,
                     void* stream, const TfbGemmTp* tp = nullptr, int force_splits = 0) {
  using namespace tfb;
  if (M <= 0 || N <= 0 || K <= 0) return TFB_ERR_ARG;
  if (out_mode != 0 && (bias || residual || act)) return TFB_ERR_ARG;
  const int gmode = grp ? grp->mode : 0;
  const int E = (gmode != 0) ? grp->num_experts : 1;
  if (gmode == 2 && out_mode == 0) return TFB_ERR_ARG;
  if (gmode == 0 && !tp && out_mode != 2 && M <= 256 && K >= 16 * BK) {
    // Few rows: the product streams the weights once and is bound by how evenly the work items cover the SMs.  Pick the
    // split count whose item count (tiles x splits) fills whole waves best, keeping at least 8 k-blocks per split;
    // accumulate the partials in fp32 and finish in a second kernel.
    const long long tiles_w = (long long)((M + BM - 1) / BM) * ((N + (N > 128 ? 255 : 127)) / (N > 128 ? 256 : 128));
    const long long ldw = (N + 3) / 4 * 4;
    const int all_sms = (max_ctas > 0 && max_ctas < sm_count()) ? max_ctas : sm_count();
    const int total_kb0 = (K + BK - 1) / BK;
    int best_s = 1;
    double best_eff = 0.0, eff1 = 0.0;
    for (int sp = 1; sp <= 16 && sp * 8 <= total_kb0; ++sp) {
      const long long items = tiles_w * sp;
      const double eff = double(items) / double((items + all_sms - 1) / all_sms * all_sms);
      if (sp == 1) eff1 = eff;
      if (eff > best_eff + 0.02) { best_eff = eff; best_s = sp; }
    }
    if (best_eff < eff1 + 0.1) best_s = 1;             // the workspace pass costs about a tenth of a weight-streaming product
    if (best_s > 1 && (long long)M * ldw <= SPLITK_WS_ELEMS) {
      cudaStream_t st0 = static_cast<cudaStream_t>(stream);
      if (float* ws = splitk_workspace(st0)) {
        if (int rc0 = gemm_impl(A, lda, a_mn, B, ldb, b_mn, ws, ldw, M, N, K, nullptr, nullptr, 0, alpha, 0, 2, max_ctas, nullptr, status,
                                stream, nullptr, best_s))
          return rc0;
        const long long quads = (long long)M * ldw / 4;
        tfb::launch_k(splitk_finalize_kernel, int((quads + 255) / 256), 256, 0, st0, ws, ldw, C, ldc, static_cast<const __nv_bfloat16*>(bias),
                                                                          static_cast<const __nv_bfloat16*>(residual), ldr, M, N, act,
                                                                          out_mode == 1);
        return int(cudaGetLastError());
      }
    }
  }
  int BN = (N > 128) ? 256 : 128;
  int sms = sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  {
    // prefer the narrower tile when it puts more SMs to work and still fits into one wave; when the narrow tiling would
    // need a second wave (8192 x 512: 256 tiles of 128 columns) the wide one finishes in a single wave and wins by
    // 12 - 27 % (measured: 13.3 against 15.2 us at K = 512, 28.8 against 39.7 us at K = 2816)
    const long long tm = (M + BM - 1) / BM;
    const long long t256 = tm * ((N + 255) / 256), t128 = tm * ((N + 127) / 128);
    static const int narrow_env = [] { const char* e = getenv("TFB_GEMM_NARROW"); return e ? atoi(e) : 1; }();
    if (narrow_env && BN == 256 && gmode != 2 && out_mode != 2 && t256 < sms && t128 > t256 && t128 <= sms) BN = 128;
  }
  CUtensorMap ta, tb;
  int rc;
  if (!a_mn) rc = make_tmap_2d(&ta, A, 2, K, M, lda * 2, BK, BM);
  else rc = make_tmap_2d(&ta, A, 2, M, K, lda * 2, 64, BK);
  if (rc) return rc;
  const int EB = gmode == 1 ? E : 1;
  const unsigned long long bes = gmode == 1 ? (unsigned long long)grp->b_expert_stride * 2 : (unsigned long long)ldb * 2 * (b_mn ? K : N);
  if (!b_mn) rc = make_tmap_3d(&tb, B, 2, K, N, EB, ldb * 2, bes, BK, BN, 1);
  else rc = make_tmap_3d(&tb, B, 2, N, K, EB, ldb * 2, bes, 64, BK, 1);
  if (rc) return rc;

  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  // C tensor map for the staged epilogue: 32-row x 128-byte boxes.  Needs a 16-byte aligned base and row pitch.
  CUtensorMap tc;
  memset(&tc, 0, sizeof(tc));
  PeerMaps tpeers;
  memset(&tpeers, 0, sizeof(tpeers));
  p.c_tma = 0;
  {
    const int esz = out_mode == 0 ? 2 : 4;
    const bool aligned = (reinterpret_cast<uintptr_t>(C) & 15) == 0 && (ldc * esz) % 16 == 0 &&
                         (gmode != 2 || (grp->c_expert_stride * esz) % 16 == 0);
    const bool rs = tp && (tp->mode & TP_RS);
    if (aligned && rs && tp->peer_c_host && tp->world <= RS_TMA_MAX_WORLD && out_mode == 0 && (ldc * 2) % 16 == 0) {
      const int rps = M / tp->world;
      bool ok = true;
      for (int d = 0; d < tp->world && ok; ++d)
        ok = (reinterpret_cast<uintptr_t>(tp->peer_c_host[d]) & 15) == 0 &&
             make_tmap_3d(&tpeers.m[d], tp->peer_c_host[d], 2, N, (unsigned long long)tp->world * rps, 1, ldc * 2,
                          (unsigned long long)ldc * 2 * tp->world * rps, 64, 32, 1) == 0;
      if (ok) p.c_tma = 1;
    }
    if (aligned && !rs) {
      const unsigned long long zs = gmode == 2 ? (unsigned long long)grp->c_expert_stride * esz : (unsigned long long)ldc * esz * M;
      if (make_tmap_3d(&tc, C, esz, N, M, gmode == 2 ? E : 1, ldc * esz, zs, 128 / esz, 32, 1) == 0) p.c_tma = 1;
    }
  }
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.alpha = alpha; p.act = act; p.out_mode = out_mode;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.status = status;
  p.group_mode = gmode; p.num_experts = E;
  p.expert_of_mtile = grp ? grp->expert_of_mtile : nullptr;
  p.seg_start = grp ? grp->seg_start : nullptr;
  p.c_expert_stride = grp ? grp->c_expert_stride : 0;
  p.tp_mode = 0; p.tp_copy_ctas = 0;
  memset(&p.ag, 0, sizeof(p.ag));
  memset(&p.wg, 0, sizeof(p.wg));
  p.wg_n_shift = -1; p.wg_k_shift = 0;
  p.rs_rank = 0; p.rs_world = 1; p.rs_rows_per_shard = M; p.rs_peer_c = nullptr;
  if (tp) {
    if (gmode != 0 || tp->mode < 1 || tp->mode > 7 || (tp->mode & (TP_AG | TP_RS)) == (TP_AG | TP_RS)) return TFB_ERR_ARG;
    if (tp->mode & (TP_AG | TP_WG)) {
      if (tp->copy_ctas < 1 || tp->copy_ctas >= sms) return TFB_ERR_ARG;
      p.tp_copy_ctas = tp->copy_ctas;
      sms -= tp->copy_ctas;
    }
    if (tp->mode & (TP_AG | TP_RS)) {
      if (tp->world < 1 || M % (tp->world * BM) || a_mn || out_mode != 0) return TFB_ERR_ARG;
    }
    if (tp->mode & TP_AG) {
      if (K % 8 || !tp->ready || !tp->peer_a) return TFB_ERR_ARG;
      p.ag.rank = tp->rank; p.ag.world = tp->world; p.ag.rows_per_shard = M / tp->world; p.ag.row_len = K;
      p.ag.epoch = tp->epoch; p.ag.rows = M; p.ag.src_is_full = 1; p.ag.skip_local = 1; p.ag.ready = tp->ready;
      p.ag.src = static_cast<const __nv_bfloat16* const*>(tp->peer_a);
      p.ag.dst = const_cast<__nv_bfloat16*>(static_cast<const __nv_bfloat16*>(A));
      p.ag.ld = lda;
    }
    if (tp->mode & TP_RS) {
      if (!tp->peer_c) return TFB_ERR_ARG;
      p.rs_rank = tp->rank; p.rs_world = tp->world; p.rs_rows_per_shard = M / tp->world;
      p.rs_peer_c = static_cast<__nv_bfloat16* const*>(tp->peer_c);
    }
    if (tp->mode & TP_WG) {
      // gathered B: rows = N (K-major B) or K (MN-major B), sharded in 128-row blocks over the data-parallel group
      const int rows = b_mn ? K : N, row_len = b_mn ? N : K;
      if (tp->wg_world < 1 || tp->wg_rows < rows || tp->wg_rows % (tp->wg_world * BM) || row_len % 8 || out_mode == 2 ||
          !tp->wg_ready || !tp->wg_src)
        return TFB_ERR_ARG;
      p.wg.rank = tp->wg_rank; p.wg.world = tp->wg_world; p.wg.rows_per_shard = tp->wg_rows / tp->wg_world;
      p.wg.row_len = row_len; p.wg.epoch = tp->wg_epoch; p.wg.rows = rows; p.wg.src_is_full = 0; p.wg.skip_local = tp->wg_skip_local ? 1 : 0;
      p.wg.ready = tp->wg_ready;
      p.wg.src = static_cast<const __nv_bfloat16* const*>(tp->wg_src);
      p.wg.dst = const_cast<__nv_bfloat16*>(static_cast<const __nv_bfloat16*>(B));
      p.wg.ld = ldb;
      if (!b_mn) p.wg_n_shift = (tp->wg_rank * (p.wg.rows_per_shard / BN)) % p.tiles_n;
      else p.wg_k_shift = (tp->wg_rank * (p.wg.rows_per_shard / BK)) % ((K + BK - 1) / BK);
    }
    p.tp_mode = tp->mode;
  }
  {
    // tile order (see decode_work): row-major unless B is wide; the activation gather / reduce-scatter orders follow the
    // row blocks and stay row-major; a gathered K-major weight is always walked in column groups
    static const int raster_env = [] { const char* e = getenv("TFB_GEMM_RASTER"); return e ? atoi(e) : -1; }();
    const int wide = (BN == 256) ? 8 : 16;
    p.raster_gn = p.tiles_n;
    if (gmode != 2 && !(p.tp_mode & (TP_AG | TP_RS))) {
      if ((p.tp_mode & TP_WG) && p.wg_n_shift >= 0) p.raster_gn = raster_env == 0 ? 1 : min(wide, p.tiles_n);
      else if (raster_env != 0 && p.tiles_n > wide + wide / 2 && p.tiles_m >= 4) p.raster_gn = raster_env > 0 ? raster_env : wide;
    }
    if (p.raster_gn < 1) p.raster_gn = 1;
  }
  const int total_kb = (K + BK - 1) / BK;
  const int tiles = p.tiles_m * p.tiles_n;
  int splits = 1;
  if (force_splits > 0 && out_mode == 2 && gmode == 0) {
    splits = force_splits;
  } else if (out_mode == 2 && gmode == 0 && tiles < sms) {
    splits = sms / tiles;                       // round down: all work items must fit in one wave
    const int max_splits = (total_kb + 7) / 8;  // keep at least 8 k-blocks (512 of K) per split
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
  }
  p.kb_per_split = (total_kb + splits - 1) / splits;
  p.splits = (total_kb + p.kb_per_split - 1) / p.kb_per_split;
  const long long work = (long long)tiles * (gmode == 2 ? E : p.splits);
  const int grid = int(work < sms ? work : sms) + p.tp_copy_ctas;   // copy CTAs take the lowest block indices
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int key = (a_mn ? 2 : 0) | (b_mn ? 1 : 0);
  if (BN == 256) {
    switch (key) {
      case 0: return launch<false, false, 256>(ta, tb, tc, tpeers, p, grid, st);
      case 1: return launch<false, true, 256>(ta, tb, tc, tpeers, p, grid, st);
      case 2: return launch<true, false, 256>(ta, tb, tc, tpeers, p, grid, st);
      default: return launch<true, true, 256>(ta, tb, tc, tpeers, p, grid, st);
    }
  } else {
    switch (key) {
      case 0: return launch<false, false, 128>(ta, tb, tc, tpeers, p, grid, st);
      case 1: return launch<false, true, 128>(ta, tb, tc, tpeers, p, grid, st);
      case 2: return launch<true, false, 128>(ta, tb, tc, tpeers, p, grid, st);
      default: return launch<true, true, 128>(ta, tb, tc, tpeers, p, grid, st);
    }
  }
}

// C[M,N] (ldc) = act(alpha * A.B + bias) + residual.
//   a_mn = 0: A is [M,K] with K contiguous (row pitch lda elements); a_mn = 1: A is stored [K,M], M contiguous.
//   b_mn = 0: B is [N,K] with K contiguous (weight layout [out,in]);  b_mn = 1: B is stored [K,N], N contiguous.
//   out_mode 0: bf16 store; 1: fp32 store; 2: fp32 atomic accumulate (C += ...), the only mode that allows split-K.
//   max_ctas > 0 limits the persistent grid (leaves SMs free for a concurrent communication kernel).
TFB_API int tfb_gemm_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn, void* C,
                          long long ldc, int M, int N, int K, const void* bias, const void* residual, long long ldr,
                          float alpha, int act, int out_mode, int max_ctas, int* status, void* stream) {
  return gemm_impl(A, lda, a_mn, B, ldb, b_mn, C, ldc, M, N, K, bias, residual, ldr, alpha, act, out_mode, max_ctas,
                   nullptr, status, stream);
}

// Grouped (mixture-of-experts) form; see TfbGemmGroup.  Mode 1: M counts the padded rows of all experts, B is
// [E, N, K] (or [E, K, N] with b_mn).  Mode 2: K counts the padded rows, C is [E, M, N] fp32 (out_mode 1 or 2).
TFB_API int tfb_gemm_bf16_grouped(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn,
                                  void* C, long long ldc, int M, int N, int K, float alpha, int out_mode,
                                  const TfbGemmGroup* grp, int* status, void* stream) {
  if (!grp || grp->mode < 1 || grp->mode > 2 || grp->num_experts < 1) return TFB_ERR_ARG;
  return gemm_impl(A, lda, a_mn, B, ldb, b_mn, C, ldc, M, N, K, nullptr, nullptr, 0, alpha, 0, out_mode, 0, grp,
                   status, stream);
}

// Fused compute + collective forms (see TfbGemmTp and tp_fused.cu).  Bit 1: C[M, N] = gathered A [M, K] . B^T where
// A's row shards live on the W tensor-parallel ranks.  Bit 2: C is ignored; partial products go to the peers' staging
// buffers (row pitch ldc) and are summed by tfb_tp_reduce.  Bit 4: B is the local gather buffer of a weight whose row
// shards live on the data-parallel ranks (tp->wg_src); the shards are pulled while the tiles of the local shard run.
// `residual` ([M, ldr] bf16, added in the epilogue) is allowed when bit 2 is clear.
TFB_API int tfb_gemm_bf16_tp(const void* A, long long lda, const void* B, long long ldb, int b_mn, void* C,
                             long long ldc, int M, int N, int K, const void* residual, long long ldr,
                             const TfbGemmTp* tp, int* status, void* stream) {
  if (!tp || tp->mode < 1 || tp->mode > 7) return TFB_ERR_ARG;
  if (residual && (tp->mode & 2)) return TFB_ERR_ARG;
  return gemm_impl(A, lda, 0, B, ldb, b_mn, C, ldc, M, N, K, nullptr, residual, ldr, 1.0f, 0, 0, 0, nullptr, status,
                   stream, tp);
}
