// Decode projections y = x W^T (+ bias) on the 5th-generation tensor cores:
// tcgen05.mma with double-buffered TMEM accumulators, operands staged by TMA, a
// persistent stream-K schedule that keeps every SM streaming weights.
//
// Replaces Matmul.forward (fastkernels/tasks/baseline/L1/linear.py:13-17) and
// the F.linear calls of the TP linear layers
// (fastkernels/tasks/baseline/L2/parallel_linear.py:78-81,157-160,237-240,
// 327-335).
//
// At decode the token count m is 1..256 while n, k are in the thousands, so the
// kernel is a WEIGHT-STREAMING kernel: its roofline is HBM bandwidth over the
// n*k*2 weight bytes, not the tensor peak.  The mapping is therefore "swap-AB":
//   MMA M (128 TMEM lanes)  <- 128 rows of W   (one n-tile)
//   MMA N (16..256 columns) <- the m tokens, zero-padded to MPAD by TMA
//   MMA K (16 per instr.)   <- 64-element k-blocks = one 128-byte swizzle row
// so every weight byte crosses HBM once and the small activation tile is re-read
// from L2.
//
// Schedule (stream-K): the work is the list of (n-tile, k-block) units in
// row-major order; CTA c of G (one per SM) owns the contiguous unit range
// [c U/G, (c+1) U/G), so all SMs stream the same number of weight bytes whatever
// n/128 is.  A range cuts tiles into segments.  A segment that starts its tile
// (k-block 0) OWNS the tile: it adds the partial sums of the following CTAs and
// writes the bf16 output.  Any other segment is necessarily the FIRST thing its
// CTA does; it parks its fp32 partial tile in the CTA's workspace slot and raises
// the slot's flag.  Owners therefore only ever wait for work that was started at
// kernel launch by a higher-numbered CTA: the waits are short, acyclic and
// bounded.  Flags are reset by the owner, so the workspace stays zeroed.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM
// owner, warps 2..5 = epilogue (TMEM lanes 32*(warp%4)..+31).  Two accumulator
// buffers in TMEM let the epilogue of one segment overlap the MMAs of the next.
#include "fk_gemm_shared.cuh"

#include <mutex>
#include <unordered_map>


namespace fk {

template <int MPAD, bool CLUSTER>
struct GemmCfg {
  // Cluster split-K with at most 64 token rows exchanges the partial tiles by
  // PUSH: every CTA stores each partial row straight into the shared memory of
  // the CTA that owns the row, one cluster barrier, local sums.  Larger batches
  // keep their partial tile at home and the owners pull rows from their peers.
  static constexpr bool kPush = CLUSTER && MPAD <= 64;
  static constexpr int kXBytes = MPAD * GEMM_BK * 2;
  static constexpr int kStageBytes = GEMM_W_BYTES + kXBytes;
  // after the ring: 2 x [16][128] bf16 output staging (stream-K) or the push slab,
  // [splits][rows per CTA][128] fp32 with rows per CTA * splits <= MPAD + 7
  static constexpr int kTailBytes = kPush ? (MPAD + 8) * GEMM_BN * 4 : 2 * 16 * GEMM_BN * 2;
  static constexpr int kStages = (204 * 1024 - kTailBytes) / kStageBytes;
  static constexpr int kOut = kStages * kStageBytes;
  static constexpr int kBars = kOut + kTailBytes;
  static constexpr int kTotal = kBars + (2 * kStages + 4) * 8 + 16;
  static constexpr int kAlloc = kTotal + 1024;
  static constexpr int kAccCols = MPAD < 32 ? 32 : MPAD;  // one accumulator buffer
  static constexpr int kTmemCols = 2 * kAccCols;
  static_assert(kStages >= 3, "pipeline too shallow");
  static_assert(kAlloc <= 232448, "shared memory budget");
  static_assert(kTmemCols <= 512, "TMEM budget");
};

struct GemmParams {
  const uint16_t* bias;  // [n] or null
  uint16_t* y; int64_t y_stride;
  int m, n, k;
  int n_tiles, kb_total;   // units = n_tiles * kb_total
  int num_ctas;
  int splits, kb_per_split;  // cluster mode: k-blocks per CTA of a cluster
  int half_n;              // SILU: rows of the gate block (= rows of the up block)
  float* part;             // [GEMM_MAX_CTAS][MPAD][128] fp32 partial tiles
  int* flags;              // [GEMM_MAX_CTAS], zero when idle
  int32_t* status;
  int trace_launch;        // diagnostic build: running number of the launch
  // fk_gemm_bf16_push (nranks > 0): instead of y, every output pair goes as an
  // 8-byte {two bf16, call number} word into the receive area of ALL tensor-parallel
  // ranks (dst[r] = this sender's area in rank r's buffer, [row][n / 2] words); the
  // call number of a row is the row's counter in this rank's header plus one.
  struct Push {
    uint8_t* dst[8];
    int nranks;
    const uint32_t* epoch;
  } push;
};

// Four consecutive outputs of one row (two packed bf16 pairs) to every rank.
__device__ __forceinline__ void push_out4(const GemmParams& p, int row, int n, uint32_t w0,
                                          uint32_t w1, uint32_t call) {
  const size_t off = ((size_t)row * (size_t)p.n + (size_t)n) * 4u;
  const uint64_t a = ((uint64_t)call << 32) | w0, b = ((uint64_t)call << 32) | w1;
#pragma unroll
  for (int r = 0; r < 8; ++r)
    if (r < p.push.nranks)
      asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1,%2};" ::"l"(p.push.dst[r] + off),
                   "l"(a), "l"(b)
                   : "memory");
}

// Diagnostic build only (-DFK_GEMM_TRACE): every CTA stamps %globaltimer at the
// points of its timeline into a table the host reads back with
// fk_debug_read_gemm_trace.  Compiled out of the library proper.
#ifdef FK_GEMM_TRACE
// (the last four launches are kept)
__device__ unsigned long long g_gemm_trace[4][GEMM_MAX_CTAS][16];
#define FK_TRACE(slot)                                                     \
  do {                                                                     \
    unsigned long long t__;                                                \
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t__));                 \
    g_gemm_trace[p.trace_launch & 3][blockIdx.x][slot] = t__;              \
  } while (0)
#else
#define FK_TRACE(slot) do {} while (0)
#endif

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_addr, uint32_t rank) {
  uint32_t raddr;
  asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(local_addr), "r"(rank));
  return raddr;
}
// Callers issue all loads of one reduction step before consuming any of them,
// so the (ordered) loads still overlap.
__device__ __forceinline__ void st_dsmem_b32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_dsmem_f32x4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(cluster_addr)
               : "memory");
  return v;
}

// CLUSTER = false: persistent stream-K over all (n-tile, k-block) units.
// CLUSTER = true : n has too few tiles to give every SM one; each tile is handled
//   by a cluster of `splits` CTAs that split its k range and reduce their fp32
//   partial tiles over distributed shared memory (each CTA reduces and writes
//   the token rows m = rank, rank + splits, ...).  No global scratch, no flags.
//   Up to 64 rows the partial rows are PUSHED into the owner's shared memory
//   (one cluster barrier, local sums); above, owners pull them from their peers.
//
// SILU (stream-K only) fuses SiluAndMul into the projection that feeds it: W is
// the merged [gate; up] matrix of 2 * half_n rows and a tile holds 64 gate rows
// (TMEM lanes 0..63) with the 64 up rows of the same output columns (lanes
// 64..127), fetched as two 64-row boxes; the owner's epilogue rounds both to bf16
// -- exactly what the separate projection would have written -- and stores
// silu(gate) * up, [m, half_n], without the [m, 2 half_n] intermediate.
template <int MPAD, bool CLUSTER, bool SILU>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_bf16_kernel(
    const __grid_constant__ CUtensorMap tmap_w,
    const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
  static_assert(!(SILU && CLUSTER), "the fused SiLU epilogue exists for stream-K only");
  using Cfg = GemmCfg<MPAD, CLUSTER>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Cfg::kBars);
  uint64_t* empty = full + Cfg::kStages;
  uint64_t* acc_full = empty + Cfg::kStages;   // [2] MMA -> epilogue
  uint64_t* acc_empty = acc_full + 2;          // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  if (threadIdx.x == 0) FK_TRACE(0);   // entry
  pdl_launch_dependents();
  const long long units = (long long)p.n_tiles * p.kb_total;
  long long u0, u1;
  int crank = 0;
  if (CLUSTER) {
    crank = (int)cluster_rank();
    const int tile = cta / p.splits;
    const int kb0 = crank * p.kb_per_split;
    const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
    u0 = (long long)tile * p.kb_total + kb0;
    u1 = (long long)tile * p.kb_total + kb1;
  } else {
    u0 = unit_begin(cta, units, p.num_ctas);
    u1 = unit_begin(cta + 1, units, p.num_ctas);
  }

  // Push mode writes into peers' shared memory later on; this first barrier phase
  // (waited for just before those writes) certifies that every CTA of the
  // cluster has started.
  if (Cfg::kPush) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  // stages of the first ring-full (requested by thread 0 during set-up)
  const int pre = (int)((u1 - u0) < Cfg::kStages ? (u1 - u0) : Cfg::kStages);
  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    // The weights are never written during a step, so the first ring-full of W
    // tiles is requested right here: before the tensor-memory allocation and the
    // CTA barrier below, and before waiting for the preceding kernels (only the
    // activation tiles, written by the predecessor, wait for those).
    tma_prefetch_desc(&tmap_w);
    int t = (int)(u0 / p.kb_total);
    int k2 = (int)(u0 - (long long)t * p.kb_total);
    for (int i = 0; i < pre; ++i) {
      mbar_arrive_expect_tx(&full[i], (uint32_t)Cfg::kStageBytes);
      load_w_tile<SILU>(smem + i * Cfg::kStageBytes, &tmap_w, &full[i], k2, t, p.half_n);
      if (++k2 == p.kb_total) { k2 = 0; ++t; }
    }
  }
  if (warp == 1) {
    asm volatile(
        "tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
            smem_u32(tmem_slot)),
        "r"((uint32_t)Cfg::kTmemCols)
        : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::
                     : "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) FK_TRACE(1);   // set-up done

  if (warp == 0 && lane == 0) {
    // ----------------------------- TMA producer ----------------------------
    tma_prefetch_desc(&tmap_x);
    int stage = 0;
    uint32_t phase = 0;
    int tile = (int)(u0 / p.kb_total);
    int kb = (int)(u0 - (long long)tile * p.kb_total);
    pdl_wait();
    FK_TRACE(2);                       // predecessors complete
    for (int i = 0; i < pre; ++i) {
      tma_load_2d(smem + i * Cfg::kStageBytes + GEMM_W_BYTES, &tmap_x, &full[i],
                  kb * GEMM_BK, 0);
      if (++kb == p.kb_total) { kb = 0; ++tile; }
    }
    if (pre == Cfg::kStages) { stage = 0; phase = 1; } else { stage = pre; }
    for (long long u = u0 + pre; u < u1; ++u) {
      if (!gemm_wait(&empty[stage], phase ^ 1, abort_flag, p.status)) break;
      uint8_t* wdst = smem + stage * Cfg::kStageBytes;
      mbar_arrive_expect_tx(&full[stage], (uint32_t)Cfg::kStageBytes);
      load_w_tile<SILU>(wdst, &tmap_w, &full[stage], kb, tile, p.half_n);
      tma_load_2d(wdst + GEMM_W_BYTES, &tmap_x, &full[stage], kb * GEMM_BK, 0);
      if (++kb == p.kb_total) { kb = 0; ++tile; }
      if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------ MMA issuer -----------------------------
    // instruction descriptor: D fp32, A/B bf16, both K-major, N = MPAD, M = 128
    constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                               ((uint32_t)(MPAD >> 3) << 17) |
                               ((uint32_t)(GEMM_BN >> 4) << 24);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int seg = 0;
    long long u = u0;
    while (u < u1 && ok) {
      const int tile = (int)(u / p.kb_total);
      const long long tile_end = (long long)(tile + 1) * p.kb_total;
      const long long seg_end = tile_end < u1 ? tile_end : u1;
      const int buf = seg & 1;
      if (!gemm_wait(&acc_empty[buf], ((seg >> 1) & 1) ^ 1, abort_flag, p.status)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + (uint32_t)(buf * Cfg::kAccCols);
      for (long long uu = u; uu < seg_end; ++uu) {
        if (!gemm_wait(&full[stage], phase, abort_flag, p.status)) { ok = false; break; }
        if (uu == u0) FK_TRACE(3);     // first stage landed
        tc_fence_after();
        const uint32_t wa = smem_u32(smem + stage * Cfg::kStageBytes);
        const uint32_t xa = wa + GEMM_W_BYTES;
#pragma unroll
        for (int kk = 0; kk < GEMM_BK / 16; ++kk) {
          tc_mma_bf16(tmem_d, smem_desc_sw128(wa + kk * 32),
                      smem_desc_sw128(xa + kk * 32), idesc,
                      (uu > u || kk > 0) ? 1u : 0u);
        }
        tc_commit(&empty[stage]);  // frees the stage when these MMAs retire
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
      }
      if (!ok) break;
      tc_commit(&acc_full[buf]);   // accumulator of this segment is complete
      FK_TRACE(4);                 // (last write wins: the last segment's MMAs issued)
      u = seg_end;
      ++seg;
    }
  } else if (warp >= 2) {
    // ------------------------------- epilogue ------------------------------
    if (Cfg::kPush) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
    pdl_wait();                    // workspace, bias and y belong to earlier kernels
    const int q = warp & 3;        // TMEM lane quarter this warp may read
    const int e = q * 32 + lane;   // row of the tile = TMEM lane
    int seg = 0, out_it = 0;
    uint16_t* out_stage = reinterpret_cast<uint16_t*>(smem + Cfg::kOut);
    long long u = u0;
    bool ok = true;
    while (u < u1 && ok) {
      const int tile = (int)(u / p.kb_total);
      const long long tile_begin = (long long)tile * p.kb_total;
      const long long tile_end = tile_begin + p.kb_total;
      const long long seg_end = tile_end < u1 ? tile_end : u1;
      const bool owner = (u == tile_begin);
      const int buf = seg & 1;
      // weight row behind TMEM lane e
      const int n = SILU ? (e < 64 ? tile * 64 + e : p.half_n + tile * 64 + (e - 64))
                         : tile * GEMM_BN + e;
      // stream-K owner of a tile that other CTAs finish: those CTAs parked their
      // partial tiles as the first thing they did, so the flags are checked and
      // (up to 64 rows) the first contributor's partial tile is fetched into
      // registers NOW, under this CTA's own k-loop, not after it
      constexpr bool PRE = !CLUSTER && MPAD <= 64;
      float pre[PRE ? MPAD : 1];
      int last = cta;
      if (!CLUSTER && owner && seg_end < tile_end) {
        // contributors: the CTAs after this one whose range starts inside the tile
        while (last + 1 < p.num_ctas &&
               unit_begin(last + 1, units, p.num_ctas) < tile_end)
          ++last;
        // wait for their partial tiles
        if (threadIdx.x == 64) {
          const uint64_t t0 = gemm_ns();
          for (int c2 = cta + 1; c2 <= last; ++c2) {
            while (ld_acquire_gpu(p.flags + c2) == 0) {
              if (gemm_ns() - t0 > 2000000000ull) {
                *abort_flag = 1;
                if (p.status) atomicOr(p.status, FK_DEV_WAIT_TIMEOUT);
                break;
              }
            }
          }
        }
        named_bar_sync(1, 128);
        if (threadIdx.x == 64) FK_TRACE(6);   // contributors' flags seen
        if (PRE) {
          const float* src = p.part + ((size_t)(cta + 1) * MPAD) * GEMM_BN + e;
#pragma unroll
          for (int j = 0; j < (PRE ? MPAD : 1); ++j) pre[j] = __ldcg(src + (size_t)j * GEMM_BN);
        }
      }
      if (!gemm_wait(&acc_full[buf], (seg >> 1) & 1, abort_flag, p.status)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (threadIdx.x == 64) FK_TRACE(5);     // accumulator of the segment complete
      const uint32_t taddr =
          tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * Cfg::kAccCols);
      if (Cfg::kPush) {
        // token row c of the tile belongs to CTA c % splits of the cluster, which
        // keeps one [rows per CTA][128] fp32 slab per sender
        const int rows_per = (p.m + p.splits - 1) / p.splits;
        const uint32_t mine = smem_u32(smem + Cfg::kOut) +
                              (uint32_t)((crank * rows_per) * GEMM_BN + e) * 4u;
        int own = 0, slot = 0;
#pragma unroll 1
        for (int c = 0; c < p.m; c += 32) {  // kAccCols is a multiple of 32
          uint32_t v[32];
          tc_ld32(taddr + (uint32_t)c, v);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (c + j < p.m)
              st_dsmem_b32(dsmem_addr(mine + (uint32_t)(slot * GEMM_BN) * 4u,
                                      (uint32_t)own),
                           v[j]);
            if (++own == p.splits) { own = 0; ++slot; }
          }
        }
      } else if (CLUSTER) {
        // park the fp32 partial tile in this CTA's own shared memory (the ring is
        // idle: every stage was consumed before acc_full fired), [m][128]
        float* dst = reinterpret_cast<float*>(smem) + e;
#pragma unroll 1
        for (int c = 0; c < p.m; c += 32) {  // kAccCols is a multiple of 32
          uint32_t v[32];
          tc_ld32(taddr + (uint32_t)c, v);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) dst[(c + j) * GEMM_BN] = __uint_as_float(v[j]);
        }
      } else if (!owner) {
        // park the fp32 partial tile in this CTA's slot, [MPAD][128]: a warp
        // writes 128 contiguous bytes per token column
        float* dst = p.part + ((size_t)cta * MPAD) * GEMM_BN + e;
#pragma unroll 1
        for (int c = 0; c < p.m; c += 16) {
          uint32_t v[16];
          tc_ld16(taddr + (uint32_t)c, v);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j)
            dst[(size_t)(c + j) * GEMM_BN] = __uint_as_float(v[j]);
        }
        __threadfence();
        named_bar_sync(1, 128);
        if (threadIdx.x == 64) st_release_gpu(p.flags + cta, 1);
      } else {
        const float bias = (p.bias && n < p.n) ? bf16_bits_to_float(p.bias[n]) : 0.f;  // p.n = all W rows
        // first output column of the tile and how many it has
        const int n0 = SILU ? tile * 64 : tile * GEMM_BN;
        const int out_n = SILU ? p.half_n : p.n;
        const int t128 = threadIdx.x - 64;
        const bool vec_store = (p.y_stride % 8 == 0) &&
                               n0 + (SILU ? 64 : GEMM_BN) <= out_n &&
                               ((reinterpret_cast<uintptr_t>(p.y) & 15u) == 0);
        constexpr int kChunkUnroll = PRE ? MPAD / 16 : 1;
#pragma unroll kChunkUnroll
        for (int ci = 0; ci < MPAD / 16; ++ci, ++out_it) {
          const int c = ci * 16;
          if (c >= p.m) break;
          uint32_t v[16];
          tc_ld16(taddr + (uint32_t)c, v);
          tc_wait_ld();
          float a[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) a[j] = __uint_as_float(v[j]);
          if (PRE && last > cta) {
#pragma unroll
            for (int j = 0; j < 16; ++j) a[j] += pre[PRE ? c + j : 0];
          }
          // partial tiles of the (other) contributors: 4 CTAs x 16 coalesced loads
          // in flight at a time, summed in CTA order (deterministic)
          for (int c2 = cta + (PRE ? 2 : 1); c2 <= last; c2 += 4) {
            float t[4][16];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              const int cc = c2 + r <= last ? c2 + r : last;
              const float* src = p.part + ((size_t)cc * MPAD + c) * GEMM_BN + e;
#pragma unroll
              for (int j = 0; j < 16; ++j) t[r][j] = __ldcg(src + (size_t)j * GEMM_BN);
            }
#pragma unroll
            for (int r = 0; r < 4; ++r)
              if (c2 + r <= last) {
#pragma unroll
                for (int j = 0; j < 16; ++j) a[j] += t[r][j];
              }
          }
          // transpose through shared memory so the output leaves in 16-byte,
          // row-contiguous stores: [16 tokens][128 columns] bf16
          uint16_t* st = out_stage + (out_it & 1) * 16 * GEMM_BN;
#pragma unroll
          for (int j = 0; j < 16; ++j)
            st[j * GEMM_BN + e] = __bfloat16_as_ushort(__float2bfloat16_rn(a[j] + bias));
          named_bar_sync(1, 128);
          if (SILU) {
            // [16 tokens][64 gate | 64 up] bf16 -> 16 x 64 outputs, 8 per thread
            const int r = t128 >> 3, ch = t128 & 7;
            if (c + r < p.m) {
              const uint4 g = *reinterpret_cast<const uint4*>(st + r * GEMM_BN + ch * 8);
              const uint4 u = *reinterpret_cast<const uint4*>(st + r * GEMM_BN + 64 + ch * 8);
              uint4 o;
              o.x = silu_mul2(g.x, u.x); o.y = silu_mul2(g.y, u.y);
              o.z = silu_mul2(g.z, u.z); o.w = silu_mul2(g.w, u.w);
              uint16_t* yrow = p.y + (int64_t)(c + r) * p.y_stride + n0 + ch * 8;
              if (vec_store) {
                *reinterpret_cast<uint4*>(yrow) = o;
              } else {
                const uint16_t* o16 = reinterpret_cast<const uint16_t*>(&o);
#pragma unroll
                for (int x = 0; x < 8; ++x)
                  if (n0 + ch * 8 + x < out_n) yrow[x] = o16[x];
              }
            }
          } else {
#pragma unroll
            for (int idx = t128; idx < 16 * 16; idx += 128) {
              const int r = idx >> 4, ch = idx & 15;
              if (c + r < p.m) {
                uint16_t* yrow = p.y + (int64_t)(c + r) * p.y_stride + n0 + ch * 8;
                const uint16_t* srow = st + r * GEMM_BN + ch * 8;
                if (p.push.nranks > 0) {
                  if (n0 + ch * 8 < p.n) {       // n % 8 == 0: the eight columns exist
                    const uint4 o = *reinterpret_cast<const uint4*>(srow);
                    const uint32_t call = p.push.epoch[c + r] + 1;
                    push_out4(p, c + r, n0 + ch * 8, o.x, o.y, call);
                    push_out4(p, c + r, n0 + ch * 8 + 4, o.z, o.w, call);
                  }
                } else if (vec_store) {
                  *reinterpret_cast<uint4*>(yrow) = *reinterpret_cast<const uint4*>(srow);
                } else {
#pragma unroll
                  for (int x = 0; x < 8; ++x)
                    if (n0 + ch * 8 + x < p.n) yrow[x] = srow[x];
                }
              }
            }
          }
        }
        if (last > cta) {
          named_bar_sync(1, 128);   // every thread has read the partials
          if (threadIdx.x == 64)
            for (int c2 = cta + 1; c2 <= last; ++c2) p.flags[c2] = 0;
        }
      }
      // this accumulator buffer may be overwritten by the next-but-one segment
      tc_fence_before();
      __syncwarp();
      if (threadIdx.x == 64) FK_TRACE(7);     // segment's epilogue done
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
      u = seg_end;
      ++seg;
    }
  }
  __syncwarp();
  if (Cfg::kPush) {
    if (warp < 2) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
    cluster_sync_all();  // every sender's rows have landed in this CTA's slabs
    if (warp >= 2) {
      const int t = threadIdx.x - 64;
      const int c4 = t & 31, rsub = t >> 5;   // 32 threads x float4 = one row
      const int tile = cta / p.splits;
      const int n = tile * GEMM_BN + c4 * 4;
      const int rows_per = (p.m + p.splits - 1) / p.splits;
      const float* slab = reinterpret_cast<const float*>(smem + Cfg::kOut) + c4 * 4;
      float b[4] = {0.f, 0.f, 0.f, 0.f};
      if (p.bias) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n + j < p.n) b[j] = bf16_bits_to_float(p.bias[n + j]);
      }
      const bool vec_ok = (n + 3 < p.n) && (p.y_stride % 4 == 0) &&
                          ((reinterpret_cast<uintptr_t>(p.y) & 7u) == 0);
      if (n < p.n) {
        for (int slot = rsub; slot * p.splits + crank < p.m; slot += 4) {
          const int row = slot * p.splits + crank;
          float4 acc = make_float4(b[0], b[1], b[2], b[3]);
#pragma unroll
          for (int r = 0; r < 8; ++r)
            if (r < p.splits) {
              const float4 v = *reinterpret_cast<const float4*>(
                  slab + (size_t)(r * rows_per + slot) * GEMM_BN);
              acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
          uint16_t* dst = p.y + (int64_t)row * p.y_stride + n;
          if (p.push.nranks > 0) {
            push_out4(p, row, n, pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w),
                      p.push.epoch[row] + 1);
          } else if (vec_ok) {
            *reinterpret_cast<uint2*>(dst) =
                make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
          } else {
            const float a[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (n + j < p.n)
                reinterpret_cast<__nv_bfloat16*>(dst)[j] = __float2bfloat16_rn(a[j]);
          }
        }
      }
    }
    // nobody reads or writes a peer's shared memory after the barrier above, so
    // the CTAs of a cluster may leave independently
  } else if (CLUSTER) {
    cluster_sync_all();  // every CTA's partial tile is visible cluster-wide
    if (warp >= 2) {
      const int t = threadIdx.x - 64;
      const int c4 = t & 31, rsub = t >> 5;   // 32 threads x float4 = one row
      const int tile = cta / p.splits;
      const int n = tile * GEMM_BN + c4 * 4;
      const uint32_t part_addr = smem_u32(smem);
      uint32_t peer[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        peer[r] = dsmem_addr(part_addr, (uint32_t)(r < p.splits ? r : 0));
      float b[4] = {0.f, 0.f, 0.f, 0.f};
      if (p.bias) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n + j < p.n) b[j] = bf16_bits_to_float(p.bias[n + j]);
      }
      const bool vec_ok = (n + 3 < p.n) && (p.y_stride % 4 == 0) &&
                          ((reinterpret_cast<uintptr_t>(p.y) & 7u) == 0);
      if (n < p.n) {
        // four token rows per pass: all their partials are requested from the
        // peers' shared memory before the first sum needs one
        constexpr int R = 4;
        const int step = p.splits * 4;
        for (int mm = crank + p.splits * rsub; mm < p.m; mm += R * step) {
          float4 v[R][8];
#pragma unroll
          for (int h = 0; h < R; ++h) {
            const int row = mm + h * step;
            const uint32_t off = (uint32_t)(row * GEMM_BN + c4 * 4) * 4u;
#pragma unroll
            for (int r = 0; r < 8; ++r)
              if (r < p.splits && row < p.m) v[h][r] = ld_dsmem_f32x4(peer[r] + off);
          }
#pragma unroll
          for (int h = 0; h < R; ++h) {
            const int row = mm + h * step;
            if (row >= p.m) break;
            float4 acc = make_float4(b[0], b[1], b[2], b[3]);
#pragma unroll
            for (int r = 0; r < 8; ++r)
              if (r < p.splits) {
                acc.x += v[h][r].x; acc.y += v[h][r].y;
                acc.z += v[h][r].z; acc.w += v[h][r].w;
              }
            uint16_t* dst = p.y + (int64_t)row * p.y_stride + n;
            if (p.push.nranks > 0) {
              push_out4(p, row, n, pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w),
                        p.push.epoch[row] + 1);
            } else if (vec_ok) {
              *reinterpret_cast<uint2*>(dst) =
                  make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
            } else {
              const float a[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (n + j < p.n)
                  reinterpret_cast<__nv_bfloat16*>(dst)[j] = __float2bfloat16_rn(a[j]);
            }
          }
        }
      }
    }
    cluster_sync_all();  // peers are done reading this CTA's shared memory
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) FK_TRACE(8);   // all roles done (incl. the cluster exchange)
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(
                     tmem_base),
                 "r"((uint32_t)Cfg::kTmemCols)
                 : "memory");
    if (lane == 0) FK_TRACE(9);        // tensor memory released
  }
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
struct G2Key {
  const void* ptr; int64_t rows, cols, stride; int box_rows;
  bool operator==(const G2Key& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols &&
           stride == o.stride && box_rows == o.box_rows;
  }
};
struct G2Hash {
  size_t operator()(const G2Key& k) const {
    return std::hash<const void*>()(k.ptr) ^
           std::hash<int64_t>()(k.rows * 1000003ll + k.cols * 7919ll + k.stride * 31ll +
                                k.box_rows);
  }
};
#ifdef FK_GEMM_TRACE
static std::atomic<int> g_trace_launches{0};
#endif
static std::mutex g_g2_mu;
static std::unordered_map<G2Key, CUtensorMap, G2Hash> g_g2_maps;

int gemm_get_2d_map(const void* ptr, int64_t rows, int64_t cols, int64_t stride,
                    int box_rows, CUtensorMap* out) {
  G2Key key{ptr, rows, cols, stride, box_rows};
  std::lock_guard<std::mutex> lk(g_g2_mu);
  auto it = g_g2_maps.find(key);
  if (it != g_g2_maps.end()) {
    *out = it->second;
    return FK_OK;
  }
  tensormap_encode_fn enc = get_tensormap_encode();
  FK_REQUIRE(enc != nullptr, FK_ERR_CUDA,
             "cuTensorMapEncodeTiled not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)stride * 2};
  cuuint32_t box[2] = {GEMM_BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                   const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FK_REQUIRE(r == CUDA_SUCCESS, FK_ERR_CUDA,
             "cuTensorMapEncodeTiled failed with code %d", (int)r);
  if (g_g2_maps.size() > 8192) g_g2_maps.clear();
  g_g2_maps.emplace(key, m);
  *out = m;
  return FK_OK;
}

template <int MPAD, bool CLUSTER, bool SILU = false>
static int launch_gemm_mode(const CUtensorMap& mw, const CUtensorMap& mx,
                            const GemmParams& p, cudaStream_t s) {
  using Cfg = GemmCfg<MPAD, CLUSTER>;
  static PerDeviceOnce attr_once;
  FK_CUDA_OK(set_max_dynamic_smem(attr_once, gemm_bf16_kernel<MPAD, CLUSTER, SILU>,
                                  Cfg::kAlloc));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)p.num_ctas, 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kAlloc;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (CLUSTER) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = (unsigned)p.splits;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
#ifdef FK_GEMM_TRACE
  GemmParams pt = p;
  pt.trace_launch = g_trace_launches.fetch_add(1);
  FK_CUDA_OK(cudaLaunchKernelEx(&cfg, gemm_bf16_kernel<MPAD, CLUSTER, SILU>, mw, mx, pt));
#else
  FK_CUDA_OK(cudaLaunchKernelEx(&cfg, gemm_bf16_kernel<MPAD, CLUSTER, SILU>, mw, mx, p));
#endif
  count_launch();
  return FK_OK;
}

// How many clusters of `splits` CTAs of this kernel can be resident at once
// (GPC boundaries make this less than sm_count / splits); cached.
template <int MPAD>
static int max_active_clusters(int splits) {
  using Cfg = GemmCfg<MPAD, true>;
  static std::mutex mu;
  static int cache_dev[64][9] = {{0}};
  static int cache_other[9] = {0};   // device index beyond the table: not cached
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  std::lock_guard<std::mutex> lk(mu);
  int* cache = cache_other;
  if (dev >= 0 && dev < 64) cache = cache_dev[dev];
  else cache[splits] = 0;
  if (cache[splits] == 0) {
    cudaFuncSetAttribute(gemm_bf16_kernel<MPAD, true, false>,
                         cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kAlloc);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(splits * 64), 1, 1);
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kAlloc;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_bf16_kernel<MPAD, true, false>, &cfg) !=
            cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = -1;  // unknown: do not use clusters of this size
    }
    cache[splits] = n;
  }
  return cache[splits];
}
static int max_active_clusters_for(int mpad, int splits) {
  switch (mpad) {
    case 16: return max_active_clusters<16>(splits);
    case 32: return max_active_clusters<32>(splits);
    case 64: return max_active_clusters<64>(splits);
    case 128: return max_active_clusters<128>(splits);
    default: return max_active_clusters<256>(splits);
  }
}

template <int MPAD>
static int launch_gemm(const CUtensorMap& mw, const CUtensorMap& mx,
                       const GemmParams& p, cudaStream_t s) {
  if (p.half_n > 0) return launch_gemm_mode<MPAD, false, true>(mw, mx, p, s);
  return p.splits > 0 ? launch_gemm_mode<MPAD, true>(mw, mx, p, s)
                      : launch_gemm_mode<MPAD, false>(mw, mx, p, s);
}

// The schedule of one call: cluster split-K (splits >= 2, one cluster per tile)
// or persistent stream-K (splits = 0).
struct GemmPlan { int splits, kb_per_split, num_ctas; };
static GemmPlan plan_gemm(int mpad, int n_tiles, int kb_total) {
  GemmPlan g{};
  const long long units = (long long)n_tiles * kb_total;
  const int sms = sm_count();
  // Few n-tiles: one cluster per tile splits k (DSMEM reduction).  A CTA streams
  // at most ~50 GB/s, so ~128 CTAs already saturate HBM; clusters are preferred
  // whenever they put at least 2 CTAs on a tile.
  int splits = sms / n_tiles;
  if (splits > 8) splits = 8;
  while (splits > 1 && (kb_total / splits < 4 ||
                        max_active_clusters_for(mpad, splits) < n_tiles))
    --splits;
  if (splits >= 2) {
    g.splits = splits;
    g.kb_per_split = (kb_total + splits - 1) / splits;
    while (g.splits > 1 && (g.splits - 1) * g.kb_per_split >= kb_total) {
      --g.splits;
      g.kb_per_split = (kb_total + g.splits - 1) / g.splits;
    }
    g.num_ctas = n_tiles * g.splits;
  } else {
    long long ctas = sms;
    if (ctas > GEMM_MAX_CTAS) ctas = GEMM_MAX_CTAS;
    // at least 4 k-blocks per CTA so the fixed cost of a CTA is amortised
    if (ctas > (units + 3) / 4) ctas = (units + 3) / 4;
    if (ctas < 1) ctas = 1;
    g.num_ctas = (int)ctas;
  }
  return g;
}

static int mpad_for(int64_t m) { return gemm_mpad_for(m); }
static size_t flags_bytes() { return GEMM_FLAGS_BYTES; }


// ---------------------------------------------------------------------------
// Scratch for fk_gemm_bf16_static: the stream-K flags followed by the partial
// tiles for m <= FK_GEMM_STATIC_MAX_M.  It lives in the library image, so every
// GPU that loads the library holds these ~5 MiB until the process exits.
// ---------------------------------------------------------------------------
constexpr int GEMM_STATIC_MAX_M = 64;
constexpr size_t GEMM_STATIC_BYTES =
    1024 + (size_t)GEMM_MAX_CTAS * GEMM_STATIC_MAX_M * GEMM_BN * sizeof(float);
static __device__ __align__(256) unsigned char g_gemm_static_scratch[GEMM_STATIC_BYTES];

// Device address of the array, looked up once per device.  In host code the
// array's name is only a handle for the runtime, never a pointer a kernel can
// use, so the address has to come from cudaGetSymbolAddress with the right
// device current.
//
// The flags must start at zero and the kernel leaves them at zero; a __device__
// array is zero when the module is loaded, so the set-up only looks the address
// up.  That look-up may load the module, which is not allowed while a stream is
// being captured: a first call on a device made during capture is refused.
static int static_scratch_for_current_device(void** out, cudaStream_t s) {
  static std::mutex mu;
  static void* ptrs[64] = {nullptr};
  int dev = 0;
  FK_CUDA_OK(cudaGetDevice(&dev));
  FK_REQUIRE(dev >= 0 && dev < 64, FK_ERR_UNSUPPORTED,
             "fk_gemm_bf16_static: device index %d out of range", dev);
  std::lock_guard<std::mutex> lk(mu);
  if (ptrs[dev] == nullptr) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    FK_CUDA_OK(cudaStreamIsCapturing(s, &cap));
    FK_REQUIRE(cap == cudaStreamCaptureStatusNone, FK_ERR_UNSUPPORTED,
               "fk_gemm_bf16_static: the first call on a device sets the scratch up and "
               "must not be made while the stream is being captured");
    void* ptr = nullptr;
    FK_CUDA_OK(cudaGetSymbolAddress(&ptr, g_gemm_static_scratch));
    ptrs[dev] = ptr;
  }
  *out = ptrs[dev];
  return FK_OK;
}

// the many-row kernel
int gemm_large_launch(const void* x, int64_t x_stride, const void* w, const void* bias,
                      void* y, int64_t y_stride, int64_t m, int64_t n, int64_t k,
                      int32_t* status, cudaStream_t stream);

}  // namespace fk

using namespace fk;

extern "C" {

size_t fk_gemm_bf16_workspace_bytes(int64_t m, int64_t n, int64_t k) {
  (void)n; (void)k;
  if (m <= 0 || m > 256) return 0;
  return flags_bytes() + (size_t)GEMM_MAX_CTAS * mpad_for(m) * GEMM_BN * sizeof(float);
}

static int gemm_bf16_impl(const void* x, int64_t x_stride, const void* w,
                          const void* bias, void* y, int64_t y_stride, int64_t m,
                          int64_t n, int64_t k, void* workspace,
                          size_t workspace_bytes, int32_t* status, fk_stream_t stream,
                          const GemmParams::Push* push) {
  FK_REQUIRE(m >= 0 && n >= 0 && k > 0, FK_ERR_INVALID_ARG, "fk_gemm_bf16: bad sizes");
  if (m == 0 || n == 0) return FK_OK;
  FK_REQUIRE(x && w && (y || push), FK_ERR_INVALID_ARG, "fk_gemm_bf16: null pointer");
  FK_REQUIRE(k % GEMM_BK == 0, FK_ERR_UNSUPPORTED,
             "fk_gemm_bf16: k = %lld must be a multiple of 64", (long long)k);
  FK_REQUIRE(n < (1ll << 31) && k < (1ll << 31), FK_ERR_UNSUPPORTED,
             "fk_gemm_bf16: dimension too large");
  FK_REQUIRE(x_stride >= k && y_stride >= n, FK_ERR_INVALID_ARG,
             "fk_gemm_bf16: row stride smaller than the row");
  FK_REQUIRE(aligned16(x) && aligned16(w) && x_stride % 8 == 0, FK_ERR_ALIGNMENT,
             "fk_gemm_bf16: x and w need 16-byte aligned rows");
  // more than 256 rows: the compute-bound tile kernel (no workspace)
  if (m > 256)
    return gemm_large_launch(x, x_stride, w, bias, y, y_stride, m, n, k, status,
                             static_cast<cudaStream_t>(stream));
  const size_t need = fk_gemm_bf16_workspace_bytes(m, n, k);
  FK_REQUIRE(workspace != nullptr && workspace_bytes >= need &&
                 (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0,
             FK_ERR_WORKSPACE,
             "fk_gemm_bf16: workspace needs %zu zero-initialised bytes, 256-byte "
             "aligned (got %zu)",
             need, workspace_bytes);

  const int mpad = mpad_for(m);
  const int n_tiles = (int)((n + GEMM_BN - 1) / GEMM_BN);
  const int kb_total = (int)(k / GEMM_BK);

  CUtensorMap mw, mx;
  int rc = gemm_get_2d_map(w, n, k, k, GEMM_BN, &mw);
  if (rc != FK_OK) return rc;
  rc = gemm_get_2d_map(x, m, k, x_stride, mpad, &mx);
  if (rc != FK_OK) return rc;

  GemmParams p{};
  p.bias = (const uint16_t*)bias;
  p.y = (uint16_t*)y; p.y_stride = y_stride;
  p.m = (int)m; p.n = (int)n; p.k = (int)k;
  p.n_tiles = n_tiles; p.kb_total = kb_total;
  const GemmPlan plan = plan_gemm(mpad, n_tiles, kb_total);
  p.splits = plan.splits; p.kb_per_split = plan.kb_per_split; p.num_ctas = plan.num_ctas;
  p.flags = reinterpret_cast<int*>(workspace);
  p.part = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + flags_bytes());
  p.status = status;
  if (push) p.push = *push;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (mpad) {
    case 16: return launch_gemm<16>(mw, mx, p, s);
    case 32: return launch_gemm<32>(mw, mx, p, s);
    case 64: return launch_gemm<64>(mw, mx, p, s);
    case 128: return launch_gemm<128>(mw, mx, p, s);
    default: return launch_gemm<256>(mw, mx, p, s);
  }
}

int fk_gemm_bf16(const void* x, int64_t x_stride, const void* w,
                 const void* bias, void* y, int64_t y_stride, int64_t m,
                 int64_t n, int64_t k, void* workspace,
                 size_t workspace_bytes, int32_t* status, fk_stream_t stream) {
  return gemm_bf16_impl(x, x_stride, w, bias, y, y_stride, m, n, k, workspace,
                        workspace_bytes, status, stream, nullptr);
}

int fk_gemm_bf16_push(const void* x, int64_t x_stride, const void* w, const void* bias,
                      int64_t m, int64_t n, int64_t k, void* workspace,
                      size_t workspace_bytes, void* const* dst, int nranks,
                      const void* call_counters, int32_t* status, fk_stream_t stream) {
  FK_REQUIRE(m >= 0 && m <= 256, FK_ERR_UNSUPPORTED,
             "fk_gemm_bf16_push: m = %lld is not a decode batch (m <= 256)", (long long)m);
  FK_REQUIRE(n > 0 && n % 8 == 0, FK_ERR_UNSUPPORTED,
             "fk_gemm_bf16_push: n = %lld must be a positive multiple of 8", (long long)n);
  FK_REQUIRE(dst != nullptr && call_counters != nullptr && nranks >= 1 && nranks <= 8,
             FK_ERR_INVALID_ARG, "fk_gemm_bf16_push: bad destination list");
  GemmParams::Push push{};
  for (int r = 0; r < nranks; ++r) {
    FK_REQUIRE(dst[r] != nullptr && aligned16(dst[r]), FK_ERR_ALIGNMENT,
               "fk_gemm_bf16_push: receive area of rank %d null or not 16-byte aligned", r);
    push.dst[r] = static_cast<uint8_t*>(dst[r]);
  }
  push.nranks = nranks;
  push.epoch = static_cast<const uint32_t*>(call_counters);
  return gemm_bf16_impl(x, x_stride, w, bias, nullptr, n, m, n, k, workspace,
                        workspace_bytes, status, stream, &push);
}

int fk_gemm_bf16_static(const void* x, int64_t x_stride, const void* w,
                        const void* bias, void* y, int64_t y_stride, int64_t m,
                        int64_t n, int64_t k, int32_t* status,
                        fk_stream_t stream) {
  FK_REQUIRE(m <= GEMM_STATIC_MAX_M, FK_ERR_UNSUPPORTED,
             "fk_gemm_bf16_static: m = %lld exceeds the built-in scratch (m <= %d); "
             "use fk_gemm_bf16 with a caller-provided workspace",
             (long long)m, GEMM_STATIC_MAX_M);
  if (m <= 0 || n <= 0) return fk_gemm_bf16(x, x_stride, w, bias, y, y_stride, m, n, k,
                                            nullptr, 0, status, stream);
  void* scratch = nullptr;
  const int rc =
      static_scratch_for_current_device(&scratch, static_cast<cudaStream_t>(stream));
  if (rc != FK_OK) return rc;
  return fk_gemm_bf16(x, x_stride, w, bias, y, y_stride, m, n, k, scratch,
                      GEMM_STATIC_BYTES, status, stream);
}

int fk_gemm_bf16_silu_mul_fusable(int64_t m, int64_t n, int64_t k) {
  // one launch when the merged [gate; up] projection takes the stream-K schedule
  // (more 128-row tiles than half the SMs) and both halves split into 64-row boxes
  if (m <= 0 || m > 256 || n <= 0 || k <= 0 || k % GEMM_BK != 0 || n % 128 != 0) return 0;
  const int n_tiles = (int)(n / GEMM_BN);
  return plan_gemm(mpad_for(m), n_tiles, (int)(k / GEMM_BK)).splits == 0 ? 1 : 0;
}

int fk_gemm_bf16_silu_mul(const void* x, int64_t x_stride, const void* w,
                          const void* bias, void* y, int64_t y_stride, int64_t m,
                          int64_t n, int64_t k, void* workspace,
                          size_t workspace_bytes, int32_t* status, fk_stream_t stream) {
  FK_REQUIRE(m >= 0 && n >= 0 && k > 0, FK_ERR_INVALID_ARG, "fk_gemm_bf16_silu_mul: bad sizes");
  if (m == 0 || n == 0) return FK_OK;
  FK_REQUIRE(x && w && y, FK_ERR_INVALID_ARG, "fk_gemm_bf16_silu_mul: null pointer");
  FK_REQUIRE(fk_gemm_bf16_silu_mul_fusable(m, n, k), FK_ERR_UNSUPPORTED,
             "fk_gemm_bf16_silu_mul: this shape (m %lld, n %lld, k %lld) has no single-launch "
             "schedule; run fk_gemm_bf16 followed by fk_silu_and_mul",
             (long long)m, (long long)n, (long long)k);
  const int64_t half = n / 2;
  FK_REQUIRE(n < (1ll << 31) && k < (1ll << 31), FK_ERR_UNSUPPORTED,
             "fk_gemm_bf16_silu_mul: dimension too large");
  FK_REQUIRE(x_stride >= k && y_stride >= half, FK_ERR_INVALID_ARG,
             "fk_gemm_bf16_silu_mul: row stride smaller than the row");
  FK_REQUIRE(aligned16(x) && aligned16(w) && x_stride % 8 == 0, FK_ERR_ALIGNMENT,
             "fk_gemm_bf16_silu_mul: x and w need 16-byte aligned rows");
  const size_t need = fk_gemm_bf16_workspace_bytes(m, n, k);
  FK_REQUIRE(workspace != nullptr && workspace_bytes >= need &&
                 (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0,
             FK_ERR_WORKSPACE,
             "fk_gemm_bf16_silu_mul: workspace needs %zu zero-initialised bytes, 256-byte "
             "aligned (got %zu)", need, workspace_bytes);
  const int mpad = mpad_for(m);
  CUtensorMap mw, mx;
  int rc = gemm_get_2d_map(w, n, k, k, GEMM_BN / 2, &mw);   // 64-row boxes
  if (rc != FK_OK) return rc;
  rc = gemm_get_2d_map(x, m, k, x_stride, mpad, &mx);
  if (rc != FK_OK) return rc;
  GemmParams p{};
  p.bias = (const uint16_t*)bias;
  p.y = (uint16_t*)y; p.y_stride = y_stride;
  p.m = (int)m; p.n = (int)n; p.k = (int)k;
  p.half_n = (int)half;
  p.n_tiles = (int)(half / 64); p.kb_total = (int)(k / GEMM_BK);
  const GemmPlan plan = plan_gemm(mpad, p.n_tiles, p.kb_total);   // stream-K (checked above)
  p.splits = 0; p.kb_per_split = 0; p.num_ctas = plan.num_ctas;
  p.flags = reinterpret_cast<int*>(workspace);
  p.part = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + flags_bytes());
  p.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (mpad) {
    case 16: return launch_gemm<16>(mw, mx, p, s);
    case 32: return launch_gemm<32>(mw, mx, p, s);
    case 64: return launch_gemm<64>(mw, mx, p, s);
    case 128: return launch_gemm<128>(mw, mx, p, s);
    default: return launch_gemm<256>(mw, mx, p, s);
  }
}

#ifdef FK_GEMM_TRACE
// diagnostic build: copy the per-CTA time stamps of the last launch to the host
int fk_debug_read_gemm_trace(void* host_buf) {
  FK_CUDA_OK(cudaDeviceSynchronize());
  FK_CUDA_OK(cudaMemcpyFromSymbol(host_buf, g_gemm_trace, sizeof(g_gemm_trace)));
  return FK_OK;
}
#endif

}  // extern "C"
