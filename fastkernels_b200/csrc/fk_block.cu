// Persistent decode-block kernel: everything a decoder layer does BETWEEN two
// attention calls, as ONE launch whose weight stream never stops.
//
// The reference runs that stretch as a chain of separate kernels
//   o_proj (RowParallelLinear.forward,  fastkernels/tasks/baseline/L2/parallel_linear.py:327-335)
//   post_attention_layernorm            (L3/llama_decoder.py:40, L1/rms_norm.py:153-164)
//   gate_up_proj + SiluAndMul + down_proj  (LlamaMLP.forward, L2/llama_mlp.py:35-38)
//   next layer: input_layernorm         (L3/llama_decoder.py:35-38)
//   qkv_proj, q/k norm, RoPE, KV store  (LlamaAttention.forward, L2/attention.py:113-150;
//                                        Attention.forward_impl, L2/attention_impl.py:313-325)
// and so did this build.  A decode GEMM is a weight-streaming kernel: measured on
// B200 its k-loop runs at the HBM peak, but every launch pays ~3 us until its
// first weight tile lands and ~2.5 us from its last MMA to the next kernel's
// first instruction, during which HBM idles; four projections per layer lose
// ~22 us of a ~95 us stretch that way.
//
// Here the stretch is a PROGRAM of phases executed by one grid of persistent CTAs
// (one per SM):
//   GEMM / GEMM+SiLU   stream-K over all CTAs, exactly the decode GEMM's tile
//                      code (tcgen05.mma, TMEM accumulators, TMA ring)
//   ADD_RMSNORM        rows dealt round-robin to the CTAs' epilogue warps
//   ROPE_STORE         (token, head) pairs dealt round-robin likewise
// A phase that consumes what the previous one produced waits at a grid-wide
// barrier (one counter in global memory; waits bounded).  Only the ACTIVATION
// side waits: the weight producer runs ahead through the whole program as ring
// slots free up, so while a barrier settles and a norm runs, the next
// projection's weights are already landing in shared memory.
//
// Roles (224 threads): warp 0 weight-tile producer, warp 1 MMA issuer + TMEM
// owner, warps 2..5 epilogue / row phases, warp 6 activation-tile producer.
#include "fk_gemm_shared.cuh"
#include "fk_rowops.cuh"

namespace fk {

constexpr int BLK_THREADS = 224;
constexpr int BLK_MAX_PHASES = 8;
constexpr int BLK_MAX_GEMMS = 4;
constexpr int BLK_BARRIER_WORD = 200;   // first of BLK_MAX_PHASES counters among the flag ints

enum : int { PH_GEMM = 1, PH_GEMM_SILU = 2, PH_ADD_RMSNORM = 3, PH_ROPE_STORE = 4 };

struct BlkPhase {
  int kind;
  int gemm;                  // GEMM phases: index of the (W, x) tensor-map pair
  // GEMM
  const uint16_t* bias; uint16_t* y; int64_t y_stride;
  int n, n_tiles, kb_total, half_n;
  int ctas;                  // CTAs the units are dealt to: every one gets >= 4 k-blocks
  // ADD_RMSNORM: residual = bf16(x + residual) (x null: none added);
  //              out = bf16(residual * rsqrt(mean(residual^2) + eps) * weight)
  const uint16_t* nx; int64_t nx_stride;
  uint16_t* residual; int64_t residual_stride;
  const uint4* norm_w; uint16_t* nout; int64_t nout_stride;
  int cols_vec; float eps;
};

struct BlkParams {
  BlkPhase ph[BLK_MAX_PHASES];
  int num_phases;
  int m;
  int num_ctas;
  float* part;               // [num_ctas][MPAD][128] fp32 partial tiles
  int* flags;                // stream-K flags + the barrier word, zero when idle
  int32_t* status;
  RopeArgs rope;
};

struct BlkMaps {
  CUtensorMap w[BLK_MAX_GEMMS];
  CUtensorMap x[BLK_MAX_GEMMS];
};

template <int MPAD>
struct BlkCfg {
  static constexpr int kXBytes = MPAD * GEMM_BK * 2;
  static constexpr int kStageBytes = GEMM_W_BYTES + kXBytes;
  static constexpr int kTailBytes = 2 * 16 * GEMM_BN * 2;       // output staging
  static constexpr int kStages = (204 * 1024 - kTailBytes) / kStageBytes;
  static constexpr int kOut = kStages * kStageBytes;
  static constexpr int kBars = kOut + kTailBytes;
  static constexpr int kRed = kBars + (2 * kStages + 4) * 8 + 16;  // norm scratch
  static constexpr int kTotal = kRed + 64;
  static constexpr int kAlloc = kTotal + 1024;
  static constexpr int kAccCols = MPAD < 32 ? 32 : MPAD;
  static constexpr int kTmemCols = 2 * kAccCols;
  static_assert(kStages >= 3, "pipeline too shallow");
  static_assert(kAlloc <= 232448, "shared memory budget");
};

// Diagnostic build only (-DFK_BLOCK_TRACE): per CTA and phase, %globaltimer when the
// activation producer got past the barrier (0), the first stage of the phase
// landed (1), its last MMA was issued (2), the epilogue warps started on it (3)
// and arrived at its barrier (4); slot 5 of phase 0 holds the kernel entry.
#ifdef FK_BLOCK_TRACE
__device__ unsigned long long g_blk_trace[GEMM_MAX_CTAS][BLK_MAX_PHASES][8];
#define BLK_TRACE(pi, slot)                                                \
  do {                                                                     \
    unsigned long long t__;                                                \
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t__));                 \
    g_blk_trace[blockIdx.x][pi][slot] = t__;                               \
  } while (0)
#else
#define BLK_TRACE(pi, slot) do {} while (0)
#endif

// Grid barrier: every CTA adds one to a phase's own counter when its share of the
// phase is written; the phase is complete (and, CTAs walking the program in order,
// so is every earlier one) when that counter has reached num_ctas.  One counter per
// phase, because a CTA without work in two successive phases arrives for both at
// once.  The waits are bounded like every other wait of the library.
__device__ __forceinline__ bool blk_wait_phases(const int* counter, int target,
                                                volatile int* abort_flag, int32_t* status) {
  if (ld_acquire_gpu(counter) >= target) return true;
  const uint64_t t0 = gemm_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (ld_acquire_gpu(counter) >= target) return true;
    if (*abort_flag) return false;
    if (gemm_ns() - t0 > 2000000000ull) {
      *abort_flag = 1;
      if (status) atomicOr(status, FK_DEV_WAIT_TIMEOUT);
      return false;
    }
  }
}

// residual-add + RMSNorm of one row by the 128 epilogue threads of a CTA
// (rounding as rmsnorm_row_kernel: fastkernels/tasks/baseline/L1/rms_norm.cu:1342-1410).
// x was written by other SMs during this launch: loads bypass L1.
template <int VPT>
__device__ __forceinline__ void blk_norm_row(const BlkPhase& ph, int row, int t128,
                                             float* red) {
  uint4 v[VPT];
  float ss = 0.f;
  uint16_t* rr = ph.residual + (int64_t)row * ph.residual_stride;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = t128 + i * 128;
    if (c < ph.cols_vec) {
      uint4 r = __ldcg(reinterpret_cast<const uint4*>(rr) + c);
      if (ph.nx != nullptr) {
        uint4 xv = __ldcg(reinterpret_cast<const uint4*>(ph.nx + (int64_t)row * ph.nx_stride) + c);
        __nv_bfloat162* a = reinterpret_cast<__nv_bfloat162*>(&xv);
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) a[j] = __hadd2(a[j], b[j]);
        r = xv;
        reinterpret_cast<uint4*>(rr)[c] = r;
      }
      v[i] = r;
      ss += sumsq8(r);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const int lane = t128 & 31, w = t128 >> 5;
  named_bar_sync(1, 128);            // previous row's readers of red[] are done
  if (lane == 0) red[w] = ss;
  named_bar_sync(1, 128);
  const float tot = red[0] + red[1] + red[2] + red[3];
  const float rs = rsqrtf(tot * (1.0f / (float)(ph.cols_vec * 8)) + ph.eps);
  uint16_t* orow = ph.nout + (int64_t)row * ph.nout_stride;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = t128 + i * 128;
    if (c < ph.cols_vec)
      reinterpret_cast<uint4*>(orow)[c] = scale8(v[i], __ldg(ph.norm_w + c), rs);
  }
}

template <int MPAD>
__global__ void __launch_bounds__(BLK_THREADS, 1) decode_block_kernel(
    const __grid_constant__ BlkMaps maps, const __grid_constant__ BlkParams p) {
  using Cfg = BlkCfg<MPAD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Cfg::kBars);
  uint64_t* empty = full + Cfg::kStages;
  uint64_t* acc_full = empty + Cfg::kStages;   // [2] MMA -> epilogue
  uint64_t* acc_empty = acc_full + 2;          // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* red = reinterpret_cast<float*>(smem + Cfg::kRed);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  const int G = p.num_ctas;
  int* counters = p.flags + BLK_BARRIER_WORD;   // [num_phases]
  if (threadIdx.x == 0) BLK_TRACE(0, 5);
  pdl_launch_dependents();

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

  if (warp == 0) {
    // ------------------- weight producer: runs ahead of everything ----------------
    // The weights never change during a step, so their tiles need no barrier: the
    // only pacing is the ring itself.
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int pi = 0; pi < p.num_phases && ok; ++pi) {
        const BlkPhase& ph = p.ph[pi];
        if (ph.kind != PH_GEMM && ph.kind != PH_GEMM_SILU) continue;
        const CUtensorMap* mw = &maps.w[ph.gemm];
        tma_prefetch_desc(mw);
        const long long units = (long long)ph.n_tiles * ph.kb_total;
        const int Gp = ph.ctas;   // CTAs that share this projection
        const long long u0 = cta < Gp ? unit_begin(cta, units, Gp) : 0;
        const long long u1 = cta < Gp ? unit_begin(cta + 1, units, Gp) : 0;
        int tile = (int)(u0 / ph.kb_total);
        int kb = (int)(u0 - (long long)tile * ph.kb_total);
        for (long long u = u0; u < u1; ++u) {
          if (!gemm_wait(&empty[stage], phase ^ 1, abort_flag, p.status)) { ok = false; break; }
          uint8_t* wdst = smem + stage * Cfg::kStageBytes;
          mbar_arrive_expect_tx(&full[stage], (uint32_t)Cfg::kStageBytes);
          if (ph.kind == PH_GEMM_SILU) load_w_tile<true>(wdst, mw, &full[stage], kb, tile, ph.half_n);
          else load_w_tile<false>(wdst, mw, &full[stage], kb, tile, 0);
          if (++kb == ph.kb_total) { kb = 0; ++tile; }
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 6) {
    // ------ activation producer: a phase's x exists once the phases before it are done ----
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      pdl_wait();                      // the first x comes from the preceding kernels
      for (int pi = 0; pi < p.num_phases && ok; ++pi) {
        const BlkPhase& ph = p.ph[pi];
        if (ph.kind != PH_GEMM && ph.kind != PH_GEMM_SILU) continue;
        const CUtensorMap* mx = &maps.x[ph.gemm];
        tma_prefetch_desc(mx);
        const long long units = (long long)ph.n_tiles * ph.kb_total;
        const int Gp = ph.ctas;   // CTAs that share this projection
        const long long u0 = cta < Gp ? unit_begin(cta, units, Gp) : 0;
        const long long u1 = cta < Gp ? unit_begin(cta + 1, units, Gp) : 0;
        if (u0 >= u1) continue;
        if (pi > 0) {
          if (!blk_wait_phases(counters + pi - 1, G, abort_flag, p.status)) break;
          // the rows were written with ordinary stores by other SMs and are read
          // by the TMA unit: order the two proxies
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        BLK_TRACE(pi, 0);
        int kb = (int)(u0 % ph.kb_total);
        for (long long u = u0; u < u1; ++u) {
          if (!gemm_wait(&empty[stage], phase ^ 1, abort_flag, p.status)) { ok = false; break; }
          tma_load_2d(smem + stage * Cfg::kStageBytes + GEMM_W_BYTES, mx, &full[stage],
                      kb * GEMM_BK, 0);
          if (++kb == ph.kb_total) kb = 0;
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer -----------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                 ((uint32_t)(MPAD >> 3) << 17) |
                                 ((uint32_t)(GEMM_BN >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int seg = 0;
      for (int pi = 0; pi < p.num_phases && ok; ++pi) {
        const BlkPhase& ph = p.ph[pi];
        if (ph.kind != PH_GEMM && ph.kind != PH_GEMM_SILU) continue;
        const long long units = (long long)ph.n_tiles * ph.kb_total;
        const int Gp = ph.ctas;   // CTAs that share this projection
        const long long u0 = cta < Gp ? unit_begin(cta, units, Gp) : 0;
        const long long u1 = cta < Gp ? unit_begin(cta + 1, units, Gp) : 0;
        long long u = u0;
        while (u < u1 && ok) {
          const int tile = (int)(u / ph.kb_total);
          const long long tile_end = (long long)(tile + 1) * ph.kb_total;
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
            if (uu == u0) BLK_TRACE(pi, 1);
            tc_fence_after();
            const uint32_t wa = smem_u32(smem + stage * Cfg::kStageBytes);
            const uint32_t xa = wa + GEMM_W_BYTES;
#pragma unroll
            for (int kk = 0; kk < GEMM_BK / 16; ++kk) {
              tc_mma_bf16(tmem_d, smem_desc_sw128(wa + kk * 32), smem_desc_sw128(xa + kk * 32),
                          idesc, (uu > u || kk > 0) ? 1u : 0u);
            }
            tc_commit(&empty[stage]);
            if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          tc_commit(&acc_full[buf]);
          BLK_TRACE(pi, 2);
          u = seg_end;
          ++seg;
        }
      }
    }
  } else {
    // ---------------- epilogue warps: GEMM tiles and the row phases ----------------
    pdl_wait();                    // workspace, outputs and row inputs belong to earlier kernels
    const int q = warp & 3;        // TMEM lane quarter this warp may read
    const int e = q * 32 + lane;   // row of the tile = TMEM lane
    const int t128 = threadIdx.x - 64;
    int seg = 0, out_it = 0;
    uint16_t* out_stage = reinterpret_cast<uint16_t*>(smem + Cfg::kOut);
    bool ok = true;
    for (int pi = 0; pi < p.num_phases && ok; ++pi) {
      const BlkPhase& ph = p.ph[pi];
      if (ph.kind == PH_ADD_RMSNORM || ph.kind == PH_ROPE_STORE) {
        // needs everything the earlier phases of every CTA wrote
        int pass = 1;
        if (pi > 0 && t128 == 0)
          pass = blk_wait_phases(counters + pi - 1, G, abort_flag, p.status) ? 1 : 0;
        named_bar_sync(1, 128);
        if (t128 == 0) BLK_TRACE(pi, 3);
        if (*abort_flag || !pass) { ok = false; break; }
        if (ph.kind == PH_ADD_RMSNORM) {
          for (int row = cta; row < p.m; row += G) {
            if (ph.cols_vec <= 128) blk_norm_row<1>(ph, row, t128, red);
            else if (ph.cols_vec <= 256) blk_norm_row<2>(ph, row, t128, red);
            else if (ph.cols_vec <= 512) blk_norm_row<4>(ph, row, t128, red);
            else blk_norm_row<8>(ph, row, t128, red);
          }
        } else {
          // (head, lane) pairs of a token in blocks of 128 threads; blocks dealt
          // round-robin over the CTAs
          const RopeArgs& a = p.rope;
          const int heads = a.hq + a.hkv + (a.v ? a.hkv : 0);
          const int gx = (heads * 8 + 127) / 128;       // head_dim 128: 8 lanes per head
          const long long blocks = (long long)gx * a.num_tokens;
          for (long long vb = cta; vb < blocks; vb += G) {
            const int bx = (int)(vb % gx);
            const int64_t tok = vb / gx;
            rope_thread<8, true, 1, true>(a, bx * 128 + t128, tok, a.num_tokens);
          }
        }
      } else {
        const bool SILU = ph.kind == PH_GEMM_SILU;
        const long long units = (long long)ph.n_tiles * ph.kb_total;
        const int Gp = ph.ctas;   // CTAs that share this projection
        const long long u0 = cta < Gp ? unit_begin(cta, units, Gp) : 0;
        const long long u1 = cta < Gp ? unit_begin(cta + 1, units, Gp) : 0;
        long long u = u0;
        while (u < u1 && ok) {
          const int tile = (int)(u / ph.kb_total);
          const long long tile_begin = (long long)tile * ph.kb_total;
          const long long tile_end = tile_begin + ph.kb_total;
          const long long seg_end = tile_end < u1 ? tile_end : u1;
          const bool owner = (u == tile_begin);
          const int buf = seg & 1;
          const int n = SILU ? (e < 64 ? tile * 64 + e : ph.half_n + tile * 64 + (e - 64))
                             : tile * GEMM_BN + e;
          constexpr bool PRE = MPAD <= 64;
          float pre[PRE ? MPAD : 1];
          int last = cta;
          if (owner && seg_end < tile_end) {
            // A flag carries the number of the phase it was raised in: the epilogue
            // warps run from one projection straight into the next, so an owner may
            // look at a contributor's flag before the previous projection's owner has
            // taken that contributor's earlier partial tile and cleared the flag.
            while (last + 1 < Gp && unit_begin(last + 1, units, Gp) < tile_end) ++last;
            if (t128 == 0) {
              const uint64_t t0 = gemm_ns();
              for (int c2 = cta + 1; c2 <= last; ++c2) {
                while (ld_acquire_gpu(p.flags + c2) != pi + 1) {
                  if (*abort_flag || gemm_ns() - t0 > 2000000000ull) {
                    *abort_flag = 1;
                    if (p.status) atomicOr(p.status, FK_DEV_WAIT_TIMEOUT);
                    break;
                  }
                }
              }
            }
            named_bar_sync(1, 128);
            if (PRE) {
              const float* src = p.part + ((size_t)(cta + 1) * MPAD) * GEMM_BN + e;
#pragma unroll
              for (int j = 0; j < (PRE ? MPAD : 1); ++j)
                pre[j] = __ldcg(src + (size_t)j * GEMM_BN);
            }
          }
          if (!gemm_wait(&acc_full[buf], (seg >> 1) & 1, abort_flag, p.status)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t taddr =
              tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * Cfg::kAccCols);
          if (!owner) {
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
            if (t128 == 0) st_release_gpu(p.flags + cta, pi + 1);
          } else {
            const float bias = (ph.bias && n < ph.n) ? bf16_bits_to_float(ph.bias[n]) : 0.f;
            const int n0 = SILU ? tile * 64 : tile * GEMM_BN;
            const int out_n = SILU ? ph.half_n : ph.n;
            const bool vec_store = (ph.y_stride % 8 == 0) &&
                                   n0 + (SILU ? 64 : GEMM_BN) <= out_n &&
                                   ((reinterpret_cast<uintptr_t>(ph.y) & 15u) == 0);
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
              uint16_t* st = out_stage + (out_it & 1) * 16 * GEMM_BN;
#pragma unroll
              for (int j = 0; j < 16; ++j)
                st[j * GEMM_BN + e] = __bfloat16_as_ushort(__float2bfloat16_rn(a[j] + bias));
              named_bar_sync(1, 128);
              if (SILU) {
                const int r = t128 >> 3, ch = t128 & 7;
                if (c + r < p.m) {
                  const uint4 g = *reinterpret_cast<const uint4*>(st + r * GEMM_BN + ch * 8);
                  const uint4 uu = *reinterpret_cast<const uint4*>(st + r * GEMM_BN + 64 + ch * 8);
                  uint4 o;
                  o.x = silu_mul2(g.x, uu.x); o.y = silu_mul2(g.y, uu.y);
                  o.z = silu_mul2(g.z, uu.z); o.w = silu_mul2(g.w, uu.w);
                  uint16_t* yrow = ph.y + (int64_t)(c + r) * ph.y_stride + n0 + ch * 8;
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
                    uint16_t* yrow = ph.y + (int64_t)(c + r) * ph.y_stride + n0 + ch * 8;
                    const uint16_t* srow = st + r * GEMM_BN + ch * 8;
                    if (vec_store) {
                      *reinterpret_cast<uint4*>(yrow) = *reinterpret_cast<const uint4*>(srow);
                    } else {
#pragma unroll
                      for (int x = 0; x < 8; ++x)
                        if (n0 + ch * 8 + x < ph.n) yrow[x] = srow[x];
                    }
                  }
                }
              }
            }
            if (last > cta) {
              named_bar_sync(1, 128);   // every thread has read the partials
              if (t128 == 0)
                for (int c2 = cta + 1; c2 <= last; ++c2) p.flags[c2] = 0;
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
          u = seg_end;
          ++seg;
        }
      }
      if (!ok) break;
      // this CTA's share of the phase is written: tell the grid
      named_bar_sync(1, 128);
      if (t128 == 0) {
        BLK_TRACE(pi, 4);
        __threadfence();
        const int old = atomicAdd(counters + pi, 1);
        // the last arrival of the last phase means every CTA is through the whole
        // program: nobody waits any more, the counters go back to zero for the
        // next launch
        if (pi == p.num_phases - 1 && old == G - 1)
          for (int i = 0; i < p.num_phases; ++i) atomicExch(counters + i, 0);
      }
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)Cfg::kTmemCols)
                 : "memory");
  }
}

template <int MPAD>
static int launch_block(const BlkMaps& maps, const BlkParams& p, cudaStream_t s) {
  using Cfg = BlkCfg<MPAD>;
  static PerDeviceOnce attr_once;
  FK_CUDA_OK(set_max_dynamic_smem(attr_once, decode_block_kernel<MPAD>, Cfg::kAlloc));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)p.num_ctas, 1, 1);
  cfg.blockDim = dim3(BLK_THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kAlloc;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  FK_CUDA_OK(cudaLaunchKernelEx(&cfg, decode_block_kernel<MPAD>, maps, p));
  count_launch();
  return FK_OK;
}

}  // namespace fk

using namespace fk;

extern "C" {

size_t fk_decode_block_workspace_bytes(int64_t m) {
  if (m <= 0 || m > 128) return 0;
  return GEMM_FLAGS_BYTES + (size_t)GEMM_MAX_CTAS * gemm_mpad_for(m) * GEMM_BN * sizeof(float);
}

int fk_decode_block(const fk_block_phase* phases, int num_phases, int64_t m,
                    void* workspace, size_t workspace_bytes, int32_t* status,
                    fk_stream_t stream) {
  FK_REQUIRE(phases != nullptr && num_phases >= 1 && num_phases <= BLK_MAX_PHASES,
             FK_ERR_INVALID_ARG, "fk_decode_block: 1..%d phases", BLK_MAX_PHASES);
  FK_REQUIRE(m >= 0, FK_ERR_INVALID_ARG, "fk_decode_block: bad row count");
  if (m == 0) return FK_OK;
  FK_REQUIRE(m <= 128, FK_ERR_UNSUPPORTED,
             "fk_decode_block: m = %lld rows; the persistent block serves decode batches of "
             "at most 128 rows", (long long)m);
  const size_t need = fk_decode_block_workspace_bytes(m);
  FK_REQUIRE(workspace != nullptr && workspace_bytes >= need &&
                 (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0,
             FK_ERR_WORKSPACE,
             "fk_decode_block: workspace needs %zu zero-initialised bytes, 256-byte aligned "
             "(got %zu)", need, workspace_bytes);
  const int mpad = gemm_mpad_for(m);
  int ctas = sm_count();
  if (ctas > GEMM_MAX_CTAS) ctas = GEMM_MAX_CTAS;
  BlkMaps maps;
  BlkParams p{};
  p.num_phases = num_phases;
  p.m = (int)m;
  p.num_ctas = ctas;
  p.flags = reinterpret_cast<int*>(workspace);
  p.part = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + GEMM_FLAGS_BYTES);
  p.status = status;
  int gemms = 0, ropes = 0;
  for (int i = 0; i < num_phases; ++i) {
    const fk_block_phase& f = phases[i];
    BlkPhase& ph = p.ph[i];
    ph.kind = f.kind;
    if (f.kind == FK_PHASE_GEMM || f.kind == FK_PHASE_GEMM_SILU_MUL) {
      const bool silu = f.kind == FK_PHASE_GEMM_SILU_MUL;
      FK_REQUIRE(gemms < BLK_MAX_GEMMS, FK_ERR_UNSUPPORTED,
                 "fk_decode_block: at most %d projections per launch", BLK_MAX_GEMMS);
      FK_REQUIRE(f.x && f.w && f.y && f.n > 0 && f.k > 0, FK_ERR_INVALID_ARG,
                 "fk_decode_block: phase %d: null pointer or empty projection", i);
      FK_REQUIRE(f.k % GEMM_BK == 0 && f.n < (1ll << 31) && f.k < (1ll << 31) &&
                     (!silu || f.n % 128 == 0),
                 FK_ERR_UNSUPPORTED,
                 "fk_decode_block: phase %d: k must be a multiple of 64 (and n of 128 with "
                 "the fused SiLU)", i);
      FK_REQUIRE(f.x_stride >= f.k && f.y_stride >= (silu ? f.n / 2 : f.n), FK_ERR_INVALID_ARG,
                 "fk_decode_block: phase %d: row stride smaller than the row", i);
      FK_REQUIRE(aligned16(f.x) && aligned16(f.w) && f.x_stride % 8 == 0, FK_ERR_ALIGNMENT,
                 "fk_decode_block: phase %d: x and w need 16-byte aligned rows", i);
      int rc = gemm_get_2d_map(f.w, f.n, f.k, f.k, silu ? GEMM_BN / 2 : GEMM_BN, &maps.w[gemms]);
      if (rc != FK_OK) return rc;
      rc = gemm_get_2d_map(f.x, m, f.k, f.x_stride, mpad, &maps.x[gemms]);
      if (rc != FK_OK) return rc;
      ph.gemm = gemms++;
      ph.bias = (const uint16_t*)f.bias;
      ph.y = (uint16_t*)f.y; ph.y_stride = f.y_stride;
      ph.n = (int)f.n;
      ph.half_n = silu ? (int)(f.n / 2) : 0;
      ph.n_tiles = silu ? (int)(f.n / 128) : (int)((f.n + GEMM_BN - 1) / GEMM_BN);
      ph.kb_total = (int)(f.k / GEMM_BK);
      // no CTA without a unit inside a projection (a tile's owner waits for every
      // CTA whose range starts inside the tile), and at least 4 k-blocks each
      long long share = ((long long)ph.n_tiles * ph.kb_total + 3) / 4;
      ph.ctas = (int)(share < ctas ? (share < 1 ? 1 : share) : ctas);
    } else if (f.kind == FK_PHASE_ADD_RMSNORM) {
      FK_REQUIRE(f.residual && f.norm_weight && f.y && f.n > 0, FK_ERR_INVALID_ARG,
                 "fk_decode_block: phase %d: null pointer", i);
      FK_REQUIRE(f.n % 8 == 0 && f.n <= 8192, FK_ERR_UNSUPPORTED,
                 "fk_decode_block: phase %d: rows of %lld elements (multiple of 8, <= 8192)", i,
                 (long long)f.n);
      FK_REQUIRE(aligned16(f.x) && aligned16(f.residual) && aligned16(f.norm_weight) &&
                     aligned16(f.y) && f.x_stride % 8 == 0 && f.residual_stride % 8 == 0 &&
                     f.y_stride % 8 == 0,
                 FK_ERR_ALIGNMENT, "fk_decode_block: phase %d: 16-byte alignment required", i);
      ph.nx = (const uint16_t*)f.x; ph.nx_stride = f.x_stride;
      ph.residual = (uint16_t*)f.residual; ph.residual_stride = f.residual_stride;
      ph.norm_w = (const uint4*)f.norm_weight;
      ph.nout = (uint16_t*)f.y; ph.nout_stride = f.y_stride;
      ph.cols_vec = (int)(f.n / 8);
      ph.eps = f.eps;
    } else if (f.kind == FK_PHASE_QKV_ROPE_STORE) {
      FK_REQUIRE(ropes++ == 0, FK_ERR_UNSUPPORTED,
                 "fk_decode_block: one split + RoPE + store phase per launch");
      FK_REQUIRE(f.head_dim == 128 && f.num_q_heads > 0 && f.num_kv_heads > 0,
                 FK_ERR_UNSUPPORTED, "fk_decode_block: phase %d: head_dim must be 128", i);
      FK_REQUIRE(f.x && f.positions && f.cos_sin_cache && f.cache_is_fp32 == 0,
                 FK_ERR_INVALID_ARG,
                 "fk_decode_block: phase %d: qkv, positions and a bf16 cos/sin cache needed", i);
      FK_REQUIRE((f.k_cache == nullptr) == (f.v_cache == nullptr) &&
                     (f.k_cache == nullptr || f.slot_mapping != nullptr),
                 FK_ERR_INVALID_ARG,
                 "fk_decode_block: phase %d: k_cache, v_cache and slot_mapping go together", i);
      FK_REQUIRE(f.x_stride >= (int64_t)(f.num_q_heads + 2 * f.num_kv_heads) * 128 &&
                     (f.kv_layout == 0 || (f.kv_layout == 1 && f.block_size > 0)),
                 FK_ERR_INVALID_ARG, "fk_decode_block: phase %d: bad qkv stride or layout", i);
      FK_REQUIRE(aligned16(f.x) && aligned16(f.cos_sin_cache) && aligned16(f.k_cache) &&
                     aligned16(f.v_cache) && aligned16(f.q_norm_weight) &&
                     aligned16(f.k_norm_weight) && f.x_stride % 8 == 0,
                 FK_ERR_ALIGNMENT, "fk_decode_block: phase %d: 16-byte alignment required", i);
      RopeArgs& a = p.rope;
      uint16_t* base = (uint16_t*)f.x;
      a.q = base; a.q_stride = f.x_stride; a.hq = f.num_q_heads;
      a.k = base + (int64_t)f.num_q_heads * 128; a.k_stride = f.x_stride;
      a.hkv = f.num_kv_heads;
      a.v = f.k_cache ? base + (int64_t)(f.num_q_heads + f.num_kv_heads) * 128 : nullptr;
      a.v_stride = f.x_stride;
      a.positions = f.positions;
      a.cache = f.cos_sin_cache; a.cache_is_fp32 = 0; a.max_position = f.max_position;
      a.q_norm_w = (const uint4*)f.q_norm_weight;
      a.k_norm_w = (const uint4*)f.k_norm_weight;
      a.eps = f.eps;
      a.k_cache = (uint16_t*)f.k_cache; a.v_cache = (uint16_t*)f.v_cache;
      a.slots = f.slot_mapping; a.num_slots = f.num_slots;
      a.page = f.block_size > 0 ? f.block_size : 1; a.hnd = f.kv_layout;
      a.num_tokens = m; a.status = status;
    } else {
      set_error("fk_decode_block: phase %d: unknown kind %d", i, f.kind);
      return FK_ERR_INVALID_ARG;
    }
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (mpad) {
    case 16: return launch_block<16>(maps, p, s);
    case 32: return launch_block<32>(maps, p, s);
    case 64: return launch_block<64>(maps, p, s);
    default: return launch_block<128>(maps, p, s);
  }
}

#ifdef FK_BLOCK_TRACE
int fk_debug_read_block_trace(void* host_buf) {
  FK_CUDA_OK(cudaDeviceSynchronize());
  FK_CUDA_OK(cudaMemcpyFromSymbol(host_buf, g_blk_trace, sizeof(g_blk_trace)));
  return FK_OK;
}
#endif

}  // extern "C"
