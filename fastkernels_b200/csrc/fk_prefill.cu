// The neighbours of the decode step on the prefill side:
//
//   fk_prefill_attn        variable-length causal attention of a batch of prompt
//                          chunks over dense K/V or over the paged KV pool
//                          (FlashAttnPrefill.forward,
//                          fastkernels/tasks/baseline/L1/flash_attn_prefill.py:28-74;
//                          PyTorch statement Attention._prefill_torch_from_tensors /
//                          _prefill_torch_from_cache,
//                          fastkernels/tasks/baseline/L2/attention_impl.py:624-652)
//   fk_merge_attn_states   log-sum-exp merge of two partial attention results
//                          (merge_attn_states,
//                          fastkernels/tasks/baseline/L1/merge_attn_states.py:32-100,
//                          kernel merge_attn_states.cu:2440-2580)
//
// Prefill attention is the one compute-bound kernel of the engine, so it runs on
// the 5th-generation tensor cores.  A work item is 256 query rows of one head as
// two 128-row tiles that take turns on the tensor pipe; one persistent CTA per SM
// walks a static list of items (heaviest first), so the Q / K fetch of the next
// item and the output write of the previous one overlap the matrix work:
//
//   warp 8        TMA producer: the two Q tiles once, then K_0 V_0 K_1 V_1 ...
//                 through a ring of five 32 KiB slots (128 keys x 128 dims,
//                 128-byte swizzle, [dim half][key][64 dims])
//   warp 9        MMA issuer and TMEM owner.  S_t = Q_t K_j^T (both operands
//                 K-major) into TMEM columns [128 t, 128 t + 128);
//                 O_t += P_t V_j with P_t read from TMEM (it overwrites the
//                 first 64 columns of S_t as bf16 pairs) and V_j read MN-major
//                 straight from the slot, accumulating in TMEM columns
//                 [256 + 128 t, ...).  Issue order
//                 S0 S1 | PV0 S0' PV1 S1' | ... so that one tile's softmax
//                 overlaps the other tile's matrix work.
//   warps 0-3     softmax of tile 0, one thread per query row (TMEM lane):
//   warps 4-7     softmax of tile 1.  Row max / exp2 / row sum in registers,
//                 P written back to TMEM as bf16, O rescaled in TMEM only when a row's running max grew by more than 2^8
//                 (the final division by the row sum makes this exact).
//
// The softmax warpgroups hold a whole score row in registers, so they take 208
// registers per thread (setmaxnreg) and the third warpgroup (TMA, MMA, two idle
// warps) drops to 80.
//
// Every wait is bounded (2 s of %globaltimer): on expiry the kernel records
// FK_DEV_WAIT_TIMEOUT, all roles leave their loops, TMEM is freed and the kernel
// returns.
#include "fk_common.cuh"
#include "fk_tcgen05.cuh"

#include <cmath>
#include <mutex>
#include <unordered_map>

namespace fk {

constexpr int PF_D = 128;
constexpr int PF_BM = 128;            // query rows per tile
constexpr int PF_BN = 128;            // keys per K/V tile
constexpr int PF_QT = 2;              // query tiles per CTA
constexpr int PF_SLOTS = 5;           // K/V ring
constexpr int PF_HALF_BYTES = 128 * 128;       // 128 rows x 64 elements
constexpr int PF_TILE_BYTES = 2 * PF_HALF_BYTES;
constexpr int PF_THREADS = 128 * (PF_QT + 1);   // softmax warpgroups + one for TMA / MMA
constexpr int PF_WARP_TMA = 4 * PF_QT;
constexpr int PF_WARP_MMA = 4 * PF_QT + 1;
// Register re-split between the warpgroups.  The CTA owns (registers per thread
// at launch) x 384 registers; setmaxnreg.inc blocks until the pool has what it
// asks for, so the split must fit that pool: the host refuses to launch otherwise.
constexpr int PF_REGS_SOFTMAX = 208;
constexpr int PF_REGS_OTHER = 80;
constexpr int PF_REGS_NEEDED = PF_QT * 128 * PF_REGS_SOFTMAX + 128 * PF_REGS_OTHER;
static_assert(PF_REGS_NEEDED <= 168 * PF_THREADS, "register split exceeds the CTA's pool");
constexpr int PF_OFF_Q = 0;
constexpr int PF_OFF_KV = PF_OFF_Q + PF_QT * PF_TILE_BYTES;
constexpr int PF_OFF_BAR = PF_OFF_KV + PF_SLOTS * PF_TILE_BYTES;
constexpr int PF_SMEM = PF_OFF_BAR + 256;
constexpr int PF_SMEM_ALLOC = PF_SMEM + 1024;
constexpr int PF_TMEM_COLS = 512;
constexpr float PF_RESCALE_LOG2 = 8.0f;
static_assert(PF_SMEM_ALLOC <= 232448, "shared memory budget");

struct PrefillParams {
  uint16_t* out; int64_t out_stride;
  float* lse; int64_t total_q;      // lse [Hq, total_q] or null
  const int32_t* cu_q; const int32_t* cu_k;
  const int32_t* block_tables; int64_t bt_stride;
  int hq, g;
  int paged, hnd, block_size, bs_shift, sub_tokens, num_blocks;
  float scale_log2;                 // softmax_scale * log2(e)
  int causal;
  int num_seqs, q_blocks;           // work items: q_blocks x num_seqs x hq
  int32_t* status;
};

// One work item: 256 query rows (two tiles) of one head of one sequence.
struct PfItem {
  int seq, head, m0;                // first query row inside the sequence
  int qs, q_len, ks, k_len;
  int n_t[PF_QT];                   // K/V tiles each query tile visits
  int nkv;                          // tiles the CTA streams = max over the tiles
};

__device__ __forceinline__ uint64_t pf_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool pf_wait(uint64_t* bar, uint32_t parity,
                                        volatile int* abort_flag, int32_t* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = pf_ns();
  for (;;) {
    for (int i = 0; i < 128; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (pf_ns() - t0 > 2000000000ull) {
      *abort_flag = 1;
      if (status) atomicOr(status, FK_DEV_WAIT_TIMEOUT);
      return false;
    }
  }
}

// Packed fp32 pairs (one instruction for two lanes of arithmetic) and the
// three-input maximum: the softmax is bound by instruction issue.
__device__ __forceinline__ uint64_t pf_pack2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void pf_unpack2(uint64_t v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t pf_fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t pf_add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float pf_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// The same wait for a converged warp: every lane gets the same answer, so the
// warp stays converged for the elect.sync that follows.
__device__ __forceinline__ bool pf_wait_warp(uint64_t* bar, uint32_t parity,
                                             volatile int* abort_flag, int32_t* status) {
  return __all_sync(0xffffffffu, pf_wait(bar, parity, abort_flag, status) ? 1 : 0) != 0;
}

// Items are numbered heaviest first (last query block first: causal rows see the
// most keys), sequences and heads inside a block adjacent so that CTAs running at
// the same time share K/V in L2.  CTA c of G takes items c, c + G, c + 2G, ...
// (a boustrophedon order measured no better).
__device__ __forceinline__ PfItem pf_load_item(const PrefillParams& p, int idx) {
  PfItem it;
  const int per_block = p.num_seqs * p.hq;
  const int qb = p.q_blocks - 1 - idx / per_block;
  const int rem = idx % per_block;
  it.seq = rem / p.hq;
  it.head = rem % p.hq;
  it.m0 = qb * (PF_QT * PF_BM);
  it.qs = p.cu_q[it.seq];
  it.q_len = p.cu_q[it.seq + 1] - it.qs;
  it.ks = p.cu_k[it.seq];
  it.k_len = p.cu_k[it.seq + 1] - it.ks;
  it.nkv = 0;
#pragma unroll
  for (int t = 0; t < PF_QT; ++t) {
    const int m0t = it.m0 + t * PF_BM;
    int n = 0;
    if (m0t < it.q_len) {
      const int last_row = min(m0t + PF_BM - 1, it.q_len - 1);
      const int hi = p.causal ? min(it.k_len - it.q_len + last_row, it.k_len - 1) : it.k_len - 1;
      if (hi >= 0) n = hi / PF_BN + 1;
    }
    it.n_t[t] = n;
    it.nkv = max(it.nkv, n);
  }
  return it;
}

__global__ void __launch_bounds__(PF_THREADS, 1)
prefill_attn_kernel(const __grid_constant__ CUtensorMap tmap_q,
                    const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v,
                    const PrefillParams p) {
  extern __shared__ uint8_t pf_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(pf_smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PF_OFF_BAR);
  uint64_t* q_full = bars;                           // Q tiles of an item landed
  uint64_t* q_empty = bars + 1;                      // ... and are no longer read
  uint64_t* slot_full = bars + 2;                    // [PF_SLOTS]
  uint64_t* slot_empty = slot_full + PF_SLOTS;       // [PF_SLOTS]
  uint64_t* s_full = slot_empty + PF_SLOTS;          // [PF_QT]
  uint64_t* p_full = s_full + PF_QT;                 // [PF_QT]
  uint64_t* o_full = p_full + PF_QT;                 // [PF_QT]
  uint64_t* o_empty = o_full + PF_QT;                // [PF_QT]: O_t read out by the epilogue
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_empty + PF_QT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(o_empty + PF_QT + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_items = p.q_blocks * p.num_seqs * p.hq;
  const int stride = gridDim.x;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int i = 0; i < PF_SLOTS; ++i) {
      mbar_init(&slot_full[i], 1);
      mbar_init(&slot_empty[i], 1);
    }
    for (int t = 0; t < PF_QT; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 4);
      mbar_init(&o_full[t], 1);
      mbar_init(&o_empty[t], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == PF_WARP_TMA && lane == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == PF_WARP_MMA) tmem_alloc(tmem_slot, PF_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // The kernel takes all 512 columns, so the allocation can only start at
  // column 0; addresses are then compile-time constants.  Anything else is
  // reported and the CTA does no work.
  const uint32_t tmem_got = *tmem_slot;
  constexpr uint32_t tmem_base = 0;
  if (tmem_got != 0) {
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, FK_DEV_TMEM_BASE);
    __syncthreads();
    if (warp == PF_WARP_MMA) tmem_dealloc(tmem_got, PF_TMEM_COLS);
    return;
  }
  pdl_wait();     // q, K/V, cu_seqlens and block tables may come from earlier kernels

  if (warp >= PF_WARP_TMA) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PF_REGS_OTHER));
  if (warp == PF_WARP_TMA) {
    // ============================ TMA producer ============================
    // Runs ahead of the other roles: the Q tiles of the next item are fetched as
    // soon as the last S product of the current one has been issued, its K/V
    // tiles as ring slots come free.
    const int st = p.sub_tokens;
    const int npieces = PF_BN / st;
    int kv_idx = 0;          // running slot-use count over all items
    int q_loads = 0;         // items whose Q has been requested
    bool ok = true;
    for (int idx = blockIdx.x; idx < total_items && ok; idx += stride) {
      const PfItem it = pf_load_item(p, idx);
      if (it.nkv == 0) continue;
      const int kvh = it.head / p.g;
      int pass = 1;
      if (lane == 0) {
        if (q_loads > 0)
          pass = pf_wait(q_empty, (uint32_t)(q_loads - 1) & 1u, abort_flag, p.status) ? 1 : 0;
        if (pass) {
          int nact = 0;
          for (int t = 0; t < PF_QT; ++t) nact += it.n_t[t] > 0 ? 1 : 0;
          mbar_arrive_expect_tx(q_full, (uint32_t)nact * PF_TILE_BYTES);
          for (int t = 0; t < PF_QT; ++t) {
            if (it.n_t[t] == 0) continue;
            for (int dh = 0; dh < 2; ++dh)
              tma_load_4d(smem + PF_OFF_Q + t * PF_TILE_BYTES + dh * PF_HALF_BYTES, &tmap_q,
                          q_full, dh * 64, it.head, it.qs + it.m0 + t * PF_BM, 0);
          }
        }
      }
      pass = __shfl_sync(0xffffffffu, pass, 0);
      if (!pass) { ok = false; break; }
      ++q_loads;
      const int32_t* bt = p.block_tables + (int64_t)it.seq * p.bt_stride;
      for (int i = 0; i < 2 * it.nkv; ++i, ++kv_idx) {
        const int slot = kv_idx % PF_SLOTS;
        const uint32_t lap = (uint32_t)(kv_idx / PF_SLOTS) & 1u;
        const int j = i >> 1;
        const bool is_v = i & 1;
        pass = 1;
        if (lane == 0) pass = pf_wait(&slot_empty[slot], lap ^ 1, abort_flag, p.status) ? 1 : 0;
        pass = __shfl_sync(0xffffffffu, pass, 0);
        if (!pass) { ok = false; break; }
        if (lane == 0) mbar_arrive_expect_tx(&slot_full[slot], PF_TILE_BYTES);
        __syncwarp();
        if (lane < npieces) {
          const int tok = j * PF_BN + lane * st;   // position inside the sequence
          uint8_t* dst = smem + PF_OFF_KV + slot * PF_TILE_BYTES + lane * st * 128;
          const CUtensorMap* map = is_v ? &tmap_v : &tmap_k;
          if (p.paged) {
            int page = p.num_blocks;     // out of range: the copy reads the zero fill
            if (tok < it.k_len) {
              page = bt[p.bs_shift >= 0 ? (tok >> p.bs_shift) : (tok / p.block_size)];
              if (page < 0 || page >= p.num_blocks) {
                page = p.num_blocks;
                if (p.status) atomicOr(p.status, FK_DEV_BAD_PAGE);
              }
            }
            const int off = p.bs_shift >= 0 ? (tok & (p.block_size - 1)) : (tok % p.block_size);
            const int c1 = p.hnd ? off : kvh, c2 = p.hnd ? kvh : off;
            tma_load_4d(dst, map, &slot_full[slot], 0, c1, c2, page);
            tma_load_4d(dst + PF_HALF_BYTES, map, &slot_full[slot], 64, c1, c2, page);
          } else {
            tma_load_4d(dst, map, &slot_full[slot], 0, kvh, it.ks + tok, 0);
            tma_load_4d(dst + PF_HALF_BYTES, map, &slot_full[slot], 64, kvh, it.ks + tok, 0);
          }
        }
      }
    }
  } else if (warp == PF_WARP_MMA) {
    // ============================= MMA issuer =============================
    // The whole warp walks the schedule converged; one elected lane issues.
    constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) |
                                 ((uint32_t)(PF_BN >> 3) << 17) |
                                 ((uint32_t)(PF_BM >> 4) << 24);
    constexpr uint32_t idesc_pv = idesc_s | (1u << 16);   // B (= V) is MN-major
    const uint32_t q_addr = smem_u32(smem + PF_OFF_Q);
    const uint32_t kv_addr = smem_u32(smem + PF_OFF_KV);
    auto issue_s = [&](int t, int slot) {
      const uint32_t a = q_addr + t * PF_TILE_BYTES;
      const uint32_t b = kv_addr + slot * PF_TILE_BYTES;
#pragma unroll
      for (int kk = 0; kk < PF_D / 16; ++kk) {
        const uint32_t o = (kk >> 2) * PF_HALF_BYTES + (kk & 3) * 32;
        tc_mma_bf16_elect(tmem_base + t * PF_BN, smem_desc_sw128(a + o),
                          smem_desc_sw128(b + o), idesc_s, kk > 0 ? 1u : 0u);
      }
    };
    auto issue_pv = [&](int t, int slot, bool acc) {
      // P_t sits in the first 64 columns of S_t (two bf16 per cell): 16 keys
      // = 8 columns per instruction
      const uint32_t a = tmem_base + t * PF_BN;
      const uint32_t b = kv_addr + slot * PF_TILE_BYTES;
#pragma unroll
      for (int kk = 0; kk < PF_BN / 16; ++kk) {
        tc_mma_bf16_ts_elect(tmem_base + 2 * PF_BN + t * PF_D, a + kk * 8,
                             smem_desc_sw128_mn(b + kk * 2048, PF_HALF_BYTES, 1024),
                             idesc_pv, (acc || kk > 0) ? 1u : 0u);
      }
    };
    int kv_base = 0;               // slot uses before this item
    int items = 0;                 // items with work so far
    uint32_t n_sp[PF_QT] = {0, 0}; // S / P hand-overs per tile so far
    uint32_t n_o[PF_QT] = {0, 0};  // items per tile so far
    bool ok = true;
    for (int idx = blockIdx.x; idx < total_items && ok; idx += stride) {
      const PfItem it = pf_load_item(p, idx);
      if (it.nkv == 0) continue;
      const int k0i = kv_base;     // K_0 of this item
      ok = pf_wait_warp(q_full, (uint32_t)items & 1u, abort_flag, p.status) &&
           pf_wait_warp(&slot_full[k0i % PF_SLOTS], (uint32_t)(k0i / PF_SLOTS) & 1u, abort_flag,
                        p.status);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int t = 0; t < PF_QT; ++t) {
        if (it.n_t[t] > 0) {
          issue_s(t, k0i % PF_SLOTS);
          tc_commit_elect(&s_full[t]);
        }
      }
      tc_commit_elect(&slot_empty[k0i % PF_SLOTS]);
      if (it.nkv == 1) tc_commit_elect(q_empty);      // Q is not read again
      for (int j = 0; j < it.nkv && ok; ++j) {
        const int vi = kv_base + 2 * j + 1, ki = kv_base + 2 * j + 2;
        const int vslot = vi % PF_SLOTS, kslot = ki % PF_SLOTS;
        ok = pf_wait_warp(&slot_full[vslot], (uint32_t)(vi / PF_SLOTS) & 1u, abort_flag,
                          p.status);
        if (!ok) break;
        bool k_ready = false;
#pragma unroll
        for (int t = 0; t < PF_QT; ++t) {
          if (!ok) break;
          if (j < it.n_t[t]) {
            if (j == 0 && n_o[t] > 0) {
              // O_t still holds the previous item until its epilogue has read it
              ok = pf_wait_warp(&o_empty[t], (n_o[t] - 1) & 1u, abort_flag, p.status);
              if (!ok) break;
            }
            ok = pf_wait_warp(&p_full[t], (n_sp[t] + (uint32_t)j) & 1u, abort_flag, p.status);
            if (!ok) break;
            tc_fence_after();
            issue_pv(t, vslot, j > 0);
            if (j == it.n_t[t] - 1) tc_commit_elect(&o_full[t]);
          }
          if (j + 1 < it.n_t[t]) {
            if (!k_ready) {
              ok = pf_wait_warp(&slot_full[kslot], (uint32_t)(ki / PF_SLOTS) & 1u, abort_flag,
                                p.status);
              if (!ok) break;
              tc_fence_after();
              k_ready = true;
            }
            issue_s(t, kslot);
            tc_commit_elect(&s_full[t]);
          }
        }
        if (!ok) break;
        tc_commit_elect(&slot_empty[vslot]);
        if (k_ready) tc_commit_elect(&slot_empty[kslot]);
        // the last S products of the item have just been issued: Q may be replaced
        if (j + 2 == it.nkv) tc_commit_elect(q_empty);
      }
      kv_base += 2 * it.nkv;
      ++items;
#pragma unroll
      for (int t = 0; t < PF_QT; ++t) {
        n_sp[t] += (uint32_t)it.n_t[t];
        if (it.n_t[t] > 0) ++n_o[t];
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(PF_REGS_SOFTMAX));
    // ============================== softmax ===============================
    const int t = warp >> 2;
    const int quad = warp & 3;                 // TMEM lanes 32 quad .. 32 quad + 31
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t s_addr = lane_addr + t * PF_BN;
    const uint32_t o_addr = lane_addr + 2 * PF_BN + t * PF_D;
    const float sc = p.scale_log2;
    const uint64_t sc2 = pf_pack2(sc, sc);
    int kv_base = 0;
    uint32_t n_sp = 0, n_o = 0;
    bool ok = true;
    for (int idx = blockIdx.x; idx < total_items && ok; idx += stride) {
      // Only what the tile loop needs stays live across it; the output pointers are
      // recomputed for the epilogue (the score row takes most of the registers).
      int my_n, nkv_item, k_len, lim;
      {
        const PfItem it = pf_load_item(p, idx);
        const int m0t = it.m0 + t * PF_BM;
        my_n = t ? it.n_t[1] : it.n_t[0];
        nkv_item = it.nkv;
        k_len = it.k_len;
        lim = p.causal ? min(it.k_len - it.q_len + m0t + row, it.k_len - 1) : it.k_len - 1;
        if (my_n == 0) {
          // a tile without visible keys (k_len == 0 or fewer keys than queries)
          if (m0t + row < it.q_len) {
            const int64_t tok = (int64_t)it.qs + m0t + row;
            uint4* dst = reinterpret_cast<uint4*>(p.out + tok * p.out_stride +
                                                  (int64_t)it.head * PF_D);
            for (int c = 0; c < 16; ++c) dst[c] = make_uint4(0u, 0u, 0u, 0u);
            if (p.lse) p.lse[(int64_t)it.head * p.total_q + tok] = -INFINITY;
          }
          kv_base += 2 * it.nkv;
          continue;
        }
      }
      float m_used = -INFINITY, l = 0.f;
      for (int j = 0; j < my_n; ++j) {
        if (!pf_wait(&s_full[t], (n_sp + (uint32_t)j) & 1u, abort_flag, p.status)) {
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t sr[128];
#pragma unroll
        for (int c = 0; c < 4; ++c) tc_ld32(s_addr + c * 32, sr + c * 32);
        tc_wait_ld();
        const int k0 = j * PF_BN;
        if (k0 + PF_BN - 1 > lim) {
          // the tile crosses this row's last visible key
#pragma unroll
          for (int c = 0; c < 128; ++c)
            if (k0 + c > lim) sr[c] = 0xff800000u;   // -inf
        }
        // row max of the raw scores (the scale is positive), four chains
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 128; c += 8) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            mx4[i] = pf_max3(mx4[i], __uint_as_float(sr[c + i]), __uint_as_float(sr[c + 4 + i]));
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sc;
        if (j == 0) {
          m_used = mx;
        } else {
          const bool grow = mx > m_used + PF_RESCALE_LOG2;
          if (__any_sync(0xffffffffu, grow)) {
            const float alpha = grow ? fast_exp2(m_used - mx) : 1.0f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t o[32];
              tc_ld32(o_addr + c * 32, o);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i)
                o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tc_st32(o_addr + c * 32, o);
            }
            tc_wait_st();
            if (grow) {
              l *= alpha;
              m_used = mx;
            }
          }
        }
        const float neg_mu = m_used == -INFINITY ? 0.f : -m_used;
        const uint64_t nm2 = pf_pack2(neg_mu, neg_mu);
        uint64_t sum2[2] = {0ull, 0ull};
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          float t0, t1, t2, t3;
          pf_unpack2(pf_fma2(pf_pack2(__uint_as_float(sr[2 * c]), __uint_as_float(sr[2 * c + 1])),
                             sc2, nm2), t0, t1);
          pf_unpack2(pf_fma2(pf_pack2(__uint_as_float(sr[2 * c + 2]),
                                      __uint_as_float(sr[2 * c + 3])), sc2, nm2), t2, t3);
          const float e0 = fast_exp2(t0), e1 = fast_exp2(t1);
          const float e2 = fast_exp2(t2), e3 = fast_exp2(t3);
          sum2[0] = pf_add2(sum2[0], pf_pack2(e0, e1));
          sum2[1] = pf_add2(sum2[1], pf_pack2(e2, e3));
          sr[c] = pack_bf16(e0, e1);
          sr[c + 1] = pack_bf16(e2, e3);
        }
        {
          float a0, a1, a2, a3;
          pf_unpack2(sum2[0], a0, a1);
          pf_unpack2(sum2[1], a2, a3);
          l += (a0 + a1) + (a2 + a3);
        }
        // P (bf16 pairs) over the first 64 columns of this row's S
        tc_st32(s_addr, sr);
        tc_st32(s_addr + 32, sr + 32);
        tc_wait_st();
        if (k0 + PF_BN > k_len) {
          // Rows of V past the end of the sequence hold whatever memory had
          // there; P is zero for them, but 0 * NaN would poison the sum.
          const int vi = kv_base + 2 * j + 1;
          const int vslot = vi % PF_SLOTS;
          if (!pf_wait(&slot_full[vslot], (uint32_t)(vi / PF_SLOTS) & 1u, abort_flag,
                       p.status)) {
            ok = false;
            break;
          }
          uint8_t* vt = smem + PF_OFF_KV + vslot * PF_TILE_BYTES;
          const int first = max(k_len - k0, 0);
          for (int i = first * 16 + row; i < PF_BN * 16; i += 128) {
            const int r = i >> 4, c = i & 15;
            *reinterpret_cast<uint4*>(vt + (c >> 3) * PF_HALF_BYTES + r * 128 +
                                      (c & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
          }
          fence_proxy_async_smem();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[t]);
      }
      if (!ok) break;
      // a row that never saw a key has no reference value: its result is zero
      if (m_used == -INFINITY) l = 0.f;
      if (!pf_wait(&o_full[t], n_o & 1u, abort_flag, p.status)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      const PfItem it = pf_load_item(p, idx);
      const bool row_valid = it.m0 + t * PF_BM + row < it.q_len;
      const int64_t tok = (int64_t)it.qs + it.m0 + t * PF_BM + row;
      uint4* dst = reinterpret_cast<uint4*>(p.out + tok * p.out_stride + (int64_t)it.head * PF_D);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tc_ld32(o_addr + c * 32, o);
        tc_wait_ld();
        if (c == 3) {
          // O_t is in registers now: the next item's first P V may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&o_empty[t]);
        }
        if (row_valid) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            dst[c * 4 + i] = make_uint4(
                pack_bf16(__uint_as_float(o[i * 8 + 0]) * inv,
                          __uint_as_float(o[i * 8 + 1]) * inv),
                pack_bf16(__uint_as_float(o[i * 8 + 2]) * inv,
                          __uint_as_float(o[i * 8 + 3]) * inv),
                pack_bf16(__uint_as_float(o[i * 8 + 4]) * inv,
                          __uint_as_float(o[i * 8 + 5]) * inv),
                pack_bf16(__uint_as_float(o[i * 8 + 6]) * inv,
                          __uint_as_float(o[i * 8 + 7]) * inv));
          }
        }
      }
      if (row_valid && p.lse) {
        p.lse[(int64_t)it.head * p.total_q + tok] =
            l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
      }
      kv_base += 2 * nkv_item;
      n_sp += (uint32_t)my_n;
      ++n_o;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == PF_WARP_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem_got, PF_TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// merge of two partial results: one thread per 8 elements of one (token, head)
// ---------------------------------------------------------------------------
struct MergeParams {
  uint16_t* out; int64_t out_st, out_sh;
  float* out_lse;
  const uint16_t* a; int64_t a_st, a_sh; const float* a_lse;
  const uint16_t* b; int64_t b_st, b_sh; const float* b_lse;
  int64_t tokens; int heads, packs;   // packs = head_dim / 8
  int64_t with_context;
};

__global__ void __launch_bounds__(256)
merge_attn_states_kernel(const MergeParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = p.tokens * p.heads * p.packs;
  if (gid >= total) return;
  const int pack = (int)(gid % p.packs);
  const int64_t th = gid / p.packs;
  const int head = (int)(th % p.heads);
  const int64_t tok = th / p.heads;
  const uint4* pa = reinterpret_cast<const uint4*>(p.a + tok * p.a_st + head * p.a_sh) + pack;
  const uint4* pb = reinterpret_cast<const uint4*>(p.b + tok * p.b_st + head * p.b_sh) + pack;
  uint4* po = reinterpret_cast<uint4*>(p.out + tok * p.out_st + head * p.out_sh) + pack;
  const int64_t li = (int64_t)head * p.tokens + tok;
  if (tok >= p.with_context) {
    // tokens without a prefix: the suffix result is the result
    *po = *pb;
    if (p.out_lse && pack == 0) p.out_lse[li] = p.b_lse[li];
    return;
  }
  float la = p.a_lse[li], lb = p.b_lse[li];
  if (isinf(la)) la = -INFINITY;
  if (isinf(lb)) lb = -INFINITY;
  const float mx = fmaxf(la, lb);
  if (isinf(mx)) {
    // neither side saw a key: pass the prefix through (zeros by convention)
    *po = *pa;
    if (p.out_lse && pack == 0) p.out_lse[li] = mx;
    return;
  }
  const float ea = expf(la - mx), eb = expf(lb - mx);
  const float se = ea + eb;
  const float wa = ea / se, wb = eb / se;
  const uint4 va = *pa, vb = *pb;
  uint4 r;
  r.x = pack_bf16(bf16lo(va.x) * wa + bf16lo(vb.x) * wb, bf16hi(va.x) * wa + bf16hi(vb.x) * wb);
  r.y = pack_bf16(bf16lo(va.y) * wa + bf16lo(vb.y) * wb, bf16hi(va.y) * wa + bf16hi(vb.y) * wb);
  r.z = pack_bf16(bf16lo(va.z) * wa + bf16lo(vb.z) * wb, bf16hi(va.z) * wa + bf16hi(vb.z) * wb);
  r.w = pack_bf16(bf16lo(va.w) * wa + bf16lo(vb.w) * wb, bf16hi(va.w) * wa + bf16hi(vb.w) * wb);
  *po = r;
  if (p.out_lse && pack == 0) p.out_lse[li] = logf(se) + mx;
}

// ---------------------------------------------------------------------------
// host: 4-D tensor maps (dims innermost first), cached by their definition
// ---------------------------------------------------------------------------
struct Map4Key {
  const void* ptr; uint64_t d[4]; uint64_t s[3]; uint32_t b[4];
  bool operator==(const Map4Key& o) const {
    if (ptr != o.ptr) return false;
    for (int i = 0; i < 4; ++i) if (d[i] != o.d[i] || b[i] != o.b[i]) return false;
    for (int i = 0; i < 3; ++i) if (s[i] != o.s[i]) return false;
    return true;
  }
};
struct Map4Hash {
  size_t operator()(const Map4Key& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    for (int i = 0; i < 4; ++i) h = h * 1000003u ^ (size_t)(k.d[i] * 31u + k.b[i]);
    for (int i = 0; i < 3; ++i) h = h * 1000003u ^ (size_t)k.s[i];
    return h;
  }
};
static std::mutex g_m4_mu;
static std::unordered_map<Map4Key, CUtensorMap, Map4Hash> g_m4;

static int get_map4(const void* ptr, const uint64_t (&dims)[4],
                    const uint64_t (&strides_bytes)[3], const uint32_t (&box)[4],
                    CUtensorMap* out) {
  Map4Key key;
  key.ptr = ptr;
  for (int i = 0; i < 4; ++i) { key.d[i] = dims[i]; key.b[i] = box[i]; }
  for (int i = 0; i < 3; ++i) key.s[i] = strides_bytes[i];
  std::lock_guard<std::mutex> lk(g_m4_mu);
  auto it = g_m4.find(key);
  if (it != g_m4.end()) {
    *out = it->second;
    return FK_OK;
  }
  tensormap_encode_fn enc = get_tensormap_encode();
  FK_REQUIRE(enc != nullptr, FK_ERR_CUDA,
             "cuTensorMapEncodeTiled not available from the driver");
  cuuint64_t d[4], s[3];
  cuuint32_t b[4], e[4] = {1, 1, 1, 1};
  for (int i = 0; i < 4; ++i) { d[i] = dims[i]; b[i] = box[i]; }
  for (int i = 0; i < 3; ++i) s[i] = strides_bytes[i];
  CUtensorMap m;
  CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), d,
                   s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FK_REQUIRE(r == CUDA_SUCCESS, FK_ERR_CUDA,
             "cuTensorMapEncodeTiled failed with code %d", (int)r);
  if (g_m4.size() > 4096) g_m4.clear();
  g_m4.emplace(key, m);
  *out = m;
  return FK_OK;
}

// [tokens, heads, 128] bf16 with a token stride: dims (D, heads, tokens, 1)
static int token_major_map(const void* ptr, int64_t tokens, int heads,
                           int64_t stride_token, uint32_t box_tokens,
                           CUtensorMap* out) {
  const uint64_t dims[4] = {PF_D, (uint64_t)heads, (uint64_t)tokens, 1};
  const uint64_t strides[3] = {(uint64_t)PF_D * 2, (uint64_t)stride_token * 2,
                               (uint64_t)stride_token * 2 * (uint64_t)tokens};
  const uint32_t box[4] = {64, 1, box_tokens, 1};
  return get_map4(ptr, dims, strides, box, out);
}

}  // namespace fk

using namespace fk;

extern "C" {

int fk_prefill_attn(const void* q, int64_t q_stride_token, void* out,
                    int64_t out_stride_token, float* out_lse, const void* k,
                    const void* v, int64_t kv_stride, int64_t num_blocks,
                    int block_size, int kv_layout, const int32_t* cu_seqlens_q,
                    const int32_t* cu_seqlens_k, const int32_t* block_tables,
                    int64_t block_table_stride, int num_seqs, int64_t total_q,
                    int64_t total_k, int max_seqlen_q, int num_q_heads,
                    int num_kv_heads, int head_dim, float softmax_scale, int causal,
                    int32_t* status, fk_stream_t stream) {
  FK_REQUIRE(num_seqs >= 0 && total_q >= 0, FK_ERR_INVALID_ARG,
             "fk_prefill_attn: negative size");
  if (num_seqs == 0 || total_q == 0 || max_seqlen_q <= 0) return FK_OK;
  FK_REQUIRE(q && out && k && v && cu_seqlens_q && cu_seqlens_k, FK_ERR_INVALID_ARG,
             "fk_prefill_attn: null pointer");
  FK_REQUIRE(head_dim == PF_D, FK_ERR_UNSUPPORTED,
             "fk_prefill_attn: head_dim %d unsupported (128 only)", head_dim);
  FK_REQUIRE(num_q_heads > 0 && num_kv_heads > 0 && num_q_heads % num_kv_heads == 0,
             FK_ERR_INVALID_ARG,
             "fk_prefill_attn: num_q_heads must be a multiple of num_kv_heads");
  FK_REQUIRE(aligned16(q) && aligned16(out) && aligned16(k) && aligned16(v) &&
                 q_stride_token % 8 == 0 && out_stride_token % 8 == 0 &&
                 kv_stride % 8 == 0,
             FK_ERR_ALIGNMENT,
             "fk_prefill_attn: pointers must be 16-byte aligned, strides multiples of 8");
  FK_REQUIRE(q_stride_token >= (int64_t)num_q_heads * PF_D &&
                 out_stride_token >= (int64_t)num_q_heads * PF_D,
             FK_ERR_INVALID_ARG, "fk_prefill_attn: token stride below heads * 128");
  const bool paged = num_blocks > 0;
  PrefillParams p{};
  CUtensorMap mq, mk, mv;
  int rc = FK_OK;
  // every argument check comes before the first driver call
  if (paged) {
    FK_REQUIRE(block_tables != nullptr, FK_ERR_INVALID_ARG,
               "fk_prefill_attn: paged K/V needs block tables");
    FK_REQUIRE(kv_layout == 0 || kv_layout == 1, FK_ERR_INVALID_ARG,
               "fk_prefill_attn: unknown kv_layout %d", kv_layout);
    FK_REQUIRE(block_size == 16 || block_size == 32 ||
                   (block_size >= 64 && block_size % 64 == 0),
               FK_ERR_UNSUPPORTED,
               "fk_prefill_attn: block_size %d must be 16, 32 or a multiple of 64",
               block_size);
    FK_REQUIRE(kv_stride >= (int64_t)block_size * num_kv_heads * PF_D,
               FK_ERR_INVALID_ARG, "fk_prefill_attn: block stride below the block size");
    const uint32_t sub = (uint32_t)(block_size < 64 ? block_size : 64);
    const bool hnd = kv_layout == 1;
    uint64_t dims[4], strides[3];
    uint32_t box[4];
    dims[0] = PF_D; dims[3] = (uint64_t)num_blocks;
    strides[0] = PF_D * 2; strides[2] = (uint64_t)kv_stride * 2;
    box[0] = 64; box[3] = 1;
    if (hnd) {
      dims[1] = (uint64_t)block_size; dims[2] = (uint64_t)num_kv_heads;
      strides[1] = (uint64_t)block_size * PF_D * 2;
      box[1] = sub; box[2] = 1;
    } else {
      dims[1] = (uint64_t)num_kv_heads; dims[2] = (uint64_t)block_size;
      strides[1] = (uint64_t)num_kv_heads * PF_D * 2;
      box[1] = 1; box[2] = sub;
    }
    rc = get_map4(k, dims, strides, box, &mk);
    if (rc != FK_OK) return rc;
    rc = get_map4(v, dims, strides, box, &mv);
    if (rc != FK_OK) return rc;
    p.paged = 1;
    p.hnd = hnd ? 1 : 0;
    p.block_size = block_size;
    p.bs_shift = (block_size & (block_size - 1)) == 0 ? __builtin_ctz(block_size) : -1;
    p.sub_tokens = (int)sub;
    p.num_blocks = (int)num_blocks;
  } else {
    FK_REQUIRE(total_k > 0, FK_ERR_INVALID_ARG, "fk_prefill_attn: total_k must be > 0");
    FK_REQUIRE(kv_stride >= (int64_t)num_kv_heads * PF_D, FK_ERR_INVALID_ARG,
               "fk_prefill_attn: token stride below heads * 128");
    rc = token_major_map(k, total_k, num_kv_heads, kv_stride, 64, &mk);
    if (rc != FK_OK) return rc;
    rc = token_major_map(v, total_k, num_kv_heads, kv_stride, 64, &mv);
    if (rc != FK_OK) return rc;
    p.paged = 0;
    p.sub_tokens = 64;
    p.bs_shift = -1;
    p.block_size = 1;
  }
  rc = token_major_map(q, total_q, num_q_heads, q_stride_token, PF_BM, &mq);
  if (rc != FK_OK) return rc;
  p.out = static_cast<uint16_t*>(out);
  p.out_stride = out_stride_token;
  p.lse = out_lse;
  p.total_q = total_q;
  p.cu_q = cu_seqlens_q;
  p.cu_k = cu_seqlens_k;
  p.block_tables = block_tables;
  p.bt_stride = block_table_stride;
  p.hq = num_q_heads;
  p.g = num_q_heads / num_kv_heads;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.causal = causal ? 1 : 0;
  p.status = status;

  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  static int launch_regs = 0;
  static PerDeviceOnce smem_once;
  FK_CUDA_OK(set_max_dynamic_smem(smem_once, prefill_attn_kernel, PF_SMEM_ALLOC));
  // registers per thread of the compiled kernel: the same on every device
  std::call_once(once, [] {
    cudaFuncAttributes fa;
    attr_err = cudaFuncGetAttributes(&fa, prefill_attn_kernel);
    if (attr_err == cudaSuccess) launch_regs = fa.numRegs;
  });
  FK_CUDA_OK(attr_err);
  FK_REQUIRE(launch_regs * PF_THREADS >= PF_REGS_NEEDED, FK_ERR_UNSUPPORTED,
             "fk_prefill_attn: this build of the kernel holds %d registers per thread, "
             "fewer than its warpgroup register split needs", launch_regs);
  const int q_blocks = (max_seqlen_q + PF_QT * PF_BM - 1) / (PF_QT * PF_BM);
  const int64_t items = (int64_t)q_blocks * num_q_heads * num_seqs;
  FK_REQUIRE(items <= 0x7fffffff, FK_ERR_UNSUPPORTED, "fk_prefill_attn: too many work items");
  p.num_seqs = num_seqs;
  p.q_blocks = q_blocks;
  const int ctas = (int)(items < sm_count() ? items : sm_count());
  dim3 grid((unsigned)ctas);
  FK_CUDA_OK(launch_kernel(prefill_attn_kernel, grid, dim3(PF_THREADS), (size_t)PF_SMEM_ALLOC,
                           static_cast<cudaStream_t>(stream), mq, mk, mv, p));
  count_launch(1);
  return FK_OK;
}

int fk_merge_attn_states(void* out, int64_t out_stride_token, int64_t out_stride_head,
                         float* out_lse, const void* prefix_out,
                         int64_t prefix_stride_token, int64_t prefix_stride_head,
                         const float* prefix_lse, const void* suffix_out,
                         int64_t suffix_stride_token, int64_t suffix_stride_head,
                         const float* suffix_lse, int64_t num_tokens, int num_heads,
                         int head_dim, int64_t prefill_tokens_with_context,
                         fk_stream_t stream) {
  FK_REQUIRE(num_tokens >= 0 && num_heads >= 0, FK_ERR_INVALID_ARG,
             "fk_merge_attn_states: negative size");
  if (num_tokens == 0 || num_heads == 0) return FK_OK;
  FK_REQUIRE(out && prefix_out && prefix_lse && suffix_out && suffix_lse,
             FK_ERR_INVALID_ARG, "fk_merge_attn_states: null pointer");
  FK_REQUIRE(head_dim > 0 && head_dim % 8 == 0, FK_ERR_UNSUPPORTED,
             "fk_merge_attn_states: head_dim %d must be a multiple of 8", head_dim);
  FK_REQUIRE(aligned16(out) && aligned16(prefix_out) && aligned16(suffix_out) &&
                 out_stride_token % 8 == 0 && out_stride_head % 8 == 0 &&
                 prefix_stride_token % 8 == 0 && prefix_stride_head % 8 == 0 &&
                 suffix_stride_token % 8 == 0 && suffix_stride_head % 8 == 0,
             FK_ERR_ALIGNMENT,
             "fk_merge_attn_states: pointers must be 16-byte aligned, strides multiples of 8");
  MergeParams p{};
  p.out = static_cast<uint16_t*>(out);
  p.out_st = out_stride_token; p.out_sh = out_stride_head;
  p.out_lse = out_lse;
  p.a = static_cast<const uint16_t*>(prefix_out);
  p.a_st = prefix_stride_token; p.a_sh = prefix_stride_head; p.a_lse = prefix_lse;
  p.b = static_cast<const uint16_t*>(suffix_out);
  p.b_st = suffix_stride_token; p.b_sh = suffix_stride_head; p.b_lse = suffix_lse;
  p.tokens = num_tokens; p.heads = num_heads; p.packs = head_dim / 8;
  p.with_context = prefill_tokens_with_context < 0 ? num_tokens
                                                   : prefill_tokens_with_context;
  const int64_t total = num_tokens * num_heads * p.packs;
  const int64_t blocks = (total + 255) / 256;
  FK_REQUIRE(blocks <= 0x7fffffff, FK_ERR_UNSUPPORTED, "fk_merge_attn_states: too large");
  FK_CUDA_OK(launch_kernel(merge_attn_states_kernel, dim3((unsigned)blocks), dim3(256), (size_t)0,
                           static_cast<cudaStream_t>(stream), p));
  count_launch(1);
  return FK_OK;
}

}  // extern "C"
