// Paged GQA decode attention for sm_100a: split-KV, TMA-staged 128-token tiles,
// warp-shuffle online softmax, log-sum-exp merge.
//
// Replaces FlashAttnDecode.forward
// (fastkernels/tasks/baseline/L1/flash_attn_decode.py:113-181); the maths is
// Attention._decode_torch (fastkernels/tasks/baseline/L2/attention_impl.py:
// 598-664).
//
// Three launches per call, all with static geometry (graph-capturable):
//   1. attn_plan_kernel   (1 CTA)  reads context_lens on the device, picks the
//      split size so that the persistent grid gets >= 4 work items per CTA,
//      and writes the per-sequence chunk prefix sum + zeroes the work counter.
//   2. attn_decode_kernel (1 persistent CTA per SM) work item = (sequence,
//      KV split, KV head).  A producer warp streams K/V tiles of 128 tokens
//      through a 3-stage shared-memory ring with cp.async.bulk.tensor (128B
//      swizzle); 8 consumer warps each own 16 tokens of a tile: S = Q K^T and
//      O += P V as bf16 m16n8k16 tensor-core tiles with all g = Hq/Hkv query
//      heads of the KV head stacked on the M dimension, so every K/V byte is
//      read from HBM exactly once; softmax state (running max / sum) lives in
//      registers and is reduced with quad shuffles.
//   3. attn_merge_kernel  merges the per-split (max, sum, un-normalised O)
//      partials of sequences that were split.
// A small self-planning call -- at most one (sequence, KV head) pair per SM and
// block tables of at most 2048 tokens -- is ONE launch instead: CTA b takes pair b
// whole, nothing is split, planned or merged.
//
// HBM traffic per call = the algorithmic bytes (K and V of every live token
// once, q, out, lens, block tables) + split partials (fp32, < 4 % at the chosen
// split sizes).
#include "fk_common.cuh"

#include <mutex>
#include <unordered_map>

namespace fk {

constexpr int ATT_D = 128;                  // head_dim
constexpr int ATT_NW = 8;                   // consumer warps
constexpr int ATT_TILE = ATT_NW * 16;       // tokens per pipeline stage
constexpr int ATT_BOX = 64;                 // tokens per TMA box
constexpr int ATT_STAGES = 3;
constexpr int ATT_THREADS = (ATT_NW + 1) * 32;
constexpr int ATT_BOX_BYTES = ATT_BOX * 128;          // 64 tokens x 64 bf16
constexpr int ATT_KV_BYTES = 4 * ATT_BOX_BYTES;       // one of K or V per stage
constexpr int ATT_STAGE_BYTES = 2 * ATT_KV_BYTES;     // 64 KiB
constexpr int ATT_QSLOT_BYTES = 16 * ATT_D * 2;       // 4 KiB
constexpr int ATT_MBUF_BYTES = 16 * 32 * 16;          // 8 KiB (16 n-tiles x 32 lanes x float4)
constexpr int ATT_PLAN_HDR = 8;                       // ints before chunk_start[]

enum : int { TILE_FIRST = 1, TILE_LAST = 2, TILE_END = 4 };

struct TileMeta {
  int seq, kvh, split, nsplits, n_valid, flags, pad0, pad1;
};

struct AttnSmem {
  static constexpr int kStages = 0;
  static constexpr int kQ = kStages + ATT_STAGES * ATT_STAGE_BYTES;
  static constexpr int kMbuf = kQ + ATT_STAGES * ATT_QSLOT_BYTES;
  static constexpr int kMl = kMbuf + 2 * ATT_MBUF_BYTES;
  static constexpr int kMeta = kMl + ATT_NW * 16 * 8;
  static constexpr int kBars = kMeta + ATT_STAGES * (int)sizeof(TileMeta);
  static constexpr int kAbort = kBars + 2 * ATT_STAGES * 8;
  static constexpr int kTotal = kAbort + 16;
  static constexpr int kAlloc = kTotal + 1024;  // manual 1024-byte alignment
};
static_assert(AttnSmem::kAlloc <= 232448, "shared memory budget");

struct AttnParams {
  const uint16_t* q; int64_t q_stride;
  uint16_t* out; int64_t out_stride;
  const int32_t* context_lens;
  const int32_t* block_tables; int64_t bt_stride;
  int batch, hq, hkv, g;
  int block_size; int num_blocks;
  int sub_tokens;     // tokens per TMA copy = min(block_size, 64)
  int fused16;        // 16-token pages: one 5-D copy brings both 64-dim halves of a page
  int bs_shift;       // log2(block_size) when it is a power of two, else -1
  int hnd;            // 1: pool is [blocks, Hkv, block, D]; 0: [blocks, block, Hkv, D]
  float scale_log2;
  int max_splits;
  int direct;         // 1: no plan, no splits: CTA b handles (sequence, KV head) item b whole
  int* plan;          // header + chunk_start[batch+1]
  int4* chunk_info;   // per chunk: {seq, split | nsplits << 16, tok_begin, tok_end}
  float* part_o;      // [batch, hq, max_splits, D]
  float2* part_ml;    // [batch, hq, max_splits]
  int32_t* status;
};

__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Wait with a wall-clock bound (2 s): returns false after recording
// FK_DEV_WAIT_TIMEOUT so the caller unwinds instead of spinning forever.
__device__ __forceinline__ bool att_wait(uint64_t* bar, uint32_t parity,
                                         volatile int* abort_flag,
                                         int32_t* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (global_ns() - t0 > 2000000000ull) {
      *abort_flag = 1;
      if (status) atomicOr(status, FK_DEV_WAIT_TIMEOUT);
      return false;
    }
  }
}

// ---------------------------------------------------------------------------
// plan
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) attn_plan_kernel(
    const int32_t* __restrict__ context_lens, int batch, int hkv,
    int max_splits, int grid_ctas, int64_t max_tokens_per_seq,
    int* __restrict__ plan, int4* __restrict__ chunk_info, int32_t* status) {
  __shared__ int red[33];
  __shared__ int s_chunk;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_launch_dependents();
  pdl_wait();

  auto block_reduce = [&](int v, bool is_max) -> int {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const int t = __shfl_xor_sync(0xffffffffu, v, o);
      v = is_max ? max(v, t) : v + t;
    }
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
      int t = red[lane];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const int u = __shfl_xor_sync(0xffffffffu, t, o);
        t = is_max ? max(t, u) : t + u;
      }
      if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
  };
  auto len_of = [&](int i) -> int {
    int L = context_lens[i];
    if (L < 0) L = 0;
    if ((int64_t)L > max_tokens_per_seq) {
      L = (int)max_tokens_per_seq;
      if (status) atomicOr(status, FK_DEV_BAD_PAGE);
    }
    return L;
  };

  int mx = 0;
  for (int i = tid; i < batch; i += blockDim.x) mx = max(mx, len_of(i));
  const int maxL = block_reduce(mx, true);

  int min_chunk = ATT_TILE;
  while ((int64_t)min_chunk * max_splits < maxL) min_chunk <<= 1;
  // 1024-token chunks measured best whenever they give every CTA >= 4 work items
  // (larger ones lengthen the tail of the dynamic schedule, smaller ones pay the
  // per-item merge more often); shrink only to keep the grid busy.
  int chunk = 1024;
  if (chunk < min_chunk) chunk = min_chunk;
  for (;;) {
    int cnt = 0;
    for (int i = tid; i < batch; i += blockDim.x)
      cnt += (len_of(i) + chunk - 1) / chunk;
    const int items = block_reduce(cnt, false) * hkv;
    if (items >= 4 * grid_ctas || (chunk >> 1) < min_chunk) break;
    chunk >>= 1;
  }
  if (tid == 0) s_chunk = chunk;
  __syncthreads();
  chunk = s_chunk;

  // exclusive prefix sum of chunks per sequence (contiguous slice per thread)
  const int per = (batch + blockDim.x - 1) / blockDim.x;
  const int lo = min(tid * per, batch), hi = min(lo + per, batch);
  int local = 0;
  for (int i = lo; i < hi; ++i) local += (len_of(i) + chunk - 1) / chunk;
  int incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  __syncthreads();
  if (lane == 31) red[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = red[lane], wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    red[lane] = wi - w;  // exclusive warp offsets
    if (lane == 31) red[32] = wi;
  }
  __syncthreads();
  int run = red[warp] + incl - local;
  int* chunk_start = plan + ATT_PLAN_HDR;
  for (int i = lo; i < hi; ++i) {
    chunk_start[i] = run;
    const int L = len_of(i);
    const int nc = (L + chunk - 1) / chunk;
    for (int c = 0; c < nc; ++c)
      chunk_info[run + c] =
          make_int4(i, c | (nc << 16), c * chunk, min(L, (c + 1) * chunk));
    run += nc;
  }
  if (tid == 0) {
    chunk_start[batch] = red[32];
    plan[0] = red[32];  // total chunks
    plan[1] = chunk;    // tokens per chunk
    plan[2] = 0;        // work counter
    plan[3] = maxL;
  }
}

// ---------------------------------------------------------------------------
// main kernel
// ---------------------------------------------------------------------------
template <bool G16>
__global__ void __launch_bounds__(ATT_THREADS, 1) attn_decode_kernel(
    const __grid_constant__ CUtensorMap tmap_k,
    const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem + AttnSmem::kStages;
  uint8_t* qslots = smem + AttnSmem::kQ;
  float4* mbuf = reinterpret_cast<float4*>(smem + AttnSmem::kMbuf);
  float2* ml = reinterpret_cast<float2*>(smem + AttnSmem::kMl);
  TileMeta* metas = reinterpret_cast<TileMeta*>(smem + AttnSmem::kMeta);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + AttnSmem::kBars);
  uint64_t* empty = full + ATT_STAGES;
  volatile int* abort_flag =
      reinterpret_cast<volatile int*>(smem + AttnSmem::kAbort);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ATT_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], ATT_NW);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  pdl_launch_dependents();
  __syncthreads();
  // everything below reads memory written by earlier kernels (plan, q, KV pool)
  pdl_wait();

  const int* plan = p.plan;

  if (warp == ATT_NW) {
    // ============================ producer warp ============================
    // Lane 0 schedules (work counter, stage hand-shake, tile descriptor, Q copy);
    // lane i issues the four K/V copies of the i-th page-sized piece of the tile,
    // so the up-to-8 page lookups and 32 copies of a 16-token-page tile go out in
    // parallel instead of through one thread.
    if (lane == 0) {
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
    }
    const int total_items = p.direct ? p.batch * p.hkv : plan[0] * p.hkv;
    int* counter = const_cast<int*>(plan) + 2;
    // direct mode: the schedule entry of item (sequence, KV head) is the whole
    // sequence as one unsplit chunk; lengths are clamped as the plan kernel does
    auto direct_info = [&](int item) -> int4 {
      const int sq = item / p.hkv;
      int L = p.context_lens[sq];
      if (L < 0) L = 0;
      const int64_t cap = p.bt_stride * (int64_t)p.block_size;
      if ((int64_t)L > cap) {
        L = (int)cap;
        if (p.status && lane == 0) atomicOr(p.status, FK_DEV_BAD_PAGE);
      }
      return make_int4(sq, 0 | (1 << 16), 0, L);
    };
    int stage = 0;
    uint32_t phase = 0;  // parity of the `empty` phase we wait for (first pass: free)
    bool ok = true;
    const int st = p.sub_tokens;
    auto page_of = [&](int t) -> int {
      return p.bs_shift >= 0 ? (t >> p.bs_shift) : (t / p.block_size);
    };
    auto off_of = [&](int t) -> int {
      return p.bs_shift >= 0 ? (t & (p.block_size - 1)) : (t % p.block_size);
    };
    // The schedule entry of the next item and each lane's page id of the next
    // tile are loaded one step ahead, so their L2 latency overlaps the wait for a
    // free stage instead of adding to it.
    int next = 0;
    if (p.direct) {
      next = (int)blockIdx.x;
    } else {
      if (lane == 0) next = atomicAdd(counter, 1);
      next = __shfl_sync(0xffffffffu, next, 0);
    }
    int4 next_info = make_int4(0, 0, 0, 0);
    if (next < total_items)
      next_info = p.direct ? direct_info(next) : p.chunk_info[next / p.hkv];
    while (ok) {
      const int item = next;
      if (item >= total_items) break;
      const int4 info = next_info;
      if (p.direct) {
        next = total_items;            // one item per CTA
      } else {
        if (lane == 0) next = atomicAdd(counter, 1);
        next = __shfl_sync(0xffffffffu, next, 0);
        if (next < total_items) next_info = p.chunk_info[next / p.hkv];
      }
      const int kvh = item % p.hkv;
      const int seq = info.x;
      const int split = info.y & 0xffff, nsplits = info.y >> 16;
      const int tok_begin = info.z, tok_end = info.w;
      if (p.direct && tok_end == 0) {
        // empty sequence: no tile reaches the consumers, the zeros are written here
        // (what the merge kernel does for such rows on the planned path)
        uint4* dst = reinterpret_cast<uint4*>(p.out + (int64_t)seq * p.out_stride +
                                              (int64_t)kvh * p.g * ATT_D);
        for (int i = lane; i < p.g * ATT_D / 8; i += 32) dst[i] = make_uint4(0u, 0u, 0u, 0u);
      }
      const int32_t* bt = p.block_tables + (int64_t)seq * p.bt_stride;
      // this lane's piece of a tile starts `lane * st` tokens into it
      const int my = lane * st;
      int pg = 0;
      if (my < ATT_TILE && tok_begin + my < tok_end) pg = bt[page_of(tok_begin + my)];
      for (int tok0 = tok_begin; tok0 < tok_end; tok0 += ATT_TILE) {
        // wait until the consumers released this stage (a fresh barrier
        // passes the parity-1 test, so the first lap does not block)
        int pass = 1;
        if (lane == 0) pass = att_wait(&empty[stage], phase ^ 1, abort_flag, p.status) ? 1 : 0;
        pass = __shfl_sync(0xffffffffu, pass, 0);
        if (!pass) {
          ok = false;
          break;
        }
        const int n_valid = min(ATT_TILE, tok_end - tok0);
        const int ncopy = (n_valid + st - 1) / st;   // pieces of this tile
        const int flags = (tok0 == tok_begin ? TILE_FIRST : 0) |
                          (tok0 + ATT_TILE >= tok_end ? TILE_LAST : 0);
        if (lane == 0) {
          TileMeta m;
          m.seq = seq; m.kvh = kvh; m.split = split; m.nsplits = nsplits;
          m.n_valid = n_valid;
          m.flags = flags;
          m.pad0 = m.pad1 = 0;
          metas[stage] = m;
          uint32_t bytes = (uint32_t)ncopy * 4u * (uint32_t)st * 128u;
          if (flags & TILE_FIRST) bytes += (uint32_t)p.g * ATT_D * 2u;
          mbar_arrive_expect_tx(&full[stage], bytes);
          if (flags & TILE_FIRST) {
            bulk_load(qslots + stage * ATT_QSLOT_BYTES,
                      p.q + (int64_t)seq * p.q_stride + (int64_t)kvh * p.g * ATT_D,
                      (uint32_t)p.g * ATT_D * 2u, &full[stage]);
          }
        }
        __syncwarp();
        if (lane < ncopy) {
          uint8_t* kdst = stages + stage * ATT_STAGE_BYTES;
          uint8_t* vdst = kdst + ATT_KV_BYTES;
          const int t = tok0 + my;
          int page = pg;
          const int off = off_of(t);
          if (page < 0 || page >= p.num_blocks) {
            // out-of-range page: the copy reads the zero fill, nothing faults
            page = p.num_blocks;
            if (p.status) atomicOr(p.status, FK_DEV_BAD_PAGE);
          }
          if (p.fused16) {
            // 16-token pages: the map's dims are (64 dims, token, dim half, head,
            // page), so one copy lands as [dim half][16 tokens][128 B] = 4 KiB, the
            // slab of consumer warp `lane`
            const int dsto = lane * 4096;
            tma_load_5d(kdst + dsto, &tmap_k, &full[stage], 0, off, 0, kvh, page);
            tma_load_5d(vdst + dsto, &tmap_v, &full[stage], 0, off, 0, kvh, page);
          } else {
            // destination: 64-token box b, rows [r0, r0 + st) of that box
            const int b = my / ATT_BOX, r0 = my % ATT_BOX;
            const int c1 = p.hnd ? off : kvh, c2 = p.hnd ? kvh : off;
#pragma unroll
            for (int dh = 0; dh < 2; ++dh) {
              const int dsto = (b * 2 + dh) * ATT_BOX_BYTES + r0 * 128;
              tma_load_4d(kdst + dsto, &tmap_k, &full[stage], dh * 64, c1, c2, page);
              tma_load_4d(vdst + dsto, &tmap_v, &full[stage], dh * 64, c1, c2, page);
            }
          }
        }
        const int tn = tok0 + ATT_TILE + my;  // this lane's piece of the next tile
        if (my < ATT_TILE && tn < tok_end) pg = bt[page_of(tn)];
        if (++stage == ATT_STAGES) { stage = 0; phase ^= 1; }
      }
    }
    // end marker (also sent after a timeout so the consumers stop)
    if (lane == 0) {
      if (att_wait(&empty[stage], phase ^ 1, abort_flag, p.status)) {
        TileMeta m{};
        m.flags = TILE_END;
        metas[stage] = m;
        mbar_arrive(&full[stage]);
      }
    }
    return;
  }

  // ========================== consumer warps ===============================
  const int w = warp;               // 0..7
  const int quad = lane & 3, row = lane >> 2;
  // Where this warp's 16-token slab sits inside the K (or V) region of a stage, and
  // how far apart its two 64-dim halves are: [box][dim half][64 tokens][128 B] for
  // 64-token copies, [slab][dim half][16 tokens][128 B] for the fused page-16 copies.
  const int slab_off = p.fused16 ? w * 4096 : (w >> 2) * 2 * ATT_BOX_BYTES + (w & 3) * 16 * 128;
  const int dh_stride = p.fused16 ? 2048 : ATT_BOX_BYTES;

  uint32_t qf[8][4];
  float o[16][4];
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) qf[i][0] = qf[i][1] = qf[i][2] = qf[i][3] = 0u;

  int stage = 0;
  uint32_t phase = 0;
  for (;;) {
    if (!att_wait(&full[stage], phase, abort_flag, p.status)) break;
    const TileMeta meta = metas[stage];
    if (meta.flags & TILE_END) break;

    if (meta.flags & TILE_FIRST) {
      const uint32_t* qs =
          reinterpret_cast<const uint32_t*>(qslots + stage * ATT_QSLOT_BYTES);
      const bool r0 = row < p.g, r1 = G16 && (row + 8 < p.g);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const int col = ks * 8 + quad;  // uint32 index inside the 64-word row
        qf[ks][0] = r0 ? qs[row * 64 + col] : 0u;
        qf[ks][1] = r1 ? qs[(row + 8) * 64 + col] : 0u;
        qf[ks][2] = r0 ? qs[row * 64 + col + 4] : 0u;
        qf[ks][3] = r1 ? qs[(row + 8) * 64 + col + 4] : 0u;
      }
      m_run[0] = m_run[1] = -INFINITY;
      l_run[0] = l_run[1] = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    }

    const int nv = min(16, meta.n_valid - w * 16);  // valid tokens in my slab
    if (nv > 0) {
      const uint32_t kbase = smem_u32(stages + stage * ATT_STAGE_BYTES) + slab_off;
      const uint32_t vbase = kbase + ATT_KV_BYTES;
      bool wrote = false;
      if (nv < 16) {
        // rows past the context end hold whatever the pool had there: clear
        // the V rows (P = 0 there, but 0 * NaN would poison the sum)
        uint8_t* vgen = stages + stage * ATT_STAGE_BYTES + ATT_KV_BYTES + slab_off;
        for (int idx = lane; idx < 16 * 16; idx += 32) {
          const int t = idx >> 4, c = idx & 15;  // row in slab, 16-byte chunk
          if (t >= nv) {
            *reinterpret_cast<uint4*>(vgen + (c >> 3) * dh_stride + t * 128 +
                                      (c & 7) * 16) = make_uint4(0, 0, 0, 0);
          }
        }
        wrote = true;
        __syncwarp();
      }

      // ---- S = Q K^T (16 x 16 per warp) ----
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      {
        const int j = lane >> 3, r = lane & 7;
        const int tb = (j >> 1) * 8 + r;          // row inside the slab
        const uint32_t rowaddr = kbase + tb * 128;
        const int sw = tb & 7;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const int c = ks * 2 + (j & 1);
          const uint32_t addr = rowaddr + (c >> 3) * dh_stride +
                                (((c & 7) ^ sw) << 4);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(addr, b0, b1, b2, b3);
          mma_bf16_16816(s[0], qf[ks], b0, b1);
          mma_bf16_16816(s[1], qf[ks], b2, b3);
        }
      }

      // ---- online softmax (base 2), state per row in registers ----
      float t[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = nt * 8 + quad * 2 + (e & 1);
          t[nt][e] = col < nv ? s[nt][e] * p.scale_log2 : -INFINITY;
        }
      float pa_f[2][4];
#pragma unroll
      for (int h = 0; h < (G16 ? 2 : 1); ++h) {
        float mx = fmaxf(fmaxf(t[0][2 * h], t[0][2 * h + 1]),
                         fmaxf(t[1][2 * h], t[1][2 * h + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[h], mx);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        const float alpha = fast_exp2(m_run[h] - m_use);
        m_run[h] = m_new;
        float ls = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float pv = fast_exp2(t[nt][2 * h + e] - m_use);
            pa_f[nt][2 * h + e] = pv;
            ls += pv;
          }
        l_run[h] = l_run[h] * alpha + ls;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          o[i][2 * h] *= alpha;
          o[i][2 * h + 1] *= alpha;
        }
      }
      uint32_t pa[4];
      pa[0] = pack_bf16(pa_f[0][0], pa_f[0][1]);
      pa[2] = pack_bf16(pa_f[1][0], pa_f[1][1]);
      if (G16) {
        pa[1] = pack_bf16(pa_f[0][2], pa_f[0][3]);
        pa[3] = pack_bf16(pa_f[1][2], pa_f[1][3]);
      } else {
        pa[1] = 0u;
        pa[3] = 0u;
      }

      // ---- O += P V (16 x 128 per warp) ----
      {
        const int j = lane >> 3, r = lane & 7;
        const int tb = (j & 1) * 8 + r;           // row inside the slab
        const uint32_t rowaddr = vbase + tb * 128;
        const int sw = tb & 7;
#pragma unroll
        for (int pr = 0; pr < 8; ++pr) {
          const int c = pr * 2 + (j >> 1);
          const uint32_t addr = rowaddr + (c >> 3) * dh_stride +
                                (((c & 7) ^ sw) << 4);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(addr, b0, b1, b2, b3);
          mma_bf16_16816(o[2 * pr], pa, b0, b1);
          mma_bf16_16816(o[2 * pr + 1], pa, b2, b3);
        }
      }
      if (wrote) fence_proxy_async_smem();
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[stage]);

    if (meta.flags & TILE_LAST) {
      // ------------- merge the 8 warps' partial states, write out ----------
      float lsum[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float v = l_run[h];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        lsum[h] = v;
      }
      if (quad == 0) {
        ml[w * 16 + row] = make_float2(m_run[0], lsum[0]);
        ml[w * 16 + row + 8] = make_float2(m_run[1], lsum[1]);
      }
      named_bar_sync(1, ATT_NW * 32);
      float m_all[2] = {-INFINITY, -INFINITY}, l_all[2] = {0.f, 0.f};
#pragma unroll
      for (int ww = 0; ww < ATT_NW; ++ww) {
        m_all[0] = fmaxf(m_all[0], ml[ww * 16 + row].x);
        m_all[1] = fmaxf(m_all[1], ml[ww * 16 + row + 8].x);
      }
      float mu[2];
      mu[0] = m_all[0] == -INFINITY ? 0.f : m_all[0];
      mu[1] = m_all[1] == -INFINITY ? 0.f : m_all[1];
#pragma unroll
      for (int ww = 0; ww < ATT_NW; ++ww) {
        const float2 a = ml[ww * 16 + row], b = ml[ww * 16 + row + 8];
        l_all[0] += a.y * fast_exp2(a.x - mu[0]);
        l_all[1] += b.y * fast_exp2(b.x - mu[1]);
      }
      const float f0 = fast_exp2(m_run[0] - mu[0]);
      const float f1 = fast_exp2(m_run[1] - mu[1]);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        o[i][0] *= f0; o[i][1] *= f0;
        o[i][2] *= f1; o[i][3] *= f1;
      }
      // tree sum through two 8 KiB buffers: (4,5)->(0,1), (6,7)->(2,3),
      // (2,3)->(0,1), 1->0
      auto send = [&](int buf) {
        float4* b = mbuf + buf * (ATT_MBUF_BYTES / 16);
#pragma unroll
        for (int i = 0; i < 16; ++i)
          b[i * 32 + lane] = make_float4(o[i][0], o[i][1], o[i][2], o[i][3]);
      };
      auto recv = [&](int buf) {
        const float4* b = mbuf + buf * (ATT_MBUF_BYTES / 16);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float4 v = b[i * 32 + lane];
          o[i][0] += v.x; o[i][1] += v.y; o[i][2] += v.z; o[i][3] += v.w;
        }
      };
      if (w == 4 || w == 5) send(w - 4);
      named_bar_sync(1, ATT_NW * 32);
      if (w == 0 || w == 1) recv(w);
      named_bar_sync(1, ATT_NW * 32);
      if (w == 6 || w == 7) send(w - 6);
      named_bar_sync(1, ATT_NW * 32);
      if (w == 2 || w == 3) recv(w - 2);
      named_bar_sync(1, ATT_NW * 32);
      if (w == 2 || w == 3) send(w - 2);
      named_bar_sync(1, ATT_NW * 32);
      if (w == 0 || w == 1) recv(w);
      named_bar_sync(1, ATT_NW * 32);
      if (w == 1) send(0);
      named_bar_sync(1, ATT_NW * 32);
      if (w == 0) {
        recv(0);
#pragma unroll
        for (int h = 0; h < (G16 ? 2 : 1); ++h) {
          const int r = row + 8 * h;
          if (r < p.g) {
            const int head = meta.kvh * p.g + r;
            if (meta.nsplits == 1) {
              const float inv = l_all[h] > 0.f ? 1.0f / l_all[h] : 0.f;
              uint32_t* dst = reinterpret_cast<uint32_t*>(
                  p.out + (int64_t)meta.seq * p.out_stride + (int64_t)head * ATT_D);
#pragma unroll
              for (int i = 0; i < 16; ++i)
                dst[i * 4 + quad] =
                    pack_bf16(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
            } else {
              const int64_t pi =
                  ((int64_t)meta.seq * p.hq + head) * p.max_splits + meta.split;
              float2* dst = reinterpret_cast<float2*>(p.part_o + pi * ATT_D);
#pragma unroll
              for (int i = 0; i < 16; ++i)
                dst[i * 4 + quad] = make_float2(o[i][2 * h], o[i][2 * h + 1]);
              if (quad == 0) p.part_ml[pi] = make_float2(m_all[h], l_all[h]);
            }
          }
        }
      }
    }
    if (++stage == ATT_STAGES) { stage = 0; phase ^= 1; }
  }
}

// ---------------------------------------------------------------------------
// merge of split partials: out = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M)
// (same rule as the reference's segment reduction,
// fastkernels/tasks/baseline/L1/triton_unified_attention.py:697-786:
// empty total -> zeros)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) attn_merge_kernel(const AttnParams p) {
  pdl_launch_dependents();
  pdl_wait();
  // the main kernel is done: clear its work counter so the same plan can serve
  // the next layer of the step without re-running the plan kernel
  if (blockIdx.x == 0 && threadIdx.x == 0) p.plan[2] = 0;
  const int gw = (int)((blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31;
  if (gw >= p.batch * p.hq) return;
  const int seq = gw / p.hq, head = gw - seq * p.hq;
  const int* chunk_start = p.plan + ATT_PLAN_HDR;
  const int n = chunk_start[seq + 1] - chunk_start[seq];
  if (n == 1) return;  // written directly by the main kernel
  uint2* dst = reinterpret_cast<uint2*>(p.out + (int64_t)seq * p.out_stride +
                                        (int64_t)head * ATT_D) + lane;
  if (n == 0) {
    *dst = make_uint2(0u, 0u);
    return;
  }
  const int64_t base = ((int64_t)seq * p.hq + head) * p.max_splits;
  float M = -INFINITY;
  for (int s = 0; s < n; ++s) M = fmaxf(M, p.part_ml[base + s].x);
  const float Mu = M == -INFINITY ? 0.f : M;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float lt = 0.f;
  for (int s = 0; s < n; ++s) {
    const float2 mlv = p.part_ml[base + s];
    const float f = fast_exp2(mlv.x - Mu);
    lt += mlv.y * f;
    const float4 v =
        reinterpret_cast<const float4*>(p.part_o + (base + s) * ATT_D)[lane];
    acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
  }
  const float inv = lt > 0.f ? 1.0f / lt : 0.f;
  *dst = make_uint2(pack_bf16(acc.x * inv, acc.y * inv),
                    pack_bf16(acc.z * inv, acc.w * inv));
}

// ---------------------------------------------------------------------------
// host: tensor-map cache
// ---------------------------------------------------------------------------
struct MapKey {
  const void* ptr; int64_t num_blocks; int block_size; int hkv; int64_t stride; int hnd;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && num_blocks == o.num_blocks &&
           block_size == o.block_size && hkv == o.hkv && stride == o.stride &&
           hnd == o.hnd;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    h ^= std::hash<int64_t>()(k.num_blocks * 1315423911ll + k.block_size * 2654435761ll +
                              k.hkv * 97ll + k.stride + k.hnd * 7919ll);
    return h;
  }
};
static std::mutex g_map_mu;
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

static int get_kv_map(const void* cache, int64_t num_blocks, int block_size,
                      int hkv, int64_t block_stride, int hnd, int fused,
                      CUtensorMap* out) {
  MapKey key{cache, num_blocks, block_size, hkv, block_stride, hnd + 2 * fused};
  std::lock_guard<std::mutex> lk(g_map_mu);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return FK_OK;
  }
  tensormap_encode_fn enc = get_tensormap_encode();
  FK_REQUIRE(enc != nullptr, FK_ERR_CUDA,
             "cuTensorMapEncodeTiled not available from the driver");
  // One copy = `sub` tokens x 64 dims of one KV head inside one page.
  //   NHD pool [blocks, block, Hkv, D]: dims (D, Hkv, token, block)
  //   HND pool [blocks, Hkv, block, D]: dims (D, token, Hkv, block)
  const cuuint32_t sub = (cuuint32_t)(block_size < ATT_BOX ? block_size : ATT_BOX);
  cuuint64_t dims[4], strides[3];
  cuuint32_t box[4];
  dims[0] = ATT_D; dims[3] = (cuuint64_t)num_blocks;
  strides[2] = (cuuint64_t)block_stride * 2;
  box[0] = 64; box[3] = 1;
  if (hnd) {
    dims[1] = (cuuint64_t)block_size; dims[2] = (cuuint64_t)hkv;
    strides[0] = (cuuint64_t)ATT_D * 2;
    strides[1] = (cuuint64_t)block_size * ATT_D * 2;
    box[1] = sub; box[2] = 1;
  } else {
    dims[1] = (cuuint64_t)hkv; dims[2] = (cuuint64_t)block_size;
    strides[0] = (cuuint64_t)ATT_D * 2;
    strides[1] = (cuuint64_t)hkv * ATT_D * 2;
    box[1] = 1; box[2] = sub;
  }
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUtensorMap m;
  CUresult r;
  if (fused) {
    // Pages of fewer than 64 tokens: the two 64-dim halves of a head become a
    // dimension of their own, (64 dims, token, dim half, head, page), so that one
    // copy of box (64, page tokens, 2, 1, 1) lands as [dim half][token][128 B].
    const cuuint64_t tok_stride = hnd ? (cuuint64_t)ATT_D * 2 : (cuuint64_t)hkv * ATT_D * 2;
    const cuuint64_t head_stride =
        hnd ? (cuuint64_t)block_size * ATT_D * 2 : (cuuint64_t)ATT_D * 2;
    cuuint64_t d5[5] = {64, (cuuint64_t)block_size, 2, (cuuint64_t)hkv, (cuuint64_t)num_blocks};
    cuuint64_t s5[4] = {tok_stride, 128, head_stride, (cuuint64_t)block_stride * 2};
    cuuint32_t b5[5] = {64, (cuuint32_t)block_size, 2, 1, 1};
    r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(cache), d5, s5, b5,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(cache), dims,
            strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  FK_REQUIRE(r == CUDA_SUCCESS, FK_ERR_CUDA,
             "cuTensorMapEncodeTiled failed with code %d", (int)r);
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps.emplace(key, m);
  *out = m;
  return FK_OK;
}

static size_t plan_hdr_bytes(int batch) {
  size_t b = (size_t)(ATT_PLAN_HDR + batch + 1) * sizeof(int);
  return (b + 255) & ~size_t(255);
}
static size_t plan_bytes(int batch, int max_splits) {
  size_t b = plan_hdr_bytes(batch) + (size_t)batch * max_splits * sizeof(int4);
  return (b + 255) & ~size_t(255);
}

}  // namespace fk

using namespace fk;

extern "C" {

size_t fk_paged_decode_attn_workspace_bytes(int batch, int num_q_heads,
                                            int head_dim, int max_splits) {
  if (batch <= 0 || num_q_heads <= 0 || head_dim <= 0 || max_splits <= 0)
    return 0;
  const size_t parts = (size_t)batch * num_q_heads * max_splits;
  return plan_bytes(batch, max_splits) + parts * head_dim * sizeof(float) +
         parts * sizeof(float2);
}

static int attn_impl(int mode, const void* q, int64_t q_stride_token, void* out,
                         int64_t out_stride_token, const void* k_cache,
                         const void* v_cache, int64_t num_blocks,
                         int block_size, int64_t kv_block_stride, int kv_layout,
                         const int32_t* context_lens,
                         const int32_t* block_tables,
                         int64_t block_table_stride, int batch,
                         int num_q_heads, int num_kv_heads, int head_dim,
                         float softmax_scale, int max_splits, void* workspace,
                         size_t workspace_bytes, int32_t* status,
                         fk_stream_t stream) {
  FK_REQUIRE(batch >= 0, FK_ERR_INVALID_ARG, "fk_paged_decode_attn: batch < 0");
  if (batch == 0) return FK_OK;
  FK_REQUIRE(context_lens && block_tables, FK_ERR_INVALID_ARG,
             "fk_paged_decode_attn: null pointer");
  FK_REQUIRE(mode == 1 || (q && out && k_cache && v_cache), FK_ERR_INVALID_ARG,
             "fk_paged_decode_attn: null pointer");
  FK_REQUIRE(head_dim == ATT_D, FK_ERR_UNSUPPORTED,
             "fk_paged_decode_attn: head_dim %d unsupported (128 only)", head_dim);
  FK_REQUIRE(num_q_heads > 0 && num_kv_heads > 0 &&
                 num_q_heads % num_kv_heads == 0,
             FK_ERR_INVALID_ARG,
             "fk_paged_decode_attn: num_q_heads must be a multiple of num_kv_heads");
  const int g = num_q_heads / num_kv_heads;
  FK_REQUIRE(g == 1 || g == 2 || g == 4 || g == 8 || g == 16, FK_ERR_UNSUPPORTED,
             "fk_paged_decode_attn: GQA ratio %d unsupported (1,2,4,8,16)", g);
  FK_REQUIRE(block_size == 16 || block_size == 32 ||
                 (block_size >= ATT_BOX && block_size % ATT_BOX == 0),
             FK_ERR_UNSUPPORTED,
             "fk_paged_decode_attn: block_size %d must be 16, 32 or a multiple of 64",
             block_size);
  FK_REQUIRE(kv_layout == 0 || kv_layout == 1, FK_ERR_INVALID_ARG,
             "fk_paged_decode_attn: kv_layout must be 0 (NHD) or 1 (HND)");
  FK_REQUIRE(num_blocks > 0 && num_blocks < (1ll << 31) && max_splits > 0 &&
                 block_table_stride > 0,
             FK_ERR_INVALID_ARG, "fk_paged_decode_attn: bad sizes");
  FK_REQUIRE(kv_block_stride >= (int64_t)block_size * num_kv_heads * head_dim,
             FK_ERR_INVALID_ARG, "fk_paged_decode_attn: kv_block_stride too small");
  FK_REQUIRE(aligned16(q) && aligned16(out) && aligned16(k_cache) &&
                 aligned16(v_cache) && q_stride_token % 8 == 0 &&
                 out_stride_token % 8 == 0 && kv_block_stride % 8 == 0,
             FK_ERR_ALIGNMENT,
             "fk_paged_decode_attn: 16-byte alignment required");
  FK_REQUIRE(q_stride_token >= (int64_t)num_q_heads * head_dim &&
                 out_stride_token >= (int64_t)num_q_heads * head_dim,
             FK_ERR_INVALID_ARG, "fk_paged_decode_attn: token stride too small");
  const size_t need = fk_paged_decode_attn_workspace_bytes(batch, num_q_heads,
                                                           head_dim, max_splits);
  FK_REQUIRE(workspace != nullptr && workspace_bytes >= need &&
                 (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0,
             FK_ERR_WORKSPACE,
             "fk_paged_decode_attn: workspace needs %zu bytes, 256-byte aligned "
             "(got %zu)",
             need, workspace_bytes);

  CUtensorMap mk, mv;
  // 16-token pages: one copy per page and pool instead of one per 64-dim half (32
  // copies per 128-token tile held the kernel at 0.74 of the HBM peak).  If the
  // driver refuses the 5-D map, the per-half copies are used.
  int fused16 = block_size == 16 ? 1 : 0;
  if (mode != 1) {
    int rc = FK_OK;
    if (fused16) {
      rc = get_kv_map(k_cache, num_blocks, block_size, num_kv_heads, kv_block_stride,
                      kv_layout, 1, &mk);
      if (rc == FK_OK)
        rc = get_kv_map(v_cache, num_blocks, block_size, num_kv_heads, kv_block_stride,
                        kv_layout, 1, &mv);
      if (rc != FK_OK) fused16 = 0;
    }
    if (!fused16) {
      rc = get_kv_map(k_cache, num_blocks, block_size, num_kv_heads, kv_block_stride,
                      kv_layout, 0, &mk);
      if (rc != FK_OK) return rc;
      rc = get_kv_map(v_cache, num_blocks, block_size, num_kv_heads, kv_block_stride,
                      kv_layout, 0, &mv);
      if (rc != FK_OK) return rc;
    }
  }

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  AttnParams p{};
  p.q = (const uint16_t*)q; p.q_stride = q_stride_token;
  p.out = (uint16_t*)out; p.out_stride = out_stride_token;
  p.context_lens = context_lens;
  p.block_tables = block_tables; p.bt_stride = block_table_stride;
  p.batch = batch; p.hq = num_q_heads; p.hkv = num_kv_heads; p.g = g;
  p.block_size = block_size; p.num_blocks = (int)num_blocks;
  p.sub_tokens = block_size < ATT_BOX ? block_size : ATT_BOX;
  p.fused16 = fused16;
  p.hnd = kv_layout;
  p.bs_shift = -1;
  for (int sh = 0; sh < 31; ++sh)
    if ((1 << sh) == block_size) p.bs_shift = sh;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.max_splits = max_splits;
  // A small self-planning call (every (sequence, KV head) pair gets its own CTA and
  // no sequence is long enough to need splitting for bandwidth) runs as ONE launch:
  // no plan kernel, no partials, no merge.
  const bool direct = mode == 0 && (int64_t)batch * num_kv_heads <= sm_count() &&
                      block_table_stride * (int64_t)block_size <= 2048;
  p.direct = direct ? 1 : 0;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  p.plan = reinterpret_cast<int*>(ws);
  const size_t parts = (size_t)batch * num_q_heads * max_splits;
  p.chunk_info = reinterpret_cast<int4*>(ws + plan_hdr_bytes(batch));
  p.part_o = reinterpret_cast<float*>(ws + plan_bytes(batch, max_splits));
  p.part_ml = reinterpret_cast<float2*>(ws + plan_bytes(batch, max_splits) +
                                        parts * head_dim * sizeof(float));
  p.status = status;

  const int grid = sm_count();
  static PerDeviceOnce attr_nhd, attr_hnd;
  FK_CUDA_OK(set_max_dynamic_smem(attr_nhd, attn_decode_kernel<false>, AttnSmem::kAlloc));
  FK_CUDA_OK(set_max_dynamic_smem(attr_hnd, attn_decode_kernel<true>, AttnSmem::kAlloc));

  if (direct) {
    const int dgrid = batch * num_kv_heads;
    if (g > 8)
      FK_LAUNCH(attn_decode_kernel<true>, dim3(dgrid), dim3(ATT_THREADS),
                (size_t)AttnSmem::kAlloc, s, mk, mv, p);
    else
      FK_LAUNCH(attn_decode_kernel<false>, dim3(dgrid), dim3(ATT_THREADS),
                (size_t)AttnSmem::kAlloc, s, mk, mv, p);
    count_launch(1);
    FK_CUDA_OK(cudaGetLastError());
    return FK_OK;
  }
  if (mode != 2) {
    FK_LAUNCH(attn_plan_kernel, dim3(1), dim3(1024), 0, s, context_lens, batch,
              num_kv_heads, max_splits, grid, block_table_stride * (int64_t)block_size,
              p.plan, p.chunk_info, status);
    count_launch(1);
  }
  if (mode == 1) {
    FK_CUDA_OK(cudaGetLastError());
    return FK_OK;
  }
  if (g > 8)
    FK_LAUNCH(attn_decode_kernel<true>, dim3(grid), dim3(ATT_THREADS),
              (size_t)AttnSmem::kAlloc, s, mk, mv, p);
  else
    FK_LAUNCH(attn_decode_kernel<false>, dim3(grid), dim3(ATT_THREADS),
              (size_t)AttnSmem::kAlloc, s, mk, mv, p);
  const int warps = batch * num_q_heads;
  FK_LAUNCH(attn_merge_kernel, dim3((warps * 32 + 255) / 256), dim3(256), 0, s, p);
  count_launch(2);
  FK_CUDA_OK(cudaGetLastError());
  return FK_OK;
}

int fk_paged_decode_attn(const void* q, int64_t q_stride_token, void* out,
                         int64_t out_stride_token, const void* k_cache,
                         const void* v_cache, int64_t num_blocks,
                         int block_size, int64_t kv_block_stride, int kv_layout,
                         const int32_t* context_lens,
                         const int32_t* block_tables,
                         int64_t block_table_stride, int batch,
                         int num_q_heads, int num_kv_heads, int head_dim,
                         float softmax_scale, int max_splits, void* workspace,
                         size_t workspace_bytes, int32_t* status,
                         fk_stream_t stream) {
  return attn_impl(0, q, q_stride_token, out, out_stride_token, k_cache, v_cache,
                   num_blocks, block_size, kv_block_stride, kv_layout, context_lens,
                   block_tables,
                   block_table_stride, batch, num_q_heads, num_kv_heads, head_dim,
                   softmax_scale, max_splits, workspace, workspace_bytes, status, stream);
}

int fk_paged_decode_attn_plan(const int32_t* context_lens,
                              const int32_t* block_tables,
                              int64_t block_table_stride, int block_size, int batch,
                              int num_q_heads, int num_kv_heads, int head_dim,
                              int max_splits, void* workspace,
                              size_t workspace_bytes, int32_t* status,
                              fk_stream_t stream) {
  return attn_impl(1, nullptr, (int64_t)num_q_heads * head_dim, nullptr,
                   (int64_t)num_q_heads * head_dim, nullptr, nullptr, 1, block_size,
                   (int64_t)block_size * num_kv_heads * head_dim, 0, context_lens,
                   block_tables, block_table_stride, batch, num_q_heads, num_kv_heads,
                   head_dim, 1.0f, max_splits, workspace, workspace_bytes, status, stream);
}

int fk_paged_decode_attn_planned(const void* q, int64_t q_stride_token, void* out,
                                 int64_t out_stride_token, const void* k_cache,
                                 const void* v_cache, int64_t num_blocks,
                                 int block_size, int64_t kv_block_stride,
                                 int kv_layout,
                                 const int32_t* context_lens,
                                 const int32_t* block_tables,
                                 int64_t block_table_stride, int batch,
                                 int num_q_heads, int num_kv_heads, int head_dim,
                                 float softmax_scale, int max_splits,
                                 void* workspace, size_t workspace_bytes,
                                 int32_t* status, fk_stream_t stream) {
  return attn_impl(2, q, q_stride_token, out, out_stride_token, k_cache, v_cache,
                   num_blocks, block_size, kv_block_stride, kv_layout, context_lens,
                   block_tables,
                   block_table_stride, batch, num_q_heads, num_kv_heads, head_dim,
                   softmax_scale, max_splits, workspace, workspace_bytes, status, stream);
}

}  // extern "C"
