// Projections y = x W^T (+ bias) for MANY rows (prefill: m in the hundreds or
// thousands), the compute-bound sibling of the weight-streaming decode kernel.
// Same interface: Matmul.forward (fastkernels/tasks/baseline/L1/linear.py:13-17)
// and the F.linear calls of the TP linear layers
// (fastkernels/tasks/baseline/L2/parallel_linear.py:78-81,157-160,237-240,327-335).
//
// With m >> 256 both operands are re-read many times, from L2: a CTA tile of
// TM x TN outputs costs (1/TM + 1/TN) operand bytes per 2 FLOP.  The tile is
// therefore 256 tokens x 256 weight rows -- two 128-lane accumulators of 256 fp32
// columns, all 512 columns of tensor memory -- which is the largest one CTA can
// hold and halves the traffic of a 128 x 256 tile:
//   MMA M (128 TMEM lanes)  <- 128 token rows of x (two halves per tile)
//   MMA N (256 columns)     <- 256 rows of W
//   MMA K (16 per instr.)   <- 64-element k-blocks = one 128-byte swizzle row
// Persistent CTAs (one per SM) take tiles round-robin with the token dimension
// fastest, so the CTAs running together share a few weight tiles in L2.
//
// Warp roles (192 threads): warp 0 = TMA producer (three 64 KiB stages),
// warp 1 = MMA issuer (converged warp, one elected lane) and TMEM owner,
// warps 2..5 = epilogue (TMEM lanes 32*(warp%4)..+31 = token rows; fp32 + bias
// -> bf16 -> 16-byte stores).  The accumulators are single-buffered: the MMAs of
// the next tile wait until the epilogue has read the previous one out, while the
// producer already fills the ring for it.  Waits are bounded (2 s).
#include "fk_common.cuh"
#include "fk_tcgen05.cuh"

#include <cstdlib>
#include <mutex>
#include <unordered_map>

namespace fk {

constexpr int GL_BM = 256;
constexpr int GL_BN = 256;
constexpr int GL_BK = 64;
constexpr int GL_STAGES = 3;
constexpr int GL_A_BYTES = GL_BM * GL_BK * 2;        // 32 KiB
constexpr int GL_B_BYTES = GL_BN * GL_BK * 2;        // 32 KiB
constexpr int GL_STAGE_BYTES = GL_A_BYTES + GL_B_BYTES;
constexpr int GL_OFF_BAR = GL_STAGES * GL_STAGE_BYTES;
constexpr int GL_SMEM = GL_OFF_BAR + 128;
constexpr int GL_SMEM_ALLOC = GL_SMEM + 1024;
constexpr int GL_THREADS = 192;
constexpr int GL_TMEM_COLS = 512;
static_assert(GL_SMEM_ALLOC <= 232448, "shared memory budget");

struct GemmLargeParams {
  const uint16_t* bias;   // [n] or null
  uint16_t* y; int64_t y_stride;
  int m, n, k;
  int m_tiles, n_tiles;
  int32_t* status;
};

__device__ __forceinline__ uint64_t gl_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool gl_wait(uint64_t* bar, uint32_t parity,
                                        volatile int* abort_flag, int32_t* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = gl_ns();
  for (;;) {
    for (int i = 0; i < 128; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (gl_ns() - t0 > 2000000000ull) {
      *abort_flag = 1;
      if (status) atomicOr(status, FK_DEV_WAIT_TIMEOUT);
      return false;
    }
  }
}
__device__ __forceinline__ bool gl_wait_warp(uint64_t* bar, uint32_t parity,
                                             volatile int* abort_flag, int32_t* status) {
  return __all_sync(0xffffffffu, gl_wait(bar, parity, abort_flag, status) ? 1 : 0) != 0;
}

__global__ void __launch_bounds__(GL_THREADS, 1)
gemm_large_kernel(const __grid_constant__ CUtensorMap tmap_x,
                  const __grid_constant__ CUtensorMap tmap_w, const GemmLargeParams p) {
  extern __shared__ uint8_t gl_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(gl_smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GL_OFF_BAR);
  uint64_t* full = bars;                       // [GL_STAGES]
  uint64_t* empty = bars + GL_STAGES;          // [GL_STAGES]
  uint64_t* acc_full = bars + 2 * GL_STAGES;   // accumulators of a tile complete
  uint64_t* acc_empty = acc_full + 1;          // ... and read out by the epilogue
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_tiles = p.m_tiles * p.n_tiles;
  const int kb_total = p.k / GL_BK;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int i = 0; i < GL_STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 4);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) tmem_alloc(tmem_slot, GL_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // all 512 columns are taken, so the allocation can only start at column 0
  const uint32_t tmem_got = *tmem_slot;
  constexpr uint32_t tmem_base = 0;
  if (tmem_got != 0) {
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, FK_DEV_TMEM_BASE);
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_got, GL_TMEM_COLS);
    return;
  }
  pdl_wait();   // x (and bias, y) may come from earlier kernels

  if (warp == 0) {
    // ------------------------------ TMA producer ---------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int ti = blockIdx.x; ti < total_tiles && ok; ti += gridDim.x) {
        const int mt = ti % p.m_tiles, nt = ti / p.m_tiles;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!gl_wait(&empty[stage], phase ^ 1, abort_flag, p.status)) { ok = false; break; }
          uint8_t* dst = smem + stage * GL_STAGE_BYTES;
          mbar_arrive_expect_tx(&full[stage], (uint32_t)GL_STAGE_BYTES);
          tma_load_2d(dst, &tmap_x, &full[stage], kb * GL_BK, mt * GL_BM);
          tma_load_2d(dst + GL_A_BYTES, &tmap_w, &full[stage], kb * GL_BK, nt * GL_BN);
          if (++stage == GL_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ----------------------------
    constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                               ((uint32_t)(GL_BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    int stage = 0;
    uint32_t phase = 0;
    uint32_t tiles_done = 0;
    bool ok = true;
    for (int ti = blockIdx.x; ti < total_tiles && ok; ti += gridDim.x) {
      // the epilogue must have read the previous tile out of tensor memory
      if (tiles_done > 0)
        ok = gl_wait_warp(acc_empty, (tiles_done - 1) & 1u, abort_flag, p.status);
      if (!ok) break;
      tc_fence_after();
      for (int kb = 0; kb < kb_total; ++kb) {
        ok = gl_wait_warp(&full[stage], phase, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a = smem_u32(smem + stage * GL_STAGE_BYTES);
        const uint32_t b = a + GL_A_BYTES;
        // the two accumulators take turns, so consecutive MMAs are independent
#pragma unroll
        for (int kk = 0; kk < GL_BK / 16; ++kk) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            tc_mma_bf16_elect(tmem_base + h * GL_BN,
                              smem_desc_sw128(a + h * (128 * 128) + kk * 32),
                              smem_desc_sw128(b + kk * 32), idesc,
                              (kb > 0 || kk > 0) ? 1u : 0u);
          }
        }
        tc_commit_elect(&empty[stage]);   // frees the stage when these MMAs retire
        if (++stage == GL_STAGES) { stage = 0; phase ^= 1; }
      }
      if (!ok) break;
      tc_commit_elect(acc_full);
      ++tiles_done;
    }
  } else {
    // -------------------------------- epilogue -----------------------------
    const int q = warp & 3;           // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;    // token row inside a 128-row half
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    uint32_t tiles_done = 0;
    bool ok = true;
    for (int ti = blockIdx.x; ti < total_tiles && ok; ti += gridDim.x) {
      const int mt = ti % p.m_tiles, nt = ti / p.m_tiles;
      if (!gl_wait(acc_full, tiles_done & 1u, abort_flag, p.status)) { ok = false; break; }
      tc_fence_after();
      const int n0 = nt * GL_BN;
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        const int64_t tok = (int64_t)mt * GL_BM + h * 128 + row;
        uint16_t* yrow = p.y + tok * p.y_stride + n0;
#pragma unroll 1
        for (int c = 0; c < GL_BN / 32; ++c) {
          uint32_t v[32];
          tc_ld32(lane_addr + h * GL_BN + c * 32, v);
          tc_wait_ld();
          if (tok < p.m) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int col = n0 + c * 32 + g * 8;
              float b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
              if (p.bias) {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  if (col + i < p.n) b[i] = bf16_bits_to_float(p.bias[col + i]);
              }
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[g * 8 + i]) + b[i];
              if (col + 8 <= p.n) {
                *reinterpret_cast<uint4*>(yrow + c * 32 + g * 8) =
                    make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]),
                               pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
              } else {
                for (int i = 0; i < 8; ++i)
                  if (col + i < p.n)
                    yrow[c * 32 + g * 8 + i] = __bfloat16_as_ushort(__float2bfloat16_rn(f[i]));
              }
            }
          }
        }
      }
      // both accumulators are in registers / memory now
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
      ++tiles_done;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_got, GL_TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// CTA-pair variant: the same 256 x 256 tile, held by TWO CTAs of a cluster.
// CTA r of the pair owns token rows [128 r, 128 r + 128) of the tile (its A
// operand and its TMEM lanes) and stages weight rows [128 r, 128 r + 128) (its
// half of B); one tcgen05.mma.cta_group::2 issued by the even CTA drives both
// tensor cores and feeds each from BOTH halves of B.  Per CTA and 64-wide k-block
// that is 32 KiB written by TMA and 32 KiB read by the MMAs (128 B/clk at full
// rate, against 160 B/clk for the single-CTA tile, which reads its whole weight
// tile twice), six stages instead of three, and two accumulator buffers of 256
// columns, so the epilogue of one tile overlaps the MMAs of the next.
//
// Barriers: full[s] lives in the even CTA and collects the bytes of both CTAs'
// copies; empty[s], acc_full[b] exist in both CTAs and are signalled by a
// multicast tcgen05.commit; acc_empty[b] lives in the even CTA and counts the
// epilogue warps of both.  All waits are bounded; both CTAs always reach the two
// cluster barriers (after set-up, before tear-down).
// ---------------------------------------------------------------------------
// NH = 1: pair tile 256 x 256, two accumulator buffers of 256 columns (the epilogue
//         of a tile overlaps the MMAs of the next), 6 stages of 32 KiB.
// NH = 2: pair tile 256 x 512 = two N halves of 256 columns, one accumulator
//         buffer (all 512 columns), 4 stages of 48 KiB: a quarter fewer operand
//         bytes per FLOP, which is what bounds the kernel (the L2 -> SM path).
template <int NH>
struct G2Cfg {
  static constexpr int kTileN = 256 * NH;
  static constexpr int kABytes = 128 * GL_BK * 2;              // this CTA's token rows
  static constexpr int kBBytes = NH * 128 * GL_BK * 2;         // this CTA's W rows
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (192 * 1024) / kStageBytes;
  static constexpr int kBufs = 2 / NH;                          // accumulator buffers
  static constexpr int kOffBar = kStages * kStageBytes;
  static constexpr int kSmem = kOffBar + 256;
  static constexpr int kAlloc = kSmem + 1024;
  static_assert(kAlloc <= 232448, "shared memory budget");
};

template <int NH>
__global__ void __launch_bounds__(GL_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_x,
                 const __grid_constant__ CUtensorMap tmap_w, const GemmLargeParams p) {
  using Cfg = G2Cfg<NH>;
  extern __shared__ uint8_t gl_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(gl_smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBar);
  uint64_t* full = bars;                         // [kStages]  (used in the even CTA)
  uint64_t* empty = bars + Cfg::kStages;         // [kStages]  (both CTAs)
  uint64_t* acc_full = bars + 2 * Cfg::kStages;  // [2]        (both CTAs)
  uint64_t* acc_empty = acc_full + 2;            // [2]        (used in the even CTA)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(acc_empty + 3);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();       // 0 = even CTA (issues the MMAs)
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int n_tiles = (p.n + Cfg::kTileN - 1) / Cfg::kTileN;
  const int total_tiles = p.m_tiles * n_tiles;
  const int kb_total = p.k / GL_BK;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int i = 0; i < Cfg::kStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);               // 4 epilogue warps of each CTA
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) tmem_alloc2(tmem_slot, GL_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  cluster_barrier_sync();      // the partner's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_got = *tmem_slot;
  constexpr uint32_t tmem_base = 0;              // all 512 columns: starts at column 0
  const bool tmem_ok = tmem_got == 0;
  if (!tmem_ok && threadIdx.x == 0 && p.status) atomicOr(p.status, FK_DEV_TMEM_BASE);
  pdl_wait();   // x (and bias, y) may come from earlier kernels

  if (tmem_ok && warp == 0) {
    // ------------------------------ TMA producer ---------------------------
    if (lane == 0) {
      const uint32_t full0 = cluster_map(smem_u32(&full[0]), 0);   // in the even CTA
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int ti = pair; ti < total_tiles && ok; ti += pairs) {
        const int mt = ti % p.m_tiles, nt = ti / p.m_tiles;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!gl_wait(&empty[stage], phase ^ 1, abort_flag, p.status)) { ok = false; break; }
          uint8_t* dst = smem + stage * Cfg::kStageBytes;
          // the even CTA announces the bytes of both CTAs for this stage
          if (rank == 0) mbar_arrive_expect_tx(&full[stage], 2u * Cfg::kStageBytes);
          const uint32_t bar = full0 + (uint32_t)stage * 8u;
          tma2_load_2d(dst, &tmap_x, bar, kb * GL_BK, mt * GL_BM + (int)rank * 128);
          // N half h of the tile = [this CTA's 128 rows | the partner's 128 rows]
#pragma unroll
          for (int h = 0; h < NH; ++h)
            tma2_load_2d(dst + Cfg::kABytes + h * (128 * GL_BK * 2), &tmap_w, bar, kb * GL_BK,
                         nt * Cfg::kTileN + h * 256 + (int)rank * 128);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (tmem_ok && warp == 1) {
    // ------------------- MMA issuer (even CTA of the pair only) ------------
    if (rank == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                 ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t tiles_done = 0;
      bool ok = true;
      for (int ti = pair; ti < total_tiles && ok; ti += pairs) {
        const uint32_t buf = tiles_done % Cfg::kBufs;
        const uint32_t use = tiles_done / Cfg::kBufs;     // how often this buffer was used
        // both epilogues must have read this buffer's previous tile out
        if (use > 0) ok = gl_wait_warp(&acc_empty[buf], (use - 1) & 1u, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        for (int kb = 0; kb < kb_total; ++kb) {
          ok = gl_wait_warp(&full[stage], phase, abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t b = a + Cfg::kABytes;
#pragma unroll
          for (int kk = 0; kk < GL_BK / 16; ++kk) {
#pragma unroll
            for (int h = 0; h < NH; ++h) {
              tc2_mma_bf16_elect(tmem_base + buf * 256 + h * 256, smem_desc_sw128(a + kk * 32),
                                 smem_desc_sw128(b + h * (128 * GL_BK * 2) + kk * 32), idesc,
                                 (kb > 0 || kk > 0) ? 1u : 0u);
            }
          }
          tc2_commit_elect(&empty[stage]);     // frees the stage in both CTAs
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc2_commit_elect(&acc_full[buf]);      // wakes the epilogues of both CTAs
        ++tiles_done;
      }
    }
  } else if (tmem_ok) {
    // -------------------------------- epilogue -----------------------------
    const int q = warp & 3;           // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;    // token row inside this CTA's 128 rows
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const uint32_t acc_empty0 = cluster_map(smem_u32(&acc_empty[0]), 0);
    uint32_t tiles_done = 0;
    bool ok = true;
    for (int ti = pair; ti < total_tiles && ok; ti += pairs) {
      const int mt = ti % p.m_tiles, nt = ti / p.m_tiles;
      const uint32_t buf = tiles_done % Cfg::kBufs;
      const uint32_t use = tiles_done / Cfg::kBufs;
      if (!gl_wait(&acc_full[buf], use & 1u, abort_flag, p.status)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int n0 = nt * Cfg::kTileN;
      const int64_t tok = (int64_t)mt * GL_BM + (int)rank * 128 + row;
      uint16_t* yrow = p.y + tok * p.y_stride + n0;
#pragma unroll 1
      for (int c = 0; c < Cfg::kTileN / 32; ++c) {
        uint32_t v[32];
        tc_ld32(lane_addr + buf * 256 + c * 32, v);
        tc_wait_ld();
        if (tok < p.m) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int col = n0 + c * 32 + g * 8;
            float b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (p.bias) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                if (col + i < p.n) b[i] = bf16_bits_to_float(p.bias[col + i]);
            }
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[g * 8 + i]) + b[i];
            if (col + 8 <= p.n) {
              *reinterpret_cast<uint4*>(yrow + c * 32 + g * 8) =
                  make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]),
                             pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
            } else {
              for (int i = 0; i < 8; ++i)
                if (col + i < p.n)
                  yrow[c * 32 + g * 8 + i] = __bfloat16_as_ushort(__float2bfloat16_rn(f[i]));
            }
          }
        }
      }
      // this warp's share of the buffer is out of tensor memory
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty0 + buf * 8u);
      ++tiles_done;
    }
  }

  // Nobody leaves while the partner may still read this CTA's shared memory,
  // write its tensor memory or signal its barriers.
  tc_fence_before();
  __syncthreads();
  cluster_barrier_sync();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_got, GL_TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
struct GLKey {
  const void* ptr; int64_t rows, cols, stride; int box_rows;
  bool operator==(const GLKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && stride == o.stride &&
           box_rows == o.box_rows;
  }
};
struct GLHash {
  size_t operator()(const GLKey& k) const {
    return std::hash<const void*>()(k.ptr) ^
           std::hash<int64_t>()(k.rows * 1315423911ll + k.cols * 2654435761ll + k.stride +
                                k.box_rows * 7919ll);
  }
};
static std::mutex g_gl_mu;
static std::unordered_map<GLKey, CUtensorMap, GLHash> g_gl_maps;

// [rows, cols] bf16 with a row stride: box = 64 columns x box_rows rows, 128B swizzle
static int gl_map(const void* ptr, int64_t rows, int64_t cols, int64_t stride, int box_rows,
                  CUtensorMap* out) {
  GLKey key{ptr, rows, cols, stride, box_rows};
  std::lock_guard<std::mutex> lk(g_gl_mu);
  auto it = g_gl_maps.find(key);
  if (it != g_gl_maps.end()) {
    *out = it->second;
    return FK_OK;
  }
  tensormap_encode_fn enc = get_tensormap_encode();
  FK_REQUIRE(enc != nullptr, FK_ERR_CUDA,
             "cuTensorMapEncodeTiled not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)stride * 2};
  cuuint32_t box[2] = {GL_BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims,
                   strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FK_REQUIRE(r == CUDA_SUCCESS, FK_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d",
             (int)r);
  if (g_gl_maps.size() > 4096) g_gl_maps.clear();
  g_gl_maps.emplace(key, m);
  *out = m;
  return FK_OK;
}

constexpr int GL_DEFAULT_PAIR_MODE = 0;

template <int NH>
static int launch_pair(const CUtensorMap& mx, const CUtensorMap& mw, const GemmLargeParams& p,
                       cudaStream_t stream) {
  using Cfg = G2Cfg<NH>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  static int max_pairs = 0;
  static PerDeviceOnce attr_once;
  FK_CUDA_OK(set_max_dynamic_smem(attr_once, gemm_pair_kernel<NH>, Cfg::kAlloc));
  // resident pairs: a property of the GPU model, asked once
  std::call_once(once, [] {
    cudaLaunchConfig_t q{};
    q.gridDim = dim3(2 * (unsigned)sm_count());
    q.blockDim = dim3(GL_THREADS);
    q.dynamicSmemBytes = Cfg::kAlloc;
    cudaLaunchAttribute a[1];
    a[0].id = cudaLaunchAttributeClusterDimension;
    a[0].val.clusterDim.x = 2; a[0].val.clusterDim.y = 1; a[0].val.clusterDim.z = 1;
    q.attrs = a; q.numAttrs = 1;
    int n_cl = 0;
    if (cudaOccupancyMaxActiveClusters(&n_cl, gemm_pair_kernel<NH>, &q) == cudaSuccess)
      max_pairs = n_cl;
  });
  FK_CUDA_OK(attr_err);
  FK_REQUIRE(max_pairs > 0, FK_ERR_CUDA, "fk_gemm_bf16: no CTA pair fits on this device");
  const int64_t tiles = (int64_t)p.m_tiles * ((p.n + Cfg::kTileN - 1) / Cfg::kTileN);
  const int pairs = (int)(tiles < max_pairs ? tiles : max_pairs);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(2u * (unsigned)pairs);
  cfg.blockDim = dim3(GL_THREADS);
  cfg.dynamicSmemBytes = Cfg::kAlloc;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  attr[na].id = cudaLaunchAttributeClusterDimension;
  attr[na].val.clusterDim.x = 2; attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = 1;
  ++na;
  cfg.attrs = attr;
  cfg.numAttrs = na;
  FK_CUDA_OK(cudaLaunchKernelEx(&cfg, gemm_pair_kernel<NH>, mx, mw, p));
  count_launch(1);
  return FK_OK;
}

// Called by fk_gemm_bf16 for m > 256 after its argument checks.
int gemm_large_launch(const void* x, int64_t x_stride, const void* w, const void* bias,
                      void* y, int64_t y_stride, int64_t m, int64_t n, int64_t k,
                      int32_t* status, cudaStream_t stream) {
  FK_REQUIRE(m < (1ll << 31), FK_ERR_UNSUPPORTED, "fk_gemm_bf16: m too large");
  FK_REQUIRE(aligned16(y) && y_stride % 8 == 0, FK_ERR_ALIGNMENT,
             "fk_gemm_bf16: y needs 16-byte aligned rows for m > 256");
  GemmLargeParams p{};
  p.bias = static_cast<const uint16_t*>(bias);
  p.y = static_cast<uint16_t*>(y);
  p.y_stride = y_stride;
  p.m = (int)m; p.n = (int)n; p.k = (int)k;
  p.m_tiles = (int)((m + GL_BM - 1) / GL_BM);
  p.n_tiles = (int)((n + GL_BN - 1) / GL_BN);
  p.status = status;
  const int64_t tiles = (int64_t)p.m_tiles * p.n_tiles;
  FK_REQUIRE(tiles <= 0x7fffffff, FK_ERR_UNSUPPORTED, "fk_gemm_bf16: too many tiles");

  // FK_B200_GEMM_PAIR: 0 = single-CTA tiles, 1 = CTA pairs with 256 x 256 tiles,
  // 2 = CTA pairs with 256 x 512 tiles
  static const int pair_mode = [] {
    const char* e = getenv("FK_B200_GEMM_PAIR");
    return e != nullptr ? atoi(e) : GL_DEFAULT_PAIR_MODE;
  }();
  CUtensorMap mx, mw;
  if (pair_mode == 1 || pair_mode == 2) {
    int rc = gl_map(x, m, k, x_stride, 128, &mx);
    if (rc != FK_OK) return rc;
    rc = gl_map(w, n, k, k, 128, &mw);
    if (rc != FK_OK) return rc;
    return pair_mode == 2 ? launch_pair<2>(mx, mw, p, stream) : launch_pair<1>(mx, mw, p, stream);
  }

  int rc = gl_map(x, m, k, x_stride, 256, &mx);
  if (rc != FK_OK) return rc;
  rc = gl_map(w, n, k, k, 256, &mw);
  if (rc != FK_OK) return rc;
  static PerDeviceOnce attr_once;
  FK_CUDA_OK(set_max_dynamic_smem(attr_once, gemm_large_kernel, GL_SMEM_ALLOC));
  const int ctas = (int)(tiles < sm_count() ? tiles : sm_count());
  FK_CUDA_OK(launch_kernel(gemm_large_kernel, dim3((unsigned)ctas), dim3(GL_THREADS),
                           (size_t)GL_SMEM_ALLOC, stream, mx, mw, p));
  count_launch(1);
  return FK_OK;
}

}  // namespace fk
