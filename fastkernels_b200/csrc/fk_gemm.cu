// Decode projections y = x W^T (+ bias) on the 5th-generation tensor cores:
// tcgen05.mma with TMEM accumulators, operands staged by TMA, split-K reduced
// through distributed shared memory inside a thread-block cluster.
//
// Replaces Matmul.forward (fastkernels/tasks/baseline/L1/linear.py:13-17) and
// the F.linear calls of the TP linear layers
// (fastkernels/tasks/baseline/L2/parallel_linear.py:78-81,157-160,237-240,
// 327-335).
//
// At decode the token count m is 1..256 while n, k are in the thousands, so the
// kernel is a WEIGHT-STREAMING kernel: its roofline is HBM bandwidth over the
// n*k*2 weight bytes, not the tensor peak.  The mapping is therefore "swap-AB":
//   MMA M (128 TMEM lanes)  <- 128 rows of W   (one n-tile per CTA)
//   MMA N (16..256 columns) <- the m tokens, zero-padded to MPAD by TMA
//   MMA K (16 per instr.)   <- 64-element k-blocks = one 128-byte swizzle row
// so every weight byte crosses HBM once and the tiny activation tile is re-read
// from L2.  To fill 148 SMs when n/128 < 148 the k range is split across the
// CTAs of a cluster (<= 8); each CTA parks its fp32 partial tile in its own
// shared memory and the cluster reduces it in a fixed order over DSMEM (no
// global workspace, no atomics, deterministic).
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM
// owner, warps 2..5 = epilogue (TMEM lanes 32*(warp%4)..+31).
#include "fk_common.cuh"

#include <mutex>
#include <unordered_map>

namespace fk {

constexpr int GEMM_BN = 128;   // weight rows per CTA (MMA M)
constexpr int GEMM_BK = 64;    // k elements per stage (128 bytes)
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_W_BYTES = GEMM_BN * GEMM_BK * 2;  // 16 KiB

template <int MPAD>
struct GemmCfg {
  static constexpr int kStages = MPAD <= 64 ? 4 : (MPAD <= 128 ? 6 : 4);
  static constexpr int kXBytes = MPAD * GEMM_BK * 2;
  static constexpr int kStageBytes = GEMM_W_BYTES + kXBytes;
  static constexpr int kPartBytes = MPAD * GEMM_BN * 4;
  static constexpr int kBars = kStages * kStageBytes;
  static constexpr int kTotal = kBars + (2 * kStages + 1) * 8 + 16;
  static constexpr int kAlloc = kTotal + 1024;
  static constexpr int kTmemCols = MPAD < 32 ? 32 : MPAD;
  static_assert(kPartBytes <= kStages * kStageBytes, "partial tile must fit");
  static_assert(kAlloc <= 232448, "shared memory budget");
};

struct GemmParams {
  const uint16_t* bias;  // [n] or null
  uint16_t* y; int64_t y_stride;
  int m, n, k;
  int splits, kb_per_split;
  int32_t* status;
};

__device__ __forceinline__ uint64_t gemm_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool gemm_wait(uint64_t* bar, uint32_t parity,
                                          volatile int* abort_flag,
                                          int32_t* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = gemm_ns();
  for (;;) {
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (gemm_ns() - t0 > 2000000000ull) {
      *abort_flag = 1;
      if (status) atomicOr(status, FK_DEV_WAIT_TIMEOUT);
      return false;
    }
  }
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
          smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t tmem_d, uint64_t desc_a,
                                            uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]),
        "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
        "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
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
// so the (ordered) loads still overlap in the memory system.
__device__ __forceinline__ float4 ld_dsmem_f32x4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(cluster_addr)
               : "memory");
  return v;
}

// K-major, 128-byte-swizzled shared-memory operand descriptor: rows of 128
// bytes, 8-row groups 1024 bytes apart (SBO), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fff);
  d |= (uint64_t)1 << 16;            // leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset
  d |= (uint64_t)1 << 46;            // version
  d |= (uint64_t)2 << 61;            // SWIZZLE_128B
  return d;
}

template <int MPAD>
__global__ void __launch_bounds__(GEMM_THREADS) gemm_bf16_kernel(
    const __grid_constant__ CUtensorMap tmap_w,
    const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
  using Cfg = GemmCfg<MPAD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Cfg::kBars);
  uint64_t* empty = full + Cfg::kStages;
  uint64_t* accum_full = empty + Cfg::kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = (int)cluster_rank();
  const int n_tile = blockIdx.x / p.splits;
  const int n0 = n_tile * GEMM_BN;
  const int kb_total = p.k / GEMM_BK;
  const int kb_begin = split * p.kb_per_split;
  const int nkb = min(kb_total, kb_begin + p.kb_per_split) - kb_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum_full, 1);
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

  if (warp == 0 && lane == 0) {
    // ----------------------------- TMA producer ----------------------------
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
    int stage = 0;
    uint32_t phase = 0;
    for (int i = 0; i < nkb; ++i) {
      if (!gemm_wait(&empty[stage], phase ^ 1, abort_flag, p.status)) break;
      uint8_t* wdst = smem + stage * Cfg::kStageBytes;
      mbar_arrive_expect_tx(&full[stage], (uint32_t)Cfg::kStageBytes);
      const int kc = (kb_begin + i) * GEMM_BK;
      tma_load_2d(wdst, &tmap_w, &full[stage], kc, n0);
      tma_load_2d(wdst + GEMM_W_BYTES, &tmap_x, &full[stage], kc, 0);
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
    for (int i = 0; i < nkb && ok; ++i) {
      if (!gemm_wait(&full[stage], phase, abort_flag, p.status)) { ok = false; break; }
      tc_fence_after();
      const uint32_t wa = smem_u32(smem + stage * Cfg::kStageBytes);
      const uint32_t xa = wa + GEMM_W_BYTES;
#pragma unroll
      for (int kk = 0; kk < GEMM_BK / 16; ++kk) {
        tc_mma_bf16(tmem_base, smem_desc_sw128(wa + kk * 32),
                    smem_desc_sw128(xa + kk * 32), idesc,
                    (i > 0 || kk > 0) ? 1u : 0u);
      }
      tc_commit(&empty[stage]);  // frees the stage when these MMAs retire
      if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
    }
    if (ok) tc_commit(accum_full);
  }
  __syncwarp();

  // ------------------------------- epilogue --------------------------------
  float* part = reinterpret_cast<float*>(smem);  // [MPAD][128] fp32, reuses the ring
  if (warp >= 2) {
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int e = q * 32 + lane;
    const bool ok = gemm_wait(accum_full, 0, abort_flag, p.status);
    tc_fence_after();
    if (ok) {
#pragma unroll 1
      for (int c = 0; c < MPAD; c += 16) {
        uint32_t v[16];
        tc_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c, v);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j)
          part[(c + j) * GEMM_BN + e] = __uint_as_float(v[j]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // every CTA's partial tile is visible cluster-wide

  if (warp >= 2) {
    // Each CTA of the cluster reduces the rows m = split, split + S, ... of the
    // tile: 32 threads x float4 cover one 128-column row, 4 rows per pass, all
    // S peer loads of a pass in flight together; summation order is r = 0..S-1.
    const int t = (warp - 2) * 32 + lane;
    const int c4 = t & 31, rsub = t >> 5;
    const int n = n0 + c4 * 4;
    const uint32_t part_addr = smem_u32(part);
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
      for (int mm = split + p.splits * rsub; mm < p.m; mm += p.splits * 4) {
        const uint32_t off = (uint32_t)(mm * GEMM_BN + c4 * 4) * 4u;
        float4 v[8];
#pragma unroll
        for (int r = 0; r < 8; ++r)
          if (r < p.splits) v[r] = ld_dsmem_f32x4(peer[r] + off);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < 8; ++r)
          if (r < p.splits) {
            acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w;
          }
        acc.x += b[0]; acc.y += b[1]; acc.z += b[2]; acc.w += b[3];
        uint16_t* dst = p.y + (int64_t)mm * p.y_stride + n;
        if (vec_ok) {
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
  __syncthreads();
  cluster_sync_all();  // peers are done reading this CTA's shared memory
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(
                     tmem_base),
                 "r"((uint32_t)Cfg::kTmemCols)
                 : "memory");
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
static std::mutex g_g2_mu;
static std::unordered_map<G2Key, CUtensorMap, G2Hash> g_g2_maps;

// Row-major [rows, cols] bf16 matrix, rows `stride` elements apart; box =
// 64 columns (128 bytes, one swizzle row) x box_rows rows.
static int get_2d_map(const void* ptr, int64_t rows, int64_t cols,
                      int64_t stride, int box_rows, CUtensorMap* out) {
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

// Split-K factor: fill the SMs, keep >= 4 k-blocks per CTA, prefer fewer splits.
static int choose_splits(int n_tiles, int kb_total, int slots) {
  int best = 1;
  double best_eff = 0.0;
  for (int s = 1; s <= 8; ++s) {
    if (kb_total / s < 4 && s > 1) break;
    const int64_t ctas = (int64_t)n_tiles * s;
    const int64_t waves = (ctas + slots - 1) / slots;
    const double eff = (double)ctas / (double)(waves * slots);
    if (eff > best_eff + 0.03) {
      best_eff = eff;
      best = s;
    }
  }
  return best;
}

template <int MPAD>
static int launch_gemm(const CUtensorMap& mw, const CUtensorMap& mx,
                       const GemmParams& p, int n_tiles, cudaStream_t s) {
  using Cfg = GemmCfg<MPAD>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_bf16_kernel<MPAD>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::kAlloc);
  });
  FK_CUDA_OK(attr_err);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)(n_tiles * p.splits), 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kAlloc;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)p.splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  FK_CUDA_OK(cudaLaunchKernelEx(&cfg, gemm_bf16_kernel<MPAD>, mw, mx, p));
  count_launch();
  return FK_OK;
}

}  // namespace fk

using namespace fk;

extern "C" {

size_t fk_gemm_bf16_workspace_bytes(int64_t m, int64_t n, int64_t k) {
  (void)m; (void)n; (void)k;
  return 0;  // split-K partials live in distributed shared memory
}

int fk_gemm_bf16(const void* x, int64_t x_stride, const void* w,
                 const void* bias, void* y, int64_t y_stride, int64_t m,
                 int64_t n, int64_t k, void* workspace,
                 size_t workspace_bytes, int32_t* status, fk_stream_t stream) {
  (void)workspace; (void)workspace_bytes;
  FK_REQUIRE(m >= 0 && n >= 0 && k > 0, FK_ERR_INVALID_ARG, "fk_gemm_bf16: bad sizes");
  if (m == 0 || n == 0) return FK_OK;
  FK_REQUIRE(x && w && y, FK_ERR_INVALID_ARG, "fk_gemm_bf16: null pointer");
  FK_REQUIRE(m <= 256, FK_ERR_UNSUPPORTED,
             "fk_gemm_bf16: m = %lld > 256 (decode kernel)", (long long)m);
  FK_REQUIRE(k % GEMM_BK == 0, FK_ERR_UNSUPPORTED,
             "fk_gemm_bf16: k = %lld must be a multiple of 64", (long long)k);
  FK_REQUIRE(n < (1ll << 31) && k < (1ll << 31), FK_ERR_UNSUPPORTED,
             "fk_gemm_bf16: dimension too large");
  FK_REQUIRE(x_stride >= k && y_stride >= n, FK_ERR_INVALID_ARG,
             "fk_gemm_bf16: row stride smaller than the row");
  FK_REQUIRE(aligned16(x) && aligned16(w) && x_stride % 8 == 0, FK_ERR_ALIGNMENT,
             "fk_gemm_bf16: x and w need 16-byte aligned rows");

  const int mpad = m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : m <= 128 ? 128 : 256;
  const int n_tiles = (int)((n + GEMM_BN - 1) / GEMM_BN);
  const int kb_total = (int)(k / GEMM_BK);
  const int ctas_per_sm = mpad <= 64 ? 2 : 1;

  CUtensorMap mw, mx;
  int rc = get_2d_map(w, n, k, k, GEMM_BN, &mw);
  if (rc != FK_OK) return rc;
  rc = get_2d_map(x, m, k, x_stride, mpad, &mx);
  if (rc != FK_OK) return rc;

  GemmParams p{};
  p.bias = (const uint16_t*)bias;
  p.y = (uint16_t*)y; p.y_stride = y_stride;
  p.m = (int)m; p.n = (int)n; p.k = (int)k;
  p.splits = choose_splits(n_tiles, kb_total, sm_count() * ctas_per_sm);
  p.kb_per_split = (kb_total + p.splits - 1) / p.splits;
  // every split must own at least one k-block
  while (p.splits > 1 && (p.splits - 1) * p.kb_per_split >= kb_total) {
    --p.splits;
    p.kb_per_split = (kb_total + p.splits - 1) / p.splits;
  }
  p.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (mpad) {
    case 16: return launch_gemm<16>(mw, mx, p, n_tiles, s);
    case 32: return launch_gemm<32>(mw, mx, p, n_tiles, s);
    case 64: return launch_gemm<64>(mw, mx, p, n_tiles, s);
    case 128: return launch_gemm<128>(mw, mx, p, n_tiles, s);
    default: return launch_gemm<256>(mw, mx, p, n_tiles, s);
  }
}

}  // extern "C"
