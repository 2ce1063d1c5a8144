// Pieces shared by the decode GEMM (fk_gemm.cu) and the persistent decode-block
// kernel (fk_block.cu): tile geometry, bounded waits, stream-K unit ranges, the
// weight-tile loads and the host-side tensor-map cache.
#pragma once

#include "fk_common.cuh"
#include "fk_tcgen05.cuh"

namespace fk {

constexpr int GEMM_BN = 128;   // weight rows per tile (MMA M)
constexpr int GEMM_BK = 64;    // k elements per stage (128 bytes)
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_W_BYTES = GEMM_BN * GEMM_BK * 2;  // 16 KiB
constexpr int GEMM_MAX_CTAS = 160;                   // workspace slots

// Row-major [rows, cols] bf16 matrix, rows `stride` elements apart; box = 64
// columns (128 bytes, one swizzle row) x box_rows rows.  Encoded maps are cached.
int gemm_get_2d_map(const void* ptr, int64_t rows, int64_t cols, int64_t stride,
                    int box_rows, CUtensorMap* out);
inline int gemm_mpad_for(int64_t m) {
  return m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : m <= 128 ? 128 : 256;
}
constexpr size_t GEMM_FLAGS_BYTES = 1024;  // GEMM_MAX_CTAS ints + the grid-barrier word

#ifdef __CUDACC__

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

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ long long unit_begin(int c, long long units, int ctas) {
  return (long long)c * units / ctas;
}

// One weight tile of a stage: 128 consecutive rows, or (SILU) 64 gate rows and the
// 64 up rows of the same columns as two boxes; the 128-byte swizzle repeats every
// 8 rows, so two 64-row boxes back to back are laid out like one 128-row box.
template <bool SILU>
__device__ __forceinline__ void load_w_tile(uint8_t* dst, const CUtensorMap* tmap_w,
                                            uint64_t* bar, int kb, int tile, int half_n) {
  if (SILU) {
    tma_load_2d(dst, tmap_w, bar, kb * GEMM_BK, tile * (GEMM_BN / 2));
    tma_load_2d(dst + GEMM_W_BYTES / 2, tmap_w, bar, kb * GEMM_BK,
                half_n + tile * (GEMM_BN / 2));
  } else {
    tma_load_2d(dst, tmap_w, bar, kb * GEMM_BK, tile * GEMM_BN);
  }
}

#endif  // __CUDACC__

}  // namespace fk
