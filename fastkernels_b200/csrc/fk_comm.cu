// Tensor-parallel exchange fused with the next op: all-reduce of the row-parallel
// projection output + residual add + RMSNorm in ONE kernel over peer memory.
//
// Replaces the pair AllReduce.forward (fastkernels/tasks/baseline/L1/allreduce.py:
// 37-55; one-shot kernel fastkernels/tasks/baseline/L1/allreduce.cu:193-212) +
// RMSNorm.forward(x, residual) (fastkernels/tasks/baseline/L1/rms_norm.py:153-164),
// i.e. what the reference's own fused path computes
// (fastkernels/tasks/baseline/L2/flashinfer_allreduce_fusion.py:227-297):
//   s        = bf16( sum over ranks r = 0..t-1 of float(y_r) )    (fp32, rank order)
//   residual = bf16( s + residual )
//   out      = bf16( float(residual) * rsqrt(mean(residual^2) + eps) * float(w) )
//
// Every rank owns one communication buffer (cudaMalloc'ed here, exported with
// CUDA IPC, mapped by the peers): a header of flag words followed by two data
// slots.  The producing GEMM writes its partial [rows, cols] straight into a slot
// of the local buffer; this kernel then, per row (one CTA per row):
//   1. tells every peer "my row of call #e is ready" (st.release.sys of the epoch
//      into the peer's header) and waits until every peer said the same (bounded,
//      2 s -> FK_DEV_WAIT_TIMEOUT),
//   2. reads the row from every rank's slot with plain peer loads (NVLink 5 through
//      NVSwitch; no multicast, no TMA), sums in rank order so all ranks get the
//      same bits, adds the residual, normalises, writes.
// One round trip per call: the two slots alternate between the two row-parallel
// projections of a layer, and a rank can only overwrite slot s (call k+2) after
// it has passed the start barrier of call k+1, which no peer signals before it
// has finished reading call k.
#include "fk_common.cuh"

#include <cstring>

namespace fk {

constexpr int COMM_MAX_ROWS = 512;
constexpr int COMM_MAX_RANKS = 8;
constexpr size_t COMM_HEADER_BYTES = 32768;

struct CommHeader {
  uint32_t start[COMM_MAX_ROWS][COMM_MAX_RANKS];  // written by peers
  uint32_t epoch[COMM_MAX_ROWS];                  // local, per row CTA
};
static_assert(sizeof(CommHeader) <= COMM_HEADER_BYTES, "header size");

struct ArParams {
  uint8_t* base[COMM_MAX_RANKS];
  int nranks, rank;
  size_t slot_offset;   // bytes from base to the slot's row 0
  uint16_t* residual; int64_t residual_stride;
  const uint4* weight;
  float eps;
  uint16_t* out; int64_t out_stride;
  int cols_vec;         // cols / 8
  float inv_cols;
  int32_t* status;
};

__device__ __forceinline__ uint64_t comm_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// peer data: bypass L1 (the line may have been cached by an earlier call)
__device__ __forceinline__ uint4 ld_peer16(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

template <int VPT>
__global__ void __launch_bounds__(256) allreduce_add_rmsnorm_kernel(const ArParams p) {
  __shared__ float red[33];
  __shared__ uint32_t s_epoch;
  pdl_launch_dependents();
  uint4 wv[VPT];  // static norm weights: fetched before the dependency wait
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    wv[i] = c < p.cols_vec ? __ldg(p.weight + c) : make_uint4(0, 0, 0, 0);
  }
  pdl_wait();  // the local GEMM's output is complete
  const int row = blockIdx.x;
  CommHeader* self = reinterpret_cast<CommHeader*>(p.base[p.rank]);
  if (threadIdx.x == 0) s_epoch = self->epoch[row] + 1;
  __syncthreads();
  const uint32_t epoch = s_epoch;
  if (threadIdx.x < p.nranks) {
    const int r = threadIdx.x;
    CommHeader* peer = reinterpret_cast<CommHeader*>(p.base[r]);
    __threadfence_system();
    st_release_sys(&peer->start[row][p.rank], epoch);
    const uint32_t* mine = &self->start[row][r];
    const uint64_t t0 = comm_ns();
    // a peer may already be one call ahead: accept any epoch >= ours
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      if (comm_ns() - t0 > 2000000000ull) {
        if (p.status) atomicOr(p.status, FK_DEV_WAIT_TIMEOUT);
        break;
      }
    }
  }
  __syncthreads();

  uint16_t* rr = p.residual + (int64_t)row * p.residual_stride;
  uint4 v[VPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < p.cols_vec) {
      uint4 part[COMM_MAX_RANKS];
#pragma unroll
      for (int r = 0; r < COMM_MAX_RANKS; ++r)
        if (r < p.nranks)
          part[r] = ld_peer16(reinterpret_cast<const uint4*>(
                                  p.base[r] + p.slot_offset) +
                              (int64_t)row * p.cols_vec + c);
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < COMM_MAX_RANKS; ++r)
        if (r < p.nranks) {
          const uint32_t w4[4] = {part[r].x, part[r].y, part[r].z, part[r].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[2 * j] += bf16lo(w4[j]);
            acc[2 * j + 1] += bf16hi(w4[j]);
          }
        }
      uint4 s;
      s.x = pack_bf16(acc[0], acc[1]); s.y = pack_bf16(acc[2], acc[3]);
      s.z = pack_bf16(acc[4], acc[5]); s.w = pack_bf16(acc[6], acc[7]);
      uint4 res = *reinterpret_cast<const uint4*>(rr + c * 8);
      __nv_bfloat162* a = reinterpret_cast<__nv_bfloat162*>(&s);
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&res);
#pragma unroll
      for (int j = 0; j < 4; ++j) a[j] = __hadd2(a[j], b[j]);
      *reinterpret_cast<uint4*>(rr + c * 8) = s;
      v[i] = s;
      const uint32_t w4[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = bf16lo(w4[j]), hi = bf16hi(w4[j]);
        ss += lo * lo + hi * hi;
      }
    }
  }
  // block reduction
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (int)(blockDim.x >> 5) ? red[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  const float rs = rsqrtf(red[32] * p.inv_cols + p.eps);
  uint16_t* orow = p.out + (int64_t)row * p.out_stride;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < p.cols_vec) {
      const uint4 w = wv[i];
      uint4 o;
      o.x = pack_bf16(bf16lo(v[i].x) * rs * bf16lo(w.x), bf16hi(v[i].x) * rs * bf16hi(w.x));
      o.y = pack_bf16(bf16lo(v[i].y) * rs * bf16lo(w.y), bf16hi(v[i].y) * rs * bf16hi(w.y));
      o.z = pack_bf16(bf16lo(v[i].z) * rs * bf16lo(w.z), bf16hi(v[i].z) * rs * bf16hi(w.z));
      o.w = pack_bf16(bf16lo(v[i].w) * rs * bf16lo(w.w), bf16hi(v[i].w) * rs * bf16hi(w.w));
      *reinterpret_cast<uint4*>(orow + c * 8) = o;
    }
  }
  if (threadIdx.x == 0) self->epoch[row] = epoch;
}

}  // namespace fk

using namespace fk;

extern "C" {

size_t fk_comm_header_bytes(void) { return COMM_HEADER_BYTES; }

int fk_comm_alloc(size_t bytes, void** ptr) {
  FK_REQUIRE(ptr != nullptr && bytes >= COMM_HEADER_BYTES, FK_ERR_INVALID_ARG,
             "fk_comm_alloc: need at least the %zu-byte header", COMM_HEADER_BYTES);
  void* p = nullptr;
  FK_CUDA_OK(cudaMalloc(&p, bytes));
  FK_CUDA_OK(cudaMemset(p, 0, bytes));
  *ptr = p;
  return FK_OK;
}

int fk_comm_free(void* ptr) {
  if (ptr) FK_CUDA_OK(cudaFree(ptr));
  return FK_OK;
}

int fk_comm_ipc_export(void* ptr, void* handle64) {
  FK_REQUIRE(ptr && handle64, FK_ERR_INVALID_ARG, "fk_comm_ipc_export: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  FK_CUDA_OK(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), ptr));
  return FK_OK;
}

int fk_comm_ipc_import(const void* handle64, void** peer_ptr) {
  FK_REQUIRE(handle64 && peer_ptr, FK_ERR_INVALID_ARG, "fk_comm_ipc_import: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  FK_CUDA_OK(cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return FK_OK;
}

int fk_comm_ipc_close(void* peer_ptr) {
  if (peer_ptr) FK_CUDA_OK(cudaIpcCloseMemHandle(peer_ptr));
  return FK_OK;
}

int fk_allreduce_add_rmsnorm(void* const* bases, int nranks, int rank,
                             size_t slot_offset_bytes, void* residual,
                             int64_t residual_stride, const void* weight,
                             float eps, void* out, int64_t out_stride,
                             int64_t rows, int64_t cols, int32_t* status,
                             fk_stream_t stream) {
  FK_REQUIRE(rows >= 0 && cols > 0, FK_ERR_INVALID_ARG,
             "fk_allreduce_add_rmsnorm: bad sizes");
  if (rows == 0) return FK_OK;
  FK_REQUIRE(bases && residual && weight && out, FK_ERR_INVALID_ARG,
             "fk_allreduce_add_rmsnorm: null pointer");
  FK_REQUIRE(nranks >= 1 && nranks <= COMM_MAX_RANKS && rank >= 0 && rank < nranks,
             FK_ERR_INVALID_ARG, "fk_allreduce_add_rmsnorm: bad rank %d of %d", rank,
             nranks);
  FK_REQUIRE(rows <= COMM_MAX_ROWS, FK_ERR_UNSUPPORTED,
             "fk_allreduce_add_rmsnorm: rows = %lld > %d", (long long)rows,
             COMM_MAX_ROWS);
  FK_REQUIRE(cols % 8 == 0 && cols <= 8 * 256 * 8, FK_ERR_UNSUPPORTED,
             "fk_allreduce_add_rmsnorm: cols must be a multiple of 8, <= 16384");
  FK_REQUIRE(slot_offset_bytes >= COMM_HEADER_BYTES && slot_offset_bytes % 16 == 0 &&
                 residual_stride % 8 == 0 && out_stride % 8 == 0 &&
                 aligned16(residual) && aligned16(weight) && aligned16(out),
             FK_ERR_ALIGNMENT, "fk_allreduce_add_rmsnorm: 16-byte alignment required");
  ArParams p{};
  for (int r = 0; r < nranks; ++r) {
    FK_REQUIRE(bases[r] != nullptr, FK_ERR_INVALID_ARG,
               "fk_allreduce_add_rmsnorm: base pointer of rank %d is null", r);
    p.base[r] = static_cast<uint8_t*>(bases[r]);
  }
  p.nranks = nranks; p.rank = rank;
  p.slot_offset = slot_offset_bytes;
  p.residual = (uint16_t*)residual; p.residual_stride = residual_stride;
  p.weight = (const uint4*)weight; p.eps = eps;
  p.out = (uint16_t*)out; p.out_stride = out_stride;
  p.cols_vec = (int)(cols / 8);
  p.inv_cols = 1.0f / (float)cols;
  p.status = status;
  const int block = p.cols_vec >= 256 ? 256 : ((p.cols_vec + 31) / 32) * 32;
  const int vpt = (p.cols_vec + block - 1) / block;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (vpt <= 1) FK_LAUNCH(allreduce_add_rmsnorm_kernel<1>, dim3((unsigned)rows), dim3(block), 0, s, p);
  else if (vpt <= 2) FK_LAUNCH(allreduce_add_rmsnorm_kernel<2>, dim3((unsigned)rows), dim3(block), 0, s, p);
  else if (vpt <= 4) FK_LAUNCH(allreduce_add_rmsnorm_kernel<4>, dim3((unsigned)rows), dim3(block), 0, s, p);
  else FK_LAUNCH(allreduce_add_rmsnorm_kernel<8>, dim3((unsigned)rows), dim3(block), 0, s, p);
  count_launch();
  FK_CUDA_OK(cudaGetLastError());
  return FK_OK;
}

}  // extern "C"
