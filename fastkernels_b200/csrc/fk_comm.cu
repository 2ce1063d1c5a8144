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
//
// Two-stage variant (large payloads on 4 or 8 ranks, the regime where the
// reference switches to reduce-scatter + all-gather,
// fastkernels/tasks/baseline/L1/allreduce.cu:214-250, 404-415): row i is OWNED by
// rank i % t.  Every rank tells only the owner that its row is ready; the owner
// alone reads the t partial rows, sums them (same rank order), PUSHES the bf16
// sum into a staging row of every peer's buffer with plain stores and raises the
// row's `done` flag there; the other ranks wait for that flag (bounded) and read
// the sum from their own memory.  Every rank then adds its residual and
// normalises locally, so all ranks still produce identical bits.  NVLink traffic
// per rank and call: 2 (t-1)/t payloads instead of (t-1).
//
// The same row routine also runs as ONE cooperative launch over all ranks of a
// group whose buffers live on one device (fk_allreduce_add_rmsnorm_group): blocks
// (row, rank) of one grid are resident together, which separate launches on one
// GPU are not guaranteed to be, so this is how a multi-rank exchange is checked
// on a single GPU.
#include "fk_common.cuh"

#include <cstddef>
#include <cstring>

namespace fk {

constexpr int COMM_MAX_ROWS = 512;
constexpr int COMM_MAX_RANKS = 8;
constexpr size_t COMM_HEADER_BYTES = 32768;

struct CommHeader {
  uint32_t start[COMM_MAX_ROWS][COMM_MAX_RANKS];  // written by peers
  uint32_t epoch[COMM_MAX_ROWS];                  // local, per row CTA
  uint32_t done[COMM_MAX_ROWS];                   // two-stage: written by the row's owner
};
static_assert(sizeof(CommHeader) <= COMM_HEADER_BYTES, "header size");

struct ArParams {
  uint8_t* base[COMM_MAX_RANKS];
  int nranks, rank;
  size_t slot_offset;     // bytes from base to the slot's row 0
  size_t reduced_offset;  // two-stage: bytes from base to the staging rows (0 = one-shot)
  uint16_t* residual; int64_t residual_stride;
  const uint4* weight;
  float eps;
  uint16_t* out; int64_t out_stride;
  int cols_vec;         // cols / 8
  float inv_cols;
  int32_t* status;
};
// per-rank tensors of a one-device group launch
struct ArGroup {
  uint16_t* residual[COMM_MAX_RANKS];
  uint16_t* out[COMM_MAX_RANKS];
  int rows;
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
__device__ __forceinline__ void st_peer16(uint4* p, const uint4& v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
// Bounded wait until *flag has reached `epoch` (a peer may already be one call
// ahead: any epoch >= ours counts).
__device__ __forceinline__ void wait_epoch(const uint32_t* flag, uint32_t epoch,
                                           int32_t* status) {
  if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return;
  const uint64_t t0 = comm_ns();
  for (;;) {
    // the clock is read once per 64 polls: reading it costs about as much as a
    // poll, and the wait is on the critical path of every call
    for (int i = 0; i < 64; ++i)
      if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return;
    if (comm_ns() - t0 > 2000000000ull) {
      if (status) atomicOr(status, FK_DEV_WAIT_TIMEOUT);
      return;
    }
  }
}

// One token row of one rank.  TWO_STAGE selects the owner-reduces-and-pushes
// exchange; otherwise every rank pulls the row from every rank.
template <int VPT, bool TWO_STAGE>
__device__ __forceinline__ void ar_row(const ArParams& p, const int rank, const int row,
                                       uint16_t* residual, uint16_t* out,
                                       const uint4 (&wv)[VPT], float* red,
                                       const uint32_t epoch) {
  CommHeader* self = reinterpret_cast<CommHeader*>(p.base[rank]);
  const int owner = TWO_STAGE ? row % p.nranks : rank;
  uint16_t* rr = residual + (int64_t)row * p.residual_stride;
  // One-stage exchange: this rank's own partial row and the residual row are local
  // and complete (the preceding kernel wrote them), so they are fetched BEFORE the
  // flag round with the peers and their latency hides under it.
  constexpr bool EARLY = !TWO_STAGE && VPT <= 4;
  uint4 own[EARLY ? VPT : 1], res_early[EARLY ? VPT : 1];
  if (EARLY) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < p.cols_vec) {
        own[i] = ld_peer16(reinterpret_cast<const uint4*>(p.base[rank] + p.slot_offset) +
                           (int64_t)row * p.cols_vec + c);
        res_early[i] = *reinterpret_cast<const uint4*>(rr + c * 8);
      }
    }
  }
  if (!TWO_STAGE) {
    if (threadIdx.x < p.nranks) {
      const int r = threadIdx.x;
      CommHeader* peer = reinterpret_cast<CommHeader*>(p.base[r]);
      // the partial row was written by the preceding kernel, whose completion this
      // grid has waited for: the release store alone publishes it system-wide
      st_release_sys(&peer->start[row][rank], epoch);
      wait_epoch(&self->start[row][r], epoch, p.status);
    }
  } else {
    if (threadIdx.x == 0) {
      // only the row's owner needs to know that this rank's partial row is ready
      CommHeader* own_hdr = reinterpret_cast<CommHeader*>(p.base[owner]);
      st_release_sys(&own_hdr->start[row][rank], epoch);
    }
    if (rank == owner && threadIdx.x < p.nranks)
      wait_epoch(&self->start[row][threadIdx.x], epoch, p.status);
    if (rank != owner && threadIdx.x == 0) wait_epoch(&self->done[row], epoch, p.status);
  }
  __syncthreads();

  uint4 v[VPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < p.cols_vec) {
      uint4 s;
      const int64_t at = (int64_t)row * p.cols_vec + c;
      if (!TWO_STAGE || rank == owner) {
        uint4 part[COMM_MAX_RANKS];
#pragma unroll
        for (int r = 0; r < COMM_MAX_RANKS; ++r)
          if (r < p.nranks) {
            if (EARLY && r == rank)
              part[r] = own[EARLY ? i : 0];
            else
              part[r] = ld_peer16(
                  reinterpret_cast<const uint4*>(p.base[r] + p.slot_offset) + at);
          }
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
        s.x = pack_bf16(acc[0], acc[1]); s.y = pack_bf16(acc[2], acc[3]);
        s.z = pack_bf16(acc[4], acc[5]); s.w = pack_bf16(acc[6], acc[7]);
        if (TWO_STAGE) {
#pragma unroll
          for (int r = 0; r < COMM_MAX_RANKS; ++r)
            if (r < p.nranks && r != rank)
              st_peer16(reinterpret_cast<uint4*>(p.base[r] + p.reduced_offset) + at, s);
        }
      } else {
        s = ld_peer16(reinterpret_cast<const uint4*>(p.base[rank] + p.reduced_offset) + at);
      }
      uint4 res = EARLY ? res_early[EARLY ? i : 0]
                        : *reinterpret_cast<const uint4*>(rr + c * 8);
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
  if (TWO_STAGE && rank == owner) {
    // the pushed row is complete in every peer's memory before its flag rises
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < p.nranks && (int)threadIdx.x != rank) {
      CommHeader* peer = reinterpret_cast<CommHeader*>(p.base[threadIdx.x]);
      st_release_sys(&peer->done[row], epoch);
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
  uint16_t* orow = out + (int64_t)row * p.out_stride;
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

template <int VPT, bool TWO_STAGE>
__global__ void __launch_bounds__(256) allreduce_add_rmsnorm_kernel(const ArParams p) {
  __shared__ float red[33];
  pdl_launch_dependents();
  uint4 wv[VPT];  // static norm weights: fetched before the dependency wait
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    wv[i] = c < p.cols_vec ? __ldg(p.weight + c) : make_uint4(0, 0, 0, 0);
  }
  pdl_wait();  // the local GEMM's output is complete, and so is this kernel's previous
               // launch, which wrote the row's call counter read next
  const uint32_t epoch =
      reinterpret_cast<CommHeader*>(p.base[p.rank])->epoch[blockIdx.x] + 1;
  ar_row<VPT, TWO_STAGE>(p, p.rank, blockIdx.x, p.residual, p.out, wv, red, epoch);
}

// All ranks of a group on ONE device: block (row, rank).  Launched cooperatively,
// so every block is resident and the waits between ranks can be satisfied.
template <int VPT, bool TWO_STAGE>
__global__ void __launch_bounds__(256) allreduce_add_rmsnorm_group_kernel(
    const ArParams p, const ArGroup g) {
  __shared__ float red[33];
  uint4 wv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    wv[i] = c < p.cols_vec ? __ldg(p.weight + c) : make_uint4(0, 0, 0, 0);
  }
  const int rank = blockIdx.y;
  // all ranks walk the rows in the same order, so the waits of one pass are
  // answered by blocks that are in the same pass
  for (int row = blockIdx.x; row < g.rows; row += gridDim.x) {
    const uint32_t epoch = reinterpret_cast<CommHeader*>(p.base[rank])->epoch[row] + 1;
    ar_row<VPT, TWO_STAGE>(p, rank, row, g.residual[rank], g.out[rank], wv, red, epoch);
    __syncthreads();   // red[] is reused by the next row
  }
}

// ---------------------------------------------------------------------------
// Pushed exchange.  The row-parallel projection itself (fk_gemm_bf16_push) stores
// every output pair straight into ALL ranks' receive areas as 8-byte
// {two bf16, call number} words, each written atomically; this kernel only ever
// reads its OWN memory: per element it polls the t senders' words until they carry
// this call's number, sums in rank order, adds the residual and normalises.  No
// flag round and no peer loads: one NVLink traversal per call instead of three.
// The call number doubles the bytes on the wire, so this form is for the small
// decode payloads (the caller decides, fk_allreduce_push_preferred).
// Receive area of one slot: [sender][row][cols / 2] 8-byte words, senders
// `sender_stride` bytes apart.
// ---------------------------------------------------------------------------
struct PushedParams {
  uint8_t* base;            // this rank's communication buffer (header first)
  int nranks;
  size_t ll_offset, sender_stride;
  uint16_t* residual; int64_t residual_stride;
  const uint4* weight; float eps;
  uint16_t* out; int64_t out_stride;
  int cols_vec; float inv_cols;
  int32_t* status;
};

__device__ __forceinline__ void ld_pairs(const uint8_t* p, uint64_t& a, uint64_t& b) {
  asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p)
               : "memory");
}

template <int VPT>
__global__ void __launch_bounds__(256) allreduce_pushed_kernel(const PushedParams p) {
  __shared__ float red[33];
  pdl_launch_dependents();
  uint4 wv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    wv[i] = c < p.cols_vec ? __ldg(p.weight + c) : make_uint4(0, 0, 0, 0);
  }
  pdl_wait();
  const int row = blockIdx.x;
  CommHeader* self = reinterpret_cast<CommHeader*>(p.base);
  const uint32_t epoch = self->epoch[row] + 1;
  uint16_t* rr = p.residual + (int64_t)row * p.residual_stride;
  const uint8_t* area = p.base + p.ll_offset + (size_t)row * (size_t)p.cols_vec * 32u;
  uint4 v[VPT];
  float ss = 0.f;
  uint64_t t0 = 0;
  bool gave_up = false;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < p.cols_vec) {
      const uint4 res = *reinterpret_cast<const uint4*>(rr + c * 8);
      // 8 columns = four {pair, call number} words = 32 bytes per sender
      uint64_t w[COMM_MAX_RANKS][4];
#pragma unroll
      for (int r = 0; r < COMM_MAX_RANKS; ++r)
        if (r < p.nranks) {
          const uint8_t* src = area + (size_t)r * p.sender_stride + (size_t)c * 32u;
          ld_pairs(src, w[r][0], w[r][1]);
          ld_pairs(src + 16, w[r][2], w[r][3]);
        }
#pragma unroll
      for (int r = 0; r < COMM_MAX_RANKS; ++r)
        if (r < p.nranks) {
          const uint8_t* src = area + (size_t)r * p.sender_stride + (size_t)c * 32u;
          int polls = 0;
          while (!gave_up && ((uint32_t)(w[r][0] >> 32) != epoch ||
                              (uint32_t)(w[r][1] >> 32) != epoch ||
                              (uint32_t)(w[r][2] >> 32) != epoch ||
                              (uint32_t)(w[r][3] >> 32) != epoch)) {
            ld_pairs(src, w[r][0], w[r][1]);
            ld_pairs(src + 16, w[r][2], w[r][3]);
            if ((++polls & 63) == 0) {      // the clock is read once per 64 polls
              const uint64_t now = comm_ns();
              if (t0 == 0) t0 = now;
              else if (now - t0 > 2000000000ull) {
                if (p.status) atomicOr(p.status, FK_DEV_WAIT_TIMEOUT);
                gave_up = true;
              }
            }
          }
        }
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < COMM_MAX_RANKS; ++r)
        if (r < p.nranks) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t d = (uint32_t)w[r][j];
            acc[2 * j] += bf16lo(d);
            acc[2 * j + 1] += bf16hi(d);
          }
        }
      uint4 s;
      s.x = pack_bf16(acc[0], acc[1]); s.y = pack_bf16(acc[2], acc[3]);
      s.z = pack_bf16(acc[4], acc[5]); s.w = pack_bf16(acc[6], acc[7]);
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

namespace {

struct ArCall {
  void* const* bases; int nranks; int rank;   // rank < 0: all ranks in one launch
  size_t slot_offset, reduced_offset;         // reduced_offset 0: one-shot
  void* const* residuals; void* const* outs;  // group launch: one per rank
  void* residual; void* out;
  int64_t residual_stride, out_stride;
  const void* weight; float eps;
  int64_t rows, cols;
  int32_t* status; cudaStream_t stream;
};

template <int VPT, bool TWO>
int ar_launch(const ArParams& p, const ArGroup* g, int64_t rows, int block, cudaStream_t s) {
  if (g == nullptr) {
    FK_LAUNCH((allreduce_add_rmsnorm_kernel<VPT, TWO>), dim3((unsigned)rows), dim3(block), 0,
              s, p);
  } else {
    // blocks of different ranks wait for one another: the grid is sized to be
    // resident all at once (each block walks several rows if need be) and is
    // launched cooperatively, which fails instead of hanging if it is not
    int per_sm = 0;
    FK_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(
        &per_sm, allreduce_add_rmsnorm_group_kernel<VPT, TWO>, block, 0));
    int64_t row_blocks = (int64_t)per_sm * sm_count() / p.nranks;
    FK_REQUIRE(row_blocks >= 1, FK_ERR_UNSUPPORTED,
               "fk_allreduce_add_rmsnorm_group: %d ranks do not fit on the device", p.nranks);
    if (row_blocks > rows) row_blocks = rows;
    ArParams pp = p;
    ArGroup gg = *g;
    gg.rows = (int)rows;
    void* args[2] = {&pp, &gg};
    FK_CUDA_OK(cudaLaunchCooperativeKernel(
        (const void*)allreduce_add_rmsnorm_group_kernel<VPT, TWO>,
        dim3((unsigned)row_blocks, (unsigned)p.nranks), dim3(block), args, 0, s));
  }
  count_launch();
  FK_CUDA_OK(cudaGetLastError());
  return FK_OK;
}

int ar_run(const ArCall& c, const char* who) {
  FK_REQUIRE(c.rows >= 0 && c.cols > 0, FK_ERR_INVALID_ARG, "%s: bad sizes", who);
  if (c.rows == 0) return FK_OK;
  const bool group = c.rank < 0;
  FK_REQUIRE(c.bases && c.weight && (group ? (c.residuals && c.outs) : (c.residual && c.out)),
             FK_ERR_INVALID_ARG, "%s: null pointer", who);
  FK_REQUIRE(c.nranks >= 1 && c.nranks <= COMM_MAX_RANKS && (group || c.rank < c.nranks),
             FK_ERR_INVALID_ARG, "%s: bad rank %d of %d", who, c.rank, c.nranks);
  FK_REQUIRE(c.rows <= COMM_MAX_ROWS, FK_ERR_UNSUPPORTED, "%s: rows = %lld > %d", who,
             (long long)c.rows, COMM_MAX_ROWS);
  FK_REQUIRE(c.cols % 8 == 0 && c.cols <= 8 * 256 * 8, FK_ERR_UNSUPPORTED,
             "%s: cols must be a multiple of 8, <= 16384", who);
  FK_REQUIRE(c.slot_offset >= COMM_HEADER_BYTES && c.slot_offset % 16 == 0 &&
                 c.residual_stride % 8 == 0 && c.out_stride % 8 == 0 && aligned16(c.weight),
             FK_ERR_ALIGNMENT, "%s: 16-byte alignment required", who);
  const bool two = c.reduced_offset != 0;
  const size_t payload = (size_t)c.rows * (size_t)c.cols * 2;
  if (two) {
    FK_REQUIRE(c.reduced_offset >= COMM_HEADER_BYTES && c.reduced_offset % 16 == 0 &&
                   (c.reduced_offset >= c.slot_offset + payload ||
                    c.slot_offset >= c.reduced_offset + payload),
               FK_ERR_INVALID_ARG,
               "%s: the staging rows must lie after the header and not overlap the slot", who);
  }
  ArParams p{};
  ArGroup g{};
  for (int r = 0; r < c.nranks; ++r) {
    FK_REQUIRE(c.bases[r] != nullptr, FK_ERR_INVALID_ARG,
               "%s: base pointer of rank %d is null", who, r);
    p.base[r] = static_cast<uint8_t*>(c.bases[r]);
    if (group) {
      FK_REQUIRE(c.residuals[r] && c.outs[r] && aligned16(c.residuals[r]) &&
                     aligned16(c.outs[r]),
                 FK_ERR_INVALID_ARG, "%s: residual / out of rank %d null or unaligned", who, r);
      g.residual[r] = static_cast<uint16_t*>(c.residuals[r]);
      g.out[r] = static_cast<uint16_t*>(c.outs[r]);
    }
  }
  if (!group)
    FK_REQUIRE(aligned16(c.residual) && aligned16(c.out), FK_ERR_ALIGNMENT,
               "%s: 16-byte alignment required", who);
  p.nranks = c.nranks; p.rank = group ? 0 : c.rank;
  p.slot_offset = c.slot_offset;
  p.reduced_offset = c.reduced_offset;
  p.residual = (uint16_t*)c.residual; p.residual_stride = c.residual_stride;
  p.weight = (const uint4*)c.weight; p.eps = c.eps;
  p.out = (uint16_t*)c.out; p.out_stride = c.out_stride;
  p.cols_vec = (int)(c.cols / 8);
  p.inv_cols = 1.0f / (float)c.cols;
  p.status = c.status;
  const int block = p.cols_vec >= 256 ? 256 : ((p.cols_vec + 31) / 32) * 32;
  const int vpt = (p.cols_vec + block - 1) / block;
  const ArGroup* gp = group ? &g : nullptr;
#define FK_AR_DISPATCH(V)                                                     \
  return two ? ar_launch<V, true>(p, gp, c.rows, block, c.stream)             \
             : ar_launch<V, false>(p, gp, c.rows, block, c.stream)
  if (vpt <= 1) { FK_AR_DISPATCH(1); }
  if (vpt <= 2) { FK_AR_DISPATCH(2); }
  if (vpt <= 4) { FK_AR_DISPATCH(4); }
  FK_AR_DISPATCH(8);
#undef FK_AR_DISPATCH
}

}  // namespace

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
  FK_REQUIRE(rank >= 0, FK_ERR_INVALID_ARG, "fk_allreduce_add_rmsnorm: bad rank %d of %d",
             rank, nranks);
  ArCall c{bases, nranks, rank, slot_offset_bytes, 0, nullptr, nullptr, residual, out,
           residual_stride, out_stride, weight, eps, rows, cols, status,
           static_cast<cudaStream_t>(stream)};
  return ar_run(c, "fk_allreduce_add_rmsnorm");
}

int fk_allreduce_two_stage_preferred(int nranks, int64_t rows, int64_t cols) {
  // The reference switches to its two-stage kernel from 512 KiB on up to 4 ranks
  // and from 256 KiB on more (allreduce.cu:404-415).  Measured on B200 over NVSwitch
  // (calls back to back inside a CUDA graph) the fused one-stage exchange is the
  // faster one at every payload a decode step produces: 512 KiB on 2 / 4 / 8 ranks
  // 12 / 13 / 17 us against 26 us, 2 MiB on 8 ranks 36 against 39 us -- the second
  // flag round costs more than the (t - 1) x payload of peer reads it saves.  Two
  // stages are chosen only beyond that, for the 8-rank payloads of a prefill chunk.
  const int64_t bytes = rows * cols * 2;
  if (nranks < 8) return 0;
  return bytes >= 4 * 1024 * 1024;
}

int fk_allreduce_add_rmsnorm_staged(void* const* bases, int nranks, int rank,
                                    size_t slot_offset_bytes, size_t staging_offset_bytes,
                                    void* residual, int64_t residual_stride,
                                    const void* weight, float eps, void* out,
                                    int64_t out_stride, int64_t rows, int64_t cols,
                                    int32_t* status, fk_stream_t stream) {
  FK_REQUIRE(rank >= 0, FK_ERR_INVALID_ARG,
             "fk_allreduce_add_rmsnorm_staged: bad rank %d of %d", rank, nranks);
  FK_REQUIRE(staging_offset_bytes != 0, FK_ERR_INVALID_ARG,
             "fk_allreduce_add_rmsnorm_staged: no staging rows given");
  ArCall c{bases, nranks, rank, slot_offset_bytes, staging_offset_bytes, nullptr, nullptr,
           residual, out, residual_stride, out_stride, weight, eps, rows, cols, status,
           static_cast<cudaStream_t>(stream)};
  return ar_run(c, "fk_allreduce_add_rmsnorm_staged");
}

int fk_allreduce_add_rmsnorm_group(void* const* bases, int nranks,
                                   size_t slot_offset_bytes, size_t staging_offset_bytes,
                                   void* const* residuals, int64_t residual_stride,
                                   const void* weight, float eps, void* const* outs,
                                   int64_t out_stride, int64_t rows, int64_t cols,
                                   int32_t* status, fk_stream_t stream) {
  ArCall c{bases, nranks, -1, slot_offset_bytes, staging_offset_bytes, residuals, outs,
           nullptr, nullptr, residual_stride, out_stride, weight, eps, rows, cols, status,
           static_cast<cudaStream_t>(stream)};
  return ar_run(c, "fk_allreduce_add_rmsnorm_group");
}

size_t fk_comm_epoch_offset(void) { return offsetof(CommHeader, epoch); }

int fk_allreduce_push_preferred(int nranks, int64_t rows, int64_t cols) {
  // Pushing costs 2 x the payload per peer on the wire (every pair travels with its
  // call number) but only one NVLink traversal; it wins while that stays small.
  // (the projection that pushes is the decode kernel: at most 256 rows)
  if (nranks < 2 || nranks > COMM_MAX_RANKS || rows < 1 || rows > 256) return 0;
  return (int64_t)(nranks - 1) * rows * cols * 4 <= 4ll * 1024 * 1024 ? 1 : 0;
}

int fk_allreduce_add_rmsnorm_pushed(void* base, int nranks, size_t ll_offset_bytes,
                                    size_t sender_stride_bytes, void* residual,
                                    int64_t residual_stride, const void* weight, float eps,
                                    void* out, int64_t out_stride, int64_t rows, int64_t cols,
                                    int32_t* status, fk_stream_t stream) {
  const char* who = "fk_allreduce_add_rmsnorm_pushed";
  FK_REQUIRE(rows >= 0 && cols > 0, FK_ERR_INVALID_ARG, "%s: bad sizes", who);
  if (rows == 0) return FK_OK;
  FK_REQUIRE(base && residual && weight && out, FK_ERR_INVALID_ARG, "%s: null pointer", who);
  FK_REQUIRE(nranks >= 1 && nranks <= COMM_MAX_RANKS, FK_ERR_INVALID_ARG,
             "%s: bad rank count %d", who, nranks);
  FK_REQUIRE(rows <= COMM_MAX_ROWS, FK_ERR_UNSUPPORTED, "%s: rows = %lld > %d", who,
             (long long)rows, COMM_MAX_ROWS);
  FK_REQUIRE(cols % 8 == 0 && cols <= 8 * 256 * 8, FK_ERR_UNSUPPORTED,
             "%s: cols must be a multiple of 8, <= 16384", who);
  FK_REQUIRE(ll_offset_bytes >= COMM_HEADER_BYTES && ll_offset_bytes % 16 == 0 &&
                 sender_stride_bytes % 16 == 0 &&
                 sender_stride_bytes >= (size_t)rows * (size_t)cols * 4 &&
                 residual_stride % 8 == 0 && out_stride % 8 == 0 && aligned16(weight) &&
                 aligned16(residual) && aligned16(out) && aligned16(base),
             FK_ERR_ALIGNMENT, "%s: offsets / strides / 16-byte alignment", who);
  PushedParams p{};
  p.base = static_cast<uint8_t*>(base);
  p.nranks = nranks;
  p.ll_offset = ll_offset_bytes; p.sender_stride = sender_stride_bytes;
  p.residual = (uint16_t*)residual; p.residual_stride = residual_stride;
  p.weight = (const uint4*)weight; p.eps = eps;
  p.out = (uint16_t*)out; p.out_stride = out_stride;
  p.cols_vec = (int)(cols / 8);
  p.inv_cols = 1.0f / (float)cols;
  p.status = status;
  const int block = p.cols_vec >= 256 ? 256 : ((p.cols_vec + 31) / 32) * 32;
  const int vpt = (p.cols_vec + block - 1) / block;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (vpt <= 1) FK_LAUNCH((allreduce_pushed_kernel<1>), dim3((unsigned)rows), dim3(block), 0, s, p);
  else if (vpt <= 2) FK_LAUNCH((allreduce_pushed_kernel<2>), dim3((unsigned)rows), dim3(block), 0, s, p);
  else if (vpt <= 4) FK_LAUNCH((allreduce_pushed_kernel<4>), dim3((unsigned)rows), dim3(block), 0, s, p);
  else FK_LAUNCH((allreduce_pushed_kernel<8>), dim3((unsigned)rows), dim3(block), 0, s, p);
  count_launch();
  FK_CUDA_OK(cudaGetLastError());
  return FK_OK;
}

}  // extern "C"
