// HBM-bound row kernels of the decode step: KV-cache scatter, RMSNorm,
// fused residual-add + RMSNorm, NeoX RoPE (+ QKV split, per-head q/k norm and
// KV store in one pass), SiLU-and-multiply.
//
// All of them move each byte once with 16-byte accesses; none is GEMM-shaped,
// so there is no tensor-core work here.  Rounding points follow the reference
// CUDA kernels (cited per kernel) so outputs agree to the last bf16 bit up to
// the order of the fp32 row reduction.
#include "fk_common.cuh"
#include "fk_rowops.cuh"

namespace fk {

// ===========================================================================
// store_kvcache: cache.view(-1, row)[slot] = src[i]   (bit-exact copy)
// reference: fastkernels/tasks/baseline/L1/store_kvcache.py:16-35
// ===========================================================================
// TOK tokens per thread and pass: their slots and 16-byte pieces are all
// requested before the first store, so a thread keeps TOK loads in flight.
template <typename SlotT, int TOK>
__global__ void __launch_bounds__(256, 4) store_kvcache_vec_kernel(
    const uint4* __restrict__ key, const uint4* __restrict__ value,
    uint4* __restrict__ k_cache, uint4* __restrict__ v_cache,
    const SlotT* __restrict__ slots, int64_t num_tokens, int vec_per_row,
    int64_t key_stride_vec, int64_t value_stride_vec, int64_t num_slots,
    int32_t* status) {
  pdl_launch_dependents();
  pdl_wait();
  // grid.x covers the 16-byte columns of a token's K row followed by its V row,
  // grid.y strides over groups of TOK tokens: no per-element index division
  const int c2 = blockIdx.x * blockDim.x + threadIdx.x;
  if (c2 >= 2 * vec_per_row) return;
  const int which = c2 >= vec_per_row ? 1 : 0;
  const int c = c2 - which * vec_per_row;
  const uint4* src = which ? value : key;
  const int64_t src_stride = which ? value_stride_vec : key_stride_vec;
  uint4* dst = which ? v_cache : k_cache;
  for (int64_t t0 = (int64_t)blockIdx.y * TOK; t0 < num_tokens;
       t0 += (int64_t)gridDim.y * TOK) {
    int64_t slot[TOK];
    uint4 v[TOK];
#pragma unroll
    for (int i = 0; i < TOK; ++i)
      slot[i] = t0 + i < num_tokens ? (int64_t)slots[t0 + i] : -1;
#pragma unroll
    for (int i = 0; i < TOK; ++i)
      if (slot[i] >= 0 && slot[i] < num_slots) v[i] = __ldg(src + (t0 + i) * src_stride + c);
#pragma unroll
    for (int i = 0; i < TOK; ++i) {
      if (slot[i] < 0) continue;
      if (slot[i] >= num_slots) {
        if (status && c == 0) atomicOr(status, FK_DEV_BAD_SLOT);
        continue;
      }
      dst[slot[i] * vec_per_row + c] = v[i];
    }
  }
}

template <typename SlotT>
__global__ void store_kvcache_elem_kernel(
    const uint16_t* __restrict__ key, const uint16_t* __restrict__ value,
    uint16_t* __restrict__ k_cache, uint16_t* __restrict__ v_cache,
    const SlotT* __restrict__ slots, int64_t num_tokens, int64_t row_elems,
    int64_t key_stride, int64_t value_stride, int64_t num_slots,
    int32_t* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = num_tokens * row_elems;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
       idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t tok = idx / row_elems;
    const int64_t c = idx - tok * row_elems;
    const int64_t slot = (int64_t)slots[tok];
    if (slot < 0) continue;
    if (slot >= num_slots) {
      if (status && c == 0) atomicOr(status, FK_DEV_BAD_SLOT);
      continue;
    }
    k_cache[slot * row_elems + c] = key[tok * key_stride + c];
    v_cache[slot * row_elems + c] = value[tok * value_stride + c];
  }
}

// HND pool [num_blocks, Hkv, page, D]: slot -> (block = slot / page, offset =
// slot % page); head h of the token lands at ((block * Hkv + h) * page + offset) * D.
// reference: fastkernels/tasks/baseline/L1/store_kvcache.py:38-68
template <typename SlotT>
__global__ void store_kvcache_hnd_kernel(
    const uint16_t* __restrict__ key, const uint16_t* __restrict__ value,
    uint16_t* __restrict__ k_cache, uint16_t* __restrict__ v_cache,
    const SlotT* __restrict__ slots, int64_t num_tokens, int hkv, int d,
    int64_t key_stride, int64_t value_stride, int page, int64_t num_slots,
    int vec, int32_t* status) {
  pdl_launch_dependents();
  pdl_wait();
  // one work item = `vec` elements (8 when everything is 16-byte aligned, else 1)
  const int per_head = d / vec;
  const int64_t total = num_tokens * hkv * per_head * 2;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
       idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = idx;
    const int c = (int)(r % per_head); r /= per_head;
    const int h = (int)(r % hkv); r /= hkv;
    const int which = (int)(r & 1);
    const int64_t tok = r >> 1;
    const int64_t slot = (int64_t)slots[tok];
    if (slot < 0) continue;
    if (slot >= num_slots) {
      if (status && c == 0 && h == 0) atomicOr(status, FK_DEV_BAD_SLOT);
      continue;
    }
    const int64_t blk = slot / page, off = slot - blk * page;
    const int64_t dst = ((blk * hkv + h) * page + off) * d + (int64_t)c * vec;
    const uint16_t* src = (which ? value + tok * value_stride : key + tok * key_stride) +
                          (int64_t)h * d + (int64_t)c * vec;
    uint16_t* out = (which ? v_cache : k_cache) + dst;
    if (vec == 8)
      *reinterpret_cast<uint4*>(out) = __ldg(reinterpret_cast<const uint4*>(src));
    else
      *out = *src;
  }
}

// ===========================================================================
// RMSNorm.  reference: fastkernels/tasks/baseline/L1/rms_norm.cu:1251-1336
//   out = bf16(float(x) * rsqrt(mean(x^2) + eps) * float(w))   (one rounding)
// ===========================================================================
__device__ __forceinline__ float block_sum(float v, float* red) {
  // red: >= 33 floats of shared memory
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? red[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// One CTA per row, the row held in registers (VPT 16-byte vectors per thread).
template <int VPT, bool FUSED_ADD>
__global__ void __launch_bounds__(256) rmsnorm_row_kernel(
    uint4* __restrict__ x, int64_t x_stride_vec, uint4* __restrict__ res_or_out,
    int64_t ro_stride_vec, const uint4* __restrict__ weight, float eps,
    int vec_per_row, float inv_cols, int64_t rows) {
  __shared__ float red[33];
  pdl_launch_dependents();
  // the norm weights never change during a step: fetch them while the
  // predecessor kernel is still finishing
  uint4 wv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    wv[i] = c < vec_per_row ? __ldg(weight + c) : make_uint4(0, 0, 0, 0);
  }
  pdl_wait();
  // A CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ...: the loads of the
  // next row are issued before the reduction of the current one, so a CTA always
  // has a row in flight (one pass when the grid has a CTA per row, as at decode).
  // (rows of more than 8192 elements are not prefetched: four row buffers would
  // not fit the register file)
  constexpr bool PREFETCH = VPT <= 4;
  uint4 nx[VPT], nr[VPT];
  int64_t row = blockIdx.x;
  if (PREFETCH && row < rows) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < vec_per_row) {
        nx[i] = x[row * x_stride_vec + c];
        if (FUSED_ADD) nr[i] = res_or_out[row * ro_stride_vec + c];
      }
    }
  }
  for (; row < rows; row += gridDim.x) {
    uint4* xr = x + row * x_stride_vec;
    uint4* rr = res_or_out + row * ro_stride_vec;
    uint4 v[VPT];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < vec_per_row) {
        if (!PREFETCH) {
          nx[i] = xr[c];
          if (FUSED_ADD) nr[i] = rr[c];
        }
        v[i] = nx[i];
        if (FUSED_ADD) {
          // residual = bf16(x + residual): packed bf16 add, one rounding
          // (fastkernels/tasks/baseline/L1/rms_norm.cu:1371-1376)
          __nv_bfloat162* a = reinterpret_cast<__nv_bfloat162*>(&v[i]);
          const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&nr[i]);
#pragma unroll
          for (int j = 0; j < 4; ++j) a[j] = __hadd2(a[j], b[j]);
          rr[c] = v[i];
        }
        ss += sumsq8(v[i]);
      }
    }
    const int64_t next = row + gridDim.x;
    if (PREFETCH && next < rows) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < vec_per_row) {
          nx[i] = x[next * x_stride_vec + c];
          if (FUSED_ADD) nr[i] = res_or_out[next * ro_stride_vec + c];
        }
      }
    }
    const float tot = block_sum(ss, red);
    const float rs = rsqrtf(tot * inv_cols + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < vec_per_row) {
        const uint4 o = scale8(v[i], wv[i], rs);
        if (FUSED_ADD)
          xr[c] = o;
        else
          rr[c] = o;
      }
    }
  }
}

// Short rows (per-head q/k norm): LPR lanes per row, rows addressed as
// (outer, inner) with separate strides so a [N, H, D] view of a packed qkv
// buffer needs no copy.
template <int LPR>
__global__ void __launch_bounds__(256) rmsnorm_short_kernel(
    const uint16_t* __restrict__ x, int64_t xs_outer, int64_t xs_inner,
    uint16_t* __restrict__ out, int64_t os_outer, int64_t os_inner,
    const uint4* __restrict__ weight, float eps, int64_t rows, int64_t inner,
    float inv_cols) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t gid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t row = gid / LPR;
  const int j = (int)(gid % LPR);
  const bool live = row < rows;
  uint4 v = make_uint4(0, 0, 0, 0);
  int64_t o = 0, i = 0;
  if (live) {
    o = row / inner;
    i = row - o * inner;
    v = *reinterpret_cast<const uint4*>(x + o * xs_outer + i * xs_inner + j * 8);
  }
  float ss = sumsq8(v);
#pragma unroll
  for (int off = LPR / 2; off > 0; off >>= 1)
    ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if (live) {
    const float rs = rsqrtf(ss * inv_cols + eps);
    *reinterpret_cast<uint4*>(out + o * os_outer + i * os_inner + j * 8) =
        scale8(v, __ldg(weight + j), rs);
  }
}

// Any shape / alignment: scalar two-pass, one CTA per row.
template <bool FUSED_ADD>
__global__ void __launch_bounds__(256) rmsnorm_generic_kernel(
    __nv_bfloat16* __restrict__ x, int64_t xs_outer, int64_t xs_inner,
    __nv_bfloat16* __restrict__ ro, int64_t ros_outer, int64_t ros_inner,
    const __nv_bfloat16* __restrict__ weight, float eps, int64_t inner,
    int64_t cols) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int64_t row = blockIdx.x;
  const int64_t o = row / inner, i = row - o * inner;
  __nv_bfloat16* xr = x + o * xs_outer + i * xs_inner;
  __nv_bfloat16* rr = ro + o * ros_outer + i * ros_inner;
  float ss = 0.f;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    __nv_bfloat16 v = xr[c];
    if (FUSED_ADD) {
      v = __hadd(v, rr[c]);
      rr[c] = v;
    }
    const float f = __bfloat162float(v);
    ss += f * f;
  }
  const float tot = block_sum(ss, red);
  const float rs = rsqrtf(tot / (float)cols + eps);
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    const float f = __bfloat162float(FUSED_ADD ? rr[c] : xr[c]);
    const __nv_bfloat16 r =
        __float2bfloat16_rn(f * rs * __bfloat162float(weight[c]));
    if (FUSED_ADD)
      xr[c] = r;
    else
      rr[c] = r;
  }
}

// ===========================================================================
// NeoX RoPE (+ optional per-head RMSNorm, + optional KV-cache store).
// references: fastkernels/tasks/baseline/L1/rotary_emb.cu:332-358 (rotation),
// fastkernels/tasks/baseline/L2/attention.py:113-144 (split, q/k norm order),
// fastkernels/tasks/baseline/L1/store_kvcache.py:16-35 (store).
// One head of one token is handled by LPH = D/16 lanes; lane j owns elements
// [8j, 8j+8) of the first half and the matching 8 of the second half.
// ===========================================================================
// Grid: x covers the (head, lane) pairs of ONE token, y strides over groups of T
// tokens, so no thread divides a flat index (see rope_thread).
template <int LPH, bool NORM, int T>
__global__ void __launch_bounds__(128) rope_heads_kernel(RopeArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  rope_thread<LPH, NORM, T, false>(a, blockIdx.x * blockDim.x + threadIdx.x,
                                   (int64_t)blockIdx.y * T, (int64_t)gridDim.y * T);
}

// ===========================================================================
// SiLU-and-multiply.  reference:
// fastkernels/tasks/baseline/L1/silu_and_mul.cu:715-740, 823-830
//   out = bf16(float(bf16(g / (1 + exp(-g)))) * float(u))
// ===========================================================================
// grid.x covers the 16-byte columns of a row, grid.y strides over groups of R
// rows: no per-element index division (a 64-bit divide costs more than the SiLU
// itself), and a thread has the 2 R loads of its group in flight before the
// first exponential.
template <int R>
__global__ void __launch_bounds__(256) silu_and_mul_vec_kernel(
    const uint4* __restrict__ x, int64_t x_stride_vec, uint4* __restrict__ out,
    int64_t out_stride_vec, int64_t rows, int d_vec) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= d_vec) return;
  for (int64_t r0 = (int64_t)blockIdx.y * R; r0 < rows; r0 += (int64_t)gridDim.y * R) {
    uint4 g[R], u[R];
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (r0 + i < rows) {
        const uint4* xr = x + (r0 + i) * x_stride_vec;
        g[i] = __ldg(xr + c);
        u[i] = __ldg(xr + d_vec + c);
      }
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (r0 + i < rows) {
        uint4 o;
        o.x = silu_mul2(g[i].x, u[i].x);
        o.y = silu_mul2(g[i].y, u[i].y);
        o.z = silu_mul2(g[i].z, u[i].z);
        o.w = silu_mul2(g[i].w, u[i].w);
        out[(r0 + i) * out_stride_vec + c] = o;
      }
  }
}

__global__ void __launch_bounds__(256) silu_and_mul_elem_kernel(
    const __nv_bfloat16* __restrict__ x, int64_t x_stride,
    __nv_bfloat16* __restrict__ out, int64_t out_stride, int64_t rows,
    int64_t d) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = rows * d;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
       idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / d, c = idx - r * d;
    const float g = __bfloat162float(x[r * x_stride + c]);
    const float u = __bfloat162float(x[r * x_stride + d + c]);
    const float a = round_bf16(silu_f32(g));
    out[r * out_stride + c] = __float2bfloat16_rn(a * u);
  }
}

// ===========================================================================
// Greedy sampling: per-row maximum and its (lowest) index over bf16 logits.
// reference: lm_logits[:bs].max(dim=-1) in the captured decode graph
// (fastkernels/infra/engine.py:6994-6996).  Ties go to the lowest index.
// ===========================================================================
__device__ __forceinline__ void amax_take(float& bv, int64_t& bi, float v,
                                          int64_t i) {
  if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}

__global__ void __launch_bounds__(1024) argmax_rows_kernel(
    const uint16_t* __restrict__ x, int64_t x_stride, int64_t cols,
    float* __restrict__ out_val, int64_t* __restrict__ out_idx) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sv[32];
  __shared__ int64_t si[32];
  const uint16_t* row = x + (int64_t)blockIdx.x * x_stride;
  float bv = -INFINITY;
  int64_t bi = 0x7fffffffffffffffll;
  const bool vec = (cols % 8 == 0) && (x_stride % 8 == 0) &&
                   ((reinterpret_cast<uintptr_t>(x) & 15u) == 0);
  if (vec) {
    const uint4* r4 = reinterpret_cast<const uint4*>(row);
    for (int64_t c = threadIdx.x; c < cols / 8; c += blockDim.x) {
      const uint4 v = __ldg(r4 + c);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        amax_take(bv, bi, bf16lo(w[j]), c * 8 + 2 * j);
        amax_take(bv, bi, bf16hi(w[j]), c * 8 + 2 * j + 1);
      }
    }
  } else {
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x)
      amax_take(bv, bi, bf16_bits_to_float(row[c]), c);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int64_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
    amax_take(bv, bi, ov, oi);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    bv = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffffffffffffll;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int64_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
      amax_take(bv, bi, ov, oi);
    }
    if (lane == 0) {
      if (bi == 0x7fffffffffffffffll) bi = 0;  // empty or all-NaN row
      if (out_val) out_val[blockIdx.x] = bv;
      out_idx[blockIdx.x] = bi;
    }
  }
}

__global__ void __launch_bounds__(256) fill_u32_kernel(uint4* __restrict__ p4,
                                                       int64_t n4, uint32_t* tail,
                                                       int ntail, uint32_t v) {
  pdl_launch_dependents();
  pdl_wait();
  const uint4 vv = make_uint4(v, v, v, v);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4;
       i += (int64_t)gridDim.x * blockDim.x)
    p4[i] = vv;
  if (blockIdx.x == 0 && threadIdx.x < ntail) tail[threadIdx.x] = v;
}

// XOR of all words: a pure read stream (eight independent 16-byte loads in flight
// per thread), the read-only counterpart of the fill above.
__global__ void __launch_bounds__(512) xor_u32_kernel(const uint4* __restrict__ p4, int64_t n4,
                                                      uint32_t* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  uint32_t acc = 0;
  for (; i + 7 * stride < n4; i += 8 * stride) {
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = ld16<true>(p4 + i + j * stride);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc ^= v[j].x ^ v[j].y ^ v[j].z ^ v[j].w;
  }
  for (; i < n4; i += stride) {
    const uint4 v = ld16<true>(p4 + i);
    acc ^= v.x ^ v.y ^ v.z ^ v.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc ^= __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0 && acc != 0) atomicXor(out, acc);
}

// Row kernels whose CTAs walk several rows: one CTA per row while all of them are
// resident at once (`per_sm` CTAs per SM: 256 threads x the registers of the
// VPT variant); beyond that every CTA takes the same number of rows, so no SM
// is left with one row more than the others at the end.
static inline unsigned row_grid(int64_t rows, int vpt) {
  const int per_sm = vpt <= 1 ? 4 : vpt <= 2 ? 3 : 2;
  const int64_t cap = (int64_t)per_sm * sm_count();
  if (rows <= cap) return (unsigned)(rows < 1 ? 1 : rows);
  const int64_t per_cta = (rows + cap - 1) / cap;
  return (unsigned)((rows + per_cta - 1) / per_cta);
}

static inline int grid_for(int64_t threads, int block) {
  int64_t g = (threads + block - 1) / block;
  const int64_t cap = (int64_t)sm_count() * 32;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace fk

using namespace fk;

extern "C" {

int fk_store_kvcache(const void* key, const void* value, void* k_cache,
                     void* v_cache, const void* slot_mapping,
                     int slot_is_int64, int64_t num_tokens, int64_t row_elems,
                     int64_t key_stride, int64_t value_stride,
                     int64_t num_slots, int32_t* status, fk_stream_t stream) {
  FK_REQUIRE(num_tokens >= 0 && row_elems > 0 && num_slots >= 0,
             FK_ERR_INVALID_ARG, "fk_store_kvcache: negative size");
  if (num_tokens == 0) return FK_OK;
  FK_REQUIRE(key && value && k_cache && v_cache && slot_mapping,
             FK_ERR_INVALID_ARG, "fk_store_kvcache: null pointer");
  FK_REQUIRE(key_stride >= row_elems && value_stride >= row_elems,
             FK_ERR_INVALID_ARG,
             "fk_store_kvcache: row stride smaller than the row");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool vec = (row_elems % 8 == 0) && (key_stride % 8 == 0) &&
                   (value_stride % 8 == 0) && aligned16(key) &&
                   aligned16(value) && aligned16(k_cache) && aligned16(v_cache);
  if (vec) {
    const int vpr = (int)(row_elems / 8);
    const int gx = (2 * vpr + 255) / 256;
    // eight tokens per thread once there are enough tokens to fill the GPU that
    // way; a block row per token (group), at most one resident wave (the slot ->
    // row -> store chain of a pass is two dependent loads long: passes are few)
    const bool many = num_tokens * gx >= 2ll * sm_count() * 8;
    const int tok_per = many ? 8 : 1;
    int64_t gy = (num_tokens + tok_per - 1) / tok_per;
    const int64_t cap = (4ll * sm_count() + gx - 1) / gx;
    if (gy > cap) gy = cap;
    if (gy > 65535) gy = 65535;
    const dim3 grid((unsigned)gx, (unsigned)gy);
#define FK_STORE(SLOT_T, TOK)                                                        \
  FK_LAUNCH((store_kvcache_vec_kernel<SLOT_T, TOK>), grid, dim3(256), 0, s,          \
            (const uint4*)key, (const uint4*)value, (uint4*)k_cache, (uint4*)v_cache, \
            (const SLOT_T*)slot_mapping, num_tokens, vpr, key_stride / 8,            \
            value_stride / 8, num_slots, status)
    if (slot_is_int64) {
      if (many) FK_STORE(int64_t, 8); else FK_STORE(int64_t, 1);
    } else {
      if (many) FK_STORE(int32_t, 8); else FK_STORE(int32_t, 1);
    }
#undef FK_STORE
  } else {
    const int grid = grid_for(num_tokens * row_elems, 256);
    if (slot_is_int64)
      FK_LAUNCH((store_kvcache_elem_kernel<int64_t>), dim3(grid), dim3(256), 0, s, 
          (const uint16_t*)key, (const uint16_t*)value, (uint16_t*)k_cache,
          (uint16_t*)v_cache, (const int64_t*)slot_mapping, num_tokens,
          row_elems, key_stride, value_stride, num_slots, status);
    else
      FK_LAUNCH((store_kvcache_elem_kernel<int32_t>), dim3(grid), dim3(256), 0, s, 
          (const uint16_t*)key, (const uint16_t*)value, (uint16_t*)k_cache,
          (uint16_t*)v_cache, (const int32_t*)slot_mapping, num_tokens,
          row_elems, key_stride, value_stride, num_slots, status);
  }
  count_launch();
  FK_CUDA_OK(cudaGetLastError());
  return FK_OK;
}

int fk_store_kvcache_hnd(const void* key, const void* value, void* k_cache,
                         void* v_cache, const void* slot_mapping,
                         int slot_is_int64, int64_t num_tokens, int num_kv_heads,
                         int head_dim, int64_t key_stride, int64_t value_stride,
                         int page_size, int64_t num_blocks, int32_t* status,
                         fk_stream_t stream) {
  FK_REQUIRE(num_tokens >= 0 && num_kv_heads > 0 && head_dim > 0 && page_size > 0 &&
                 num_blocks >= 0,
             FK_ERR_INVALID_ARG, "fk_store_kvcache_hnd: bad sizes");
  if (num_tokens == 0) return FK_OK;
  FK_REQUIRE(key && value && k_cache && v_cache && slot_mapping, FK_ERR_INVALID_ARG,
             "fk_store_kvcache_hnd: null pointer");
  const int64_t row = (int64_t)num_kv_heads * head_dim;
  FK_REQUIRE(key_stride >= row && value_stride >= row, FK_ERR_INVALID_ARG,
             "fk_store_kvcache_hnd: row stride smaller than the row");
  const bool al = head_dim % 8 == 0 && key_stride % 8 == 0 && value_stride % 8 == 0 &&
                  aligned16(key) && aligned16(value) && aligned16(k_cache) &&
                  aligned16(v_cache);
  const int vec = al ? 8 : 1;
  const int grid = grid_for(num_tokens * num_kv_heads * (head_dim / vec) * 2, 256);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t num_slots = num_blocks * page_size;
  if (slot_is_int64)
    FK_LAUNCH(store_kvcache_hnd_kernel<int64_t>, dim3(grid), dim3(256), 0, s,
              (const uint16_t*)key, (const uint16_t*)value, (uint16_t*)k_cache,
              (uint16_t*)v_cache, (const int64_t*)slot_mapping, num_tokens, num_kv_heads,
              head_dim, key_stride, value_stride, page_size, num_slots, vec, status);
  else
    FK_LAUNCH(store_kvcache_hnd_kernel<int32_t>, dim3(grid), dim3(256), 0, s,
              (const uint16_t*)key, (const uint16_t*)value, (uint16_t*)k_cache,
              (uint16_t*)v_cache, (const int32_t*)slot_mapping, num_tokens, num_kv_heads,
              head_dim, key_stride, value_stride, page_size, num_slots, vec, status);
  count_launch();
  FK_CUDA_OK(cudaGetLastError());
  return FK_OK;
}

int fk_rmsnorm(const void* x, int64_t x_stride_outer, int64_t x_stride_inner,
               int64_t inner, void* out, int64_t out_stride_outer,
               int64_t out_stride_inner, const void* weight, float eps,
               int64_t outer, int64_t cols, fk_stream_t stream) {
  FK_REQUIRE(outer >= 0 && inner > 0 && cols > 0, FK_ERR_INVALID_ARG,
             "fk_rmsnorm: bad sizes");
  const int64_t rows = outer * inner;
  if (rows == 0) return FK_OK;
  FK_REQUIRE(x && out && weight, FK_ERR_INVALID_ARG, "fk_rmsnorm: null pointer");
  FK_REQUIRE(rows < (1ll << 31), FK_ERR_UNSUPPORTED, "fk_rmsnorm: too many rows");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool al = aligned16(x) && aligned16(out) && aligned16(weight) &&
                  cols % 8 == 0 && x_stride_outer % 8 == 0 &&
                  x_stride_inner % 8 == 0 && out_stride_outer % 8 == 0 &&
                  out_stride_inner % 8 == 0;
  const int vpr = (int)(cols / 8);
  const float inv = 1.0f / (float)cols;
  if (al && (vpr == 4 || vpr == 8 || vpr == 16 || vpr == 32)) {
    const int64_t threads = rows * vpr;
    const int grid = (int)((threads + 255) / 256);
#define FK_SHORT(L)                                                          \
  FK_LAUNCH((rmsnorm_short_kernel<L>), dim3(grid), dim3(256), 0, s,                               \
      (const uint16_t*)x, x_stride_outer, x_stride_inner, (uint16_t*)out,    \
      out_stride_outer, out_stride_inner, (const uint4*)weight, eps, rows,   \
      inner, inv)
    if (vpr == 4) FK_SHORT(4);
    else if (vpr == 8) FK_SHORT(8);
    else if (vpr == 16) FK_SHORT(16);
    else FK_SHORT(32);
#undef FK_SHORT
  } else if (al && inner == 1 && vpr <= 256 * 8) {
    const int block = vpr >= 256 ? 256 : ((vpr + 31) / 32) * 32;
    const int vpt = (vpr + block - 1) / block;
#define FK_ROW(V)                                                            \
  FK_LAUNCH((rmsnorm_row_kernel<V, false>), dim3(row_grid(rows, V)), dim3(block), 0, s,         \
      (uint4*)const_cast<void*>(x), x_stride_outer / 8, (uint4*)out,         \
      out_stride_outer / 8, (const uint4*)weight, eps, vpr, inv, rows)
    if (vpt <= 1) FK_ROW(1);
    else if (vpt <= 2) FK_ROW(2);
    else if (vpt <= 4) FK_ROW(4);
    else FK_ROW(8);
#undef FK_ROW
  } else {
    FK_LAUNCH((rmsnorm_generic_kernel<false>), dim3((int)rows), dim3(256), 0, s, 
        (__nv_bfloat16*)const_cast<void*>(x), x_stride_outer, x_stride_inner,
        (__nv_bfloat16*)out, out_stride_outer, out_stride_inner,
        (const __nv_bfloat16*)weight, eps, inner, cols);
  }
  count_launch();
  FK_CUDA_OK(cudaGetLastError());
  return FK_OK;
}

int fk_fused_add_rmsnorm(void* x, int64_t x_stride, void* residual,
                         int64_t residual_stride, const void* weight,
                         float eps, int64_t rows, int64_t cols,
                         fk_stream_t stream) {
  FK_REQUIRE(rows >= 0 && cols > 0, FK_ERR_INVALID_ARG,
             "fk_fused_add_rmsnorm: bad sizes");
  if (rows == 0) return FK_OK;
  FK_REQUIRE(x && residual && weight, FK_ERR_INVALID_ARG,
             "fk_fused_add_rmsnorm: null pointer");
  FK_REQUIRE(rows < (1ll << 31), FK_ERR_UNSUPPORTED,
             "fk_fused_add_rmsnorm: too many rows");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool al = aligned16(x) && aligned16(residual) && aligned16(weight) &&
                  cols % 8 == 0 && x_stride % 8 == 0 && residual_stride % 8 == 0;
  const int vpr = (int)(cols / 8);
  if (al && vpr <= 256 * 8) {
    const int block = vpr >= 256 ? 256 : ((vpr + 31) / 32) * 32;
    const int vpt = (vpr + block - 1) / block;
    const float inv = 1.0f / (float)cols;
#define FK_ROW(V)                                                          \
  FK_LAUNCH((rmsnorm_row_kernel<V, true>), dim3(row_grid(rows, V)), dim3(block), 0, s,          \
      (uint4*)x, x_stride / 8, (uint4*)residual, residual_stride / 8,      \
      (const uint4*)weight, eps, vpr, inv, rows)
    if (vpt <= 1) FK_ROW(1);
    else if (vpt <= 2) FK_ROW(2);
    else if (vpt <= 4) FK_ROW(4);
    else FK_ROW(8);
#undef FK_ROW
  } else {
    FK_LAUNCH((rmsnorm_generic_kernel<true>), dim3((int)rows), dim3(256), 0, s, 
        (__nv_bfloat16*)x, x_stride, 0, (__nv_bfloat16*)residual,
        residual_stride, 0, (const __nv_bfloat16*)weight, eps, 1, cols);
  }
  count_launch();
  FK_CUDA_OK(cudaGetLastError());
  return FK_OK;
}

static int launch_rope(const RopeArgs& a, int head_dim, cudaStream_t s) {
  const int heads = a.hq + a.hkv + (a.v ? a.hkv : 0);
  const int lph = head_dim / 16;
  FK_REQUIRE(a.num_tokens < (1ll << 31), FK_ERR_UNSUPPORTED, "rope: too many tokens");
  // x: the (head, lane) pairs of one token in blocks of 128 threads; y: tokens, two
  // per thread once that still leaves several blocks per SM
  const unsigned gx = (unsigned)((heads * lph + 127) / 128);
  const bool many = a.num_tokens * gx >= 16ll * sm_count();
  const int64_t groups = many ? (a.num_tokens + 1) / 2 : a.num_tokens;
  const unsigned gy = (unsigned)(groups < 65535 ? groups : 65535);
  const dim3 grid(gx, gy);
  const bool norm = a.q_norm_w != nullptr || a.k_norm_w != nullptr;
#define FK_ROPE(L)                                                                     \
  do {                                                                                 \
    if (norm) {                                                                        \
      if (many) FK_LAUNCH((rope_heads_kernel<L, true, 2>), grid, dim3(128), 0, s, a);  \
      else FK_LAUNCH((rope_heads_kernel<L, true, 1>), grid, dim3(128), 0, s, a);       \
    } else {                                                                           \
      if (many) FK_LAUNCH((rope_heads_kernel<L, false, 2>), grid, dim3(128), 0, s, a); \
      else FK_LAUNCH((rope_heads_kernel<L, false, 1>), grid, dim3(128), 0, s, a);      \
    }                                                                                  \
  } while (0)
  switch (lph) {
    case 2: FK_ROPE(2); break;
    case 4: FK_ROPE(4); break;
    case 8: FK_ROPE(8); break;
    case 16: FK_ROPE(16); break;
    default:
      set_error("rope: head_dim %d unsupported (32, 64, 128, 256)", head_dim);
      return FK_ERR_UNSUPPORTED;
  }
#undef FK_ROPE
  count_launch();
  FK_CUDA_OK(cudaGetLastError());
  return FK_OK;
}

int fk_rope_neox(const int64_t* positions, void* query, int64_t q_stride,
                 int num_q_heads, void* key, int64_t k_stride,
                 int num_kv_heads, int head_dim, const void* cos_sin_cache,
                 int cache_is_fp32, int64_t max_position, int64_t num_tokens,
                 int32_t* status, fk_stream_t stream) {
  FK_REQUIRE(num_tokens >= 0 && num_q_heads >= 0 && num_kv_heads >= 0,
             FK_ERR_INVALID_ARG, "fk_rope_neox: negative size");
  if (num_tokens == 0 || num_q_heads + num_kv_heads == 0) return FK_OK;
  FK_REQUIRE(positions && cos_sin_cache && (query || num_q_heads == 0) &&
                 (key || num_kv_heads == 0),
             FK_ERR_INVALID_ARG, "fk_rope_neox: null pointer");
  FK_REQUIRE(aligned16(query) && aligned16(key) && aligned16(cos_sin_cache) &&
                 q_stride % 8 == 0 && k_stride % 8 == 0,
             FK_ERR_ALIGNMENT, "fk_rope_neox: 16-byte alignment required");
  RopeArgs a{};
  a.q = (uint16_t*)query; a.q_stride = q_stride; a.hq = num_q_heads;
  a.k = (uint16_t*)key; a.k_stride = k_stride; a.hkv = num_kv_heads;
  a.v = nullptr; a.v_stride = 0;
  a.positions = positions;
  a.cache = cos_sin_cache; a.cache_is_fp32 = cache_is_fp32;
  a.max_position = max_position;
  a.q_norm_w = nullptr; a.k_norm_w = nullptr; a.eps = 0.f;
  a.k_cache = nullptr; a.v_cache = nullptr; a.slots = nullptr; a.num_slots = 0;
  a.page = 1; a.hnd = 0;
  a.num_tokens = num_tokens; a.status = status;
  return launch_rope(a, head_dim, static_cast<cudaStream_t>(stream));
}

int fk_qkv_rope_store(void* qkv, int64_t qkv_stride, int num_q_heads,
                      int num_kv_heads, int head_dim,
                      const int64_t* positions, const void* cos_sin_cache,
                      int cache_is_fp32, int64_t max_position,
                      const void* q_norm_weight, const void* k_norm_weight,
                      float norm_eps, void* k_cache, void* v_cache,
                      const int32_t* slot_mapping, int64_t num_slots,
                      int block_size, int kv_layout, int64_t num_tokens,
                      int32_t* status, fk_stream_t stream) {
  FK_REQUIRE(num_tokens >= 0 && num_q_heads > 0 && num_kv_heads > 0,
             FK_ERR_INVALID_ARG, "fk_qkv_rope_store: bad sizes");
  FK_REQUIRE((kv_layout == 0 || kv_layout == 1) && (kv_layout == 0 || block_size > 0),
             FK_ERR_INVALID_ARG, "fk_qkv_rope_store: bad cache layout");
  if (num_tokens == 0) return FK_OK;
  FK_REQUIRE(qkv && positions && cos_sin_cache, FK_ERR_INVALID_ARG,
             "fk_qkv_rope_store: null pointer");
  FK_REQUIRE((k_cache == nullptr) == (v_cache == nullptr) &&
                 (k_cache == nullptr || slot_mapping != nullptr),
             FK_ERR_INVALID_ARG,
             "fk_qkv_rope_store: k_cache, v_cache and slot_mapping go together");
  FK_REQUIRE(qkv_stride >= (int64_t)(num_q_heads + 2 * num_kv_heads) * head_dim,
             FK_ERR_INVALID_ARG, "fk_qkv_rope_store: row stride too small");
  FK_REQUIRE(aligned16(qkv) && aligned16(cos_sin_cache) && aligned16(k_cache) &&
                 aligned16(v_cache) && aligned16(q_norm_weight) &&
                 aligned16(k_norm_weight) && qkv_stride % 8 == 0,
             FK_ERR_ALIGNMENT, "fk_qkv_rope_store: 16-byte alignment required");
  RopeArgs a{};
  uint16_t* base = (uint16_t*)qkv;
  a.q = base; a.q_stride = qkv_stride; a.hq = num_q_heads;
  a.k = base + (int64_t)num_q_heads * head_dim; a.k_stride = qkv_stride;
  a.hkv = num_kv_heads;
  a.v = base + (int64_t)(num_q_heads + num_kv_heads) * head_dim;
  a.v_stride = qkv_stride;
  a.positions = positions;
  a.cache = cos_sin_cache; a.cache_is_fp32 = cache_is_fp32;
  a.max_position = max_position;
  a.q_norm_w = (const uint4*)q_norm_weight;
  a.k_norm_w = (const uint4*)k_norm_weight;
  a.eps = norm_eps;
  a.k_cache = (uint16_t*)k_cache; a.v_cache = (uint16_t*)v_cache;
  a.slots = slot_mapping; a.num_slots = num_slots;
  a.page = block_size > 0 ? block_size : 1; a.hnd = kv_layout;
  a.num_tokens = num_tokens; a.status = status;
  if (k_cache == nullptr) a.v = nullptr;  // nothing to do for v without a store
  return launch_rope(a, head_dim, static_cast<cudaStream_t>(stream));
}

int fk_silu_and_mul(const void* x, int64_t x_stride, void* out,
                    int64_t out_stride, int64_t rows, int64_t d,
                    fk_stream_t stream) {
  FK_REQUIRE(rows >= 0 && d > 0, FK_ERR_INVALID_ARG, "fk_silu_and_mul: bad sizes");
  if (rows == 0) return FK_OK;
  FK_REQUIRE(x && out, FK_ERR_INVALID_ARG, "fk_silu_and_mul: null pointer");
  FK_REQUIRE(x_stride >= 2 * d && out_stride >= d, FK_ERR_INVALID_ARG,
             "fk_silu_and_mul: row stride smaller than the row");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (d % 8 == 0 && x_stride % 8 == 0 && out_stride % 8 == 0 && aligned16(x) &&
      aligned16(out)) {
    const int gx = ((int)(d / 8) + 255) / 256;
    // four rows per thread once that still leaves several blocks per SM, else a
    // block row per matrix row; at most ~16 blocks per SM, the rest by striding
    const bool many = rows * gx >= 8ll * sm_count() * 4;
    int64_t gy = many ? (rows + 3) / 4 : rows;
    const int64_t cap = (16ll * sm_count() + gx - 1) / gx;
    if (gy > cap) gy = cap;
    if (gy > 65535) gy = 65535;
    if (many)
      FK_LAUNCH((silu_and_mul_vec_kernel<4>), dim3((unsigned)gx, (unsigned)gy), dim3(256), 0, s,
                (const uint4*)x, x_stride / 8, (uint4*)out, out_stride / 8, rows, (int)(d / 8));
    else
      FK_LAUNCH((silu_and_mul_vec_kernel<1>), dim3((unsigned)gx, (unsigned)gy), dim3(256), 0, s, 
        (const uint4*)x, x_stride / 8, (uint4*)out, out_stride / 8, rows,
        (int)(d / 8));
  } else {
    const int grid = grid_for(rows * d, 256);
    FK_LAUNCH((silu_and_mul_elem_kernel), dim3(grid), dim3(256), 0, s, 
        (const __nv_bfloat16*)x, x_stride, (__nv_bfloat16*)out, out_stride, rows,
        d);
  }
  count_launch();
  FK_CUDA_OK(cudaGetLastError());
  return FK_OK;
}

int fk_argmax_bf16(const void* x, int64_t x_stride, int64_t rows, int64_t cols,
                   float* out_val, int64_t* out_idx, fk_stream_t stream) {
  FK_REQUIRE(rows >= 0 && cols > 0, FK_ERR_INVALID_ARG, "fk_argmax_bf16: bad sizes");
  if (rows == 0) return FK_OK;
  FK_REQUIRE(x && out_idx, FK_ERR_INVALID_ARG, "fk_argmax_bf16: null pointer");
  FK_REQUIRE(x_stride >= cols && rows < (1ll << 31), FK_ERR_INVALID_ARG,
             "fk_argmax_bf16: bad stride or row count");
  FK_LAUNCH((argmax_rows_kernel), dim3((int)rows), dim3(1024), 0, static_cast<cudaStream_t>(stream), 
      (const uint16_t*)x, x_stride, cols, out_val, out_idx);
  count_launch();
  FK_CUDA_OK(cudaGetLastError());
  return FK_OK;
}

int fk_fill_u32(void* dst, int64_t count, uint32_t value, fk_stream_t stream) {
  FK_REQUIRE(count >= 0, FK_ERR_INVALID_ARG, "fk_fill_u32: negative count");
  if (count == 0) return FK_OK;
  FK_REQUIRE(dst != nullptr, FK_ERR_INVALID_ARG, "fk_fill_u32: null pointer");
  FK_REQUIRE(aligned16(dst), FK_ERR_ALIGNMENT, "fk_fill_u32: 16-byte alignment required");
  const int64_t n4 = count / 4;
  const int grid = grid_for(n4 > 0 ? n4 : 1, 256);
  FK_LAUNCH((fill_u32_kernel), dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), 
      (uint4*)dst, n4, (uint32_t*)dst + n4 * 4, (int)(count - n4 * 4), value);
  count_launch();
  FK_CUDA_OK(cudaGetLastError());
  return FK_OK;
}

int fk_xor_u32(const void* src, int64_t count, uint32_t* out, fk_stream_t stream) {
  FK_REQUIRE(count >= 0 && count % 4 == 0, FK_ERR_INVALID_ARG,
             "fk_xor_u32: count must be a non-negative multiple of 4");
  if (count == 0) return FK_OK;
  FK_REQUIRE(src != nullptr && out != nullptr, FK_ERR_INVALID_ARG, "fk_xor_u32: null pointer");
  FK_REQUIRE(aligned16(src), FK_ERR_ALIGNMENT, "fk_xor_u32: 16-byte alignment required");
  const int64_t n4 = count / 4;
  int64_t grid = (n4 + 511) / 512;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (grid > cap) grid = cap;
  FK_LAUNCH((xor_u32_kernel), dim3((unsigned)grid), dim3(512), 0,
            static_cast<cudaStream_t>(stream), (const uint4*)src, n4, out);
  count_launch();
  FK_CUDA_OK(cudaGetLastError());
  return FK_OK;
}

}  // extern "C"
