// Row operations shared by the stand-alone row kernels and by the phases of the
// persistent decode-block kernel: RMSNorm pieces and the fused split + per-head
// q/k RMSNorm + NeoX RoPE + KV store.
#pragma once

#include "fk_common.cuh"

namespace fk {

#ifdef __CUDACC__

// 16-byte load; CG bypasses L1 (data written by other SMs earlier in the SAME
// kernel: L1 is not coherent across SMs)
template <bool CG>
__device__ __forceinline__ uint4 ld16(const void* p) {
  if (CG) return __ldcg(reinterpret_cast<const uint4*>(p));
  return *reinterpret_cast<const uint4*>(p);
}

__device__ __forceinline__ float sumsq8(const uint4& v) {
  float s = 0.f, t;
  t = bf16lo(v.x); s += t * t; t = bf16hi(v.x); s += t * t;
  t = bf16lo(v.y); s += t * t; t = bf16hi(v.y); s += t * t;
  t = bf16lo(v.z); s += t * t; t = bf16hi(v.z); s += t * t;
  t = bf16lo(v.w); s += t * t; t = bf16hi(v.w); s += t * t;
  return s;
}
__device__ __forceinline__ uint32_t scale2(uint32_t x, uint32_t w, float rs) {
  return pack_bf16(bf16lo(x) * rs * bf16lo(w), bf16hi(x) * rs * bf16hi(w));
}
__device__ __forceinline__ uint4 scale8(const uint4& x, const uint4& w,
                                        float rs) {
  uint4 o;
  o.x = scale2(x.x, w.x, rs);
  o.y = scale2(x.y, w.y, rs);
  o.z = scale2(x.z, w.z, rs);
  o.w = scale2(x.w, w.w, rs);
  return o;
}

#endif  // __CUDACC__

struct RopeArgs {
  uint16_t* q; int64_t q_stride; int hq;
  uint16_t* k; int64_t k_stride; int hkv;
  const uint16_t* v; int64_t v_stride;   // null: no value path
  const int64_t* positions;
  const void* cache; int cache_is_fp32; int64_t max_position;
  const uint4* q_norm_w; const uint4* k_norm_w; float eps;
  uint16_t* k_cache; uint16_t* v_cache;  // null: no store
  const int32_t* slots; int64_t num_slots;
  int page; int hnd;                     // cache layout (hnd: [blocks, Hkv, page, D])
  int64_t num_tokens;
  int32_t* status;
};

#ifdef __CUDACC__
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = bf16lo(v.x); f[1] = bf16hi(v.x); f[2] = bf16lo(v.y); f[3] = bf16hi(v.y);
  f[4] = bf16lo(v.z); f[5] = bf16hi(v.z); f[6] = bf16lo(v.w); f[7] = bf16hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]);
  o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
  return o;
}
__device__ __forceinline__ void load_cs8(const void* cache, int is_fp32,
                                         int64_t elem_off, float (&f)[8]) {
  if (is_fp32) {
    const float4* p =
        reinterpret_cast<const float4*>(static_cast<const float*>(cache) + elem_off);
    const float4 a = __ldg(p), b = __ldg(p + 1);
    // the reference casts the fp32 cache to the activation dtype before use
    // (fastkernels/tasks/baseline/L1/rotary_emb.py:171-173)
    f[0] = round_bf16(a.x); f[1] = round_bf16(a.y); f[2] = round_bf16(a.z);
    f[3] = round_bf16(a.w); f[4] = round_bf16(b.x); f[5] = round_bf16(b.y);
    f[6] = round_bf16(b.z); f[7] = round_bf16(b.w);
  } else {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(
        static_cast<const uint16_t*>(cache) + elem_off));
    unpack8(v, f);
  }
}

// One thread's share of the fused split + norm + RoPE + store: lane t of the
// (head, lane) pairs of a token (t / LPH = head, t % LPH = lane), tokens
// tok_start, tok_start + tok_step, ... in groups of T.  Everything that depends
// on the head only (q / k / v, norm weights) is set up once.  Per group a thread
// first requests positions and slots of its T tokens, then their two 16-byte
// pieces, then the cos / sin pieces, and only then starts the arithmetic: 2 T +
// 2 T loads in flight per thread.  NORM compiles the per-head RMSNorm in.  All
// threads of a warp must call it together (the norm shuffles across the LPH
// lanes of a head).
template <int LPH, bool NORM, int T, bool CG>
__device__ __forceinline__ void rope_thread(const RopeArgs& a, const int t,
                                            const int64_t tok_start, const int64_t tok_step) {
  constexpr int D = LPH * 16;
  constexpr int HALF = D / 2;
  const int heads = a.hq + a.hkv + (a.v ? a.hkv : 0);
  int h = t / LPH;          // LPH is a power of two: a shift
  const int j = t % LPH;
  // all lanes of a group share `live`; the shuffles of the norm stay convergent
  // because dead groups still execute them with zeros.
  const bool live = h < heads;
  int kind = 0;  // 0 q, 1 k, 2 v
  uint16_t* base = nullptr;
  int64_t stride = 0;
  if (live) {
    if (h < a.hq) {
      kind = 0;
      base = a.q + (int64_t)h * D;
      stride = a.q_stride;
    } else if (h < a.hq + a.hkv) {
      kind = 1;
      h -= a.hq;
      base = a.k + (int64_t)h * D;
      stride = a.k_stride;
    } else {
      kind = 2;
      h -= a.hq + a.hkv;
      base = const_cast<uint16_t*>(a.v) + (int64_t)h * D;
      stride = a.v_stride;
    }
  }
  const bool store = live && kind != 0 && a.k_cache != nullptr;
  uint16_t* cache_out = kind == 1 ? a.k_cache : a.v_cache;
  float w1[8], w2[8];
  bool normed = false;
  if (NORM) {
    const uint4* nw = kind == 0 ? a.q_norm_w : (kind == 1 ? a.k_norm_w : nullptr);
    normed = live && nw != nullptr;
    if (normed) {
      unpack8(__ldg(nw + j), w1);
      unpack8(__ldg(nw + LPH + j), w2);
    }
  }
  const bool cache_bf16 = !a.cache_is_fp32;
  const uint16_t* cache16 = static_cast<const uint16_t*>(a.cache);

  for (int64_t t0 = tok_start; t0 < a.num_tokens; t0 += tok_step) {
    bool on[T];
    int64_t pos[T], slot[T];
    uint4 r1[T], r2[T], cs1[T], cs2[T];
#pragma unroll
    for (int i = 0; i < T; ++i) {
      on[i] = live && t0 + i < a.num_tokens;
      pos[i] = (on[i] && kind != 2) ? a.positions[t0 + i] : 0;
      slot[i] = (on[i] && store) ? (int64_t)a.slots[t0 + i] : -1;
    }
#pragma unroll
    for (int i = 0; i < T; ++i) {
      r1[i] = r2[i] = make_uint4(0, 0, 0, 0);
      if (on[i]) {
        const uint16_t* src = base + (t0 + i) * stride;
        r1[i] = ld16<CG>(src + j * 8);
        r2[i] = ld16<CG>(src + HALF + j * 8);
      }
    }
    bool pos_ok[T];
#pragma unroll
    for (int i = 0; i < T; ++i) {
      pos_ok[i] = pos[i] >= 0 && pos[i] < a.max_position;
      cs1[i] = cs2[i] = make_uint4(0, 0, 0, 0);
      if (on[i] && kind != 2 && pos_ok[i] && cache_bf16) {
        cs1[i] = __ldg(reinterpret_cast<const uint4*>(cache16 + pos[i] * D + j * 8));
        cs2[i] = __ldg(reinterpret_cast<const uint4*>(cache16 + pos[i] * D + HALF + j * 8));
      }
    }
#pragma unroll
    for (int i = 0; i < T; ++i) {
      uint4 o1 = r1[i], o2 = r2[i];
      if (kind != 2 || NORM) {
        float x1[8], x2[8];
        unpack8(r1[i], x1);
        unpack8(r2[i], x2);
        if (NORM) {
          // per-head RMSNorm first (Qwen3 order), rounded to bf16 like the separate
          // kernel's output would be
          float ss = 0.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) ss += x1[e] * x1[e] + x2[e] * x2[e];
#pragma unroll
          for (int off = LPH / 2; off > 0; off >>= 1)
            ss += __shfl_xor_sync(0xffffffffu, ss, off);
          if (normed) {
            const float rs = rsqrtf(ss * (1.0f / D) + a.eps);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              x1[e] = round_bf16(x1[e] * rs * w1[e]);
              x2[e] = round_bf16(x2[e] * rs * w2[e]);
            }
          }
        }
        if (on[i] && kind != 2) {
          if (pos_ok[i]) {
            float c[8], sn[8], y1[8], y2[8];
            if (cache_bf16) {
              unpack8(cs1[i], c);
              unpack8(cs2[i], sn);
            } else {
              load_cs8(a.cache, 1, pos[i] * D + j * 8, c);
              load_cs8(a.cache, 1, pos[i] * D + HALF + j * 8, sn);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              y1[e] = x1[e] * c[e] - x2[e] * sn[e];
              y2[e] = x2[e] * c[e] + x1[e] * sn[e];
            }
            o1 = pack8(y1);
            o2 = pack8(y2);
          } else {
            if (a.status && j == 0) atomicOr(a.status, FK_DEV_BAD_POSITION);
            o1 = pack8(x1);
            o2 = pack8(x2);
          }
          uint16_t* src = base + (t0 + i) * stride;
          *reinterpret_cast<uint4*>(src + j * 8) = o1;
          *reinterpret_cast<uint4*>(src + HALF + j * 8) = o2;
        }
      }
      if (on[i] && store && slot[i] >= 0) {
        if (slot[i] < a.num_slots) {
          int64_t row = slot[i] * a.hkv + h;          // NHD: [slot][head]
          if (a.hnd) {
            const int64_t blk = slot[i] / a.page, off = slot[i] - blk * a.page;
            row = (blk * a.hkv + h) * a.page + off;   // HND: [block][head][offset]
          }
          uint16_t* dst = cache_out + row * (int64_t)D;
          *reinterpret_cast<uint4*>(dst + j * 8) = o1;
          *reinterpret_cast<uint4*>(dst + HALF + j * 8) = o2;
        } else if (a.status && j == 0 && h == 0) {
          atomicOr(a.status, FK_DEV_BAD_SLOT);
        }
      }
    }
  }
}

#endif  // __CUDACC__

}  // namespace fk
