"""CPU oracle for the decode hot path -- TEST INFRASTRUCTURE, not product code.

A numpy restatement of the reference's algorithms for the decode step of the
FastKernels serving engine.  Only tests/, __graft_entry__.smoke() and the
cpu_baseline / --impl reference legs of bench.py may import this module; the
product path (fastkernels_b200/) never does.

Parity pin: every function here is checked against the reference's own Python
code (imported from the reference tree when the fixtures were generated) through
the golden vectors in tests/golden/*.npz, produced by tests/golden/make_golden.py.
The reference ships no golden vectors of its own for this path.

Each function cites the reference file:line it follows (paths relative to the
reference repository root).  bf16 tensors travel as uint16 bit patterns; all
arithmetic is float32 (float64 where stated) with explicit bf16 rounding at the
points where the reference rounds.
"""
from __future__ import annotations

import numpy as np

# --------------------------------------------------------------------------- bf16


def bf16_round_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit pattern (uint16), round-to-nearest-even, NaN kept."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    rounding = ((u >> 16) & 1) + np.uint32(0x7FFF)
    r = ((u + rounding) >> 16).astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        r = np.where(nan, ((u >> 16) | 0x40).astype(np.uint16), r)
    return r


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest bf16 value, returned as float32."""
    return bf16_bits_to_f32(bf16_round_bits(x))


# --------------------------------------------------------------------------- store


def store_kvcache(key, value, k_cache, v_cache, slot_mapping) -> None:
    """fastkernels/tasks/baseline/L1/store_kvcache.py:16-35 (NHD kernel) and
    71-82 (module): for each token i with slot >= 0,
    cache.view(-1, Hkv*D)[slot] = key[i].view(Hkv*D).  In place; any dtype."""
    n = key.shape[0]
    row = int(np.prod(key.shape[1:]))
    kc = k_cache.reshape(-1, row)
    vc = v_cache.reshape(-1, row)
    slots = np.asarray(slot_mapping).astype(np.int64)
    for i in range(n):
        s = int(slots[i])
        if s < 0:
            continue
        kc[s] = key[i].reshape(row)
        vc[s] = value[i].reshape(row)


def store_kvcache_hnd(key, value, k_cache, v_cache, slot_mapping) -> None:
    """fastkernels/tasks/baseline/L1/store_kvcache.py:38-68 (HND kernel) and 85-101:
    caches [num_blocks, Hkv, page, D]; block = slot // page, offset = slot % page,
    head h of token i goes to cache[block, h, offset, :].  In place; any dtype."""
    page = k_cache.shape[2]
    slots = np.asarray(slot_mapping).astype(np.int64)
    for i in range(key.shape[0]):
        s = int(slots[i])
        if s < 0:
            continue
        k_cache[s // page, :, s % page, :] = key[i]
        v_cache[s // page, :, s % page, :] = value[i]


def hnd_to_nhd(cache):
    """View an HND pool [blocks, Hkv, page, D] as NHD [blocks, page, Hkv, D]."""
    return np.transpose(cache, (0, 2, 1, 3))


# ----------------------------------------------------------------------- attention


def _cache_seq(cache, block_table, length, block_size):
    """fastkernels/tasks/baseline/L2/attention_impl.py:598-604."""
    pages = (length + block_size - 1) // block_size
    ids = np.asarray(block_table[:pages]).astype(np.int64)
    hkv, d = cache.shape[-2], cache.shape[-1]
    return cache[ids].reshape(-1, hkv, d)[:length]


def paged_decode_attention(q, k_cache, v_cache, context_lens, block_tables, scale,
                           dtype=np.float32, kv_layout="NHD"):
    """fastkernels/tasks/baseline/L2/attention_impl.py:654-664 (_decode_torch)
    with _sdpa_one (606-622) and _repeat_kv_for_heads (592-596).

    q [B, Hq, D], caches [num_blocks, block, Hkv, D] (float arrays),
    context_lens [B], block_tables [B, cols].  One query token per sequence
    attends to all L_i cached keys (the causal mask k_pos <= q_pos with
    q_pos = L_i - 1 keeps every key).  Returns [B, Hq, D] in `dtype`.
    A sequence of length 0 yields zeros (the reference never issues one)."""
    if kv_layout == "HND":
        # the HND page-table kernel the reference calls on B200
        # (fastkernels/tasks/baseline/L1/flashinfer_decode.py:92-107, third-party
        # trtllm-gen) computes the same attention over pages laid out
        # [blocks, Hkv, page, D]
        k_cache, v_cache = hnd_to_nhd(k_cache), hnd_to_nhd(v_cache)
    b, hq, d = q.shape
    block_size, hkv = k_cache.shape[1], k_cache.shape[2]
    g = hq // hkv
    out = np.zeros((b, hq, d), dtype=dtype)
    for i in range(b):
        length = int(context_lens[i])
        if length <= 0:
            continue
        ks = _cache_seq(k_cache, block_tables[i], length, block_size)
        vs = _cache_seq(v_cache, block_tables[i], length, block_size)
        # repeat_interleave of the KV heads to Hq == grouping the query heads by
        # KV head: [Hkv, g, D] x [Hkv, D, L]
        kk = np.ascontiguousarray(ks.transpose(1, 0, 2), dtype=dtype)   # [Hkv, L, D]
        vv = np.ascontiguousarray(vs.transpose(1, 0, 2), dtype=dtype)
        qi = q[i].astype(dtype).reshape(hkv, g, d)
        s = np.matmul(qi, kk.transpose(0, 2, 1)) * dtype(scale)          # [Hkv, g, L]
        s = s - s.max(axis=2, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(axis=2, keepdims=True)
        out[i] = np.matmul(p, vv).reshape(hq, d)
    return out



# ------------------------------------------------------------------------- prefill


def prefill_attention(q, k, v, cu_q, cu_k, scale, causal=True, block_tables=None,
                      block_size=None, kv_layout="NHD"):
    """Variable-length prefill attention in fp32.

    Dense K/V: fastkernels/tasks/baseline/L2/attention_impl.py:624-636
    (_prefill_torch_from_tensors); paged: 638-652 (_prefill_torch_from_cache);
    both through _sdpa_one (606-622): key j is visible to query t of a sequence
    iff j <= (k_len - q_len) + t.
    q [Tq, Hq, D]; dense k, v [Tk, Hkv, D]; paged: the pools and block_tables.
    Returns (out [Tq, Hq, D] fp32, lse [Hq, Tq] fp32, natural log; -inf and a
    zero row where no key is visible)."""
    q = np.asarray(q, dtype=np.float32)
    tq, hq, d = q.shape
    if block_tables is not None and kv_layout == "HND":
        k, v = hnd_to_nhd(k), hnd_to_nhd(v)
    hkv = k.shape[-2]
    g = hq // hkv
    out = np.zeros((tq, hq, d), dtype=np.float32)
    lse = np.full((hq, tq), -np.inf, dtype=np.float32)
    for i in range(len(cu_q) - 1):
        qs, qe = int(cu_q[i]), int(cu_q[i + 1])
        k_len = int(cu_k[i + 1]) - int(cu_k[i])
        q_len = qe - qs
        if q_len == 0:
            continue
        if block_tables is None:
            ks = int(cu_k[i])
            kk = np.asarray(k[ks:ks + k_len], dtype=np.float32)
            vv = np.asarray(v[ks:ks + k_len], dtype=np.float32)
        else:
            kk = _cache_seq(k, block_tables[i], k_len, block_size).astype(np.float32)
            vv = _cache_seq(v, block_tables[i], k_len, block_size).astype(np.float32)
        if k_len == 0:
            continue
        kh = np.repeat(kk.transpose(1, 0, 2), g, axis=0)      # [Hq, k_len, D]
        vh = np.repeat(vv.transpose(1, 0, 2), g, axis=0)
        s = np.einsum("thd,hkd->htk", q[qs:qe], kh).astype(np.float32) * np.float32(scale)
        if causal:
            qpos = (k_len - q_len) + np.arange(q_len)
            mask = np.arange(k_len)[None, :] <= qpos[:, None]
            s = np.where(mask[None], s, -np.inf)
        m = s.max(axis=-1, keepdims=True)
        msafe = np.where(np.isfinite(m), m, 0.0)
        e = np.exp(s - msafe)
        l = e.sum(axis=-1, keepdims=True)
        o = np.einsum("htk,hkd->thd", e / np.where(l > 0, l, 1.0), vh)
        out[qs:qe] = o
        with np.errstate(divide="ignore"):
            lse[:, qs:qe] = np.where(l[..., 0] > 0, np.log(l[..., 0]) + msafe[..., 0], -np.inf)
    return out, lse


def merge_attn_states(prefix_out, prefix_lse, suffix_out, suffix_lse,
                      prefill_tokens_with_context=None):
    """fastkernels/tasks/baseline/L1/merge_attn_states.cu:2470-2575 (the Triton
    statement of the same maths: triton_merge_attn_states.py:100-175).
    Outputs [T, H, D] float32 arrays of bf16 values, lse [H, T] fp32.  +inf lse
    counts as -inf; both -inf: the prefix row passes through, lse -inf.  Tokens
    >= prefill_tokens_with_context copy the suffix.  Returns (out bf16-rounded
    fp32, out_lse)."""
    a = np.asarray(prefix_out, dtype=np.float32)
    b = np.asarray(suffix_out, dtype=np.float32)
    la = np.asarray(prefix_lse, dtype=np.float32).T.copy()    # [T, H]
    lb = np.asarray(suffix_lse, dtype=np.float32).T.copy()
    la[np.isinf(la)] = -np.inf
    lb[np.isinf(lb)] = -np.inf
    mx = np.maximum(la, lb)
    dead = np.isinf(mx)
    ms = np.where(dead, 0.0, mx).astype(np.float32)
    ea = np.exp(la - ms).astype(np.float32)
    eb = np.exp(lb - ms).astype(np.float32)
    se = (ea + eb).astype(np.float32)
    se_safe = np.where(dead, 1.0, se).astype(np.float32)
    wa = (ea / se_safe).astype(np.float32)[..., None]
    wb = (eb / se_safe).astype(np.float32)[..., None]
    out = bf16_round((a * wa).astype(np.float32) + (b * wb).astype(np.float32))
    out = np.where(dead[..., None], a, out)
    with np.errstate(divide="ignore"):
        out_lse = np.where(dead, -np.inf, np.log(se_safe) + ms).astype(np.float32)
    if prefill_tokens_with_context is not None:
        n = int(prefill_tokens_with_context)
        out[n:] = b[n:]
        out_lse[n:] = np.asarray(suffix_lse, dtype=np.float32).T[n:]
    return out.astype(np.float32), out_lse.T.copy()


# --------------------------------------------------------------------------- norms


def rmsnorm_native(x, weight, eps, residual=None):
    """fastkernels/tasks/baseline/L1/rms_norm.py:97-118 (forward_native), for
    bf16 activations given as float32 arrays holding bf16 values:
    fp32 promote, [add residual, round to bf16 for the returned residual but
    keep the UNROUNDED sum for the variance], x*rsqrt(var+eps) rounded to bf16,
    then multiplied by the weight in bf16 (second rounding)."""
    x = x.astype(np.float32)
    res_out = None
    if residual is not None:
        x = x + residual.astype(np.float32)
        res_out = bf16_round(x)
    var = np.mean(x * x, axis=-1, keepdims=True, dtype=np.float32)
    y = bf16_round(x * (1.0 / np.sqrt(var + np.float32(eps))).astype(np.float32))
    y = bf16_round(y * weight.astype(np.float32))
    return y if residual is None else (y, res_out)


def rmsnorm_kernel(x, weight, eps, residual=None):
    """The reference's CUDA kernel semantics, which is what the engine runs in
    eager / CUDA-graph mode: fastkernels/tasks/baseline/L1/rms_norm.cu:1251-1336
    (rms_norm) and 1342-1410 (fused_add_rms_norm).  The residual sum is rounded
    to bf16 BEFORE the variance; out = bf16(x * rsqrt(mean(x^2)+eps) * w), one
    rounding.  Inputs: float32 arrays holding bf16 values."""
    x = x.astype(np.float32)
    res_out = None
    if residual is not None:
        x = bf16_round(x + residual.astype(np.float32))
        res_out = x
    var = (x.astype(np.float64) ** 2).mean(axis=-1, keepdims=True)
    rs = (1.0 / np.sqrt(var + eps)).astype(np.float32)
    y = bf16_round(x * rs * weight.astype(np.float32))
    return y if residual is None else (y, res_out)


# ----------------------------------------------------------------------- all-reduce


def allreduce_sum(partials):
    """Sum of the ranks' bf16 tensors the way the reference's custom all-reduce
    forms it (fastkernels/tasks/baseline/L1/allreduce.cu:184-191, packed_reduce:
    the first rank's value is widened to fp32, the others are added in rank
    order, one rounding back to bf16); its one-stage and two-stage kernels give
    the same bits (193-250).  `partials`: sequence of float32 arrays holding bf16
    values, one per rank."""
    acc = np.asarray(partials[0], dtype=np.float32).copy()
    for part in partials[1:]:
        acc = (acc + np.asarray(part, dtype=np.float32)).astype(np.float32)
    return bf16_round(acc)


def allreduce_add_rmsnorm(partials, residual, weight, eps):
    """AllReduce.forward (fastkernels/tasks/baseline/L1/allreduce.py:37-55) followed
    by RMSNorm.forward(x, residual) with the CUDA kernel's rounding
    (rms_norm.cu:1342-1410): what a row-parallel projection plus the next norm
    compute on every rank.  Returns (out, new residual)."""
    return rmsnorm_kernel(allreduce_sum(partials), weight, eps, residual)


# ---------------------------------------------------------------------------- rope


def rope_cos_sin_cache(head_dim, max_position, theta):
    """fastkernels/tasks/baseline/L1/rotary_emb.py:93-107 with
    rope_scaling_factor == 1.0: fp32 [max_position, head_dim] = cat(cos, sin)."""
    inv_freq = (1.0 / (np.float32(theta) ** (np.arange(0, head_dim, 2, dtype=np.float32)
                                              / np.float32(head_dim)))).astype(np.float32)
    t = np.arange(max_position, dtype=np.float32)
    freqs = np.outer(t, inv_freq).astype(np.float32)
    return np.concatenate([np.cos(freqs), np.sin(freqs)], axis=-1).astype(np.float32)


def rope_neox(positions, query, key, head_dim, cos_sin_cache, rounding="kernel"):
    """NeoX rotation.  cos_sin_cache must already be rounded to the activation
    dtype (the reference casts it per call, rotary_emb.py:171-173).

    rounding="kernel": fastkernels/tasks/baseline/L1/rotary_emb.cu:332-358 --
      fp32 maths, one rounding of each output.
    rounding="native": fastkernels/tasks/baseline/L1/rotary_emb.py:109-139 run
      on bf16 tensors -- every elementwise product and the sum/difference round
      to bf16.
    query [T, Hq*D], key [T, Hkv*D] float32 arrays of bf16 values; returns
    rotated copies."""
    cs = cos_sin_cache[np.asarray(positions).astype(np.int64)].astype(np.float32)
    half = head_dim // 2
    cos = cs[:, None, :half]
    sin = cs[:, None, half:]

    def rot(x):
        t = x.shape[0]
        xv = x.reshape(t, -1, head_dim).astype(np.float32)
        x1, x2 = xv[..., :half], xv[..., half:]
        if rounding == "kernel":
            o1 = bf16_round(x1 * cos - x2 * sin)
            o2 = bf16_round(x2 * cos + x1 * sin)
        else:
            o1 = bf16_round(bf16_round(x1 * cos) - bf16_round(x2 * sin))
            o2 = bf16_round(bf16_round(x2 * cos) + bf16_round(x1 * sin))
        return np.concatenate([o1, o2], axis=-1).reshape(x.shape)

    return rot(query), (rot(key) if key is not None else None)


# ---------------------------------------------------------------------------- silu


def silu_and_mul(x, rounding="kernel"):
    """rounding="kernel": fastkernels/tasks/baseline/L1/silu_and_mul.cu:715-740,
    823-830: bf16(float(bf16(g / (1 + exp(-g)))) * u).
    rounding="native": fastkernels/tasks/baseline/L1/silu_and_mul.py:18-22 on
    bf16 tensors (F.silu rounds to bf16, the product rounds again) -- the same
    two roundings."""
    d = x.shape[-1] // 2
    g = x[..., :d].astype(np.float32)
    u = x[..., d:].astype(np.float32)
    a = bf16_round(g / (1.0 + np.exp(-g)))
    return bf16_round(a * u)


# -------------------------------------------------------------------------- linear


def linear(x, w, bias=None):
    """F.linear (fastkernels/tasks/baseline/L1/linear.py:13-17;
    L2/parallel_linear.py:81,160,240,332): fp32 accumulate, bf16 output."""
    y = np.asarray(x, dtype=np.float32) @ np.asarray(w, dtype=np.float32).T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float32)
    return bf16_round(y)


# ------------------------------------------------------------------- decode layers


class DecoderOracle:
    """One tensor-parallel rank (tp=1) of a Llama/Qwen3-style decoder run for
    decode, composed as the reference composes it:
      LlamaModel.forward            fastkernels/tasks/baseline/L4/llama.py:100-116
      LlamaDecoderLayer.forward     fastkernels/tasks/baseline/L3/llama_decoder.py:34-42
      LlamaAttention.forward        fastkernels/tasks/baseline/L2/attention.py:113-156
      Attention.forward_impl        fastkernels/tasks/baseline/L2/attention_impl.py:313-363
      LlamaMLP.forward              fastkernels/tasks/baseline/L2/llama_mlp.py:35-38
      lm-head + greedy max          fastkernels/infra/engine.py:6994-6996
    Weights: dict of float32 arrays holding bf16 values.  Rounding points follow
    the CUDA-kernel semantics the engine runs under CUDA graphs."""

    def __init__(self, cfg: dict, weights: dict, cos_sin_cache_bf16: np.ndarray):
        self.cfg = cfg
        self.w = weights
        self.cs = cos_sin_cache_bf16

    def layer(self, li, h, residual, positions, k_cache, v_cache, slot_mapping,
              context_lens, block_tables, cu_seqlens=None):
        """One LlamaDecoderLayer.forward (llama_decoder.py:34-42): decode over the
        paged cache, or -- with cu_seqlens -- prefill of whole prompts
        (attention_impl.py:401-433 with k_len == q_len)."""
        c = self.cfg
        hq, hkv, d = c["num_heads"], c["num_kv_heads"], c["head_dim"]
        eps = c["eps"]
        p = f"l{li}."
        if residual is None:
            residual = h
            x = rmsnorm_kernel(h, self.w[p + "ln1"], eps)
        else:
            x, residual = rmsnorm_kernel(h, self.w[p + "ln1"], eps, residual)
        qkv = linear(x, self.w[p + "qkv"])
        q, k, v = np.split(qkv, [hq * d, (hq + hkv) * d], axis=-1)
        t = q.shape[0]
        if c.get("qk_norm", False):
            q = rmsnorm_kernel(q.reshape(t, hq, d), self.w[p + "qn"], eps).reshape(t, -1)
            k = rmsnorm_kernel(k.reshape(t, hkv, d), self.w[p + "kn"], eps).reshape(t, -1)
        q, k = rope_neox(positions, q, k, d, self.cs)
        store_kvcache(k.reshape(t, hkv, d), v.reshape(t, hkv, d), k_cache, v_cache,
                      slot_mapping)
        if cu_seqlens is None:
            o = paged_decode_attention(q.reshape(t, hq, d), k_cache, v_cache, context_lens,
                                       block_tables, d ** -0.5)
        else:
            o, _ = prefill_attention(q.reshape(t, hq, d), k.reshape(t, hkv, d),
                                     v.reshape(t, hkv, d), cu_seqlens, cu_seqlens, d ** -0.5)
        o = bf16_round(o).reshape(t, hq * d)
        h = linear(o, self.w[p + "o"])
        x, residual = rmsnorm_kernel(h, self.w[p + "ln2"], eps, residual)
        gu = linear(x, self.w[p + "gate_up"])
        h = linear(silu_and_mul(gu), self.w[p + "down"])
        return h, residual

    def head(self, h, residual):
        """Final norm, lm-head projection and greedy max (lowest index on ties)."""
        x, _ = rmsnorm_kernel(h, self.w["norm"], self.cfg["eps"], residual)
        logits = linear(x, self.w["lm_head"])
        return logits, logits.argmax(axis=-1)

    def prefill(self, input_ids, positions, cu_seqlens, k_caches, v_caches, slot_mapping):
        """Whole prompts (concatenated, cu_seqlens [num_seqs + 1]): fills the caches
        and returns the logits / greedy token after each prompt's last token
        (fastkernels/infra/engine.py:6048-6063 with is_prefill=True; the LM head
        runs on the last row of every sequence)."""
        h = self.w["embed"][np.asarray(input_ids).astype(np.int64)]
        residual = None
        for li in range(self.cfg["num_layers"]):
            h, residual = self.layer(li, h, residual, positions, k_caches[li], v_caches[li],
                                     slot_mapping, None, None, cu_seqlens=cu_seqlens)
        rows = np.asarray(cu_seqlens[1:]).astype(np.int64) - 1
        return self.head(h[rows], residual[rows])

    def step(self, input_ids, positions, k_caches, v_caches, slot_mapping, context_lens,
             block_tables):
        h = self.w["embed"][np.asarray(input_ids).astype(np.int64)]
        residual = None
        for li in range(self.cfg["num_layers"]):
            h, residual = self.layer(li, h, residual, positions, k_caches[li], v_caches[li],
                                     slot_mapping, context_lens, block_tables)
        return self.head(h, residual)
