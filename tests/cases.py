"""Seeded synthetic inputs for the decode hot path (numpy, platform-stable).

np.random.RandomState is used everywhere because its streams are frozen across
numpy versions, so the fixtures in tests/golden/ stay valid on any machine.
Shapes follow the benchmark configurations: paged decode attention + KV store
(config 1), fused add+RMSNorm + split + RoPE + store (config 2), the skewed
long-context stress (config 5), and scaled-down decoders for the whole step.
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle.decode_oracle import bf16_round  # noqa: E402


def randn_bf16(rs: np.random.RandomState, shape, scale=1.0) -> np.ndarray:
    """float32 array whose values are exactly representable in bf16."""
    return bf16_round((rs.standard_normal(size=shape) * scale).astype(np.float32))


def attention_case(seed, batch, hq, hkv, d, block_size, num_blocks, lens=None,
                   len_range=(1, 256), log_uniform=False, extra_cols=0):
    """q, paged K/V pool, context lengths and block tables.

    Block tables are a random permutation of pool blocks (each sequence gets
    ceil(L/block) distinct blocks), padded with -1, as the engine pads them
    (fastkernels/infra/engine.py:1974-1975)."""
    rs = np.random.RandomState(seed)
    if lens is None:
        if log_uniform:
            lo, hi = np.log(len_range[0]), np.log(len_range[1])
            lens = np.floor(np.exp(rs.uniform(lo, hi, size=batch))).astype(np.int32)
        else:
            lens = rs.randint(len_range[0], len_range[1] + 1, size=batch).astype(np.int32)
    lens = np.asarray(lens, dtype=np.int32)
    pages = (lens + block_size - 1) // block_size
    need = int(pages.sum())
    if num_blocks is None:
        num_blocks = max(need, 1)
    assert need <= num_blocks, (need, num_blocks)
    perm = rs.permutation(num_blocks).astype(np.int32)
    cols = int(max(pages.max(), 1)) + extra_cols
    bt = np.full((batch, cols), -1, dtype=np.int32)
    o = 0
    for i in range(batch):
        bt[i, :pages[i]] = perm[o:o + pages[i]]
        o += pages[i]
    q = randn_bf16(rs, (batch, hq, d), 0.5)
    k_cache = randn_bf16(rs, (num_blocks, block_size, hkv, d), 0.5)
    v_cache = randn_bf16(rs, (num_blocks, block_size, hkv, d), 0.5)
    return dict(q=q, k_cache=k_cache, v_cache=v_cache, context_lens=lens,
                block_tables=bt, scale=float(d) ** -0.5, block_size=block_size)


def prefill_case(seed, q_lens, k_lens, hq, hkv, d=128, block_size=64, extra_blocks=3):
    """A batch of prompt chunks: sequence i has k_lens[i] keys of which the last
    q_lens[i] are its queries' own tokens (k_lens[i] - q_lens[i] cached before).

    Returns dense q [Tq, Hq, D], k / v [Tk, Hkv, D], cu_seqlens (int32), and the
    same keys laid out in an NHD paged pool (random block permutation, slack
    after each sequence's end filled with large values so that a kernel reading
    past the end shows up)."""
    rs = np.random.RandomState(seed)
    q_lens = np.asarray(q_lens, dtype=np.int32)
    k_lens = np.asarray(k_lens, dtype=np.int32)
    cu_q = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    cu_k = np.concatenate([[0], np.cumsum(k_lens)]).astype(np.int32)
    tq, tk = int(cu_q[-1]), int(cu_k[-1])
    q = randn_bf16(rs, (tq, hq, d), 0.5)
    k = randn_bf16(rs, (max(tk, 1), hkv, d), 0.5)
    v = randn_bf16(rs, (max(tk, 1), hkv, d), 0.5)
    pages = (k_lens + block_size - 1) // block_size
    num_blocks = int(pages.sum()) + extra_blocks
    perm = rs.permutation(num_blocks).astype(np.int32)
    cols = int(max(pages.max(), 1)) + 1
    bt = np.full((len(q_lens), cols), -1, dtype=np.int32)
    k_cache = np.full((num_blocks, block_size, hkv, d), 3.0e4, dtype=np.float32)
    v_cache = np.full((num_blocks, block_size, hkv, d), 3.0e4, dtype=np.float32)
    o = 0
    for i in range(len(q_lens)):
        bt[i, :pages[i]] = perm[o:o + pages[i]]
        o += pages[i]
        for t in range(int(k_lens[i])):
            blk = bt[i, t // block_size]
            k_cache[blk, t % block_size] = k[cu_k[i] + t]
            v_cache[blk, t % block_size] = v[cu_k[i] + t]
    return dict(q=q, k=k, v=v, cu_q=cu_q, cu_k=cu_k, q_lens=q_lens, k_lens=k_lens,
                k_cache=k_cache, v_cache=v_cache, block_tables=bt, block_size=block_size,
                scale=float(d) ** -0.5, max_q=int(q_lens.max()), max_k=int(k_lens.max()))


def config1_case(seed=201):
    """Config 1: batch 8, 32 q / 8 kv heads, D 128, block 256, pool of 128
    blocks, lens uniform in [128, 2048]; each sequence's new token is stored at
    slot = block_table[len // 256] * 256 + len % 256 before attention, and
    attention then covers len + 1 tokens."""
    rs = np.random.RandomState(seed)
    b, hq, hkv, d, bs, nb = 8, 32, 8, 128, 256, 128
    lens = rs.randint(128, 2049, size=b).astype(np.int32)
    case = attention_case(seed + 1000, b, hq, hkv, d, bs, nb, lens=lens + 1)
    case["new_k"] = randn_bf16(rs, (b, hkv, d), 0.5)
    case["new_v"] = randn_bf16(rs, (b, hkv, d), 0.5)
    bt = case["block_tables"]
    case["slot_mapping"] = np.array(
        [bt[i, lens[i] // bs] * bs + lens[i] % bs for i in range(b)], dtype=np.int32)
    return case


def rope_store_case(seed, tokens, hidden, hq, hkv, d, num_blocks, block_size, max_pos,
                    qk_norm=False):
    """Config-2-shaped inputs: x/residual, norm weights, packed qkv rows,
    positions, distinct random slots over the pool."""
    rs = np.random.RandomState(seed)
    out = dict(
        x=randn_bf16(rs, (tokens, hidden)),
        residual=randn_bf16(rs, (tokens, hidden)),
        norm_w=bf16_round((1.0 + 0.02 * rs.standard_normal(hidden)).astype(np.float32)),
        qkv=randn_bf16(rs, (tokens, (hq + 2 * hkv) * d)),
        positions=rs.randint(0, max_pos, size=tokens).astype(np.int64),
        slots=rs.permutation(num_blocks * block_size)[:tokens].astype(np.int32),
    )
    if qk_norm:
        out["q_norm_w"] = bf16_round((1.0 + 0.1 * rs.standard_normal(d)).astype(np.float32))
        out["k_norm_w"] = bf16_round((1.0 + 0.1 * rs.standard_normal(d)).astype(np.float32))
    return out


def decoder_weights(seed, cfg, scale=0.02):
    """Random-init decoder weights (randn * scale, norm weights 1.0), as float32
    arrays of bf16 values.  Layout matches the reference modules: qkv
    [(Hq+2Hkv)*D, hidden], o [hidden, Hq*D], gate_up [2*ffn, hidden],
    down [hidden, ffn], embed/lm_head [vocab, hidden]."""
    rs = np.random.RandomState(seed)
    h, f, v = cfg["hidden"], cfg["ffn"], cfg["vocab"]
    hq, hkv, d = cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    w = {"embed": randn_bf16(rs, (v, h), scale), "lm_head": randn_bf16(rs, (v, h), scale),
         "norm": np.ones(h, dtype=np.float32)}
    for li in range(cfg["num_layers"]):
        p = f"l{li}."
        w[p + "ln1"] = np.ones(h, dtype=np.float32)
        w[p + "ln2"] = np.ones(h, dtype=np.float32)
        w[p + "qkv"] = randn_bf16(rs, ((hq + 2 * hkv) * d, h), scale)
        w[p + "o"] = randn_bf16(rs, (h, hq * d), scale)
        w[p + "gate_up"] = randn_bf16(rs, (2 * f, h), scale)
        w[p + "down"] = randn_bf16(rs, (h, f), scale)
        if cfg.get("qk_norm", False):
            w[p + "qn"] = np.ones(d, dtype=np.float32)
            w[p + "kn"] = np.ones(d, dtype=np.float32)
    return w


TINY_QWEN3 = dict(num_layers=2, hidden=256, ffn=512, num_heads=4, num_kv_heads=2,
                  head_dim=128, vocab=1024, eps=1e-6, theta=1e6, qk_norm=True,
                  max_pos=1024)

# 16 query / 8 KV heads: shards over 2, 4 or 8 tensor-parallel ranks
TINY_TP8 = dict(num_layers=2, hidden=1024, ffn=2048, num_heads=16, num_kv_heads=8,
                head_dim=128, vocab=2048, eps=1e-6, theta=1e6, qk_norm=True,
                max_pos=1024)
