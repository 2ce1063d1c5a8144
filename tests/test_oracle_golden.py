"""The numpy oracle against the reference's own outputs (tests/golden/), CPU only.

This is the pin of the oracle: every restated function must reproduce what the
reference's Python code produced on the same seeded inputs.
"""
import numpy as np

import cases
from oracle import decode_oracle as O


def ulp_diff(a_bits, b_bits):
    """bf16 ulp distance between two uint16 bit-pattern arrays (same sign assumed
    for nearby values; sign-magnitude mapped to a monotone integer line)."""
    def mono(b):
        b = b.astype(np.int32)
        return np.where(b & 0x8000, -(b & 0x7FFF), b & 0x7FFF)
    return np.abs(mono(a_bits) - mono(b_bits))


def test_bf16_round_matches_torch():
    import torch
    rs = np.random.RandomState(0)
    x = np.concatenate([rs.standard_normal(4096).astype(np.float32) * 10.0 ** rs.randint(-6, 6, 4096),
                        np.array([0.0, -0.0, 1.0, 65280.0, 3.3895314e38, np.inf, -np.inf],
                                 dtype=np.float32)])
    ref = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(O.bf16_round_bits(x), ref)
    # ties go to even
    tie = np.array([0x3F808000, 0x3F818000], dtype=np.uint32).view(np.float32)
    assert O.bf16_round_bits(tie).tolist() == [0x3F80, 0x3F82]


def test_attention_small_ragged(golden):
    c = cases.attention_case(11, 5, 8, 2, 128, 64, 12, lens=[1, 63, 64, 65, 200])
    out = O.paged_decode_attention(c["q"], c["k_cache"], c["v_cache"], c["context_lens"],
                                   c["block_tables"], c["scale"])
    np.testing.assert_allclose(out, golden["attn_small"], rtol=2e-5, atol=2e-6)


def test_attention_gqa16(golden):
    c = cases.attention_case(12, 3, 16, 1, 128, 64, 16, lens=[7, 129, 500])
    out = O.paged_decode_attention(c["q"], c["k_cache"], c["v_cache"], c["context_lens"],
                                   c["block_tables"], c["scale"])
    np.testing.assert_allclose(out, golden["attn_g16"], rtol=2e-5, atol=2e-6)


def test_config1_store_then_attention(golden):
    c = cases.config1_case()
    O.store_kvcache(c["new_k"], c["new_v"], c["k_cache"], c["v_cache"], c["slot_mapping"])
    rows = c["slot_mapping"].astype(np.int64)
    assert np.array_equal(O.bf16_round_bits(c["k_cache"].reshape(-1, 1024)[rows]),
                          golden["store_c1_k_rows"])
    assert np.array_equal(O.bf16_round_bits(c["v_cache"].reshape(-1, 1024)[rows]),
                          golden["store_c1_v_rows"])
    out = O.paged_decode_attention(c["q"], c["k_cache"], c["v_cache"], c["context_lens"],
                                   c["block_tables"], c["scale"])
    np.testing.assert_allclose(out, golden["attn_c1"], rtol=2e-5, atol=2e-6)


def test_store_skips_negative_slots():
    rs = np.random.RandomState(3)
    k = rs.randint(0, 65536, size=(4, 2, 8)).astype(np.uint16)
    v = rs.randint(0, 65536, size=(4, 2, 8)).astype(np.uint16)
    kc = np.zeros((2, 4, 2, 8), dtype=np.uint16)
    vc = np.zeros_like(kc)
    O.store_kvcache(k, v, kc, vc, np.array([5, -1, 0, 7]))
    flat = kc.reshape(-1, 16)
    assert np.array_equal(flat[5], k[0].reshape(-1)) and np.array_equal(flat[0], k[2].reshape(-1))
    assert np.array_equal(flat[7], k[3].reshape(-1))
    assert not flat[[1, 2, 3, 4, 6]].any()
    assert np.array_equal(vc.reshape(-1, 16)[7], v[3].reshape(-1))


def _rc():
    return cases.rope_store_case(21, 6, 256, 4, 2, 128, 4, 64, 64, qk_norm=True)


def test_rmsnorm_native(golden):
    rc = _rc()
    y = O.rmsnorm_native(rc["x"], rc["norm_w"], 1e-6)
    assert ulp_diff(O.bf16_round_bits(y), golden["rms_plain"]).max() <= 1
    assert (ulp_diff(O.bf16_round_bits(y), golden["rms_plain"]) > 0).mean() < 0.01
    y, r = O.rmsnorm_native(rc["x"], rc["norm_w"], 1e-6, rc["residual"])
    assert np.array_equal(O.bf16_round_bits(r), golden["rms_fused_res"])
    assert ulp_diff(O.bf16_round_bits(y), golden["rms_fused_y"]).max() <= 1
    q3 = rc["qkv"][:, :512].reshape(6, 4, 128)
    y = O.rmsnorm_native(q3, rc["q_norm_w"], 1e-6)
    assert ulp_diff(O.bf16_round_bits(y), golden["rms_heads"]).max() <= 1


def test_rmsnorm_kernel_semantics_close_to_native(golden):
    """The CUDA-kernel rounding (one rounding, residual rounded first) stays
    within 2 bf16 ulp of the native path the golden vectors hold."""
    rc = _rc()
    y = O.rmsnorm_kernel(rc["x"], rc["norm_w"], 1e-6)
    assert ulp_diff(O.bf16_round_bits(y), golden["rms_plain"]).max() <= 2
    y, r = O.rmsnorm_kernel(rc["x"], rc["norm_w"], 1e-6, rc["residual"])
    assert np.array_equal(O.bf16_round_bits(r), golden["rms_fused_res"])
    np.testing.assert_allclose(y, O.bf16_bits_to_f32(golden["rms_fused_y"]), rtol=2e-2,
                               atol=2e-2)


def test_rope_cache_and_rotation(golden):
    cache = O.rope_cos_sin_cache(128, 64, 1e6)
    # numpy's and torch's float32 pow differ in the last bit of inv_freq; the
    # angle error grows with the position (63 here), far below bf16 resolution
    np.testing.assert_allclose(cache, golden["rope_cache"], rtol=0, atol=1e-5)
    np.testing.assert_allclose(O.rope_cos_sin_cache(128, 32, 5e5), golden["rope_cache_5e5"],
                               rtol=0, atol=1e-5)
    assert (O.bf16_round_bits(cache) != O.bf16_round_bits(golden["rope_cache"])).mean() < 2e-3
    rc = _rc()
    cache_bf = O.bf16_round(golden["rope_cache"])
    q, k = rc["qkv"][:, :512], rc["qkv"][:, 512:768]
    qo, ko = O.rope_neox(rc["positions"], q, k, 128, cache_bf, rounding="native")
    assert np.array_equal(O.bf16_round_bits(qo), golden["rope_q"])
    assert np.array_equal(O.bf16_round_bits(ko), golden["rope_k"])
    qk, kk = O.rope_neox(rc["positions"], q, k, 128, cache_bf, rounding="kernel")
    # one rounding (kernel) vs three (native): results differ by rounding only
    np.testing.assert_allclose(qk, O.bf16_bits_to_f32(golden["rope_q"]), rtol=1.6e-2, atol=1e-2)
    np.testing.assert_allclose(kk, O.bf16_bits_to_f32(golden["rope_k"]), rtol=1.6e-2, atol=1e-2)


def test_silu_and_mul(golden):
    rs = np.random.RandomState(31)
    sx = cases.randn_bf16(rs, (7, 2 * 96), 2.0)
    d = ulp_diff(O.bf16_round_bits(O.silu_and_mul(sx)), golden["silu"])
    assert d.max() <= 1 and (d > 0).mean() < 0.01


def test_linear(golden):
    rs = np.random.RandomState(31)
    cases.randn_bf16(rs, (7, 2 * 96), 2.0)
    lx, lw = cases.randn_bf16(rs, (5, 192)), cases.randn_bf16(rs, (130, 192), 0.05)
    lb = cases.randn_bf16(rs, (130,), 0.1)
    d = ulp_diff(O.bf16_round_bits(O.linear(lx, lw)), golden["linear"])
    assert d.max() <= 1
    # the reference's CPU bf16 addmm rounds the product before adding the bias
    np.testing.assert_allclose(O.linear(lx, lw, lb), O.bf16_bits_to_f32(golden["linear_bias"]),
                               rtol=2e-2, atol=2e-2)


def test_decoder_oracle_runs_and_is_deterministic():
    cfg = cases.TINY_QWEN3
    w = cases.decoder_weights(5, cfg)
    cs = O.bf16_round(O.rope_cos_sin_cache(cfg["head_dim"], cfg["max_pos"], cfg["theta"]))
    dec = O.DecoderOracle(cfg, w, cs)
    nb, bs = 8, 64
    kcs = [np.zeros((nb, bs, cfg["num_kv_heads"], cfg["head_dim"]), np.float32)
           for _ in range(cfg["num_layers"])]
    vcs = [np.zeros_like(kcs[0]) for _ in range(cfg["num_layers"])]
    bt = np.array([[0, 1], [2, 3]], dtype=np.int32)
    ids = np.array([3, 900])
    toks = []
    for step in range(3):
        n = step + 1
        logits, ids = dec.step(ids, np.array([n - 1, n - 1]), kcs, vcs,
                               np.array([bt[0, 0] * bs + n - 1, bt[1, 0] * bs + n - 1]),
                               np.array([n, n], dtype=np.int32), bt)
        assert logits.shape == (2, cfg["vocab"]) and np.isfinite(logits).all()
        toks.append(ids.copy())
    assert kcs[0].reshape(-1, 256)[0].any() and kcs[1].reshape(-1, 256)[2 * bs + 2].any()


def test_hnd_store_and_attention_equal_nhd_under_permutation():
    """The HND restatements against the golden-pinned NHD ones: storing through
    the HND rule and viewing the pool as NHD gives the NHD store's pool, and
    attention over either layout is the same."""
    rs = np.random.RandomState(8)
    nb, page, hkv, d, n = 6, 16, 2, 128, 9
    k = cases.randn_bf16(rs, (n, hkv, d))
    v = cases.randn_bf16(rs, (n, hkv, d))
    slots = np.array([0, 15, 16, 95, -1, 40, 41, 42, 7])
    kc_n = np.zeros((nb, page, hkv, d), np.float32)
    vc_n = np.zeros_like(kc_n)
    kc_h = np.zeros((nb, hkv, page, d), np.float32)
    vc_h = np.zeros_like(kc_h)
    O.store_kvcache(k, v, kc_n, vc_n, slots)
    O.store_kvcache_hnd(k, v, kc_h, vc_h, slots)
    assert np.array_equal(O.hnd_to_nhd(kc_h), kc_n) and np.array_equal(O.hnd_to_nhd(vc_h), vc_n)
    c = cases.attention_case(14, 3, 8, 2, 128, 16, 24, lens=[1, 16, 100])
    ref = O.paged_decode_attention(c["q"], c["k_cache"], c["v_cache"], c["context_lens"],
                                   c["block_tables"], c["scale"])
    kh = np.ascontiguousarray(np.transpose(c["k_cache"], (0, 2, 1, 3)))
    vh = np.ascontiguousarray(np.transpose(c["v_cache"], (0, 2, 1, 3)))
    got = O.paged_decode_attention(c["q"], kh, vh, c["context_lens"], c["block_tables"],
                                   c["scale"], kv_layout="HND")
    assert np.array_equal(got, ref)


# ----------------------------------------------------------------- prefill side
def test_prefill_oracle_matches_reference_vectors():
    """oracle.prefill_attention against outputs of the reference's
    _prefill_torch_from_tensors / _prefill_torch_from_cache (fp32, CPU)."""
    import os
    from golden.make_golden_prefill import CASES
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "prefill_vectors.npz"))
    for name, (seed, ql, kl, hq, hkv, bs) in CASES.items():
        c = cases.prefill_case(seed, ql, kl, hq, hkv, block_size=bs)
        dense, _ = O.prefill_attention(c["q"], c["k"], c["v"], c["cu_q"], c["cu_k"], c["scale"])
        paged, _ = O.prefill_attention(c["q"], c["k_cache"], c["v_cache"], c["cu_q"], c["cu_k"],
                                         c["scale"], block_tables=c["block_tables"],
                                         block_size=bs)
        keep = 1 if name == "chunked" else 2
        assert np.abs(dense[::keep] - g[f"{name}_dense"]).max() < 2e-5, name
        assert np.abs(paged[::4] - g[f"{name}_paged_every4"]).max() < 2e-5, name


def test_merge_oracle_reproduces_whole_attention():
    """merge(prefix part, suffix part) equals attention over all keys -- pinned to
    the reference vectors of the 'chunked' case through that identity."""
    import os
    from golden.make_golden_prefill import CASES
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "prefill_vectors.npz"))
    seed, ql, kl, hq, hkv, bs = CASES["chunked"]
    c = cases.prefill_case(seed, ql, kl, hq, hkv, block_size=bs)
    # sequence 2: 100 queries after 233 cached keys
    qs, ks, n, pre = int(c["cu_q"][2]), int(c["cu_k"][2]), 100, 233
    q = c["q"][qs:qs + n]
    k, v = c["k"][ks:ks + pre + n], c["v"][ks:ks + pre + n]
    cu_q = np.array([0, n])
    a, la = O.prefill_attention(q, k[:pre], v[:pre], cu_q, np.array([0, pre]), c["scale"],
                                  causal=False)
    b, lb = O.prefill_attention(q, k[pre:], v[pre:], cu_q, np.array([0, n]), c["scale"])
    # keep the parts in fp32 here: the merge's own rounding is checked on the GPU
    w = np.exp(la - np.maximum(la, lb)), np.exp(lb - np.maximum(la, lb))
    mix = (a * w[0].T[..., None] + b * w[1].T[..., None]) / (w[0] + w[1]).T[..., None]
    assert np.abs(mix - g["chunked_dense"][qs:qs + n]).max() < 2e-5
    m, ml = O.merge_attn_states(O.bf16_round(a), la, O.bf16_round(b), lb)
    assert np.abs(m - g["chunked_dense"][qs:qs + n]).max() < 1.5e-2
    empty = np.full_like(la, -np.inf)
    m2, ml2 = O.merge_attn_states(O.bf16_round(a), la, O.bf16_round(b), empty)
    assert (m2 == O.bf16_round(O.bf16_round(a) * 1.0)).all() and np.allclose(ml2, la)
