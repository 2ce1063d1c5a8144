"""Parity at the benchmark configurations' OWN widths (not scaled-down stand-ins):

  config 3  a composed decode step at hidden 4096, 32 / 8 heads, FFN 12288, vocab
            151 936, q/k norm, batch 64 under CUDA graphs, in lockstep with the
            oracle (2 layers: the oracle's host time is per layer);
  config 2  the fused chain at its size: 4096 tokens x hidden 4096 through fused
            add + RMSNorm, then split + RoPE + store on 4096 x 6144 packed rows;
  config 5  the attention call at batch 256 (oracle on a seeded subset, the
            V == 1 property on every sequence);
  config 4  the per-rank attention shapes of the 70B-shape decoder at tp 2 / 4 / 8
            (32/4, 16/2, 8/1 heads, batch 128).

All through the C-ABI; the oracle is the checker only.
"""
import numpy as np
import pytest
import torch

import cases
from gpu_util import assert_bf16_close, dev, host_bits, host_f32
from oracle import decode_oracle as O
from test_gpu_engine import lockstep, make_engine, seed_context

pytestmark = pytest.mark.gpu

ATOL = RTOL = 2e-2


@pytest.fixture(scope="module")
def ops():
    from fastkernels_b200 import ops as _ops
    return _ops


# ------------------------------------------------------------------ config 3 width
C3_WIDTH = dict(num_layers=2, hidden=4096, ffn=12288, num_heads=32, num_kv_heads=8,
                head_dim=128, vocab=151936, eps=1e-6, theta=1e6, qk_norm=True, max_pos=2048)


def wide_weights(seed, cfg, scale=0.02):
    """decoder_weights at full width.  The values are drawn on the device (the
    host generator needs minutes for the 151 936 x 4096 matrices) and come back
    as float32 arrays of bf16 values; embedding and LM head share one matrix."""
    g = torch.Generator(device="cuda").manual_seed(seed)

    def rnd(shape, mean=0.0, std=scale):
        t = torch.randn(shape, generator=g, device="cuda") * std + mean
        return t.to(torch.bfloat16).float().cpu().numpy()

    h, f, v = cfg["hidden"], cfg["ffn"], cfg["vocab"]
    hq, hkv, d = cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    head = rnd((v, h))
    w = {"embed": head, "lm_head": head, "norm": np.ones(h, np.float32)}
    for li in range(cfg["num_layers"]):
        p = f"l{li}."
        w[p + "ln1"] = rnd((h,), 1.0, 0.02)
        w[p + "ln2"] = rnd((h,), 1.0, 0.02)
        w[p + "qkv"] = rnd(((hq + 2 * hkv) * d, h))
        w[p + "o"] = rnd((h, hq * d))
        w[p + "gate_up"] = rnd((2 * f, h))
        w[p + "down"] = rnd((h, f))
        w[p + "qn"] = rnd((d,), 1.0, 0.1)
        w[p + "kn"] = rnd((d,), 1.0, 0.1)
    return w


@pytest.fixture(scope="module")
def wide():
    return wide_weights(41, C3_WIDTH)


@pytest.mark.timeout(1500)
@pytest.mark.parametrize("decode_block", [False, True], ids=["kernels", "persistent_block"])
def test_config3_width_graph_decode_in_lockstep_with_oracle(wide, decode_block):
    cfg_d, w = C3_WIDTH, wide
    rs = np.random.RandomState(42)
    lens = rs.randint(256, 1025, size=64).tolist()
    eng = make_engine(cfg_d, w, lens, block=256, eager=False, graphs=(64,),
                      decode_block=decode_block)
    first, kcs, vcs = seed_context(eng, lens, 43)
    steps = 8
    equal, near, first_logits = lockstep(cfg_d, w, eng, first, kcs, vcs, steps)
    assert int(eng.status.item()) == 0
    total = steps * len(lens)
    # lockstep() has already verified that every differing token sits within two
    # bf16 steps of the oracle's maximum logit
    assert equal + near == total, f"{equal} equal + {near} near ties of {total}"
    assert equal >= 0.95 * total, f"only {equal} of {total} tokens equal ({near} near ties)"


def test_config3_width_first_step_logits_within_tolerance(wide):
    cfg_d, w = dict(C3_WIDTH, num_layers=1), wide      # the first layer of the same weights
    rs = np.random.RandomState(45)
    lens = rs.randint(256, 1025, size=64).tolist()
    eng = make_engine(cfg_d, w, lens, block=256, eager=True)
    first, kcs, vcs = seed_context(eng, lens, 46)
    _, _, ref = lockstep(cfg_d, w, eng, first, kcs, vcs, 1)
    got = eng.graph_vars["lm_logits"][:64].float().cpu().numpy()
    inside = np.abs(got - ref) <= ATOL + RTOL * np.abs(ref)
    assert inside.mean() >= 0.99, inside.mean()
    assert np.abs(got - ref).max() <= 0.0625, np.abs(got - ref).max()


# ------------------------------------------------------------------- config 2 size
def test_config2_chain_at_its_size(ops):
    t, hidden, hq, hkv, d = 4096, 4096, 32, 8, 128
    nb, bs, max_pos = 256, 256, 8192
    rc = cases.rope_store_case(202, t, hidden, hq, hkv, d, nb, bs, max_pos, qk_norm=False)
    # fused residual add + RMSNorm (eps 1e-6, weights 1 + 0.02 randn), in place
    x, r = dev(rc["x"]), dev(rc["residual"])
    ops.fused_add_rmsnorm(x, r, dev(rc["norm_w"]), 1e-6)
    y_ref, r_ref = O.rmsnorm_kernel(rc["x"], rc["norm_w"], 1e-6, rc["residual"])
    assert np.array_equal(host_bits(r), O.bf16_round_bits(r_ref)), "residual not bit-exact"
    assert_bf16_close(x, y_ref, max_ulp=1, frac=0.02)
    # split + NeoX RoPE (theta 1e6) + store of the 4096 packed rows
    cache = O.rope_cos_sin_cache(d, max_pos, 1e6)
    qkv = rc["qkv"]
    q_np, k_np, v_np = np.split(qkv, [hq * d, (hq + hkv) * d], axis=1)
    q_ref, k_ref = O.rope_neox(rc["positions"], q_np, k_np, d, O.bf16_round(cache))
    buf = dev(qkv)
    kc = torch.zeros((nb, bs, hkv, d), dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    st = ops.new_status("cuda")
    ops.qkv_rope_store(buf, hq, hkv, d, dev(rc["positions"]), dev(cache, torch.float32),
                       None, None, 1e-6, kc, vc, dev(rc["slots"]), st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert_bf16_close(buf[:, :hq * d], q_ref, max_ulp=1, frac=0.02)
    assert_bf16_close(buf[:, hq * d:(hq + hkv) * d], k_ref, max_ulp=1, frac=0.02)
    # cache rows: exactly the rotated k the kernel wrote in place, and raw v;
    # every slot that no token maps to is still zero
    k_gpu = host_bits(buf[:, hq * d:(hq + hkv) * d].contiguous()).reshape(t, hkv, d)
    kc_ref = np.zeros((nb * bs, hkv, d), np.uint16)
    vc_ref = np.zeros_like(kc_ref)
    O.store_kvcache(k_gpu, O.bf16_round_bits(v_np).reshape(t, hkv, d), kc_ref, vc_ref,
                    rc["slots"])
    assert np.array_equal(host_bits(kc).reshape(kc_ref.shape), kc_ref)
    assert np.array_equal(host_bits(vc).reshape(vc_ref.shape), vc_ref)
    # v columns of the packed rows untouched
    assert np.array_equal(host_bits(buf[:, (hq + hkv) * d:].contiguous()),
                          O.bf16_round_bits(v_np))


# ---------------------------------------------------------- attention at full batch
def device_attention_case(seed, batch, hq, hkv, lens, block=256, d=128):
    """The pool is made on the device (gigabytes at these sizes); block tables are
    a random permutation of the pool."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    lens_t = torch.as_tensor(np.asarray(lens, np.int32), device="cuda")
    pages = (np.asarray(lens) + block - 1) // block
    nb = int(pages.sum())
    perm = torch.randperm(nb, generator=g, device="cuda").to(torch.int32).cpu().numpy()
    bt = np.full((batch, int(pages.max())), -1, np.int32)
    o = 0
    for i in range(batch):
        bt[i, :pages[i]] = perm[o:o + pages[i]]
        o += pages[i]
    q = (torch.randn((batch, hq, d), generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    kc = (torch.randn((nb, block, hkv, d), generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    vc = (torch.randn((nb, block, hkv, d), generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    return q, kc, vc, lens_t, torch.as_tensor(bt, device="cuda"), bt


def check_subset(q, kc, vc, lens, bt_np, out, subset, scale):
    """Oracle on the sequences of `subset`: only their pages travel to the host."""
    for i in subset:
        L = int(lens[i])
        pages = bt_np[i, :(L + kc.shape[1] - 1) // kc.shape[1]]
        idx = torch.as_tensor(pages.astype(np.int64), device="cuda")
        k_host, v_host = host_f32(kc[idx]), host_f32(vc[idx])
        local_bt = np.arange(len(pages), dtype=np.int32)[None, :]
        ref = O.paged_decode_attention(host_f32(q[i:i + 1]), k_host, v_host,
                                       np.array([L], np.int32), local_bt, scale)
        got = host_f32(out[i:i + 1])
        np.testing.assert_allclose(got, ref, atol=ATOL, rtol=RTOL)
        assert np.abs(got - ref).max() <= 6e-3, (i, L, np.abs(got - ref).max())


def test_config5_attention_at_batch_256(ops):
    b, hq, hkv, d = 256, 64, 4, 128
    rs = np.random.RandomState(205)
    lens = np.floor(np.exp(rs.uniform(np.log(64), np.log(32768), size=b))).astype(np.int32)
    q, kc, vc, lens_t, bt, bt_np = device_attention_case(5, b, hq, hkv, lens)
    ws = torch.empty(ops.attn_workspace_bytes(b, hq, d, 64), dtype=torch.uint8, device="cuda")
    st = ops.new_status("cuda")
    out = ops.paged_decode_attn(q, kc, vc, lens_t, bt, d ** -0.5, ws, 64, status=st)
    one = ops.paged_decode_attn(q, kc, torch.ones_like(vc), lens_t, bt, d ** -0.5, ws, 64,
                                status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    # softmax weights sum to one: with V == 1 every output of all 256 sequences is 1
    assert torch.allclose(one.float(), torch.ones_like(one, dtype=torch.float32), atol=8e-3)
    # oracle on 32 seeded sequences, always including the shortest and the longest
    subset = set(rs.choice(b, size=30, replace=False).tolist())
    subset |= {int(np.argmin(lens)), int(np.argmax(lens))}
    check_subset(q, kc, vc, lens, bt_np, out, sorted(subset), d ** -0.5)


@pytest.mark.parametrize("hq,hkv", [(32, 4), (16, 2), (8, 1)])
def test_config4_per_rank_attention_shapes(ops, hq, hkv):
    """Llama-3-70B shape (64 / 8 heads) split over 2, 4 and 8 ranks: batch 128,
    contexts uniform in [512, 8192]."""
    b, d = 128, 128
    rs = np.random.RandomState(400 + hq)
    lens = rs.randint(512, 8193, size=b).astype(np.int32)
    q, kc, vc, lens_t, bt, bt_np = device_attention_case(40 + hq, b, hq, hkv, lens)
    ws = torch.empty(ops.attn_workspace_bytes(b, hq, d, 64), dtype=torch.uint8, device="cuda")
    st = ops.new_status("cuda")
    out = ops.paged_decode_attn(q, kc, vc, lens_t, bt, d ** -0.5, ws, 64, status=st)
    one = ops.paged_decode_attn(q, kc, torch.ones_like(vc), lens_t, bt, d ** -0.5, ws, 64,
                                status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert torch.allclose(one.float(), torch.ones_like(one, dtype=torch.float32), atol=8e-3)
    subset = set(rs.choice(b, size=10, replace=False).tolist())
    subset |= {int(np.argmin(lens)), int(np.argmax(lens))}
    check_subset(q, kc, vc, lens, bt_np, out, sorted(subset), d ** -0.5)
