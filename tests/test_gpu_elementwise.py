"""GPU parity (through the C-ABI) of the row kernels against the CPU oracle."""
import numpy as np
import pytest
import torch

import cases
from gpu_util import assert_bf16_close, dev, host_bits, host_f32
from oracle import decode_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from fastkernels_b200 import ops as _ops
    return _ops


# ------------------------------------------------------------------ store_kvcache
@pytest.mark.parametrize("slot_dtype", [torch.int32, torch.int64])
def test_store_kvcache_bit_exact_strided_views(ops, slot_dtype):
    rs = np.random.RandomState(1)
    n, hq, hkv, d, nb, bs = 37, 4, 2, 128, 3, 64
    qkv = rs.randint(0, 65536, size=(n, (hq + 2 * hkv) * d)).astype(np.uint16)
    slots = rs.permutation(nb * bs)[:n].astype(np.int64)
    slots[[3, 11]] = -1
    kc0 = rs.randint(0, 65536, size=(nb, bs, hkv, d)).astype(np.uint16)
    vc0 = rs.randint(0, 65536, size=(nb, bs, hkv, d)).astype(np.uint16)
    k_np = qkv[:, hq * d:(hq + hkv) * d].reshape(n, hkv, d)
    v_np = qkv[:, (hq + hkv) * d:].reshape(n, hkv, d)
    kc_ref, vc_ref = kc0.copy(), vc0.copy()
    O.store_kvcache(k_np, v_np, kc_ref, vc_ref, slots)

    t = torch.from_numpy(qkv.view(np.int16)).cuda().view(torch.bfloat16)
    k = t[:, hq * d:(hq + hkv) * d].view(n, hkv, d)       # strided views
    v = t[:, (hq + hkv) * d:].view(n, hkv, d)
    kc = torch.from_numpy(kc0.view(np.int16)).cuda().view(torch.bfloat16)
    vc = torch.from_numpy(vc0.view(np.int16)).cuda().view(torch.bfloat16)
    st = ops.new_status("cuda")
    ops.store_kvcache(k, v, kc, vc, torch.from_numpy(slots).to(slot_dtype).cuda(), st)
    assert np.array_equal(host_bits(kc), kc_ref)
    assert np.array_equal(host_bits(vc), vc_ref)
    assert int(st.item()) == 0


def test_store_kvcache_unaligned_rows_and_bad_slot(ops):
    rs = np.random.RandomState(2)
    n, hkv, d, slots_total = 9, 1, 12, 20           # 24-byte rows: element path
    k_np = rs.randint(0, 65536, size=(n, hkv, d)).astype(np.uint16)
    v_np = rs.randint(0, 65536, size=(n, hkv, d)).astype(np.uint16)
    slots = np.array([0, 19, 5, -1, 7, 25, 3, 2, 1], dtype=np.int32)  # 25 is out of range
    kc_ref = np.zeros((slots_total, hkv, d), np.uint16)
    vc_ref = np.zeros_like(kc_ref)
    ok = slots.copy()
    ok[5] = -1
    O.store_kvcache(k_np, v_np, kc_ref, vc_ref, ok)
    k = torch.from_numpy(k_np.view(np.int16)).cuda().view(torch.bfloat16)
    v = torch.from_numpy(v_np.view(np.int16)).cuda().view(torch.bfloat16)
    kc = torch.zeros((slots_total, 1, hkv, d), dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    st = ops.new_status("cuda")
    ops.store_kvcache(k, v, kc, vc, torch.from_numpy(slots).cuda(), st)
    assert np.array_equal(host_bits(kc).reshape(kc_ref.shape), kc_ref)
    assert np.array_equal(host_bits(vc).reshape(vc_ref.shape), vc_ref)
    assert int(st.item()) == 1        # FK_DEV_BAD_SLOT, row skipped


@pytest.mark.parametrize("slot_dtype", [torch.int32, torch.int64])
def test_store_kvcache_hnd_bit_exact(ops, slot_dtype):
    rs = np.random.RandomState(6)
    n, hq, hkv, d, nb, page = 41, 4, 2, 128, 9, 16
    qkv = rs.randint(0, 65536, size=(n, (hq + 2 * hkv) * d)).astype(np.uint16)
    slots = rs.permutation(nb * page)[:n].astype(np.int64)
    slots[[0, 7]] = -1
    kc0 = rs.randint(0, 65536, size=(nb, hkv, page, d)).astype(np.uint16)
    vc0 = rs.randint(0, 65536, size=(nb, hkv, page, d)).astype(np.uint16)
    k_np = qkv[:, hq * d:(hq + hkv) * d].reshape(n, hkv, d)
    v_np = qkv[:, (hq + hkv) * d:].reshape(n, hkv, d)
    kc_ref, vc_ref = kc0.copy(), vc0.copy()
    O.store_kvcache_hnd(k_np, v_np, kc_ref, vc_ref, slots)
    t = torch.from_numpy(qkv.view(np.int16)).cuda().view(torch.bfloat16)
    k = t[:, hq * d:(hq + hkv) * d].view(n, hkv, d)
    v = t[:, (hq + hkv) * d:].view(n, hkv, d)
    kc = torch.from_numpy(kc0.view(np.int16)).cuda().view(torch.bfloat16)
    vc = torch.from_numpy(vc0.view(np.int16)).cuda().view(torch.bfloat16)
    st = ops.new_status("cuda")
    ops.store_kvcache_hnd(k, v, kc, vc, torch.from_numpy(slots).to(slot_dtype).cuda(), st)
    assert np.array_equal(host_bits(kc), kc_ref) and np.array_equal(host_bits(vc), vc_ref)
    assert int(st.item()) == 0


def test_qkv_rope_store_hnd_cache_matches_nhd(ops):
    """The fused kernel writing an HND pool stores the same rows as the NHD one."""
    t, hq, hkv, d, nb, page, max_pos = 30, 4, 2, 128, 8, 16, 512
    rc = cases.rope_store_case(78, t, 256, hq, hkv, d, nb, page, max_pos, qk_norm=True)
    cache = dev(O.rope_cos_sin_cache(d, max_pos, 1e6), torch.float32)
    outs = {}
    for layout in ("NHD", "HND"):
        buf = dev(rc["qkv"])
        shape = (nb, page, hkv, d) if layout == "NHD" else (nb, hkv, page, d)
        kc = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
        vc = torch.zeros_like(kc)
        ops.qkv_rope_store(buf, hq, hkv, d, dev(rc["positions"]), cache, dev(rc["q_norm_w"]),
                           dev(rc["k_norm_w"]), 1e-6, kc, vc, dev(rc["slots"]),
                           kv_layout=layout)
        if layout == "HND":
            kc, vc = kc.permute(0, 2, 1, 3).contiguous(), vc.permute(0, 2, 1, 3).contiguous()
        outs[layout] = (host_bits(buf), host_bits(kc), host_bits(vc))
    for a, b in zip(outs["NHD"], outs["HND"]):
        assert np.array_equal(a, b)
    assert outs["NHD"][1].any()


def test_store_kvcache_empty(ops):
    kc = torch.zeros((2, 64, 2, 128), dtype=torch.bfloat16, device="cuda")
    e = torch.empty((0, 2, 128), dtype=torch.bfloat16, device="cuda")
    ops.store_kvcache(e, e, kc, kc.clone(), torch.empty(0, dtype=torch.int32, device="cuda"))


def test_store_roundtrip_config2_size(ops):
    """Full config-2 size: 4096 tokens scattered to distinct slots of a 256x256
    pool, then gathered back: must reproduce the inputs bit for bit and leave
    every other slot untouched."""
    g = torch.Generator(device="cuda").manual_seed(7)
    n, hkv, d = 4096, 8, 128
    k = torch.randn((n, hkv, d), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((n, hkv, d), generator=g, device="cuda").to(torch.bfloat16)
    slots = torch.randperm(256 * 256, generator=g, device="cuda")[:n].to(torch.int32)
    kc = torch.zeros((256, 256, hkv, d), dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    ops.store_kvcache(k, v, kc, vc, slots)
    idx = slots.long()
    assert torch.equal(kc.view(-1, hkv, d)[idx].view(torch.int16), k.view(torch.int16))
    assert torch.equal(vc.view(-1, hkv, d)[idx].view(torch.int16), v.view(torch.int16))
    assert int((kc.view(-1, hkv * d).abs().sum(-1) != 0).sum()) <= n


# ------------------------------------------------------------------------- norms
@pytest.mark.parametrize("rows,cols", [(6, 256), (64, 4096), (3, 8192), (5, 1000), (2, 16384)])
def test_rmsnorm_and_fused(ops, rows, cols):
    rs = np.random.RandomState(rows * 131 + cols)
    x = cases.randn_bf16(rs, (rows, cols))
    r = cases.randn_bf16(rs, (rows, cols))
    w = O.bf16_round((1.0 + 0.02 * rs.standard_normal(cols)).astype(np.float32))
    y = ops.rmsnorm(dev(x), dev(w), 1e-6)
    assert_bf16_close(y, O.rmsnorm_kernel(x, w, 1e-6))
    xd, rd = dev(x), dev(r)
    ops.fused_add_rmsnorm(xd, rd, dev(w), 1e-6)
    y_ref, r_ref = O.rmsnorm_kernel(x, w, 1e-6, r)
    assert np.array_equal(host_bits(rd), O.bf16_round_bits(r_ref))   # the add is exact
    assert_bf16_close(xd, y_ref)
    # and within the stated tolerance of the reference's native formulation
    yn, _ = O.rmsnorm_native(x, w, 1e-6, r)
    np.testing.assert_allclose(host_f32(xd), yn, atol=2e-2, rtol=2e-2)


def test_rmsnorm_golden_inputs(ops, golden):
    rc = cases.rope_store_case(21, 6, 256, 4, 2, 128, 4, 64, 64, qk_norm=True)
    y = ops.rmsnorm(dev(rc["x"]), dev(rc["norm_w"]), 1e-6)
    np.testing.assert_allclose(host_f32(y), O.bf16_bits_to_f32(golden["rms_plain"]),
                               atol=2e-2, rtol=2e-2)
    xd, rd = dev(rc["x"]), dev(rc["residual"])
    ops.fused_add_rmsnorm(xd, rd, dev(rc["norm_w"]), 1e-6)
    assert np.array_equal(host_bits(rd), golden["rms_fused_res"])
    np.testing.assert_allclose(host_f32(xd), O.bf16_bits_to_f32(golden["rms_fused_y"]),
                               atol=2e-2, rtol=2e-2)


def test_rmsnorm_per_head_strided_view(ops, golden):
    rc = cases.rope_store_case(21, 6, 256, 4, 2, 128, 4, 64, 64, qk_norm=True)
    qkv = dev(rc["qkv"])
    q3 = qkv[:, :512].view(6, 4, 128)                   # row stride 1024, not 512
    y = ops.rmsnorm(q3, dev(rc["q_norm_w"]), 1e-6)
    want = O.rmsnorm_kernel(rc["qkv"][:, :512].reshape(6, 4, 128), rc["q_norm_w"], 1e-6)
    assert_bf16_close(y, want)
    np.testing.assert_allclose(host_f32(y), O.bf16_bits_to_f32(golden["rms_heads"]),
                               atol=2e-2, rtol=2e-2)


def test_strided_rows_fused(ops):
    rs = np.random.RandomState(9)
    big = cases.randn_bf16(rs, (4, 1024))
    r = cases.randn_bf16(rs, (4, 512))
    w = np.ones(512, np.float32)
    bd = dev(big)
    xv, rd = bd[:, 512:], dev(r)                        # x is a strided view
    ops.fused_add_rmsnorm(xv, rd, dev(w), 1e-5)
    y_ref, r_ref = O.rmsnorm_kernel(big[:, 512:], w, 1e-5, r)
    assert_bf16_close(xv, y_ref)
    assert np.array_equal(host_bits(bd[:, :512].contiguous()), O.bf16_round_bits(big[:, :512]))


# -------------------------------------------------------------------------- rope
@pytest.mark.parametrize("cache_dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("d", [128, 64])
def test_rope_neox_in_place(ops, cache_dtype, d):
    rs = np.random.RandomState(5 + d)
    t, hq, hkv, max_pos = 33, 6, 2, 512
    cache = O.rope_cos_sin_cache(d, max_pos, 1e6)
    qkv = cases.randn_bf16(rs, (t, (hq + 2 * hkv) * d))
    pos = rs.randint(0, max_pos, size=t).astype(np.int64)
    q_np, k_np = qkv[:, :hq * d], qkv[:, hq * d:(hq + hkv) * d]
    q_ref, k_ref = O.rope_neox(pos, q_np, k_np, d, O.bf16_round(cache))
    buf = dev(qkv)
    q, k = buf[:, :hq * d], buf[:, hq * d:(hq + hkv) * d]
    cd = dev(cache, torch.float32) if cache_dtype == "fp32" else dev(cache)
    st = ops.new_status("cuda")
    ops.rope_neox(dev(pos), q, k, d, cd, st)
    assert_bf16_close(q, q_ref, frac=0.01)
    assert_bf16_close(k, k_ref, frac=0.01)
    # v part of the packed rows untouched
    assert np.array_equal(host_bits(buf[:, (hq + hkv) * d:].contiguous()),
                          O.bf16_round_bits(qkv[:, (hq + hkv) * d:]))
    assert int(st.item()) == 0


def test_rope_golden(ops, golden):
    rc = cases.rope_store_case(21, 6, 256, 4, 2, 128, 4, 64, 64, qk_norm=True)
    buf = dev(rc["qkv"])
    ops.rope_neox(dev(rc["positions"]), buf[:, :512], buf[:, 512:768], 128,
                  dev(golden["rope_cache"], torch.float32))
    np.testing.assert_allclose(host_f32(buf[:, :512]), O.bf16_bits_to_f32(golden["rope_q"]),
                               atol=2e-2, rtol=2e-2)
    np.testing.assert_allclose(host_f32(buf[:, 512:768]), O.bf16_bits_to_f32(golden["rope_k"]),
                               atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("qk_norm", [False, True])
def test_qkv_rope_store_fused_chain(ops, qk_norm):
    t, hq, hkv, d, nb, bs, max_pos = 50, 8, 2, 128, 4, 64, 2048
    rc = cases.rope_store_case(77, t, 256, hq, hkv, d, nb, bs, max_pos, qk_norm=qk_norm)
    rc["slots"][[4, 9]] = -1
    cache = O.rope_cos_sin_cache(d, max_pos, 1e6)
    qkv = rc["qkv"]
    q_np, k_np, v_np = np.split(qkv, [hq * d, (hq + hkv) * d], axis=1)
    if qk_norm:
        q_np = O.rmsnorm_kernel(q_np.reshape(t, hq, d), rc["q_norm_w"], 1e-6).reshape(t, -1)
        k_np = O.rmsnorm_kernel(k_np.reshape(t, hkv, d), rc["k_norm_w"], 1e-6).reshape(t, -1)
    q_ref, k_ref = O.rope_neox(rc["positions"], q_np, k_np, d, O.bf16_round(cache))

    buf = dev(qkv)
    kc = torch.zeros((nb, bs, hkv, d), dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    st = ops.new_status("cuda")
    ops.qkv_rope_store(buf, hq, hkv, d, dev(rc["positions"]), dev(cache, torch.float32),
                       dev(rc["q_norm_w"]) if qk_norm else None,
                       dev(rc["k_norm_w"]) if qk_norm else None, 1e-6, kc, vc,
                       dev(rc["slots"]), st)
    assert int(st.item()) == 0
    # with the per-head norm in the chain, a 1-ulp difference of the normed
    # value (fp32 reduction order) can become 2 ulp after the rotation
    ulp = 2 if qk_norm else 1
    assert_bf16_close(buf[:, :hq * d], q_ref, max_ulp=ulp, frac=0.03)
    assert_bf16_close(buf[:, hq * d:(hq + hkv) * d], k_ref, max_ulp=ulp, frac=0.03)
    # the cache holds exactly the rotated k the kernel wrote in place, and raw v
    k_gpu = host_bits(buf[:, hq * d:(hq + hkv) * d].contiguous()).reshape(t, hkv, d)
    kc_ref = np.zeros((nb * bs, hkv, d), np.uint16)
    vc_ref = np.zeros_like(kc_ref)
    O.store_kvcache(k_gpu, O.bf16_round_bits(v_np).reshape(t, hkv, d), kc_ref, vc_ref,
                    rc["slots"])
    assert np.array_equal(host_bits(kc).reshape(kc_ref.shape), kc_ref)
    assert np.array_equal(host_bits(vc).reshape(vc_ref.shape), vc_ref)


def test_rope_bad_position_is_flagged_not_faulted(ops):
    t, d = 4, 128
    cache = dev(O.rope_cos_sin_cache(d, 16, 1e4), torch.float32)
    q = torch.ones((t, 2 * d), dtype=torch.bfloat16, device="cuda")
    k = torch.ones((t, d), dtype=torch.bfloat16, device="cuda")
    st = ops.new_status("cuda")
    ops.rope_neox(torch.tensor([0, 3, 99, 2], device="cuda"), q, k, d, cache, st)
    assert int(st.item()) == 8
    assert torch.equal(q[2], torch.ones(2 * d, dtype=torch.bfloat16, device="cuda"))


# -------------------------------------------------------------------------- silu
@pytest.mark.parametrize("rows,d", [(7, 96), (64, 12288), (3, 100), (1, 8)])
def test_silu_and_mul(ops, rows, d):
    rs = np.random.RandomState(d)
    x = cases.randn_bf16(rs, (rows, 2 * d), 2.0)
    y = ops.silu_and_mul(dev(x))
    assert_bf16_close(y, O.silu_and_mul(x), frac=0.01)


def test_silu_golden(ops, golden):
    rs = np.random.RandomState(31)
    sx = cases.randn_bf16(rs, (7, 2 * 96), 2.0)
    y = ops.silu_and_mul(dev(sx))
    np.testing.assert_allclose(host_f32(y), O.bf16_bits_to_f32(golden["silu"]), atol=2e-2,
                               rtol=2e-2)


# ------------------------------------------------------------------ argmax / fill
def test_argmax_rows_lowest_index_on_ties(ops):
    rs = np.random.RandomState(4)
    x = cases.randn_bf16(rs, (9, 151936), 1.0)
    x[0, 70000] = x[0, 5] = 9.0            # exact tie: the lower index wins
    x[1, 151935] = 11.0                    # last column
    x[2, :] = -3.0                         # all equal -> index 0
    vals, idx = ops.argmax_rows(dev(x))
    assert np.array_equal(idx.cpu().numpy(), x.argmax(axis=1))
    np.testing.assert_array_equal(vals.cpu().numpy(), x.max(axis=1))
    # ragged width / strided rows take the scalar path
    y = cases.randn_bf16(rs, (5, 1003), 1.0)
    big = dev(np.concatenate([y, y], axis=1))
    vals, idx = ops.argmax_rows(big[:, :1003])
    assert np.array_equal(idx.cpu().numpy(), y.argmax(axis=1))


def test_fill_u32(ops):
    t = torch.full((1000003,), 7, dtype=torch.int32, device="cuda")[:1000000]
    ops.fill_u32(t, 0xDEADBEEF)
    assert int((t.view(torch.int32) != -559038737).sum()) == 0
    small = torch.ones(3, dtype=torch.float32, device="cuda")
    ops.fill_u32(small, 0)
    assert not small.any()


def test_xor_checksum_matches_numpy():
    """fk_xor_u32: XOR of all 32-bit words, accumulated into *out; sizes around the
    unrolled loop's stride, and a second call folding into the same word."""
    from fastkernels_b200 import ops
    rs = np.random.RandomState(11)
    acc = 0
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    for words in (4, 36, 4096, 148 * 16 * 512 * 4 * 8 + 12, 3 * 1000 * 1000 * 4):
        a = rs.randint(0, 2 ** 32, size=words, dtype=np.uint64).astype(np.uint32)
        t = torch.from_numpy(a.view(np.int32)).cuda()
        single = ops.xor_u32(t)
        ops.xor_u32(t, out)
        torch.cuda.synchronize()
        ref = int(np.bitwise_xor.reduce(a))
        acc ^= ref
        assert int(single.item()) & 0xffffffff == ref
        assert int(out.item()) & 0xffffffff == acc
