"""The persistent decode block (fk_decode_block) through the C-ABI: programs of
projections, residual-add + RMSNorms and the split + RoPE + KV store, against the
oracle's composition of the same ops (LlamaDecoderLayer.forward,
fastkernels/tasks/baseline/L3/llama_decoder.py:34-42, between two attention
calls) and against this build's one-kernel-per-op entry points."""
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


def close(got, ref, max_ulp=3, beyond=1e-4, differing=0.12):
    """Inside the bf16 tolerance of the path (2e-2) everywhere; bit-identical to the
    oracle except for `differing` of the elements; further than `max_ulp` bf16 steps
    only where a rotation or a sum nearly cancels (at most `beyond` of the elements:
    a step is relative to the result, the rounding error to the operands)."""
    g = host_f32(got)
    np.testing.assert_allclose(g, ref, atol=2e-2, rtol=2e-2)
    gb, wb = O.bf16_round_bits(g).astype(np.int32), O.bf16_round_bits(ref).astype(np.int32)
    big = (np.abs(ref) >= 1e-3) & (((gb ^ wb) & 0x8000) == 0)
    steps = np.abs((gb & 0x7FFF) - (wb & 0x7FFF))[big]
    assert (steps > max_ulp).mean() <= beyond, (steps > max_ulp).mean()
    assert (steps > 0).mean() <= differing, (steps > 0).mean()


@pytest.mark.parametrize("m,hidden,ffn,hq,hkv", [
    (64, 1024, 2048, 8, 2),      # a few tiles: most CTAs idle in some phases
    (5, 512, 1024, 4, 2),        # a handful of rows (16-row accumulator)
    (100, 1024, 3072, 8, 8),     # 128-row accumulator, no prefetch of partial tiles
    (64, 4096, 12288, 32, 8),    # the 8B shape at its own width
])
def test_layer_program_matches_oracle(ops, m, hidden, ffn, hq, hkv):
    d, eps, nb, bs, max_pos = 128, 1e-6, 8, 64, 2048
    rs = np.random.RandomState(m + hidden)
    sc = 1.0 / np.sqrt(hidden)
    w_o = cases.randn_bf16(rs, (hidden, hq * d), 1.0 / np.sqrt(hq * d))
    w_gu = cases.randn_bf16(rs, (2 * ffn, hidden), sc)
    w_dn = cases.randn_bf16(rs, (hidden, ffn), 1.0 / np.sqrt(ffn))
    w_qkv = cases.randn_bf16(rs, ((hq + 2 * hkv) * d, hidden), sc)
    ln2 = O.bf16_round((1 + 0.05 * rs.standard_normal(hidden)).astype(np.float32))
    ln1 = O.bf16_round((1 + 0.05 * rs.standard_normal(hidden)).astype(np.float32))
    qn = O.bf16_round((1 + 0.1 * rs.standard_normal(d)).astype(np.float32))
    kn = O.bf16_round((1 + 0.1 * rs.standard_normal(d)).astype(np.float32))
    attn_out = cases.randn_bf16(rs, (m, hq * d), 0.5)
    residual = cases.randn_bf16(rs, (m, hidden))
    pos = rs.randint(0, max_pos, size=m).astype(np.int64)
    slots = rs.permutation(nb * bs)[:m].astype(np.int32)
    slots[m // 2] = -1                                   # a padded row
    cache = O.bf16_round(O.rope_cos_sin_cache(d, max_pos, 1e6))

    res_d = dev(residual)
    kc = torch.zeros((nb, bs, hkv, d), dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    st = ops.new_status("cuda")
    prog = ops.BlockProgram(m, "cuda")
    yd = prog.gemm(dev(attn_out), dev(w_o))
    xd = prog.add_rmsnorm(yd, res_d, dev(ln2), eps)
    act = prog.gemm_silu_mul(xd, dev(w_gu))
    y2d = prog.gemm(act, dev(w_dn))
    hd = prog.add_rmsnorm(y2d, res_d, dev(ln1), eps)
    qkv = prog.gemm(hd, dev(w_qkv))
    prog.qkv_rope_store(qkv, hq, hkv, d, dev(pos), dev(cache), dev(qn), dev(kn), eps, kc, vc,
                        dev(slots))
    prog.launch(status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0, f"device status {int(st.item())}"
    # Every op is checked from the inputs the kernel itself gave it (the GPU's own
    # intermediate tensors), so each comparison carries the tolerance of ONE op and
    # differences do not pile up along the chain.
    f = host_f32
    assert_bf16_close(yd, O.linear(attn_out, w_o), max_ulp=1, frac=0.03)
    x_ref, res1 = O.rmsnorm_kernel(f(yd), ln2, eps, residual)
    assert_bf16_close(xd, x_ref, max_ulp=1, frac=0.03)
    act_ref = O.silu_and_mul(O.linear(f(xd), w_gu))
    np.testing.assert_allclose(f(act), act_ref, atol=2e-2, rtol=2e-2)
    gb = O.bf16_round_bits(f(act)).astype(np.int32)
    wb = O.bf16_round_bits(act_ref).astype(np.int32)
    big = (np.abs(act_ref) >= 1e-3) & (((gb ^ wb) & 0x8000) == 0)
    assert (np.abs((gb & 0x7FFF) - (wb & 0x7FFF))[big] > 2).mean() <= 1e-4
    assert_bf16_close(y2d, O.linear(f(act), w_dn), max_ulp=1, frac=0.03)
    h_ref, res2 = O.rmsnorm_kernel(f(y2d), ln1, eps, res1)
    assert np.array_equal(host_bits(res_d), O.bf16_round_bits(res2)), "residual not bit-exact"
    assert_bf16_close(hd, h_ref, max_ulp=1, frac=0.03)
    qkv_ref = O.linear(f(hd), w_qkv)
    q_np, k_np, v_np = np.split(qkv_ref, [hq * d, (hq + hkv) * d], axis=1)
    q_np = O.rmsnorm_kernel(q_np.reshape(m, hq, d), qn, eps).reshape(m, -1)
    k_np = O.rmsnorm_kernel(k_np.reshape(m, hkv, d), kn, eps).reshape(m, -1)
    q_ref, k_ref = O.rope_neox(pos, q_np, k_np, d, cache)
    # projection, per-head norm and rotation each round once: up to three steps
    close(qkv[:, :hq * d], q_ref)
    close(qkv[:, hq * d:(hq + hkv) * d], k_ref)
    assert_bf16_close(qkv[:, (hq + hkv) * d:], v_np, max_ulp=1, frac=0.03)
    # the cache rows are the kernel's own rotated k / raw v rows, bit for bit
    k_gpu = host_bits(qkv[:, hq * d:(hq + hkv) * d].contiguous()).reshape(m, hkv, d)
    v_gpu = host_bits(qkv[:, (hq + hkv) * d:].contiguous()).reshape(m, hkv, d)
    kc_ref = np.zeros((nb * bs, hkv, d), np.uint16)
    vc_ref = np.zeros_like(kc_ref)
    O.store_kvcache(k_gpu, v_gpu, kc_ref, vc_ref, slots)
    assert np.array_equal(host_bits(kc).reshape(kc_ref.shape), kc_ref)
    assert np.array_equal(host_bits(vc).reshape(vc_ref.shape), vc_ref)

    # the workspace (stream-K flags, barrier counter) is left zeroed: a second,
    # different launch right behind the first gives the right answer too
    prog2 = ops.BlockProgram(m, "cuda")
    y_again = prog2.gemm(dev(attn_out), dev(w_o))
    prog2.launch(status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert torch.equal(y_again.view(torch.int16), yd.view(torch.int16))
    # and against the stand-alone projection kernel (same arithmetic, other split points)
    assert_bf16_close(yd, host_f32(ops.gemm_bf16(dev(attn_out), dev(w_o))), max_ulp=1, frac=0.03)


def test_first_layer_program_and_final_norm(ops):
    """[norm without add, qkv, RoPE + store] as run before the first attention call,
    and [down, add + final norm] as run after the last layer; no q/k norm weights,
    a projection bias, HND pages of 16 tokens."""
    m, hidden, hq, hkv, d, eps = 7, 512, 4, 2, 128, 1e-5
    nb, page, max_pos = 6, 16, 512
    rs = np.random.RandomState(9)
    emb = cases.randn_bf16(rs, (m, hidden))
    ln = O.bf16_round((1 + 0.05 * rs.standard_normal(hidden)).astype(np.float32))
    w_qkv = cases.randn_bf16(rs, ((hq + 2 * hkv) * d, hidden), 0.05)
    b_qkv = cases.randn_bf16(rs, ((hq + 2 * hkv) * d,), 0.1)
    pos = rs.randint(0, max_pos, size=m).astype(np.int64)
    slots = rs.permutation(nb * page)[:m].astype(np.int32)
    cache = O.bf16_round(O.rope_cos_sin_cache(d, max_pos, 5e5))
    x_ref = O.rmsnorm_kernel(emb, ln, eps)
    qkv_ref = O.linear(x_ref, w_qkv, b_qkv)
    q_np, k_np, v_np = np.split(qkv_ref, [hq * d, (hq + hkv) * d], axis=1)
    q_ref, k_ref = O.rope_neox(pos, q_np, k_np, d, cache)
    kc = torch.zeros((nb, hkv, page, d), dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    res_d = dev(emb)
    st = ops.new_status("cuda")
    prog = ops.BlockProgram(m, "cuda")
    xd = prog.add_rmsnorm(None, res_d, dev(ln), eps)
    qkv = prog.gemm(xd, dev(w_qkv), dev(b_qkv))
    prog.qkv_rope_store(qkv, hq, hkv, d, dev(pos), dev(cache), None, None, eps, kc, vc,
                        dev(slots), kv_layout="HND")
    prog.launch(status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert np.array_equal(host_bits(res_d), O.bf16_round_bits(emb))      # residual untouched
    assert_bf16_close(xd, x_ref, max_ulp=1, frac=0.02)
    close(qkv[:, :hq * d], q_ref)
    close(qkv[:, hq * d:(hq + hkv) * d], k_ref)
    k_gpu = host_bits(qkv[:, hq * d:(hq + hkv) * d].contiguous()).reshape(m, hkv, d)
    v_gpu = host_bits(qkv[:, (hq + hkv) * d:].contiguous()).reshape(m, hkv, d)
    kc_ref = np.zeros((nb, hkv, page, d), np.uint16)
    vc_ref = np.zeros_like(kc_ref)
    O.store_kvcache_hnd(k_gpu, v_gpu, kc_ref, vc_ref, slots)
    assert np.array_equal(host_bits(kc), kc_ref) and np.array_equal(host_bits(vc), vc_ref)

    # [down projection, add + final norm]
    ffn = 1024
    act = cases.randn_bf16(rs, (m, ffn), 0.5)
    w_dn = cases.randn_bf16(rs, (hidden, ffn), 0.03)
    res = cases.randn_bf16(rs, (m, hidden))
    out_ref, res_ref = O.rmsnorm_kernel(O.linear(act, w_dn), ln, eps, res)
    res_d = dev(res)
    prog = ops.BlockProgram(m, "cuda")
    y = prog.gemm(dev(act), dev(w_dn))
    out = prog.add_rmsnorm(y, res_d, dev(ln), eps)
    prog.launch(status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    close(res_d, res_ref)
    close(out, out_ref)


def test_block_validation_refuses_before_launch(ops):
    from fastkernels_b200 import _lib
    before = _lib.lib.fk_launch_count()
    x = torch.zeros((129, 256), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((256, 256), dtype=torch.bfloat16, device="cuda")
    prog = ops.BlockProgram(129, "cuda")
    prog.gemm(x, w)
    with pytest.raises(_lib.FkError, match="FK_ERR_UNSUPPORTED"):
        prog.launch()
    prog = ops.BlockProgram(4, "cuda")
    for _ in range(5):                                    # five projections: one too many
        prog.gemm(x[:4], w)
    with pytest.raises(_lib.FkError, match="FK_ERR_UNSUPPORTED"):
        prog.launch()
    assert _lib.lib.fk_launch_count() == before
