"""GPU parity of the prefill-side kernels (through the C-ABI) against the oracle:
variable-length causal attention over dense and paged K/V, and the merge of two
partial attention results.  Tolerance of the bf16 path: atol = rtol = 2e-2."""
import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

ATOL = RTOL = 2e-2


def _dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def _close(got, want, what):
    got = got.float().cpu().numpy()
    err = np.abs(got - want)
    bad = err > ATOL + RTOL * np.abs(want)
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside tolerance, max err {err.max():.4g}"
    return float(err.max())


SHAPES = [
    # q_lens, k_lens, hq, hkv
    ([1], [1], 2, 1),
    ([5, 127, 128, 129], [5, 127, 128, 129], 4, 2),
    ([256, 257, 300], [256, 257, 300], 4, 1),
    ([1, 64, 200], [300, 64, 777], 8, 2),        # chunks after a cached prefix
    ([513], [1100], 2, 2),
]


@pytest.mark.parametrize("q_lens,k_lens,hq,hkv", SHAPES)
@pytest.mark.parametrize("causal", [True, False])
def test_prefill_dense(q_lens, k_lens, hq, hkv, causal):
    from fastkernels_b200 import ops
    from oracle import decode_oracle as orc
    c = cases.prefill_case(31, q_lens, k_lens, hq, hkv)
    want, want_lse = orc.prefill_attention(c["q"], c["k"], c["v"], c["cu_q"], c["cu_k"],
                                           c["scale"], causal=causal)
    st = ops.new_status("cuda")
    out, lse = ops.prefill_attn(_dev(c["q"], torch.bfloat16), _dev(c["k"], torch.bfloat16),
                                _dev(c["v"], torch.bfloat16), _dev(c["cu_q"]), _dev(c["cu_k"]),
                                c["max_q"], c["scale"], causal=causal, return_lse=True, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    _close(out, want, "out")
    _close(lse, want_lse, "lse")


@pytest.mark.parametrize("block_size,layout", [(64, "NHD"), (256, "NHD"), (16, "HND"), (32, "NHD")])
def test_prefill_paged(block_size, layout):
    from fastkernels_b200 import ops
    from oracle import decode_oracle as orc
    c = cases.prefill_case(32, [3, 190, 260], [260, 190, 700], 8, 2, block_size=block_size)
    want, want_lse = orc.prefill_attention(c["q"], c["k_cache"], c["v_cache"], c["cu_q"],
                                           c["cu_k"], c["scale"], block_tables=c["block_tables"],
                                           block_size=block_size)
    kc, vc = _dev(c["k_cache"], torch.bfloat16), _dev(c["v_cache"], torch.bfloat16)
    if layout == "HND":
        kc, vc = kc.permute(0, 2, 1, 3).contiguous(), vc.permute(0, 2, 1, 3).contiguous()
    st = ops.new_status("cuda")
    out, lse = ops.prefill_attn(_dev(c["q"], torch.bfloat16), kc, vc, _dev(c["cu_q"]),
                                _dev(c["cu_k"]), c["max_q"], c["scale"],
                                block_table=_dev(c["block_tables"]), kv_layout=layout,
                                return_lse=True, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    _close(out, want, "out")
    _close(lse, want_lse, "lse")


def test_prefill_strided_views_and_no_keys():
    """q / k / v as views into a packed qkv buffer (the engine's layout), plus a
    sequence with no keys at all."""
    from fastkernels_b200 import ops
    from oracle import decode_oracle as orc
    hq, hkv, d = 4, 2, 128
    c = cases.prefill_case(33, [70, 0, 140], [70, 0, 140], hq, hkv)
    tq = c["q"].shape[0]
    qkv = torch.zeros((tq, (hq + 2 * hkv) * d), dtype=torch.bfloat16, device="cuda")
    qkv[:, :hq * d] = _dev(c["q"], torch.bfloat16).view(tq, -1)
    qkv[:, hq * d:(hq + hkv) * d] = _dev(c["k"], torch.bfloat16).view(tq, -1)
    qkv[:, (hq + hkv) * d:] = _dev(c["v"], torch.bfloat16).view(tq, -1)
    q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
    want, _ = orc.prefill_attention(c["q"], c["k"], c["v"], c["cu_q"], c["cu_k"], c["scale"])
    out = ops.prefill_attn(q.view(tq, hq, d), k.view(tq, hkv, d), v.view(tq, hkv, d),
                           _dev(c["cu_q"]), _dev(c["cu_k"]), c["max_q"], c["scale"])
    torch.cuda.synchronize()
    _close(out, want, "out")


def test_prefill_bad_page_is_flagged():
    from fastkernels_b200 import ops
    c = cases.prefill_case(34, [100], [100], 2, 1, block_size=64)
    bt = c["block_tables"].copy()
    bt[0, 1] = 10 ** 6
    st = ops.new_status("cuda")
    ops.prefill_attn(_dev(c["q"], torch.bfloat16), _dev(c["k_cache"], torch.bfloat16),
                     _dev(c["v_cache"], torch.bfloat16), _dev(c["cu_q"]), _dev(c["cu_k"]),
                     c["max_q"], c["scale"], block_table=_dev(bt), status=st)
    torch.cuda.synchronize()
    assert int(st.item()) & 2


def test_prefill_split_and_merge_equals_whole():
    """Attention over [prefix | suffix] keys = merge(attention over the prefix,
    attention over the suffix): ties the two kernels together at a larger size."""
    from fastkernels_b200 import ops
    from oracle import decode_oracle as orc
    hq, hkv, d, n, cut = 8, 2, 128, 640, 384
    c = cases.prefill_case(35, [n], [n + cut], hq, hkv)
    q = _dev(c["q"], torch.bfloat16)
    k, v = _dev(c["k"], torch.bfloat16), _dev(c["v"], torch.bfloat16)
    cu_q = _dev(c["cu_q"])
    whole, whole_lse = ops.prefill_attn(q, k, v, cu_q, _dev(c["cu_k"]), n, c["scale"],
                                        return_lse=True)
    cu_pre = _dev(np.array([0, cut], dtype=np.int32))
    cu_suf = _dev(np.array([0, n], dtype=np.int32))
    pre, pre_lse = ops.prefill_attn(q, k[:cut], v[:cut], cu_q, cu_pre, n, c["scale"],
                                    causal=False, return_lse=True)
    suf, suf_lse = ops.prefill_attn(q, k[cut:], v[cut:], cu_q, cu_suf, n, c["scale"],
                                    causal=True, return_lse=True)
    merged = torch.empty_like(whole)
    merged_lse = torch.empty_like(whole_lse)
    ops.merge_attn_states(merged, pre, pre_lse, suf, suf_lse, merged_lse)
    torch.cuda.synchronize()
    want, want_lse = orc.prefill_attention(c["q"], c["k"], c["v"], c["cu_q"], c["cu_k"], c["scale"])
    _close(whole, want, "whole")
    _close(merged, want, "merged")
    _close(merged_lse, want_lse, "merged lse")


def test_merge_attn_states_matches_oracle():
    from fastkernels_b200 import ops
    from oracle import decode_oracle as orc
    rs = np.random.RandomState(36)
    t, h, d = 37, 5, 128
    a = cases.randn_bf16(rs, (t, h, d), 1.0)
    b = cases.randn_bf16(rs, (t, h, d), 1.0)
    la = rs.randn(h, t).astype(np.float32) * 3
    lb = rs.randn(h, t).astype(np.float32) * 3
    la[0, 0] = -np.inf                       # one side empty
    lb[1, 1] = np.inf                        # +inf counts as -inf
    la[2, 2] = lb[2, 2] = -np.inf            # both empty: prefix passes through
    for ctx in (None, 20):
        want, want_lse = orc.merge_attn_states(a, la, b, lb, prefill_tokens_with_context=ctx)
        out = torch.empty((t, h, d), dtype=torch.bfloat16, device="cuda")
        out_lse = torch.empty((h, t), dtype=torch.float32, device="cuda")
        ops.merge_attn_states(out, _dev(a, torch.bfloat16), _dev(la), _dev(b, torch.bfloat16),
                              _dev(lb), out_lse, prefill_tokens_with_context=ctx)
        torch.cuda.synchronize()
        got = out.float().cpu().numpy()
        # one bf16 rounding of an fp32 expression: at most 1 ulp apart
        assert np.abs(got - want).max() <= np.abs(want).max() * 2 ** -7
        assert (got == want).mean() > 0.97
        gl = out_lse.cpu().numpy()
        fin = np.isfinite(want_lse)
        assert (np.isfinite(gl) == fin).all()
        assert np.abs(gl[fin] - want_lse[fin]).max() < 1e-5


def test_prefill_many_items_per_cta():
    """More work items than SMs (several rounds of the persistent CTAs), ragged
    lengths, prefixes, empty sequences in between; paged pool."""
    from fastkernels_b200 import ops
    from oracle import decode_oracle as orc
    rs = np.random.RandomState(37)
    q_lens = [int(x) for x in rs.randint(0, 700, size=12)]
    q_lens[3] = 0
    k_lens = [q + int(rs.randint(0, 300)) if q else 0 for q in q_lens]
    c = cases.prefill_case(37, q_lens, k_lens, 16, 4, block_size=64)
    want, want_lse = orc.prefill_attention(c["q"], c["k"], c["v"], c["cu_q"], c["cu_k"], c["scale"])
    st = ops.new_status("cuda")
    out, lse = ops.prefill_attn(_dev(c["q"], torch.bfloat16), _dev(c["k_cache"], torch.bfloat16),
                                _dev(c["v_cache"], torch.bfloat16), _dev(c["cu_q"]),
                                _dev(c["cu_k"]), c["max_q"], c["scale"],
                                block_table=_dev(c["block_tables"]), return_lse=True, status=st)
    out2 = ops.prefill_attn(_dev(c["q"], torch.bfloat16), _dev(c["k"], torch.bfloat16),
                            _dev(c["v"], torch.bfloat16), _dev(c["cu_q"]), _dev(c["cu_k"]),
                            c["max_q"], c["scale"])
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    _close(out, want, "paged")
    _close(out2, want, "dense")
    _close(lse, want_lse, "lse")


@pytest.mark.parametrize("seed", list(range(10)))
def test_prefill_random_shapes(seed):
    """Seeded random batches: head counts, GQA ratios, page sizes, layouts, ragged
    query / key lengths (prefixes, empty sequences), causal or not."""
    from fastkernels_b200 import ops
    from oracle import decode_oracle as orc
    rs = np.random.RandomState(1000 + seed)
    g = int(rs.choice([1, 2, 4, 8]))
    hkv = int(rs.choice([1, 2, 3]))
    hq = g * hkv
    nseq = int(rs.randint(1, 6))
    q_lens = [int(rs.choice([0, 1, 7, 100, 128, 129, 255, 256, 257, 400, 520])) for _ in range(nseq)]
    if sum(q_lens) == 0:
        q_lens[0] = 33
    k_lens = [q + int(rs.choice([0, 0, 5, 128, 300])) if q else int(rs.choice([0, 40])) for q in q_lens]
    causal = bool(rs.randint(0, 2))
    block = int(rs.choice([16, 32, 64, 128, 256]))
    layout = str(rs.choice(["NHD", "HND"]))
    c = cases.prefill_case(2000 + seed, q_lens, k_lens, hq, hkv, block_size=block)
    want, want_lse = orc.prefill_attention(c["q"], c["k"], c["v"], c["cu_q"], c["cu_k"], c["scale"],
                                           causal=causal)
    kc, vc = _dev(c["k_cache"], torch.bfloat16), _dev(c["v_cache"], torch.bfloat16)
    if layout == "HND":
        kc, vc = kc.permute(0, 2, 1, 3).contiguous(), vc.permute(0, 2, 1, 3).contiguous()
    st = ops.new_status("cuda")
    q = _dev(c["q"], torch.bfloat16)
    paged, lse = ops.prefill_attn(q, kc, vc, _dev(c["cu_q"]), _dev(c["cu_k"]), max(c["max_q"], 1),
                                  c["scale"], causal=causal, block_table=_dev(c["block_tables"]),
                                  kv_layout=layout, return_lse=True, status=st)
    dense = ops.prefill_attn(q, _dev(c["k"], torch.bfloat16), _dev(c["v"], torch.bfloat16),
                             _dev(c["cu_q"]), _dev(c["cu_k"]), max(c["max_q"], 1), c["scale"],
                             causal=causal, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    what = f"g={g} hkv={hkv} q={q_lens} k={k_lens} causal={causal} block={block} {layout}"
    _close(paged, want, "paged " + what)
    _close(dense, want, "dense " + what)
    fin = np.isfinite(want_lse)
    got_lse = lse.cpu().numpy()
    assert (np.isfinite(got_lse) == fin).all(), what
    assert np.abs(got_lse[fin] - want_lse[fin]).max() < 2e-2, what
