"""GPU parity (through the C-ABI) of paged GQA decode attention."""
import numpy as np
import pytest
import torch

import cases
from gpu_util import dev, host_f32
from oracle import decode_oracle as O

pytestmark = pytest.mark.gpu

ATOL = RTOL = 2e-2          # the stated bf16 tolerance
TIGHT = 6e-3                # what the kernel is expected to achieve


@pytest.fixture(scope="module")
def ops():
    from fastkernels_b200 import ops as _ops
    return _ops


def run(ops, c, max_splits=16, bt_pad=0, status=None):
    q, kc, vc = dev(c["q"]), dev(c["k_cache"]), dev(c["v_cache"])
    bt = c["block_tables"]
    if bt_pad:
        bt = np.concatenate([bt, np.full((bt.shape[0], bt_pad), -1, np.int32)], axis=1)
    b, hq, d = c["q"].shape
    ws = torch.empty(ops.attn_workspace_bytes(b, hq, d, max_splits), dtype=torch.uint8,
                     device="cuda")
    out = ops.paged_decode_attn(q, kc, vc, dev(c["context_lens"]), dev(bt), c["scale"], ws,
                                max_splits, status=status)
    torch.cuda.synchronize()
    return out


def check(out, ref, tight=TIGHT):
    g = host_f32(out)
    np.testing.assert_allclose(g, ref, atol=ATOL, rtol=RTOL)
    assert np.abs(g - ref).max() <= tight, np.abs(g - ref).max()


def oracle(c):
    return O.paged_decode_attention(c["q"], c["k_cache"], c["v_cache"], c["context_lens"],
                                    c["block_tables"], c["scale"])


def test_small_ragged_matches_golden(ops, golden):
    c = cases.attention_case(11, 5, 8, 2, 128, 64, 12, lens=[1, 63, 64, 65, 200])
    st = ops.new_status("cuda")
    out = run(ops, c, status=st)
    check(out, golden["attn_small"])
    assert int(st.item()) == 0


def test_gqa16_matches_golden(ops, golden):
    c = cases.attention_case(12, 3, 16, 1, 128, 64, 16, lens=[7, 129, 500])
    check(run(ops, c), golden["attn_g16"])


def test_config1_store_then_attend_matches_golden(ops, golden):
    c = cases.config1_case()
    kc, vc = dev(c["k_cache"]), dev(c["v_cache"])
    ops.store_kvcache(dev(c["new_k"]), dev(c["new_v"]), kc, vc, dev(c["slot_mapping"]))
    b, hq, d = c["q"].shape
    ws = torch.empty(ops.attn_workspace_bytes(b, hq, d, 32), dtype=torch.uint8, device="cuda")
    out = ops.paged_decode_attn(dev(c["q"]), kc, vc, dev(c["context_lens"]),
                                dev(c["block_tables"]), c["scale"], ws, 32)
    check(out, golden["attn_c1"])


@pytest.mark.parametrize("g,hkv", [(1, 4), (2, 2), (4, 2), (8, 1), (16, 2)])
def test_gqa_ratios(ops, g, hkv):
    c = cases.attention_case(100 + g, 6, g * hkv, hkv, 128, 128, None, len_range=(1, 900))
    check(run(ops, c), oracle(c))


@pytest.mark.parametrize("max_splits", [1, 2, 64])
def test_split_bounds(ops, max_splits):
    """max_splits = 1 forces one chunk per sequence (no merge); 64 lets the
    planner cut 128-token chunks: same answer either way."""
    c = cases.attention_case(7, 4, 8, 2, 128, 256, None, lens=[2047, 300, 1, 1025])
    check(run(ops, c, max_splits=max_splits), oracle(c))


@pytest.mark.parametrize("layout,page", [("HND", 16), ("HND", 32), ("HND", 64),
                                         ("NHD", 16), ("NHD", 32)])
def test_small_pages_and_hnd_layout(ops, layout, page):
    """Page sizes below the 64-token TMA box (one copy per page) and the HND
    pool the reference uses by default on B200 (page 16)."""
    c = cases.attention_case(40 + page, 7, 16, 2, 128, page, None,
                             lens=[1, page - 1, page, page + 1, 129, 1000, 2500])
    ref = oracle(c)
    q = dev(c["q"])
    kc, vc = c["k_cache"], c["v_cache"]
    if layout == "HND":
        kc = np.ascontiguousarray(np.transpose(kc, (0, 2, 1, 3)))
        vc = np.ascontiguousarray(np.transpose(vc, (0, 2, 1, 3)))
    b, hq, d = c["q"].shape
    ws = torch.empty(ops.attn_workspace_bytes(b, hq, d, 32), dtype=torch.uint8, device="cuda")
    st = ops.new_status("cuda")
    out = ops.paged_decode_attn(q, dev(kc), dev(vc), dev(c["context_lens"]),
                                dev(c["block_tables"]), c["scale"], ws, 32, status=st,
                                kv_layout=layout)
    check(out, ref)
    assert int(st.item()) == 0


def test_one_plan_serves_several_layers(ops):
    """The engine plans the split schedule once per step; every layer then calls
    the planned entry point with its own q / K / V but the same lengths, block
    tables and workspace.  Results must equal the self-planning call."""
    c = cases.attention_case(21, 6, 16, 4, 128, 128, None, lens=[1500, 7, 128, 129, 3000, 640])
    b, hq, d = c["q"].shape
    ws = torch.empty(ops.attn_workspace_bytes(b, hq, d, 16), dtype=torch.uint8, device="cuda")
    lens, bt = dev(c["context_lens"]), dev(c["block_tables"])
    st = ops.new_status("cuda")
    ops.paged_decode_attn_plan(lens, bt, 128, hq, 4, d, ws, 16, status=st)
    rs = np.random.RandomState(5)
    for layer in range(3):
        q = cases.randn_bf16(rs, c["q"].shape, 0.5)
        kc = cases.randn_bf16(rs, c["k_cache"].shape, 0.5)
        vc = cases.randn_bf16(rs, c["v_cache"].shape, 0.5)
        out = ops.paged_decode_attn(dev(q), dev(kc), dev(vc), lens, bt, c["scale"], ws, 16,
                                    status=st, planned=True)
        ref = O.paged_decode_attention(q, kc, vc, c["context_lens"], c["block_tables"],
                                       c["scale"])
        check(out, ref)
    assert int(st.item()) == 0


@pytest.mark.parametrize("hq,hkv", [(8, 2), (16, 1)])
def test_small_call_runs_as_one_launch_and_matches_the_planned_path(ops, hq, hkv):
    """A self-planning call with at most one (sequence, KV head) pair per SM and
    short block tables is a single launch (no plan, no merge); empty sequences give
    zero rows there too.  Same oracle, same tolerance as the three-launch path,
    which the planned entry point still takes for the same inputs."""
    from fastkernels_b200 import _lib
    c = cases.attention_case(31, 6, hq, hkv, 128, 64, None, lens=[0, 1, 130, 700, 0, 64])
    ref = oracle(c)
    before = _lib.lib.fk_launch_count()
    out = run(ops, c)
    assert _lib.lib.fk_launch_count() - before == 1
    check(out, ref)
    assert (host_f32(out)[[0, 4]] == 0).all()
    # the planned path on the same tensors
    b, _, d = c["q"].shape
    ws = torch.empty(ops.attn_workspace_bytes(b, hq, d, 16), dtype=torch.uint8, device="cuda")
    lens, bt = dev(c["context_lens"]), dev(c["block_tables"])
    st = ops.new_status("cuda")
    ops.paged_decode_attn_plan(lens, bt, 64, hq, hkv, d, ws, 16, status=st)
    before = _lib.lib.fk_launch_count()
    out2 = ops.paged_decode_attn(dev(c["q"]), dev(c["k_cache"]), dev(c["v_cache"]), lens, bt,
                                 c["scale"], ws, 16, status=st, planned=True)
    torch.cuda.synchronize()
    assert _lib.lib.fk_launch_count() - before == 2
    check(out2, ref)
    assert int(st.item()) == 0


def test_padded_rows_and_wide_block_table(ops):
    """context_len 0 rows (graph padding) give zeros; extra -1 columns and a
    row stride larger than the live column count are ignored."""
    c = cases.attention_case(8, 5, 8, 2, 128, 64, 40, lens=[130, 0, 64, 0, 5])
    out = run(ops, c, bt_pad=7)
    ref = oracle(c)
    check(out, ref)
    assert not host_f32(out)[[1, 3]].any()


def test_strided_q_and_out_views(ops):
    c = cases.attention_case(9, 3, 8, 2, 128, 64, None, lens=[100, 257, 31])
    hq, hkv, d = 8, 2, 128
    qkv = torch.zeros((3, (hq + 2 * hkv) * d), dtype=torch.bfloat16, device="cuda")
    qkv[:, :hq * d] = dev(c["q"]).view(3, -1)
    q = qkv[:, :hq * d].view(3, hq, d)
    ws = torch.empty(ops.attn_workspace_bytes(3, hq, d, 8), dtype=torch.uint8, device="cuda")
    out = ops.paged_decode_attn(q, dev(c["k_cache"]), dev(c["v_cache"]), dev(c["context_lens"]),
                                dev(c["block_tables"]), c["scale"], ws, 8)
    check(out, oracle(c))


def test_nan_beyond_context_is_ignored(ops):
    """Pool contents past the context end (stale or never written) must not
    leak into the result, even if they are NaN bit patterns."""
    c = cases.attention_case(10, 2, 8, 2, 128, 64, None, lens=[70, 3])
    ref = oracle(c)
    for i, L in enumerate(c["context_lens"]):
        for t in range(int(L), ((int(L) + 63) // 64) * 64):
            blk = c["block_tables"][i, t // 64]
            c["k_cache"][blk, t % 64] = np.nan
            c["v_cache"][blk, t % 64] = np.nan
    check(run(ops, c), ref)


def test_bad_page_is_flagged_not_faulted(ops):
    c = cases.attention_case(13, 2, 8, 2, 128, 64, 8, lens=[100, 100])
    c["block_tables"][1, 1] = 999
    st = ops.new_status("cuda")
    out = run(ops, c, status=st)
    assert int(st.item()) & 2
    np.testing.assert_allclose(host_f32(out)[0], oracle(dict(c, block_tables=np.where(
        c["block_tables"] == 999, 0, c["block_tables"])))[0], atol=ATOL, rtol=RTOL)


def test_skewed_long_context_config5_sample(ops):
    """Config-5 shape at reduced batch: 64 q / 4 kv heads (ratio 16), log-uniform
    lengths up to 32768, blocks scattered over the pool."""
    c = cases.attention_case(205, 24, 64, 4, 128, 256, None, len_range=(64, 32768),
                             log_uniform=True)
    check(run(ops, c, max_splits=32), oracle(c))


@pytest.mark.parametrize("tp", [2, 4])
def test_config5_heads_sharded_like_tensor_parallel(ops, tp):
    """Config 5 under TP 2/4: query heads split across ranks, KV heads split where
    divisible; every rank owns its Hkv/tp slice of every page, block tables and
    lengths are replicated, and no collective is involved.  The per-rank outputs,
    concatenated along the head axis, must equal the unsharded oracle."""
    c = cases.attention_case(305, 12, 64, 4, 128, 256, None, len_range=(64, 16384),
                             log_uniform=True)
    ref = oracle(c)
    hq, hkv = 64, 4
    outs = []
    for r in range(tp):
        qs, ks = hq // tp, hkv // tp
        shard = dict(c, q=c["q"][:, r * qs:(r + 1) * qs],
                     k_cache=np.ascontiguousarray(c["k_cache"][:, :, r * ks:(r + 1) * ks]),
                     v_cache=np.ascontiguousarray(c["v_cache"][:, :, r * ks:(r + 1) * ks]))
        outs.append(host_f32(run(ops, shard, max_splits=32)))
    check_np = np.concatenate(outs, axis=1)
    np.testing.assert_allclose(check_np, ref, atol=ATOL, rtol=RTOL)
    assert np.abs(check_np - ref).max() <= TIGHT


def test_linearity_in_v_at_config3_size(ops):
    """Size-independent property at the benchmark's batch/length scale (one
    layer of config 3): attention is linear in V, and with V == 1 every output
    is exactly 1 (softmax weights sum to one)."""
    g = torch.Generator(device="cuda").manual_seed(3)
    b, hq, hkv, d, bs = 64, 32, 8, 128, 256
    lens = torch.randint(1024, 8193, (b,), generator=g, device="cuda", dtype=torch.int32)
    pages = (lens + bs - 1) // bs
    nb = int(pages.sum())
    perm = torch.randperm(nb, generator=g, device="cuda").to(torch.int32)
    bt = torch.full((b, 33), -1, dtype=torch.int32, device="cuda")
    o = 0
    for i in range(b):
        n = int(pages[i])
        bt[i, :n] = perm[o:o + n]
        o += n
    q = (torch.randn((b, hq, d), generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    kc = (torch.randn((nb, bs, hkv, d), generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    v1 = (torch.randn((nb, bs, hkv, d), generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    ones = torch.ones_like(v1)
    ws = torch.empty(ops.attn_workspace_bytes(b, hq, d, 64), dtype=torch.uint8, device="cuda")
    st = ops.new_status("cuda")
    o1 = ops.paged_decode_attn(q, kc, v1, lens, bt, d ** -0.5, ws, 64, status=st).float()
    o_one = ops.paged_decode_attn(q, kc, ones, lens, bt, d ** -0.5, ws, 64, status=st).float()
    o_sum = ops.paged_decode_attn(q, kc, (v1.float() + 1).to(torch.bfloat16), lens, bt,
                                  d ** -0.5, ws, 64, status=st).float()
    assert int(st.item()) == 0
    assert torch.allclose(o_one, torch.ones_like(o_one), atol=8e-3)
    assert torch.allclose(o_sum, o1 + 1.0, atol=3e-2, rtol=2e-2)
    # spot-check two sequences against the oracle
    for i in (0, 37):
        L = int(lens[i])
        ref = O.paged_decode_attention(
            host_f32(q[i:i + 1]), host_f32(kc), host_f32(v1), np.array([L], np.int32),
            bt[i:i + 1].cpu().numpy(), d ** -0.5)
        np.testing.assert_allclose(o1[i:i + 1].cpu().numpy(), ref, atol=ATOL, rtol=RTOL)
