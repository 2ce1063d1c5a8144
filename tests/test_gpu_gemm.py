"""GPU parity (through the C-ABI) of the tcgen05 decode GEMM."""
import numpy as np
import pytest
import torch

import cases
from gpu_util import dev, host_f32
from oracle import decode_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from fastkernels_b200 import ops as _ops
    return _ops


def check(y, ref, k):
    g = host_f32(y)
    np.testing.assert_allclose(g, ref, atol=2e-2, rtol=2e-2)
    # fp32 accumulation in a different order: at most one bf16 step away
    scale = np.maximum(np.abs(ref), 1e-2)
    assert (np.abs(g - ref) / scale).max() <= 2.0 ** -7, (np.abs(g - ref) / scale).max()


@pytest.mark.parametrize("m,n,k", [
    (5, 130, 192),       # ragged n tile, tiny k (golden shape)
    (1, 128, 64),        # single k-block
    (16, 256, 512),
    (33, 1000, 1024),    # n not a multiple of 128
    (64, 512, 4096),
    (64, 6144, 4096),    # qkv projection of the 8B shape
    (128, 1024, 2048),
    (200, 384, 1024),    # m padded to 256
    (7, 256, 4096),      # clusters of 8 with fewer rows than CTAs: one CTA owns no row
    (63, 5760, 1024),    # 45 tiles: clusters of 3, 21 rows per CTA
    (64, 4096, 12288),   # down projection of the 8B shape: clusters of 4
    (64, 3072, 4096),    # 24 tiles: clusters of 5, 13 rows per CTA (65 slab rows)
    (50, 2560, 2048),    # 20 tiles: clusters of 6
    (64, 768, 4096),     # qkv shard at tp8: 6 tiles, clusters of 8
])
def test_gemm_matches_oracle(ops, m, n, k):
    rs = np.random.RandomState(m * 7 + n)
    x = cases.randn_bf16(rs, (m, k))
    w = cases.randn_bf16(rs, (n, k), 0.05)
    st = ops.new_status("cuda")
    y = ops.gemm_bf16(dev(x), dev(w), status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    check(y, O.linear(x, w), k)


def test_gemm_golden_and_bias(ops, golden):
    rs = np.random.RandomState(31)
    cases.randn_bf16(rs, (7, 2 * 96), 2.0)
    lx, lw = cases.randn_bf16(rs, (5, 192)), cases.randn_bf16(rs, (130, 192), 0.05)
    lb = cases.randn_bf16(rs, (130,), 0.1)
    y = ops.gemm_bf16(dev(lx), dev(lw))
    np.testing.assert_allclose(host_f32(y), O.bf16_bits_to_f32(golden["linear"]), atol=2e-2,
                               rtol=2e-2)
    yb = ops.gemm_bf16(dev(lx), dev(lw), bias=dev(lb))
    np.testing.assert_allclose(host_f32(yb), O.bf16_bits_to_f32(golden["linear_bias"]),
                               atol=2e-2, rtol=2e-2)
    check(yb, O.linear(lx, lw, lb), 192)


@pytest.mark.parametrize("m,n,k", [(64, 520, 2048),      # cluster split-K, ragged n
                                   (40, 24576, 1024),    # stream-K, many tiles
                                   (128, 4096, 8192)])   # cluster split-K, m = 128
def test_gemm_bias_both_schedules(ops, m, n, k):
    rs = np.random.RandomState(n + k)
    x = cases.randn_bf16(rs, (m, k))
    w = cases.randn_bf16(rs, (n, k), 0.03)
    b = cases.randn_bf16(rs, (n,), 0.5)
    out = torch.zeros((m, n + 8), dtype=torch.bfloat16, device="cuda")
    st = ops.new_status("cuda")
    ops.gemm_bf16(dev(x), dev(w), bias=dev(b), out=out[:, :n], status=st)
    assert int(st.item()) == 0
    check(out[:, :n], O.linear(x, w, b), k)
    assert not out[:, n:].any()
    # same call again: the schedule's scratch (flags, partial tiles) was left clean
    out2 = torch.zeros_like(out)
    ops.gemm_bf16(dev(x), dev(w), bias=dev(b), out=out2[:, :n])
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))


def test_gemm_strided_input_and_output(ops):
    rs = np.random.RandomState(4)
    m, n, k = 24, 256, 256
    big = cases.randn_bf16(rs, (m, 2 * k))
    w = cases.randn_bf16(rs, (n, k), 0.05)
    xd = dev(big)[:, k:]                      # row stride 2k
    out = torch.zeros((m, 2 * n), dtype=torch.bfloat16, device="cuda")
    ops.gemm_bf16(xd, dev(w), out=out[:, :n])
    check(out[:, :n], O.linear(big[:, k:], w), k)
    assert not out[:, n:].any()


def test_gemm_down_proj_shape_split_k(ops):
    """k = 12288 (down projection of the 8B shape): long split-K reduction."""
    g = torch.Generator(device="cuda").manual_seed(1)
    m, n, k = 64, 4096, 12288
    x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn((n, k), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    y = ops.gemm_bf16(x, w)
    ref = O.linear(host_f32(x), host_f32(w))
    check(y, ref, k)


@pytest.mark.parametrize("m,n,k,bias", [(257, 256, 64, False), (300, 520, 192, True),
                                        (1000, 1032, 512, False), (2048, 768, 1024, True)])
def test_gemm_many_rows_matches_oracle(m, n, k, bias):
    """m > 256 takes the 256 x 256 tile kernel: ragged row and column tails, bias."""
    import numpy as np
    import torch
    import cases
    from fastkernels_b200 import ops
    from oracle import decode_oracle as O
    rs = np.random.RandomState(m + n)
    x = cases.randn_bf16(rs, (m, k), 1.0)
    w = cases.randn_bf16(rs, (n, k), 0.05)
    b = cases.randn_bf16(rs, (n,), 0.5) if bias else None
    want = O.linear(x, w, b)
    dev = lambda a: torch.from_numpy(a).to(torch.bfloat16).cuda()          # noqa: E731
    st = ops.new_status("cuda")
    got = ops.gemm_bf16(dev(x), dev(w), dev(b) if bias else None, status=st).float().cpu().numpy()
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    # one bf16 rounding of an fp32 sum whose order differs from numpy's
    err = np.abs(got - want)
    assert (err <= 2e-2 + 2e-2 * np.abs(want)).all(), err.max()
    assert (got == want).mean() > 0.9


def test_gemm_many_rows_strided_views():
    """x as a column slice of a wider buffer, y into a strided destination."""
    import numpy as np
    import torch
    import cases
    from fastkernels_b200 import ops
    from oracle import decode_oracle as O
    rs = np.random.RandomState(77)
    m, n, k = 600, 512, 256
    xw = cases.randn_bf16(rs, (m, k + 64), 1.0)
    w = cases.randn_bf16(rs, (n, k), 0.05)
    xd = torch.from_numpy(xw).to(torch.bfloat16).cuda()[:, 64:]
    out = torch.zeros((m, n + 128), dtype=torch.bfloat16, device="cuda")
    ops.gemm_bf16(xd, torch.from_numpy(w).to(torch.bfloat16).cuda(), out=out[:, :n])
    torch.cuda.synchronize()
    want = O.linear(xw[:, 64:], w)
    got = out[:, :n].float().cpu().numpy()
    assert (np.abs(got - want) <= 2e-2 + 2e-2 * np.abs(want)).all()
    assert float(out[:, n:].abs().max()) == 0.0


@pytest.mark.parametrize("mode", ["1", "2"])
def test_gemm_many_rows_cta_pair_kernels(mode):
    """The CTA-pair variants of the many-row kernel (tcgen05 cta_group::2, selected by
    FK_B200_GEMM_PAIR, read once per process) against the oracle, in a child process."""
    import os
    import subprocess
    import sys
    code = r"""
import sys
import numpy as np, torch
sys.path.insert(0, 'tests')
import cases
from fastkernels_b200 import ops
from oracle import decode_oracle as O
for (m, n, k, bias) in [(257, 256, 64, False), (300, 520, 192, True), (1000, 1032, 512, False),
                        (1536, 2048, 256, True)]:
    rs = np.random.RandomState(m + n)
    x = cases.randn_bf16(rs, (m, k), 1.0)
    w = cases.randn_bf16(rs, (n, k), 0.05)
    b = cases.randn_bf16(rs, (n,), 0.5) if bias else None
    want = O.linear(x, w, b)
    dev = lambda a: torch.from_numpy(a).to(torch.bfloat16).cuda()
    st = ops.new_status('cuda')
    got = ops.gemm_bf16(dev(x), dev(w), dev(b) if bias else None, status=st).float().cpu().numpy()
    torch.cuda.synchronize()
    assert int(st.item()) == 0, int(st.item())
    err = np.abs(got - want)
    assert (err <= 2e-2 + 2e-2 * np.abs(want)).all(), (m, n, k, float(err.max()))
    assert (got == want).mean() > 0.9
print('pair ok')
"""
    env = dict(os.environ, FK_B200_GEMM_PAIR=mode)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0 and "pair ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


# ---------------------------------------------------- gate/up projection + SiLU fused
@pytest.mark.parametrize("m,n,k,bias", [
    (64, 24576, 4096, False),    # the 8B-shape MLP at batch 64
    (5, 24576, 1024, True),      # a handful of rows, with bias
    (128, 28672, 2048, False),   # the 70B-shape MLP shard at tp2 (k shortened)
    (200, 20480, 512, True),     # m padded to 256
])
def test_gemm_silu_mul_matches_the_two_ops(ops, m, n, k, bias):
    """One launch for silu_and_mul(x W^T): against the oracle's linear followed by
    its SiLU-and-multiply (the rounding points are those of the two ops: <= 1 bf16
    step, as for each op alone), and against this build's own two-kernel path."""
    from gpu_util import assert_bf16_close
    assert ops.gemm_silu_mul_fusable(m, n, k)
    rs = np.random.RandomState(n + k + m)
    x = cases.randn_bf16(rs, (m, k))
    w = cases.randn_bf16(rs, (n, k), 0.03)
    b = cases.randn_bf16(rs, (n,), 0.3) if bias else None
    st = ops.new_status("cuda")
    xd, wd, bd = dev(x), dev(w), (dev(b) if bias else None)
    out = torch.full((m, n // 2 + 8), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_silu_mul(xd, wd, bias=bd, out=out[:, :n // 2], status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert torch.isnan(out[:, n // 2:].float()).all()      # nothing written past the row
    got = out[:, :n // 2]
    ref = O.silu_and_mul(O.linear(x, w, b))
    np.testing.assert_allclose(host_f32(got), ref, atol=2e-2, rtol=2e-2)
    # The product of two projection outputs that may each be one bf16 step away from
    # the oracle's (fp32 summation order): almost every element is within two steps;
    # where silu(gate) * up nearly cancels, a few in a million are further off in
    # relative terms while far inside the tolerance checked above.
    gb = O.bf16_round_bits(host_f32(got)).astype(np.int32)
    wb = O.bf16_round_bits(ref).astype(np.int32)
    steps = np.abs((gb & 0x7FFF) - (wb & 0x7FFF))
    big = (np.abs(ref) >= 1e-3) & (((gb ^ wb) & 0x8000) == 0)
    assert (steps[big] > 2).mean() <= 1e-4, (steps[big] > 2).mean()
    assert (steps[big] > 0).mean() <= 0.03, (steps[big] > 0).mean()
    two = ops.silu_and_mul(ops.gemm_bf16(xd, wd, bias=bd))
    np.testing.assert_allclose(host_f32(got), host_f32(two), atol=2e-2, rtol=2e-2)
    assert (got.view(torch.int16) == two.view(torch.int16)).float().mean() >= 0.97


def test_gemm_silu_mul_refuses_shapes_without_single_launch_form(ops):
    from fastkernels_b200 import _lib
    assert not ops.gemm_silu_mul_fusable(64, 3072, 4096)       # few tiles: cluster split-K
    assert not ops.gemm_silu_mul_fusable(64, 24576 + 64, 4096)
    x = torch.zeros((64, 4096), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((3072, 4096), dtype=torch.bfloat16, device="cuda")
    before = _lib.lib.fk_launch_count()
    with pytest.raises(_lib.FkError, match="FK_ERR_UNSUPPORTED"):
        ops.gemm_silu_mul(x, w)
    assert _lib.lib.fk_launch_count() == before
