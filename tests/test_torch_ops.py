"""torch.library registration: schemas and fake (shape-only) implementations,
checked on CPU with FakeTensorMode; on a GPU, a candidate MLP block must trace
with torch.compile(fullgraph=True) and give the eager result."""
import pytest
import torch


def test_fake_impls_describe_shapes():
    import fastkernels_b200.torch_ops  # noqa: F401
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        x = torch.empty((5, 256), dtype=torch.bfloat16, device="cuda")
        w = torch.empty((256,), dtype=torch.bfloat16, device="cuda")
        assert torch.ops.fk_b200.rmsnorm(x, w, 1e-6).shape == (5, 256)
        assert torch.ops.fk_b200.fused_add_rmsnorm(x, x.clone(), w, 1e-6) is None
        wt = torch.empty((384, 256), dtype=torch.bfloat16, device="cuda")
        y = torch.ops.fk_b200.gemm_bf16(x, wt, None)
        assert y.shape == (5, 384) and y.dtype == torch.bfloat16
        assert torch.ops.fk_b200.silu_and_mul(y).shape == (5, 192)
        pos = torch.empty((5,), dtype=torch.int64, device="cuda")
        cache = torch.empty((64, 128), dtype=torch.float32, device="cuda")
        assert torch.ops.fk_b200.rope_neox(pos, x, None, 128, cache) is None


def test_schemas_declare_mutations():
    import fastkernels_b200.torch_ops  # noqa: F401
    s = torch.ops.fk_b200.fused_add_rmsnorm.default._schema
    assert [a.alias_info is not None and a.alias_info.is_write for a in s.arguments] == \
        [True, True, False, False]
    s = torch.ops.fk_b200.rope_neox.default._schema
    assert s.arguments[1].alias_info.is_write and s.arguments[2].alias_info.is_write


@pytest.mark.gpu
def test_fullgraph_compile_of_candidate_block_matches_eager():
    from fastkernels_b200.candidate.L1.rms_norm import RMSNorm
    from fastkernels_b200.candidate.L1.silu_and_mul import SiluAndMul
    from fastkernels_b200.candidate.L2.parallel_linear import (MergedColumnParallelLinear,
                                                                RowParallelLinear)

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.norm = RMSNorm(256)
            self.up = MergedColumnParallelLinear(256, [512, 512])
            self.act = SiluAndMul()
            self.down = RowParallelLinear(512, 256)

        def forward(self, x, residual):
            x, residual = self.norm(x, residual)
            return self.down(self.act(self.up(x))), residual

    torch.manual_seed(0)
    blk = Block().cuda().to(torch.bfloat16)
    for p in blk.parameters():
        p.data.normal_(0, 0.05)
    blk.norm.weight.data.fill_(1.0)
    x = torch.randn(7, 256, device="cuda").to(torch.bfloat16)
    r = torch.randn(7, 256, device="cuda").to(torch.bfloat16)
    want, want_r = blk(x.clone(), r.clone())
    compiled = torch.compile(blk, fullgraph=True, backend="eager")
    got, got_r = compiled(x.clone(), r.clone())
    assert torch.equal(got, want) and torch.equal(got_r, want_r)
