"""The C-ABI library loads on a machine without a GPU, exports every symbol the
header declares, and rejects bad arguments on the host (no kernel is launched)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "fk_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fk_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def fklib():
    from fastkernels_b200 import build
    build.build()
    from fastkernels_b200 import _lib
    return _lib


def test_every_declared_symbol_is_exported_and_bound(fklib):
    syms = header_symbols()
    assert len(syms) >= 12
    raw = ctypes.CDLL(str(fklib.LIB_PATH))
    for s in syms:
        assert hasattr(raw, s), f"{s} declared in fk_b200.h but not exported"
        assert s in fklib.PROTOTYPES, f"{s} has no ctypes prototype"
    assert sorted(fklib.PROTOTYPES) == syms


def test_version_and_error_text(fklib):
    assert fklib.lib.fk_version() >= 100
    rc = fklib.lib.fk_store_kvcache(None, None, None, None, None, 0, 4, 16, 16, 16, 8, None, None)
    assert rc == -1
    assert b"null pointer" in fklib.lib.fk_last_error()
    with pytest.raises(fklib.FkError, match="FK_ERR_INVALID_ARG"):
        fklib.check(rc, "fk_store_kvcache")


def test_host_side_validation_codes(fklib):
    L = fklib.lib
    one = ctypes.c_void_p(4096)  # never dereferenced: validation fails first
    # unsupported head_dim
    rc = L.fk_paged_decode_attn(one, 64 * 8, one, 64 * 8, one, one, 4, 64, 64 * 2 * 64, 0, one, one, 4,
                                2, 8, 2, 64, 0.1, 4, one, 1 << 20, None, None)
    assert rc == -2 and b"head_dim" in L.fk_last_error()
    # unsupported block size
    rc = L.fk_paged_decode_attn(one, 1024, one, 1024, one, one, 4, 48, 48 * 2 * 128, 0, one, one, 4,
                                2, 8, 2, 128, 0.1, 4, one, 1 << 20, None, None)
    assert rc == -2 and b"block_size" in L.fk_last_error()
    # workspace too small
    need = L.fk_paged_decode_attn_workspace_bytes(2, 8, 128, 4)
    assert need > 2 * 8 * 4 * 128 * 4
    rc = L.fk_paged_decode_attn(one, 1024, one, 1024, one, one, 4, 64, 64 * 2 * 128, 0, one, one, 4,
                                2, 8, 2, 128, 0.1, 4, one, need - 1, None, None)
    assert rc == -3
    # misaligned pointer
    rc = L.fk_rope_neox(one, ctypes.c_void_p(4098), 512, 4, one, 256, 2, 128, one, 1, 64, 3,
                        None, None)
    assert rc == -4
    # gemm: k not a multiple of 64; more than 256 rows need no workspace
    assert L.fk_gemm_bf16(one, 100, one, None, one, 128, 4, 128, 100, None, 0, None, None) == -2
    assert L.fk_gemm_bf16_workspace_bytes(300, 128, 128) == 0
    # gemm: missing stream-K workspace
    assert L.fk_gemm_bf16_workspace_bytes(64, 4096, 4096) >= 160 * 64 * 128 * 4
    assert L.fk_gemm_bf16(one, 128, one, None, one, 128, 4, 128, 128, None, 0, None, None) == -3
    # empty problems are fine and launch nothing
    before = L.fk_launch_count()
    assert L.fk_silu_and_mul(None, 0, None, 0, 0, 8, None) == 0
    assert L.fk_fused_add_rmsnorm(None, 0, None, 0, None, 1e-6, 0, 8, None) == 0
    assert L.fk_launch_count() == before


def test_ops_refuse_cpu_tensors(fklib):
    import torch
    from fastkernels_b200 import ops
    x = torch.zeros(2, 8, dtype=torch.bfloat16)
    with pytest.raises(fklib.FkError, match="CUDA tensor"):
        ops.silu_and_mul(x)
