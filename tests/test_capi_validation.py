"""The C-ABI refuses bad arguments on the host, before any CUDA call: these run
without a GPU.  Every refusal returns a negative fk_status and leaves a message
in fk_last_error()."""
import ctypes

import pytest

from fastkernels_b200 import _lib

L = _lib.lib
INVALID, UNSUPPORTED, WORKSPACE, ALIGNMENT = -1, -2, -3, -4
P = 0x10000          # a non-null, 16-byte aligned stand-in; never dereferenced


def err():
    return L.fk_last_error().decode()


def prefill(**kw):
    a = dict(q=P, q_stride=512, out=P, out_stride=512, lse=None, k=P, v=P, kv_stride=256,
             num_blocks=0, block_size=0, layout=0, cu_q=P, cu_k=P, bt=None, bt_stride=0,
             num_seqs=1, total_q=8, total_k=8, max_q=8, hq=4, hkv=2, d=128, scale=0.1, causal=1)
    a.update(kw)
    return L.fk_prefill_attn(a["q"], a["q_stride"], a["out"], a["out_stride"], a["lse"], a["k"],
                             a["v"], a["kv_stride"], a["num_blocks"], a["block_size"],
                             a["layout"], a["cu_q"], a["cu_k"], a["bt"], a["bt_stride"],
                             a["num_seqs"], a["total_q"], a["total_k"], a["max_q"], a["hq"],
                             a["hkv"], a["d"], a["scale"], a["causal"], None, None)


def test_prefill_refusals():
    assert prefill(num_seqs=0) == 0                      # empty batch: nothing to do
    assert prefill(total_q=0) == 0
    assert prefill(q=None) == INVALID and "null" in err()
    assert prefill(d=64) == UNSUPPORTED and "head_dim" in err()
    assert prefill(hq=5) == INVALID and "multiple" in err()
    assert prefill(q=P + 2) == ALIGNMENT
    assert prefill(q_stride=509) == ALIGNMENT
    assert prefill(q_stride=128) == INVALID and "stride" in err()
    assert prefill(num_blocks=4, block_size=64, kv_stride=64 * 2 * 128) == INVALID  # no tables
    assert prefill(num_blocks=4, block_size=48, kv_stride=48 * 2 * 128, bt=P,
                   bt_stride=4) == UNSUPPORTED and "block_size" in err()
    assert prefill(num_blocks=4, block_size=64, kv_stride=64 * 2 * 128, bt=P, bt_stride=4,
                   layout=7) == INVALID and "kv_layout" in err()
    assert prefill(total_k=0) == INVALID


def test_merge_refusals():
    def merge(**kw):
        a = dict(out=P, st=512, sh=128, lse=None, a=P, b=P, al=P, bl=P, tokens=4, heads=4, d=128)
        a.update(kw)
        return L.fk_merge_attn_states(a["out"], a["st"], a["sh"], a["lse"], a["a"], a["st"],
                                      a["sh"], a["al"], a["b"], a["st"], a["sh"], a["bl"],
                                      a["tokens"], a["heads"], a["d"], -1, None)
    assert merge(tokens=0) == 0
    assert merge(a=None) == INVALID
    assert merge(d=12) == UNSUPPORTED and "multiple of 8" in err()
    assert merge(out=P + 4) == ALIGNMENT
    assert merge(sh=100) == ALIGNMENT


def test_decode_side_refusals():
    # head_dim other than 128, GQA ratio not a power of two up to 16, odd page size
    args = lambda **kw: _attn(**kw)                        # noqa: E731
    assert _attn(d=64) == UNSUPPORTED
    assert _attn(hq=6, hkv=2) == UNSUPPORTED and "GQA" in err()
    assert _attn(block=48) == UNSUPPORTED
    assert _attn(ws=None) == WORKSPACE
    # GEMM: k not a multiple of 64, missing workspace
    assert L.fk_gemm_bf16(P, 4096, P, None, P, 4096, 8, 4096, 4000, P, 1 << 30, None,
                          None) == UNSUPPORTED and "64" in err()
    assert L.fk_gemm_bf16(P, 4096, P, None, P, 4096, 8, 4096, 4096, None, 0, None,
                          None) == WORKSPACE
    assert L.fk_gemm_bf16_static(P, 4096, P, None, P, 4096, 65, 4096, 4096, None,
                                 None) == UNSUPPORTED and "scratch" in err()


def _attn(d=128, hq=8, hkv=2, block=64, ws=P):
    return L.fk_paged_decode_attn(P, hq * d, P, hq * d, P, P, 16, block, block * hkv * d, 0, P, P,
                                  4, 2, hq, hkv, d, 0.1, 8, ws, 1 << 24, None, None)
