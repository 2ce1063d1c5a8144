"""ctypes binding of libfk_b200.so (the C-ABI declared in include/fk_b200.h).

There is no fallback: if the library is missing or a symbol is absent the import
of this module raises, and every op wrapper raises on a non-zero status.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = Path(os.environ.get("FK_B200_LIB", _PKG / "libfk_b200.so"))

FK_OK = 0
STATUS_NAMES = {
    0: "FK_OK",
    -1: "FK_ERR_INVALID_ARG",
    -2: "FK_ERR_UNSUPPORTED",
    -3: "FK_ERR_WORKSPACE",
    -4: "FK_ERR_ALIGNMENT",
    -5: "FK_ERR_CUDA",
}
DEV_BAD_SLOT, DEV_BAD_PAGE, DEV_WAIT_TIMEOUT, DEV_BAD_POSITION = 1, 2, 4, 8

_vp, _i32, _i64, _f32, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

class BlockPhase(C.Structure):
    """struct fk_block_phase of include/fk_b200.h (same field order and types)."""
    _fields_ = [
        ("kind", C.c_int32),
        ("x", _vp), ("x_stride", _i64),
        ("w", _vp), ("bias", _vp),
        ("y", _vp), ("y_stride", _i64),
        ("n", _i64), ("k", _i64),
        ("residual", _vp), ("residual_stride", _i64),
        ("norm_weight", _vp), ("eps", _f32),
        ("num_q_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("positions", _vp),
        ("cos_sin_cache", _vp), ("cache_is_fp32", C.c_int32), ("max_position", _i64),
        ("q_norm_weight", _vp), ("k_norm_weight", _vp),
        ("k_cache", _vp), ("v_cache", _vp),
        ("slot_mapping", _vp), ("num_slots", _i64),
        ("block_size", C.c_int32), ("kv_layout", C.c_int32),
    ]


PHASE_GEMM, PHASE_GEMM_SILU_MUL, PHASE_ADD_RMSNORM, PHASE_QKV_ROPE_STORE = 1, 2, 3, 4

# name -> (restype, argtypes); must list every symbol include/fk_b200.h declares
PROTOTYPES = {
    "fk_version": (_i32, []),
    "fk_last_error": (C.c_char_p, []),
    "fk_launch_count": (_i64, []),
    "fk_set_pdl": (_i32, [_i32]),
    "fk_store_kvcache": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64,
                                _i64, _vp, _vp]),
    "fk_paged_decode_attn_workspace_bytes": (_sz, [_i32, _i32, _i32, _i32]),
    "fk_paged_decode_attn": (_i32, [_vp, _i64, _vp, _i64, _vp, _vp, _i64, _i32, _i64, _i32,
                                    _vp, _vp, _i64, _i32, _i32, _i32, _i32, _f32, _i32,
                                    _vp, _sz, _vp, _vp]),
    "fk_paged_decode_attn_plan": (_i32, [_vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _i32,
                                         _vp, _sz, _vp, _vp]),
    "fk_paged_decode_attn_planned": (_i32, [_vp, _i64, _vp, _i64, _vp, _vp, _i64, _i32, _i64,
                                            _i32, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _f32, _i32,
                                            _vp, _sz, _vp, _vp]),
    "fk_rmsnorm": (_i32, [_vp, _i64, _i64, _i64, _vp, _i64, _i64, _vp, _f32, _i64, _i64,
                          _vp]),
    "fk_fused_add_rmsnorm": (_i32, [_vp, _i64, _vp, _i64, _vp, _f32, _i64, _i64, _vp]),
    "fk_rope_neox": (_i32, [_vp, _vp, _i64, _i32, _vp, _i64, _i32, _i32, _vp, _i32, _i64,
                            _i64, _vp, _vp]),
    "fk_qkv_rope_store": (_i32, [_vp, _i64, _i32, _i32, _i32, _vp, _vp, _i32, _i64, _vp,
                                 _vp, _f32, _vp, _vp, _vp, _i64, _i32, _i32, _i64, _vp, _vp]),
    "fk_store_kvcache_hnd": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i64, _i32, _i32, _i64,
                                    _i64, _i32, _i64, _vp, _vp]),
    "fk_silu_and_mul": (_i32, [_vp, _i64, _vp, _i64, _i64, _i64, _vp]),
    "fk_argmax_bf16": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _vp]),
    "fk_comm_header_bytes": (_sz, []),
    "fk_comm_alloc": (_i32, [_sz, C.POINTER(_vp)]),
    "fk_comm_free": (_i32, [_vp]),
    "fk_comm_ipc_export": (_i32, [_vp, _vp]),
    "fk_comm_ipc_import": (_i32, [_vp, C.POINTER(_vp)]),
    "fk_comm_ipc_close": (_i32, [_vp]),
    "fk_allreduce_add_rmsnorm": (_i32, [C.POINTER(_vp), _i32, _i32, _sz, _vp, _i64, _vp, _f32,
                                        _vp, _i64, _i64, _i64, _vp, _vp]),
    "fk_allreduce_two_stage_preferred": (_i32, [_i32, _i64, _i64]),
    "fk_comm_epoch_offset": (_sz, []),
    "fk_allreduce_push_preferred": (_i32, [_i32, _i64, _i64]),
    "fk_gemm_bf16_push": (_i32, [_vp, _i64, _vp, _vp, _i64, _i64, _i64, _vp, _sz,
                                 C.POINTER(_vp), _i32, _vp, _vp, _vp]),
    "fk_allreduce_add_rmsnorm_pushed": (_i32, [_vp, _i32, _sz, _sz, _vp, _i64, _vp, _f32,
                                               _vp, _i64, _i64, _i64, _vp, _vp]),
    "fk_allreduce_add_rmsnorm_staged": (_i32, [C.POINTER(_vp), _i32, _i32, _sz, _sz, _vp, _i64,
                                               _vp, _f32, _vp, _i64, _i64, _i64, _vp, _vp]),
    "fk_allreduce_add_rmsnorm_group": (_i32, [C.POINTER(_vp), _i32, _sz, _sz, C.POINTER(_vp),
                                              _i64, _vp, _f32, C.POINTER(_vp), _i64, _i64,
                                              _i64, _vp, _vp]),
    "fk_fill_u32": (_i32, [_vp, _i64, C.c_uint32, _vp]),
    "fk_xor_u32": (_i32, [_vp, _i64, _vp, _vp]),
    "fk_prefill_attn": (_i32, [_vp, _i64, _vp, _i64, _vp, _vp, _vp, _i64, _i64, _i32, _i32,
                               _vp, _vp, _vp, _i64, _i32, _i64, _i64, _i32, _i32, _i32, _i32,
                               _f32, _i32, _vp, _vp]),
    "fk_merge_attn_states": (_i32, [_vp, _i64, _i64, _vp, _vp, _i64, _i64, _vp, _vp, _i64,
                                    _i64, _vp, _i64, _i32, _i32, _i64, _vp]),
    "fk_gemm_bf16_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "fk_gemm_bf16_silu_mul_fusable": (_i32, [_i64, _i64, _i64]),
    "fk_gemm_bf16_silu_mul": (_i32, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _sz,
                                     _vp, _vp]),
    "fk_decode_block_workspace_bytes": (_sz, [_i64]),
    "fk_decode_block": (_i32, [C.POINTER(BlockPhase), _i32, _i64, _vp, _sz, _vp, _vp]),
    "fk_gemm_bf16_static": (_i32, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp]),
    "fk_gemm_bf16": (_i32, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _sz,
                            _vp, _vp]),
}


class FkError(RuntimeError):
    """A C-ABI call returned a negative fk_status."""


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python -m fastkernels_b200.build` "
            "(there is no CPU or library fallback)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is missing
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(rc: int, what: str) -> None:
    if rc != FK_OK:
        msg = lib.fk_last_error().decode("utf-8", "replace")
        raise FkError(f"{what}: {STATUS_NAMES.get(rc, rc)}: {msg}")
