"""Tensor-level wrappers over the C-ABI: take torch CUDA tensors, pass raw
pointers / sizes / strides and the current CUDA stream to libfk_b200.so.

torch is only the owner of device memory and streams here; every wrapper fails
loudly (FkError) instead of falling back to a torch implementation, and no
wrapper calls a library kernel.

Kernels report device-side anomalies (a slot, page or position out of range, a
bounded wait that ran out) by OR-ing fk_device_status bits into an int32 device
word.  A wrapper called without `status=` uses the per-device word of
`default_status`, so a caller that does not thread a status tensor through its
modules can still read one word per device after a step.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import check, lib

BF16 = torch.bfloat16


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype, name: str) -> None:
    if not t.is_cuda:
        raise _lib.FkError(f"{name} must be a CUDA tensor (no CPU path exists)")
    if t.dtype != dtype:
        raise _lib.FkError(f"{name} must be {dtype}, got {t.dtype}")


def new_status(device) -> torch.Tensor:
    """One int32 device word the kernels OR their fk_device_status bits into."""
    return torch.zeros(1, dtype=torch.int32, device=device)


_DEFAULT_STATUS: dict = {}


def default_status(device=None) -> torch.Tensor:
    """The status word (one per device, made on first use) that wrappers called
    without `status=` hand to their kernels."""
    key = torch.device("cuda", torch.cuda.current_device()) if device is None \
        else torch.device(device)
    if key.index is None:
        key = torch.device("cuda", torch.cuda.current_device())
    st = _DEFAULT_STATUS.get(key)
    if st is None:
        st = _DEFAULT_STATUS[key] = new_status(key)
    return st


def _status_ptr(status, like: torch.Tensor) -> int:
    return (status if status is not None else default_status(like.device)).data_ptr()


# --------------------------------------------------------------------------- store
def store_kvcache(key, value, k_cache, v_cache, slot_mapping, status=None) -> None:
    """cache.view(-1, Hkv*D)[slot] = key[i] / value[i] for slot >= 0 (bit-exact)."""
    _need(key, k_cache.dtype, "key")
    _need(value, v_cache.dtype, "value")
    if key.element_size() != 2:
        raise _lib.FkError("store_kvcache moves 16-bit elements")
    n = key.shape[0]
    row = key[0].numel() if n else int(k_cache.shape[-1] * k_cache.shape[-2])
    if n and (key.stride(-1) != 1 or (key.dim() == 3 and key.stride(1) != key.shape[2])):
        raise _lib.FkError("key rows must be dense")
    if n and (value.stride(-1) != 1 or (value.dim() == 3 and value.stride(1) != value.shape[2])):
        raise _lib.FkError("value rows must be dense")
    if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise _lib.FkError("caches must be contiguous")
    if slot_mapping.dtype not in (torch.int32, torch.int64):
        raise _lib.FkError("slot_mapping must be int32 or int64")
    num_slots = k_cache.numel() // row
    check(lib.fk_store_kvcache(
        _ptr(key), _ptr(value), _ptr(k_cache), _ptr(v_cache), _ptr(slot_mapping),
        int(slot_mapping.dtype == torch.int64), n, row,
        key.stride(0) if n else row, value.stride(0) if n else row, num_slots,
        _status_ptr(status, key), _stream()), "fk_store_kvcache")


def store_kvcache_hnd(key, value, k_cache, v_cache, slot_mapping, status=None) -> None:
    """HND pool [blocks, Hkv, page, D]: head h of token i goes to
    [slot // page, h, slot % page, :] (bit-exact)."""
    _need(key, k_cache.dtype, "key")
    _need(value, v_cache.dtype, "value")
    n = key.shape[0]
    nb, hkv, page, d = k_cache.shape
    if n and (key.stride(-1) != 1 or key.stride(1) != d or value.stride(-1) != 1
              or value.stride(1) != d):
        raise _lib.FkError("key/value heads must be dense")
    if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise _lib.FkError("caches must be contiguous")
    if slot_mapping.dtype not in (torch.int32, torch.int64):
        raise _lib.FkError("slot_mapping must be int32 or int64")
    check(lib.fk_store_kvcache_hnd(
        _ptr(key), _ptr(value), _ptr(k_cache), _ptr(v_cache), _ptr(slot_mapping),
        int(slot_mapping.dtype == torch.int64), n, hkv, d,
        key.stride(0) if n else hkv * d, value.stride(0) if n else hkv * d, page, nb,
        _status_ptr(status, key), _stream()), "fk_store_kvcache_hnd")


# ----------------------------------------------------------------------- attention
def attn_workspace_bytes(batch, num_q_heads, head_dim, max_splits) -> int:
    return int(lib.fk_paged_decode_attn_workspace_bytes(batch, num_q_heads, head_dim,
                                                        max_splits))


def max_splits_for(max_seq_len: int, floor: int = 16) -> int:
    """Splits needed so the smallest split (128 tokens) can cover max_seq_len,
    capped: larger contexts simply use proportionally larger splits."""
    return max(1, min(64, max(floor, (max_seq_len + 127) // 128)))


def paged_decode_attn_plan(context_lens, block_tables, block_size, num_q_heads, num_kv_heads,
                           head_dim, workspace, max_splits, status=None) -> None:
    """Compute the split-KV schedule of a decode step once; layers then call
    paged_decode_attn(..., planned=True) with the same workspace."""
    _need(context_lens, torch.int32, "context_lens")
    _need(block_tables, torch.int32, "block_tables")
    b = context_lens.shape[0]
    check(lib.fk_paged_decode_attn_plan(
        _ptr(context_lens), _ptr(block_tables), block_tables.stride(0) if b else 1,
        block_size, b, num_q_heads, num_kv_heads, head_dim, int(max_splits),
        _ptr(workspace), workspace.numel() * workspace.element_size(),
        _status_ptr(status, context_lens), _stream()), "fk_paged_decode_attn_plan")


def paged_decode_attn(q, k_cache, v_cache, context_lens, block_tables, softmax_scale,
                      workspace, max_splits, out=None, status=None, planned=False,
                      kv_layout="NHD"):
    """out[i,h] = softmax(scale q[i,h] K_i^T) V_i over the paged cache:
    NHD [blocks, block, Hkv, D] or HND [blocks, Hkv, block, D]."""
    _need(q, BF16, "q")
    _need(k_cache, BF16, "k_cache")
    _need(v_cache, BF16, "v_cache")
    _need(context_lens, torch.int32, "context_lens")
    _need(block_tables, torch.int32, "block_tables")
    b, hq, d = q.shape
    if kv_layout == "NHD":
        nb, bs, hkv, d2 = k_cache.shape
        dense = (hkv * d, d, 1)
    elif kv_layout == "HND":
        nb, hkv, bs, d2 = k_cache.shape
        dense = (bs * d, d, 1)
    else:
        raise _lib.FkError("kv_layout must be 'NHD' or 'HND'")
    if d2 != d or v_cache.shape != k_cache.shape:
        raise _lib.FkError("cache shape mismatch")
    if q.stride(2) != 1 or q.stride(1) != d:
        raise _lib.FkError("q heads must be contiguous")
    if k_cache.stride()[1:] != dense or v_cache.stride() != k_cache.stride():
        raise _lib.FkError("caches must be dense within a block")
    if block_tables.stride(1) != 1:
        raise _lib.FkError("block_tables rows must be dense")
    if out is None:
        out = torch.empty((b, hq, d), dtype=BF16, device=q.device)
    fn = lib.fk_paged_decode_attn_planned if planned else lib.fk_paged_decode_attn
    check(fn(
        _ptr(q), q.stride(0) if b else hq * d, _ptr(out), out.stride(0) if b else hq * d,
        _ptr(k_cache), _ptr(v_cache), nb, bs, k_cache.stride(0), int(kv_layout == "HND"),
        _ptr(context_lens), _ptr(block_tables), block_tables.stride(0) if b else 1,
        b, hq, hkv, d, float(softmax_scale), int(max_splits),
        _ptr(workspace), workspace.numel() * workspace.element_size(),
        _status_ptr(status, q), _stream()), "fk_paged_decode_attn")
    return out


def prefill_attn(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, softmax_scale,
                 causal=True, block_table=None, kv_layout="NHD", out=None,
                 return_lse=False, status=None):
    """Variable-length prefill attention on q [total_q, Hq, 128].

    Without block_table, k / v are dense [total_k, Hkv, 128] (token-strided views
    allowed) and sequence i owns rows cu_seqlens_k[i]..cu_seqlens_k[i+1].  With
    block_table [num_seqs, cols] they are the paged pools (NHD
    [blocks, page, Hkv, 128] or HND [blocks, Hkv, page, 128]) and only the
    per-sequence key counts of cu_seqlens_k are used.  Causal masking is aligned
    to the END of each sequence's keys (a chunk of q_len queries after a cached
    prefix sees the prefix plus its own past).  Returns out, or (out, lse) with
    lse fp32 [Hq, total_q]."""
    _need(q, BF16, "q")
    _need(k, BF16, "k")
    _need(v, BF16, "v")
    _need(cu_seqlens_q, torch.int32, "cu_seqlens_q")
    _need(cu_seqlens_k, torch.int32, "cu_seqlens_k")
    if q.dim() != 3 or q.stride(2) != 1 or q.stride(1) != q.shape[2]:
        raise _lib.FkError("q must be [total_q, Hq, D] with dense heads")
    total_q, hq, d = q.shape
    num_seqs = cu_seqlens_q.numel() - 1
    if cu_seqlens_k.numel() != num_seqs + 1:
        raise _lib.FkError("cu_seqlens_q and cu_seqlens_k must have the same length")
    if out is None:
        out = torch.empty((total_q, hq, d), dtype=BF16, device=q.device)
    elif out.stride(2) != 1 or out.stride(1) != d:
        raise _lib.FkError("out heads must be dense")
    lse = torch.empty((hq, total_q), dtype=torch.float32, device=q.device) if return_lse else None
    if block_table is None:
        if k.dim() != 3 or k.stride(2) != 1 or k.stride(1) != d or v.stride() != k.stride() \
                or v.shape != k.shape:
            raise _lib.FkError("dense k / v must be [total_k, Hkv, D] with dense heads")
        total_k, hkv = k.shape[0], k.shape[1]
        nb, bs, kv_stride, bt_stride = 0, 0, k.stride(0) if total_k else hkv * d, 0
    else:
        _need(block_table, torch.int32, "block_table")
        if block_table.stride(1) != 1:
            raise _lib.FkError("block_table rows must be dense")
        if kv_layout == "HND":
            nb, hkv, bs, d2 = k.shape
            dense = (bs * d2, d2, 1)
        else:
            nb, bs, hkv, d2 = k.shape
            dense = (hkv * d2, d2, 1)
        if d2 != d or v.shape != k.shape:
            raise _lib.FkError("cache shape mismatch")
        if k.stride()[1:] != dense or v.stride() != k.stride():
            raise _lib.FkError("caches must be dense within a block")
        total_k, kv_stride, bt_stride = 0, k.stride(0), block_table.stride(0)
    check(lib.fk_prefill_attn(
        _ptr(q), q.stride(0) if total_q else hq * d, _ptr(out),
        out.stride(0) if total_q else hq * d, _ptr(lse), _ptr(k), _ptr(v), kv_stride, nb, bs,
        int(kv_layout == "HND"), _ptr(cu_seqlens_q), _ptr(cu_seqlens_k), _ptr(block_table),
        bt_stride, num_seqs, total_q, total_k, int(max_seqlen_q), hq, hkv, d,
        float(softmax_scale), int(bool(causal)), _status_ptr(status, q), _stream()),
        "fk_prefill_attn")
    return (out, lse) if return_lse else out


def merge_attn_states(output, prefix_output, prefix_lse, suffix_output, suffix_lse,
                      output_lse=None, prefill_tokens_with_context=None) -> None:
    """output = log-sum-exp weighted mix of two partial attention results
    [T, H, D] bf16 with lse fp32 [H, T]; written in place (output_lse optional)."""
    for name, t in (("output", output), ("prefix_output", prefix_output),
                    ("suffix_output", suffix_output)):
        _need(t, BF16, name)
        if t.dim() != 3 or t.stride(2) != 1:
            raise _lib.FkError(f"{name} must be [T, H, D] with dense rows")
    for name, t in (("prefix_lse", prefix_lse), ("suffix_lse", suffix_lse)):
        _need(t, torch.float32, name)
        if not t.is_contiguous():
            raise _lib.FkError(f"{name} must be contiguous [H, T]")
    if output_lse is not None:
        _need(output_lse, torch.float32, "output_lse")
        if not output_lse.is_contiguous():
            raise _lib.FkError("output_lse must be contiguous [H, T]")
    t, h, d = output.shape
    if prefix_output.shape != output.shape or suffix_output.shape != output.shape:
        raise _lib.FkError("merge_attn_states: shape mismatch")
    check(lib.fk_merge_attn_states(
        _ptr(output), output.stride(0), output.stride(1), _ptr(output_lse),
        _ptr(prefix_output), prefix_output.stride(0), prefix_output.stride(1),
        _ptr(prefix_lse), _ptr(suffix_output), suffix_output.stride(0),
        suffix_output.stride(1), _ptr(suffix_lse), t, h, d,
        -1 if prefill_tokens_with_context is None else int(prefill_tokens_with_context),
        _stream()), "fk_merge_attn_states")


# --------------------------------------------------------------------------- norms
def rmsnorm(x, weight, eps, out=None):
    """out = bf16(x * rsqrt(mean(x^2)+eps) * w); x is [..., cols], last dim dense.
    2-D [T, cols] and 3-D [N, H, cols] (strided views allowed) are supported."""
    _need(x, BF16, "x")
    _need(weight, BF16, "weight")
    if x.stride(-1) != 1:
        raise _lib.FkError("x rows must be dense")
    cols = x.shape[-1]
    if out is None:
        out = torch.empty(x.shape, dtype=BF16, device=x.device)
    if x.dim() == 2:
        outer, inner = x.shape[0], 1
        xs = (x.stride(0) if outer else cols, 0)
        os_ = (out.stride(0) if outer else cols, 0)
    elif x.dim() == 3:
        outer, inner = x.shape[0], x.shape[1]
        xs = (x.stride(0), x.stride(1))
        os_ = (out.stride(0), out.stride(1))
    else:
        raise _lib.FkError("rmsnorm supports 2-D and 3-D inputs")
    check(lib.fk_rmsnorm(_ptr(x), xs[0], xs[1], inner, _ptr(out), os_[0], os_[1],
                         _ptr(weight), float(eps), outer, cols, _stream()), "fk_rmsnorm")
    return out


def fused_add_rmsnorm(x, residual, weight, eps) -> None:
    """In place: residual = bf16(x + residual); x = rmsnorm(residual) * w."""
    _need(x, BF16, "x")
    _need(residual, BF16, "residual")
    _need(weight, BF16, "weight")
    if x.dim() != 2 or residual.shape != x.shape or x.stride(1) != 1 or residual.stride(1) != 1:
        raise _lib.FkError("fused_add_rmsnorm needs matching 2-D row-dense tensors")
    rows, cols = x.shape
    check(lib.fk_fused_add_rmsnorm(_ptr(x), x.stride(0) if rows else cols, _ptr(residual),
                                   residual.stride(0) if rows else cols, _ptr(weight),
                                   float(eps), rows, cols, _stream()),
          "fk_fused_add_rmsnorm")


# ---------------------------------------------------------------------------- rope
def rope_neox(positions, query, key, head_dim, cos_sin_cache, status=None) -> None:
    """In-place NeoX rotation of query [T, Hq*D] and key [T, Hkv*D]."""
    _need(query, BF16, "query")
    _need(positions, torch.int64, "positions")
    t = query.shape[0]
    q2 = query.view(t, -1)
    hq = q2.shape[1] // head_dim
    if key is not None:
        _need(key, BF16, "key")
        k2 = key.view(t, -1)
        hkv = k2.shape[1] // head_dim
        ks = k2.stride(0) if t else k2.shape[1]
    else:
        k2, hkv, ks = None, 0, 0
    if cos_sin_cache.dtype not in (torch.float32, BF16):
        raise _lib.FkError("cos_sin_cache must be fp32 or bf16")
    check(lib.fk_rope_neox(_ptr(positions), _ptr(q2), q2.stride(0) if t else q2.shape[1], hq,
                           _ptr(k2), ks, hkv, head_dim, _ptr(cos_sin_cache),
                           int(cos_sin_cache.dtype == torch.float32),
                           cos_sin_cache.shape[0], t, _status_ptr(status, query),
                           _stream()),
          "fk_rope_neox")


def qkv_rope_store(qkv, num_q_heads, num_kv_heads, head_dim, positions, cos_sin_cache,
                   q_norm_weight, k_norm_weight, eps, k_cache, v_cache, slot_mapping,
                   status=None, kv_layout="NHD") -> None:
    """Split + [per-head q/k RMSNorm] + NeoX RoPE in place on the packed qkv rows,
    and store rotated k / raw v into the paged cache at slot_mapping."""
    _need(qkv, BF16, "qkv")
    _need(positions, torch.int64, "positions")
    if qkv.dim() != 2 or qkv.stride(1) != 1:
        raise _lib.FkError("qkv must be 2-D row-dense")
    t = qkv.shape[0]
    num_slots, page = 0, 0
    if k_cache is not None:
        page = k_cache.shape[2] if kv_layout == "HND" else k_cache.shape[1]
        _need(slot_mapping, torch.int32, "slot_mapping")
        if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
            raise _lib.FkError("caches must be contiguous")
        num_slots = k_cache.numel() // (num_kv_heads * head_dim)
    check(lib.fk_qkv_rope_store(
        _ptr(qkv), qkv.stride(0) if t else qkv.shape[1], num_q_heads, num_kv_heads, head_dim,
        _ptr(positions), _ptr(cos_sin_cache), int(cos_sin_cache.dtype == torch.float32),
        cos_sin_cache.shape[0], _ptr(q_norm_weight), _ptr(k_norm_weight), float(eps),
        _ptr(k_cache), _ptr(v_cache), _ptr(slot_mapping), num_slots, page,
        int(kv_layout == "HND"), t, _status_ptr(status, qkv), _stream()), "fk_qkv_rope_store")


# ---------------------------------------------------------------------------- silu
def silu_and_mul(x, out=None):
    _need(x, BF16, "x")
    if x.dim() != 2 or x.stride(1) != 1:
        raise _lib.FkError("silu_and_mul needs a 2-D row-dense input")
    rows, d2 = x.shape
    d = d2 // 2
    if out is None:
        out = torch.empty((rows, d), dtype=BF16, device=x.device)
    check(lib.fk_silu_and_mul(_ptr(x), x.stride(0) if rows else d2, _ptr(out),
                              out.stride(0) if rows else d, rows, d, _stream()),
          "fk_silu_and_mul")
    return out


# ---------------------------------------------------------------------------- fill
def fill_u32(t: torch.Tensor, value: int = 0) -> None:
    """Fill a contiguous tensor (byte size a multiple of 4) with a 32-bit pattern."""
    nbytes = t.numel() * t.element_size()
    if not t.is_contiguous() or nbytes % 4:
        raise _lib.FkError("fill_u32 needs a contiguous tensor of whole 32-bit words")
    check(lib.fk_fill_u32(_ptr(t), nbytes // 4, value, _stream()), "fk_fill_u32")


def xor_u32(t: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """XOR of all 32-bit words of a contiguous tensor (byte size a multiple of 16)
    into the one-element int32 tensor `out` (made and zeroed when not given): a
    checksum, and a pure read stream for bandwidth measurements."""
    nbytes = t.numel() * t.element_size()
    if not t.is_contiguous() or nbytes % 16:
        raise _lib.FkError("xor_u32 needs a contiguous tensor of whole 16-byte groups")
    if out is None:
        out = torch.zeros(1, dtype=torch.int32, device=t.device)
    check(lib.fk_xor_u32(_ptr(t), nbytes // 4, _ptr(out), _stream()), "fk_xor_u32")
    return out


# -------------------------------------------------------------------------- argmax
def argmax_rows(x, out_val=None, out_idx=None):
    """(max as fp32, lowest index of the max) per row of a bf16 [rows, cols] matrix."""
    _need(x, BF16, "x")
    if x.dim() != 2 or x.stride(1) != 1:
        raise _lib.FkError("argmax_rows needs a 2-D row-dense input")
    rows, cols = x.shape
    if out_val is None:
        out_val = torch.empty(rows, dtype=torch.float32, device=x.device)
    if out_idx is None:
        out_idx = torch.empty(rows, dtype=torch.int64, device=x.device)
    check(lib.fk_argmax_bf16(_ptr(x), x.stride(0) if rows else cols, rows, cols,
                             _ptr(out_val), _ptr(out_idx), _stream()), "fk_argmax_bf16")
    return out_val, out_idx


# ---------------------------------------------------------------------------- gemm
def gemm_workspace_bytes(m, n, k) -> int:
    return int(lib.fk_gemm_bf16_workspace_bytes(m, n, k))


_GEMM_WS: dict = {}


def gemm_workspace(device) -> torch.Tensor:
    """Per-device stream-K workspace (flags + fp32 partial tiles), sized for the
    largest m, zero-initialised once.  The kernel leaves it zeroed, and GEMMs on
    one stream run one after the other, so a single buffer serves them all; a
    caller that runs GEMMs concurrently on several streams passes its own."""
    key = torch.device(device)
    if key.index is None and key.type == "cuda":
        key = torch.device("cuda", torch.cuda.current_device())
    ws = _GEMM_WS.get(key)
    if ws is None:
        ws = torch.zeros(gemm_workspace_bytes(256, 1, 64), dtype=torch.uint8, device=key)
        _GEMM_WS[key] = ws
    return ws


def gemm_bf16(x, w, bias=None, out=None, workspace=None, status=None):
    """y = x @ w.T (+ bias): x [m, k], w [n, k] contiguous, y [m, n] bf16."""
    _need(x, BF16, "x")
    _need(w, BF16, "w")
    if x.dim() != 2 or x.stride(1) != 1 or not w.is_contiguous():
        raise _lib.FkError("gemm_bf16 needs row-dense x and contiguous w")
    m, k = x.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=BF16, device=x.device)
    if workspace is None:
        workspace = gemm_workspace(x.device)
    # m <= 256: the weight-streaming decode kernel; more rows (prefill): the 256 x 256
    # tile kernel inside the same entry point
    check(lib.fk_gemm_bf16(_ptr(x), x.stride(0) if m else k, _ptr(w), _ptr(bias), _ptr(out),
                           out.stride(0) if m else n, m, n, k, _ptr(workspace),
                           workspace.numel() * workspace.element_size(),
                           _status_ptr(status, x), _stream()), "fk_gemm_bf16")
    return out


def gemm_bf16_push(x, w, bias, dst, nranks: int, call_counters: int, workspace=None,
                   status=None) -> None:
    """x @ w.T (+ bias) stored tile by tile into the receive areas `dst` (ctypes
    array of `nranks` device addresses) of all tensor-parallel ranks instead of a
    local y; `call_counters` = device address of this rank's per-row call counters."""
    _need(x, BF16, "x")
    _need(w, BF16, "w")
    if x.dim() != 2 or x.stride(1) != 1 or not w.is_contiguous():
        raise _lib.FkError("gemm_bf16_push needs row-dense x and contiguous w")
    m, k = x.shape
    n = w.shape[0]
    if workspace is None:
        workspace = gemm_workspace(x.device)
    check(lib.fk_gemm_bf16_push(_ptr(x), x.stride(0) if m else k, _ptr(w), _ptr(bias), m, n, k,
                                _ptr(workspace), workspace.numel() * workspace.element_size(),
                                dst, nranks, call_counters, _status_ptr(status, x), _stream()),
          "fk_gemm_bf16_push")


def gemm_silu_mul_fusable(m: int, n: int, k: int) -> bool:
    """True when silu_and_mul(x @ w.T) for x [m, k], w [n, k] runs as one launch."""
    return bool(lib.fk_gemm_bf16_silu_mul_fusable(m, n, k))


def gemm_silu_mul(x, w, bias=None, out=None, workspace=None, status=None):
    """silu_and_mul(x @ w.T (+ bias)) in one launch: w = [gate; up] rows, result
    [m, n / 2].  Raises for shapes without the single-launch form (see
    gemm_silu_mul_fusable)."""
    _need(x, BF16, "x")
    _need(w, BF16, "w")
    if x.dim() != 2 or x.stride(1) != 1 or not w.is_contiguous():
        raise _lib.FkError("gemm_silu_mul needs row-dense x and contiguous w")
    m, k = x.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n // 2), dtype=BF16, device=x.device)
    if workspace is None:
        workspace = gemm_workspace(x.device)
    check(lib.fk_gemm_bf16_silu_mul(_ptr(x), x.stride(0) if m else k, _ptr(w), _ptr(bias),
                                    _ptr(out), out.stride(0) if m else n // 2, m, n, k,
                                    _ptr(workspace),
                                    workspace.numel() * workspace.element_size(),
                                    _status_ptr(status, x), _stream()), "fk_gemm_bf16_silu_mul")
    return out


# -------------------------------------------------------------------- decode block
class BlockProgram:
    """Builder for one fk_decode_block launch: the projections, residual-add +
    RMSNorms and the split + RoPE + KV store a decoder layer runs between two
    attention calls, executed by one persistent kernel.  Phases run in the order
    they are added; every tensor is bf16, row-dense, with m rows."""

    def __init__(self, m: int, device):
        self.m, self.device = int(m), torch.device(device)
        self.phases: list = []
        self._keep: list = []          # tensors referenced by raw pointers

    def _phase(self, kind):
        ph = _lib.BlockPhase()
        ph.kind = kind
        self.phases.append(ph)
        return ph

    def _gemm(self, kind, x, w, bias, out):
        _need(x, BF16, "x")
        _need(w, BF16, "w")
        if x.dim() != 2 or x.shape[0] != self.m or x.stride(1) != 1 or not w.is_contiguous():
            raise _lib.FkError("block projection needs row-dense x [m, k] and contiguous w")
        n, k = w.shape
        cols = n // 2 if kind == _lib.PHASE_GEMM_SILU_MUL else n
        if out is None:
            out = torch.empty((self.m, cols), dtype=BF16, device=x.device)
        ph = self._phase(kind)
        ph.x, ph.x_stride = x.data_ptr(), x.stride(0)
        ph.w, ph.bias = w.data_ptr(), _ptr(bias)
        ph.y, ph.y_stride = out.data_ptr(), out.stride(0)
        ph.n, ph.k = n, k
        self._keep += [x, w, bias, out]
        return out

    def gemm(self, x, w, bias=None, out=None):
        """out = x @ w.T (+ bias)"""
        return self._gemm(_lib.PHASE_GEMM, x, w, bias, out)

    def gemm_silu_mul(self, x, w, bias=None, out=None):
        """out = silu_and_mul(x @ w.T (+ bias)), w = [gate; up]"""
        if w.shape[0] % 128:
            raise _lib.FkError("gate/up projection rows must be a multiple of 128")
        return self._gemm(_lib.PHASE_GEMM_SILU_MUL, x, w, bias, out)

    def add_rmsnorm(self, x, residual, weight, eps, out=None):
        """residual += x (x None: nothing added); out = rmsnorm(residual) * weight"""
        _need(residual, BF16, "residual")
        _need(weight, BF16, "weight")
        if residual.dim() != 2 or residual.shape[0] != self.m or residual.stride(1) != 1:
            raise _lib.FkError("block norm needs a row-dense residual [m, cols]")
        if out is None:
            out = torch.empty_like(residual)
        ph = self._phase(_lib.PHASE_ADD_RMSNORM)
        if x is not None:
            _need(x, BF16, "x")
            if x.shape != residual.shape or x.stride(1) != 1:
                raise _lib.FkError("block norm: x and residual must have the same shape")
            ph.x, ph.x_stride = x.data_ptr(), x.stride(0)
        ph.residual, ph.residual_stride = residual.data_ptr(), residual.stride(0)
        ph.norm_weight, ph.eps = weight.data_ptr(), float(eps)
        ph.y, ph.y_stride = out.data_ptr(), out.stride(0)
        ph.n = residual.shape[1]
        self._keep += [x, residual, weight, out]
        return out

    def qkv_rope_store(self, qkv, num_q_heads, num_kv_heads, head_dim, positions,
                       cos_sin_cache, q_norm_weight, k_norm_weight, eps, k_cache, v_cache,
                       slot_mapping, kv_layout="NHD"):
        """ops.qkv_rope_store on the packed qkv rows (bf16 cos/sin cache)."""
        _need(qkv, BF16, "qkv")
        _need(positions, torch.int64, "positions")
        _need(cos_sin_cache, BF16, "cos_sin_cache")
        if qkv.dim() != 2 or qkv.shape[0] != self.m or qkv.stride(1) != 1:
            raise _lib.FkError("qkv must be row-dense [m, (Hq + 2 Hkv) * D]")
        ph = self._phase(_lib.PHASE_QKV_ROPE_STORE)
        ph.x, ph.x_stride = qkv.data_ptr(), qkv.stride(0)
        ph.num_q_heads, ph.num_kv_heads, ph.head_dim = num_q_heads, num_kv_heads, head_dim
        ph.positions = positions.data_ptr()
        ph.cos_sin_cache, ph.cache_is_fp32 = cos_sin_cache.data_ptr(), 0
        ph.max_position = cos_sin_cache.shape[0]
        ph.q_norm_weight, ph.k_norm_weight = _ptr(q_norm_weight), _ptr(k_norm_weight)
        ph.eps = float(eps)
        if k_cache is not None:
            _need(slot_mapping, torch.int32, "slot_mapping")
            if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
                raise _lib.FkError("caches must be contiguous")
            ph.k_cache, ph.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
            ph.slot_mapping = slot_mapping.data_ptr()
            ph.num_slots = k_cache.numel() // (num_kv_heads * head_dim)
            ph.block_size = k_cache.shape[2] if kv_layout == "HND" else k_cache.shape[1]
            ph.kv_layout = int(kv_layout == "HND")
        self._keep += [qkv, positions, cos_sin_cache, q_norm_weight, k_norm_weight, k_cache,
                       v_cache, slot_mapping]

    def launch(self, workspace=None, status=None) -> None:
        if not self.phases:
            return
        if workspace is None:
            workspace = gemm_workspace(self.device)
        arr = (_lib.BlockPhase * len(self.phases))(*self.phases)
        st = status if status is not None else default_status(self.device)
        check(lib.fk_decode_block(arr, len(self.phases), self.m, _ptr(workspace),
                                  workspace.numel() * workspace.element_size(), st.data_ptr(),
                                  _stream()), "fk_decode_block")


def decode_block_max_rows() -> int:
    return 128
