"""Library reference points for bench.py: what the reference's own GPU path costs
on the same tensors, timed beside this build's kernels.

The reference runs its decode step on library kernels: cuBLAS through F.linear
for the projections (fastkernels/tasks/baseline/L1/linear.py:13-17), vLLM's
bundled flash-attention for NHD pools
(fastkernels/tasks/baseline/L1/flash_attn_decode.py:164-181) and FlashInfer's
trtllm-gen decode for the HND / 16 pool it selects on Blackwell
(fastkernels/tasks/baseline/L1/flashinfer_decode.py:92-107,
fastkernels/infra/context.py:57-67).  Nothing here is on the product path: the
functions are called by bench.py AFTER its timed region, each library inside
try/except so that a missing or failing import becomes a string in the report.

Timing follows the reference's harness (fastkernels/bench.py:1938-2020): warm-up
10, then 50 calls, before each one a buffer of twice the L2 size is zeroed, CUDA
events around each call, median.
"""
from __future__ import annotations

import statistics

import numpy as np
import torch

from . import ops

WARMUP, ITERS = 10, 50


def _flush_buffer(device) -> torch.Tensor:
    l2 = torch.cuda.get_device_properties(device).L2_cache_size
    return torch.empty(int(2 * l2), dtype=torch.int8, device=device)


def median_us(fn, flush: torch.Tensor, warmup: int = WARMUP, iters: int = ITERS) -> float:
    for _ in range(warmup):
        flush.zero_()
        fn()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    for i in range(iters):
        flush.zero_()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    return statistics.median(s.elapsed_time(e) for s, e in zip(starts, ends)) * 1e3


def _try(report: dict, key: str, make):
    """report[key] = make() or the error text."""
    try:
        report[key] = make()
    except Exception as exc:  # noqa: BLE001 - depends on the installed library builds
        report[key] = f"unavailable: {type(exc).__name__}: {exc}"[:200]


def projection_points(eng, batch: int, flush) -> dict:
    """Own tcgen05 GEMM vs cuBLAS (F.linear) on the decoder's five decode shapes,
    with the engine's own weights."""
    layer = eng.model.model.layers[0]
    shapes = {
        "qkv": layer.self_attn.qkv_proj.weight,
        "o": layer.self_attn.o_proj.weight,
        "gate_up": layer.mlp.gate_up_proj.weight,
        "down": layer.mlp.down_proj.weight,
        "lm_head": eng.model.lm_head.embedding_op.emb.weight,
    }
    out = {}
    g = torch.Generator(device=eng.device).manual_seed(7)
    for name, w in shapes.items():
        n, k = w.shape
        x = torch.randn((batch, k), generator=g, device=eng.device).to(torch.bfloat16)
        y = torch.empty((batch, n), dtype=torch.bfloat16, device=eng.device)
        entry = {"m": batch, "n": n, "k": k,
                 "own_us": median_us(lambda: ops.gemm_bf16(x, w, out=y), flush)}
        _try(entry, "cublas_us",
             lambda: median_us(lambda: torch.nn.functional.linear(x, w), flush))
        out[name] = entry
    return out


def attention_points(batch, hq, hkv, lens, flush, d=128, block=256) -> dict:
    """Paged decode attention of ONE layer of the workload (seeded contexts `lens`):
    this build on an NHD / 256 pool and on an HND / 16 pool, vLLM's flash-attention
    as FlashAttnDecode calls it, FlashInfer's trtllm-gen decode as TRTLLMDecode
    calls it.  Runs in a process of its own (see `attention_points_in_child`)."""
    dev = torch.device("cuda", torch.cuda.current_device())
    b = batch
    lens = np.asarray(lens, dtype=np.int64)
    lens_d = torch.from_numpy(lens.astype(np.int32)).to(dev)
    g = torch.Generator(device=dev).manual_seed(11)
    q = (torch.randn((b, hq, d), generator=g, device=dev) * 0.5).to(torch.bfloat16)
    scale = d ** -0.5
    out = {}

    def pool(page, hnd):
        """Pool with one spare page per sequence and a dense block table."""
        pages = (lens + page - 1) // page + 1
        nb = int(pages.sum())
        perm = torch.randperm(nb, generator=g, device=dev).to(torch.int32).cpu().numpy()
        bt = np.zeros((b, int(pages.max())), np.int32)
        o_ = 0
        for i in range(b):
            bt[i, :pages[i]] = perm[o_:o_ + pages[i]]
            o_ += pages[i]
        shape = (nb, hkv, page, d) if hnd else (nb, page, hkv, d)
        k = torch.empty(shape, dtype=torch.bfloat16, device=dev).normal_(0, 0.5, generator=g)
        v = torch.empty(shape, dtype=torch.bfloat16, device=dev).normal_(0, 0.5, generator=g)
        return k, v, torch.from_numpy(bt).to(dev)

    ws = torch.empty(ops.attn_workspace_bytes(b, hq, d, 64), dtype=torch.uint8, device=dev)
    kc, vc, bt = pool(block, False)
    o = torch.empty_like(q)
    out["own_nhd_us"] = median_us(lambda: ops.paged_decode_attn(
        q, kc, vc, lens_d, bt, scale, ws, 64, out=o), flush)
    # as inside a decode step: the split schedule is computed once per step and
    # shared by all layers, a layer's call is the main kernel + the merge kernel
    ops.paged_decode_attn_plan(lens_d, bt, block, hq, hkv, d, ws, 64)
    out["own_nhd_planned_us"] = median_us(lambda: ops.paged_decode_attn(
        q, kc, vc, lens_d, bt, scale, ws, 64, out=o, planned=True), flush)

    def vllm_fa():
        from vllm.vllm_flash_attn import flash_attn_varlen_func
        cu_q = torch.arange(0, b + 1, device=dev, dtype=torch.int32)
        kw = dict(q=q, k=kc, v=vc, cu_seqlens_q=cu_q, max_seqlen_q=1, seqused_k=lens_d,
                  max_seqlen_k=int(lens.max()), softmax_scale=scale, causal=True,
                  block_table=bt)
        res = flash_attn_varlen_func(**kw)
        torch.cuda.synchronize()
        out["vllm_flash_attn_max_abs_diff_vs_own"] = float((res.float() - o.float()).abs().max())
        return median_us(lambda: flash_attn_varlen_func(**kw), flush)
    _try(out, "vllm_flash_attn_nhd_us", vllm_fa)
    del kc, vc
    # the reference's default pool on this GPU: HND, 16-token pages, same contexts
    k16, v16, bt16 = pool(16, True)
    o16 = torch.empty_like(q)
    out["own_hnd16_us"] = median_us(lambda: ops.paged_decode_attn(
        q, k16, v16, lens_d, bt16, scale, ws, 64, out=o16, kv_layout="HND"), flush)
    ops.paged_decode_attn_plan(lens_d, bt16, 16, hq, hkv, d, ws, 64)
    out["own_hnd16_planned_us"] = median_us(lambda: ops.paged_decode_attn(
        q, k16, v16, lens_d, bt16, scale, ws, 64, out=o16, kv_layout="HND", planned=True),
        flush)

    def trtllm():
        from flashinfer.decode import trtllm_batch_decode_with_kv_cache
        wsb = torch.zeros(512 * 1024 * 1024, dtype=torch.uint8, device=dev)
        kw = dict(query=q, kv_cache=(k16, v16), workspace_buffer=wsb, block_tables=bt16,
                  seq_lens=lens_d, max_seq_len=int(lens.max()), bmm1_scale=scale,
                  bmm2_scale=1.0, window_left=-1, sinks=None, kv_layout="HND")
        res = trtllm_batch_decode_with_kv_cache(**kw)
        torch.cuda.synchronize()
        out["flashinfer_trtllm_max_abs_diff_vs_own"] = \
            float((res.float() - o16.float()).abs().max())
        return median_us(lambda: trtllm_batch_decode_with_kv_cache(**kw), flush)
    _try(out, "flashinfer_trtllm_hnd16_us", trtllm)
    out["layer_kv_tokens"] = int(lens.sum())
    out["layer_kv_bytes"] = int(2 * lens.sum() * hkv * d * 2)
    return out


def attention_points_in_child(wl, lens, device_index: int) -> dict:
    """Runs `python -m fastkernels_b200.library_points` as a child process: the
    library kernels get a CUDA context of their own (a failure there cannot take
    the benchmark's context with it) and their pools do not sit on top of the
    benchmark's."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([root, env.get("PYTHONPATH", "")])
    cmd = [sys.executable, "-m", "fastkernels_b200.library_points", "--device", str(device_index),
           "--batch", str(wl["batch"]), "--hq", str(wl["hq"]), "--hkv", str(wl["hkv"]),
           "--lens", ",".join(str(int(x)) for x in lens)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    if r.returncode != 0 or not lines:
        return {"unavailable": f"child exit code {r.returncode}: {r.stderr.strip()[-300:]}"}
    return json.loads(lines[-1])


def step_with_library_projections(eng, batch: int, steps: int) -> dict:
    """Timing only: the same CUDA graph captured once more with every projection
    of the step routed to F.linear (cuBLAS), replayed `steps` times.  The patch
    lives for the duration of this call; tokens of this pass are discarded."""
    import fastkernels_b200.ops as ops_mod

    own = ops_mod.gemm_bf16
    own_fusable = ops_mod.gemm_silu_mul_fusable

    def library_gemm(x, w, bias=None, out=None, workspace=None, status=None):
        y = torch.nn.functional.linear(x, w, bias)
        if out is not None:
            out.copy_(y)
            return out
        return y

    def replay_ms():
        for _ in range(3):
            eng.step(sync=False)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            eng.step(sync=False)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    # own, library, own, library: the order is alternated because a long run drifts
    # with the power state of the GPU
    own_ms, lib_ms, err = [], [], None
    for rnd in range(2):
        eng.capture_cudagraph([batch])
        own_ms.append(replay_ms())
        try:
            # every projection through F.linear; the gate/up projection then feeds
            # the separate SiLU kernel, as in the reference
            ops_mod.gemm_bf16 = library_gemm
            ops_mod.gemm_silu_mul_fusable = lambda m, n, k: False
            eng.capture_cudagraph([batch])
            lib_ms.append(replay_ms())
        except Exception as exc:  # noqa: BLE001
            err = f"unavailable: {type(exc).__name__}: {exc}"[:200]
        finally:
            ops_mod.gemm_bf16 = own
            ops_mod.gemm_silu_mul_fusable = own_fusable
    eng.capture_cudagraph([batch])
    return {"own_projections_ms_per_step": own_ms,
            "cublas_projections_ms_per_step": lib_ms if err is None else err}


def collect(eng, wl, steps: int) -> dict:
    flush = _flush_buffer(eng.device)
    report = {"method": f"L2 flushed before each call, median of {ITERS} after {WARMUP} warm-up "
                        "calls, CUDA events (the reference harness' timing)"}
    _try(report, "projections", lambda: projection_points(eng, wl["batch"], flush))
    lens = eng.graph_vars["context_lens"][:wl["batch"]].cpu().numpy()
    _try(report, "decode_attention",
         lambda: attention_points_in_child(wl, lens, eng.device.index or 0))
    _try(report, "step", lambda: step_with_library_projections(eng, wl["batch"], steps))
    return report


if __name__ == "__main__":
    import argparse
    import json
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--batch", type=int, required=True)
    ap.add_argument("--hq", type=int, required=True)
    ap.add_argument("--hkv", type=int, required=True)
    ap.add_argument("--lens", required=True, help="comma-separated context lengths")
    a = ap.parse_args()
    torch.cuda.set_device(a.device)
    lens_ = [int(x) for x in a.lens.split(",")]
    assert len(lens_) == a.batch
    print(json.dumps(attention_points(a.batch, a.hq, a.hkv, lens_,
                                      _flush_buffer(torch.device("cuda", a.device)))),
          flush=True)
