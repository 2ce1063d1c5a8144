"""Single-kernel micro-benchmarks through the C-ABI (CUDA-event timing, L2 flush
between iterations); also the small, bounded cases used for ncu captures.

    python -m fastkernels_b200.microbench attn  --batch 64 --hq 32 --hkv 8 --lo 1024 --hi 8192
    python -m fastkernels_b200.microbench gemm  --m 64 --n 6144 --k 4096 [--cublas]
    python -m fastkernels_b200.microbench gemm_silu --m 64 --n 24576 --k 4096   (gate/up + SiLU)
    python -m fastkernels_b200.microbench chain --tokens 4096          (config-2 fused chain)
    python -m fastkernels_b200.microbench prefill --batch 4 --hq 32 --hkv 8 --seqlen 4096
    python -m fastkernels_b200.microbench engine_prefill --batch 8 --seqlen 1024   (whole model)
    python -m fastkernels_b200.microbench suite                        (all benchmark shapes)

Each run prints one JSON object per case: median / min time, algorithmic bytes,
achieved GB/s and the fraction of the measured HBM peak.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch

from . import ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def hbm_peak() -> float:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"])
    return 6650.0


_flush = None


def timeit(fn, iters=20, warm=3, flush=True):
    global _flush
    if flush and _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            ops.fill_u32(_flush, 0)   # the library's own kernel: same carveout
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def report(name, med_ms, min_ms, nbytes, extra=None):
    peak = hbm_peak()
    d = dict(case=name, ms_med=med_ms, ms_min=min_ms, bytes=int(nbytes),
             gbs_med=nbytes / med_ms / 1e6, gbs_min=nbytes / min_ms / 1e6,
             frac_of_measured_hbm=nbytes / med_ms / 1e6 / peak)
    if extra:
        d.update(extra)
    print(json.dumps(d), flush=True)
    return d


def attn_case(batch, hq, hkv, lens, block=256, max_splits=64, iters=20, name="attn",
              layout="NHD", libs=False):
    d, dev = 128, "cuda"
    g = torch.Generator(device=dev).manual_seed(1)
    lens = np.asarray(lens, dtype=np.int64)
    pages = (lens + block - 1) // block
    nb = int(pages.sum())
    perm = torch.randperm(nb, generator=g, device=dev).to(torch.int32).cpu().numpy()
    bt = np.full((batch, int(pages.max())), -1, np.int32)
    o = 0
    for i in range(batch):
        bt[i, :pages[i]] = perm[o:o + pages[i]]
        o += pages[i]
    bt_d = torch.from_numpy(bt).cuda()
    lens_d = torch.from_numpy(lens.astype(np.int32)).cuda()
    q = (torch.randn((batch, hq, d), generator=g, device=dev) * 0.5).to(torch.bfloat16)
    shape = (nb, block, hkv, d) if layout == "NHD" else (nb, hkv, block, d)
    kc = torch.empty(shape, dtype=torch.bfloat16, device=dev).normal_(0, 0.5, generator=g)
    vc = torch.empty(shape, dtype=torch.bfloat16, device=dev).normal_(0, 0.5, generator=g)
    ws = torch.empty(ops.attn_workspace_bytes(batch, hq, d, max_splits), dtype=torch.uint8,
                     device=dev)
    out = torch.empty_like(q)
    st = ops.new_status(dev)

    def fn():
        ops.paged_decode_attn(q, kc, vc, lens_d, bt_d, d ** -0.5, ws, max_splits, out=out,
                              status=st, kv_layout=layout)

    med, mn = timeit(fn, iters=iters)
    nbytes = 2 * int(lens.sum()) * hkv * d * 2 + 2 * batch * hq * d * 2 + 4 * batch + 4 * nb
    plan = ws[:16].view(torch.int32).tolist()
    extra = dict(batch=batch, hq=hq, hkv=hkv, tokens=int(lens.sum()), chunks=plan[0],
                 chunk_tokens=plan[1], status=int(st.item()))
    if libs and layout == "NHD":
        extra.update(_library_decode_attention(q, kc, vc, lens, lens_d, bt, bt_d, block, iters))
    return report(name, med, mn, nbytes, extra)


def _library_decode_attention(q, kc, vc, lens, lens_d, bt, bt_d, block, iters):
    """Reference points: the paged decode attention of the libraries installed next
    to torch, on the same tensors and with the same timing method.  vLLM's bundled
    flash-attention is the call behind the reference's FlashAttnDecode
    (fastkernels/tasks/baseline/L1/flash_attn_decode.py:164-181)."""
    b, hq, d = q.shape
    hkv = kc.shape[2]
    res = {}
    try:
        from flash_attn import flash_attn_with_kvcache
        q4 = q.view(b, 1, hq, d)
        ms, _ = timeit(lambda: flash_attn_with_kvcache(q4, kc, vc, cache_seqlens=lens_d,
                                                       block_table=bt_d, causal=True),
                       iters=iters)
        res["flash_attn_kvcache_us"] = ms * 1e3
    except Exception as e:  # pragma: no cover - depends on the installed build
        res["flash_attn_error"] = repr(e)[:120]
    try:
        from vllm.vllm_flash_attn import flash_attn_varlen_func
        cu_q = torch.arange(0, b + 1, device=q.device, dtype=torch.int32)
        ms, _ = timeit(lambda: flash_attn_varlen_func(
            q, kc, vc, max_seqlen_q=1, cu_seqlens_q=cu_q, max_seqlen_k=int(lens.max()),
            seqused_k=lens_d, causal=True, block_table=bt_d), iters=iters)
        res["vllm_flash_attn_us"] = ms * 1e3
    except Exception as e:  # pragma: no cover
        res["vllm_flash_attn_error"] = repr(e)[:120]
    try:
        import flashinfer
        pages = (lens + block - 1) // block
        wsb = torch.empty(256 << 20, dtype=torch.uint8, device=q.device)
        w = flashinfer.BatchDecodeWithPagedKVCacheWrapper(wsb, "NHD")
        indptr = torch.from_numpy(np.concatenate([[0], np.cumsum(pages)]).astype(np.int32)).cuda()
        indices = torch.from_numpy(
            np.concatenate([bt[i, :pages[i]] for i in range(b)]).astype(np.int32)).cuda()
        last = torch.from_numpy(((lens - 1) % block + 1).astype(np.int32)).cuda()
        w.plan(indptr, indices, last, hq, hkv, d, block, q_data_type=torch.bfloat16)
        ms, _ = timeit(lambda: w.run(q, (kc, vc)), iters=iters)
        res["flashinfer_decode_us"] = ms * 1e3
    except Exception as e:  # pragma: no cover
        res["flashinfer_error"] = repr(e)[:120]
    return res


def tensor_peak() -> float:
    """Measured cuBLAS bf16 burst throughput in TFLOP/s (fallback: an earlier
    measurement on the same GPU type)."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f).get("bf16_tflops", 1590.0))
    return 1590.0


def prefill_case(batch, hq, hkv, seqlen, prefix=0, paged=False, block=256, iters=20,
                 name="prefill", sdpa=False):
    """Causal prefill attention of `batch` prompts of `seqlen` tokens each (after
    `prefix` cached tokens).  FLOPs counted: 4 * Hq * D * visible (query, key)
    pairs, i.e. the causal half only."""
    d = 128
    tq, tk = batch * seqlen, batch * (seqlen + prefix)
    g = torch.Generator(device="cuda").manual_seed(7)
    q = (torch.randn((tq, hq, d), device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    cu_q = torch.arange(0, batch + 1, device="cuda", dtype=torch.int32) * seqlen
    cu_k = torch.arange(0, batch + 1, device="cuda", dtype=torch.int32) * (seqlen + prefix)
    bt = None
    if paged:
        pages = (seqlen + prefix + block - 1) // block
        nb = batch * pages
        k = (torch.randn((nb, block, hkv, d), device="cuda", generator=g) * 0.5).to(torch.bfloat16)
        v = (torch.randn((nb, block, hkv, d), device="cuda", generator=g) * 0.5).to(torch.bfloat16)
        bt = torch.randperm(nb, device="cuda", generator=g).to(torch.int32).view(batch, pages)
    else:
        k = (torch.randn((tk, hkv, d), device="cuda", generator=g) * 0.5).to(torch.bfloat16)
        v = (torch.randn((tk, hkv, d), device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    out = torch.empty_like(q)
    st = ops.new_status("cuda")
    scale = d ** -0.5

    def run():
        ops.prefill_attn(q, k, v, cu_q, cu_k, seqlen, scale, causal=True, block_table=bt,
                         out=out, status=st)

    med, mn = timeit(run, iters=iters)
    pairs = batch * (seqlen * prefix + seqlen * (seqlen + 1) // 2)
    flops = 4.0 * hq * d * pairs
    peak = tensor_peak()
    res = dict(case=name, ms_med=med, ms_min=mn, flops=flops, tflops_med=flops / med / 1e9,
               tflops_min=flops / mn / 1e9, frac_of_measured_bf16=flops / med / 1e9 / peak,
               status=int(st.item()))
    if sdpa and not paged and prefix == 0:
        # torch's fused attention on the same problem (library reference point)
        q4 = q.view(batch, seqlen, hq, d).transpose(1, 2)
        k4 = k.view(batch, seqlen, hkv, d).transpose(1, 2)
        v4 = v.view(batch, seqlen, hkv, d).transpose(1, 2)
        f = lambda: torch.nn.functional.scaled_dot_product_attention(  # noqa: E731
            q4, k4, v4, is_causal=True, enable_gqa=True)
        try:
            m2, _ = timeit(f, iters=iters)
            res["torch_sdpa_ms"] = m2
            res["torch_sdpa_tflops"] = flops / m2 / 1e9
        except Exception as e:  # pragma: no cover - depends on the torch build
            res["torch_sdpa_error"] = str(e)[:80]
    print(json.dumps(res), flush=True)
    return res


def engine_prefill_case(batch, seqlen, layers=36, iters=3, chunk=None):
    """Whole-model prefill of `batch` prompts of `seqlen` tokens through
    DecodeEngine.prefill on the Qwen3-8B shape (random-init weights): prompt tokens
    per second, host preparation and the first-token D2H included."""
    from .candidate.L4.llama import LlamaConfig
    from .engine import DecodeEngine
    cfg = LlamaConfig(hidden_size=4096, intermediate_size=12288, num_hidden_layers=layers,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                      vocab_size=151936, max_position_embeddings=seqlen + 64,
                      rms_norm_eps=1e-6, rope_theta=1e6, qk_norm=True, kv_block_size=256)
    pages = (seqlen + 1 + 255) // 256 + 1
    rs = np.random.RandomState(5)
    prompts = [rs.randint(0, 151936, size=seqlen).tolist() for _ in range(batch)]
    ts = []
    eng = DecodeEngine(cfg, max_num_seqs=batch * (iters + 1), max_model_len=seqlen + 64,
                       num_kv_blocks=pages * batch * (iters + 1) + 2, device="cuda", seed=1)
    for it in range(iters + 1):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.prefill(prompts, chunk_tokens=chunk)
        b.record()
        torch.cuda.synchronize()
        if it:                      # the first pass warms allocators and tensor maps
            ts.append(a.elapsed_time(b))
    ts.sort()
    med = ts[len(ts) // 2]
    params = layers * (4096 * 6144 + 4096 * 4096 + 4096 * 24576 + 12288 * 4096)
    flops = 2.0 * params * batch * seqlen + 4.0 * 32 * 128 * layers * batch * seqlen * (seqlen + 1) / 2
    res = dict(case="engine_prefill", batch=batch, seqlen=seqlen, layers=layers, ms_med=med,
               prompt_tokens_per_s=batch * seqlen / med * 1e3, tflops=flops / med / 1e9,
               frac_of_measured_bf16=flops / med / 1e9 / tensor_peak(),
               status=int(eng.status.item()))
    print(json.dumps(res), flush=True)
    return res


def gemm_case(m, n, k, cublas=False, iters=20, name="gemm"):
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(2)
    x = torch.randn((m, k), generator=g, device=dev).to(torch.bfloat16)
    w = torch.empty((n, k), dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=g)
    y = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    st = ops.new_status(dev)
    med, mn = timeit(lambda: ops.gemm_bf16(x, w, out=y, status=st), iters=iters)
    nbytes = n * k * 2 + m * k * 2 + m * n * 2
    extra = dict(m=m, n=n, k=k, tflops_med=2.0 * m * n * k / med / 1e9, status=int(st.item()))
    if cublas:
        cm, _ = timeit(lambda: torch.nn.functional.linear(x, w), iters=iters)
        extra["cublas_ms_med"] = cm
        extra["cublas_gbs_med"] = nbytes / cm / 1e6
        extra["max_abs_diff_vs_cublas"] = float(
            (y.float() - torch.nn.functional.linear(x, w).float()).abs().max())
    return report(name, med, mn, nbytes, extra)


def gemm_silu_case(m, n, k, iters=20, name="gemm_silu"):
    """silu_and_mul(x W^T): the single-launch form against gate/up projection +
    SiLU kernel as two launches."""
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(4)
    x = torch.randn((m, k), generator=g, device=dev).to(torch.bfloat16)
    w = torch.empty((n, k), dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=g)
    y = torch.empty((m, n // 2), dtype=torch.bfloat16, device=dev)
    mid = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    st = ops.new_status(dev)
    med, mn = timeit(lambda: ops.gemm_silu_mul(x, w, out=y, status=st), iters=iters)

    def two():
        ops.gemm_bf16(x, w, out=mid, status=st)
        ops.silu_and_mul(mid, y)
    med2, _ = timeit(two, iters=iters)
    nbytes = n * k * 2 + m * k * 2 + m * (n // 2) * 2
    return report(name, med, mn, nbytes, dict(m=m, n=n, k=k, two_launches_ms_med=med2,
                                              status=int(st.item())))


def chain_case(tokens=4096, hidden=4096, hq=32, hkv=8, d=128, iters=20):
    """Config 2: fused add+RMSNorm on [T, hidden], then split + RoPE + KV store on
    a packed qkv [T, (Hq+2Hkv)*D] (positions < 8192, distinct slots of a 256x256 pool)."""
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(3)
    x = torch.randn((tokens, hidden), generator=g, device=dev).to(torch.bfloat16)
    r = torch.randn((tokens, hidden), generator=g, device=dev).to(torch.bfloat16)
    w = (1 + 0.02 * torch.randn(hidden, generator=g, device=dev)).to(torch.bfloat16)
    qkv = torch.randn((tokens, (hq + 2 * hkv) * d), generator=g, device=dev).to(torch.bfloat16)
    pos = torch.randint(0, 8192, (tokens,), generator=g, device=dev)
    slots = torch.randperm(256 * 256, generator=g, device=dev)[:tokens].to(torch.int32)
    kc = torch.zeros((256, 256, hkv, d), dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    from .candidate.L1.rotary_emb import RotaryEmbedding
    cache = RotaryEmbedding(d, 8192, 1e6).cos_sin_cache.cuda().to(torch.bfloat16)
    e = 2
    med, mn = timeit(lambda: ops.fused_add_rmsnorm(x, r, w, 1e-6), iters=iters)
    report("fused_add_rmsnorm", med, mn, 4 * tokens * hidden * e + hidden * e)
    med, mn = timeit(lambda: ops.qkv_rope_store(qkv, hq, hkv, d, pos, cache, None, None, 1e-6,
                                                kc, vc, slots), iters=iters)
    report("qkv_rope_store", med, mn,
           tokens * (hq + 2 * hkv) * d * e + tokens * (hq + hkv) * d * e + 2 * tokens * hkv * d * e
           + tokens * d * e + 12 * tokens)
    k = qkv[:, hq * d:(hq + hkv) * d].view(tokens, hkv, d)
    v = qkv[:, (hq + hkv) * d:].view(tokens, hkv, d)
    med, mn = timeit(lambda: ops.store_kvcache(k, v, kc, vc, slots), iters=iters)
    report("store_kvcache", med, mn, 4 * tokens * hkv * d * e + 4 * tokens)
    gu = torch.randn((tokens, 2 * 12288), generator=g, device=dev).to(torch.bfloat16)
    out = torch.empty((tokens, 12288), dtype=torch.bfloat16, device=dev)
    med, mn = timeit(lambda: ops.silu_and_mul(gu, out), iters=iters)
    report("silu_and_mul", med, mn, 3 * tokens * 12288 * e)


def timeline_case():
    """Per-CTA time stamps of the decode projections and of the persistent decode
    block on the 8B shape (batch 64).  Needs a diagnostic copy of the library:

        python -m fastkernels_b200.build --define FK_GEMM_TRACE --define FK_BLOCK_TRACE
        FK_B200_LIB=build/libfk_b200_diag.so python -m fastkernels_b200.microbench timeline

    Prints, per kernel and stamp, min / median / max over the CTAs in microseconds
    from the first CTA's entry."""
    import ctypes
    from . import _lib
    L = _lib.lib
    if not hasattr(L, "fk_debug_read_gemm_trace") or not hasattr(L, "fk_debug_read_block_trace"):
        raise SystemExit("timeline needs the diagnostic build (see --help of this case)")
    for f in (L.fk_debug_read_gemm_trace, L.fk_debug_read_block_trace):
        f.restype, f.argtypes = ctypes.c_int, [ctypes.c_void_p]
    m, hidden, ffn, hq, hkv, d = 64, 4096, 12288, 32, 8, 128
    g = torch.Generator(device="cuda").manual_seed(5)

    def t(*shape, s=0.02):
        return (torch.randn(shape, generator=g, device="cuda") * s).to(torch.bfloat16)

    w = dict(qkv=t((hq + 2 * hkv) * d, hidden), o=t(hidden, hq * d), gate_up=t(2 * ffn, hidden),
             down=t(hidden, ffn))
    x = dict(qkv=t(m, hidden, s=0.5), o=t(m, hq * d, s=0.5), gate_up=t(m, hidden, s=0.5))
    ctas = dict(qkv=96, o=128, gate_up=148, down=128)
    act = torch.empty((m, ffn), dtype=torch.bfloat16, device="cuda")
    y = {k: torch.empty((m, v.shape[0]), dtype=torch.bfloat16, device="cuda") for k, v in w.items()}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    gemm_names = ["entry", "setup_done", "predecessors_done", "first_stage_landed",
                  "last_mma_issued", "accumulator_complete", "contributor_flags_seen",
                  "epilogue_done", "all_roles_done", "tmem_released"]

    def show(label, table, names, t0):
        print(label)
        for i, n in enumerate(names):
            col = table[:, i]
            col = col[col > 0]
            if len(col):
                print(f"    {n:24s} min {(col.min() - t0) / 1e3:7.2f}  med "
                      f"{(np.median(col) - t0) / 1e3:7.2f}  max {(col.max() - t0) / 1e3:7.2f}")

    def gemm_trace():
        buf = np.zeros(4 * 160 * 16, dtype=np.uint64)
        L.fk_debug_read_gemm_trace(buf.ctypes.data)
        return buf.reshape(4, 160, 16).astype(np.int64)

    # the four projections of a layer back to back, as in a decode step
    for _ in range(2):
        ops.fill_u32(flush, 0)
        torch.cuda.synchronize()
        for _ in range(2):
            ops.gemm_bf16(x["qkv"], w["qkv"], out=y["qkv"])
            ops.gemm_bf16(x["o"], w["o"], out=y["o"])
            ops.gemm_silu_mul(x["gate_up"], w["gate_up"], out=act)
            ops.gemm_bf16(act, w["down"], out=y["down"])
        torch.cuda.synchronize()
    tr = gemm_trace()
    order = sorted(range(4), key=lambda i: tr[i, 0, 0])
    t0 = tr[order[0], :96, 0].min()
    for i, name in zip(order, ["qkv", "o", "gate_up + SiLU", "down"]):
        n = ctas["gate_up" if "gate" in name else name]
        show(f"--- chain: {name} projection ({n} CTAs)", tr[i][:n], gemm_names, t0)

    # the persistent decode block on the same shapes
    from .candidate.L1.rotary_emb import RotaryEmbedding
    ln = torch.ones(hidden, dtype=torch.bfloat16, device="cuda")
    hn = torch.ones(d, dtype=torch.bfloat16, device="cuda")
    res = t(m, hidden, s=1.0)
    pos = torch.randint(0, 2048, (m,), generator=g, device="cuda")
    slots = torch.randperm(8 * 256, generator=g, device="cuda")[:m].to(torch.int32)
    cache = RotaryEmbedding(d, 2048, 1e6).cos_sin_cache.cuda().to(torch.bfloat16)
    kc = torch.zeros((8, 256, hkv, d), dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)

    def block():
        prog = ops.BlockProgram(m, "cuda")
        y1 = prog.gemm(x["o"], w["o"])
        h2 = prog.add_rmsnorm(y1, res, ln, 1e-6)
        a2 = prog.gemm_silu_mul(h2, w["gate_up"])
        y2 = prog.gemm(a2, w["down"])
        h = prog.add_rmsnorm(y2, res, ln, 1e-6)
        qkv = prog.gemm(h, w["qkv"])
        prog.qkv_rope_store(qkv, hq, hkv, d, pos, cache, hn, hn, 1e-6, kc, vc, slots)
        prog.launch()

    for _ in range(3):
        ops.fill_u32(flush, 0)
        torch.cuda.synchronize()
        block()
        torch.cuda.synchronize()
    buf = np.zeros(160 * 8 * 8, dtype=np.uint64)
    L.fk_debug_read_block_trace(buf.ctypes.data)
    bt = buf.reshape(160, 8, 8).astype(np.int64)[:148]
    t0 = bt[:, 0, 5].min()
    kinds = ["o projection", "add + norm", "gate_up + SiLU", "down projection", "add + norm",
             "qkv projection", "RoPE + store"]
    for pi, kind in enumerate(kinds):
        show(f"--- decode block phase {pi}: {kind}", bt[:, pi, :5],
             ["activations_released", "first_stage_landed", "last_mma_issued",
              "row_phase_started", "arrived_at_barrier"], t0)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(20):
        block()
    b.record()
    torch.cuda.synchronize()
    print(f"decode block, 20 launches back to back: {a.elapsed_time(b) * 1e3 / 20:.1f} us each")


def read_peak_case(gib=4, iters=10):
    """Read-only stream (fk_xor_u32) and write-only stream (fk_fill_u32) over a
    buffer far larger than L2, back to back between one event pair: what HBM gives
    a kernel that only reads (decode attention, weight streaming) as opposed to
    the copy figure of MEASURED_PEAKS.json."""
    buf = torch.empty(gib << 30, dtype=torch.uint8, device="cuda")
    ops.fill_u32(buf, 0x01010101)
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    res = {}
    for name, fn in (("read", lambda: ops.xor_u32(buf, out)), ("write", lambda: ops.fill_u32(buf, 7))):
        for _ in range(3):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        res[name + "_gbs"] = buf.numel() * iters / a.elapsed_time(b) / 1e6
    res.update(case="read_peak", bytes=buf.numel(), copy_peak_gbs=hbm_peak())
    print(json.dumps(res), flush=True)
    return res


def suite():
    rs = np.random.RandomState(3)
    attn_case(64, 32, 8, rs.randint(1024, 8193, 64), name="attn_c3_layer")
    attn_case(256, 64, 4, np.floor(np.exp(rs.uniform(np.log(64), np.log(32768), 256))),
              name="attn_c5")
    attn_case(8, 32, 8, rs.randint(128, 2049, 8) + 1, name="attn_c1")
    attn_case(64, 32, 8, rs.randint(1024, 8193, 64), block=16, layout="HND",
              name="attn_c3_layer_hnd16")
    attn_case(128, 32, 4, rs.randint(512, 8193, 128), name="attn_c4_tp2_layer")
    attn_case(128, 8, 1, rs.randint(512, 8193, 128), name="attn_c4_tp8_layer")
    for name, (m, n, k) in dict(qkv=(64, 6144, 4096), o=(64, 4096, 4096),
                                gate_up=(64, 24576, 4096), down=(64, 4096, 12288),
                                lm_head=(64, 151936, 4096), c4tp2_qkv=(128, 5120, 8192),
                                c4tp2_o=(128, 8192, 4096), c4tp2_gate_up=(128, 28672, 8192),
                                c4tp2_down=(128, 8192, 14336)).items():
        gemm_case(m, n, k, cublas=True, name="gemm_" + name)
    gemm_silu_case(64, 24576, 4096, name="gemm_silu_gate_up")
    chain_case()
    # prefill side (tensor-bound: TFLOP/s against the measured bf16 peak)
    prefill_case(4, 32, 8, 4096, name="prefill_4x4096")
    prefill_case(1, 32, 8, 16384, name="prefill_1x16384")
    prefill_case(16, 32, 8, 1024, name="prefill_16x1024")
    prefill_case(4, 32, 8, 4096, paged=True, name="prefill_4x4096_paged")
    for name, (m, n, k) in dict(gate_up=(8192, 24576, 4096), down=(8192, 4096, 12288),
                                qkv=(8192, 6144, 4096), o=(8192, 4096, 4096)).items():
        gemm_case(m, n, k, cublas=True, name="gemm_prefill_" + name)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["attn", "gemm", "gemm_silu", "chain", "prefill", "read_peak",
                                     "engine_prefill", "timeline", "suite"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--lo", type=int, default=1024)
    ap.add_argument("--hi", type=int, default=8192)
    ap.add_argument("--m", type=int, default=64)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--block", type=int, default=256)
    ap.add_argument("--layout", default="NHD", choices=["NHD", "HND"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--cublas", action="store_true")
    ap.add_argument("--seqlen", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--prefix", type=int, default=0)
    ap.add_argument("--paged", action="store_true")
    ap.add_argument("--sdpa", action="store_true")
    ap.add_argument("--libs", action="store_true",
                    help="attn: also time the installed libraries' paged decode attention")
    a = ap.parse_args()
    if a.what == "attn":
        rs = np.random.RandomState(3)
        attn_case(a.batch, a.hq, a.hkv, rs.randint(a.lo, a.hi + 1, a.batch), iters=a.iters,
                  block=a.block, layout=a.layout, libs=a.libs)
    elif a.what == "gemm":
        gemm_case(a.m, a.n, a.k, cublas=a.cublas, iters=a.iters)
    elif a.what == "gemm_silu":
        gemm_silu_case(a.m, a.n, a.k, iters=a.iters)
    elif a.what == "timeline":
        timeline_case()
    elif a.what == "chain":
        chain_case(a.tokens, iters=a.iters)
    elif a.what == "read_peak":
        read_peak_case()
    elif a.what == "engine_prefill":
        engine_prefill_case(a.batch, a.seqlen, layers=a.layers, iters=a.iters)
    elif a.what == "prefill":
        prefill_case(a.batch, a.hq, a.hkv, a.seqlen, prefix=a.prefix, paged=a.paged,
                     block=a.block, iters=a.iters, sdpa=a.sdpa)
    else:
        suite()


if __name__ == "__main__":
    main()
