#!/usr/bin/env python
"""Decode-throughput benchmark of the B200 decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c3|c4|c5]

Workload (synthetic, seeded): config "c3" = one decode step of a random-init
Qwen3-8B-architecture decoder (36 layers, hidden 4096, FFN 12288, 32 q / 8 kv
heads, head_dim 128, q/k RMSNorm, vocab 151936, bf16), batch 64, context lengths
uniform in [1024, 8192], paged KV block 256, CUDA-graph decode, greedy sampling.
"c4" = the Llama-3-70B-architecture decoder (80 layers, hidden 8192, FFN 28672,
64 q / 8 kv heads, vocab 128256, rope theta 5e5), batch 128, lengths in
[512, 8192]; it needs tensor parallelism (N >= 2).

A step = one decode step of the whole batch.  With N > 1 the script is launched
once per GPU (torch.distributed.run) and the model is tensor-parallel over the
N ranks (strong scaling: the total work is fixed).  Rank 0 prints ONE JSON line.

`value`   tokens/s with the step inputs already resident on the device: K graph
          replays timed with CUDA events on the launching stream (barrier +
          synchronize on both sides, max over ranks).  Every step streams all
          weights and the whole live KV cache (tens of GB) from HBM, far more
          than the 126 MB L2, so no explicit L2 flush is needed.
`e2e`     the same K steps through DecodeEngine.step(): per step the host
          prepares positions / slots / lengths / token ids in pinned memory,
          copies them to the device, replays the graph and reads the sampled
          token ids back before the next step starts.
`roofline` of the dominant kernel (paged decode attention, HBM-bound).
`cpu_baseline` the numpy oracle (a port of the reference's PyTorch CPU path) on
          this box's host cores, on a bounded sample of the same workload.
`library_points` (1 GPU) the reference's GPU path beside this build's kernels,
          measured after the timed region: cuBLAS on the five projection shapes,
          vLLM's flash-attention and FlashInfer's trtllm-gen decode on one
          layer's KV, and the whole step with the projections on cuBLAS.

--impl reference times that CPU port alone (no GPU work in the timed region).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "c3": dict(name="qwen3-8b-shape decode, batch 64, ctx U[1024,8192], block 256",
               layers=36, hidden=4096, ffn=12288, hq=32, hkv=8, d=128, vocab=151936,
               theta=1e6, eps=1e-6, qk_norm=True, batch=64, len_lo=1024, len_hi=8192,
               seed=202),
    "c4": dict(name="llama3-70b-shape decode, batch 128, ctx U[512,8192], block 256",
               layers=80, hidden=8192, ffn=28672, hq=64, hkv=8, d=128, vocab=128256,
               theta=5e5, eps=1e-5, qk_norm=False, batch=128, len_lo=512, len_hi=8192,
               seed=203),
}
WORKLOADS["c5"] = dict(
    name="skewed long-context paged decode attention, batch 256, 64 q / 4 kv heads, "
         "ctx log-U[64,32768], block 256",
    attention_only=True, hq=64, hkv=4, d=128, batch=256, len_lo=64, len_hi=32768, seed=205)
BLOCK = 256
METRIC = "decode_tokens_per_s"
UNIT = "tok/s"


def workload_lens(wl):
    rs = np.random.RandomState(wl["seed"])
    if wl.get("attention_only"):       # log-uniform lengths
        lo, hi = np.log(wl["len_lo"]), np.log(wl["len_hi"])
        return np.floor(np.exp(rs.uniform(lo, hi, size=wl["batch"]))).astype(np.int64)
    return rs.randint(wl["len_lo"], wl["len_hi"] + 1, size=wl["batch"]).astype(np.int64)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


# ------------------------------------------------------------------ clock sampling
class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons during the timed region."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        busy = [c for c in sm if mx and c > 0.25 * mx] or sm
        return {"sm_mhz": float(np.median(busy)) if busy else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------- CPU sample
def cpu_sample(wl, lens, kv_layer=None, steps=1, warmup=0):
    """The oracle's decode step on the host cores for ONE of the decoder's layers
    at the full batch, plus the final norm / lm-head / greedy max once; the full
    step is `layers` x the layer time + the head time.  Returns (tok/s, text)."""
    from oracle import decode_oracle as O
    rng = np.random.default_rng(wl["seed"])
    b, h, f = wl["batch"], wl["hidden"], wl["ffn"]
    hq, hkv, d = wl["hq"], wl["hkv"], wl["d"]
    cfg = dict(num_layers=1, hidden=h, ffn=f, num_heads=hq, num_kv_heads=hkv, head_dim=d,
               vocab=wl["vocab"], eps=wl["eps"], qk_norm=wl["qk_norm"])

    def rnd(shape, scale):
        return O.bf16_round(rng.standard_normal(shape, dtype=np.float32) * np.float32(scale))

    w = {"l0.ln1": np.ones(h, np.float32), "l0.ln2": np.ones(h, np.float32),
         "l0.qkv": rnd(((hq + 2 * hkv) * d, h), 0.02), "l0.o": rnd((h, hq * d), 0.02),
         "l0.gate_up": rnd((2 * f, h), 0.02), "l0.down": rnd((h, f), 0.02),
         "l0.qn": np.ones(d, np.float32), "l0.kn": np.ones(d, np.float32),
         "norm": np.ones(h, np.float32), "lm_head": rnd((wl["vocab"], h), 0.02)}
    pages = (lens + BLOCK - 1) // BLOCK
    nb = int(pages.sum())
    bt = np.full((b, int(pages.max())), -1, np.int32)
    o = 0
    for i in range(b):
        bt[i, :pages[i]] = np.arange(o, o + pages[i])
        o += pages[i]
    if kv_layer is None:
        kc = rnd((nb, BLOCK, hkv, d), 0.5)
        vc = rnd((nb, BLOCK, hkv, d), 0.5)
    else:
        kc, vc = kv_layer
    cs = O.bf16_round(O.rope_cos_sin_cache(d, int(lens.max()) + 8, wl["theta"]))
    dec = O.DecoderOracle(cfg, w, cs)
    x = rnd((b, h), 1.0)
    res = rnd((b, h), 1.0)
    slots = np.array([bt[i, (L - 1) // BLOCK] * BLOCK + (L - 1) % BLOCK
                      for i, L in enumerate(lens)])
    t_layer = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        hh, rr = dec.layer(0, x, res, lens - 1, kc, vc, slots, lens.astype(np.int32), bt)
        t1 = time.perf_counter()
        if it >= warmup:
            t_layer.append(t1 - t0)
    t0 = time.perf_counter()
    dec.head(hh, rr)
    t_head = time.perf_counter() - t0
    step_s = wl["layers"] * float(np.mean(t_layer)) + t_head
    text = (f"1 of {wl['layers']} decoder layers at the full batch of {b} "
            f"({int(lens.sum())} cached tokens) timed {steps}x, plus final norm + lm-head + "
            f"argmax once; step time = {wl['layers']} x layer + head "
            f"(layer {np.mean(t_layer):.3f} s, head {t_head:.3f} s)")
    return b / step_s, step_s, text


def use_all_host_threads() -> int:
    """torch.distributed.run starts its workers with OMP_NUM_THREADS=1, which
    would pin the BLAS behind numpy to one core: raise the limit of every thread
    pool in the process to the core count and return the number in effect."""
    want = os.cpu_count() or 1
    try:
        import threadpoolctl
        threadpoolctl.threadpool_limits(limits=want)
        pools = threadpoolctl.threadpool_info()
        got = max([p_.get("num_threads", 1) for p_ in pools] or [1])
    except Exception:
        got = 1
    try:
        import torch
        torch.set_num_threads(want)
    except Exception:
        pass
    return got


def run_reference(args, wl):
    """--impl reference: the CPU port of the reference path, rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    lens = workload_lens(wl)
    cores = use_all_host_threads()
    toks, step_s, text = cpu_sample(wl, lens, steps=max(args.steps, 1), warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": toks, "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl["name"], "global_batch": wl["batch"],
                   "parallelism": "host cores (no GPU)"},
        "cpu_baseline": {"value": toks, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": text},
        "e2e": {"value": toks, "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------ our arm
def attention_bytes(lens, hq, hkv, d, e=2):
    """Algorithmic bytes of one paged decode attention call: K and V of every
    live token once, q in, out, lens, block-table entries."""
    pages = (lens + BLOCK - 1) // BLOCK
    b = len(lens)
    return int(2 * lens.sum() * hkv * d * e + 2 * b * hq * d * e + 4 * b + 4 * pages.sum())


def run_attention_only(args, wl):
    """Config 5: ONE paged decode attention call per step over a skewed batch, with
    the heads sharded over the ranks (query heads and KV heads split, block tables
    and lengths replicated, no collective: every rank owns its Hkv/N slice of
    every page).  value = algorithmic bytes of all ranks per second."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    if wl["hkv"] % world or wl["hq"] % world:
        raise SystemExit(f"{world} ranks do not divide the head counts")
    from fastkernels_b200 import _lib, ops
    b, d = wl["batch"], wl["d"]
    hq, hkv = wl["hq"] // world, wl["hkv"] // world
    lens = workload_lens(wl)
    pages = (lens + BLOCK - 1) // BLOCK
    nb = int(pages.sum())
    rs = np.random.RandomState(wl["seed"] + 1)
    perm = rs.permutation(nb).astype(np.int32)      # blocks scattered over the pool
    bt = np.full((b, int(pages.max())), -1, np.int32)
    o = 0
    for i in range(b):
        bt[i, :pages[i]] = perm[o:o + pages[i]]
        o += pages[i]
    g = torch.Generator(device=dev).manual_seed(wl["seed"] * 31 + rank)
    kc = torch.empty((nb, BLOCK, hkv, d), dtype=torch.bfloat16, device=dev).normal_(0, 0.5, generator=g)
    vc = torch.empty((nb, BLOCK, hkv, d), dtype=torch.bfloat16, device=dev).normal_(0, 0.5, generator=g)
    q_host = (torch.randn((b, hq, d)) * 0.5).to(torch.bfloat16).pin_memory()
    lens_host = torch.from_numpy(lens.astype(np.int32)).pin_memory()
    bt_host = torch.from_numpy(bt).pin_memory()
    out_host = torch.empty((b, hq, d), dtype=torch.bfloat16).pin_memory()
    q = q_host.to(dev)
    lens_d, bt_d = lens_host.to(dev), bt_host.to(dev)
    out = torch.empty_like(q)
    ws = torch.empty(ops.attn_workspace_bytes(b, hq, d, 64), dtype=torch.uint8, device=dev)
    st = ops.new_status(dev)
    scale = d ** -0.5

    def call():
        ops.paged_decode_attn(q, kc, vc, lens_d, bt_d, scale, ws, 64, out=out, status=st)

    def call_e2e():
        q.copy_(q_host, non_blocking=True)
        lens_d.copy_(lens_host, non_blocking=True)
        bt_d.copy_(bt_host, non_blocking=True)
        call()
        out_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    c0 = _lib.lib.fk_launch_count()
    call()
    torch.cuda.synchronize()
    launches = int(_lib.lib.fk_launch_count() - c0)
    sampler = ClockSampler(local)
    for _ in range(args.warmup):
        call()
    if rank == 0:
        sampler.start()
    ms_dev = timed(call, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    for _ in range(args.warmup):
        call_e2e()
    ms_e2e = timed(call_e2e, args.steps)
    status = int(st.item())
    rank_bytes = attention_bytes(lens, hq, hkv, d)
    total_bytes = rank_bytes * world
    if rank != 0:
        sys.stdout.flush()
        if world > 1:
            dist.barrier()
            os._exit(0)
        return
    peaks, peak_kind = measured_peaks()
    per_rank = rank_bytes / (ms_dev / args.steps * 1e-3) / 1e9
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        from oracle import decode_oracle as O
        cores = use_all_host_threads()
        pick = np.argsort(lens)[::16][:16]            # 16 sequences across the length range
        t0 = time.perf_counter()
        sub_bytes = 0
        for i in pick:
            L = int(lens[i])
            idx = torch.as_tensor(bt[i, :pages[i]].astype(np.int64), device=dev)
            O.paged_decode_attention(q[i:i + 1].float().cpu().numpy(),
                                     kc[idx].float().cpu().numpy(), vc[idx].float().cpu().numpy(),
                                     np.array([L], np.int32),
                                     np.arange(pages[i], dtype=np.int32)[None, :], scale)
            sub_bytes += attention_bytes(lens[i:i + 1], hq, hkv, d)
        dt = time.perf_counter() - t0
        cpu = {"value": sub_bytes / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
               "sample": f"the oracle's attention on 16 of the {b} sequences "
                         f"({sub_bytes / 1e6:.0f} MB of K/V, device-to-host copies included)"}
    line = {
        "metric": "paged_attention_hbm_gbs", "value": total_bytes / (ms_dev / args.steps * 1e-3) / 1e9,
        "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": wl["name"], "global_batch": b,
                   "parallelism": f"heads sharded over {world} ranks, no collective",
                   "per_rank_heads": f"{hq} q / {hkv} kv", "kv_tokens": int(lens.sum()),
                   "l2": f"one call streams {rank_bytes / 1e6:.0f} MB per rank: no flush needed",
                   "device_status_word": status},
        "e2e": {"value": total_bytes / (ms_e2e / args.steps * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": int(q_host.numel() * 2 + lens_host.numel() * 4
                                          + bt_host.numel() * 4),
                "d2h_bytes_per_step": int(out_host.numel() * 2),
                "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": launches * args.steps, "clocks": clocks,
        "roofline": {"kernel": "attn_plan_kernel + attn_decode_kernel + attn_merge_kernel, "
                               "one call on one rank", "bound": "hbm", "achieved": per_rank,
                     "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": per_rank / peaks["hbm_gbs"], "peak_source": peak_kind,
                     "traffic": rank_bytes * ATTN_TRAFFIC_RATIO,
                     "algorithmic_bytes": rank_bytes},
        "cpu_baseline": cpu,
    }
    print(json.dumps(line), flush=True)
    sys.stdout.flush()
    if world > 1:
        dist.barrier()
        os._exit(0)


def run_ours(args, wl):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback "
                         "(use --impl reference for the CPU port)")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE {world}", file=sys.stderr)
    tp = world
    if wl["hkv"] % tp or wl["hq"] % tp:
        raise SystemExit(f"tensor parallel degree {tp} does not divide the head counts")

    from fastkernels_b200 import _lib, ops
    from fastkernels_b200.candidate.L4.llama import LlamaConfig
    from fastkernels_b200.engine import DecodeEngine

    lens = workload_lens(wl)
    library_points = world == 1 and not args.no_library_points
    total_steps = 2 * (args.steps + args.warmup) + 8
    if library_points:
        total_steps += 4 * (args.steps + 3)      # the A/B passes of the step
    max_len = int(lens.max()) + total_steps
    # KV pool layout: the benchmark configuration is NHD pages of 256 tokens; the
    # reference's own default on this GPU (HND, 16) can be asked for
    block, layout = args.kv_block, args.kv_layout
    default_pool = block == BLOCK and layout == "NHD"
    max_model_len = ((max_len + block - 1) // block) * block
    nblocks = int(((lens + total_steps + block - 1) // block).sum()) + 1
    layers = args.layers or wl["layers"]
    cfg = LlamaConfig(hidden_size=wl["hidden"], intermediate_size=wl["ffn"],
                      num_hidden_layers=layers, num_attention_heads=wl["hq"],
                      num_key_value_heads=wl["hkv"], head_dim=wl["d"],
                      vocab_size=wl["vocab"], max_position_embeddings=max_model_len,
                      rms_norm_eps=wl["eps"], rope_theta=wl["theta"], qk_norm=wl["qk_norm"],
                      kv_block_size=block, kv_layout=layout, decode_block=args.decode_block)
    eng = DecodeEngine(cfg, max_num_seqs=wl["batch"], max_model_len=max_model_len,
                       num_kv_blocks=nblocks, device=f"cuda:{local}", seed=wl["seed"])
    eng.fill_kv_random(wl["seed"])
    rs = np.random.RandomState(wl["seed"] + 1)
    eng.add_sequences(lens.tolist(), rs.randint(0, wl["vocab"], size=wl["batch"]).tolist())

    # launches of one step (counted on an eager pass before capture)
    bs = wl["batch"]
    n = eng.prepare_decode(use_host_ids=True)
    eng.stage_inputs(n, bs, use_host_ids=True)
    c0 = _lib.lib.fk_launch_count()
    eng.enforce_eager = True
    eng.run_step_device(bs)
    eng.enforce_eager = False
    eng._mark_slot_in_flight()
    torch.cuda.synchronize()
    launches_per_step = int(_lib.lib.fk_launch_count() - c0)
    for s in eng.seqs:
        s.num_tokens += 1
    eng.capture_cudagraph([bs])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(sync: bool, steps: int) -> float:
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            eng.step(sync=sync)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=f"cuda:{local}")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    sampler = ClockSampler(local)
    for _ in range(args.warmup):
        eng.step(sync=False)
    if rank == 0:
        sampler.start()
    ms_dev = timed(False, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    for _ in range(args.warmup):
        eng.step(sync=True)
    h0, d0 = eng.h2d_bytes, eng.d2h_bytes
    ms_e2e = timed(True, args.steps)
    h2d = (eng.h2d_bytes - h0) / args.steps
    d2h = (eng.d2h_bytes - d0) / args.steps
    status = eng.device_status()

    # roofline of the dominant kernel: layer-0 attention on the live workload
    cur = np.array([s.num_tokens - 1 for s in eng.seqs], dtype=np.int64)  # last step
    att = eng.model.model.layers[0].self_attn.attn
    gv = eng.graph_vars
    hq_l, hkv_l = wl["hq"] // tp, wl["hkv"] // tp
    q = torch.randn((bs, hq_l, wl["d"]), device=f"cuda:{local}").to(torch.bfloat16)
    out = torch.empty_like(q)
    op = att.decode_op
    # as inside the step: the split schedule is planned once, layers call the
    # planned entry point (main kernel + merge kernel)
    ops.paged_decode_attn_plan(gv["context_lens"][:bs], gv["block_tables"][:bs], block,
                               hq_l, hkv_l, wl["d"], eng.attn_workspace, op._max_splits,
                               status=op._status)
    # `reps` launches back to back between two events on the launching stream (one
    # layer's K/V is > 1 GB, so nothing survives in L2 from one launch to the next)
    def attn_once():
        ops.paged_decode_attn(q, att.k_cache, att.v_cache, gv["context_lens"][:bs],
                              gv["block_tables"][:bs], wl["d"] ** -0.5, eng.attn_workspace,
                              op._max_splits, out=out, status=op._status, planned=True,
                              kv_layout=cfg.kv_layout)

    reps = 20
    for _ in range(3):
        attn_once()
    torch.cuda.synchronize()
    a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        attn_once()
    b_.record()
    torch.cuda.synchronize()
    att_ms = a.elapsed_time(b_) / reps
    att_bytes = attention_bytes(cur, hq_l, hkv_l, wl["d"])
    peaks, peak_kind = measured_peaks()
    achieved = att_bytes / (att_ms * 1e-3) / 1e9
    roofline = {"kernel": "attn_decode_kernel (+ merge kernel; split plan shared per step), one layer of this workload",
                "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peak_kind,
                "traffic": (att_bytes * ATTN_TRAFFIC_RATIO if ATTN_TRAFFIC_RATIO else None),
                "algorithmic_bytes": att_bytes, "ms_per_launch": att_ms}
    # for context only (the fraction above stays on the measured copy peak): what this
    # GPU gives a kernel that only reads, measured now with the library's read stream
    # over up to 8 GiB of the live K pools (far larger than L2)
    try:
        pool = eng.kv_cache[0].reshape(-1)               # the K pools of all layers
        nb = min(pool.numel() * 2, 8 << 30) // 16 * 16
        flat = pool.view(torch.uint8)[:nb]
        if nb >= (1 << 30):
            acc = torch.zeros(1, dtype=torch.int32, device=f"cuda:{local}")
            for _ in range(2):
                ops.xor_u32(flat, acc)
            a.record()
            for _ in range(5):
                ops.xor_u32(flat, acc)
            b_.record()
            torch.cuda.synchronize()
            roofline["read_stream_gbs"] = nb * 5 / (a.elapsed_time(b_) * 1e-3) / 1e9
    except Exception as e:          # informational: never fails the bench line
        roofline["read_stream_gbs"] = f"unavailable: {e}"

    # the fused all-reduce + add + RMSNorm alone, at the step's payload, both exchanges
    # (every rank issues the same calls; max over ranks)
    allreduce = None
    if eng.comm is not None:
        comm = eng.comm
        res = torch.zeros((bs, wl["hidden"]), dtype=torch.bfloat16, device=f"cuda:{local}")
        wn = torch.ones(wl["hidden"], dtype=torch.bfloat16, device=f"cuda:{local}")
        o_ = torch.empty_like(res)
        allreduce = {"payload_bytes": bs * wl["hidden"] * 2,
                     "selected": "push" if comm.pushed(bs) else
                                 "two_stage" if comm.two_stage(bs) else "one_stage"}
        keep = comm.algo
        for algo in ("one_stage", "two_stage"):
            comm.algo = algo
            for i in range(6):
                comm.allreduce_add_rmsnorm(i & 1, bs, res, wn, wl["eps"], out=o_)
            barrier()
            if int(comm.status.item()) != 0:      # a wait ran out: do not time 100 more
                allreduce[algo + "_us_per_call"] = "device status %d" % int(comm.status.item())
                continue
            # 50 calls in one CUDA graph: device time, not the host's launch rate
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(50):
                    comm.allreduce_add_rmsnorm(i & 1, bs, res, wn, wl["eps"], out=o_)
            g.replay()
            barrier()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            g.replay()
            t1.record()
            barrier()
            us = torch.tensor([t0.elapsed_time(t1) * 1e3 / 50], device=f"cuda:{local}")
            dist.all_reduce(us, op=dist.ReduceOp.MAX)
            allreduce[algo + "_us_per_call"] = float(us.item())
        # the pair the layer runs: row-parallel output projection + all-reduce + add +
        # norm, with the exchange pulled by the norm kernel or pushed by the projection
        kdim = wl["hq"] * wl["d"] // tp
        xo = (torch.randn((bs, kdim), device=f"cuda:{local}") * 0.1).to(torch.bfloat16)
        wo = (torch.randn((wl["hidden"], kdim), device=f"cuda:{local}") * 0.02).to(torch.bfloat16)
        for algo in ("one_stage", "push"):
            comm.algo = algo

            def pair(i):
                if algo == "push":
                    comm.gemm_push(xo, wo, None, i & 1)
                else:
                    ops.gemm_bf16(xo, wo, out=comm.slot_view(i & 1, bs, wl["hidden"]))
                comm.allreduce_add_rmsnorm(i & 1, bs, res, wn, wl["eps"], out=o_)
            for i in range(6):
                pair(i)
            barrier()
            if int(comm.status.item()) != 0:
                allreduce["o_proj_plus_" + algo + "_us"] = \
                    "device status %d" % int(comm.status.item())
                continue
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(50):
                    pair(i)
            g.replay()
            barrier()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            g.replay()
            t1.record()
            barrier()
            us = torch.tensor([t0.elapsed_time(t1) * 1e3 / 50], device=f"cuda:{local}")
            dist.all_reduce(us, op=dist.ReduceOp.MAX)
            allreduce["o_proj_plus_" + algo + "_us"] = float(us.item())
        comm.algo = keep
        status |= int(comm.status.item())

    def finish():
        """Leave without tearing NCCL down: communicators captured in CUDA graphs
        make destroy_process_group block, so every rank meets at a last barrier
        and exits."""
        sys.stdout.flush()
        sys.stderr.flush()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
            os._exit(0)

    if rank != 0:
        finish()
        return

    # CPU baseline on rank 0: the oracle on layer 0's live K/V
    cpu = None
    if not args.no_cpu_baseline and tp == 1 and default_pool:
        pages = (cur + BLOCK - 1) // BLOCK
        kparts, vparts = [], []
        for s in eng.seqs:
            idx = torch.tensor(s.block_table, device=f"cuda:{local}")
            kparts.append(att.k_cache[idx].float().cpu().numpy())
            vparts.append(att.v_cache[idx].float().cpu().numpy())
        kv = (np.concatenate(kparts), np.concatenate(vparts))
        cores = use_all_host_threads()
        toks, _, text = cpu_sample(wl, cur, kv_layer=kv, steps=1, warmup=0)
        cpu = {"value": toks, "unit": UNIT, "cores": cores, "kind": "port", "sample": text}
        del kv, kparts, vparts
    elif tp > 1:
        cpu = None

    b = wl["batch"]
    line = {
        "metric": METRIC, "value": b * args.steps / (ms_dev * 1e-3), "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": wl["name"] if default_pool else
                   wl["name"].replace("block 256", f"{layout} pages of {block}"),
                   "global_batch": b, "layers": layers,
                   "parallelism": f"tp{tp}", "cuda_graphs": True,
                   "layer_kernels": "persistent decode block" if args.decode_block and tp == 1
                   else "one kernel per op",
                   "l2": "inputs (weights + live KV) exceed L2 by >100x; no flush needed",
                   "device_status_word": status},
        "e2e": {"value": b * args.steps / (ms_e2e * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
    }
    if allreduce is not None:
        line["allreduce_add_rmsnorm"] = allreduce
    if args.layers and args.layers != wl["layers"]:
        line["config"]["note"] = "REDUCED layer count: debug run, not a valid measurement"
    if library_points and default_pool:
        from fastkernels_b200 import library_points as lp
        line["library_points"] = lp.collect(eng, wl, args.steps)
    print(json.dumps(line), flush=True)
    finish()


# DRAM bytes (read + write) per launch / algorithmic bytes for attn_decode_kernel:
# 294.6 MB / 287.0 MB in an ncu capture of a 287 MB case.  The bench's layer is
# too large to capture with --set full; traffic grows in proportion to the cached
# tokens, so the ratio is applied to the live workload's algorithmic bytes.
ATTN_TRAFFIC_RATIO = 1.027


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-library-points", action="store_true",
                    help="skip the library reference points (1 GPU only)")
    ap.add_argument("--kv-block", type=int, default=BLOCK,
                    help="tokens per KV page (default: the benchmark's 256)")
    ap.add_argument("--kv-layout", default="NHD", choices=["NHD", "HND"])
    ap.add_argument("--decode-block", action="store_true",
                    help="run the kernels between two attention calls as one persistent "
                         "launch (fk_decode_block; 1 GPU)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        if wl.get("attention_only"):
            raise SystemExit("--impl reference times the decode-step workloads (c3, c4)")
        run_reference(args, wl)
    elif wl.get("attention_only"):
        run_attention_only(args, wl)
    else:
        run_ours(args, wl)


if __name__ == "__main__":
    main()
