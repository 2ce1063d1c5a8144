"""Worker for the multi-GPU tensor-parallel test (spawned once per rank; 2, 4 or 8
ranks)."""
import os
import sys
import traceback

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
for p in (os.path.dirname(HERE), HERE):
    if p not in sys.path:
        sys.path.insert(0, p)


def run_engine(cfg_d, w, lens, rank, world, steps, seed, graph):
    import cases
    from fastkernels_b200.candidate.L4.llama import LlamaConfig
    from fastkernels_b200.engine import DecodeEngine
    block = 64
    cfg = LlamaConfig(hidden_size=cfg_d["hidden"], intermediate_size=cfg_d["ffn"],
                      num_hidden_layers=cfg_d["num_layers"],
                      num_attention_heads=cfg_d["num_heads"],
                      num_key_value_heads=cfg_d["num_kv_heads"], head_dim=cfg_d["head_dim"],
                      vocab_size=cfg_d["vocab"], max_position_embeddings=cfg_d["max_pos"],
                      rms_norm_eps=cfg_d["eps"], rope_theta=cfg_d["theta"],
                      qk_norm=cfg_d["qk_norm"], kv_block_size=block)
    nb = sum((L + 40 + block - 1) // block for L in lens) + 2
    eng = DecodeEngine(cfg, max_num_seqs=len(lens), max_model_len=max(lens) + 64,
                       num_kv_blocks=nb, device=f"cuda:{rank}", enforce_eager=not graph)
    eng.load_full_weights(w)
    rs = np.random.RandomState(seed)
    first = rs.randint(0, cfg.vocab_size, size=len(lens))
    eng.add_sequences(lens, first)
    hkv = cfg.num_key_value_heads
    hl = hkv // world
    shape = (nb, block, hkv, cfg.head_dim)
    kcs, vcs = [], []
    for li in range(cfg.num_hidden_layers):
        k = cases.randn_bf16(rs, shape, 0.5)
        v = cases.randn_bf16(rs, shape, 0.5)
        eng.kv_cache[0, li].copy_(torch.from_numpy(k[:, :, rank * hl:(rank + 1) * hl]))
        eng.kv_cache[1, li].copy_(torch.from_numpy(v[:, :, rank * hl:(rank + 1) * hl]))
        kcs.append(k)
        vcs.append(v)
    if graph:
        eng.capture_cudagraph([len(lens)])
    toks, logits, sched = [], [], []
    for _ in range(steps):
        lens_now = [s.num_tokens for s in eng.seqs]
        t = eng.step(sync=True)
        toks.append(t.copy())
        # all ranks hold a vocab shard of the logits
        logits.append(eng.graph_vars["lm_logits"][:len(lens)].float().cpu().numpy())
        sched.append((lens_now, [list(s.block_table) for s in eng.seqs]))
    status = int(eng.status.item()) | (int(eng.comm.status.item()) if eng.comm else 0)
    return eng, first, kcs, vcs, np.stack(toks), logits, sched, status


def worker(rank, world, port, ret):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world,
                                device_id=torch.device("cuda", rank))
        import cases
        from oracle import decode_oracle as O
        # 4 q / 2 kv heads shard over two ranks; more ranks take the 16 / 8 model
        cfg_d = cases.TINY_QWEN3 if world == 2 else cases.TINY_TP8
        # The oracle is the unsharded model.  Every rank rounds its partial
        # projection to bf16 before the exchange (as the reference's ranks do), so
        # the more ranks, the further a logit may sit from the oracle's: a token
        # counts as a near tie within 2 bf16 steps of the oracle's maximum on two
        # ranks, within 4 on more.  The exact check is the one against the NCCL path.
        near_ulps = 2 if world == 2 else 4
        w = cases.decoder_weights(5, cfg_d, scale=0.05)
        lens = [1, 30, 64, 65, 127, 200]
        steps = 16
        out = {}
        # The automatic rule gives this small model the pushed exchange (the projection
        # stores into every rank's receive area); "one_stage" forces the pull by the norm
        # kernel, "two_stage" the owner-reduces-and-pushes exchange, which the rule only
        # picks for payloads far larger than this model's
        for mode in ("fused_eager", "fused_graph", "fused_one_stage_graph",
                     "fused_two_stage_graph", "nccl_eager"):
            os.environ["FK_B200_NCCL_ALLREDUCE"] = "1" if mode.startswith("nccl") else "0"
            os.environ["FK_B200_ALLREDUCE_ALGO"] = \
                "two_stage" if "two_stage" in mode else \
                "one_stage" if "one_stage" in mode else "auto"
            from fastkernels_b200 import comm as comm_mod
            comm_mod.set_tp_comm(None)
            res = run_engine(cfg_d, w, lens, rank, world, steps, 17, mode.endswith("graph"))
            out[mode] = res
            dist.barrier()
        msgs = []
        for mode, res in out.items():
            if res[7] != 0:
                msgs.append(f"{mode}: device status {res[7]}")
        # prefill through the tensor-parallel engine (chunks of the communicator's row
        # capacity over the pages; the fused all-reduce serves [chunk, hidden] partials)
        rs = np.random.RandomState(29)
        plens = [3, 70, 300]
        prompts = [rs.randint(0, cfg_d["vocab"], size=n).tolist() for n in plens]
        first_tokens = {}
        os.environ["FK_B200_ALLREDUCE_ALGO"] = "auto"
        for mode in ("fused_eager", "nccl_eager"):
            os.environ["FK_B200_NCCL_ALLREDUCE"] = "1" if mode.startswith("nccl") else "0"
            comm_mod.set_tp_comm(None)
            eng = out[mode][0].__class__(out[mode][0].config, max_num_seqs=len(plens),
                                         max_model_len=max(plens) + 64, num_kv_blocks=12,
                                         device=f"cuda:{rank}", enforce_eager=True)
            eng.load_full_weights(w)
            first_tokens[mode] = eng.prefill(prompts)
            st = int(eng.status.item()) | (int(eng.comm.status.item()) if eng.comm else 0)
            if st != 0:
                msgs.append(f"prefill {mode}: device status {st}")
            dist.barrier()
        if world == 2 and not np.array_equal(first_tokens["fused_eager"],
                                             first_tokens["nccl_eager"]):
            msgs.append("prefill: fused and NCCL all-reduce paths sample different tokens")
        if rank == 0:
            cs = O.bf16_round(eng.model.model.rotary_emb.cos_sin_cache.cpu().numpy())
            dec = O.DecoderOracle(cfg_d, w, cs)
            shape = (12, 64, cfg_d["num_kv_heads"], cfg_d["head_dim"])
            kz = [np.zeros(shape, np.float32) for _ in range(cfg_d["num_layers"])]
            vz = [np.zeros(shape, np.float32) for _ in range(cfg_d["num_layers"])]
            cu = np.concatenate([[0], np.cumsum(plens)]).astype(np.int32)
            slots = np.concatenate([[s.block_table[t // 64] * 64 + t % 64 for t in range(n)]
                                    for s, n in zip(eng.seqs, plens)])
            lg, want = dec.prefill(np.concatenate(prompts),
                                   np.concatenate([np.arange(n) for n in plens]), cu, kz, vz,
                                   slots)
            for i, (g, wv) in enumerate(zip(first_tokens["fused_eager"], want)):
                if g != wv:
                    gap = float(lg[i, wv] - lg[i, g])
                    ulp = 2.0 ** (np.floor(np.log2(max(abs(float(lg[i, wv])), 1e-30))) - 7)
                    if gap > near_ulps * ulp:
                        msgs.append(f"prefill seq {i}: token {g} vs oracle {wv}")
        ref_toks = out["nccl_eager"][4]
        for mode in ("fused_eager", "fused_graph", "fused_one_stage_graph",
                     "fused_two_stage_graph"):
            # the fused runs take the same sums in the same order
            if not np.array_equal(out[mode][4], out["fused_eager"][4]):
                msgs.append(f"{mode}: tokens differ from the eager fused run")
            if world == 2:
                # a sum of two terms has one order: the NCCL path gives the same bits
                if not np.array_equal(out[mode][4], ref_toks):
                    msgs.append(f"{mode}: tokens differ from the NCCL all-reduce path")
                for a, b in zip(out[mode][5], out["nccl_eager"][5]):
                    if not np.allclose(a, b, atol=2e-2, rtol=2e-2):
                        msgs.append(f"{mode}: logits differ from the NCCL path")
                        break
            else:
                # NCCL adds 4 or 8 bf16 terms in its own order with its own rounding,
                # the fused kernel in rank order in fp32: same inputs (first step),
                # logits within tolerance; later steps may follow different tokens
                a, b = out[mode][5][0], out["nccl_eager"][5][0]
                # (measured on 4 ranks: 96 % of the logits inside 2e-2, none further
                # than 0.07 apart: NCCL rounds its partial sums to bf16 on the way)
                inside = np.abs(a - b) <= 2e-2 + 2e-2 * np.abs(b)
                if inside.mean() < 0.90 or np.abs(a - b).max() > 0.125:
                    msgs.append(f"{mode}: first-step logits differ from the NCCL path "
                                f"({inside.mean():.4f} inside, max {np.abs(a - b).max():.3f})")
        if rank == 0:
            # teacher-forced oracle over the fused run's own tokens and schedule
            eng, first, kcs, vcs, toks, logits, sched, _ = out["fused_graph"]
            cs = O.bf16_round(eng.model.model.rotary_emb.cos_sin_cache.cpu().numpy())
            dec = O.DecoderOracle(cfg_d, w, cs)
            ids = np.array(first)
            bs = 64
            equal = near = 0
            for step in range(steps):
                lens_now, tables = sched[step]
                lens_a = np.array(lens_now)
                cols = max(len(t) for t in tables)
                bt = np.full((len(lens_a), cols), -1, np.int32)
                for i, t in enumerate(tables):
                    bt[i, :len(t)] = t
                slots = np.array([tables[i][(L - 1) // bs] * bs + (L - 1) % bs
                                  for i, L in enumerate(lens_a)])
                lg, want = dec.step(ids, lens_a - 1, kcs, vcs, slots, lens_a.astype(np.int32), bt)
                for i in range(len(lens_a)):
                    if toks[step][i] == want[i]:
                        equal += 1
                    else:
                        gap = float(lg[i, want[i]] - lg[i, toks[step][i]])
                        ulp = 2.0 ** (np.floor(np.log2(max(abs(float(lg[i, want[i]])), 1e-30))) - 7)
                        if gap <= near_ulps * ulp:
                            near += 1
                        else:
                            msgs.append(f"step {step} seq {i}: token {toks[step][i]} vs oracle {want[i]}")
                ids = toks[step].copy()
            # each rank rounds its partial sums to bf16 before the exchange, so TP
            # sees a few more bf16 near-ties than one GPU does; every mismatch
            # was verified above to be within 2 bf16 steps of the oracle's maximum
            if equal < 0.90 * steps * len(lens):
                msgs.append(f"only {equal} of {steps * len(lens)} tokens equal the oracle ({near} near ties)")
        ret[rank] = "ok" if not msgs else "\n".join(msgs)
    except Exception:
        ret[rank] = traceback.format_exc()
    finally:
        try:
            dist.barrier()
        except Exception:
            pass
        sys.stdout.flush()
        os._exit(0)
