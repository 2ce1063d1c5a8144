"""Tensor-parallel host logic on CPU: two gloo ranks shard full weights through
the candidates' weight loaders and must reproduce the unsharded result.  The GPU
GEMM is replaced by torch's CPU matmul here (test only): what is checked is the
sharding arithmetic, the all-reduce placement and the greedy (max, index) gather."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import fastkernels_b200.candidate.L2.parallel_linear as pl
        import fastkernels_b200.candidate.L1.linear as l1
        from fastkernels_b200.candidate.L2.parallel_embedding import (ParallelLMHead,
                                                                       VocabParallelEmbedding)
        from fastkernels_b200.candidate.L4.llama import LlamaConfig
        from fastkernels_b200.engine import DecodeEngine
        from fastkernels_b200.infra.tp import _tp_rank, _tp_size

        cpu_linear = lambda x, w, b: torch.nn.functional.linear(x, w, b)
        pl._linear = cpu_linear
        l1.Matmul.forward = lambda self, i, w, b=None: cpu_linear(i, w, b)
        assert _tp_size() == world and _tp_rank() == rank

        g = torch.Generator().manual_seed(0)
        hidden, d, hq, hkv, ffn, vocab, t = 64, 16, 8, 4, 96, 40, 5
        x = torch.randn(t, hidden, generator=g)
        wq = torch.randn(hq * d, hidden, generator=g)
        wk = torch.randn(hkv * d, hidden, generator=g)
        wv = torch.randn(hkv * d, hidden, generator=g)
        wgu = torch.randn(2 * ffn, hidden, generator=g)
        wdown = torch.randn(hidden, ffn, generator=g)
        emb = torch.randn(vocab, hidden, generator=g)

        def gather(y):
            out = [torch.empty_like(y) for _ in range(world)]
            dist.all_gather(out, y.contiguous())
            return out

        # QKV: per-rank [q_r | k_r | v_r]; concatenating the per-rank q blocks gives q
        qkv = pl.QKVParallelLinear(hidden, d, hq, hkv)
        for sid, w in (("q", wq), ("k", wk), ("v", wv)):
            qkv.weight.weight_loader(qkv.weight, w, sid)
        parts = gather(qkv(x))
        qs, ks = hq * d // world, hkv * d // world
        q = torch.cat([p[:, :qs] for p in parts], 1)
        k = torch.cat([p[:, qs:qs + ks] for p in parts], 1)
        v = torch.cat([p[:, qs + ks:] for p in parts], 1)
        torch.testing.assert_close(q, x @ wq.T)
        torch.testing.assert_close(k, x @ wk.T)
        torch.testing.assert_close(v, x @ wv.T)

        # merged gate/up (each block sharded independently) -> row-parallel down + all-reduce
        gu = pl.MergedColumnParallelLinear(hidden, [ffn, ffn])
        gu.weight.weight_loader(gu.weight, wgu)
        down = pl.RowParallelLinear(ffn, hidden)
        down.weight.weight_loader(down.weight, wdown)
        y = gu(x)
        f = ffn // world
        act = torch.nn.functional.silu(y[:, :f]) * y[:, f:]
        out = down(act)                                   # all-reduced inside
        full = x @ wgu.T
        ref = (torch.nn.functional.silu(full[:, :ffn]) * full[:, ffn:]) @ wdown.T
        torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-4)

        # vocab-parallel embedding and greedy gather
        e = VocabParallelEmbedding(vocab, hidden)
        w = e.embedding_op.emb.weight
        w.weight_loader(w, emb)
        ids = torch.tensor([0, 19, 20, 39, 7])
        with torch.no_grad():
            torch.testing.assert_close(e(ids), emb[ids])
            head = ParallelLMHead(vocab, hidden)
            hw = head.embedding_op.emb.weight
            hw.weight_loader(hw, emb)
            logits = head.project(x)
            vals, idxs = logits.max(dim=-1)
            tok = head.greedy_pairs(vals, idxs)
        assert torch.equal(tok, (x @ emb.T).argmax(-1))

        # engine: the KV pool holds Hkv / tp heads per rank
        cfg = LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=1,
                          num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                          vocab_size=64, max_position_embeddings=256, kv_block_size=64)
        eng = DecodeEngine(cfg, max_num_seqs=2, max_model_len=128, num_kv_blocks=4, device="cpu")
        assert tuple(eng.kv_cache.shape) == (2, 1, 4, 64, 1, 128)
        assert eng.model.model.layers[0].self_attn.num_heads == 2
        assert eng.graph_vars["lm_logits"].shape[1] == 32
        ret[rank] = "ok"
    except Exception as ex:  # surfaced by the parent
        import traceback
        ret[rank] = traceback.format_exc()
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_two_rank_sharding_matches_unsharded():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert dict(ret) == {0: "ok", 1: "ok"}, "\n".join(str(v) for v in ret.values())
