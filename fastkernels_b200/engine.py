"""Decode-step engine: paged KV pool, block manager, CUDA-graph decode, greedy
sampling, tensor parallelism (one process per GPU, NCCL).

Mirror of the decode path of the reference engine (fastkernels/infra/engine.py):
  BlockManager.maybe_append_pages            engine.py:530-537
  ModelRunner.allocate_kv_cache              engine.py:1783-1793  (pool layout)
  ModelRunner._prepare_decode_arrays         engine.py:5767-5838  (positions / slots / lens)
  ModelRunner._run_graph_from_numpy          engine.py:5386-5427  (H2D staging + replay)
  ModelRunner.capture_cudagraph              engine.py:6701-7025  (graph body, graph_vars)
  ModelRunner._greedy_from_hidden            engine.py:5711-5746  (argmax, tp all-gather)
plus the prefill side of ModelRunner.run (engine.py:4902-4990, 6048-6063): whole
or chunked prompts fill their KV pages and join the running batch.  Scheduling
of mixed prefill + decode batches, HTTP serving and checkpoint loading are
outside this build; sequences may also enter with their context already in the
cache (synthetic contexts for the benchmark, or whatever the caller wrote).

Every rank of a tensor-parallel group runs this same host code on the same
inputs (deterministic scheduling), so no control-plane exchange is needed; the
data-path exchanges are the NCCL all-reduces after o_proj / down_proj / the
vocab-parallel embedding and the (max, index) all-gather of greedy sampling,
all captured in the CUDA graph.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field

import numpy as np
import torch

from . import ops
from .candidate.L4.llama import LlamaConfig, LlamaForCausalLM
from .infra.context import get_context, reset_context, set_context
from .infra.tp import _tp_rank, _tp_size

# FK_B200_PREPARE_AHEAD=0: stage every step's host arrays only when the step is
# called (for A/B timing of the look-ahead in DecodeEngine.step)
_NO_PREPARE_AHEAD = os.environ.get("FK_B200_PREPARE_AHEAD", "1") == "0"


@dataclass
class Sequence:
    """One running request: `num_tokens` counts the tokens whose K/V are (or, for
    the newest one, are about to be) in the cache; `block_table` lists its pages."""
    seq_id: int
    num_tokens: int
    block_table: list[int] = field(default_factory=list)
    last_token: int = 0
    output: list[int] = field(default_factory=list)


def pack_prefill_chunk(prompt_lens, done, budget):
    """Next prefill forward: walk the sequences in order and take as many of each
    one's remaining prompt tokens as the token budget allows (None = no limit).
    Returns [(sequence index, first token, count)]; every sequence appears at most
    once, so a forward holds at most one chunk per sequence."""
    left = budget if budget is not None else 1 << 62
    part = []
    for i, n in enumerate(prompt_lens):
        take = min(n - done[i], left)
        if take > 0:
            part.append((i, done[i], take))
            left -= take
        if left == 0:
            break
    return part


class BlockManager:
    """Free-list page allocator (decode subset of engine.py:380-586)."""

    def __init__(self, num_blocks: int, block_size: int):
        self.block_size = block_size
        self.free = list(range(num_blocks - 1, -1, -1))

    def allocate(self, seq: Sequence) -> None:
        need = (seq.num_tokens + self.block_size - 1) // self.block_size
        while len(seq.block_table) < need:
            seq.block_table.append(self._pop())

    def maybe_append_page(self, seq: Sequence) -> bool:
        """Called with num_tokens INCLUDING the token sampled last step: a new
        page is needed when that token is the first of a page (engine.py:530-533)."""
        if seq.num_tokens % self.block_size == 1 and \
                len(seq.block_table) * self.block_size < seq.num_tokens:
            seq.block_table.append(self._pop())
            return True
        return False

    def _pop(self) -> int:
        if not self.free:
            raise RuntimeError("KV pool exhausted")
        return self.free.pop()

    def release(self, seq: Sequence) -> None:
        self.free.extend(reversed(seq.block_table))
        seq.block_table.clear()


class DecodeEngine:
    def __init__(self, config: LlamaConfig, *, max_num_seqs: int, max_model_len: int,
                 num_kv_blocks: int, device="cuda", seed: int = 0,
                 enforce_eager: bool = False, init_scale: float = 0.02,
                 attn_max_splits: int | None = None):
        self.config = config
        self.device = torch.device(device)
        self.tp, self.rank = _tp_size(), _tp_rank()
        self.block_size = config.kv_block_size
        self.max_num_seqs = max_num_seqs
        self.max_model_len = max_model_len
        self.max_num_blocks = (max_model_len + self.block_size - 1) // self.block_size
        self.enforce_eager = enforce_eager
        self.h2d_bytes = 0
        self.d2h_bytes = 0

        prev = torch.get_default_dtype()
        torch.set_default_dtype(config.dtype)
        try:
            with torch.device(self.device):
                self.model = LlamaForCausalLM(config)
        finally:
            torch.set_default_dtype(prev)
        self.init_random_weights(seed, init_scale)
        if attn_max_splits is None:
            attn_max_splits = ops.max_splits_for(max_model_len)
        for layer in self.model.model.layers:
            layer.self_attn.attn.decode_op._max_splits = attn_max_splits

        # tensor parallel: fused all-reduce + add + RMSNorm over peer memory unless
        # FK_B200_NCCL_ALLREDUCE=1 asks for the plain NCCL path
        self.comm = None
        if self.tp > 1 and self.device.type == "cuda" and \
                os.environ.get("FK_B200_NCCL_ALLREDUCE", "0") != "1":
            from .comm import TpComm, set_tp_comm
            # rows: one prefill chunk (512, the most a fused call takes); a decode
            # batch has to fit the same limit
            if max_num_seqs > 512:
                raise ValueError("tensor-parallel decode batches are limited to 512 sequences "
                                 "by the fused all-reduce (set FK_B200_NCCL_ALLREDUCE=1 for more)")
            self.comm = TpComm(512, config.hidden_size, self.device)
            algo = os.environ.get("FK_B200_ALLREDUCE_ALGO", "auto")
            if algo not in ("auto", "one_stage", "two_stage", "push"):
                raise ValueError("FK_B200_ALLREDUCE_ALGO must be auto, one_stage, two_stage "
                                 "or push")
            self.comm.algo = algo
            set_tp_comm(self.comm)
        self.allocate_kv_cache(num_kv_blocks)
        self.blocks = BlockManager(num_kv_blocks, self.block_size)
        self.seqs: list[Sequence] = []
        self._init_buffers()
        self.graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self.graph_pool = None
        self._bt_dirty = True

    # ------------------------------------------------------------------ weights
    @torch.no_grad()
    def init_random_weights(self, seed: int, scale: float) -> None:
        """Random-init every parameter (randn * scale; norm weights 1.0).  Shards
        are drawn per rank: statistically the same model at every tp degree."""
        g = torch.Generator(device=self.device).manual_seed(seed * 1000003 + self.rank)
        for name, p in self.model.named_parameters():
            if "norm" in name or "layernorm" in name:
                p.fill_(1.0)
            else:
                p.normal_(0.0, scale, generator=g)

    @torch.no_grad()
    def load_full_weights(self, w: dict) -> None:
        """Load UNSHARDED weights (dict of tensors in the layout of
        tests/cases.py:decoder_weights) through each parameter's weight_loader,
        which takes this rank's shard exactly as the reference loaders do."""
        m, c = self.model, self.config
        dev = self.device

        def t(a):
            return torch.as_tensor(a).to(device=dev, dtype=c.dtype)

        emb = m.model.embed_tokens.embedding_op.emb.weight
        emb.weight_loader(emb, t(w["embed"]))
        lm = m.lm_head.embedding_op.emb.weight
        lm.weight_loader(lm, t(w["lm_head"]))
        m.model.norm.weight.copy_(t(w["norm"]))
        hq, hkv, d = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        for li, layer in enumerate(m.model.layers):
            p = f"l{li}."
            layer.input_layernorm.weight.copy_(t(w[p + "ln1"]))
            layer.post_attention_layernorm.weight.copy_(t(w[p + "ln2"]))
            qkv = t(w[p + "qkv"])
            qp = layer.self_attn.qkv_proj.weight
            qp.weight_loader(qp, qkv[:hq * d], "q")
            qp.weight_loader(qp, qkv[hq * d:(hq + hkv) * d], "k")
            qp.weight_loader(qp, qkv[(hq + hkv) * d:], "v")
            op = layer.self_attn.o_proj.weight
            op.weight_loader(op, t(w[p + "o"]))
            gu = layer.mlp.gate_up_proj.weight
            gu.weight_loader(gu, t(w[p + "gate_up"]))
            dn = layer.mlp.down_proj.weight
            dn.weight_loader(dn, t(w[p + "down"]))
            if c.qk_norm:
                layer.self_attn.q_norm.weight.copy_(t(w[p + "qn"]))
                layer.self_attn.k_norm.weight.copy_(t(w[p + "kn"]))

    # ----------------------------------------------------------------- KV cache
    def allocate_kv_cache(self, num_blocks: int) -> None:
        """Pool [2, layers, num_blocks, BLOCK, Hkv/tp, D] (NHD) or
        [2, layers, num_blocks, Hkv/tp, BLOCK, D] (HND); every attention layer gets
        its K and V views (engine.py:1783-1793)."""
        c = self.config
        hkv = max(c.num_key_value_heads // self.tp, 1)
        self.num_kv_blocks = num_blocks
        shape = (num_blocks, hkv, self.block_size, c.head_dim) if c.kv_layout == "HND" \
            else (num_blocks, self.block_size, hkv, c.head_dim)
        self.kv_cache = torch.zeros((2, c.num_hidden_layers, *shape), dtype=c.dtype,
                                    device=self.device)
        for li, layer in enumerate(self.model.model.layers):
            layer.self_attn.attn.k_cache = self.kv_cache[0, li]
            layer.self_attn.attn.v_cache = self.kv_cache[1, li]

    @torch.no_grad()
    def fill_kv_random(self, seed: int, scale: float = 0.5) -> None:
        """Synthetic contexts: fill the whole pool with randn * scale."""
        g = torch.Generator(device=self.device).manual_seed(seed * 7919 + self.rank)
        for li in range(self.config.num_hidden_layers):
            self.kv_cache[:, li].normal_(0.0, scale, generator=g)

    # ------------------------------------------------------------------ buffers
    def _init_buffers(self) -> None:
        n, dev, c = self.max_num_seqs, self.device, self.config
        vocab_local = c.vocab_size // self.tp
        # The per-step inputs live in ONE buffer, [input_ids i64 | positions i64 |
        # slot_mapping i32 | context_lens i32], so that a step stages them with a
        # single host-to-device copy (all four, or the last three when the token ids
        # stay on the device).
        def packed_views(buf):
            return dict(input_ids=buf[:8 * n].view(torch.int64),
                        positions=buf[8 * n:16 * n].view(torch.int64),
                        slot_mapping=buf[16 * n:20 * n].view(torch.int32),
                        context_lens=buf[20 * n:24 * n].view(torch.int32))

        self._packed_dev = torch.zeros(24 * n, dtype=torch.uint8, device=dev)
        self._packed_dev[16 * n:20 * n].view(torch.int32).fill_(-1)   # slot_mapping: no slot
        self.graph_vars = dict(
            **packed_views(self._packed_dev),
            block_tables=torch.full((n, self.max_num_blocks), -1, dtype=torch.int32,
                                    device=dev),
            outputs=torch.zeros((n, c.hidden_size), dtype=c.dtype, device=dev),
            lm_logits=torch.zeros((n, vocab_local), dtype=c.dtype, device=dev),
            lm_max_vals=torch.zeros(n, dtype=torch.float32, device=dev),
            lm_max_idxs=torch.zeros(n, dtype=torch.int64, device=dev),
            token_ids=torch.zeros(n, dtype=torch.int64, device=dev),
        )

        def pinned(shape, dtype):
            return torch.zeros(shape, dtype=dtype).pin_memory() if dev.type == "cuda" \
                else torch.zeros(shape, dtype=dtype)

        # Ring of pinned staging slots: an async H2D copy reads the pinned buffer
        # when the copy EXECUTES, so a slot may be rewritten only after the copies
        # issued from it have completed (the slot's event).  The host can therefore
        # run up to RING - 1 steps ahead of the device.
        self.RING = 4
        self._ring = []
        for _ in range(self.RING):
            packed = pinned(24 * n, torch.uint8)
            packed[16 * n:20 * n].view(torch.int32).fill_(-1)   # slot_mapping: no slot
            self._ring.append(dict(
                **packed_views(packed), packed=packed,
                block_tables=pinned((n, self.max_num_blocks), torch.int32),
                token_ids=pinned(n, torch.int64)))
        self._ring_np = [{k: v.numpy() for k, v in slot.items()} for slot in self._ring]
        self._ring_events = [None] * self.RING
        self._ring_pos = 0
        # (sequence-set version, count) the staging slot was prepared ahead for, or None
        self._ahead = None
        self._seq_epoch = 0
        self.host, self.host_np = self._ring[0], self._ring_np[0]
        # one split-KV workspace serves every layer (they run back to back on
        # one stream)
        first = self.model.model.layers[0].self_attn.attn.decode_op
        first.preallocate(n, dev)
        ws_attr = "_fk_workspace" if hasattr(first, "_fk_workspace") else "_workspace"
        for layer in self.model.model.layers[1:]:
            op = layer.self_attn.attn.decode_op
            setattr(op, ws_attr, getattr(first, ws_attr))
            op._ws_batch, op._status = first._ws_batch, first._status
        self.attn_workspace = getattr(first, ws_attr)
        self.status = first._status

    # ---------------------------------------------------------------- sequences
    def add_sequences(self, context_lens, first_tokens) -> list[Sequence]:
        """Register running sequences whose first `L - 1` tokens are already in
        the cache and whose L-th token (`first_tokens[i]`) is the next input."""
        out = []
        for L, tok in zip(context_lens, first_tokens):
            if len(self.seqs) >= self.max_num_seqs:
                raise RuntimeError("max_num_seqs exceeded")
            if L < 1 or L > self.max_model_len:
                raise ValueError(f"context length {L} outside [1, {self.max_model_len}]")
            s = Sequence(len(self.seqs), int(L), last_token=int(tok))
            self.blocks.allocate(s)
            self.seqs.append(s)
            out.append(s)
        self._bt_dirty = True
        self._seq_epoch += 1
        return out

    @torch.no_grad()
    def prefill(self, prompts, chunk_tokens: int | None = None,
                use_block_tables: bool = True) -> np.ndarray:
        """Run whole prompts through the model, fill their KV pages and sample the
        first new token of each (greedy); the sequences then join the running
        batch, ready for step().  Prefill side of ModelRunner.run
        (fastkernels/infra/engine.py:6048-6063) with the metadata of
        prepare_prefill (engine.py:4902-4990): cu_seqlens, per-token slots and the
        block tables, so attention reads the pages the store has just written.

        chunk_tokens=C splits the work into forwards of at most C tokens; a chunk
        attends over the pages written by earlier chunks plus itself (the
        reference's chunked prefill).  With a tensor-parallel communicator the
        chunk defaults to its row capacity.  use_block_tables=False (whole prompts
        only) attends over the batch's own dense K/V instead, the reference's
        path when no block table exists (its warm-up)."""
        from .comm import get_tp_comm
        comm = get_tp_comm()
        if chunk_tokens is None and comm is not None and comm.world > 1:
            chunk_tokens = comm.max_rows
        dev, bs_ = self.device, self.block_size
        new = []
        for prompt in prompts:
            n = len(prompt)
            if n < 1 or n + 1 > self.max_model_len:
                raise ValueError(f"prompt length {n} outside [1, {self.max_model_len - 1}]")
            if len(self.seqs) + len(new) >= self.max_num_seqs:
                raise RuntimeError("max_num_seqs exceeded")
            s = Sequence(len(self.seqs) + len(new), n)
            self.blocks.allocate(s)
            new.append(s)
        done = [0] * len(new)
        first = np.zeros(len(new), dtype=np.int64)
        while any(d < len(pr) for d, pr in zip(done, prompts)):
            part = pack_prefill_chunk([len(pr) for pr in prompts], done, chunk_tokens)
            ids = np.concatenate([np.asarray(prompts[i][a:a + c], dtype=np.int64)
                                  for i, a, c in part])
            pos = np.concatenate([np.arange(a, a + c, dtype=np.int64) for i, a, c in part])
            tabs = [np.asarray(new[i].block_table, dtype=np.int64) for i, a, c in part]
            slots = np.concatenate([tabs[j][np.arange(a, a + c) // bs_] * bs_
                                    + np.arange(a, a + c) % bs_
                                    for j, (i, a, c) in enumerate(part)]).astype(np.int32)
            cu_q = np.concatenate([[0], np.cumsum([c for _, _, c in part])]).astype(np.int32)
            cu_k = np.concatenate([[0], np.cumsum([a + c for _, a, c in part])]).astype(np.int32)
            paged = use_block_tables or chunk_tokens is not None
            bt = None
            if paged:
                cols = max(len(t) for t in tabs)
                bt_np = np.full((len(part), cols), -1, dtype=np.int32)
                for j, t in enumerate(tabs):
                    bt_np[j, :len(t)] = t
                bt = torch.from_numpy(bt_np).to(dev)
            set_context(True, cu_seqlens_q=torch.from_numpy(cu_q).to(dev),
                        cu_seqlens_k=torch.from_numpy(cu_k).to(dev),
                        max_seqlen_q=max(c for _, _, c in part),
                        max_seqlen_k=max(a + c for _, a, c in part),
                        slot_mapping=torch.from_numpy(slots).to(dev), block_tables=bt)
            hidden = self.model(torch.from_numpy(ids).to(dev), torch.from_numpy(pos).to(dev))
            reset_context()
            ends = [(j, i) for j, (i, a, c) in enumerate(part) if a + c == len(prompts[i])]
            if ends:
                rows = torch.from_numpy(cu_q[[j + 1 for j, _ in ends]].astype(np.int64) - 1).to(dev)
                logits = self.model.lm_head.project(hidden.index_select(0, rows))
                vals, idxs = ops.argmax_rows(logits)
                tok = self.model.lm_head.greedy_pairs(vals, idxs).cpu().numpy()
                for (j, i), t in zip(ends, tok):
                    first[i] = int(t)
            for i, a, c in part:
                done[i] = a + c
        for s, t in zip(new, first):
            s.num_tokens += 1          # the sampled token is the next step's input
            s.last_token = int(t)
            s.output.append(int(t))
            self.seqs.append(s)
        self._bt_dirty = True
        self._seq_epoch += 1
        return first

    def graph_batch_size(self, n: int) -> int:
        for bs in sorted(self.graphs):
            if bs >= n:
                return bs
        return n

    # ----------------------------------------------------------- host-side prep
    def prepare_decode(self, use_host_ids: bool) -> int:
        """Fill the pinned staging arrays for this step (engine.py:5793-5798):
        position = n - 1, context_len = n,
        slot = block_table[-1] * BLOCK + ((n % BLOCK) - 1 if n % BLOCK else BLOCK - 1).
        Everything but the token ids may already have been written while the previous
        step ran on the device (`_prepare_ahead`)."""
        if self._ahead is not None and self._ahead == (self._seq_epoch, len(self.seqs)):
            n = len(self.seqs)
        else:
            n = self._prepare_layout()
        self._ahead = None
        if use_host_ids:
            ids = self.host_np["input_ids"]
            for i, s in enumerate(self.seqs):
                ids[i] = s.last_token
        return n

    def _prepare_ahead(self) -> None:
        """Called between the launch of a step and the wait for its tokens: the next
        step's positions, lengths, slots and block-table changes depend on no token
        value, so they are written into the next staging slot while the device is
        busy.  Skipped when the next step could fail (length limit, pool nearly
        empty), so that such errors are still raised by the step they belong to."""
        if not self.seqs or _NO_PREPARE_AHEAD:
            return
        bs_, pages = self.block_size, 0
        for s in self.seqs:
            if s.num_tokens > self.max_model_len:
                return
            if s.num_tokens % bs_ == 1 and len(s.block_table) * bs_ < s.num_tokens:
                pages += 1
        if pages > len(self.blocks.free):
            return
        self._prepare_layout()
        self._ahead = (self._seq_epoch, len(self.seqs))

    def _prepare_layout(self) -> int:
        self._ring_pos = (self._ring_pos + 1) % self.RING
        ev = self._ring_events[self._ring_pos]
        if ev is not None:
            ev.synchronize()            # copies issued from this slot have landed
        self.host, self.host_np = self._ring[self._ring_pos], self._ring_np[self._ring_pos]
        h, bs_ = self.host_np, self.block_size
        n = len(self.seqs)
        for i, s in enumerate(self.seqs):
            if self.blocks.maybe_append_page(s):
                self._bt_dirty = True
            if s.num_tokens > self.max_model_len:
                raise RuntimeError("sequence exceeds max_model_len")
            m = s.num_tokens % bs_
            h["positions"][i] = s.num_tokens - 1
            h["context_lens"][i] = s.num_tokens
            h["slot_mapping"][i] = s.block_table[-1] * bs_ + (m - 1 if m else bs_ - 1)
        if self._bt_dirty:
            bt = h["block_tables"]
            bt[:n].fill(-1)
            for i, s in enumerate(self.seqs):
                bt[i, :len(s.block_table)] = s.block_table
        return n

    def _mark_slot_in_flight(self) -> None:
        if self.device.type == "cuda":
            ev = self._ring_events[self._ring_pos]
            if ev is None:
                ev = self._ring_events[self._ring_pos] = torch.cuda.Event()
            ev.record()

    def stage_inputs(self, n: int, bs: int, use_host_ids: bool) -> None:
        """H2D copies from pinned memory into the graph's input buffers; padded
        rows get slot -1 / context_len 0 (engine.py:5404-5406)."""
        gv, h = self.graph_vars, self.host
        if bs > n:
            h["slot_mapping"][n:bs] = -1
            h["context_lens"][n:bs] = 0
            h["positions"][n:bs] = 0
        first = 0 if use_host_ids else 8 * self.max_num_seqs
        self._packed_dev[first:].copy_(h["packed"][first:], non_blocking=True)
        self.h2d_bytes += h["packed"].numel() - first
        if self._bt_dirty:
            gv["block_tables"][:bs].copy_(h["block_tables"][:bs], non_blocking=True)
            self.h2d_bytes += h["block_tables"][:bs].numel() * 4
            self._bt_dirty = False

    # -------------------------------------------------------------- graph body
    def _forward(self, bs: int) -> None:
        gv = self.graph_vars
        # one split-KV schedule per step, shared by every layer
        ctx = get_context()
        att = self.model.model.layers[0].self_attn.attn
        op = att.decode_op
        ops.paged_decode_attn_plan(ctx.context_lens, ctx.block_tables, self.block_size,
                                   att.num_heads, att.num_kv_heads, att.head_size,
                                   self.attn_workspace, op._max_splits, status=op._status)
        ctx.attn_plan_ready = True
        hidden = self.model(gv["input_ids"][:bs], gv["positions"][:bs])
        gv["outputs"][:bs] = hidden
        logits = self.model.lm_head.project(hidden)
        gv["lm_logits"][:bs] = logits
        ops.argmax_rows(gv["lm_logits"][:bs], gv["lm_max_vals"][:bs], gv["lm_max_idxs"][:bs])
        ids = self.model.lm_head.greedy_pairs(gv["lm_max_vals"][:bs], gv["lm_max_idxs"][:bs])
        gv["token_ids"][:bs] = ids
        # hand the sampled ids to the next step on the device (engine.py:5689-5705)
        gv["input_ids"][:bs] = ids

    def _set_context(self, bs: int, max_ctx: int) -> None:
        gv = self.graph_vars
        set_context(False, slot_mapping=gv["slot_mapping"][:bs],
                    context_lens=gv["context_lens"][:bs],
                    block_tables=gv["block_tables"][:bs], max_context_len=max_ctx)

    @torch.no_grad()
    def capture_cudagraph(self, batch_sizes) -> None:
        """Capture one graph per batch size with the persistent graph_vars as
        inputs; max_context_len is max_model_len at capture (engine.py:6832-6836)
        and the real lengths are read on the device at replay."""
        gv = self.graph_vars
        saved = {k: gv[k].clone() for k in ("input_ids", "positions", "slot_mapping",
                                             "context_lens", "block_tables")}
        gv["slot_mapping"].fill_(-1)
        gv["context_lens"].fill_(1)
        gv["block_tables"].fill_(0)
        gv["positions"].zero_()
        gv["input_ids"].zero_()
        for bs in sorted(batch_sizes, reverse=True):
            self._set_context(bs, self.max_model_len)
            for _ in range(2):          # warm-up outside capture (lazy allocations, NCCL)
                self._forward(bs)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, self.graph_pool):
                self._forward(bs)
            if self.graph_pool is None:
                self.graph_pool = graph.pool()
            self.graphs[bs] = graph
            torch.cuda.synchronize()
            reset_context()
        for k, v in saved.items():
            gv[k].copy_(v)

    # -------------------------------------------------------------------- steps
    @torch.no_grad()
    def run_step_device(self, bs: int) -> None:
        """Replay (or eagerly run) the step for batch size `bs` on inputs that
        are already in the graph buffers."""
        g = self.graphs.get(bs)
        if g is not None and not self.enforce_eager:
            g.replay()
        else:
            self._set_context(bs, self.max_model_len)
            self._forward(bs)
            reset_context()

    @torch.no_grad()
    def step(self, sync: bool = True) -> np.ndarray | None:
        """One decode step for all running sequences through the public path:
        host prep -> pinned H2D staging -> graph replay -> D2H of the token ids.
        With sync=True the sampled ids come back to the host before returning
        and feed the next step from the host; with sync=False the next step
        reads them from the device buffer and the host copy is deferred."""
        n = self.prepare_decode(use_host_ids=sync)
        bs = self.graph_batch_size(n)
        self.stage_inputs(n, bs, use_host_ids=sync)
        self.run_step_device(bs)
        self.host["token_ids"][:n].copy_(self.graph_vars["token_ids"][:n], non_blocking=True)
        self._mark_slot_in_flight()
        self.d2h_bytes += n * 8
        for s in self.seqs:
            s.num_tokens += 1
        if not sync:
            return None
        landing = self.host_np["token_ids"]     # this step's slot (the next call moves on)
        self._prepare_ahead()
        torch.cuda.current_stream().synchronize()
        ids = landing[:n].copy()
        for s, t in zip(self.seqs, ids.tolist()):
            s.last_token = t
            s.output.append(t)
        return ids

    def device_status(self) -> int:
        """OR of every device status word this engine's kernels write (attention
        workspace word, the per-device default word of the row kernels and GEMMs,
        the tensor-parallel communicator's): 0 = no slot / page / position out of
        range and no wait ran out.  Synchronises; call between steps."""
        st = int(self.status.item()) | int(ops.default_status(self.device).item())
        if self.comm is not None:
            st |= int(self.comm.status.item())
        return st

    def decode(self, steps: int) -> np.ndarray:
        """Greedy-decode `steps` tokens for every running sequence; [steps, n].
        Raises if a kernel reported a device-side anomaly on the way."""
        toks = np.stack([self.step(sync=True) for _ in range(steps)])
        st = self.device_status()
        if st:
            if st & 4:
                # a wait ran out: a late stream-K contributor may have left its flag
                # raised, so the shared GEMM workspace starts the next call zeroed again
                ops.gemm_workspace(self.device)[:1024].zero_()
            raise RuntimeError(f"device status word {st} after decoding (fk_device_status bits)")
        return toks
