"""Host-side logic of the decode engine on CPU (no kernel is launched): block
manager, per-step positions / slots / context lengths, block-table staging."""
import numpy as np
import pytest
import torch

from fastkernels_b200.candidate.L4.llama import LlamaConfig
from fastkernels_b200.engine import BlockManager, DecodeEngine, Sequence


def tiny_cfg(block=64):
    return LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=1,
                       num_attention_heads=2, num_key_value_heads=1, head_dim=128,
                       vocab_size=256, max_position_embeddings=512, qk_norm=True,
                       kv_block_size=block)


def test_block_manager_appends_on_first_token_of_page():
    bm = BlockManager(8, 4)
    s = Sequence(0, 4)
    bm.allocate(s)
    assert len(s.block_table) == 1
    assert not bm.maybe_append_page(s)          # n = 4: page full, nothing new yet
    s.num_tokens = 5                            # the sampled token opens a page
    assert bm.maybe_append_page(s) and len(s.block_table) == 2
    assert not bm.maybe_append_page(s)          # idempotent within the step
    s.num_tokens = 6
    assert not bm.maybe_append_page(s)
    bm.release(s)
    assert len(bm.free) == 8
    small = BlockManager(1, 4)
    a = Sequence(0, 4)
    small.allocate(a)
    with pytest.raises(RuntimeError, match="exhausted"):
        small.allocate(Sequence(1, 1))


def test_prepare_decode_matches_reference_arithmetic():
    """position = n-1, context_len = n,
    slot = bt[-1]*B + ((n % B) - 1 if n % B else B - 1)  (engine.py:5793-5798)."""
    eng = DecodeEngine(tiny_cfg(64), max_num_seqs=4, max_model_len=256, num_kv_blocks=16,
                       device="cpu")
    lens = [1, 64, 65, 130]
    eng.add_sequences(lens, [7, 8, 9, 10])
    dev_bt = None                                # what the device would hold
    for step in range(70):
        n = eng.prepare_decode(use_host_ids=True)
        assert n == 4
        h = eng.host_np
        if eng._bt_dirty:                        # staged only when a page was added
            dev_bt = h["block_tables"].copy()
        for i, s in enumerate(eng.seqs):
            L = lens[i] + step
            assert s.num_tokens == L
            assert h["positions"][i] == L - 1 and h["context_lens"][i] == L
            page = s.block_table[(L - 1) // 64]
            assert h["slot_mapping"][i] == page * 64 + (L - 1) % 64
            assert len(s.block_table) == (L + 63) // 64
            assert list(dev_bt[i, :len(s.block_table)]) == s.block_table
            assert (dev_bt[i, len(s.block_table):] == -1).all()
        eng._bt_dirty = False
        for s in eng.seqs:
            s.num_tokens += 1
    all_pages = sum((s.block_table for s in eng.seqs), [])
    assert len(set(all_pages)) == len(all_pages)          # no page shared


@pytest.mark.parametrize("ahead", [False, True])
def test_layout_prepared_ahead_equals_layout_prepared_on_time(ahead):
    """step(sync=True) writes the next step's positions / lengths / slots / block
    tables while the device still runs the current one (`_prepare_ahead`).  The
    staged values must be the ones an engine without that look-ahead stages, the
    look-ahead must be dropped when sequences join in between, and it must not run
    when the next step could fail (more pages needed than the pool has left)."""
    def make():
        e = DecodeEngine(tiny_cfg(64), max_num_seqs=6, max_model_len=256, num_kv_blocks=18,
                         device="cpu")
        e.add_sequences([1, 64, 65, 130], [7, 8, 9, 10])
        return e
    eng, ref = make(), make()
    for step in range(120):
        if step == 50:                            # a sequence joins between two steps
            eng.add_sequences([33], [5])
            ref.add_sequences([33], [5])
        slot_before = eng._ring_pos
        n = eng.prepare_decode(use_host_ids=True)
        assert n == ref.prepare_decode(use_host_ids=True)
        if ahead and step and step != 50 and used_ahead:
            assert eng._ring_pos == slot_before   # the slot written ahead is the one used
        for k in ("positions", "context_lens", "slot_mapping", "input_ids"):
            assert (eng.host_np[k][:n] == ref.host_np[k][:n]).all(), (k, step)
        assert eng._bt_dirty == ref._bt_dirty
        if eng._bt_dirty:
            assert (eng.host_np["block_tables"][:n] == ref.host_np["block_tables"][:n]).all()
        eng._bt_dirty = ref._bt_dirty = False
        for e in (eng, ref):
            for i, s in enumerate(e.seqs):
                s.num_tokens += 1
                s.last_token = 100 + step + i
        used_ahead = False
        if ahead:
            free = len(eng.blocks.free)
            need = sum(1 for s in eng.seqs
                       if s.num_tokens % 64 == 1 and len(s.block_table) * 64 < s.num_tokens)
            eng._prepare_ahead()
            used_ahead = eng._ahead is not None
            assert used_ahead == (need <= free)
    assert [s.block_table for s in eng.seqs] == [s.block_table for s in ref.seqs]


def test_look_ahead_leaves_errors_to_the_step_they_belong_to():
    eng = DecodeEngine(tiny_cfg(64), max_num_seqs=2, max_model_len=128, num_kv_blocks=2,
                       device="cpu")
    eng.add_sequences([64, 1], [0, 0])            # both pages of the pool taken
    eng.prepare_decode(True)
    for s in eng.seqs:
        s.num_tokens += 1                         # 65 tokens: the next step needs a page
    eng._prepare_ahead()                          # nothing staged, nothing raised
    assert eng._ahead is None and len(eng.seqs[0].block_table) == 1
    with pytest.raises(RuntimeError, match="exhausted"):
        eng.prepare_decode(True)


def test_limits_are_enforced():
    eng = DecodeEngine(tiny_cfg(64), max_num_seqs=2, max_model_len=128, num_kv_blocks=4,
                       device="cpu")
    with pytest.raises(ValueError):
        eng.add_sequences([129], [0])
    eng.add_sequences([128, 5], [0, 0])
    with pytest.raises(RuntimeError, match="max_num_seqs"):
        eng.add_sequences([1], [0])
    eng.seqs[0].num_tokens = 129
    with pytest.raises(RuntimeError):
        eng.prepare_decode(True)


def test_kv_pool_layout_and_views():
    eng = DecodeEngine(tiny_cfg(64), max_num_seqs=2, max_model_len=128, num_kv_blocks=4,
                       device="cpu")
    assert tuple(eng.kv_cache.shape) == (2, 1, 4, 64, 1, 128)
    att = eng.model.model.layers[0].self_attn.attn
    assert att.k_cache.data_ptr() == eng.kv_cache[0, 0].data_ptr()
    assert att.v_cache.data_ptr() == eng.kv_cache[1, 0].data_ptr()
    assert att.k_cache.is_contiguous()


def test_prefill_chunk_packing_covers_every_token_once():
    from fastkernels_b200.engine import pack_prefill_chunk
    lens = [1, 17, 64, 130, 201]
    for budget in (None, 1, 48, 64, 1000):
        done = [0] * len(lens)
        seen = [[] for _ in lens]
        rounds = 0
        while any(d < n for d, n in zip(done, lens)):
            part = pack_prefill_chunk(lens, done, budget)
            assert part, "no progress"
            assert len({i for i, _, _ in part}) == len(part)        # one chunk per sequence
            assert budget is None or sum(c for _, _, c in part) <= budget
            for i, a, c in part:
                assert a == done[i] and c > 0
                seen[i].extend(range(a, a + c))
                done[i] = a + c
            rounds += 1
            assert rounds < 10000
        assert all(s_ == list(range(n)) for s_, n in zip(seen, lens))
        if budget is None:
            assert rounds == 1
