"""The candidates drop into the reference's `tasks/candidate/` slot.

Drives the reference's own loader and swapper (fastkernels/list.py:443-523, the
round trip of the reference's tests/test_bench.py:162-212) over
fastkernels_b200/candidate on CPU.  Needs a checkout of the reference: its root
is taken from FK_REFERENCE_ROOT, else from a directory `reference` beside this
repository; without one the test is skipped.  The work happens in a child
process (tests/candidate_slot_probe.py) because the reference reads
FASTKERNELS_CANDIDATE_DIR at import time and its modules must not leak into the
other tests' process.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]


def _reference_root() -> Path | None:
    for cand in (os.environ.get("FK_REFERENCE_ROOT"), REPO.parent / "reference"):
        if cand and (Path(cand) / "fastkernels" / "list.py").is_file():
            return Path(cand)
    return None


@pytest.fixture(scope="module")
def report():
    root = _reference_root()
    if root is None:
        pytest.skip("no reference checkout (set FK_REFERENCE_ROOT)")
    env = dict(os.environ)
    env["FASTKERNELS_CANDIDATE_DIR"] = str(REPO / "fastkernels_b200" / "candidate")
    env["PYTHONPATH"] = os.pathsep.join([str(root), str(REPO), env.get("PYTHONPATH", "")])
    r = subprocess.run([sys.executable, str(REPO / "tests" / "candidate_slot_probe.py")],
                       env=env, cwd=str(REPO / "tests"), capture_output=True, text=True,
                       timeout=900)
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("REPORT ")]
    assert r.returncode == 0 and lines, f"probe failed:\n{r.stdout[-3000:]}\n{r.stderr[-3000:]}"
    return json.loads(lines[-1][len("REPORT "):])


EXPECTED = {
    "L1/allreduce:AllReduce", "L1/embedding:Embedding", "L1/flash_attn_decode:FlashAttnDecode",
    "L1/flash_attn_prefill:FlashAttnPrefill", "L1/flashinfer_decode:TRTLLMDecode",
    "L1/flashinfer_prefill:TRTLLMPrefill", "L1/linear:Matmul", "L1/linear:Linear",
    "L1/merge_attn_states:MergeAttnStates", "L1/rms_norm:RMSNorm",
    "L1/rotary_emb:RotaryEmbedding", "L1/silu_and_mul:SiluAndMul",
    "L1/store_kvcache:StoreKVCache", "L1/store_kvcache:StoreKVCacheHND",
    "L2/attention:LlamaAttention", "L2/attention_impl:Attention", "L2/llama_mlp:LlamaMLP",
    "L2/parallel_embedding:VocabParallelEmbedding", "L2/parallel_embedding:ParallelLMHead",
    "L2/parallel_linear:ColumnParallelLinear", "L2/parallel_linear:MergedColumnParallelLinear",
    "L2/parallel_linear:QKVParallelLinear", "L2/parallel_linear:RowParallelLinear",
    "L3/llama_decoder:LlamaDecoderLayer", "L4/llama:LlamaForCausalLM",
}


def test_loader_finds_every_candidate_class(report):
    """_load_candidate_class returns a class of the target's own name for every
    operator class of every baseline file that has a candidate file: the classes
    this build replaces, and the baseline's own for the ones it does not (so the
    loader's last-Module-in-file fallback never binds an unrelated class)."""
    assert report["wrong_class"] == []
    replaced = {t["key"] for t in report["targets"] if not t["kept_baseline"]}
    assert replaced == EXPECTED, sorted(replaced ^ EXPECTED)


def test_signatures_accept_what_the_baseline_accepts(report):
    """__init__ and forward of every replaced class take the baseline's parameters
    (same order, same defaults); additions are keyword-only with defaults."""
    assert report["signature_problems"] == {}


def test_swap_and_restore_round_trip(report):
    sw = report["swap"]
    # baseline files that import without CUDA extensions are all paired
    cpu_importable = EXPECTED - {"L1/flash_attn_decode:FlashAttnDecode",
                                 "L1/flash_attn_prefill:FlashAttnPrefill",
                                 "L1/flashinfer_prefill:TRTLLMPrefill"}
    assert cpu_importable <= set(sw["pairs"]), sorted(cpu_importable - set(sw["pairs"]))
    assert sw["l3_sees_l2"] and sw["l3_sees_l1"] and sw["l2_sees_l2"]
    assert sw["baseline_l3_uses_candidate_attention"] and sw["baseline_l3_uses_candidate_mlp"]
    assert sw["baseline_l4_submodule_packages"] == ["fastkernels_b200"]
    assert sw["decode_op_isinstance"]
    assert sw["attention_layout"] == [256, "NHD"]      # the reference's CPU default backend
    assert sw["restored"]


def test_parameter_names_and_shapes_match_the_baseline(report):
    assert report["swap"]["state_dict_mismatch"] == {}
    assert len(report["swap"]["state_dict_classes"]) >= 10


def test_candidates_read_the_reference_engine_context(report):
    assert report["context"] == {"reads_reference": True, "own_wins_while_set": True,
                                 "back_to_reference": True}
