"""Child process of tests/test_candidate_slot.py.

Runs with the reference checkout on sys.path and FASTKERNELS_CANDIDATE_DIR
pointing at fastkernels_b200/candidate, drives the reference's OWN loader
(fastkernels/list.py: discover_operator_targets, _load_candidate_class,
discover_candidate_impls, apply_candidates, restore_candidates) over this
package's candidate files on CPU, and prints one JSON object with what it saw.
No kernel is launched: only imports, constructors and signatures.
"""
from __future__ import annotations

import ast
import importlib
import inspect
import json
import sys
from pathlib import Path


def baseline_signatures(path: Path) -> dict:
    """{class: {method: [(name, kind, has_default, default_repr)]}} read from the
    baseline source with ast (some baseline files need CUDA extensions to import)."""
    tree = ast.parse(path.read_text())
    out = {}
    for node in tree.body:
        if not isinstance(node, ast.ClassDef):
            continue
        methods = {}
        for item in node.body:
            if isinstance(item, ast.FunctionDef) and item.name in ("__init__", "forward"):
                a = item.args
                params = []
                pos = a.posonlyargs + a.args
                defaults = [None] * (len(pos) - len(a.defaults)) + list(a.defaults)
                for arg, d in zip(pos, defaults):
                    params.append((arg.arg, "pos", d is not None,
                                   ast.unparse(d) if d is not None else None))
                if a.vararg:
                    params.append((a.vararg.arg, "var", False, None))
                for arg, d in zip(a.kwonlyargs, a.kw_defaults):
                    params.append((arg.arg, "kw", d is not None,
                                   ast.unparse(d) if d is not None else None))
                if a.kwarg:
                    params.append((a.kwarg.arg, "varkw", False, None))
                methods[item.name] = params
        out[node.name] = methods
    return out


def compare(base_params, cand_sig: inspect.Signature) -> list[str]:
    """Everything the baseline accepts must be accepted, in the same position and
    with the same default; what the candidate adds must be optional and
    keyword-only (or swallowed by *args / **kwargs)."""
    problems = []
    cand = list(cand_sig.parameters.values())
    cand_by_name = {p.name: p for p in cand}
    cand_varkw = any(p.kind is p.VAR_KEYWORD for p in cand)
    cand_var = any(p.kind is p.VAR_POSITIONAL for p in cand)
    cand_pos = [p for p in cand if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
    base_pos = [b for b in base_params if b[1] == "pos"]
    for i, (name, kind, has_default, default) in enumerate(base_pos):
        if name == "self":
            continue
        if i < len(cand_pos):
            c = cand_pos[i]
            if c.name != name and not (cand_var and cand_varkw):
                problems.append(f"positional {i}: baseline '{name}', candidate '{c.name}'")
                continue
            if c.name == name and has_default:
                if c.default is inspect.Parameter.empty:
                    problems.append(f"'{name}' lost its default")
                elif repr(c.default) != default and str(c.default) != default:
                    try:
                        same = c.default == ast.literal_eval(default)
                    except Exception:
                        same = False
                    if not same:
                        problems.append(f"'{name}' default {default} -> {c.default!r}")
        elif not (cand_var and cand_varkw):
            if name not in cand_by_name and not cand_varkw:
                problems.append(f"missing parameter '{name}'")
    for name, kind, has_default, default in base_params:
        if kind == "kw" and name not in cand_by_name and not cand_varkw:
            problems.append(f"missing keyword '{name}'")
    base_names = {b[0] for b in base_params}
    base_open = any(b[1] in ("var", "varkw") for b in base_params)
    for p in cand:
        if p.name in base_names or p.kind in (p.VAR_POSITIONAL, p.VAR_KEYWORD):
            continue
        if base_open:
            continue
        if p.kind is not p.KEYWORD_ONLY or p.default is inspect.Parameter.empty:
            problems.append(f"extra parameter '{p.name}' must be keyword-only with a default")
    return problems


def main() -> None:
    import torch
    import fastkernels
    import fastkernels.list as L

    report: dict = {"candidate_dir": str(fastkernels.CANDIDATE_DIR), "targets": [],
                    "signature_problems": {}, "wrong_class": [], "swap": {}, "context": {}}
    baseline_dir = Path(fastkernels.BASELINE_DIR)
    for t in L.discover_operator_targets():
        f = fastkernels.CANDIDATE_DIR / f"L{t.level}" / f"{t.name}.py"
        if not f.is_file():
            continue
        key = f"L{t.level}/{t.name}:{t.class_name}"
        cand = L._load_candidate_class(f, t.class_name)
        base_mod_name = f"fastkernels.tasks.baseline.L{t.level}.{t.name}"
        kept = cand is not None and cand.__module__ == base_mod_name
        report["targets"].append({"key": key, "kept_baseline": kept})
        if cand is None or cand.__name__ != t.class_name:
            report["wrong_class"].append(f"{key} -> {getattr(cand, '__name__', None)}")
            continue
        if kept:
            continue
        sigs = baseline_signatures(baseline_dir / f"L{t.level}" / f"{t.name}.py")
        for method, base_params in sigs.get(t.class_name, {}).items():
            probs = compare(base_params, inspect.signature(getattr(cand, method)))
            if probs:
                report["signature_problems"][f"{key}.{method}"] = probs

    # swap / restore round trip through the reference's own functions
    pairs = L.discover_candidate_impls()
    report["swap"]["pairs"] = sorted(f"L{t.level}/{t.name}:{t.class_name}" for t, _b, _c in pairs)
    by_name = {t.class_name: (b, c) for t, b, c in pairs}
    undo = L.apply_candidates(pairs)
    l3 = importlib.import_module("fastkernels.tasks.baseline.L3.llama_decoder")
    l4 = importlib.import_module("fastkernels.tasks.baseline.L4.llama")
    l2a = importlib.import_module("fastkernels.tasks.baseline.L2.attention")
    report["swap"]["l3_sees_l2"] = l3.LlamaAttention is by_name["LlamaAttention"][1]
    report["swap"]["l3_sees_l1"] = l3.RMSNorm is by_name["RMSNorm"][1]
    report["swap"]["l2_sees_l2"] = l2a.Attention is by_name["Attention"][1]
    cfg = l4.LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                         vocab_size=1024, max_position_embeddings=512,
                         rope_scaling_factor=1.0)
    # the BASELINE L3 / L4 classes, built after the swap, are made of candidates
    base_l3 = by_name["LlamaDecoderLayer"][0]
    layer = base_l3(cfg, rotary_emb=None, bias=False, qk_norm=True)
    report["swap"]["baseline_l3_uses_candidate_attention"] = \
        type(layer.self_attn) is by_name["LlamaAttention"][1]
    report["swap"]["baseline_l3_uses_candidate_mlp"] = type(layer.mlp) is by_name["LlamaMLP"][1]
    report["swap"]["attention_layout"] = [layer.self_attn.attn._block_size,
                                          layer.self_attn.attn.kv_layout]
    base_l4 = by_name["LlamaForCausalLM"][0]
    model = base_l4(cfg)
    kinds = {type(m).__module__.split(".")[0] for m in model.modules()
             if type(m).__module__.split(".")[0] in ("fastkernels", "fastkernels_b200")
             and type(m) is not base_l4 and type(m).__name__ != "LlamaModel"}
    report["swap"]["baseline_l4_submodule_packages"] = sorted(kinds)
    # class identity: the engine looks decode ops up with isinstance against the
    # (swapped) name in the baseline module
    if "FlashAttnDecode" in by_name:
        fa = importlib.import_module("fastkernels.tasks.baseline.L1.flash_attn_decode")
        report["swap"]["decode_op_isinstance"] = isinstance(
            layer.self_attn.attn.decode_op, fa.FlashAttnDecode)
    else:
        cand_fa = L._load_candidate_class(
            fastkernels.CANDIDATE_DIR / "L1" / "flash_attn_decode.py", "FlashAttnDecode")
        report["swap"]["decode_op_isinstance"] = isinstance(
            layer.self_attn.attn.decode_op, cand_fa)
    L.restore_candidates(undo)
    report["swap"]["restored"] = l3.LlamaAttention is by_name["LlamaAttention"][0] \
        and l3.RMSNorm is by_name["RMSNorm"][0]
    # load_state_dict(strict=False) copies the baseline's weights into a candidate
    # (fastkernels/bench.py:2177): names and shapes of parameters and buffers must
    # match, class by class (the baseline attention layer itself needs CUDA
    # extensions to construct, so it is compared through its parts)
    mismatched = {}
    builds = {
        "RMSNorm": ((256,), {"eps": 1e-6}),
        "RotaryEmbedding": ((128, 512, 1e6), {}),
        "Linear": ((64, 32), {"bias": True}),
        "Embedding": ((100, 32), {"padding_idx": 0}),
        "ColumnParallelLinear": ((256, 512), {"bias": True}),
        "MergedColumnParallelLinear": ((256, [512, 512]), {}),
        "QKVParallelLinear": ((256, 128, 4, 2), {"bias": True}),
        "RowParallelLinear": ((512, 256), {"bias": True}),
        "VocabParallelEmbedding": ((1024, 256), {}),
        "ParallelLMHead": ((1024, 256), {}),
        "LlamaMLP": ((cfg,), {}),
    }
    for name, (args, kwargs) in builds.items():
        base_cls, cand_cls = by_name[name]
        b, c = base_cls(*args, **kwargs), cand_cls(*args, **kwargs)
        sb = {k: (tuple(v.shape), str(v.dtype)) for k, v in b.state_dict().items()}
        sc = {k: (tuple(v.shape), str(v.dtype)) for k, v in c.state_dict().items()}
        bb = {k: tuple(v.shape) for k, v in b.named_buffers() if not k.startswith("_")}
        cb = {k: tuple(v.shape) for k, v in c.named_buffers() if not k.startswith("_")}
        if sb != sc or bb != cb:
            mismatched[name] = {"baseline": sorted(sb) + sorted(bb),
                                "candidate": sorted(sc) + sorted(cb)}
    report["swap"]["state_dict_mismatch"] = mismatched
    report["swap"]["state_dict_classes"] = sorted(builds)

    # the candidates read the context the reference engine sets
    import fastkernels.infra.context as ref_ctx
    from fastkernels_b200.infra import context as own_ctx
    lens = torch.arange(3, dtype=torch.int32)
    ref_ctx.set_context(False, slot_mapping=lens, context_lens=lens, block_tables=None)
    seen = own_ctx.get_context()
    report["context"]["reads_reference"] = seen is ref_ctx.get_context() \
        and seen.context_lens is lens
    own_ctx.set_context(False, context_lens=lens + 1)
    report["context"]["own_wins_while_set"] = own_ctx.get_context() is not ref_ctx.get_context()
    own_ctx.reset_context()
    report["context"]["back_to_reference"] = own_ctx.get_context() is ref_ctx.get_context()
    ref_ctx.reset_context()
    print("REPORT " + json.dumps(report))


if __name__ == "__main__":
    main()
