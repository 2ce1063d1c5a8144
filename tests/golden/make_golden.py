"""Generate tests/golden/reference_vectors.npz from the reference's own Python
code (CPU), imported from a checkout of Snowflake-AI-Research/fastkernels.

    python tests/golden/make_golden.py /path/to/fastkernels-checkout

The inputs come from tests/cases.py (seeded, numpy-only), so only the reference
OUTPUTS are stored.  Functions exercised (reference paths):
  Attention._decode_torch / _cache_seq / _sdpa_one   L2/attention_impl.py:598-664
  RMSNorm.forward_native                             L1/rms_norm.py:97-118
  RotaryEmbedding.__init__ cache, forward_native     L1/rotary_emb.py:93-139
  SiluAndMul.forward_native                          L1/silu_and_mul.py:18-22
  F.linear as called by the parallel linears         L2/parallel_linear.py:81
  store: index_copy_ restatement of                  L1/store_kvcache.py:16-35
    (the reference has only a Triton kernel for the store, so the fixture is the
     three-line torch restatement of its semantics)
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import cases  # noqa: E402
from oracle.decode_oracle import bf16_round_bits  # noqa: E402


def t_bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a).to(torch.bfloat16)


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    torch.manual_seed(0)
    torch.set_num_threads(8)
    from fastkernels.tasks.baseline.L1.rms_norm import RMSNorm
    from fastkernels.tasks.baseline.L1.rotary_emb import RotaryEmbedding
    from fastkernels.tasks.baseline.L1.silu_and_mul import SiluAndMul
    from fastkernels.tasks.baseline.L2.attention_impl import Attention

    out: dict[str, np.ndarray] = {}

    # ---- attention: small ragged case + config 1 ---------------------------
    def run_attn(case, hq, hkv, d):
        att = object.__new__(Attention)
        torch.nn.Module.__init__(att)
        att.num_heads, att.num_kv_heads, att.head_size = hq, hkv, d
        att.scale, att._block_size = case["scale"], case["block_size"]
        o = att._decode_torch(
            torch.from_numpy(case["q"]), torch.from_numpy(case["k_cache"]),
            torch.from_numpy(case["v_cache"]), torch.from_numpy(case["context_lens"]),
            torch.from_numpy(case["block_tables"]))
        return o.numpy().astype(np.float32)

    small = cases.attention_case(11, 5, 8, 2, 128, 64, 12, lens=[1, 63, 64, 65, 200])
    out["attn_small"] = run_attn(small, 8, 2, 128)
    c1 = cases.config1_case()
    # store the new token first (engine order), then attend over len + 1
    kc, vc = torch.from_numpy(c1["k_cache"]), torch.from_numpy(c1["v_cache"])
    slots = torch.from_numpy(c1["slot_mapping"]).long()
    kc.view(-1, 8 * 128).index_copy_(0, slots, torch.from_numpy(c1["new_k"]).view(8, -1))
    vc.view(-1, 8 * 128).index_copy_(0, slots, torch.from_numpy(c1["new_v"]).view(8, -1))
    out["attn_c1"] = run_attn(c1, 32, 8, 128)
    out["store_c1_k_rows"] = bits(t_bf16(kc.view(-1, 8 * 128)[slots].numpy()))
    out["store_c1_v_rows"] = bits(t_bf16(vc.view(-1, 8 * 128)[slots].numpy()))
    g16 = cases.attention_case(12, 3, 16, 1, 128, 64, 16, lens=[7, 129, 500])
    out["attn_g16"] = run_attn(g16, 16, 1, 128)

    # ---- rmsnorm native ------------------------------------------------------
    rc = cases.rope_store_case(21, 6, 256, 4, 2, 128, 4, 64, 64, qk_norm=True)
    x, r, w = t_bf16(rc["x"]), t_bf16(rc["residual"]), t_bf16(rc["norm_w"])
    out["rms_plain"] = bits(RMSNorm.forward_native(x, w, 1e-6, 256))
    y, rr = RMSNorm.forward_native(x, w, 1e-6, 256, r)
    out["rms_fused_y"], out["rms_fused_res"] = bits(y), bits(rr)
    q3 = t_bf16(rc["qkv"])[:, :4 * 128].view(6, 4, 128)
    out["rms_heads"] = bits(RMSNorm.forward_native(q3, t_bf16(rc["q_norm_w"]), 1e-6, 128))

    # ---- rope ----------------------------------------------------------------
    rope = RotaryEmbedding(128, 64, 1e6)
    out["rope_cache"] = rope.cos_sin_cache.numpy().astype(np.float32)
    cache_bf = rope.cos_sin_cache.to(torch.bfloat16)
    qkv = t_bf16(rc["qkv"])
    q, k = qkv[:, :512].contiguous(), qkv[:, 512:768].contiguous()
    pos = torch.from_numpy(rc["positions"])
    qo, ko = RotaryEmbedding.forward_native(pos, q, k, 128, cache_bf)
    out["rope_q"], out["rope_k"] = bits(qo), bits(ko)
    rope5 = RotaryEmbedding(128, 32, 5e5)
    out["rope_cache_5e5"] = rope5.cos_sin_cache.numpy().astype(np.float32)

    # ---- silu ------------------------------------------------------------------
    rs = np.random.RandomState(31)
    sx = cases.randn_bf16(rs, (7, 2 * 96), 2.0)
    out["silu"] = bits(SiluAndMul.forward_native(t_bf16(sx)))

    # ---- linear ----------------------------------------------------------------
    lx, lw = cases.randn_bf16(rs, (5, 192)), cases.randn_bf16(rs, (130, 192), 0.05)
    lb = cases.randn_bf16(rs, (130,), 0.1)
    out["linear"] = bits(torch.nn.functional.linear(t_bf16(lx), t_bf16(lw)))
    out["linear_bias"] = bits(torch.nn.functional.linear(t_bf16(lx), t_bf16(lw), t_bf16(lb)))

    path = os.path.join(HERE, "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
