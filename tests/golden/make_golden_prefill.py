"""Generate tests/golden/prefill_vectors.npz from the reference's own Python code
(CPU), imported from a checkout of Snowflake-AI-Research/fastkernels.

    python tests/golden/make_golden_prefill.py /path/to/fastkernels-checkout

Inputs come from tests/cases.py (seeded, numpy-only); only the reference OUTPUTS
are stored.  Reference paths exercised:
  Attention._prefill_torch_from_tensors   L2/attention_impl.py:624-636
  Attention._prefill_torch_from_cache     L2/attention_impl.py:638-652
  (both through _sdpa_one, 606-622)
The merge of two partial results has no CPU code in the reference (CUDA and
Triton only), so its fixture is the identity the reference documents for it
(merge_attn_states.py:1-6): attention over [prefix | suffix] computed by the
functions above.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

import cases  # noqa: E402

CASES = {
    # name: (seed, q_lens, k_lens, hq, hkv, block_size)
    "ragged": (41, [5, 127, 129], [5, 127, 129], 2, 1, 64),
    "chunked": (42, [1, 64, 100], [300, 64, 333], 4, 2, 64),
    "gqa8_page16": (43, [33, 50], [33, 200], 8, 1, 16),
}


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    torch.set_num_threads(8)
    from fastkernels.tasks.baseline.L2.attention_impl import Attention

    out: dict[str, np.ndarray] = {}
    for name, (seed, ql, kl, hq, hkv, bs) in CASES.items():
        c = cases.prefill_case(seed, ql, kl, hq, hkv, block_size=bs)
        att = object.__new__(Attention)
        torch.nn.Module.__init__(att)
        att.num_heads, att.num_kv_heads, att.head_size = hq, hkv, 128
        att.scale, att._block_size = c["scale"], bs
        q = torch.from_numpy(c["q"])
        cu_q, cu_k = torch.from_numpy(c["cu_q"]), torch.from_numpy(c["cu_k"])
        dense = att._prefill_torch_from_tensors(
            q, torch.from_numpy(c["k"]), torch.from_numpy(c["v"]), cu_q, cu_k)
        paged = att._prefill_torch_from_cache(
            q, torch.from_numpy(c["k_cache"]), torch.from_numpy(c["v_cache"]), cu_q, cu_k,
            torch.from_numpy(c["block_tables"]))
        keep = 1 if name == "chunked" else 2     # every token / every 2nd token
        out[f"{name}_dense"] = dense.numpy().astype(np.float32)[::keep]
        # the paged path must agree with the dense one; every 4th token is kept
        out[f"{name}_paged_every4"] = paged.numpy().astype(np.float32)[::4]
    path = os.path.join(HERE, "prefill_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
