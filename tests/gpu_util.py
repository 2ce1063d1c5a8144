"""Helpers shared by the GPU parity tests (numpy <-> torch CUDA bf16)."""
import numpy as np
import torch

from oracle import decode_oracle as O


def dev(a: np.ndarray, dtype=None) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a))
    if t.dtype == torch.float32 and dtype is None:
        dtype = torch.bfloat16
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def host_f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def host_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def assert_bf16_close(got: torch.Tensor, want_f32: np.ndarray, max_ulp=1, frac=0.02,
                      atol=2e-2, rtol=2e-2):
    """Within the stated tolerance (atol/rtol 2e-2) everywhere, and identical
    to the oracle's bf16 value except for `frac` of the elements, which may be
    off by at most `max_ulp` bf16 steps (fp32 reduction order)."""
    g = host_f32(got)
    np.testing.assert_allclose(g, want_f32, atol=atol, rtol=rtol)
    gb = O.bf16_round_bits(g).astype(np.int32)
    wb = O.bf16_round_bits(want_f32).astype(np.int32)
    same_sign = (gb & 0x8000) == (wb & 0x8000)
    d = np.abs((gb & 0x7FFF) - (wb & 0x7FFF))
    tiny = np.abs(want_f32) < 1e-3
    bad = (~same_sign & ~tiny) | ((d > max_ulp) & ~tiny)
    assert not bad.any(), f"{bad.sum()} elements beyond {max_ulp} ulp"
    assert ((d > 0) & ~tiny).mean() <= frac, f"{((d > 0) & ~tiny).mean():.4f} of elements differ"
