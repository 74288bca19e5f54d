"""Helpers shared by the tests: fixtures loading, seeded inputs, masks and error metrics."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"
GOLDEN_CASES = sorted(p.stem for p in GOLDEN.glob("*.npz"))

# Acceptance thresholds for bf16 kernels against the fp32 oracle on the same inputs.
MAX_ABS = 2e-2
MIN_COS = 0.9995


def bits_to_bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.astype(np.int16)).view(torch.bfloat16)


def load_golden(name: str) -> dict:
    d = np.load(GOLDEN / f"{name}.npz")
    out = {k: bits_to_bf16(d[k]) for k in ("q", "k", "v", "do")}
    out.update({k: torch.from_numpy(d[k]) for k in ("o", "dq", "dk", "dv")})
    out["block_mask"] = torch.from_numpy(d["block_mask"])
    out["q_block"] = int(d["q_block"])
    out["kv_block"] = int(d["kv_block"])
    return out


def rand_qkv(B, Hq, Hkv, Sq, Skv, seed, scale=1.0, device="cpu", dtype=torch.bfloat16):
    g = torch.Generator(device="cpu").manual_seed(seed)
    mk = lambda h, s: (torch.randn((B, h, s, 128), generator=g) * scale).to(dtype).to(device)
    return mk(Hq, Sq), mk(Hkv, Skv), mk(Hkv, Skv), mk(Hq, Sq)


def bernoulli_mask(shape, keep, seed, force_diag=True):
    g = torch.Generator(device="cpu").manual_seed(seed)
    m = torch.rand(shape, generator=g) < keep
    if force_diag:
        nQ, nK = shape[-2:]
        i = torch.arange(nQ)
        m[..., i, (i * nK) // nQ] = True
    return m


def reference_rule_mask(nQ, nK):
    """The reference test's block-mask rule |i - j| < 2 or j == 4 (test_flex_block_attn.py:25)."""
    i = torch.arange(nQ)[:, None]
    j = torch.arange(nK)[None, :]
    return ((i - j).abs() < 2) | (j == 4)


def err_stats(got: torch.Tensor, want: torch.Tensor):
    g = got.detach().double().flatten().cpu()
    w = want.detach().double().flatten().cpu()
    max_abs = (g - w).abs().max().item()
    denom = (g.norm() * w.norm()).item()
    cos = (g @ w).item() / denom if denom > 0 else (1.0 if g.norm().item() == w.norm().item() else 0.0)
    return max_abs, cos


PARITY_LOG: list = []   # (what, raw max-abs, cosine, max|want|) of every assert_close, in call order


def assert_close(got, want, what, max_abs=MAX_ABS, min_cos=MIN_COS, rel_to_max=True, report=False):
    """max-abs (relative to max|want| when that exceeds 1, so large-magnitude inputs are judged on
    the same bf16 footing) and cosine similarity.  Returns (raw max-abs, cosine, max|want|); with
    ``report`` the raw figures are also printed as one line (shown by ``pytest -s`` / ``-rP``)."""
    ma, cos = err_stats(got, want)
    mx = want.detach().abs().max().item()
    ref = max(1.0, mx) if rel_to_max else 1.0
    PARITY_LOG.append((what, ma, cos, mx))
    if report:
        print(f"PARITY {what}: max_abs={ma:.3e} cos={cos:.7f} max|ref|={mx:.3f} bound={max_abs * ref:.3e}")
    assert torch.isfinite(got.float()).all(), f"{what}: non-finite values"
    assert ma <= max_abs * ref, f"{what}: max-abs {ma:.4g} > {max_abs * ref:.4g} (cos {cos:.6f})"
    assert cos >= min_cos, f"{what}: cosine {cos:.6f} < {min_cos} (max-abs {ma:.4g})"
    return ma, cos, mx
