"""Block-mask builders for the workloads this operator is measured on.

The reference advertises sliding-tile (STA), MoBA and hybrid SSTA masks but does not ship their
builders (reference flex_block_attn/__init__.py:7-12 is commented out; README.md:54-55), and its
benchmark harness draws random masks with numpy on the host (benchmark/utils/utils.py:69-103).
These builders produce the same kinds of bool block masks directly on the device, in the shapes
``flex_block_attn_func`` accepts: [nQ, nK] or [B, H, nQ, nK], True = attend.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch


def full_mask(nQ: int, nK: int, device="cuda") -> torch.Tensor:
    """All-ones [nQ, nK] mask (dense attention)."""
    return torch.ones((nQ, nK), dtype=torch.bool, device=device)


def bernoulli_mask(B: int, H: int, nQ: int, nK: int, keep: float, seed: int, device="cuda",
                   force_diagonal: bool = True) -> torch.Tensor:
    """Per-(batch, head) i.i.d. Bernoulli(keep) mask [B, H, nQ, nK] with the (scaled) diagonal
    forced on, drawn from a seeded generator on ``device``."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    m = torch.rand((B, H, nQ, nK), generator=g, device=device) < keep
    if force_diagonal:
        i = torch.arange(nQ, device=device)
        m[:, :, i, (i * nK) // nQ] = True
    return m


def tile_major_permutation(grid: Sequence[int], tile: Sequence[int], device="cpu") -> torch.Tensor:
    """Permutation that reorders a raster-order (t, h, w) token sequence into tile-major order.

    ``perm[new_pos] = old_pos``: tokens of one ``tile`` (e.g. 6x8x8 = 384 tokens) become contiguous
    and tiles are ordered raster-wise over the tile grid, so one tile is one attention block.
    Apply as ``x[:, :, perm]``; invert with ``torch.argsort(perm)``.
    """
    T, Hh, W = grid
    tt, th, tw = tile
    assert T % tt == 0 and Hh % th == 0 and W % tw == 0, "grid must be a multiple of the tile"
    idx = torch.arange(T * Hh * W, device=device).reshape(T // tt, tt, Hh // th, th, W // tw, tw)
    return idx.permute(0, 2, 4, 1, 3, 5).reshape(-1)


def sta_mask(tile_grid: Sequence[int], window: Sequence[int] = (1, 1, 1), device="cuda") -> torch.Tensor:
    """3-D sliding-tile attention: tile i attends tile j iff |dt|<=wt, |dh|<=wh and |dw|<=ww in
    tile coordinates.  Returns [n_tiles, n_tiles] with tile id = (t * Gh + h) * Gw + w."""
    Gt, Gh, Gw = tile_grid
    t, h, w = torch.meshgrid(torch.arange(Gt, device=device), torch.arange(Gh, device=device),
                             torch.arange(Gw, device=device), indexing="ij")
    c = torch.stack([t.reshape(-1), h.reshape(-1), w.reshape(-1)], dim=-1)  # [n, 3]
    d = (c[:, None, :] - c[None, :, :]).abs()
    return (d[..., 0] <= window[0]) & (d[..., 1] <= window[1]) & (d[..., 2] <= window[2])


def moba_topk_mask(q: torch.Tensor, k: torch.Tensor, q_block: int, kv_block: int, topk: int) -> torch.Tensor:
    """MoBA-style selection: for every query block the ``topk`` key blocks with the largest
    (mean-pooled query block) . (mean-pooled key block) score.  q: [B, Hq, Sq, D], k: [B, Hkv, Skv, D];
    returns [B, Hq, Sq/q_block, Skv/kv_block]."""
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    qp = q.float().reshape(B, Hq, Sq // q_block, q_block, D).mean(3)
    kp = k.float().reshape(B, Hkv, Skv // kv_block, kv_block, D).mean(3)
    if Hq != Hkv:
        kp = kp.repeat_interleave(Hq // Hkv, dim=1)
    score = torch.matmul(qp, kp.transpose(-1, -2))
    top = score.topk(min(topk, score.shape[-1]), dim=-1).indices
    m = torch.zeros_like(score, dtype=torch.bool)
    m.scatter_(-1, top, True)
    return m


def ssta_mask(q: torch.Tensor, k: torch.Tensor, tile_grid: Sequence[int], q_block: int, kv_block: int,
              topk: int = 8, window: Sequence[int] = (1, 1, 1)) -> torch.Tensor:
    """Hybrid SSTA mask = STA tile window UNION MoBA top-k, for tile-major token order.

    One key block is one tile (kv_block = tokens per tile); a query block is ``q_block`` tokens and
    belongs to tile ``r * q_block // kv_block``.  Returns [B, Hq, Sq/q_block, n_tiles].
    """
    n_tiles = tile_grid[0] * tile_grid[1] * tile_grid[2]
    assert k.shape[2] == n_tiles * kv_block and kv_block % q_block == 0
    win = sta_mask(tile_grid, window, device=q.device)                    # [n_tiles, n_tiles]
    win_q = win.repeat_interleave(kv_block // q_block, dim=0)              # [nQ, n_tiles]
    assert win_q.shape[0] == q.shape[2] // q_block
    return moba_topk_mask(q, k, q_block, kv_block, topk) | win_q[None, None]


def to_tile_major(x: torch.Tensor, grid: Sequence[int], tile: Sequence[int]) -> torch.Tensor:
    """[B, S, H, 128] bf16, raster (t, h, w) token order -> [B, H, S, 128], tile-major token order.

    One CUDA pass (transpose + token permutation); equal to
    ``x.transpose(1, 2)[:, :, tile_major_permutation(grid, tile)]``.
    """
    return _tile_major(x, grid, tile, True)


def from_tile_major(x: torch.Tensor, grid: Sequence[int], tile: Sequence[int]) -> torch.Tensor:
    """Inverse of ``to_tile_major``: [B, H, S, 128] tile-major -> [B, S, H, 128] raster order."""
    return _tile_major(x, grid, tile, False)


def _tile_major(x, grid, tile, forward: bool):
    from . import _cabi

    if not x.is_cuda or x.dtype != torch.bfloat16 or x.dim() != 4 or x.shape[-1] != 128 or not x.is_contiguous():
        raise ValueError("expected a contiguous CUDA bf16 tensor with a last dimension of 128")
    T, H, W = grid
    S = T * H * W
    if forward:
        B, S_in, Hn, _ = x.shape
        out = torch.empty((B, Hn, S, 128), dtype=x.dtype, device=x.device)
    else:
        B, Hn, S_in, _ = x.shape
        out = torch.empty((B, S, Hn, 128), dtype=x.dtype, device=x.device)
    if S_in != S:
        raise ValueError(f"sequence length {S_in} does not match the {T}x{H}x{W} grid")
    with torch.cuda.device(x.device):
        rc = _cabi.lib().fba_tile_major(x.data_ptr(), out.data_ptr(), B, Hn, T, H, W, tile[0], tile[1], tile[2],
                                        1 if forward else 0, torch.cuda.current_stream(x.device).cuda_stream)
    _cabi.check(rc, "fba_tile_major")
    return out
