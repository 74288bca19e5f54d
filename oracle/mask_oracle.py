"""Definitions of the structured block masks and of the work-item order.  TEST INFRASTRUCTURE ONLY.

Nothing in the product path imports this module; the tests use it as the checker for the
list-emitting mask builders (fba_sta_index, fba_ssta_index) and for fba_fwd_order / fba_bwd_order.

The reference advertises sliding-tile (STA), MoBA and hybrid SSTA masks (reference README.md:54-55)
but ships no builder for them (flex_block_attn/__init__.py:7-12 is commented out), so there is no
reference code to restate; what is restated here is the published definition of each mask, once
with plain Python loops (``*_loops``, for by-hand sized cases) and once vectorised with torch for
the sizes the GPU tests use.  The two forms are checked against each other in tests/test_oracle.py.

  STA    tile i attends tile j iff |dt| <= wt, |dh| <= wh and |dw| <= ww, tile id = (t*Gh + h)*Gw + w.
  MoBA   query block r attends the `topk` key blocks with the largest
         mean(q rows of block r) . mean(k rows of block c); grouped-query heads read kv head h // (Hq/Hkv).
  SSTA   MoBA united with the STA window of the tile that contains the query block
         (one key block = one tile; tile of query block r = r * q_block // kv_block).
  order  stable descending argsort of each work item's summed list length.
"""
from __future__ import annotations

from typing import Sequence

import torch


def sta_mask_loops(tile_grid: Sequence[int], window: Sequence[int]) -> torch.Tensor:
    Gt, Gh, Gw = tile_grid
    n = Gt * Gh * Gw
    m = torch.zeros((n, n), dtype=torch.bool)
    for i in range(n):
        ti, hi, wi = i // (Gh * Gw), (i // Gw) % Gh, i % Gw
        for j in range(n):
            tj, hj, wj = j // (Gh * Gw), (j // Gw) % Gh, j % Gw
            m[i, j] = abs(ti - tj) <= window[0] and abs(hi - hj) <= window[1] and abs(wi - wj) <= window[2]
    return m


def sta_mask(tile_grid: Sequence[int], window: Sequence[int] = (1, 1, 1), device="cpu") -> torch.Tensor:
    Gt, Gh, Gw = tile_grid
    ids = torch.arange(Gt * Gh * Gw, device=device)
    c = torch.stack([ids // (Gh * Gw), (ids // Gw) % Gh, ids % Gw], dim=-1)
    d = (c[:, None, :] - c[None, :, :]).abs()
    return (d[..., 0] <= window[0]) & (d[..., 1] <= window[1]) & (d[..., 2] <= window[2])


def pooled_scores(q: torch.Tensor, k: torch.Tensor, q_block: int, kv_block: int) -> torch.Tensor:
    """[B, Hq, nQ, nK] fp32: (mean of the query block) . (mean of the key block)."""
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    qp = q.float().reshape(B, Hq, Sq // q_block, q_block, D).mean(3)
    kp = k.float().reshape(B, Hkv, Skv // kv_block, kv_block, D).mean(3)
    if Hq != Hkv:
        kp = kp.repeat_interleave(Hq // Hkv, dim=1)
    return torch.matmul(qp, kp.transpose(-1, -2))


def moba_topk_mask_loops(q, k, q_block: int, kv_block: int, topk: int) -> torch.Tensor:
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    nQ, nK = Sq // q_block, Skv // kv_block
    m = torch.zeros((B, Hq, nQ, nK), dtype=torch.bool)
    for b in range(B):
        for h in range(Hq):
            hk = h // (Hq // Hkv)
            for r in range(nQ):
                qm = q[b, h, r * q_block:(r + 1) * q_block].float().mean(0)
                scores = [float(qm @ k[b, hk, c * kv_block:(c + 1) * kv_block].float().mean(0)) for c in range(nK)]
                best = sorted(range(nK), key=lambda c: (-scores[c], c))[: min(topk, nK)]
                for c in best:
                    m[b, h, r, c] = True
    return m


def moba_topk_mask(q, k, q_block: int, kv_block: int, topk: int) -> torch.Tensor:
    score = pooled_scores(q, k, q_block, kv_block)
    top = score.topk(min(topk, score.shape[-1]), dim=-1).indices
    m = torch.zeros_like(score, dtype=torch.bool)
    m.scatter_(-1, top, True)
    return m


def ssta_mask(q, k, tile_grid: Sequence[int], q_block: int, kv_block: int, topk: int = 8,
              window: Sequence[int] = (1, 1, 1)) -> torch.Tensor:
    n_tiles = tile_grid[0] * tile_grid[1] * tile_grid[2]
    assert k.shape[2] == n_tiles * kv_block and kv_block % q_block == 0
    win = sta_mask(tile_grid, window, device=q.device)
    win_q = win.repeat_interleave(kv_block // q_block, dim=0)[: q.shape[2] // q_block]
    return moba_topk_mask(q, k, q_block, kv_block, topk) | win_q[None, None]


def ssta_mask_loops(q, k, tile_grid, q_block, kv_block, topk, window) -> torch.Tensor:
    m = moba_topk_mask_loops(q, k, q_block, kv_block, topk)
    win = sta_mask_loops(tile_grid, window)
    for r in range(m.shape[2]):
        m[:, :, r] |= win[r * q_block // kv_block]
    return m


def explain_selection_differences(mask: torch.Tensor, want: torch.Tensor, score: torch.Tensor,
                                  rtol: float = 1e-4, atol: float = 1e-5) -> int:
    """Rows where two top-k selections differ must differ only by blocks whose pooled scores tie to
    within fp32 summation-order noise.  Returns the number of differing rows, every one of which was
    explained this way; raises AssertionError on the first unexplained one."""
    diff_rows = (mask != want).any(-1)
    n = 0
    for b, h, r in diff_rows.nonzero().tolist():
        a, w = mask[b, h, r], want[b, h, r]
        only_a, only_w = (a & ~w).nonzero().flatten(), (w & ~a).nonzero().flatten()
        assert len(only_a) == len(only_w), f"row ({b},{h},{r}): different number of selected blocks"
        sa, sw = score[b, h, r, only_a].sort().values, score[b, h, r, only_w].sort().values
        assert torch.allclose(sa, sw, rtol=rtol, atol=atol), f"row ({b},{h},{r}): selection differs beyond a numerical tie"
        n += 1
    return n


def work_order(cnt: torch.Tensor, rows_per_bh: int, per_head: bool, n_groups: int, rows_div: int, n_tiles: int,
               tiles_per_item: int, heads_per_item: int) -> torch.Tensor:
    """int32 [n_groups or 1, n_items]: stable descending argsort of the work of each item.

    ``cnt`` holds the list lengths, [n_heads * rows_per_bh] for a per-head list or [rows_per_bh] for
    a list shared by every head.  Item i of group g covers tiles i*tiles_per_item .. (+tiles_per_item-1)
    (those below n_tiles) of heads g*heads_per_item .. (+heads_per_item-1); a tile's list row is
    tile // rows_div.
    """
    n_items = (n_tiles + tiles_per_item - 1) // tiles_per_item
    groups = n_groups if per_head else 1
    cnt = cnt.to(torch.int64).cpu()
    key = torch.zeros((groups, n_items), dtype=torch.int64)
    for g in range(groups):
        for r in range(heads_per_item):
            base = (g * heads_per_item + r) * rows_per_bh if per_head else 0
            for u in range(tiles_per_item):
                tile = torch.arange(n_items) * tiles_per_item + u
                ok = tile < n_tiles
                key[g, ok] += cnt[base + tile[ok] // rows_div]
    return torch.argsort(key, dim=-1, descending=True, stable=True).to(torch.int32)
