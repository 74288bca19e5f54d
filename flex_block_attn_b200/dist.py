"""Multi-GPU use of the operator: one process per GPU over ``torch.distributed``.

The reference is single-GPU (its kernels' grid is (tiles, heads, batch) with no cross-head
traffic, reference flex_block_attn_h100.cu:924), so every (batch, head) is an independent unit:

  * ``head_shard``: contiguous head range of a rank -- head-sharded inputs need no collective at
    all, each rank just runs the operator on its heads;
  * ``seq_to_head`` / ``head_to_seq``: the one real exchange, for inputs that arrive
    sequence-sharded (Ulysses layout).  [B, H, S/P, D] on every rank  <->  [B, H/P, S, D].
    Each (peer, batch, local head) chunk [S/P, D] is contiguous on both sides, so the exchange is
    a group of point-to-point sends/receives that lands directly in the layout the kernels read
    (no pack / unpack pass); over NCCL the group runs as one fused all-to-all on NVLink.
  * ``ulysses_flex_block_attn``: all-to-all in, block-sparse attention on the local heads,
    all-to-all out, differentiable end to end.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def head_shard(n_heads: int, world_size: int, rank: int) -> slice:
    """Contiguous head range owned by ``rank`` (n_heads must divide evenly)."""
    if n_heads % world_size != 0:
        raise ValueError(f"{n_heads} heads do not divide over {world_size} ranks")
    per = n_heads // world_size
    return slice(rank * per, (rank + 1) * per)


def _exchange(ops) -> None:
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()


def seq_to_head(x: torch.Tensor, group=None) -> torch.Tensor:
    """[B, H, S/P, D] (all heads, local sequence chunk) -> [B, H/P, S, D] (local heads, all of S)."""
    P = dist.get_world_size(group)
    rank = dist.get_rank(group)
    B, H, Sl, D = x.shape
    if H % P != 0:
        raise ValueError(f"{H} heads do not divide over {P} ranks")
    Hl = H // P
    x = x.contiguous()
    out = torch.empty((B, Hl, Sl * P, D), dtype=x.dtype, device=x.device)
    ops = []
    for peer in range(P):
        gpeer = dist.get_global_rank(group, peer) if group is not None else peer
        for b in range(B):
            for h in range(Hl):
                src = x[b, peer * Hl + h]                       # [Sl, D] contiguous
                dst = out[b, h, peer * Sl:(peer + 1) * Sl]      # [Sl, D] contiguous
                if peer == rank:
                    dst.copy_(x[b, rank * Hl + h])
                else:
                    ops.append(dist.P2POp(dist.isend, src, gpeer, group))
                    ops.append(dist.P2POp(dist.irecv, dst, gpeer, group))
    _exchange(ops)
    return out


def head_to_seq(x: torch.Tensor, group=None) -> torch.Tensor:
    """Inverse of ``seq_to_head``: [B, H/P, S, D] -> [B, H, S/P, D]."""
    P = dist.get_world_size(group)
    rank = dist.get_rank(group)
    B, Hl, S, D = x.shape
    if S % P != 0:
        raise ValueError(f"sequence length {S} does not divide over {P} ranks")
    Sl = S // P
    x = x.contiguous()
    out = torch.empty((B, Hl * P, Sl, D), dtype=x.dtype, device=x.device)
    ops = []
    for peer in range(P):
        gpeer = dist.get_global_rank(group, peer) if group is not None else peer
        for b in range(B):
            for h in range(Hl):
                src = x[b, h, peer * Sl:(peer + 1) * Sl]        # [Sl, D] contiguous
                dst = out[b, peer * Hl + h]                     # [Sl, D] contiguous
                if peer == rank:
                    dst.copy_(x[b, h, rank * Sl:(rank + 1) * Sl])
                else:
                    ops.append(dist.P2POp(dist.isend, src, gpeer, group))
                    ops.append(dist.P2POp(dist.irecv, dst, gpeer, group))
    _exchange(ops)
    return out


class _SeqToHead(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return seq_to_head(x, group)

    @staticmethod
    def backward(ctx, g):
        return head_to_seq(g, ctx.group), None


class _HeadToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return head_to_seq(x, group)

    @staticmethod
    def backward(ctx, g):
        return seq_to_head(g, ctx.group), None


def ulysses_flex_block_attn(q, k, v, q_block_size, kv_block_size, mask_fn: Callable, group=None,
                            attn_fn: Optional[Callable] = None):
    """Block-sparse attention for sequence-sharded inputs.

    q, k, v: [B, H, S/P, 128] local sequence chunks holding all heads.  ``mask_fn(q_h, k_h)`` gets
    the head-sharded, full-sequence tensors ([B, H/P, S, 128]) and returns the block mask for the
    local heads ([nQ, nK] or [B, H/P, nQ, nK]); it runs after the exchange because data-dependent
    masks (top-k of pooled q.k) need the whole sequence of a head.  Returns o: [B, H, S/P, 128].
    ``attn_fn`` defaults to ``flex_block_attn_func`` (a CPU stand-in can be injected for tests of
    the exchange logic).
    """
    if attn_fn is None:
        from .interface import flex_block_attn_func as attn_fn  # noqa: N813
    qh = _SeqToHead.apply(q, group)
    kh = _SeqToHead.apply(k, group)
    vh = _SeqToHead.apply(v, group)
    with torch.no_grad():
        mask = mask_fn(qh, kh)
    oh = attn_fn(qh, kh, vh, q_block_size, kv_block_size, mask)
    return _HeadToSeq.apply(oh, group)
