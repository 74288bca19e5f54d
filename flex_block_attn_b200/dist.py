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
  * ``PeerExchange``: the same exchange for activations held as [B, S/P, H, D] in raster token
    order, fused with the transpose and the raster <-> tile-major token reorder: one kernel per
    GPU stores every row into its final place in the owning GPU's buffer over NVLink peer memory.
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


# ---------------------------------------------------------------------------------------------
# Exchange fused with the layout change, over peer memory.
# ---------------------------------------------------------------------------------------------
def peer_exchange_rows(rank: int, world: int, B: int, H: int, grid, tile, to_head: bool):
    """Where ``fba_peer_exchange`` puts every 128-element row of rank ``rank``'s source tensor.

    Plain-torch statement of the kernel's index arithmetic (CPU; used by the tests and as the
    definition of the layouts): returns ``(dest_rank, dest_row)``, one entry per source row in
    source order.  ``to_head``: source [B, S/P, H] raster chunk -> [B, H/P, S] tile-major on the
    rank owning the head; otherwise source [B, H/P, S] tile-major -> [B, S/P, H] raster chunk on
    the rank owning the token.
    """
    from .masks import tile_major_permutation

    T, Hh, W = grid
    S = T * Hh * W
    if H % world or S % world:
        raise ValueError("heads and sequence must divide over the ranks")
    Hl, Sl = H // world, S // world
    perm = tile_major_permutation(grid, tile)          # perm[tile_major_pos] = raster_pos
    inv = torch.argsort(perm)                          # inv[raster_pos] = tile_major_pos
    if to_head:
        b, sl, h = torch.meshgrid(torch.arange(B), torch.arange(Sl), torch.arange(H), indexing="ij")
        dest = h // Hl
        row = (b * Hl + (h - dest * Hl)) * S + inv[rank * Sl + sl]
    else:
        b, hl, s = torch.meshgrid(torch.arange(B), torch.arange(Hl), torch.arange(S), indexing="ij")
        r = perm[s]
        dest = r // Sl
        row = (b * Sl + (r - dest * Sl)) * H + rank * Hl + hl
    return dest.reshape(-1), row.reshape(-1)


class _RawDeviceMemory:
    """Device memory owned elsewhere, exposed to torch through the CUDA array interface."""

    def __init__(self, ptr: int, n_elems: int):
        self.__cuda_array_interface__ = {"shape": (n_elems,), "typestr": "<i2", "data": (ptr, False),
                                         "version": 2, "strides": None}


class PeerExchange:
    """Sequence <-> head exchange fused with the raster <-> tile-major token reorder.

    Every rank holds ``[B, S/P, H, 128]`` (bf16, raster (t, h, w) token order, its contiguous
    chunk of the sequence) and needs ``[B, H/P, S, 128]`` for its heads with tokens in tile-major
    order.  One kernel per rank stores each row straight into its final place in the owning
    rank's buffer over NVLink (``fba_peer_exchange``); there is no pack, unpack, transpose or
    permutation pass on either side.  NCCL is used only for two one-element all-reduces that
    order the stores against the readers on the other GPUs.

    The destination buffers (``slots`` per direction, so that q, k and v can be in flight
    together) are allocated once and shared through CUDA IPC.  The tensors returned by
    ``seq_to_head`` / ``head_to_seq`` ALIAS those buffers: they stay valid until the next call
    with the same slot and direction.  Collective: every rank of ``group`` must make the same
    calls in the same order.  Call ``close()`` (collective) when done.
    """

    def __init__(self, B: int, H: int, grid, tile=(1, 1, 1), group=None, device=None, slots: int = 1):
        import ctypes

        from . import _cabi

        self._lib = _cabi.lib()
        self._check = _cabi.check
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.B, self.H, self.grid, self.tile = B, H, tuple(grid), tuple(tile)
        T, Hh, W = self.grid
        self.S = T * Hh * W
        if H % self.world or self.S % self.world:
            raise ValueError("heads and sequence must divide over the ranks")
        if self.world > 16:
            raise ValueError("at most 16 ranks")
        self.Hl, self.Sl = H // self.world, self.S // self.world
        self._n_elems = B * self.Hl * self.S * 128          # same count for both layouts
        self.slots = slots
        self._own, self._peer_ptrs, self._opened = [], [], []
        self._closed = False
        handles = []
        with torch.cuda.device(self.device):
            for _ in range(2 * slots):                       # [to_head slots..., to_seq slots...]
                p = ctypes.c_void_p()
                self._check(self._lib.fba_peer_alloc(self._n_elems * 2, ctypes.byref(p)), "fba_peer_alloc")
                self._own.append(p.value)
                h = ctypes.create_string_buffer(64)
                self._check(self._lib.fba_peer_export(p.value, h), "fba_peer_export")
                handles.append(h.raw)
            gathered = [None] * self.world
            dist.all_gather_object(gathered, handles, group=group)
            for i in range(2 * slots):
                ptrs = (ctypes.c_void_p * self.world)()
                for r in range(self.world):
                    if r == self.rank:
                        ptrs[r] = self._own[i]
                    else:
                        p = ctypes.c_void_p()
                        self._check(self._lib.fba_peer_open(gathered[r][i], ctypes.byref(p)), "fba_peer_open")
                        self._opened.append(p.value)
                        ptrs[r] = p.value
                self._peer_ptrs.append(ptrs)
            self._flag = torch.zeros(1, device=self.device)
            self._views = [torch.as_tensor(_RawDeviceMemory(p, self._n_elems), device=self.device).view(torch.bfloat16)
                           for p in self._own]
        self._barrier()

    def _barrier(self):
        # stream-ordered on every rank: completes only after all ranks' earlier work on their
        # current streams has completed
        dist.all_reduce(self._flag, group=self.group)

    def _run(self, x, to_head: bool, slot: int):
        if self._closed:
            raise RuntimeError("PeerExchange is closed")
        if not 0 <= slot < self.slots:
            raise ValueError(f"slot {slot} out of range")
        want = (self.B, self.Sl, self.H, 128) if to_head else (self.B, self.Hl, self.S, 128)
        if tuple(x.shape) != want or x.dtype != torch.bfloat16 or not x.is_cuda or not x.is_contiguous():
            raise ValueError(f"expected a contiguous CUDA bf16 tensor of shape {want}")
        i = slot if to_head else self.slots + slot
        lo, hi = self._own[i], self._own[i] + self._n_elems * 2
        if lo < x.data_ptr() + x.numel() * 2 and x.data_ptr() < hi:
            raise ValueError("the source tensor lies inside the destination slot of this exchange; clone it or use "
                             "another slot")
        T, Hh, W = self.grid
        self._barrier()
        with torch.cuda.device(self.device):
            rc = self._lib.fba_peer_exchange(x.data_ptr(), self._peer_ptrs[i], self.world, self.rank, self.B, self.H,
                                             T, Hh, W, self.tile[0], self.tile[1], self.tile[2], 1 if to_head else 0,
                                             torch.cuda.current_stream(self.device).cuda_stream)
        self._check(rc, "fba_peer_exchange")
        self._barrier()
        shape = (self.B, self.Hl, self.S, 128) if to_head else (self.B, self.Sl, self.H, 128)
        return self._views[i].view(shape)

    def seq_to_head(self, x: torch.Tensor, slot: int = 0) -> torch.Tensor:
        """[B, S/P, H, 128] raster chunk -> [B, H/P, S, 128] tile-major, local heads (aliases slot)."""
        return self._run(x, True, slot)

    def head_to_seq(self, y: torch.Tensor, slot: int = 0) -> torch.Tensor:
        """[B, H/P, S, 128] tile-major, local heads -> [B, S/P, H, 128] raster chunk (aliases slot)."""
        return self._run(y, False, slot)

    def close(self):
        """Unmap the peers' buffers and free the local ones (collective; idempotent).  Tensors
        returned earlier must no longer be used."""
        if self._closed:
            return
        self._closed = True
        torch.cuda.synchronize(self.device)
        self._barrier()
        torch.cuda.synchronize(self.device)
        self._views = []
        with torch.cuda.device(self.device):
            for p in self._opened:
                self._lib.fba_peer_close(p)
            self._barrier()   # nobody frees while a peer still has the buffer mapped
            torch.cuda.synchronize(self.device)
            for p in self._own:
                self._lib.fba_peer_free(p)
        self._opened, self._own = [], []


class _PeerSeqToHead(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ex, slot, grad_slot, keep):
        ctx.ex, ctx.grad_slot = ex, grad_slot
        y = ex.seq_to_head(x.contiguous(), slot)
        # `keep`: the result will be saved for a backward pass.  The slot is raw peer-written memory
        # that the next exchange through it overwrites behind autograd's back (no version counter
        # sees those stores), so what outlives this call must be a private copy.
        return y.clone() if keep else y

    @staticmethod
    def backward(ctx, g):
        # cloned: autograd may keep the returned tensor as the leaf's .grad, and the slot is reused
        return ctx.ex.head_to_seq(g.contiguous(), ctx.grad_slot).clone(), None, None, None, None


class _PeerHeadToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ex, slot, grad_slot, keep):
        ctx.ex, ctx.grad_slot = ex, grad_slot
        y = ex.head_to_seq(x.contiguous(), slot)
        return y.clone() if keep else y

    @staticmethod
    def backward(ctx, g):
        # consumed at once by the attention backward (which copies nothing out of it after it
        # returns), so the slot view is enough here
        return ctx.ex.seq_to_head(g.contiguous(), ctx.grad_slot), None, None, None, None


def ulysses_tile_major_attn(q, k, v, q_block_size, kv_block_size, mask_fn: Callable, exchange: PeerExchange,
                            attn_fn: Optional[Callable] = None):
    """Block-sparse attention for sequence-sharded activations in their native layout.

    q, k, v: [B, S/P, H, 128] bf16, this rank's contiguous chunk of the raster-order (t, h, w)
    sequence with all heads (self-attention: q and k/v have the same heads and length).  The
    fused peer exchange delivers [B, H/P, S, 128] in the tile-major order of ``exchange``;
    ``mask_fn(q_h, k_h)`` returns the block mask (or ``SparseLists``) for the local heads in that
    order; the output comes back as [B, S/P, H, 128] raster order.  Differentiable: the gradients
    take the same two kernels in the opposite direction.  ``exchange`` needs at least 4 slots
    (q, k, v and dO travel towards the heads; O, dQ, dK, dV back).

    Lifetime of the exchanged tensors: with grad mode on, the head-major q, k, v that the attention
    saves for its backward and the returned output are private copies, so any number of layers (or
    micro-batches, or checkpointed recomputations) may share one ``exchange``.  Without grad mode
    nothing is saved; the inputs of the attention and the returned output then ALIAS the exchange's
    slots and are valid until the next call through the same ``exchange``.
    """
    if exchange.slots < 4:
        raise ValueError("ulysses_tile_major_attn needs a PeerExchange with at least 4 slots")
    if attn_fn is None:
        from .interface import flex_block_attn_func as attn_fn  # noqa: N813
    keep = torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v))
    qh = _PeerSeqToHead.apply(q, exchange, 0, 1, keep)
    kh = _PeerSeqToHead.apply(k, exchange, 1, 2, keep)
    vh = _PeerSeqToHead.apply(v, exchange, 2, 3, keep)
    with torch.no_grad():
        mask = mask_fn(qh, kh)
    oh = attn_fn(qh, kh, vh, q_block_size, kv_block_size, mask)
    return _PeerHeadToSeq.apply(oh, exchange, 0, 3, keep)
