"""CPU, world_size 2 over gloo: head sharding and the Ulysses sequence<->head exchange are exact
re-layouts, forward and backward, and compose with an attention function into the same result as
one process computing everything."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _cpu_attn(q, k, v, qb, kb, mask):
    from oracle import dense_oracle as orc

    return orc.sdpa_dense(q, k, v, mask, qb, kb)


def _worker(rank, world, port, ret):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flex_block_attn_b200 import dist as fd

        assert fd.head_shard(24, world, rank) == slice(rank * 12, rank * 12 + 12)
        B, H, S, D = 2, 4, 6 * 32, 128
        g = torch.Generator().manual_seed(0)
        full = [torch.randn((B, H, S, D), generator=g) for _ in range(4)]  # q k v do, same on all ranks
        Sl = S // world
        loc = [t[:, :, rank * Sl:(rank + 1) * Sl].clone() for t in full]
        # exchange is an exact re-layout
        qh = fd.seq_to_head(loc[0])
        hs = fd.head_shard(H, world, rank)
        assert torch.equal(qh, full[0][:, hs])
        assert torch.equal(fd.head_to_seq(qh), loc[0])
        # composed operator == single-process result, forward and backward
        mask = (torch.rand((6, 6), generator=g) < 0.5) | torch.eye(6, dtype=torch.bool)
        ql, kl, vl = (t.clone().requires_grad_() for t in loc[:3])
        o = fd.ulysses_flex_block_attn(ql, kl, vl, 32, 32, lambda qh_, kh_: mask, attn_fn=_cpu_attn)
        o.backward(loc[3])
        qf, kf, vf = (t.clone().requires_grad_() for t in full[:3])
        of = _cpu_attn(qf, kf, vf, 32, 32, mask)
        of.backward(full[3])
        sl = slice(rank * Sl, (rank + 1) * Sl)
        assert torch.allclose(o, of[:, :, sl], atol=1e-5)
        assert torch.allclose(ql.grad, qf.grad[:, :, sl], atol=1e-5)
        assert torch.allclose(kl.grad, kf.grad[:, :, sl], atol=1e-5)
        assert torch.allclose(vl.grad, vf.grad[:, :, sl], atol=1e-5)

        # the autograd wiring of the native-layout path ([B, S/P, H, D] raster in and out), with a
        # stand-in for PeerExchange that does the same re-layout over gloo
        from flex_block_attn_b200.masks import tile_major_permutation

        grid, tile = (2, 4, 24), (1, 4, 8)                 # S = 192, tiles of 32 tokens
        perm = tile_major_permutation(grid, tile)
        inv = torch.argsort(perm)

        class GlooExchange:
            slots = 4

            def seq_to_head(self, x, slot=0):             # [B, S/P, H, D] raster -> [B, H/P, S, D] tile-major
                return fd.seq_to_head(x.transpose(1, 2).contiguous())[:, :, perm].contiguous()

            def head_to_seq(self, y, slot=0):
                return fd.head_to_seq(y[:, :, inv].contiguous()).transpose(1, 2).contiguous()

        raster = [t.transpose(1, 2).contiguous() for t in full]             # [B, S, H, D]
        rl = [t[:, sl].clone() for t in raster]
        q2, k2, v2 = (t.clone().requires_grad_() for t in rl[:3])
        o2 = fd.ulysses_tile_major_attn(q2, k2, v2, 32, 32, lambda qh_, kh_: mask, GlooExchange(), attn_fn=_cpu_attn)
        o2.backward(rl[3])
        qt, kt, vt = (t[:, :, perm].clone().requires_grad_() for t in full[:3])   # tile-major, all heads
        ot = _cpu_attn(qt, kt, vt, 32, 32, mask)
        ot.backward(full[3][:, :, perm])
        back = lambda t: t[:, :, inv].transpose(1, 2)[:, sl]                 # -> this rank's raster chunk
        assert torch.allclose(o2, back(ot.detach()), atol=1e-5)
        assert torch.allclose(q2.grad, back(qt.grad), atol=1e-5)
        assert torch.allclose(k2.grad, back(kt.grad), atol=1e-5)
        assert torch.allclose(v2.grad, back(vt.grad), atol=1e-5)

        # Two chained layers through ONE exchange whose results alias per-slot buffers, as the real
        # PeerExchange's do: the second layer's exchanges overwrite the slots the first layer's q, k,
        # v came from.  Autograd cannot see such stores, so the wiring must have kept private copies.
        class AliasingExchange(GlooExchange):
            def __init__(self):
                self.to_head, self.to_seq = {}, {}

            def seq_to_head(self, x, slot=0):
                y = GlooExchange.seq_to_head(self, x, slot)
                buf = self.to_head.setdefault(slot, torch.empty_like(y))
                buf.copy_(y)
                return buf

            def head_to_seq(self, y, slot=0):
                x = GlooExchange.head_to_seq(self, y, slot)
                buf = self.to_seq.setdefault(slot, torch.empty_like(x))
                buf.copy_(x)
                return buf

        ex = AliasingExchange()
        q3, k3, v3 = (t.clone().requires_grad_() for t in rl[:3])
        h1 = fd.ulysses_tile_major_attn(q3, k3, v3, 32, 32, lambda qh_, kh_: mask, ex, attn_fn=_cpu_attn)
        h2 = fd.ulysses_tile_major_attn(h1, k3 * 0.5, v3 + 1.0, 32, 32, lambda qh_, kh_: mask, ex, attn_fn=_cpu_attn)
        h2.backward(rl[3])
        qt, kt, vt = (t[:, :, perm].clone().requires_grad_() for t in full[:3])
        g1 = _cpu_attn(qt, kt, vt, 32, 32, mask)
        g2 = _cpu_attn(g1, kt * 0.5, vt + 1.0, 32, 32, mask)
        g2.backward(full[3][:, :, perm])
        assert torch.allclose(h2, back(g2.detach()), atol=1e-5)
        assert torch.allclose(q3.grad, back(qt.grad), atol=1e-5), "two layers sharing one exchange: dQ"
        assert torch.allclose(k3.grad, back(kt.grad), atol=1e-5), "two layers sharing one exchange: dK"
        assert torch.allclose(v3.grad, back(vt.grad), atol=1e-5), "two layers sharing one exchange: dV"
        ret[rank] = "ok"
    except Exception as e:  # pragma: no cover - surfaced through ret
        ret[rank] = f"{type(e).__name__}: {e}"
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_ulysses_exchange_world2():
    world = 2
    port = _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: "ok", 1: "ok"}


@pytest.mark.parametrize("world,grid,tile", [(2, (2, 4, 4), (1, 2, 2)), (4, (4, 4, 8), (2, 2, 4)), (2, (1, 1, 64), (1, 1, 1))])
def test_peer_exchange_row_map_is_transpose_plus_tile_major(world, grid, tile):
    """The row map of the fused peer exchange, emulated for all ranks in one process: scattering
    every rank's [B, S/P, H] raster chunk by it gives transpose + tile-major permutation + head
    sharding; the way back restores the chunks."""
    from flex_block_attn_b200.dist import peer_exchange_rows
    from flex_block_attn_b200.masks import tile_major_permutation

    B, H, D = 2, 4, 3
    S = grid[0] * grid[1] * grid[2]
    Hl, Sl = H // world, S // world
    x = torch.arange(B * S * H * D, dtype=torch.float32).reshape(B, S, H, D)      # global, raster order
    want_heads = x.transpose(1, 2)[:, :, tile_major_permutation(grid, tile)]     # [B, H, S, D] tile-major
    head_bufs = [torch.full((B * Hl * S, D), -1.0) for _ in range(world)]
    for r in range(world):
        chunk = x[:, r * Sl:(r + 1) * Sl].reshape(-1, D)
        dest, row = peer_exchange_rows(r, world, B, H, grid, tile, True)
        assert dest.numel() == chunk.shape[0]
        for d in range(world):
            sel = dest == d
            head_bufs[d][row[sel]] = chunk[sel]
    for r in range(world):
        assert torch.equal(head_bufs[r].reshape(B, Hl, S, D), want_heads[:, r * Hl:(r + 1) * Hl])
    seq_bufs = [torch.full((B * Sl * H, D), -1.0) for _ in range(world)]
    for r in range(world):
        src = head_bufs[r]
        dest, row = peer_exchange_rows(r, world, B, H, grid, tile, False)
        for d in range(world):
            sel = dest == d
            seq_bufs[d][row[sel]] = src[sel]
    for r in range(world):
        assert torch.equal(seq_bufs[r].reshape(B, Sl, H, D), x[:, r * Sl:(r + 1) * Sl])
