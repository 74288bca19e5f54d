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
