"""GPU: the list-emitting mask builders (fba_sta_index, fba_ssta_index) against the mask definitions
in oracle/mask_oracle.py and the nonzero()-based list oracle; the package's own torch builders
(flex_block_attn_b200/masks.py) are held to the same definitions."""
import pytest
import torch

from oracle import dense_oracle as orc
from oracle import mask_oracle as mo
from tests.util import rand_qkv

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("grid,window", [((3, 6, 10), (1, 1, 1)), ((1, 1, 5), (0, 0, 2)), ((2, 3, 4), (1, 0, 1)),
                                         ((4, 4, 4), (3, 3, 3))])
def test_sta_lists_equal_compacted_mask(grid, window):
    import flex_block_attn_b200 as fba
    from flex_block_attn_b200 import masks

    lists = fba.sta_lists(grid, window, tile_tokens=384)
    mask = mo.sta_mask(grid, window)
    assert torch.equal(masks.sta_mask(grid, window, device="cpu"), mask)
    q2k_idx, q2k_cnt, k2q_idx, k2q_cnt = orc.block_index_oracle(mask)
    assert torch.equal(lists.fwd_idx.cpu(), q2k_idx) and torch.equal(lists.fwd_cnt.cpu(), q2k_cnt)
    assert torch.equal(lists.bwd_idx.cpu(), k2q_idx) and torch.equal(lists.bwd_cnt.cpu(), k2q_cnt)


def test_sta_lists_drive_the_operator():
    import flex_block_attn_b200 as fba
    from flex_block_attn_b200 import masks

    grid = (2, 2, 3)
    S = 12 * 384
    q, k, v, do = rand_qkv(1, 2, 2, S, S, seed=90, device="cuda")
    outs = []
    for bm in (masks.sta_mask(grid), fba.sta_lists(grid)):
        qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
        o = fba.flex_block_attn_func(qq, kk, vv, 384, 384, bm)
        o.backward(do)
        outs.append((o.detach(), qq.grad, kk.grad, vv.grad))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][2], outs[1][2]) and torch.equal(outs[0][3], outs[1][3])
    assert (outs[0][1].float() - outs[1][1].float()).abs().max().item() <= 1e-2


@pytest.mark.parametrize("B,Hq,Hkv,grid,qb,kb,topk", [(1, 2, 2, (1, 2, 4), 128, 384, 2), (2, 4, 2, (3, 2, 2), 128, 384, 3),
                                                     (1, 2, 2, (3, 6, 10), 128, 384, 8), (1, 1, 1, (1, 1, 6), 384, 384, 6)])
def test_ssta_lists_match_torch_builder(B, Hq, Hkv, grid, qb, kb, topk):
    import flex_block_attn_b200 as fba
    from flex_block_attn_b200 import masks

    n_tiles = grid[0] * grid[1] * grid[2]
    S = n_tiles * kb
    q, k, _, _ = rand_qkv(B, Hq, Hkv, S, S, seed=91 + topk, device="cuda")
    lists, mask = fba.ssta_lists(q, k, grid, qb, kb, topk=topk)
    want = mo.ssta_mask(q, k, grid, qb, kb, topk=topk)
    assert torch.equal(masks.ssta_mask(q, k, grid, qb, kb, topk=topk), want)
    assert mask.shape == want.shape and mask.dtype == torch.bool
    # the lists are exactly the compaction of the mask the kernel produced
    q2k_idx, q2k_cnt, k2q_idx, k2q_cnt = orc.block_index_oracle(mask.cpu())
    assert torch.equal(lists.fwd_idx.cpu(), q2k_idx) and torch.equal(lists.fwd_cnt.cpu(), q2k_cnt)
    assert torch.equal(lists.bwd_idx.cpu(), k2q_idx) and torch.equal(lists.bwd_cnt.cpu(), k2q_cnt)
    # and the mask is the definition's; a row may differ only where pooled scores tie to within fp32
    # summation-order noise, every differing row is checked for that, and such rows must be rare
    n_explained = mo.explain_selection_differences(mask, want, mo.pooled_scores(q, k, qb, kb))
    assert n_explained == int((mask != want).any(-1).sum())
    assert n_explained <= 0.01 * mask[..., 0].numel()
    assert bool((mask.sum(-1) >= min(topk, n_tiles)).all())


@pytest.mark.parametrize("qb,kb,topk", [(128, 384, 3), (384, 384, 5), (128, 128, 1)])
def test_moba_lists_match_torch_builder(qb, kb, topk):
    """Top-k selection alone (window switched off): same mask as masks.moba_topk_mask up to
    numerical ties, exactly ``topk`` blocks per row, lists = compaction of the mask, and attention
    over the lists matches the oracle over the mask."""
    import flex_block_attn_b200 as fba
    from flex_block_attn_b200 import masks
    from tests.util import assert_close

    B, Hq, Hkv, S = 1, 4, 2, 3072
    q, k, v, do = rand_qkv(B, Hq, Hkv, S, S, seed=70 + topk, device="cuda")
    lists, mask = fba.moba_lists(q, k, qb, kb, topk)
    want = mo.moba_topk_mask(q, k, qb, kb, topk)
    assert torch.equal(masks.moba_topk_mask(q, k, qb, kb, topk), want)
    assert mask.shape == want.shape and bool((mask.sum(-1) == topk).all())
    n_explained = mo.explain_selection_differences(mask, want, mo.pooled_scores(q, k, qb, kb))
    assert n_explained <= 0.01 * mask[..., 0].numel()
    q2k_idx, q2k_cnt, k2q_idx, k2q_cnt = orc.block_index_oracle(mask.cpu())
    assert torch.equal(lists.fwd_idx.cpu(), q2k_idx) and torch.equal(lists.fwd_cnt.cpu(), q2k_cnt)
    assert torch.equal(lists.bwd_idx.cpu(), k2q_idx) and torch.equal(lists.bwd_cnt.cpu(), k2q_cnt)
    q1, k1, v1 = (t.clone().requires_grad_() for t in (q, k, v))
    o = fba.flex_block_attn_func(q1, k1, v1, qb, kb, lists)
    o.backward(do)
    ref = orc.attention_slab(q.float(), k.float(), v.float(), mask, qb, kb, do.float())
    for g, w, nm in zip((o.detach(), q1.grad, k1.grad, v1.grad), (ref[0], ref[2], ref[3], ref[4]), ("O", "dQ", "dK", "dV")):
        assert_close(g.float(), w, f"moba {nm}")


@pytest.mark.parametrize("grid,tile", [((6, 8, 16), (6, 8, 8)), ((4, 4, 6), (2, 2, 3)), ((18, 48, 80), (6, 8, 8))])
def test_tile_major_layout_change_is_exact(grid, tile):
    from flex_block_attn_b200 import masks

    S = grid[0] * grid[1] * grid[2]
    B, Hn = (1, 2) if S > 10000 else (2, 3)
    g = torch.Generator().manual_seed(S)
    x = torch.randn((B, S, Hn, 128), generator=g).to(torch.bfloat16).cuda()
    perm = masks.tile_major_permutation(grid, tile, device="cuda")
    want = x.transpose(1, 2)[:, :, perm].contiguous()
    got = masks.to_tile_major(x, grid, tile)
    assert got.shape == (B, Hn, S, 128) and torch.equal(got, want)
    back = masks.from_tile_major(got, grid, tile)
    assert torch.equal(back, x)


@pytest.mark.parametrize("world,grid,tile,H", [(2, (2, 8, 8), (2, 4, 4), 8), (4, (3, 8, 16), (3, 4, 8), 8),
                                               (8, (4, 8, 8), (1, 1, 1), 8), (2, (2, 8, 8), (1, 8, 8), 16),
                                               (1, (2, 4, 8), (1, 2, 8), 24), (2, (1, 3, 6), (1, 1, 3), 6)])
def test_peer_exchange_kernel_with_emulated_ranks(world, grid, tile, H):
    """fba_peer_exchange with every "rank" on one GPU (its peer pointers are local buffers): the
    union of all ranks' stores is transpose + tile-major reorder + head sharding, bit for bit, and
    the way back restores every rank's raster chunk."""
    import ctypes

    from flex_block_attn_b200 import _cabi, masks

    lib = _cabi.lib()
    B = 2
    S = grid[0] * grid[1] * grid[2]
    Hl, Sl = H // world, S // world     # covers both row enumerations of the kernel in both directions
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((B, S, H, 128), generator=g, device="cuda").to(torch.bfloat16)
    want = masks.to_tile_major(x, grid, tile)                                   # [B, H, S, 128]
    stream = torch.cuda.current_stream().cuda_stream
    head_bufs = [torch.zeros((B, Hl, S, 128), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[t.data_ptr() for t in head_bufs])
    chunks = [x[:, r * Sl:(r + 1) * Sl].contiguous() for r in range(world)]
    for r in range(world):
        rc = lib.fba_peer_exchange(chunks[r].data_ptr(), ptrs, world, r, B, H, *grid, *tile, 1, stream)
        _cabi.check(rc, "fba_peer_exchange")
    for r in range(world):
        assert torch.equal(head_bufs[r], want[:, r * Hl:(r + 1) * Hl])
    seq_bufs = [torch.zeros((B, Sl, H, 128), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    ptrs2 = (ctypes.c_void_p * world)(*[t.data_ptr() for t in seq_bufs])
    for r in range(world):
        rc = lib.fba_peer_exchange(head_bufs[r].data_ptr(), ptrs2, world, r, B, H, *grid, *tile, 0, stream)
        _cabi.check(rc, "fba_peer_exchange")
    for r in range(world):
        assert torch.equal(seq_bufs[r], chunks[r])
    # argument checks
    assert lib.fba_peer_exchange(chunks[0].data_ptr(), ptrs, 0, 0, B, H, *grid, *tile, 1, stream) == -1
    assert lib.fba_peer_exchange(chunks[0].data_ptr(), ptrs, world, world, B, H, *grid, *tile, 1, stream) == -1
