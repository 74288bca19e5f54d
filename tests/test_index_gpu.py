"""GPU: the compaction kernels must be bit-identical to the nonzero()-based oracle."""
import pytest
import torch

from oracle import dense_oracle as orc
from tests.util import bernoulli_mask, reference_rule_mask

pytestmark = pytest.mark.gpu


def _masks():
    yield "2d_4x4", bernoulli_mask((4, 4), 0.5, 0)
    yield "2d_1x1", torch.ones((1, 1), dtype=torch.bool)
    yield "2d_rule_48x12", reference_rule_mask(48, 12)
    yield "2d_allfalse_row", torch.tensor([[1, 0, 1], [0, 0, 0], [1, 1, 1]], dtype=torch.bool)
    yield "2d_alltrue_80", torch.ones((80, 80), dtype=torch.bool)
    for n in (31, 32, 33, 180):
        yield f"4d_{n}", bernoulli_mask((1, 3, n, n), 0.4, n)
    yield "4d_540x180", bernoulli_mask((2, 3, 540, 180), 0.1, 7)
    yield "4d_empty", torch.zeros((1, 2, 5, 7), dtype=torch.bool)


@pytest.mark.parametrize("name,mask", list(_masks()), ids=[n for n, _ in _masks()])
def test_build_index_bit_exact(name, mask):
    import flex_block_attn_b200 as fba

    got = fba.build_index(mask.cuda())
    want = orc.block_index_oracle(mask)
    for g, w, nm in zip(got, want, ("q2k_idx", "q2k_cnt", "k2q_idx", "k2q_cnt")):
        assert g.dtype == torch.int32
        assert torch.equal(g.cpu(), w), (name, nm)


@pytest.mark.parametrize("qb,kb,nQ,nK", [(16, 64, 24, 6), (32, 128, 20, 5), (64, 384, 12, 2), (48, 192, 7, 2),
                                         (64, 64, 3, 3), (192, 64, 2, 6), (16, 384, 48, 2)])
@pytest.mark.parametrize("dim", [2, 4])
def test_build_tile_lists_bit_exact(qb, kb, nQ, nK, dim):
    import flex_block_attn_b200 as fba

    Sq, Skv = qb * nQ, kb * nK
    shape = (nQ, nK) if dim == 2 else (2, 2, nQ, nK)
    mask = bernoulli_mask(shape, 0.5, seed=qb + kb + dim)
    lists = fba.build_lists(mask.cuda(), qb, kb, Sq, Skv, need_bwd=True)
    assert not lists.aligned
    want = orc.tile_lists_oracle(mask, qb, kb, Sq, Skv)
    got = (lists.fwd_idx, lists.fwd_cnt, lists.fwd_msk, lists.bwd_idx, lists.bwd_cnt, lists.bwd_msk)
    for g, w, nm in zip(got, want, ("fwd_idx", "fwd_cnt", "fwd_msk", "bwd_idx", "bwd_cnt", "bwd_msk")):
        gi = g.cpu().to(torch.int32)
        if nm.endswith("msk"):
            gi = gi & 0xFFFF
        assert torch.equal(gi, w), (nm, gi, w)
