"""CPU tests that pin the oracle: against the golden vectors produced by the reference's own
oracle code, and against itself (explicit == slab == SDPA; integer list restatements)."""
import pytest
import torch

from oracle import dense_oracle as orc
from tests.util import GOLDEN_CASES, bernoulli_mask, load_golden, rand_qkv, reference_rule_mask


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_explicit_matches_reference_golden(name):
    g = load_golden(name)
    o, lse, dq, dk, dv = orc.attention_explicit(g["q"], g["k"], g["v"], g["block_mask"], g["q_block"],
                                                g["kv_block"], g["do"])
    scale = max(1.0, g["o"].abs().max().item())
    for got, want, nm in ((o, g["o"], "o"), (dq, g["dq"], "dq"), (dk, g["dk"], "dk"), (dv, g["dv"], "dv")):
        tol = 2e-5 * max(1.0, want.abs().max().item())
        assert torch.allclose(got, want, rtol=1e-4, atol=tol), (name, nm, (got - want).abs().max().item(), scale)


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_slab_matches_reference_golden(name):
    g = load_golden(name)
    o, lse, dq, dk, dv = orc.attention_slab(g["q"], g["k"], g["v"], g["block_mask"], g["q_block"],
                                            g["kv_block"], g["do"])
    for got, want, nm in ((o, g["o"], "o"), (dq, g["dq"], "dq"), (dk, g["dk"], "dk"), (dv, g["dv"], "dv")):
        tol = 2e-5 * max(1.0, want.abs().max().item())
        assert torch.allclose(got, want, rtol=1e-4, atol=tol), (name, nm)


def test_config1_explicit_slab_sdpa_agree():
    """Benchmark configuration 1 (the CPU-runnable case): B=1, H=2, S=1536, D=128, 384-blocks, Bernoulli(0.5)|diag mask, fp32."""
    q, k, v, do = rand_qkv(1, 2, 2, 1536, 1536, seed=0, dtype=torch.float32)
    mask = bernoulli_mask((4, 4), 0.5, seed=0)
    qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
    o_ref = orc.sdpa_dense(qr, kr, vr, mask, 384, 384)
    o_ref.backward(do)
    for fn in (orc.attention_explicit, orc.attention_slab):
        o, lse, dq, dk, dv = fn(q, k, v, mask, 384, 384, do)
        assert torch.allclose(o, o_ref, atol=1e-5, rtol=1e-4)
        assert torch.allclose(dq, qr.grad, atol=2e-5, rtol=1e-4)
        assert torch.allclose(dk, kr.grad, atol=2e-5, rtol=1e-4)
        assert torch.allclose(dv, vr.grad, atol=2e-5, rtol=1e-4)


def test_softmax_scale_explicit_slab_sdpa_agree():
    """The optional softmax_scale of the three oracle forms means the same thing (SDPA's ``scale``)."""
    q, k, v, do = rand_qkv(1, 2, 1, 768, 768, seed=3, dtype=torch.float32)
    mask = bernoulli_mask((1, 2, 6, 6), 0.5, seed=3)
    qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
    o_ref = orc.sdpa_dense(qr, kr, vr, mask, 128, 128, softmax_scale=0.2)
    o_ref.backward(do)
    for fn in (orc.attention_explicit, orc.attention_slab):
        o, lse, dq, dk, dv = fn(q, k, v, mask, 128, 128, do, softmax_scale=0.2)
        assert torch.allclose(o, o_ref, atol=1e-5, rtol=1e-4)
        assert torch.allclose(dq, qr.grad, atol=5e-5, rtol=1e-4)
        assert torch.allclose(dk, kr.grad, atol=5e-5, rtol=1e-4)
        assert torch.allclose(dv, vr.grad, atol=5e-5, rtol=1e-4)
    o_default = orc.attention_slab(q, k, v, mask, 128, 128)[0]
    assert not torch.allclose(o_default, o_ref, atol=1e-3)


def test_gqa_4d_mask_and_asymmetric_blocks():
    q, k, v, do = rand_qkv(2, 4, 2, 256, 384, seed=3, dtype=torch.float32)
    mask = bernoulli_mask((2, 4, 256 // 32, 384 // 128), 0.5, seed=4)
    a = orc.attention_explicit(q, k, v, mask, 32, 128, do)
    b = orc.attention_slab(q, k, v, mask, 32, 128, do)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, atol=2e-5, rtol=1e-4)
    qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
    o_ref = orc.sdpa_dense(qr, kr, vr, mask, 32, 128)
    o_ref.backward(do)
    assert torch.allclose(a[0], o_ref, atol=1e-5, rtol=1e-4)
    assert torch.allclose(a[3], kr.grad, atol=2e-5, rtol=1e-4)


def test_dead_rows_are_zero():
    q, k, v, do = rand_qkv(1, 1, 1, 256, 256, seed=5, dtype=torch.float32)
    mask = torch.tensor([[True, False], [False, False]])
    o, lse, dq, dk, dv = orc.attention_explicit(q, k, v, mask, 128, 128, do)
    assert (o[:, :, 128:] == 0).all() and torch.isinf(lse[:, :, 128:]).all()
    assert (dq[:, :, 128:] == 0).all() and (dk[:, :, 128:] == 0).all()
    assert torch.isfinite(dq).all() and torch.isfinite(dk).all() and torch.isfinite(dv).all()


def test_index_lists_by_hand():
    m = torch.tensor([[1, 0, 1, 1], [0, 0, 0, 0], [0, 1, 0, 0]], dtype=torch.bool)
    q2k_idx, q2k_cnt, k2q_idx, k2q_cnt = orc.block_index_oracle(m)
    assert q2k_idx.tolist() == [[0, 2, 3, -1], [-1, -1, -1, -1], [1, -1, -1, -1]]
    assert q2k_cnt.tolist() == [3, 0, 1]
    assert k2q_idx.tolist() == [[0, -1, -1], [2, -1, -1], [0, -1, -1], [0, -1, -1]]
    assert k2q_cnt.tolist() == [1, 1, 1, 1]


def test_tile_words_by_loops():
    q_block, kv_block, Sq, Skv = 48, 192, 48 * 7, 192 * 2
    m = reference_rule_mask(7, 2)
    w = orc.tile_mask_words(m, q_block, kv_block, Sq, Skv)
    n_mt, n_nt = (Sq + 127) // 128, (Skv + 127) // 128
    assert tuple(w.shape) == (n_mt, n_nt)
    for mt in range(n_mt):
        for nt in range(n_nt):
            exp = 0
            for h in range(2):
                for g in range(8):
                    r, c = mt * 128 + g * 16, nt * 128 + h * 64
                    if r < Sq and c < Skv and m[r // q_block, c // kv_block]:
                        exp |= 1 << (8 * h + g)
            assert int(w[mt, nt]) == exp
    fi, fc, fm, bi, bc, bm = orc.tile_lists_oracle(m, q_block, kv_block, Sq, Skv)
    assert fi.shape == (n_mt, n_nt) and bi.shape == (n_nt, n_mt)
    assert int(fc.sum()) == int(bc.sum()) == int((w != 0).sum())


# ------------------------------------------------------------------------------------------------
# Structured-mask definitions and the work-item order (oracle/mask_oracle.py)
# ------------------------------------------------------------------------------------------------
def test_sta_mask_by_hand():
    from oracle import mask_oracle as mo

    # 1 x 2 x 3 grid of tiles, ids 0 1 2 / 3 4 5; window (0, 1, 1): neighbours in h and w
    m = mo.sta_mask_loops((1, 2, 3), (0, 1, 1))
    assert m.int().tolist() == [[1, 1, 0, 1, 1, 0], [1, 1, 1, 1, 1, 1], [0, 1, 1, 0, 1, 1],
                                [1, 1, 0, 1, 1, 0], [1, 1, 1, 1, 1, 1], [0, 1, 1, 0, 1, 1]]
    # window (0, 0, 1) on a 1 x 1 x 4 line is tridiagonal
    assert mo.sta_mask_loops((1, 1, 4), (0, 0, 1)).int().tolist() == [[1, 1, 0, 0], [1, 1, 1, 0], [0, 1, 1, 1], [0, 0, 1, 1]]
    for grid, win in (((3, 6, 10), (1, 1, 1)), ((2, 3, 4), (1, 0, 1)), ((4, 4, 4), (3, 3, 3))):
        assert torch.equal(mo.sta_mask(grid, win), mo.sta_mask_loops(grid, win))


def test_moba_and_ssta_masks_by_hand():
    from oracle import mask_oracle as mo

    # one head, 2 query blocks of 16 rows, 3 key blocks of 64 rows, every row of a block equal, so the
    # pooled vectors are the rows themselves: q0 = e0, q1 = e1; k0 = 3 e0, k1 = 2 e0 + 5 e1, k2 = e1
    D = 128
    e = torch.eye(D)
    q = torch.cat([e[0].expand(16, D), e[1].expand(16, D)])[None, None]
    k = torch.cat([(3 * e[0]).expand(64, D), (2 * e[0] + 5 * e[1]).expand(64, D), e[1].expand(64, D)])[None, None]
    score = mo.pooled_scores(q, k, 16, 64)
    assert score[0, 0].tolist() == [[3.0, 2.0, 0.0], [0.0, 5.0, 1.0]]
    assert mo.moba_topk_mask(q, k, 16, 64, 1)[0, 0].int().tolist() == [[1, 0, 0], [0, 1, 0]]
    assert mo.moba_topk_mask(q, k, 16, 64, 2)[0, 0].int().tolist() == [[1, 1, 0], [0, 1, 1]]
    assert torch.equal(mo.moba_topk_mask_loops(q, k, 16, 64, 2), mo.moba_topk_mask(q, k, 16, 64, 2))
    # SSTA: kv_block 64 = one tile, q_block 16 -> both query blocks sit in tile 0 of a 1 x 1 x 3 line;
    # window (0, 0, 1) adds tiles {0, 1} to both rows
    m = mo.ssta_mask(q, k, (1, 1, 3), 16, 64, topk=1, window=(0, 0, 1))
    assert m[0, 0].int().tolist() == [[1, 1, 0], [1, 1, 0]]
    assert torch.equal(m, mo.ssta_mask_loops(q, k, (1, 1, 3), 16, 64, 1, (0, 0, 1)))
    # random inputs, grouped-query heads: loops == vectorised
    g = torch.Generator().manual_seed(1)
    q = torch.randn((2, 4, 96, D), generator=g)
    k = torch.randn((2, 2, 192, D), generator=g)
    assert torch.equal(mo.moba_topk_mask_loops(q, k, 32, 64, 2), mo.moba_topk_mask(q, k, 32, 64, 2))
    assert torch.equal(mo.ssta_mask_loops(q[:, :, :96], k, (1, 3, 1), 32, 64, 1, (0, 1, 0)),
                       mo.ssta_mask(q[:, :, :96], k, (1, 3, 1), 32, 64, 1, (0, 1, 0)))
    # the package's own torch builders state the same definitions
    from flex_block_attn_b200 import masks

    assert torch.equal(masks.moba_topk_mask(q, k, 32, 64, 2), mo.moba_topk_mask(q, k, 32, 64, 2))
    assert torch.equal(masks.sta_mask((2, 3, 4), (1, 0, 1), device="cpu"), mo.sta_mask((2, 3, 4), (1, 0, 1)))


def test_work_order_by_hand():
    from oracle import mask_oracle as mo

    # shared list, one tile per item: descending, ties keep index order
    assert mo.work_order(torch.tensor([3, 1, 3, 0, 2, 2]), 6, False, 1, 1, 6, 1, 1).tolist() == [[0, 2, 4, 5, 1, 3]]
    # forward items are tile pairs; 5 tiles, rows_div 1: keys (3+1, 3+0, 2) -> order 0, 1, 2
    assert mo.work_order(torch.tensor([3, 1, 3, 0, 2]), 5, False, 1, 1, 5, 2, 1).tolist() == [[0, 1, 2]]
    # 384-row blocks (rows_div 3), 6 tiles, pairs (0,1) (2,3) (4,5): keys (2a, a+b, 2b) with a=1, b=4
    assert mo.work_order(torch.tensor([1, 4]), 2, False, 1, 3, 6, 2, 1).tolist() == [[2, 1, 0]]
    # per-head list, two kv heads with two query heads each: keys are sums over the group
    cnt = torch.tensor([1, 5,  4, 0,   2, 2,  0, 9])   # heads 0..3, 2 rows each
    assert mo.work_order(cnt, 2, True, 2, 1, 2, 1, 2).tolist() == [[0, 1], [1, 0]]
