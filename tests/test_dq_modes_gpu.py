"""GPU: the two dQ strategies of the backward.  "atomic" (key-major kernel + fp32 reductions) is the
default everywhere else in the suite; here the query-major pass ("qmajor") is held to the same
oracle and tolerances on the same cases, dK / dV must not depend on the mode, and in query-major
mode dQ must be bit-reproducible."""
import pytest
import torch

from oracle import dense_oracle as orc
from tests.util import assert_close, bernoulli_mask, rand_qkv

pytestmark = pytest.mark.gpu

CASES = {
    # name: (B, Hq, Hkv, Sq, Skv, qb, kb, mask shape, keep)
    "c1_2d": (1, 2, 2, 1536, 1536, 384, 384, (4, 4), 0.5),
    "c3_like": (1, 3, 3, 3840, 3840, 384, 384, (1, 3, 10, 10), 0.4),
    "c5_like": (2, 2, 2, 3072, 3072, 128, 384, (2, 2, 24, 8), 0.4),
    "gqa": (2, 4, 2, 1024, 768, 128, 384, (2, 4, 8, 2), 0.5),
    "cross": (1, 2, 2, 512, 1280, 128, 128, (4, 10), 0.4),
    "tile_mask_64_192": (1, 4, 2, 1536, 1536, 64, 192, (1, 4, 24, 8), 0.5),
    "tile_mask_16_64": (1, 1, 1, 768, 768, 16, 64, (48, 12), 0.3),
    "q_gt_kv": (1, 1, 1, 384, 384, 192, 64, (2, 6), 0.5),
    "ragged": (1, 1, 1, 336, 384, 48, 192, (7, 2), 0.6),
    "odd_tiles": (1, 2, 2, 640, 640, 128, 128, (1, 2, 5, 5), 0.5),
}


def _run(case, mode, seed=0):
    import flex_block_attn_b200 as fba

    B, Hq, Hkv, Sq, Skv, qb, kb, mshape, keep = CASES[case]
    q, k, v, do = rand_qkv(B, Hq, Hkv, Sq, Skv, seed=100 + seed, device="cuda")
    mask = bernoulli_mask(mshape, keep, 100 + seed).cuda()
    lists = fba.build_lists(mask, qb, kb, Sq, Skv, need_bwd=True)
    o, lse = fba.forward_with_lists(q, k, v, lists)
    dq, dk, dv = fba.backward_with_lists(q, k, v, o, lse, do, lists, dq_mode=mode)
    torch.cuda.synchronize()
    fba.check_status()
    return (q, k, v, do, mask, qb, kb), (dq, dk, dv)


@pytest.mark.parametrize("case", list(CASES))
def test_query_major_dq_against_oracle(case):
    (q, k, v, do, mask, qb, kb), got = _run(case, "qmajor")
    want = orc.attention_slab(q.float(), k.float(), v.float(), mask, qb, kb, do.float())
    for g, w, nm in zip(got, want[2:], ("dQ", "dK", "dV")):
        assert_close(g.float(), w, f"qmajor {case} {nm}")


@pytest.mark.parametrize("case", ["c3_like", "gqa", "tile_mask_64_192", "ragged"])
def test_modes_agree_and_query_major_is_bit_reproducible(case):
    _, a = _run(case, "atomic")
    _, b = _run(case, "qmajor")
    _, c = _run(case, "qmajor")
    assert torch.equal(a[1], b[1]) and torch.equal(a[2], b[2]), "dK / dV depend on the dQ mode"
    assert torch.equal(b[0], c[0]) and torch.equal(b[1], c[1]) and torch.equal(b[2], c[2])
    assert_close(a[0].float(), b[0].float(), f"dQ atomic vs qmajor {case}", max_abs=1e-2)


def test_dead_rows_in_query_major_mode():
    import flex_block_attn_b200 as fba

    q, k, v, do = rand_qkv(1, 1, 1, 512, 512, seed=8, device="cuda")
    m = bernoulli_mask((1, 1, 4, 4), 0.5, 8)
    m[0, 0, 2, :] = False
    m[0, 0, :, 1] = False
    m = m.cuda()
    lists = fba.build_lists(m, 128, 128, 512, 512, need_bwd=True)
    o, lse = fba.forward_with_lists(q, k, v, lists)
    dq, dk, dv = fba.backward_with_lists(q, k, v, o, lse, do, lists, dq_mode="qmajor")
    assert (dq[:, :, 256:384] == 0).all() and (dk[:, :, 128:256] == 0).all() and (dv[:, :, 128:256] == 0).all()
    want = orc.attention_slab(q.float(), k.float(), v.float(), m, 128, 128, do.float())
    for g, w, nm in zip((dq, dk, dv), want[2:], ("dQ", "dK", "dV")):
        assert_close(g.float(), w, f"qmajor dead {nm}")


def test_autograd_uses_the_mode_from_the_environment(monkeypatch):
    import flex_block_attn_b200 as fba

    monkeypatch.setenv("FBA_DQ_MODE", "qmajor")
    q, k, v, do = rand_qkv(1, 2, 2, 1536, 1536, seed=3, device="cuda")
    mask = bernoulli_mask((1, 2, 4, 4), 0.5, 3).cuda()
    grads = []
    for _ in range(2):
        qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
        fba.flex_block_attn_func(qq, kk, vv, 384, 384, mask).backward(do)
        grads.append(qq.grad)
    assert torch.equal(grads[0], grads[1])
    want = orc.attention_slab(q.float(), k.float(), v.float(), mask, 384, 384, do.float())
    assert_close(grads[0].float(), want[2], "qmajor through autograd dQ")
    monkeypatch.setenv("FBA_DQ_MODE", "bogus")
    with pytest.raises(ValueError):
        fba.interface.default_dq_mode()


@pytest.mark.parametrize("case", ["c1_2d", "c3_like", "c5_like", "gqa", "cross", "tile_mask_64_192", "tile_mask_16_64",
                                  "ragged", "odd_tiles"])
def test_alternative_key_major_kernel(case):
    """The second key-major kernel (query-row orientation, selectable with fba_set_bwd_kernel(2) or
    FBA_BWD_KERNEL=2) against the oracle, and against the default kernel."""
    from flex_block_attn_b200 import _cabi

    lib = _cabi.lib()
    prev = lib.fba_set_bwd_kernel(2)
    try:
        assert prev in (1, 2)
        (q, k, v, do, mask, qb, kb), got = _run(case, "atomic")
    finally:
        assert lib.fba_set_bwd_kernel(prev) == 2
    want = orc.attention_slab(q.float(), k.float(), v.float(), mask, qb, kb, do.float())
    for g, w, nm in zip(got, want[2:], ("dQ", "dK", "dV")):
        assert_close(g.float(), w, f"kernel 2 {case} {nm}")
    _, ref = _run(case, "atomic")
    for g, w, nm in zip(got, ref, ("dQ", "dK", "dV")):
        assert_close(g.float(), w.float(), f"kernel 2 vs 1 {case} {nm}", max_abs=1e-2)
    assert lib.fba_set_bwd_kernel(3) == -1
