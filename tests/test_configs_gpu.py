"""GPU: the benchmark workloads (full, random-sparse, STA, SSTA) at (or near) their full sizes.  Full-size parity against the fp32 slab
oracle run on the same device for a subset of heads, plus size-independent properties
(constant-V rows, linearity in V and dO, run-to-run determinism) on the full head count."""
import pytest
import torch

from oracle import dense_oracle as orc
from tests.util import assert_close, rand_qkv

pytestmark = pytest.mark.gpu


def _fwd_bwd(q, k, v, do, qb, kb, mask):
    import flex_block_attn_b200 as fba

    lists = fba.build_lists(mask, qb, kb, q.shape[2], k.shape[2], need_bwd=True)
    o, lse = fba.forward_with_lists(q, k, v, lists)
    dq, dk, dv = fba.backward_with_lists(q, k, v, o, lse, do, lists)
    torch.cuda.synchronize()
    fba.check_status()
    return o, dq, dk, dv


def _parity(q, k, v, do, qb, kb, mask, tag):
    torch.backends.cuda.matmul.allow_tf32 = False
    got = _fwd_bwd(q, k, v, do, qb, kb, mask)
    want = orc.attention_slab(q.float(), k.float(), v.float(), mask, qb, kb, do.float())
    for g, w, nm in zip(got, (want[0], want[2], want[3], want[4]), ("O", "dQ", "dK", "dV")):
        assert_close(g.float(), w, f"{tag} {nm}")


def test_c2_full_attention_s30720():
    from flex_block_attn_b200 import masks

    q, k, v, do = rand_qkv(1, 2, 2, 30720, 30720, seed=20, scale=0.5, device="cuda")
    _parity(q, k, v, do, 384, 384, masks.full_mask(80, 80), "C2")


@pytest.mark.parametrize("S", [11520, 69120])
def test_c3_random_sparse(S):
    from flex_block_attn_b200 import masks

    H = 2
    q, k, v, do = rand_qkv(1, H, H, S, S, seed=30 + S % 7, device="cuda")
    mask = masks.bernoulli_mask(1, H, S // 384, S // 384, 0.4, seed=S)
    _parity(q, k, v, do, 384, 384, mask, f"C3 S{S}")


def test_c4_sta_s69120():
    from flex_block_attn_b200 import masks

    q, k, v, do = rand_qkv(1, 2, 2, 69120, 69120, seed=40, device="cuda")
    _parity(q, k, v, do, 384, 384, masks.sta_mask((3, 6, 10)), "C4")


def test_c5_ssta_asymmetric_s69120():
    from flex_block_attn_b200 import masks

    q, k, v, do = rand_qkv(1, 2, 2, 69120, 69120, seed=50, device="cuda")
    mask = masks.ssta_mask(q, k, (3, 6, 10), 128, 384, topk=8)
    assert mask.shape == (1, 2, 540, 180)
    _parity(q, k, v, do, 128, 384, mask, "C5")


def test_full_head_count_properties_c3_s69120():
    """H=24 at S=69120 (the headline workload): constant V gives constant O rows; O is linear in V,
    dQ/dK are linear in dO; forward / dK / dV are bit-reproducible."""
    from flex_block_attn_b200 import masks

    S, H = 69120, 24
    q, k, v, do = rand_qkv(1, H, H, S, S, seed=60, device="cuda")
    mask = masks.bernoulli_mask(1, H, S // 384, S // 384, 0.4, seed=61)
    ones = torch.ones_like(v)
    o1, dq1, dk1, dv1 = _fwd_bwd(q, k, ones, do, 384, 384, mask)
    assert (o1.float() - 1).abs().max().item() <= 8e-3  # softmax rows sum to 1 (bf16 P rounding)
    a = _fwd_bwd(q, k, v, do, 384, 384, mask)
    b = _fwd_bwd(q, k, v, do, 384, 384, mask)
    assert torch.equal(a[0], b[0]) and torch.equal(a[2], b[2]) and torch.equal(a[3], b[3])
    c = _fwd_bwd(q, k, v, (2 * do.float()).to(torch.bfloat16), 384, 384, mask)
    assert torch.equal(c[0], a[0])
    assert_close(c[3].float(), 2 * a[3].float(), "dV linear in dO", max_abs=1e-2)
    assert_close(c[2].float(), 2 * a[2].float(), "dK linear in dO", max_abs=1e-2)
    assert_close(c[1].float(), 2 * a[1].float(), "dQ linear in dO", max_abs=1e-2)
    d = _fwd_bwd(q, k, (2 * v.float()).to(torch.bfloat16), do, 384, 384, mask)
    assert_close(d[0].float(), 2 * a[0].float(), "O linear in V", max_abs=2e-2)
