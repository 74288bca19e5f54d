"""GPU: the benchmark workloads (full, random-sparse at all eight sweep lengths, STA, SSTA at B=2) at
their full sequence lengths.  Parity against the fp32 slab oracle run on the same device, on two
heads per configuration and on sampled heads of the full 24-head launch, plus size-independent
properties (constant-V rows, linearity in V and dO, run-to-run determinism) on the full head count.
Every compared tensor's raw max-abs error is printed in the terminal summary."""
import pytest
import torch

from oracle import dense_oracle as orc
from tests.util import assert_close, rand_qkv

pytestmark = pytest.mark.gpu

C3_SWEEP = [11520, 19200, 30720, 38400, 46080, 53760, 61440, 69120]


def _fwd_bwd(q, k, v, do, qb, kb, mask):
    import flex_block_attn_b200 as fba

    lists = fba.build_lists(mask, qb, kb, q.shape[2], k.shape[2], need_bwd=True)
    o, lse = fba.forward_with_lists(q, k, v, lists)
    dq, dk, dv = fba.backward_with_lists(q, k, v, o, lse, do, lists)
    torch.cuda.synchronize()
    fba.check_status()
    return o, dq, dk, dv


def _compare(got, q, k, v, do, qb, kb, mask, tag):
    torch.backends.cuda.matmul.allow_tf32 = False
    want = orc.attention_slab(q.float(), k.float(), v.float(), mask, qb, kb, do.float())
    for g, w, nm in zip(got, (want[0], want[2], want[3], want[4]), ("O", "dQ", "dK", "dV")):
        assert_close(g.float(), w, f"{tag} {nm}", report=True)


def _parity(q, k, v, do, qb, kb, mask, tag):
    _compare(_fwd_bwd(q, k, v, do, qb, kb, mask), q, k, v, do, qb, kb, mask, tag)


def test_c2_full_attention_s30720():
    from flex_block_attn_b200 import masks

    q, k, v, do = rand_qkv(1, 2, 2, 30720, 30720, seed=20, scale=0.5, device="cuda")
    _parity(q, k, v, do, 384, 384, masks.full_mask(80, 80), "C2 S30720")


@pytest.mark.parametrize("S", C3_SWEEP)
def test_c3_random_sparse(S):
    from flex_block_attn_b200 import masks

    H = 2
    q, k, v, do = rand_qkv(1, H, H, S, S, seed=30 + S % 7, device="cuda")
    mask = masks.bernoulli_mask(1, H, S // 384, S // 384, 0.4, seed=S)
    _parity(q, k, v, do, 384, 384, mask, f"C3 S{S}")


def test_c4_sta_s69120():
    from flex_block_attn_b200 import masks

    q, k, v, do = rand_qkv(1, 2, 2, 69120, 69120, seed=40, device="cuda")
    _parity(q, k, v, do, 384, 384, masks.sta_mask((3, 6, 10)), "C4 S69120")


def test_c5_ssta_asymmetric_s69120_b2():
    """B = 2 as the configuration states; per-(batch, head) mask [2, H, 540, 180]."""
    from flex_block_attn_b200 import masks

    q, k, v, do = rand_qkv(2, 2, 2, 69120, 69120, seed=50, device="cuda")
    mask = masks.ssta_mask(q, k, (3, 6, 10), 128, 384, topk=8)
    assert mask.shape == (2, 2, 540, 180)
    assert not torch.equal(mask[0], mask[1])
    _parity(q, k, v, do, 128, 384, mask, "C5 B2 S69120")


def test_full_head_count_c3_s69120():
    """H=24 at S=69120 (the headline workload).  Three heads (first, middle, last) of the 24-head
    launch are compared with the oracle run on those heads' own masks; on all heads: constant V
    gives constant O rows, O is linear in V, dQ/dK are linear in dO, and forward / dK / dV are
    bit-reproducible."""
    from flex_block_attn_b200 import masks

    S, H = 69120, 24
    q, k, v, do = rand_qkv(1, H, H, S, S, seed=60, device="cuda")
    mask = masks.bernoulli_mask(1, H, S // 384, S // 384, 0.4, seed=61)
    a = _fwd_bwd(q, k, v, do, 384, 384, mask)
    for h in (0, 11, 23):
        hs = slice(h, h + 1)
        _compare(tuple(t[:, hs] for t in a), q[:, hs], k[:, hs], v[:, hs], do[:, hs], 384, 384, mask[:, hs],
                 f"C3 S69120 H24 head{h}")
    b = _fwd_bwd(q, k, v, do, 384, 384, mask)
    assert torch.equal(a[0], b[0]) and torch.equal(a[2], b[2]) and torch.equal(a[3], b[3])
    del b
    ones = torch.ones_like(v)
    o1 = _fwd_bwd(q, k, ones, do, 384, 384, mask)[0]
    assert (o1.float() - 1).abs().max().item() <= 8e-3  # softmax rows sum to 1 (bf16 P rounding)
    del o1, ones
    c = _fwd_bwd(q, k, v, (2 * do.float()).to(torch.bfloat16), 384, 384, mask)
    assert torch.equal(c[0], a[0])
    assert_close(c[3].float(), 2 * a[3].float(), "dV linear in dO", max_abs=1e-2)
    assert_close(c[2].float(), 2 * a[2].float(), "dK linear in dO", max_abs=1e-2)
    assert_close(c[1].float(), 2 * a[1].float(), "dQ linear in dO", max_abs=1e-2)
    del c
    d = _fwd_bwd(q, k, (2 * v.float()).to(torch.bfloat16), do, 384, 384, mask)
    assert_close(d[0].float(), 2 * a[0].float(), "O linear in V", max_abs=2e-2)
