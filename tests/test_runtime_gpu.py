"""GPU: the pieces around the attention kernels -- work-item order, the reference-shaped C entry
points, the bounded-wait self-test, status reporting and device handling."""
import ctypes

import pytest
import torch

from oracle import dense_oracle as orc
from oracle import mask_oracle as mo
from tests.util import assert_close, bernoulli_mask, rand_qkv

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", ["c3_4d", "shared_2d", "gqa_4d", "tile_lists", "asym_4d"])
def test_work_order_is_the_stable_descending_argsort(case):
    import flex_block_attn_b200 as fba

    if case == "c3_4d":
        B, Hq, Hkv, S, qb, kb, shape = 1, 3, 3, 69120, 384, 384, (1, 3, 180, 180)
    elif case == "shared_2d":
        B, Hq, Hkv, S, qb, kb, shape = 2, 2, 2, 3840, 384, 384, (10, 10)
    elif case == "gqa_4d":
        B, Hq, Hkv, S, qb, kb, shape = 2, 4, 2, 2560, 128, 256, (2, 4, 20, 10)
    elif case == "tile_lists":
        B, Hq, Hkv, S, qb, kb, shape = 1, 2, 2, 1344, 48, 192, (1, 2, 28, 7)
    else:
        B, Hq, Hkv, S, qb, kb, shape = 1, 2, 1, 4608, 128, 384, (1, 2, 36, 12)
    mask = bernoulli_mask(shape, 0.4, seed=len(case)).cuda()
    lists = fba.build_lists(mask, qb, kb, S, S, need_bwd=True)
    per_head = mask.dim() == 4
    n_mt, n_nt = (S + 127) // 128, (S + 127) // 128
    fl = lists.fwd_list(ordered=True)
    bl = lists.bwd_list(Hq, Hkv)
    assert fl.order and bl.order
    want_f = mo.work_order(lists.fwd_cnt, fl.rows_per_bh, per_head, B * Hq, fl.rows_div, n_mt, 2, 1)
    want_b = mo.work_order(lists.bwd_cnt, bl.rows_per_bh, per_head, B * Hkv, bl.rows_div, n_nt, 1,
                           Hq // Hkv if per_head else 1)
    assert torch.equal(lists.fwd_order.cpu(), want_f)
    assert torch.equal(lists.bwd_order[(Hq, Hkv)].cpu(), want_b)
    # every row is a permutation
    assert torch.equal(lists.fwd_order.sort(-1).values.cpu(), torch.arange(want_f.shape[1], dtype=torch.int32).expand_as(want_f))


def test_work_order_changes_no_result(monkeypatch):
    """Forward, dK and dV are bit-identical with and without the longest-first order (each CTA does
    the same work, only the dispatch order changes); dQ agrees to reduction-order noise."""
    import flex_block_attn_b200 as fba

    q, k, v, do = rand_qkv(1, 4, 2, 3840, 3840, seed=17, device="cuda")
    mask = bernoulli_mask((1, 4, 30, 10), 0.4, 17).cuda()
    outs = []
    for flag in ("1", "0"):
        monkeypatch.setenv("FBA_WORK_ORDER", flag)
        lists = fba.build_lists(mask, 128, 384, 3840, 3840, need_bwd=True)
        o, lse = fba.forward_with_lists(q, k, v, lists)
        outs.append((o,) + fba.backward_with_lists(q, k, v, o, lse, do, lists))
        assert (lists.fwd_order is not None) == (flag == "1")
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][2], outs[1][2]) and torch.equal(outs[0][3], outs[1][3])
    assert_close(outs[0][1].float(), outs[1][1].float(), "dQ with / without order", max_abs=1e-2)
    want = orc.attention_slab(q.float(), k.float(), v.float(), mask, 128, 384, do.float())
    for g, w, nm in zip(outs[0], (want[0], want[2], want[3], want[4]), ("O", "dQ", "dK", "dV")):
        assert_close(g.float(), w, f"ordered {nm}")


@pytest.mark.parametrize("qb,kb,dim,small", [(384, 384, 4, False), (128, 384, 4, True), (64, 192, 2, True),
                                             (192, 64, 2, True), (16, 64, 4, False)])
def test_reference_shaped_entry_points(qb, kb, dim, small):
    """fba_attn_forward / fba_attn_backward through the pass-throughs that carry the reference
    extension's call shape: bool masks in (the backward's transposed), o, lse / dq, dk, dv out."""
    import flex_block_attn_b200 as fba

    B, Hq, Hkv, S = 2, 4, 2, 1536
    q, k, v, do = rand_qkv(B, Hq, Hkv, S, S, seed=qb + kb, device="cuda")
    shape = (S // qb, S // kb) if dim == 2 else (B, Hq, S // qb, S // kb)
    mask = bernoulli_mask(shape, 0.5, qb + kb).cuda()
    # what the reference's Python layer passes: block_mask = pooled mask (unused here), small = fine mask
    coarse = torch.ones_like(mask[..., :1, :1]) if small else mask
    o, lse = fba._flex_block_attn_forward(q, k, v, qb, kb, coarse, mask, small)
    mt = mask.transpose(-1, -2).contiguous()
    ct = coarse.transpose(-1, -2).contiguous()
    dq, dk, dv = fba._flex_block_attn_backward(q, k, v, o, lse, do, qb, kb, ct, mt, small)
    torch.cuda.synchronize()
    fba.check_status()
    want = orc.attention_slab(q.float(), k.float(), v.float(), mask, qb, kb, do.float())
    assert torch.allclose(lse[..., 0], want[1], atol=2e-3, rtol=1e-4)
    for g, w, nm in zip((o, dq, dk, dv), (want[0], want[2], want[3], want[4]), ("O", "dQ", "dK", "dV")):
        assert_close(g.float(), w, f"attn entry qb{qb} kb{kb} {nm}")
    # bit-identical to the list-based entry points
    lists = fba.build_lists(mask, qb, kb, S, S, need_bwd=True)
    o2, lse2 = fba.forward_with_lists(q, k, v, lists)
    _, dk2, dv2 = fba.backward_with_lists(q, k, v, o2, lse2, do, lists)
    assert torch.equal(o, o2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)


def test_attn_entry_rejects_small_workspace():
    from flex_block_attn_b200 import _cabi

    lib = _cabi.lib()
    x = torch.zeros(1024, device="cuda")
    p = x.data_ptr()
    rc = lib.fba_attn_forward(p, p, p, p, p, 1, 1, 1, 1536, 1536, 384, 384, p, p, 2, 0, p, 16, p, None)
    assert rc == -1 and b"workspace smaller" in lib.fba_last_error()


def test_bounded_wait_runs_out_and_is_reported():
    """A wait on a barrier nobody arrives at gives up after its cycle budget, the kernel ends by
    itself, the status words say where, and the host helper maps them to FBA_ERR_TIMEOUT."""
    import flex_block_attn_b200 as fba
    from flex_block_attn_b200 import _cabi

    lib = _cabi.lib()
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.fba_check_status(status.data_ptr(), stream) == 0
    limit = 1_000_000
    _cabi.check(lib.fba_selftest_wait_timeout(status.data_ptr(), limit, waited.data_ptr(), stream), "selftest")
    torch.cuda.synchronize()                               # returns: the kernel ended by itself
    words = status.tolist()
    assert words[0] == 1 and words[1] == 9 and words[2] == 1 and words[6] == 777, words
    assert limit <= int(waited.item()) < 50 * limit        # gave up soon after the budget, not much later
    assert lib.fba_check_status(status.data_ptr(), stream) == -4
    assert b"timed out" in lib.fba_last_error() and b"kernel=9" in lib.fba_last_error()
    assert lib.fba_check_status(status.data_ptr(), stream) == 0      # cleared by the report
    # the Python layer raises from the same words
    _cabi.check(lib.fba_selftest_wait_timeout(fba.interface._status(torch.device("cuda", 0)).data_ptr(), limit, None,
                                              stream), "selftest")
    with pytest.raises(RuntimeError, match="timed out"):
        fba.check_status(torch.device("cuda", 0))
    fba.check_status(torch.device("cuda", 0))              # and is clean again
    # the context is still usable
    q, k, v, _ = rand_qkv(1, 1, 1, 256, 256, seed=1, device="cuda")
    fba.flex_block_attn_func(q, k, v, 128, 128, torch.ones((2, 2), dtype=torch.bool, device="cuda"))
    fba.check_status()


def test_timeout_is_noticed_without_an_explicit_check(monkeypatch):
    """With per-call checking off (the default outside the tests), the asynchronous host mirror of
    the status words makes a later call raise."""
    import flex_block_attn_b200 as fba
    from flex_block_attn_b200 import _cabi

    monkeypatch.setenv("FBA_CHECK_STATUS", "0")
    dev = torch.device("cuda", 0)
    q, k, v, _ = rand_qkv(1, 1, 1, 256, 256, seed=2, device="cuda")
    m = torch.ones((2, 2), dtype=torch.bool, device="cuda")
    lib = _cabi.lib()
    _cabi.check(lib.fba_selftest_wait_timeout(fba.interface._status(dev).data_ptr(), 100_000, None,
                                              torch.cuda.current_stream().cuda_stream), "selftest")
    fba.flex_block_attn_func(q, k, v, 128, 128, m)          # refreshes the mirror after its kernels
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="timed out"):
        fba.flex_block_attn_func(q, k, v, 128, 128, m)
    fba.check_status(dev)


def test_entry_points_leave_the_current_device_alone():
    import flex_block_attn_b200 as fba

    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    q, k, v, _ = rand_qkv(1, 1, 1, 256, 256, seed=3, device="cuda:1")
    m = torch.ones((2, 2), dtype=torch.bool, device="cuda:1")
    torch.cuda.set_device(0)
    rt = ctypes.CDLL("libcudart.so.12")
    dev = ctypes.c_int(-1)
    o = fba.flex_block_attn_func(q, k, v, 128, 128, m)
    assert rt.cudaGetDevice(ctypes.byref(dev)) == 0 and dev.value == 0
    assert o.device.index == 1
    fba.check_status(torch.device("cuda", 1))
