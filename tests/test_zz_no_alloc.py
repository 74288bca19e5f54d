"""GPU: the scratch-free backward entry point (fba_bwd_static_scratch) against fba_bwd.

fba_bwd_static_scratch is for hosts that cannot allocate device memory when they need a backward
pass (all HBM already in a fixed arena or a foreign pool, or no tolerance for cudaMalloc's
device-wide synchronisation): its scratch is an array inside the library.  It must return what
fba_bwd returns with caller-allocated scratch -- dK and dV bit for bit, dQ within the tolerance
the other tests use for it (its fp32 accumulation order is not fixed) -- on two calls in a row
(the array is shared and keeps the previous call's contents), and must refuse sizes beyond its
stated capacity.  Runs last so that a failure here cannot hide the other tests' results.
"""
import ctypes

import pytest
import torch

from oracle import dense_oracle as orc
from tests.util import assert_close, bernoulli_mask, rand_qkv

pytestmark = pytest.mark.gpu


def _bwd(entry, q, k, v, o, lse, do, lists, scratch=None):
    import flex_block_attn_b200 as fba
    from flex_block_attn_b200 import _cabi
    from flex_block_attn_b200.interface import _status, _stream_ptr

    lib = _cabi.lib()
    B, Hq, Sq, _ = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    lst = lists.bwd_list()
    common = (q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), do.data_ptr(),
              dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, Hq, Hkv, Sq, Skv, ctypes.byref(lst))
    if entry == "static":
        rc = lib.fba_bwd_static_scratch(*common, _status(q.device).data_ptr(), _stream_ptr(q.device))
    else:
        rc = lib.fba_bwd(*common, scratch[0].data_ptr(), scratch[1].data_ptr(), _status(q.device).data_ptr(),
                         _stream_ptr(q.device))
    _cabi.check(rc, entry)
    torch.cuda.synchronize()
    fba.check_status(q.device)
    return dq, dk, dv


def test_static_scratch_matches_fba_bwd_twice_in_a_row():
    import flex_block_attn_b200 as fba
    from flex_block_attn_b200 import _cabi

    lib = _cabi.lib()
    assert lib.fba_bwd_static_scratch_max_rows() == 131072
    shapes = [(1, 2, 2, 1536, 1536, 384, 384, (1, 2, 4, 4)),      # first call
              (2, 4, 2, 1024, 768, 128, 384, (2, 4, 8, 2))]       # second call: other shape, GQA, more rows
    for n, (B, Hq, Hkv, Sq, Skv, qb, kb, mshape) in enumerate(shapes):
        q, k, v, do = rand_qkv(B, Hq, Hkv, Sq, Skv, seed=70 + n, device="cuda")
        mask = bernoulli_mask(mshape, 0.5, 70 + n).cuda()
        lists = fba.build_lists(mask, qb, kb, Sq, Skv, need_bwd=True)
        o, lse = fba.forward_with_lists(q, k, v, lists)
        n1, n2 = ctypes.c_uint64(), ctypes.c_uint64()
        assert lib.fba_bwd_scratch_bytes(B, Hq, Sq, ctypes.byref(n1), ctypes.byref(n2)) == 0
        scratch = (torch.empty(n1.value // 4, dtype=torch.float32, device="cuda"),
                   torch.empty(n2.value // 4, dtype=torch.float32, device="cuda"))
        want = _bwd("dynamic", q, k, v, o, lse, do, lists, scratch)
        ref = orc.attention_slab(q.float(), k.float(), v.float(), mask, qb, kb, do.float())
        for rep in range(2):
            got = _bwd("static", q, k, v, o, lse, do, lists)
            assert torch.equal(got[1], want[1]), f"dK differs (shape {n}, call {rep})"
            assert torch.equal(got[2], want[2]), f"dV differs (shape {n}, call {rep})"
            assert_close(got[0].float(), want[0].float(), f"dQ (shape {n}, call {rep})", max_abs=1e-2)
            for g, w, nm in zip(got, ref[2:], ("dQ", "dK", "dV")):
                assert_close(g.float(), w, f"static scratch vs oracle {nm} (shape {n}, call {rep})")


def test_static_scratch_at_exact_capacity_and_one_tile_beyond():
    """B * Hq * ceil(Sq/128) * 128 == 131072 rows uses the array to its last byte (an off-by-one in
    the split between its two regions would corrupt the last query tile of the last head, which
    the oracle comparison on that head sees); one 128-row tile more is refused before any launch."""
    import flex_block_attn_b200 as fba
    from flex_block_attn_b200 import _cabi
    from flex_block_attn_b200._cabi import FbaList

    lib = _cabi.lib()
    B, Hq, Hkv, Sq, Skv, qb, kb = 1, 8, 8, 16384, 1024, 128, 128
    assert B * Hq * Sq == lib.fba_bwd_static_scratch_max_rows()
    q, k, v, do = rand_qkv(B, Hq, Hkv, Sq, Skv, seed=77, device="cuda")
    mask = bernoulli_mask((B, Hq, Sq // qb, Skv // kb), 0.5, 77).cuda()
    lists = fba.build_lists(mask, qb, kb, Sq, Skv, need_bwd=True)
    o, lse = fba.forward_with_lists(q, k, v, lists)
    n1, n2 = ctypes.c_uint64(), ctypes.c_uint64()
    assert lib.fba_bwd_scratch_bytes(B, Hq, Sq, ctypes.byref(n1), ctypes.byref(n2)) == 0
    scratch = (torch.empty(n1.value // 4, dtype=torch.float32, device="cuda"),
               torch.empty(n2.value // 4, dtype=torch.float32, device="cuda"))
    want = _bwd("dynamic", q, k, v, o, lse, do, lists, scratch)
    hs = slice(Hq - 1, Hq)   # the head whose scratch sits at the very end of the array
    ref = orc.attention_slab(q[:, hs].float(), k[:, hs].float(), v[:, hs].float(), mask[:, hs], qb, kb, do[:, hs].float())
    for rep in range(2):
        got = _bwd("static", q, k, v, o, lse, do, lists)
        assert torch.equal(got[1], want[1]) and torch.equal(got[2], want[2])
        assert_close(got[0].float(), want[0].float(), f"dQ at capacity (call {rep})", max_abs=1e-2)
        for g, w, nm in zip(got, ref[2:], ("dQ", "dK", "dV")):
            assert_close(g[:, hs].float(), w, f"static scratch at capacity vs oracle {nm} (call {rep})")
    x = torch.zeros(16, device="cuda")
    p = x.data_ptr()
    lst = FbaList()
    rc = lib.fba_bwd_static_scratch(p, p, p, p, p, p, p, p, p, B, Hq, Hkv, Sq + 128, Skv, ctypes.byref(lst), p, None)
    assert rc == -5 and b"exceeds the built-in scratch capacity" in lib.fba_last_error()


def test_static_scratch_rejects_oversize():
    from flex_block_attn_b200 import _cabi
    from flex_block_attn_b200._cabi import FbaList

    lib = _cabi.lib()
    x = torch.zeros(16, device="cuda")
    lst = FbaList()
    p = x.data_ptr()
    # 1 * 24 * 69120 rows is far beyond 131072: refused before anything is launched.
    rc = lib.fba_bwd_static_scratch(p, p, p, p, p, p, p, p, p, 1, 24, 24, 69120, 69120, ctypes.byref(lst), p, None)
    assert rc == -5
    assert b"exceeds the built-in scratch capacity" in lib.fba_last_error()
