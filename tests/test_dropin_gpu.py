"""GPU: the reference's own, unmodified Python layer on top of this library.

``oracle/_ref/flex_block_attn_interface.py`` is the reference's file, byte for byte (fetched by
oracle/fetch_ref_interface.py; it is not part of this repository).  It imports ``attn_forward`` /
``attn_backward`` from the compiled module ``flex_block_attn_cuda``; here that name is bound to
``flex_block_attn_b200.compat``, the stand-in INTEGRATION.md describes, and the reference's
``flex_block_attn_func`` -- its asserts, its mask pooling for asymmetric blocks, its transposes in
backward -- then runs the reference's own test grid against the oracle.
"""
import importlib.util
import sys
from pathlib import Path

import pytest
import torch

from oracle import dense_oracle as orc
from tests.util import assert_close, bernoulli_mask, rand_qkv, reference_rule_mask

pytestmark = pytest.mark.gpu
REF_FILE = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "flex_block_attn_interface.py"


@pytest.fixture(scope="module")
def ref_iface():
    if not REF_FILE.exists():
        pytest.skip("oracle/_ref/flex_block_attn_interface.py is absent (run oracle/fetch_ref_interface.py on a "
                    "machine that has the reference checkout)")
    import flex_block_attn_b200.compat as compat

    saved = sys.modules.get("flex_block_attn_cuda")
    sys.modules["flex_block_attn_cuda"] = compat
    try:
        spec = importlib.util.spec_from_file_location("ref_flex_block_attn_interface", REF_FILE)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        yield mod
    finally:
        if saved is None:
            sys.modules.pop("flex_block_attn_cuda", None)
        else:
            sys.modules["flex_block_attn_cuda"] = saved


def _run(ref_iface, q, k, v, do, qb, kb, mask, tag):
    import flex_block_attn_b200 as fba

    qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
    o = ref_iface.flex_block_attn_func(qq, kk, vv, qb, kb, mask)
    o.backward(do)
    torch.cuda.synchronize()
    fba.check_status()
    want = orc.attention_slab(q.float(), k.float(), v.float(), mask, qb, kb, do.float())
    for g, w, nm in zip((o.detach(), qq.grad, kk.grad, vv.grad), (want[0], want[2], want[3], want[4]),
                        ("O", "dQ", "dK", "dV")):
        assert_close(g.float(), w, f"drop-in {tag} {nm}")
    return o.detach()


# The reference's grid (test/test_flex_block_attn.py:66-71) with its mask rule (:25), 4-D masks.
@pytest.mark.parametrize("seq_len", [768, 1536, 3072])
@pytest.mark.parametrize("heads", [1, 4])
@pytest.mark.parametrize("qb,kb", [(16, 64), (32, 128), (64, 64), (128, 128), (64, 256), (128, 384), (384, 384)])
def test_reference_python_layer_on_this_library(ref_iface, seq_len, heads, qb, kb):
    q, k, v, do = rand_qkv(1, heads, heads, seq_len, seq_len, seed=seq_len + heads + qb + kb, device="cuda")
    mask2d = reference_rule_mask(seq_len // qb, seq_len // kb)
    mask = mask2d[None, None].expand(1, heads, -1, -1).contiguous().cuda()
    _run(ref_iface, q, k, v, do, qb, kb, mask, f"S{seq_len} H{heads} qb{qb} kb{kb}")


def test_reference_python_layer_2d_mask_and_same_bits_as_native(ref_iface):
    """2-D mask, equal block sizes: the reference layer's output equals this package's own
    flex_block_attn_func bit for bit (same kernels underneath)."""
    import flex_block_attn_b200 as fba

    q, k, v, do = rand_qkv(2, 2, 2, 1536, 1536, seed=5, device="cuda")
    mask = bernoulli_mask((4, 4), 0.5, 5).cuda()
    o_ref = _run(ref_iface, q, k, v, do, 384, 384, mask, "2d")
    assert torch.equal(o_ref, fba.flex_block_attn_func(q, k, v, 384, 384, mask))
