"""CPU: the Python layer keeps the reference's argument checks (flex_block_attn_interface.py:18-32)
and refuses CPU tensors instead of falling back."""
import pytest
import torch

import flex_block_attn_b200 as fba
from flex_block_attn_b200 import masks


def _qkv(S=256, H=1):
    q = torch.zeros((1, H, S, 128), dtype=torch.bfloat16)
    return q, q.clone(), q.clone()


@pytest.mark.parametrize("qb,kb,msg", [
    (24, 64, "q_block_size (24) must be divisible by 16"),
    (16, 96, "kv_block_size (96) must be divisible by 64"),
    (48, 64, "must be divisible by q_block_size (48), or vice versa"),
])
def test_block_size_assertions(qb, kb, msg):
    q, k, v = _qkv()
    with pytest.raises(AssertionError) as e:
        fba.flex_block_attn_func(q, k, v, qb, kb, torch.ones((2, 2), dtype=torch.bool))
    assert msg in str(e.value)


def test_length_and_mask_shape_assertions():
    q, k, v = _qkv(S=200)
    with pytest.raises(AssertionError, match="q_seq_len \\(200\\) must be divisible by q_block_size"):
        fba.flex_block_attn_func(q, k, v, 128, 128, torch.ones((2, 2), dtype=torch.bool))
    q, k, v = _qkv(S=256)
    with pytest.raises(AssertionError, match="must equal q_seq_len"):
        fba.flex_block_attn_func(q, k, v, 128, 128, torch.ones((3, 2), dtype=torch.bool))


def test_cpu_tensors_are_refused_not_emulated():
    q, k, v = _qkv()
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        fba.flex_block_attn_func(q, k, v, 128, 128, torch.ones((2, 2), dtype=torch.bool))


def test_mask_builders_on_cpu():
    m = masks.sta_mask((3, 6, 10), device="cpu")
    assert m.shape == (180, 180) and int(m.sum()) == 3136 and bool((m == m.T).all())
    assert int(m.sum(1).min()) == 8 and int(m.sum(1).max()) == 27
    perm = masks.tile_major_permutation((18, 48, 80), (6, 8, 8))
    assert perm.shape == (69120,) and torch.equal(torch.sort(perm).values, torch.arange(69120))
    first = perm[:384]
    t, h, w = first // (48 * 80), (first // 80) % 48, first % 80
    assert int(t.max()) == 5 and int(h.max()) == 7 and int(w.max()) == 7
    g = torch.Generator().manual_seed(0)
    q = torch.randn((1, 2, 3 * 128 * 2, 128), generator=g)
    k = torch.randn((1, 2, 2 * 384, 128), generator=g)
    mb = masks.moba_topk_mask(q, k, 128, 384, 1)
    assert mb.shape == (1, 2, 6, 2) and bool((mb.sum(-1) == 1).all())
    ms = masks.ssta_mask(q, k, (1, 1, 2), 128, 384, topk=1, window=(0, 0, 0))
    assert ms.shape == (1, 2, 6, 2) and bool(ms[0, 0, 0, 0]) and bool(ms[0, 0, 5, 1])
    bm = masks.bernoulli_mask(1, 2, 6, 3, 0.0, 0, device="cpu")
    assert int(bm.sum()) == 12  # only the forced (scaled) diagonal


def test_prebuilt_lists_are_checked_against_the_call():
    """A SparseLists passed instead of a mask must fit the block sizes, (batch, head) and device."""
    q, k, v = _qkv(S=256, H=2)
    z = torch.zeros((4, 2), dtype=torch.int32)
    c = torch.zeros((4,), dtype=torch.int32)
    lists = fba.SparseLists(True, 4, 1, 3, 2, 2, 128, 128, 256, 256, z, c, None, z, c, None)   # built for 3 heads
    with pytest.raises(AssertionError, match="batch and head sizes of q"):
        fba.flex_block_attn_func(q, k, v, 128, 128, lists)
    with pytest.raises(AssertionError, match="other block sizes"):
        fba.flex_block_attn_func(q, k, v, 256, 256, lists)
    with pytest.raises(ValueError, match="softmax_scale"):
        lists2 = fba.SparseLists(True, 2, 1, 2, 2, 2, 128, 128, 256, 256, z, c, None, z, c, None)
        fba.flex_block_attn_func(q, k, v, 128, 128, lists2, softmax_scale=float("nan"))


def test_bench_reads_roofline_traffic_from_the_committed_profile():
    """bench.py takes the backward kernel's DRAM bytes per active block pair from the ncu summary
    under profiles/ (no hand-copied constant)."""
    import importlib.util
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    spec = importlib.util.spec_from_file_location("bench_mod", root / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    got = bench.bwd_dram_bytes_per_pair()
    assert got is not None and got[1].startswith("fba_bwd_kernel_")
    text = (root / "profiles" / got[1]).read_text()
    assert f"dram_bytes_per_active_pair = {int(got[0])}" in text
    # the figure is the capture's read + write bytes over its active pairs
    import re
    rd = int(re.search(r"dram__bytes_read.sum \| byte \| (\d+)", text).group(1))
    wr = int(re.search(r"dram__bytes_write.sum \| byte \| (\d+)", text).group(1))
    pairs = int(re.search(r"([\d ]+) active block pairs\n\n    python bench.py --seq 46080", text).group(1).replace(" ", ""))
    assert abs((rd + wr) / pairs - got[0]) < 1.0
    # the step's FLOP count per active pair: 4 + 10 GEMM-flops per (q, kv, d) triple
    class A:  # minimal stand-in for parsed arguments
        seq, heads, keep = None, 24, 0.4
    wl = bench.Workload("c3", A, 24, 0, "cpu")
    assert wl.flops == 14 * 384 * 384 * 128 and wl.shape == (1, 24, 69120, 128)
    wl5 = bench.Workload("c5", A, 3, 0, "cpu")
    assert wl5.flops == 14 * 128 * 384 * 128 and wl5.shape == (2, 3, 69120, 128)


def test_compat_module_has_the_reference_extension_signatures():
    """flex_block_attn_b200.compat stands in for the reference's compiled module: same two names, same
    positional parameters as attention_forward / attention_backward (reference attn.cpp:12-21)."""
    import inspect

    from flex_block_attn_b200 import compat

    fwd = list(inspect.signature(compat.attn_forward).parameters)
    bwd = list(inspect.signature(compat.attn_backward).parameters)
    assert fwd == ["q", "k", "v", "q_block_size", "kv_block_size", "load_block_mask", "compute_block_mask",
                   "use_small_block_mode"]
    assert bwd == ["q", "k", "v", "o", "l_vec", "og", "q_block_size", "kv_block_size", "load_block_mask",
                   "compute_block_mask", "use_small_block_mode"]
