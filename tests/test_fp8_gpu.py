"""GPU: the e4m3 key / value cache path (fba_quantize_kv_e4m3, fba_fwd_fp8kv).

The cache writer is integer / byte work and is held bit-exactly to the oracle's restatement.  The
forward is compared with the oracle evaluated on the DEQUANTISED cache and the per-row e4m3 round
trip of q, i.e. on exactly the operands the kernel's arithmetic stands for; what remains is the
kernel's 8-bit rounding of the probabilities and fp32 summation order.  Tolerance for that:
cosine >= 0.999 and max-abs <= 5e-2 * max(1, max|expected|), stated here because it is wider than
the bf16 kernels' 2e-2 / 0.9995 (e4m3 keeps 3 mantissa bits).
"""
import pytest
import torch

from oracle import dense_oracle as orc
from tests.util import assert_close, bernoulli_mask, rand_qkv

pytestmark = pytest.mark.gpu
FP8_MAX_ABS, FP8_MIN_COS = 5e-2, 0.999


@pytest.mark.parametrize("S,block,scale", [(768, 128, 1.0), (1536, 384, 1.0), (1536, 768, 3.0), (256, 256, 0.01)])
def test_cache_writer_is_bit_exact(S, block, scale):
    import flex_block_attn_b200 as fba

    _, k, v, _ = rand_qkv(2, 2, 2, 128, S, seed=S + block, scale=scale, device="cuda")
    if S >= 2 * block:
        k[0, 1, block:2 * block] = 0          # an all-zero block gets scale 1
    cache = fba.quantize_kv(k, v, block)
    k8, ks = orc.quantize_e4m3_blocks(k, block)
    v8, vs = orc.quantize_e4m3_blocks(v, block)
    assert torch.equal(cache.k_scale, ks) and torch.equal(cache.v_scale, vs)
    assert torch.equal(cache.k8, k8)
    assert torch.equal(cache.v8t, v8.transpose(-1, -2).contiguous())
    kd, vd = cache.dequantize()
    assert torch.equal(kd, orc.dequantize_e4m3_blocks(k8, ks, block))
    assert (kd - k.float()).abs().max().item() <= 0.07 * k.float().abs().max().item()
    assert (vd - v.float()).abs().max().item() <= 0.07 * v.float().abs().max().item()


CASES = {
    # name: (B, Hq, Hkv, Sq, Skv, qb, kb, mask shape, keep, scale_block)
    "c1": (1, 2, 2, 1536, 1536, 384, 384, (4, 4), 0.5, 384),
    "c3_like": (1, 3, 3, 3840, 3840, 384, 384, (1, 3, 10, 10), 0.4, 384),
    "c5_like_gqa": (2, 4, 2, 3072, 3072, 128, 384, (2, 4, 24, 8), 0.4, 384),
    "cross_small_scale_block": (1, 2, 2, 512, 1280, 128, 128, (4, 10), 0.4, 128),
    "tile_mask": (1, 2, 1, 1536, 1536, 64, 192, (1, 2, 24, 8), 0.5, 768),
    "odd_tiles": (1, 2, 2, 640, 640, 128, 128, (1, 2, 5, 5), 0.5, 128),
}


@pytest.mark.parametrize("case", list(CASES))
def test_fp8_forward_against_oracle_on_the_dequantised_cache(case):
    import flex_block_attn_b200 as fba

    B, Hq, Hkv, Sq, Skv, qb, kb, mshape, keep, sblock = CASES[case]
    q, k, v, _ = rand_qkv(B, Hq, Hkv, Sq, Skv, seed=len(case), device="cuda")
    # blocks of different magnitude, so that a wrong scale index cannot pass
    ramp = torch.linspace(0.5, 2.0, Skv // sblock, device="cuda").repeat_interleave(sblock)[None, None, :, None]
    k = (k.float() * ramp).to(torch.bfloat16)
    v = (v.float() * ramp.flip(2)).to(torch.bfloat16)
    mask = bernoulli_mask(mshape, keep, len(case)).cuda()
    cache = fba.quantize_kv(k, v, sblock)
    o, lse = fba.flex_block_attn_fp8kv(q, cache, qb, kb, mask, need_lse=True)
    torch.cuda.synchronize()
    fba.check_status()
    kd, vd = cache.dequantize()
    want_o, want_lse = orc.attention_slab(orc.quantize_rows_e4m3(q), kd, vd, mask, qb, kb)
    ma, cos, mx = assert_close(o.float(), want_o, f"fp8 {case} O", max_abs=FP8_MAX_ABS, min_cos=FP8_MIN_COS, report=True)
    live = torch.isfinite(want_lse)
    assert torch.equal(torch.isfinite(lse), live)
    assert torch.allclose(lse[live], want_lse[live], atol=5e-3, rtol=1e-3)
    # and it stays close to the bf16 forward on the original K, V (cache rounding included)
    o16 = fba.flex_block_attn_func(q, k, v, qb, kb, mask)
    assert_close(o.float(), o16.float(), f"fp8 vs bf16 {case}", max_abs=0.12, min_cos=0.995)
    o2 = fba.flex_block_attn_fp8kv(q, cache, qb, kb, mask)
    assert torch.equal(o, o2)


def test_fp8_forward_bad_arguments():
    import flex_block_attn_b200 as fba

    q, k, v, _ = rand_qkv(1, 2, 2, 256, 384, seed=1, device="cuda")
    with pytest.raises(ValueError):
        fba.quantize_kv(k, v, 96)
    with pytest.raises(ValueError):
        fba.quantize_kv(k, v, 256)          # does not divide 384
    cache = fba.quantize_kv(k, v, 128)
    with pytest.raises(ValueError):
        fba.flex_block_attn_fp8kv(q.float(), cache, 128, 128, torch.ones((2, 3), dtype=torch.bool, device="cuda"))
