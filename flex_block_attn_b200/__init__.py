"""B200-native (sm_100a) block-sparse attention, drop-in for Tencent-Hunyuan/flex-block-attn's
``flex_block_attn_func`` (same exported names as the reference's flex_block_attn/__init__.py:1-5)."""
from .interface import (  # noqa: F401
    FlexBlockAttnFunc,
    Fp8KVCache,
    SparseLists,
    _flex_block_attn_backward,
    _flex_block_attn_forward,
    backward_with_lists,
    build_index,
    build_lists,
    check_status,
    flex_block_attn_fp8kv,
    flex_block_attn_func,
    forward_with_lists,
    moba_lists,
    quantize_kv,
    ssta_lists,
    sta_lists,
)

__all__ = [
    "flex_block_attn_func",
    "_flex_block_attn_forward",
    "_flex_block_attn_backward",
    "FlexBlockAttnFunc",
    "build_index",
    "build_lists",
    "forward_with_lists",
    "backward_with_lists",
    "check_status",
    "SparseLists",
    "sta_lists",
    "ssta_lists",
    "moba_lists",
    "Fp8KVCache",
    "quantize_kv",
    "flex_block_attn_fp8kv",
]
