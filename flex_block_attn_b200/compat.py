"""Stand-in for the reference's compiled module ``flex_block_attn_cuda``.

The reference's Python layer does ``from flex_block_attn_cuda import attn_forward, attn_backward``
(reference flex_block_attn/flex_block_attn_interface.py:4) and calls them with torch tensors
(attn.cpp:12-21, 29-30).  This module offers the same two functions with the same positional
arguments and return values on top of libfba_b200.so's ``fba_attn_forward`` / ``fba_attn_backward``,
so a reference checkout can be pointed at this library with

    import sys, flex_block_attn_b200.compat
    sys.modules["flex_block_attn_cuda"] = flex_block_attn_b200.compat

before ``flex_block_attn`` is imported, and nothing else changes.  Differences a caller can see:
``l_vec`` holds the natural-log sum-exp (the reference stores -sqrt(128) times it); it is only ever
handed back to ``attn_backward``, which expects what ``attn_forward`` wrote.  The gradients come
back in bf16.
"""
from __future__ import annotations

from .interface import _flex_block_attn_backward, _flex_block_attn_forward


def attn_forward(q, k, v, q_block_size, kv_block_size, load_block_mask, compute_block_mask, use_small_block_mode):
    """-> [o bf16 [B,H,Sq,128], l_vec fp32 [B,H,Sq,1]] (reference attention_forward, .cu:810-1007)."""
    o, lse = _flex_block_attn_forward(q, k, v, q_block_size, kv_block_size, load_block_mask, compute_block_mask,
                                      use_small_block_mode)
    return [o, lse]


def attn_backward(q, k, v, o, l_vec, og, q_block_size, kv_block_size, load_block_mask, compute_block_mask,
                  use_small_block_mode):
    """-> [qg, kg, vg] (reference attention_backward, .cu:1009-1267); the masks arrive transposed."""
    dq, dk, dv = _flex_block_attn_backward(q, k, v, o, l_vec, og, q_block_size, kv_block_size, load_block_mask,
                                           compute_block_mask, use_small_block_mode)
    return [dq, dk, dv]
