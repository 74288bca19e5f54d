"""Python API and autograd wrapper of the B200 block-sparse attention operator.

Mirrors the reference's public layer (flex_block_attn/flex_block_attn_interface.py):
``flex_block_attn_func`` (:91-106), ``FlexBlockAttnFunc`` (:14-89) and the two pass-throughs
``_flex_block_attn_forward`` / ``_flex_block_attn_backward`` (:6-12), with the same argument
meaning, the same assertion texts (:18-32) and the same return convention
(``dq, dk, dv, None x 5``, :89).  Underneath, PyTorch only allocates device buffers and supplies
the current stream; all compute runs in libfba_b200.so through the C ABI in include/fba.h.

Differences that a caller can observe:
  * gradients come back in bf16 directly (the reference returns fp32 and lets autograd cast);
  * the saved log-sum-exp is the natural-log one, shape [B, H, Sq, 1] (the reference stores
    -sqrt(128) * LSE, flex_block_attn_h100.cu:303-307);
  * the block mask is compacted once in forward into index lists that backward reuses; the
    reference max-pools the mask (:38-66) and transposes it on every backward (:85-86);
  * ``q_block_size > kv_block_size`` with a 2-D mask works (the reference reshapes it wrongly,
    :55-57) and a query row that attends to nothing yields a zero output row and zero gradients;
  * sequences shorter than 128 rows are padded to 128 around the kernels (which want one full tile).
"""
from __future__ import annotations

import ctypes
import math
import os
from dataclasses import dataclass
from typing import Optional

import torch

from . import _cabi
from ._cabi import FbaList

HEAD_DIM = 128
TILE = 128

class _StatusMonitor:
    """Per-device status words (written by a kernel whose bounded wait gave up) and a pinned host
    mirror that is refreshed asynchronously after every call, so that a timeout is noticed at the
    next call without any synchronisation."""

    def __init__(self, device: torch.device):
        self.device = device
        self.buf = torch.zeros(8, dtype=torch.int32, device=device)
        self.host = torch.zeros(8, dtype=torch.int32).pin_memory()
        self.event = torch.cuda.Event()
        self.pending = False

    def after_call(self) -> None:
        self.host.copy_(self.buf, non_blocking=True)
        self.event.record(torch.cuda.current_stream(self.device))
        self.pending = True

    def poll(self) -> None:
        """Raise if a mirror copy that has already completed shows a timed-out wait."""
        if self.pending and self.event.query():
            self.pending = False
            if int(self.host[0]) != 0:
                self.raise_from(self.host.tolist())

    def raise_from(self, words) -> None:
        self.buf.zero_()
        self.host.zero_()
        raise RuntimeError(
            "flex_block_attn_b200: a device-side wait timed out; the outputs of that call are undefined "
            f"(kernel={words[1]} role={words[2]} block=({words[3]},{words[4]}) iter={words[5]} tag={words[6]})"
        )


_monitors: dict[int, _StatusMonitor] = {}


def _monitor(device: torch.device) -> _StatusMonitor:
    key = device.index if device.index is not None else torch.cuda.current_device()
    mon = _monitors.get(key)
    if mon is None:
        mon = _StatusMonitor(torch.device("cuda", key))
        _monitors[key] = mon
    return mon


def _status(device: torch.device) -> torch.Tensor:
    """Per-device 8-word status buffer the kernels write when a bounded wait gives up."""
    return _monitor(device).buf


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronise the current stream of ``device`` and raise if any kernel reported a timed-out
    wait.  Every call of this package also polls, without synchronising, a host mirror of the status
    words refreshed after the previous calls; a training loop that wants the check to be exact calls
    this once per step, where it synchronises anyway."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    mon = _monitor(device)
    rc = _cabi.lib().fba_check_status(mon.buf.data_ptr(), _stream_ptr(device))
    mon.pending = False
    if rc == _cabi.FBA_ERR_TIMEOUT:
        mon.host.zero_()
        raise RuntimeError("flex_block_attn_b200: " + _cabi.lib().fba_last_error().decode("utf-8", "replace"))
    _cabi.check(rc, "fba_check_status")


def _maybe_check(device: torch.device) -> None:
    if os.environ.get("FBA_CHECK_STATUS", "0") == "1":
        check_status(device)
    else:
        _monitor(device).after_call()


def _new(shape_or_like, dtype=None, device=None) -> torch.Tensor:
    """Output / scratch allocation: uninitialised, or NaN-filled under FBA_POISON_OUTPUTS=1 (the test
    suite sets it so that an element no kernel wrote shows up in every comparison)."""
    if isinstance(shape_or_like, torch.Tensor):
        t = torch.empty_like(shape_or_like)
    else:
        t = torch.empty(shape_or_like, dtype=dtype, device=device)
    if os.environ.get("FBA_POISON_OUTPUTS", "0") == "1" and t.is_floating_point():
        t.fill_(float("nan"))
    return t


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


@dataclass
class SparseLists:
    """Compacted index lists of one block mask, in the layout the kernels walk.

    ``q2k_*`` / ``k2q_*`` are the block-granular lists (always built when both block sizes are
    multiples of 128; they are then exactly what the kernels consume).  For other block sizes the
    kernels consume 128x128 tile lists with 16-bit sub-tile masks (``fwd_*`` / ``bwd_*``).
    """

    aligned: bool
    mask_dim: int
    B: int
    H: int
    nQ: int
    nK: int
    q_block: int
    kv_block: int
    Sq: int
    Skv: int
    fwd_idx: torch.Tensor
    fwd_cnt: torch.Tensor
    fwd_msk: Optional[torch.Tensor]
    bwd_idx: Optional[torch.Tensor]
    bwd_cnt: Optional[torch.Tensor]
    bwd_msk: Optional[torch.Tensor]
    # work-item orders (longest list first), built on first use; the backward one depends on the
    # number of kv heads (a CTA walks the lists of a whole grouped-query group)
    fwd_order: Optional[torch.Tensor] = None
    bwd_order: Optional[dict] = None

    def fwd_list(self, ordered: bool = False) -> FbaList:
        n_mt = (self.Sq + TILE - 1) // TILE
        rows = self.nQ if self.aligned else n_mt
        lst = FbaList(
            self.fwd_idx.data_ptr(), self.fwd_cnt.data_ptr(), _ptr(self.fwd_msk),
            self.fwd_idx.shape[-1], rows, rows if self.mask_dim == 4 else 0,
            self.q_block // TILE if self.aligned else 1,
            self.kv_block // TILE if self.aligned else 1,
        )
        if ordered and _work_order_enabled():
            if self.fwd_order is None:
                dev = self.fwd_idx.device
                n_rows = self.B * self.H if self.mask_dim == 4 else 1
                order = torch.empty((n_rows, (n_mt + 1) // 2), dtype=torch.int32, device=dev)
                with torch.cuda.device(dev):
                    rc = _cabi.lib().fba_fwd_order(ctypes.byref(lst), self.B, self.H, self.Sq, order.data_ptr(),
                                                   _stream_ptr(dev))
                if rc != _cabi.FBA_ERR_TOO_LARGE:
                    _cabi.check(rc, "fba_fwd_order")
                    self.fwd_order = order
            lst.order = _ptr(self.fwd_order)
        return lst

    def bwd_list(self, Hq: Optional[int] = None, Hkv: Optional[int] = None) -> FbaList:
        """``Hq`` / ``Hkv`` given: also attach the longest-first work order for that head grouping."""
        assert self.bwd_idx is not None and self.bwd_cnt is not None
        n_nt = (self.Skv + TILE - 1) // TILE
        rows = self.nK if self.aligned else n_nt
        lst = FbaList(
            self.bwd_idx.data_ptr(), self.bwd_cnt.data_ptr(), _ptr(self.bwd_msk),
            self.bwd_idx.shape[-1], rows, rows if self.mask_dim == 4 else 0,
            self.kv_block // TILE if self.aligned else 1,
            self.q_block // TILE if self.aligned else 1,
        )
        if Hq is not None and Hkv is not None and _work_order_enabled():
            if self.bwd_order is None:
                self.bwd_order = {}
            B = self.B if self.mask_dim == 4 else 1
            if (Hq, Hkv) not in self.bwd_order:
                dev = self.bwd_idx.device
                n_rows = B * Hkv if self.mask_dim == 4 else 1
                order = torch.empty((n_rows, n_nt), dtype=torch.int32, device=dev)
                with torch.cuda.device(dev):
                    rc = _cabi.lib().fba_bwd_order(ctypes.byref(lst), B, Hq, Hkv, self.Skv, order.data_ptr(),
                                                   _stream_ptr(dev))
                if rc == _cabi.FBA_ERR_TOO_LARGE:
                    order = None
                else:
                    _cabi.check(rc, "fba_bwd_order")
                self.bwd_order[(Hq, Hkv)] = order
            lst.order = _ptr(self.bwd_order[(Hq, Hkv)])
        return lst


def _work_order_enabled() -> bool:
    """FBA_WORK_ORDER=0 launches the attention grids in natural tile order (for A/B timing)."""
    return os.environ.get("FBA_WORK_ORDER", "1") != "0"


def build_index(block_mask: torch.Tensor, want_q2k: bool = True, want_k2q: bool = True):
    """Block-granular compaction: returns (q2k_idx, q2k_cnt, k2q_idx, k2q_cnt), int32.

    ``q2k_idx[r, :q2k_cnt[r]]`` are the ascending kv-block indices q-block row r attends to (rows
    are flattened over batch and head for a 4-D mask); unused slots are -1.  ``k2q_*`` is the same
    for the transposed mask.  Bit-exact against a ``torch.nonzero`` restatement.
    """
    if block_mask.dtype != torch.bool:
        raise TypeError("block_mask must be a torch.bool tensor")
    if not block_mask.is_cuda:
        raise RuntimeError("block_mask must be a CUDA tensor (there is no CPU path)")
    if block_mask.dim() not in (2, 4):
        raise ValueError("block_mask must have 2 or 4 dimensions")
    m = block_mask.contiguous()
    dev = m.device
    if m.dim() == 2:
        B = H = 1
        nQ, nK = m.shape
    else:
        B, H, nQ, nK = m.shape
    n_bh = B * H if m.dim() == 4 else 1
    q2k_idx = q2k_cnt = k2q_idx = k2q_cnt = None
    if want_q2k:
        q2k_idx = torch.empty((n_bh * nQ, nK), dtype=torch.int32, device=dev)
        q2k_cnt = torch.empty((n_bh * nQ,), dtype=torch.int32, device=dev)
    if want_k2q:
        k2q_idx = torch.empty((n_bh * nK, nQ), dtype=torch.int32, device=dev)
        k2q_cnt = torch.empty((n_bh * nK,), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        rc = _cabi.lib().fba_build_index(
            m.data_ptr(), m.dim(), B, H, nQ, nK, _ptr(q2k_idx), _ptr(q2k_cnt), _ptr(k2q_idx),
            _ptr(k2q_cnt), _stream_ptr(dev))
    _cabi.check(rc, "fba_build_index")
    return q2k_idx, q2k_cnt, k2q_idx, k2q_cnt


def build_lists(block_mask: torch.Tensor, q_block: int, kv_block: int, Sq: int, Skv: int,
                need_bwd: bool = True) -> SparseLists:
    """Compact ``block_mask`` into the lists the forward (and backward) kernels walk."""
    if block_mask.dtype != torch.bool:
        raise TypeError("block_mask must be a torch.bool tensor")
    if not block_mask.is_cuda:
        raise RuntimeError("block_mask must be a CUDA tensor (there is no CPU path)")
    m = block_mask.contiguous()
    dev = m.device
    if m.dim() == 2:
        B = H = 1
        nQ, nK = m.shape
    else:
        B, H, nQ, nK = m.shape
    aligned = q_block % TILE == 0 and kv_block % TILE == 0
    if aligned:
        q2k_idx, q2k_cnt, k2q_idx, k2q_cnt = build_index(m, True, need_bwd)
        return SparseLists(aligned, m.dim(), B, H, nQ, nK, q_block, kv_block, Sq, Skv,
                           q2k_idx, q2k_cnt, None, k2q_idx, k2q_cnt, None)
    n_bh = B * H if m.dim() == 4 else 1
    n_mt = (Sq + TILE - 1) // TILE
    n_nt = (Skv + TILE - 1) // TILE
    fwd_idx = torch.empty((n_bh * n_mt, n_nt), dtype=torch.int32, device=dev)
    fwd_cnt = torch.empty((n_bh * n_mt,), dtype=torch.int32, device=dev)
    fwd_msk = torch.empty((n_bh * n_mt, n_nt), dtype=torch.int16, device=dev)
    bwd_idx = bwd_cnt = bwd_msk = None
    if need_bwd:
        bwd_idx = torch.empty((n_bh * n_nt, n_mt), dtype=torch.int32, device=dev)
        bwd_cnt = torch.empty((n_bh * n_nt,), dtype=torch.int32, device=dev)
        bwd_msk = torch.empty((n_bh * n_nt, n_mt), dtype=torch.int16, device=dev)
    with torch.cuda.device(dev):
        rc = _cabi.lib().fba_build_tile_lists(
            m.data_ptr(), m.dim(), B, H, nQ, nK, q_block, kv_block, Sq, Skv,
            fwd_idx.data_ptr(), fwd_cnt.data_ptr(), fwd_msk.data_ptr(),
            _ptr(bwd_idx), _ptr(bwd_cnt), _ptr(bwd_msk), _stream_ptr(dev))
    _cabi.check(rc, "fba_build_tile_lists")
    return SparseLists(aligned, m.dim(), B, H, nQ, nK, q_block, kv_block, Sq, Skv,
                       fwd_idx, fwd_cnt, fwd_msk, bwd_idx, bwd_cnt, bwd_msk)


def sta_lists(tile_grid, window=(1, 1, 1), tile_tokens: int = 384, device="cuda") -> SparseLists:
    """Lists of the 3-D sliding-tile mask, built on the device without a bool mask.

    One attention block = one tile of ``tile_tokens`` tokens (a multiple of 128), tokens in
    tile-major order (``masks.tile_major_permutation``).  Same lists as
    ``build_lists(masks.sta_mask(tile_grid, window), tile_tokens, tile_tokens, ...)``.
    """
    if tile_tokens % TILE != 0:
        raise ValueError("tile_tokens must be a multiple of 128")
    Gt, Gh, Gw = tile_grid
    n = Gt * Gh * Gw
    dev = torch.device(device)
    idx = torch.empty((n, n), dtype=torch.int32, device=dev)
    cnt = torch.empty((n,), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        rc = _cabi.lib().fba_sta_index(Gt, Gh, Gw, window[0], window[1], window[2], idx.data_ptr(), cnt.data_ptr(),
                                       _stream_ptr(dev))
    _cabi.check(rc, "fba_sta_index")
    S = n * tile_tokens
    return SparseLists(True, 2, 1, 1, n, n, tile_tokens, tile_tokens, S, S, idx, cnt, None, idx, cnt, None)


def ssta_lists(q, k, tile_grid, q_block: int, kv_block: int, topk: int = 8, window=(1, 1, 1),
               need_bwd: bool = True):
    """Hybrid SSTA mask (STA window united with the MoBA top-k of pooled q.k) built by CUDA kernels.

    Returns ``(lists, mask)``: the ``SparseLists`` the attention kernels walk and the bool mask
    [B, Hq, Sq/q_block, Skv/kv_block] (same definition as ``masks.ssta_mask``).  Both block sizes
    must be multiples of 128 and q_block must divide kv_block (one key block = one tile).
    """
    _check_qkv(q, k, k)
    if q_block % TILE != 0 or kv_block % TILE != 0:
        raise ValueError("ssta_lists needs block sizes that are multiples of 128")
    B, Hq, Sq, _ = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    nQ, nK = Sq // q_block, Skv // kv_block
    dev = q.device
    n = ctypes.c_uint64(0)
    _cabi.check(_cabi.lib().fba_ssta_scratch_floats(B, Hq, Hkv, nQ, nK, ctypes.byref(n)), "fba_ssta_scratch_floats")
    scratch = torch.empty((n.value,), dtype=torch.float32, device=dev)
    mask = torch.empty((B, Hq, nQ, nK), dtype=torch.bool, device=dev)
    q2k_idx = torch.empty((B * Hq * nQ, nK), dtype=torch.int32, device=dev)
    q2k_cnt = torch.empty((B * Hq * nQ,), dtype=torch.int32, device=dev)
    k2q_idx = k2q_cnt = None
    if need_bwd:
        k2q_idx = torch.empty((B * Hq * nK, nQ), dtype=torch.int32, device=dev)
        k2q_cnt = torch.empty((B * Hq * nK,), dtype=torch.int32, device=dev)
    Gt, Gh, Gw = tile_grid
    with torch.cuda.device(dev):
        rc = _cabi.lib().fba_ssta_index(q.data_ptr(), k.data_ptr(), B, Hq, Hkv, Sq, Skv, q_block, kv_block,
                                        Gt, Gh, Gw, window[0], window[1], window[2], topk, scratch.data_ptr(),
                                        mask.data_ptr(), q2k_idx.data_ptr(), q2k_cnt.data_ptr(), _ptr(k2q_idx),
                                        _ptr(k2q_cnt), _stream_ptr(dev))
    _cabi.check(rc, "fba_ssta_index")
    lists = SparseLists(True, 4, B, Hq, nQ, nK, q_block, kv_block, Sq, Skv, q2k_idx, q2k_cnt, None, k2q_idx,
                        k2q_cnt, None)
    return lists, mask


def moba_lists(q, k, q_block: int, kv_block: int, topk: int, need_bwd: bool = True):
    """MoBA mask (for every query block the ``topk`` key blocks with the largest pooled q.k score,
    same definition as ``masks.moba_topk_mask``) built by the SSTA kernels with the window switched
    off.  Returns ``(lists, mask)`` like ``ssta_lists``."""
    return ssta_lists(q, k, (1, 1, k.shape[2] // kv_block), q_block, kv_block, topk=topk, window=(-1, -1, -1),
                      need_bwd=need_bwd)


def _check_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor (there is no CPU path)")
        if t.dtype != torch.bfloat16:
            raise TypeError(f"{name} must be torch.bfloat16")
        if t.dim() != 4:
            raise ValueError(f"{name} must have shape [batch, heads, seq, head_dim]")
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
    if q.shape[-1] != HEAD_DIM or k.shape[-1] != HEAD_DIM or v.shape[-1] != HEAD_DIM:
        raise ValueError("head_dim must be 128")
    if k.shape != v.shape:
        raise ValueError("k and v must have the same shape")
    if q.shape[0] != k.shape[0]:
        raise ValueError("q and k must have the same batch size")
    if q.shape[1] % k.shape[1] != 0:
        raise ValueError("the number of query heads must be a multiple of the number of kv heads")
    if q.device != k.device or q.device != v.device:
        raise RuntimeError("q, k and v must be on the same device")


def _scale_of(softmax_scale) -> float:
    if softmax_scale is None:
        return 1.0 / math.sqrt(HEAD_DIM)
    softmax_scale = float(softmax_scale)
    if not (softmax_scale > 0.0 and math.isfinite(softmax_scale)):
        raise ValueError("softmax_scale must be positive and finite")
    return softmax_scale


def forward_with_lists(q, k, v, lists: SparseLists, softmax_scale=None, need_lse: bool = True):
    """Run the forward kernel; returns (o bf16 [B,H,Sq,128], lse fp32 [B,H,Sq]).

    ``softmax_scale`` (default 1/sqrt(128), the reference's fixed value) multiplies q k^T before the
    softmax.  With ``need_lse=False`` (inference) no log-sum-exp is written and ``lse`` is None.
    """
    _check_qkv(q, k, v)
    B, Hq, Sq, _ = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    dev = q.device
    o = _new(q)
    lse = _new((B, Hq, Sq), torch.float32, dev) if need_lse else None
    _monitor(dev).poll()
    lst = lists.fwd_list(ordered=True)
    with torch.cuda.device(dev):
        rc = _cabi.lib().fba_fwd_scaled(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                        lse.data_ptr() if need_lse else None, B, Hq, Hkv, Sq, Skv,
                                        ctypes.byref(lst), _scale_of(softmax_scale), _status(dev).data_ptr(),
                                        _stream_ptr(dev))
    _cabi.check(rc, "fba_fwd_scaled")
    _maybe_check(dev)
    return o, lse


@dataclass
class Fp8KVCache:
    """Key / value cache in e4m3 with per-(batch, kv head, block) fp32 scales (``quantize_kv``).

    ``k8``: uint8 [B, Hkv, Skv, 128]; ``v8t``: uint8 [B, Hkv, 128, Skv] (V is stored transposed);
    ``k_scale`` / ``v_scale``: fp32 [B, Hkv, Skv / scale_block].
    """

    k8: torch.Tensor
    v8t: torch.Tensor
    k_scale: torch.Tensor
    v_scale: torch.Tensor
    scale_block: int

    def dequantize(self):
        """(k, v) in fp32, [B, Hkv, Skv, 128]: what the kernel's arithmetic stands for."""
        B, Hkv, Skv, _ = self.k8.shape
        k = self.k8.view(torch.float8_e4m3fn).float() * self.k_scale.repeat_interleave(self.scale_block, dim=-1)[..., None]
        v = self.v8t.view(torch.float8_e4m3fn).float().transpose(-1, -2) * \
            self.v_scale.repeat_interleave(self.scale_block, dim=-1)[..., None]
        return k, v


def quantize_kv(k: torch.Tensor, v: torch.Tensor, scale_block: int) -> Fp8KVCache:
    """Quantise bf16 K and V [B, Hkv, Skv, 128] to e4m3 with one scale per block of ``scale_block``
    key rows (a multiple of 128 that divides Skv)."""
    _check_qkv(k, k, v)
    B, Hkv, Skv, _ = k.shape
    if scale_block % TILE != 0 or Skv % scale_block != 0:
        raise ValueError("scale_block must be a multiple of 128 that divides the key length")
    dev = k.device
    k8 = torch.empty((B, Hkv, Skv, HEAD_DIM), dtype=torch.uint8, device=dev)
    v8t = torch.empty((B, Hkv, HEAD_DIM, Skv), dtype=torch.uint8, device=dev)
    ks = torch.empty((B, Hkv, Skv // scale_block), dtype=torch.float32, device=dev)
    vs = torch.empty_like(ks)
    with torch.cuda.device(dev):
        lib = _cabi.lib()
        _cabi.check(lib.fba_quantize_kv_e4m3(k.data_ptr(), k8.data_ptr(), ks.data_ptr(), B * Hkv, Skv, scale_block, 0,
                                             _stream_ptr(dev)), "fba_quantize_kv_e4m3(k)")
        _cabi.check(lib.fba_quantize_kv_e4m3(v.data_ptr(), v8t.data_ptr(), vs.data_ptr(), B * Hkv, Skv, scale_block, 1,
                                             _stream_ptr(dev)), "fba_quantize_kv_e4m3(v)")
    return Fp8KVCache(k8, v8t, ks, vs, scale_block)


def flex_block_attn_fp8kv(q, cache: Fp8KVCache, q_block_size, kv_block_size, block_mask, softmax_scale=None,
                          need_lse: bool = False):
    """Inference forward over an e4m3 key / value cache: same arguments as ``flex_block_attn_func``
    with ``cache`` in place of k and v.  Not differentiable.  Returns o (and lse when asked)."""
    if not q.is_cuda or q.dtype != torch.bfloat16 or q.dim() != 4 or q.shape[-1] != HEAD_DIM or not q.is_contiguous():
        raise ValueError("q must be a contiguous CUDA bf16 tensor [batch, heads, seq, 128]")
    B, Hq, Sq, _ = q.shape
    Bk, Hkv, Skv, _ = cache.k8.shape
    if Bk != B or Hq % Hkv != 0:
        raise ValueError("batch / head counts of q and the cache do not fit")
    lists = block_mask if isinstance(block_mask, SparseLists) else \
        build_lists(block_mask, q_block_size, kv_block_size, Sq, Skv, need_bwd=False)
    dev = q.device
    o = _new(q)
    lse = _new((B, Hq, Sq), torch.float32, dev) if need_lse else None
    _monitor(dev).poll()
    lst = lists.fwd_list(ordered=True)
    with torch.cuda.device(dev):
        rc = _cabi.lib().fba_fwd_fp8kv(q.data_ptr(), cache.k8.data_ptr(), cache.v8t.data_ptr(), cache.k_scale.data_ptr(),
                                       cache.v_scale.data_ptr(), cache.scale_block, o.data_ptr(), _ptr(lse), B, Hq, Hkv,
                                       Sq, Skv, ctypes.byref(lst), _scale_of(softmax_scale), _status(dev).data_ptr(),
                                       _stream_ptr(dev))
    _cabi.check(rc, "fba_fwd_fp8kv")
    _maybe_check(dev)
    return (o, lse) if need_lse else o


DQ_MODES = {"atomic": 0, "qmajor": 1}


def default_dq_mode() -> str:
    """dQ strategy used when a call does not name one: ``FBA_DQ_MODE`` (atomic | qmajor), else atomic."""
    mode = os.environ.get("FBA_DQ_MODE", "atomic").lower()
    if mode not in DQ_MODES:
        raise ValueError(f"FBA_DQ_MODE must be one of {sorted(DQ_MODES)}, got {mode!r}")
    return mode


def backward_with_lists(q, k, v, o, lse, dout, lists: SparseLists, softmax_scale=None, dq_mode: Optional[str] = None):
    """Run the backward kernels; returns (dq, dk, dv) in bf16.  ``softmax_scale`` must be the
    forward's.

    ``dq_mode``: "atomic" (default) -- the key-major kernel adds dQ partials into an fp32
    accumulator with vector reductions (fastest; dQ is reproducible to fp32 rounding only);
    "qmajor" -- a second, query-major kernel accumulates dQ in tensor memory and writes it once
    (bit-reproducible dQ, no fp32 accumulator; more tensor-core work).  None = ``FBA_DQ_MODE``.
    """
    _check_qkv(q, k, v)
    mode = default_dq_mode() if dq_mode is None else dq_mode
    if mode not in DQ_MODES:
        raise ValueError(f"dq_mode must be one of {sorted(DQ_MODES)}")
    B, Hq, Sq, _ = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    dev = q.device
    if dout.dtype != torch.bfloat16:
        dout = dout.to(torch.bfloat16)
    dout = dout.contiguous()
    o = o.contiguous()
    lse = lse.reshape(B, Hq, Sq).contiguous()
    if lse.dtype != torch.float32:
        raise TypeError("lse must be torch.float32")
    dq, dk, dv = _new(q), _new(k), _new(v)
    n1, n2 = ctypes.c_uint64(0), ctypes.c_uint64(0)
    _cabi.check(_cabi.lib().fba_bwd_scratch_bytes(B, Hq, Sq, ctypes.byref(n1), ctypes.byref(n2)),
                "fba_bwd_scratch_bytes")
    lse_delta = _new((n1.value // 4,), torch.float32, dev)
    dq_accum = _new((n2.value // 4,), torch.float32, dev) if mode == "atomic" else None
    _monitor(dev).poll()
    lst = lists.bwd_list(Hq, Hkv)
    q2k = lists.fwd_list(ordered=True) if mode == "qmajor" else None
    with torch.cuda.device(dev):
        rc = _cabi.lib().fba_bwd_ex(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                    dout.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                    B, Hq, Hkv, Sq, Skv, ctypes.byref(lst),
                                    ctypes.byref(q2k) if q2k is not None else None, _scale_of(softmax_scale),
                                    DQ_MODES[mode], lse_delta.data_ptr(), _ptr(dq_accum), _status(dev).data_ptr(),
                                    _stream_ptr(dev))
    _cabi.check(rc, "fba_bwd_ex")
    _maybe_check(dev)
    return dq, dk, dv


def _mask_ptr(m: Optional[torch.Tensor], like: torch.Tensor):
    if m is None:
        return None, None
    if m.dtype != torch.bool:
        raise TypeError("block_mask must be a torch.bool tensor")
    if m.device != like.device:
        raise RuntimeError("block_mask must be on the device of q (there is no CPU path)")
    m = m.contiguous()
    return m, m.data_ptr()


def _attn_workspace(B, Hq, Hkv, Sq, Skv, q_block_size, kv_block_size, mask_dim, backward, dev):
    n = ctypes.c_uint64(0)
    _cabi.check(_cabi.lib().fba_attn_workspace_bytes(B, Hq, Hkv, Sq, Skv, q_block_size, kv_block_size, mask_dim,
                                                     1 if backward else 0, ctypes.byref(n)),
                "fba_attn_workspace_bytes")
    return torch.empty((max(n.value, 256),), dtype=torch.uint8, device=dev), n.value


def _flex_block_attn_forward(q, k, v, q_block_size, kv_block_size, block_mask, small_block_mask=None,
                             use_small_block_mode=False):
    """Same call shape as the reference pass-through (interface.py:6-8); returns (o, lse).

    Binds ``fba_attn_forward``, the C entry point that stands where the reference extension's
    ``attn_forward`` stood: the bool masks go in as they are (``small_block_mask`` is the mask at
    [Sq/q_block, Skv/kv_block] granularity and is the one used when ``use_small_block_mode`` is
    set; ``block_mask`` is then the pooled mask, which this implementation does not need).
    ``lse`` is fp32 [B, H, Sq, 1], natural log.
    """
    _check_qkv(q, k, v)
    B, Hq, Sq, _ = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    dev = q.device
    bm, bm_ptr = _mask_ptr(block_mask, q)
    sm, sm_ptr = _mask_ptr(small_block_mask, q)
    fine = sm if (use_small_block_mode and sm is not None) else bm
    if fine is None or fine.dim() not in (2, 4):
        raise ValueError("block_mask must have 2 or 4 dimensions")
    o = _new(q)
    lse = _new((B, Hq, Sq), torch.float32, dev)
    ws, ws_bytes = _attn_workspace(B, Hq, Hkv, Sq, Skv, q_block_size, kv_block_size, fine.dim(), False, dev)
    _monitor(dev).poll()
    with torch.cuda.device(dev):
        rc = _cabi.lib().fba_attn_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                          B, Hq, Hkv, Sq, Skv, q_block_size, kv_block_size, bm_ptr, sm_ptr,
                                          fine.dim(), 1 if use_small_block_mode else 0, ws.data_ptr(), ws_bytes,
                                          _status(dev).data_ptr(), _stream_ptr(dev))
    _cabi.check(rc, "fba_attn_forward")
    _maybe_check(dev)
    return o, lse.unsqueeze(-1)


def _flex_block_attn_backward(q, k, v, o, lse, do, q_block_size, kv_block_size, block_mask,
                              small_block_mask=None, use_small_block_mode=False):
    """Same call shape as the reference pass-through (interface.py:10-12); returns (dq, dk, dv).

    Binds ``fba_attn_backward``.  Like the reference's, the masks arrive TRANSPOSED
    ([.., Skv/kv_block, Sq/q_block], reference interface.py:85-86).
    """
    _check_qkv(q, k, v)
    B, Hq, Sq, _ = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    dev = q.device
    bm, bm_ptr = _mask_ptr(block_mask, q)
    sm, sm_ptr = _mask_ptr(small_block_mask, q)
    fine = sm if (use_small_block_mode and sm is not None) else bm
    if fine is None or fine.dim() not in (2, 4):
        raise ValueError("block_mask must have 2 or 4 dimensions")
    if do.dtype != torch.bfloat16:
        do = do.to(torch.bfloat16)
    do = do.contiguous()
    o = o.contiguous()
    lse = lse.reshape(B, Hq, Sq).contiguous()
    if lse.dtype != torch.float32:
        raise TypeError("lse must be torch.float32")
    dq, dk, dv = _new(q), _new(k), _new(v)
    ws, ws_bytes = _attn_workspace(B, Hq, Hkv, Sq, Skv, q_block_size, kv_block_size, fine.dim(), True, dev)
    _monitor(dev).poll()
    with torch.cuda.device(dev):
        rc = _cabi.lib().fba_attn_backward(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                           do.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                           B, Hq, Hkv, Sq, Skv, q_block_size, kv_block_size, bm_ptr, sm_ptr,
                                           fine.dim(), 1 if use_small_block_mode else 0, ws.data_ptr(), ws_bytes,
                                           _status(dev).data_ptr(), _stream_ptr(dev))
    _cabi.check(rc, "fba_attn_backward")
    _maybe_check(dev)
    return dq, dk, dv


class FlexBlockAttnFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, q_block_size, kv_block_size, block_mask, is_grad_enabled, softmax_scale=None):
        _scale_of(softmax_scale)   # reject a bad scale before anything else
        assert q_block_size % 16 == 0, f"q_block_size ({q_block_size}) must be divisible by 16"
        assert kv_block_size % 64 == 0, f"kv_block_size ({kv_block_size}) must be divisible by 64"
        assert kv_block_size % q_block_size == 0 or q_block_size % kv_block_size == 0, \
            f"kv_block_size ({kv_block_size}) must be divisible by q_block_size ({q_block_size}), or vice versa."
        _, _, q_seq_len, _ = q.shape
        _, _, kv_seq_len, _ = k.shape
        assert q_seq_len % q_block_size == 0, \
            f"q_seq_len ({q_seq_len}) must be divisible by q_block_size ({q_block_size})"
        assert kv_seq_len % kv_block_size == 0, \
            f"kv_seq_len ({kv_seq_len}) must be divisible by kv_block_size ({kv_block_size})"
        prebuilt = block_mask if isinstance(block_mask, SparseLists) else None
        if prebuilt is not None:
            # lists built ahead of time (sta_lists / ssta_lists / build_lists) instead of a bool mask
            assert (prebuilt.q_block, prebuilt.kv_block) == (q_block_size, kv_block_size), \
                "the lists were built for other block sizes"
            assert prebuilt.mask_dim == 2 or (prebuilt.B, prebuilt.H) == (q.shape[0], q.shape[1]), \
                "per-(batch, head) lists must have the batch and head sizes of q"
            assert prebuilt.fwd_idx.device == q.device, "the lists live on another device than q"
            q_block_num, kv_block_num = prebuilt.nQ, prebuilt.nK
        elif block_mask.dim() == 2:
            q_block_num, kv_block_num = block_mask.shape
        else:
            _, _, q_block_num, kv_block_num = block_mask.shape
            assert block_mask.shape[0] == q.shape[0] and block_mask.shape[1] == q.shape[1], \
                "a 4-D block_mask must have the batch and head sizes of q"
        assert q_block_size * q_block_num == q_seq_len, \
            f"q_block_size ({q_block_size}) * q_block_num ({q_block_num}) must equal q_seq_len ({q_seq_len}"
        assert kv_block_size * kv_block_num == kv_seq_len, \
            f"kv_block_size ({kv_block_size}) * kv_block_num ({kv_block_num}) must equal kv_seq_len ({kv_seq_len}"

        is_grad = is_grad_enabled and any(x.requires_grad for x in [q, k, v])
        if prebuilt is not None:
            lists = prebuilt
            assert not is_grad or lists.bwd_idx is not None, "these lists were built without the key-major direction"
        else:
            lists = build_lists(block_mask, q_block_size, kv_block_size, q_seq_len, kv_seq_len, need_bwd=is_grad)
        o, lse = forward_with_lists(q, k, v, lists, softmax_scale, need_lse=is_grad)
        if is_grad:
            ctx.save_for_backward(q, k, v, o, lse)
            ctx.lists = lists
            ctx.softmax_scale = softmax_scale
        return o

    @staticmethod
    def backward(ctx, dout, *args):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = backward_with_lists(q, k, v, o, lse, dout, ctx.lists, ctx.softmax_scale)
        return dq, dk, dv, None, None, None, None, None


def flex_block_attn_func(q, k, v, q_block_size, kv_block_size, block_mask, softmax_scale=None):
    """Block-sparse attention, drop-in for the reference's function of the same name.

    Args:
        q: [batch, heads, q_seq_len, 128] bf16 CUDA tensor
        k, v: [batch, kv_heads, kv_seq_len, 128] bf16 CUDA tensors (heads % kv_heads == 0)
        q_block_size: query block size (multiple of 16)
        kv_block_size: key/value block size (multiple of 64; one block size divides the other)
        block_mask: bool [q_seq_len/q_block_size, kv_seq_len/kv_block_size] or
            [batch, heads, ...same...]; True = the query block attends to the key block.
            (Extension: a ``SparseLists`` from ``build_lists`` / ``sta_lists`` / ``ssta_lists`` is
            accepted in its place and skips the compaction.)
        softmax_scale: extension, not in the reference (which fixes 1/sqrt(128)): factor applied
            to q k^T before the softmax; None = 1/sqrt(128).  Without grad mode (inference) the
            forward also skips writing the log-sum-exp.

    Returns:
        [batch, heads, q_seq_len, 128] bf16; differentiable w.r.t. q, k and v.
    """
    if (q.shape[2] < TILE or k.shape[2] < TILE) and isinstance(block_mask, torch.Tensor):
        return _short_sequence_call(q, k, v, q_block_size, kv_block_size, block_mask, softmax_scale)
    return FlexBlockAttnFunc.apply(q, k, v, q_block_size, kv_block_size, block_mask, torch.is_grad_enabled(),
                                   softmax_scale)


def _short_sequence_call(q, k, v, q_block_size, kv_block_size, block_mask, softmax_scale):
    """Sequences shorter than one 128-row tile (the reference accepts e.g. one 64-row block,
    flex_block_attn_interface.py:19; the kernels want at least 128 rows): pad q, k, v with whole zero
    blocks up to 128 rows, give the added blocks an all-False mask, run, and cut the padding off again.
    The pad and the slice are torch ops, so gradients flow through them."""
    Sq, Skv = q.shape[2], k.shape[2]
    assert Sq % q_block_size == 0, f"q_seq_len ({Sq}) must be divisible by q_block_size ({q_block_size})"
    assert Skv % kv_block_size == 0, f"kv_seq_len ({Skv}) must be divisible by kv_block_size ({kv_block_size})"
    Sq2 = Sq if Sq >= TILE else q_block_size * -(-TILE // q_block_size)
    Skv2 = Skv if Skv >= TILE else kv_block_size * -(-TILE // kv_block_size)
    pad = torch.nn.functional.pad
    q2 = pad(q, (0, 0, 0, Sq2 - Sq))
    k2 = pad(k, (0, 0, 0, Skv2 - Skv))
    v2 = pad(v, (0, 0, 0, Skv2 - Skv))
    nQ, nK = block_mask.shape[-2:]
    m2 = pad(block_mask, (0, Skv2 // kv_block_size - nK, 0, Sq2 // q_block_size - nQ), value=False)
    out = FlexBlockAttnFunc.apply(q2.contiguous(), k2.contiguous(), v2.contiguous(), q_block_size, kv_block_size,
                                  m2.contiguous(), torch.is_grad_enabled(), softmax_scale)
    return out[:, :, :Sq]
