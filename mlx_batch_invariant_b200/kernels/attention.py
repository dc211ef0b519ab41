"""Batch-invariant attention with a fixed KV split size (host wrappers).

Mirrors the reference wrappers (mlx_batch_invariant/kernels/attention.py:299-397): keys in
fixed splits of SPLIT_SIZE = 256, key-by-key online softmax inside a split, split
partials merged left to right; decode (T_q == 1) and prefill run the same per-key and
merge code, so a token's bits do not depend on which of them produced it.

Extension over the reference: ``kv_lens`` (int32 [B]) gives each sequence of a decode
batch its own key count, and K/V may be strided views of a larger cache (no copy).
A row's arithmetic depends on its own length only.
"""

from __future__ import annotations

import torch

from .. import _lib
from ._util import adopt, dtype_code, give_back, require_cuda

SPLIT_SIZE = 256
SUPPORTED_HEAD_DIMS = (32, 64, 128, 256)


def supports(q, k, v, mask, sinks) -> bool:
    """Same predicate as the reference (mlx_batch_invariant/kernels/attention.py:299-310), with the
    head dims this build has kernels for."""
    return (
        q.ndim == 4 and k.ndim == 4 and v.ndim == 4
        and (mask is None or (isinstance(mask, str) and mask == "causal"))
        and sinks is None
        and q.shape[1] % k.shape[1] == 0
        and k.shape == v.shape
        and q.shape[-1] == k.shape[-1]
        and q.shape[-1] in SUPPORTED_HEAD_DIMS
        and q.shape[0] == k.shape[0]
        and (mask is None or q.shape[2] <= k.shape[2])
        and q.dtype in _lib.DTYPE_CODE
    )


def _prep(q, k, v):
    qt, foreign = adopt(q)
    kt, vt = adopt(k)[0], adopt(v)[0]
    dev = require_cuda(qt, kt, vt)
    dt = qt.dtype
    if kt.dtype != dt:
        kt = kt.to(dt)
    if vt.dtype != dt:
        vt = vt.to(dt)
    return qt, kt, vt, dev, foreign


def _kv_layout(k: torch.Tensor, v: torch.Tensor):
    """K and V must share one (batch, head, key) stride triple with unit stride along D and
    16-byte aligned rows; copy if they do not."""
    per = 16 // k.element_size()

    def ok(t):
        return (t.stride(3) == 1 and t.data_ptr() % 16 == 0 and t.stride(2) >= t.shape[3]
                and all(s % per == 0 for s in t.stride()[:3]))

    if not (ok(k) and ok(v) and k.stride() == v.stride()):
        k, v = k.contiguous(), v.contiguous()
    return k, v, k.stride(0), k.stride(1), k.stride(2)


def batch_invariant_decode_attention(q, k, v, *, scale: float, split_size: int = SPLIT_SIZE, kv_lens=None, push=None):
    """T_q == 1. Per-split partials (query heads of a kv head share K/V rows), then an ordered combine.
    ``push`` (``PushGather.sink()``): the output is this rank's head slice of a gathered [B, world * Hq * D]
    activation; the combine kernel stores it into every rank's destination and shakes hands
    (``bi_attn_decode_push``); nothing is returned."""
    assert q.shape[2] == 1 and q.shape[3] % 32 == 0
    qt, kt, vt, dev, foreign = _prep(q, k, v)
    B, Hq, Tq, D = qt.shape
    _, Hkv, L, _ = kt.shape
    code = dtype_code(qt.dtype)
    qc = qt.contiguous()
    kt, vt, sb, sh, sl = _kv_layout(kt, vt)
    lens = None
    if kv_lens is not None:
        lens = adopt(kv_lens)[0].to(device=dev, dtype=torch.int32).contiguous()
        if lens.shape != (B,):
            raise ValueError(f"kv_lens must have shape ({B},), got {tuple(lens.shape)}")
    lib = _lib.load()
    nbytes = lib.bi_attn_decode_workspace_bytes(B, Hq, L, D, split_size)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
    if push is not None:
        with torch.cuda.device(dev):
            _lib.check(lib.bi_attn_decode_push(qc.data_ptr(), kt.data_ptr(), vt.data_ptr(), _lib.ptr(lens), ws.data_ptr(), nbytes,
                                               B, Hq, Hkv, L, D, sb, sh, sl, float(scale), int(split_size), code,
                                               _lib.stream_ptr(dev), *push, _lib.status_word(dev).data_ptr()))
        return None
    out = torch.empty_like(qc)
    with torch.cuda.device(dev):
        _lib.check(lib.bi_attn_decode(qc.data_ptr(), kt.data_ptr(), vt.data_ptr(), out.data_ptr(), _lib.ptr(lens),
                                      ws.data_ptr(), nbytes, B, Hq, Hkv, L, D, sb, sh, sl, float(scale),
                                      int(split_size), code, _lib.stream_ptr(dev)))
    return give_back(out, q, foreign)


def batch_invariant_paged_decode_attention(q, k_pages, v_pages, block_table, kv_lens, *, scale: float,
                                           split_size: int = SPLIT_SIZE):
    """Decode attention over a paged cache (an extension; the reference reads one contiguous cache).
    ``k_pages`` / ``v_pages``: [pages, Hkv, page_size, D]; ``block_table`` int32 [B, max_pages] names the pages of
    every sequence in order; ``kv_lens`` int32 [B]. Same bits as the same keys in a contiguous cache."""
    assert q.shape[2] == 1 and q.shape[3] == 128
    qt, kt, vt, dev, foreign = _prep(q, k_pages, v_pages)
    B, Hq, _, D = qt.shape
    _, Hkv, page, _ = kt.shape
    code = dtype_code(qt.dtype)
    qc = qt.contiguous()
    kt, vt, sp, sh, sl = _kv_layout(kt, vt)
    table = adopt(block_table)[0].to(device=dev, dtype=torch.int32).contiguous()
    lens = adopt(kv_lens)[0].to(device=dev, dtype=torch.int32).contiguous()
    if table.ndim != 2 or table.shape[0] != B or lens.shape != (B,):
        raise ValueError("block_table must be [B, max_pages] and kv_lens [B]")
    max_pages = table.shape[1]
    out = torch.empty_like(qc)
    lib = _lib.load()
    nbytes = lib.bi_attn_decode_workspace_bytes(B, Hq, max_pages * page, D, split_size)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.bi_attn_decode_paged(qc.data_ptr(), kt.data_ptr(), vt.data_ptr(), out.data_ptr(), lens.data_ptr(),
                                            table.data_ptr(), ws.data_ptr(), nbytes, B, Hq, Hkv, max_pages, page, D, sp, sh, sl,
                                            table.stride(0), float(scale), int(split_size), code, _lib.stream_ptr(dev)))
    return give_back(out, q, foreign)


def batch_invariant_prefill_attention(q, k, v, *, scale: float, causal: bool, split_size: int = SPLIT_SIZE):
    """Any T_q. Queries are right-aligned to the cache end when causal; same split loop and merge as decode."""
    assert q.shape[3] % 32 == 0
    qt, kt, vt, dev, foreign = _prep(q, k, v)
    B, Hq, Tq, D = qt.shape
    _, Hkv, L, _ = kt.shape
    code = dtype_code(qt.dtype)
    qc = qt.contiguous()
    kt, vt, sb, sh, sl = _kv_layout(kt, vt)
    out = torch.empty_like(qc)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().bi_attn_prefill(qc.data_ptr(), kt.data_ptr(), vt.data_ptr(), out.data_ptr(), B, Hq, Hkv,
                                               Tq, L, D, sb, sh, sl, float(scale), 1 if causal else 0,
                                               int(split_size), code, _lib.stream_ptr(dev)))
    return give_back(out, q, foreign)


def batch_invariant_attention(q, k, v, *, scale: float, mask=None, kv_lens=None):
    """Dispatch: decode path for T_q == 1, prefill path otherwise."""
    if q.shape[2] == 1:
        return batch_invariant_decode_attention(q, k, v, scale=scale, kv_lens=kv_lens)
    if kv_lens is not None:
        raise ValueError("kv_lens is a decode-only option")
    return batch_invariant_prefill_attention(q, k, v, scale=scale, causal=(mask == "causal"))
