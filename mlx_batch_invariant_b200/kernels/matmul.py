"""Batch-invariant dense matmul ``a @ b`` for 2-D ``b`` (host wrapper).

Mirrors batch_invariant_matmul / launch_tiled of the reference
(mlx_batch_invariant/kernels/matmul.py:279-340): K is cut into fixed groups of
GROUP_K = 256, each group partial starts from zero, the fp32 partials are folded
left to right, and the launch shape (split: one CTA per K group plus a combine
kernel; fused: one CTA folds all groups) depends on M while the arithmetic does not.
``b`` is read through its strides, so the ``W.T`` view nn.Linear passes is consumed
in place.
"""

from __future__ import annotations

import torch

from .. import _lib
from ._util import adopt, dtype_code, give_back, require_cuda, rows_16b

GROUP_K = 256

_PATHS = {"auto": _lib.PATH_AUTO, "split": _lib.PATH_SPLIT, "fused": _lib.PATH_FUSED, "fold": _lib.PATH_SPLIT_FOLD}


def _launch_shape(path: str, batch_tile: int | None, M: int, N: int, K: int, ws_bytes_auto: int, dev: torch.device):
    """(path word, workspace tensor or None, workspace bytes) for a call. The workspace is the stream's
    persistent one, whose head holds the zeroed arrival counters of the in-kernel fold."""
    G = (K + GROUP_K - 1) // GROUP_K
    nbytes = ws_bytes_auto if path in ("auto", "fused") else _lib.COUNTER_BYTES + G * M * N * 4
    word = _PATHS[path] | _lib.WS_ZEROED | (_lib.batch_tile(batch_tile) if batch_tile else 0)
    ws = _lib.matmul_workspace(dev, nbytes) if nbytes else None
    return word, ws, (ws.numel() if ws is not None else 0)


def _weight_is_tensor_core(b: torch.Tensor, K: int) -> bool:
    """The predicate bi_matmul applies to the weight (16-bit, rows of K contiguous elements
    that TMA can address). Used only to decide whether the activation needs an aligned copy."""
    es = b.element_size()
    return (b.dtype != torch.float32 and b.stride(0) == 1 and K % 8 == 0 and b.data_ptr() % 16 == 0
            and (b.shape[1] == 1 or ((b.stride(1) * es) % 16 == 0 and b.stride(1) >= K)))


def batch_invariant_matmul(a, b, *, path: str = "auto", batch_tile: int | None = None, awaiting=None, bias=None, push=None,
                           rope=None):
    """``a @ b`` with a batch-invariant reduction order.

    ``a`` may have extra leading dims (flattened into M); ``b`` must be 2-D (a transposed
    view is fine). fp32 accumulation; the output dtype is the promoted input dtype.
    ``path`` ("auto", "split", "fused", "fold") and ``batch_tile`` (16, 32, 64, 128 batch rows per tile)
    force a launch shape; all give the same bits. ``awaiting`` (flags pointer, epoch pointer, rank, world) says
    that ``a`` is the destination of a peer gather nobody has waited for yet: the kernel waits for it itself,
    after it has started streaming the weight (runner/peer.py). ``bias`` ([N], the output dtype) is added to the
    rounded product in the kernel's epilogue: the bits of ``batch_invariant_matmul(a, b) + bias``.
    ``push`` (destination table, flag table, counters pointer, rank, world, wait -- ``PushGather.sink()``): the
    product is this rank's column slice of a gathered activation; the fold kernel stores it into every rank's
    destination and shakes hands (``bi_matmul_push``); nothing is returned.
    ``rope`` (the arguments of ``bi_rope_append`` after ``qkv``, up to ``capacity``): the product is a decoder's qkv
    projection; the fold kernel rotates q and k and appends k and v to the cache itself (``bi_matmul_rope``);
    nothing is returned.
    """
    at, foreign = adopt(a)
    bt, _ = adopt(b)
    if bt.ndim != 2:
        raise ValueError("batch_invariant_matmul: b must be 2-D")
    if at.ndim < 1:
        raise ValueError("batch_invariant_matmul: a must have at least one dim")
    lead = at.shape[:-1]
    K = at.shape[-1]
    if K != bt.shape[0]:
        raise ValueError(f"shape mismatch {tuple(at.shape)} @ {tuple(bt.shape)}")
    dev = require_cuda(at, bt)
    N = bt.shape[1]
    out_dtype = torch.result_type(at, bt)
    code = dtype_code(out_dtype)
    a2 = at.reshape(-1, K)
    if a2.dtype != out_dtype:
        a2 = a2.to(out_dtype)
    if bt.dtype != out_dtype:
        bt = bt.to(out_dtype)
    M = a2.shape[0]
    if K == 0:
        return give_back(torch.zeros((*lead, N), dtype=out_dtype, device=dev), a, foreign)
    if M > 0 and _weight_is_tensor_core(bt, K):
        a2 = rows_16b(a2)
    lib = _lib.load()
    if rope is not None:
        if bias is not None or push is not None or awaiting is not None or M == 0:
            raise ValueError("rope cannot be combined with bias, push, awaiting or an empty batch")
        with torch.cuda.device(dev):
            word, ws, nbytes = _launch_shape("split", batch_tile, M, N, K, 0, dev)
            _lib.check(lib.bi_matmul_rope(a2.data_ptr(), bt.data_ptr(), _lib.ptr(ws), nbytes, M, N, K,
                                          a2.stride(0) if M > 1 else K, a2.stride(1), bt.stride(0), bt.stride(1), code, word,
                                          _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev), *rope))
        return None
    if push is not None:
        if bias is not None or M == 0:
            raise ValueError("push cannot be combined with bias or an empty batch")
        with torch.cuda.device(dev):
            word, ws, nbytes = _launch_shape("split", batch_tile, M, N, K, 0, dev)
            aw = awaiting[:2] if awaiting is not None else (None, None)
            _lib.check(lib.bi_matmul_push(a2.data_ptr(), bt.data_ptr(), _lib.ptr(ws), nbytes, M, N, K,
                                          a2.stride(0) if M > 1 else K, a2.stride(1), bt.stride(0), bt.stride(1), code, word,
                                          _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev), *aw, *push))
        return None
    out = torch.empty((M, N), dtype=out_dtype, device=dev)
    with torch.cuda.device(dev):
        word, ws, nbytes = _launch_shape(path, batch_tile, M, N, K, lib.bi_matmul_workspace_bytes(M, N, K, code), dev)
        args = (a2.data_ptr(), bt.data_ptr(), out.data_ptr(), _lib.ptr(ws), nbytes, M, N, K,
                a2.stride(0) if M > 1 else K, a2.stride(1), bt.stride(0), bt.stride(1), code,
                word, _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))
        if bias is not None:
            bias_t = adopt(bias)[0]
            if bias_t.shape != (N,) or bias_t.dtype != out_dtype or not bias_t.is_cuda or awaiting is not None:
                raise ValueError("bias must be a CUDA tensor of shape [N] in the output dtype (and cannot be combined with awaiting)")
            bias_t = bias_t.contiguous()
            _lib.check(lib.bi_matmul_bias(args[0], args[1], bias_t.data_ptr(), *args[2:]))
        else:
            _lib.check(lib.bi_matmul(*args) if awaiting is None else lib.bi_matmul_awaiting(*args, *awaiting))
    return give_back(out.reshape(*lead, N), a, foreign)
