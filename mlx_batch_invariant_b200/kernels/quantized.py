"""Batch-invariant affine quantized matmul ``y[M, N] = x[M, K] @ W[N, K].T`` (host wrapper).

``W`` is the packed affine format of the reference (mlx_batch_invariant/kernels/quantized.py:3-7):
``bits``-wide unsigned codes packed low to high in uint32 words, one scale and bias
per ``group_size`` consecutive codes of a row::

    w[n, k] = code(n, k) * scales[n, k // group_size] + biases[n, k // group_size]

The kernel dequantizes while it stages the weight tile (fp32 fma, one rounding to the
input dtype) and then runs the dense kernel's MMA sequence and fold.
"""

from __future__ import annotations

import torch

from .. import _lib
from ._util import adopt, dtype_code, give_back, require_cuda, rows_16b
from .matmul import _launch_shape

SUPPORTED_BITS = (4, 8)
SUPPORTED_GROUPS = (32, 64, 128)


def supports(x, w, scales, biases, transpose, group_size, bits, mode) -> bool:
    """Same predicate as the reference (mlx_batch_invariant/kernels/quantized.py:91-103)."""
    return (
        mode == "affine"
        and bool(transpose)
        and biases is not None
        and bits in SUPPORTED_BITS
        and group_size in SUPPORTED_GROUPS
        and isinstance(x, torch.Tensor) and x.is_floating_point() and x.dtype in _lib.DTYPE_CODE
        and isinstance(w, torch.Tensor) and w.dtype in (torch.uint32, torch.int32) and w.ndim == 2
        and scales.ndim == 2 and biases.ndim == 2
        and x.shape[-1] % group_size == 0
        and w.shape[1] * (32 // bits) == x.shape[-1]
    )


_STAGES = {None: 0, "smem": _lib.QMM_STAGE_SMEM, "tmem": _lib.QMM_STAGE_TMEM}


def batch_invariant_quantized_matmul(x, w, scales, biases, *, group_size: int, bits: int, path: str = "auto",
                                     batch_tile: int | None = None, stage: str | None = None, awaiting=None, push=None,
                                     rope=None):
    """``x @ dequant(w).T``. ``path`` / ``batch_tile`` force a launch shape as for the dense matmul; ``stage``
    ("smem", "tmem") forces how the dequantized weight reaches the tensor core. All give the same bits.
    ``awaiting`` / ``push`` / ``rope``: as for ``batch_invariant_matmul`` (``bi_qmm_awaiting`` / ``bi_qmm_push`` /
    ``bi_qmm_rope``)."""
    xt, foreign = adopt(x)
    wt, st, bt = adopt(w)[0], adopt(scales)[0], adopt(biases)[0]
    dev = require_cuda(xt, wt, st, bt)
    if bits not in SUPPORTED_BITS or group_size not in SUPPORTED_GROUPS:
        raise ValueError(f"unsupported quantization: bits={bits}, group_size={group_size}")
    lead = xt.shape[:-1]
    K = xt.shape[-1]
    N = wt.shape[0]
    if wt.ndim != 2 or wt.shape[1] * (32 // bits) != K:
        raise ValueError(f"packed weight shape {tuple(wt.shape)} does not match K={K} at {bits} bits")
    if K % group_size or st.shape != (N, K // group_size) or bt.shape != st.shape:
        raise ValueError(f"scales/biases shape {tuple(st.shape)} does not match (N={N}, K/group_size={K // group_size})")
    dt = xt.dtype
    code = dtype_code(dt)
    x2 = rows_16b(xt.reshape(-1, K))
    M = x2.shape[0]
    st = st.to(dt).contiguous()
    bt = bt.to(dt).contiguous()
    wt = wt.contiguous()
    lib = _lib.load()
    if rope is not None:
        if push is not None or awaiting is not None or M == 0:
            raise ValueError("rope cannot be combined with push, awaiting or an empty batch")
        with torch.cuda.device(dev):
            word, ws, nbytes = _launch_shape("split", batch_tile, M, N, K, 0, dev)
            _lib.check(lib.bi_qmm_rope(x2.data_ptr(), wt.data_ptr(), st.data_ptr(), bt.data_ptr(), _lib.ptr(ws), nbytes, M, N, K,
                                       x2.stride(0) if M > 1 else K, group_size, bits, code, word | _STAGES[stage],
                                       _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev), *rope))
        return None
    if push is not None:
        if M == 0:
            raise ValueError("push cannot be combined with an empty batch")
        with torch.cuda.device(dev):
            word, ws, nbytes = _launch_shape("split", batch_tile, M, N, K, 0, dev)
            aw = awaiting[:2] if awaiting is not None else (None, None)
            _lib.check(lib.bi_qmm_push(x2.data_ptr(), wt.data_ptr(), st.data_ptr(), bt.data_ptr(), _lib.ptr(ws), nbytes, M, N, K,
                                       x2.stride(0) if M > 1 else K, group_size, bits, code, word | _STAGES[stage],
                                       _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev), *aw, *push))
        return None
    out = torch.empty((M, N), dtype=dt, device=dev)
    with torch.cuda.device(dev):
        word, ws, nbytes = _launch_shape(path, batch_tile, M, N, K, lib.bi_qmm_workspace_bytes(M, N, K, code), dev)
        args = (x2.data_ptr(), wt.data_ptr(), st.data_ptr(), bt.data_ptr(), out.data_ptr(),
                _lib.ptr(ws), nbytes, M, N, K, x2.stride(0) if M > 1 else K, group_size, bits, code,
                word | _STAGES[stage], _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))
        _lib.check(lib.bi_qmm(*args) if awaiting is None else lib.bi_qmm_awaiting(*args, *awaiting))
    return give_back(out.reshape(*lead, N), x, foreign)
