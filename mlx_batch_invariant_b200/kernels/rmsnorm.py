"""Batch-invariant RMSNorm (host wrapper).

Mirrors batch_invariant_rms_norm of the reference (mlx_batch_invariant/kernels/rmsnorm.py:64-79):
one CTA of 256 threads per row, fixed-stride partial sums, fixed tree, so a row's
result is the same alone or among thousands.
"""

from __future__ import annotations

import torch

from .. import _lib
from ._util import adopt, dtype_code, give_back, require_cuda


def batch_invariant_rms_norm(x, weight, eps: float):
    """``x * rsqrt(mean(x^2, -1) + eps) * weight`` over the last axis; ``weight`` may be None."""
    xt, foreign = adopt(x)
    wt = None if weight is None else adopt(weight)[0]
    dev = require_cuda(xt, wt)
    code = dtype_code(xt.dtype)
    D = xt.shape[-1]
    if wt is not None:
        if wt.shape != (D,):
            raise ValueError(f"weight shape {tuple(wt.shape)} does not match last dim {D}")
        if wt.dtype != xt.dtype:
            wt = wt.to(xt.dtype)
        wt = wt.contiguous()
    rows = xt.numel() // D if D else 0
    x2 = xt.reshape(rows, D).contiguous()
    out = torch.empty_like(x2)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().bi_rms_norm(x2.data_ptr(), _lib.ptr(wt), out.data_ptr(), rows, D, float(eps), code,
                                           _lib.stream_ptr(dev)))
    return give_back(out.reshape(xt.shape), x, foreign)
