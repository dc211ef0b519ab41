"""Batch-invariant LayerNorm (host wrapper).

The reference has no LayerNorm kernel yet; it names one as the next norm to cover (README.md:261-263 there).
This one follows its RMSNorm (mlx_batch_invariant/kernels/rmsnorm.py:19-47, 64-79): one CTA of 256 threads per
row, fixed-stride fp32 partials and a fixed tree -- once for the mean, once for the squared deviations -- so a
row's result is the same alone or among thousands.
"""

from __future__ import annotations

import torch

from .. import _lib
from ._util import adopt, dtype_code, give_back, require_cuda


def batch_invariant_layer_norm(x, weight, bias, eps: float):
    """``(x - mean) * rsqrt(var + eps) * weight + bias`` over the last axis; ``weight`` / ``bias`` may be None."""
    xt, foreign = adopt(x)
    wt = None if weight is None else adopt(weight)[0]
    bt = None if bias is None else adopt(bias)[0]
    dev = require_cuda(xt, wt, bt)
    code = dtype_code(xt.dtype)
    D = xt.shape[-1]
    for name, t in (("weight", wt), ("bias", bt)):
        if t is not None and t.shape != (D,):
            raise ValueError(f"{name} shape {tuple(t.shape)} does not match last dim {D}")
    wt = None if wt is None else wt.to(xt.dtype).contiguous()
    bt = None if bt is None else bt.to(xt.dtype).contiguous()
    rows = xt.numel() // D if D else 0
    x2 = xt.reshape(rows, D).contiguous()
    out = torch.empty_like(x2)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().bi_layer_norm(x2.data_ptr(), _lib.ptr(wt), _lib.ptr(bt), out.data_ptr(), rows, D, float(eps),
                                             code, _lib.stream_ptr(dev)))
    return give_back(out.reshape(xt.shape), x, foreign)
