"""The MLX half of the mode: wrappers with MLX's signatures for the six symbols the reference patches
(mlx_batch_invariant/_mode.py:37-50 there).

An ``mx.array`` reaches the kernels through DLPack (no copy): the wrapper views every array argument as a
torch tensor, applies the same support rules as the torch entry points in ``ops``, and hands the result
back as an MLX array. Whatever the kernels do not take -- arrays that do not export DLPack, arrays that are
not on a CUDA device, unsupported shapes or options -- is counted as a fallback under the reference's key
strings and then goes to the *MLX* stock callable that was installed before the mode was entered, exactly
as the reference falls back to stock MLX (mlx_batch_invariant/ops.py:36-39, 46-95 there); strict mode raises
instead.
"""

from __future__ import annotations

import torch

from . import ops
from .kernels import (
    batch_invariant_attention,
    batch_invariant_matmul,
    batch_invariant_quantized_matmul,
    batch_invariant_rms_norm,
)
from .kernels import attention as _attn
from .kernels import quantized as _quant
from .kernels._util import give_back


def _view(x):
    """torch view of an array that exports DLPack, else None (None stays None only for optional arguments)."""
    if isinstance(x, torch.Tensor):
        return x
    if hasattr(x, "__dlpack__"):
        try:
            return torch.from_dlpack(x)
        except Exception:
            return None
    return None


def _call(orig, args, kwargs, stream):
    if stream is not None:
        kwargs = dict(kwargs, stream=stream)
    return orig(*args, **kwargs)


def patches(mx) -> list:
    """(owner, attribute, replacement) triples for ``mlx.core`` module ``mx``. The stock callables are read
    here, at the moment the mode is entered, so a fallback reaches whatever was installed before."""
    o_matmul, o_addmm, o_qmm = mx.matmul, mx.addmm, mx.quantized_matmul
    o_rms, o_sdpa, o_arr_matmul = mx.fast.rms_norm, mx.fast.scaled_dot_product_attention, mx.array.__matmul__

    def _mm(a, b, op):
        ta, tb = _view(a), _view(b)
        if ta is None or tb is None:
            return None, None, "non-2d-rhs-or-non-float"
        return ta, tb, ops._mm_reason(ta, tb)

    def matmul(a, b, *, stream=None):
        ta, tb, reason = _mm(a, b, "matmul")
        if reason is None:
            ops.handled["matmul"] += 1
            return give_back(batch_invariant_matmul(ta, tb), a, True)
        ops._fallback("matmul", reason)
        return _call(o_matmul, (a, b), {}, stream)

    def array_matmul(self, other):
        ta, tb, reason = _mm(self, other, "matmul")
        if reason is None:
            ops.handled["matmul"] += 1
            return give_back(batch_invariant_matmul(ta, tb), self, True)
        ops._fallback("matmul", reason)
        return o_arr_matmul(self, other)

    def addmm(c, a, b, /, alpha: float = 1.0, beta: float = 1.0, *, stream=None):
        ta, tb, reason = _mm(a, b, "addmm")
        tc = _view(c)
        if reason is None and tc is None:
            reason = "non-2d-rhs-or-non-float"
        if reason is None:
            ops.handled["addmm"] += 1
            prod = batch_invariant_matmul(ta, tb)
            if alpha != 1.0:
                prod = prod * alpha
            return give_back(prod + (tc if beta == 1.0 else tc * beta), a, True)
        ops._fallback("addmm", reason)
        return _call(o_addmm, (c, a, b), {"alpha": alpha, "beta": beta}, stream)

    def quantized_matmul(x, w, /, scales, biases=None, transpose: bool = True, group_size=None, bits=None,
                         mode: str = "affine", *, stream=None):
        gs = 64 if group_size is None else group_size
        nb = 4 if bits is None else bits
        tx, tw, ts = _view(x), _view(w), _view(scales)
        tb = None if biases is None else _view(biases)
        ok = (tx is not None and tw is not None and ts is not None and (biases is None or tb is not None)
              and _quant.supports(tx, tw, ts, tb, transpose, gs, nb, mode) and ops._on_cuda(tx, tw, ts, tb))
        if ok:
            ops.handled["quantized_matmul"] += 1
            return give_back(batch_invariant_quantized_matmul(tx, tw, ts, tb, group_size=gs, bits=nb), x, True)
        ops._fallback("quantized_matmul", f"{mode}-{nb}bit-g{gs}-{'T' if transpose else 'N'}")
        kw = {"scales": scales, "biases": biases, "transpose": transpose, "group_size": group_size, "bits": bits}
        if mode != "affine":
            kw["mode"] = mode
        return _call(o_qmm, (x, w), kw, stream)

    def rms_norm(x, weight, eps: float, *, stream=None):
        tx = _view(x)
        tw = None if weight is None else _view(weight)
        if tx is not None and (weight is None or tw is not None) and ops._is_float(tx) and ops._on_cuda(tx, tw):
            ops.handled["rms_norm"] += 1
            return give_back(batch_invariant_rms_norm(tx, tw, eps), x, True)
        ops._fallback("rms_norm", "non-float" if tx is None or not ops._is_float(tx) else "not-cuda")
        return _call(o_rms, (x, weight, eps), {}, stream)

    def scaled_dot_product_attention(q, k, v, *, scale: float, mask=None, sinks=None, stream=None, **extra):
        tq, tk, tv = _view(q), _view(k), _view(v)
        plain_mask = mask is None or isinstance(mask, str)
        if (tq is not None and tk is not None and tv is not None and plain_mask
                and _attn.supports(tq, tk, tv, mask, sinks) and ops._on_cuda(tq, tk, tv)):
            ops.handled["sdpa_decode" if tq.shape[2] == 1 else "sdpa_prefill"] += 1
            return give_back(batch_invariant_attention(tq, tk, tv, scale=scale, mask=mask), q, True)
        ops._fallback("sdpa", "sinks-or-shape" if plain_mask else "array-mask")
        kw = dict(extra, scale=scale, mask=mask)
        if sinks is not None:
            kw["sinks"] = sinks
        return _call(o_sdpa, (q, k, v), kw, stream)

    return [
        (mx, "matmul", matmul),
        (mx, "addmm", addmm),
        (mx, "quantized_matmul", quantized_matmul),
        (mx.fast, "rms_norm", rms_norm),
        (mx.fast, "scaled_dot_product_attention", scaled_dot_product_attention),
        (mx.array, "__matmul__", array_matmul),
    ]
