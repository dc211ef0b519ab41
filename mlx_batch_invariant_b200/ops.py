"""Functional entry points with explicit fallback accounting.

Same contract as the reference (mlx_batch_invariant/ops.py:1-104): each op returns the
batch-invariant result when a kernel supports the inputs; otherwise the fallback is
counted first, then strict mode raises ``RuntimeError`` and non-strict mode runs the
stock op. ``stats()`` exposes the counters so a run can be audited: "deterministic" with
ten silent fallbacks is not deterministic.

The stock ops here are PyTorch's CUDA kernels (cuBLAS, SDPA), captured at import so the
mode's patching never recurses. There is no CPU implementation of any kernel: tensors
that are not on a CUDA device are a counted fallback like any other unsupported input.
"""

from __future__ import annotations

import math
from collections import Counter

import torch
import torch.nn.functional as F

from .kernels import (
    batch_invariant_attention,
    batch_invariant_matmul,
    batch_invariant_quantized_matmul,
    batch_invariant_rms_norm,
)
from .kernels import batch_invariant_layer_norm
from .kernels import attention as _attn
from .kernels import quantized as _quant

# Stock implementations, captured at import so patching never recurses.
_orig_matmul = torch.matmul
_orig_mm = torch.mm
_orig_addmm = torch.addmm
_orig_linear = F.linear
_orig_rms_norm = F.rms_norm
_orig_layer_norm = F.layer_norm
_orig_sdpa = F.scaled_dot_product_attention
_orig_tensor_matmul = torch.Tensor.__matmul__
_orig_tensor_rmatmul = torch.Tensor.__rmatmul__
_orig_tensor_matmul_method = torch.Tensor.matmul
_orig_tensor_mm_method = torch.Tensor.mm

handled: Counter = Counter()
fallbacks: Counter = Counter()
strict: bool = False


def _fallback(op: str, reason: str):
    fallbacks[f"{op}:{reason}"] += 1
    if strict:
        raise RuntimeError(f"batch-invariant mode: no kernel for {op} ({reason})")


def _is_float(x) -> bool:
    return isinstance(x, torch.Tensor) and x.is_floating_point() and x.dtype in (
        torch.float32, torch.float16, torch.bfloat16)


def _on_cuda(*xs) -> bool:
    return all(x.is_cuda for x in xs if isinstance(x, torch.Tensor))


def _mm_reason(a, b):
    """None when the dense kernel takes (a, b), else the fallback reason."""
    if not (_is_float(a) and _is_float(b) and b.ndim == 2 and a.ndim >= 1):
        return "non-2d-rhs-or-non-float"
    if not _on_cuda(a, b):
        return "not-cuda"
    return None


def matmul(a, b, *, stream=None, out=None):
    reason = _mm_reason(a, b) if out is None else "non-2d-rhs-or-non-float"
    if reason is None:
        handled["matmul"] += 1
        return batch_invariant_matmul(a, b)
    _fallback("matmul", reason)
    return _orig_matmul(a, b) if out is None else _orig_matmul(a, b, out=out)


def addmm(c, a, b, /, alpha: float = 1.0, beta: float = 1.0, *, stream=None):
    """``beta * c + alpha * (a @ b)``. As in the reference (mlx_batch_invariant/ops.py:54-62) the
    product is rounded to the output dtype first, then scaled and added with ordinary
    elementwise ops, which are batch-invariant by themselves."""
    reason = _mm_reason(a, b)
    if reason is None:
        handled["addmm"] += 1
        if (alpha == 1.0 and beta == 1.0 and isinstance(c, torch.Tensor) and c.is_cuda and c.ndim == 1
                and c.shape[0] == b.shape[1] and c.dtype == torch.result_type(a, b)):
            return batch_invariant_matmul(a, b, bias=c)      # a linear layer's bias: added in the kernel's epilogue, same bits
        prod = batch_invariant_matmul(a, b)
        if alpha != 1.0:
            prod = prod * alpha
        return prod + (c if beta == 1.0 else c * beta)
    _fallback("addmm", reason)
    return _orig_addmm(c, a, b, beta=beta, alpha=alpha)


def _stock_quantized_matmul(x, w, scales, biases, transpose, group_size, bits):
    """Stock path for quantized weights: dequantize with torch ops, then torch.matmul."""
    per = 32 // bits
    shifts = torch.arange(per, device=w.device, dtype=torch.int64) * bits
    codes = (w.to(torch.int64).bitwise_and(0xFFFFFFFF).unsqueeze(-1) >> shifts) & ((1 << bits) - 1)
    codes = codes.reshape(w.shape[0], -1).to(x.dtype)
    s = scales.to(x.dtype).repeat_interleave(group_size, dim=1)
    b = biases.to(x.dtype).repeat_interleave(group_size, dim=1)
    wd = codes * s + b
    return _orig_matmul(x, wd.T if transpose else wd)


def quantized_matmul(x, w, /, scales, biases=None, transpose: bool = True, group_size=None, bits=None,
                     mode: str = "affine", *, stream=None):
    gs = 64 if group_size is None else group_size
    b = 4 if bits is None else bits
    if _quant.supports(x, w, scales, biases, transpose, gs, b, mode) and _on_cuda(x, w, scales, biases):
        handled["quantized_matmul"] += 1
        return batch_invariant_quantized_matmul(x, w, scales, biases, group_size=gs, bits=b)
    _fallback("quantized_matmul", f"{mode}-{b}bit-g{gs}-{'T' if transpose else 'N'}")
    if mode != "affine" or biases is None:
        raise NotImplementedError(f"no stock implementation for quantization mode {mode!r}")
    return _stock_quantized_matmul(x, w, scales, biases, transpose, gs, b)


def rms_norm(x, weight, eps: float, *, stream=None):
    if _is_float(x) and _on_cuda(x, weight):
        handled["rms_norm"] += 1
        return batch_invariant_rms_norm(x, weight, eps)
    _fallback("rms_norm", "non-float" if not _is_float(x) else "not-cuda")
    return _orig_rms_norm(x, (x.shape[-1],), weight, eps)


def _stock_sdpa(q, k, v, scale, mask):
    """Stock attention with the reference's mask convention ("causal" is right-aligned to the
    end of the keys)."""
    Hq, Hkv = q.shape[1], k.shape[1]
    attn_mask = None
    if isinstance(mask, str) and mask == "causal":
        Tq, L = q.shape[2], k.shape[2]
        attn_mask = torch.ones(Tq, L, dtype=torch.bool, device=q.device).tril(diagonal=L - Tq)
    elif isinstance(mask, torch.Tensor):
        attn_mask = mask
    return _orig_sdpa(q, k, v, attn_mask=attn_mask, scale=scale, enable_gqa=(Hq != Hkv))


def scaled_dot_product_attention(q, k, v, *, scale: float, mask=None, sinks=None, force_fused=False, stream=None):
    if _attn.supports(q, k, v, mask, sinks) and _on_cuda(q, k, v):
        handled["sdpa_decode" if q.shape[2] == 1 else "sdpa_prefill"] += 1
        return batch_invariant_attention(q, k, v, scale=scale, mask=mask)
    _fallback("sdpa", "array-mask" if isinstance(mask, torch.Tensor) else "sinks-or-shape")
    if sinks is not None:
        raise NotImplementedError("no stock implementation for attention sinks")
    return _stock_sdpa(q, k, v, scale, mask)


# ---- adapters with PyTorch's own signatures (installed by the mode) -------------------

def torch_mm(a, b, *, out=None):
    return matmul(a, b, out=out)


def torch_tensor_matmul(self, other):
    return matmul(self, other)


def torch_tensor_rmatmul(self, other):
    return matmul(other, self)


def torch_addmm(input, mat1, mat2, *, beta=1, alpha=1, out=None):
    if out is not None:
        _fallback("addmm", "non-2d-rhs-or-non-float")
        return _orig_addmm(input, mat1, mat2, beta=beta, alpha=alpha, out=out)
    return addmm(input, mat1, mat2, alpha=float(alpha), beta=float(beta))


def torch_linear(input, weight, bias=None):
    """F.linear: ``input @ weight.T (+ bias)``; counted as matmul, or addmm when biased
    (what nn.Linear maps to in the reference)."""
    if bias is None:
        return matmul(input, weight.T if isinstance(weight, torch.Tensor) and weight.ndim == 2 else weight)
    if isinstance(weight, torch.Tensor) and weight.ndim == 2:
        return addmm(bias, input, weight.T)
    _fallback("addmm", "non-2d-rhs-or-non-float")
    return _orig_linear(input, weight, bias)


def torch_rms_norm(input, normalized_shape, weight=None, eps=None):
    shape = tuple(normalized_shape) if not isinstance(normalized_shape, int) else (normalized_shape,)
    if len(shape) == 1 and shape[0] == input.shape[-1]:
        e = torch.finfo(input.dtype).eps if eps is None and _is_float(input) else (eps or 0.0)
        return rms_norm(input, weight, e)
    _fallback("rms_norm", "non-float")
    return _orig_rms_norm(input, normalized_shape, weight, eps)


def torch_sdpa(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, enable_gqa=False):
    D = query.shape[-1]
    sc = (1.0 / math.sqrt(D)) if scale is None else scale
    square = query.ndim == 4 and key.ndim == 4 and query.shape[2] == key.shape[2]
    plain = dropout_p == 0.0 and (not is_causal or square)  # torch aligns a causal mask top-left
    if attn_mask is None and plain:
        if query.ndim == 4 and key.ndim == 4 and query.shape[1] != key.shape[1] and not enable_gqa:
            plain = False
    if plain:
        mask = attn_mask if attn_mask is not None else ("causal" if is_causal else None)
        if not (isinstance(mask, torch.Tensor)) and _attn.supports(query, key, value, mask, None) and _on_cuda(query, key, value):
            return scaled_dot_product_attention(query, key, value, scale=sc, mask=mask)
    _fallback("sdpa", "array-mask" if isinstance(attn_mask, torch.Tensor) else "sinks-or-shape")
    return _orig_sdpa(query, key, value, attn_mask=attn_mask, dropout_p=dropout_p, is_causal=is_causal, scale=scale,
                      enable_gqa=enable_gqa)


def torch_layer_norm(input, normalized_shape, weight=None, bias=None, eps=1e-5):
    """F.layer_norm over the last axis (an extension: the reference does not patch a LayerNorm; counted under
    ``layer_norm``)."""
    shape = tuple(normalized_shape) if not isinstance(normalized_shape, int) else (normalized_shape,)
    if len(shape) == 1 and shape[0] == input.shape[-1] and _is_float(input):
        if _on_cuda(input, weight, bias):
            handled["layer_norm"] += 1
            return batch_invariant_layer_norm(input, weight, bias, eps)
        _fallback("layer_norm", "not-cuda")
    else:
        _fallback("layer_norm", "non-float")
    return _orig_layer_norm(input, normalized_shape, weight, bias, eps)


def reset_stats():
    handled.clear()
    fallbacks.clear()


def stats() -> dict:
    return {"handled": dict(handled), "fallbacks": dict(fallbacks)}
