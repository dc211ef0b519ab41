"""A stand-in for ``mlx.core`` for tests of the MLX half of the mode and of the DLPack boundary: an array
type that owns a torch tensor and exports it through ``__dlpack__`` only (it is not a torch.Tensor), and
the six stock callables the mode patches, each recording that it ran. Real MLX is not installable here."""

from __future__ import annotations

import importlib.machinery
import sys
import types

import torch


def _mm(a, b):
    return torch.einsum("...k,kj->...j", a, b)          # not one of the symbols the mode patches


def install():
    """Put fake ``mlx`` / ``mlx.core`` modules into sys.modules; returns (mx, calls, uninstall)."""
    calls: list[str] = []

    class array:
        def __init__(self, t):
            self.t = t

        def __dlpack__(self, stream=None):
            return self.t.__dlpack__()

        def __dlpack_device__(self):
            return self.t.__dlpack_device__()

        def __matmul__(self, other):
            calls.append("array.__matmul__")
            return array(_mm(self.t, other.t))

        @property
        def shape(self):
            return tuple(self.t.shape)

    array.__module__ = "mlx.core"
    mlx = types.ModuleType("mlx")
    mx = types.ModuleType("mlx.core")
    fast = types.ModuleType("mlx.core.fast")
    for m in (mlx, mx, fast):
        m.__spec__ = importlib.machinery.ModuleSpec(m.__name__, None)
    mlx.__path__ = []

    def matmul(a, b, *, stream=None):
        calls.append("matmul")
        return array(_mm(a.t, b.t))

    def addmm(c, a, b, alpha=1.0, beta=1.0, *, stream=None):
        calls.append("addmm")
        return array(beta * c.t + alpha * _mm(a.t, b.t))

    def quantized_matmul(x, w, scales, biases=None, transpose=True, group_size=None, bits=None, *, stream=None):
        calls.append("quantized_matmul")
        return array(torch.zeros(x.t.shape[:-1] + (w.t.shape[0],), dtype=x.t.dtype, device=x.t.device))

    def rms_norm(x, weight, eps, *, stream=None):
        calls.append("rms_norm")
        y = x.t * torch.rsqrt((x.t * x.t).mean(-1, keepdim=True) + eps)
        return array(y if weight is None else y * weight.t)

    def sdpa(q, k, v, *, scale, mask=None, sinks=None, stream=None):
        calls.append("sdpa")
        return array(torch.zeros_like(q.t))

    mx.array, mx.matmul, mx.addmm, mx.quantized_matmul = array, matmul, addmm, quantized_matmul
    mx.from_dlpack = lambda t: array(torch.from_dlpack(t))
    fast.rms_norm, fast.scaled_dot_product_attention = rms_norm, sdpa
    mx.fast = fast
    mlx.core = mx
    saved = {k: sys.modules.get(k) for k in ("mlx", "mlx.core", "mlx.core.fast")}
    sys.modules.update({"mlx": mlx, "mlx.core": mx, "mlx.core.fast": fast})

    def uninstall():
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v

    return mx, calls, uninstall
