"""The override mechanism.

Same contract as the reference (mlx_batch_invariant/_mode.py:66-91): a re-entrant context
manager that, on entering the outermost block, swaps the module-level functions model
code reaches for and restores them on leaving it, under one process-global lock;
``strict`` is scoped to each ``with`` and restored to the outer value.

Patched while the mode is on:
  * PyTorch: ``torch.matmul``, ``torch.mm``, ``torch.addmm``, ``Tensor.__matmul__`` /
    ``__rmatmul__`` / ``.matmul`` / ``.mm``, ``F.linear``, ``F.rms_norm``, ``F.layer_norm``,
    ``F.scaled_dot_product_attention`` -- what ``nn.Linear``, ``nn.RMSNorm`` and attention
    modules call.
  * MLX, when ``mlx.core`` is importable: the six symbols the reference patches
    (``mx.matmul``, ``mx.addmm``, ``mx.quantized_matmul``, ``mx.fast.rms_norm``,
    ``mx.fast.scaled_dot_product_attention``, ``mx.array.__matmul__``), through wrappers of
    their own (``_mlx.py``): arrays cross over DLPack, and a fallback goes to the MLX stock op.
Code that captured a stock callable before the block was entered bypasses the mode, as in
the reference.
"""

from __future__ import annotations

import contextlib
import importlib.util
import threading

import torch
import torch.nn.functional as F

from . import ops

_lock = threading.Lock()
_depth = 0
_saved: list = []


def _torch_patches():
    return [
        (torch, "matmul", ops.matmul),
        (torch, "mm", ops.torch_mm),
        (torch, "addmm", ops.torch_addmm),
        (torch.Tensor, "__matmul__", ops.torch_tensor_matmul),
        (torch.Tensor, "__rmatmul__", ops.torch_tensor_rmatmul),
        (torch.Tensor, "matmul", ops.torch_tensor_matmul),
        (torch.Tensor, "mm", ops.torch_tensor_matmul),
        (F, "linear", ops.torch_linear),
        (F, "rms_norm", ops.torch_rms_norm),
        (F, "layer_norm", ops.torch_layer_norm),
        (F, "scaled_dot_product_attention", ops.torch_sdpa),
    ]


def _mlx_patches():
    if importlib.util.find_spec("mlx") is None:
        return []
    try:
        import mlx.core as mx
    except Exception:  # an MLX install that cannot initialise is the same as none
        return []
    from . import _mlx

    return _mlx.patches(mx)


def _apply():
    global _saved
    _saved = []
    for owner, name, repl in _torch_patches() + _mlx_patches():
        _saved.append((owner, name, getattr(owner, name)))
        setattr(owner, name, repl)


def _restore():
    global _saved
    for owner, name, orig in reversed(_saved):
        setattr(owner, name, orig)
    _saved = []


def is_batch_invariant_mode_enabled() -> bool:
    return _depth > 0


@contextlib.contextmanager
def set_batch_invariant_mode(enabled: bool = True, *, strict: bool = False):
    """Route matmul / addmm / quantized matmul / rms_norm / attention through the
    batch-invariant kernels for the duration of the block.

    ``strict=True`` raises instead of falling back to a stock kernel for unsupported
    inputs. Re-entrant; process-global.
    """
    global _depth
    if not enabled:
        yield
        return
    with _lock:
        if _depth == 0:
            _apply()
        _depth += 1
        prev_strict = ops.strict
        ops.strict = strict
    try:
        yield
    finally:
        with _lock:
            ops.strict = prev_strict
            _depth -= 1
            if _depth == 0:
                _restore()
