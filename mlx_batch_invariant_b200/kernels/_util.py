"""Shared helpers of the kernel wrappers: input adoption (torch / DLPack) and checks."""

from __future__ import annotations

import torch

from .. import _lib


def adopt(x):
    """Return (tensor, was_foreign). Anything exposing __dlpack__ (for instance an MLX
    CUDA-backend array) is viewed as a torch tensor without a copy."""
    if isinstance(x, torch.Tensor):
        return x, False
    if hasattr(x, "__dlpack__"):
        return torch.from_dlpack(x), True
    raise TypeError(f"expected a torch.Tensor or a DLPack-capable array, got {type(x).__name__}")


def give_back(out: torch.Tensor, like, foreign: bool):
    """Hand the result back in the caller's array type when the inputs were foreign."""
    if not foreign:
        return out
    mod = type(like).__module__.split(".")[0]
    if mod == "mlx":
        import mlx.core as mx  # only reachable when the caller passed MLX arrays

        return mx.from_dlpack(out) if hasattr(mx, "from_dlpack") else mx.array(out)
    return out


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(
                "batch-invariant kernels run on CUDA tensors only (there is no CPU path); "
                f"got a tensor on {t.device}"
            )
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    return dev


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _lib.DTYPE_CODE[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt} (float32, float16, bfloat16)") from None


def rows_16b(x2: torch.Tensor) -> torch.Tensor:
    """A [M, K] view whose rows are k-contiguous and 16-byte aligned (copy if needed).
    The copy moves data only; which kernel a weight takes never depends on it."""
    es = x2.element_size()
    ok = x2.stride(-1) == 1 and x2.data_ptr() % 16 == 0 and (x2.shape[0] == 1 or (x2.stride(0) * es) % 16 == 0)
    if ok and (x2.shape[0] == 1 or x2.stride(0) >= x2.shape[1]):
        return x2
    if (x2.shape[1] * es) % 16 == 0:
        return x2.contiguous()
    # pad the row pitch up to a multiple of 16 bytes
    per = 16 // es
    pitch = (x2.shape[1] + per - 1) // per * per
    buf = torch.empty((x2.shape[0], pitch), dtype=x2.dtype, device=x2.device)
    view = buf[:, : x2.shape[1]]
    view.copy_(x2)
    return view
