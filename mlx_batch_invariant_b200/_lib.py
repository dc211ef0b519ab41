"""ctypes binding of libbi_b200.so (the C ABI declared in include/bi_abi.h).

The library is the product: there is no Python or CPU stand-in for any kernel.
If the shared object is missing the first kernel call raises, loudly.
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p, POINTER
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libbi_b200.so"

BI_OK = 0
BI_ERR_UNSUPPORTED, BI_ERR_BAD_ARG, BI_ERR_MISALIGNED, BI_ERR_WORKSPACE, BI_ERR_CUDA, BI_ERR_DEVICE_WAIT = 1, 2, 3, 4, 5, 6
BI_F32, BI_F16, BI_BF16 = 0, 1, 2
PATH_AUTO, PATH_SPLIT, PATH_FUSED, PATH_SPLIT_FOLD = 0, 1, 2, 3
WS_ZEROED = 0x100                 # BI_MATMUL_WS_ZEROED
QMM_STAGE_SMEM, QMM_STAGE_TMEM = 0x1000000, 0x2000000
COUNTER_BYTES = 16384             # BI_MATMUL_COUNTER_BYTES


def batch_tile(n: int) -> int:    # BI_MATMUL_BATCH_TILE(n)
    return n << 16

DTYPE_CODE = {torch.float32: BI_F32, torch.float16: BI_F16, torch.bfloat16: BI_BF16}

# name -> (restype, argtypes); mirrors include/bi_abi.h one to one
SIGNATURES = {
    "bi_version": (c_int, []),
    "bi_last_error": (c_char_p, []),
    "bi_launch_count": (ctypes.c_ulonglong, []),
    "bi_read_device_status": (c_int, [c_void_p, POINTER(c_int32), c_void_p]),
    "bi_rms_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_int, c_void_p]),
    "bi_layer_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_int, c_void_p]),
    "bi_matmul_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int]),
    "bi_matmul": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int64, c_int64, c_int64, c_int64,
                          c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "bi_matmul_bias": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int64, c_int64, c_int64, c_int64,
                               c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "bi_qmm_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int]),
    "bi_qmm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int64, c_int64,
                       c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "bi_attn_decode_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int64, c_int]),
    "bi_attn_decode": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int64,
                               c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_float, c_int, c_int,
                               c_void_p]),
    "bi_attn_decode_paged": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int64,
                                     c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_float,
                                     c_int, c_int, c_void_p]),
    "bi_attn_decode_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                      c_int64, c_int64, c_int64, c_int64, c_int64, c_float, c_int, c_int, c_void_p]),
    "bi_rope_append": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                               c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int, c_void_p]),
    "bi_swiglu": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "bi_peer_alloc": (c_int, [ctypes.POINTER(c_void_p), c_size_t]),
    "bi_peer_free": (c_int, [c_void_p]),
    "bi_peer_export": (c_int, [c_void_p, ctypes.c_char_p]),
    "bi_peer_open": (c_int, [ctypes.c_char_p, ctypes.POINTER(c_void_p)]),
    "bi_peer_close": (c_int, [c_void_p]),
    "bi_push_gather": (c_int, [c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), c_void_p, c_int64, c_int64,
                               c_int, c_int, c_int, c_void_p, c_void_p]),
    "bi_push_gather_swiglu": (c_int, [c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), c_void_p, c_int64, c_int64,
                                      c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "bi_matmul_awaiting": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int64, c_int64, c_int64, c_int64,
                                   c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int]),
    "bi_qmm_awaiting": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int64, c_int64,
                                c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int]),
    "bi_add_rms_norm_awaiting": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_int,
                                         c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "bi_add_rms_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_int, c_void_p]),
    "bi_matmul_rope": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                               c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64]),
    "bi_qmm_rope": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int64, c_int64, c_int64, c_int64,
                            c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64]),
    "bi_matmul_push": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                               c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.POINTER(c_void_p),
                               ctypes.POINTER(c_void_p), c_void_p, c_int, c_int, c_int]),
    "bi_qmm_push": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int64, c_int64, c_int64, c_int64,
                            c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.POINTER(c_void_p),
                            ctypes.POINTER(c_void_p), c_void_p, c_int, c_int, c_int]),
    "bi_attn_decode_push": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int64, c_int64, c_int64,
                                    c_int64, c_int64, c_int64, c_int64, c_int64, c_float, c_int, c_int, c_void_p,
                                    ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), c_void_p, c_int, c_int, c_int,
                                    c_void_p]),
    "bi_attn_prefill": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                                c_int64, c_int64, c_int64, c_int64, c_float, c_int, c_int, c_int, c_void_p]),
}

_lib = None
_lock = threading.Lock()


class KernelError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"libbi_b200 status {code}: {message}")
        self.code = code


def load() -> ctypes.CDLL:
    """Load the shared library once and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not LIB_PATH.exists():
                raise RuntimeError(
                    f"{LIB_PATH} is missing: build it with `python -m mlx_batch_invariant_b200.build` "
                    "(there is no fallback implementation)"
                )
            lib = ctypes.CDLL(str(LIB_PATH))
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def last_error() -> str:
    return load().bi_last_error().decode("utf-8", "replace")


def check(code: int) -> None:
    if code != BI_OK:
        raise KernelError(code, last_error())


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


# One int32 status word per device, written by kernels whose bounded waits run out.
_status: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


# Matmul workspaces: one per (device, stream), kept between calls. Its first COUNTER_BYTES are the per-tile
# arrival counters of the split path's in-kernel fold; they are zero between calls (the kernel leaves them so),
# which is what the WS_ZEROED flag promises the library. Calls on one stream are ordered, so they can share it.
_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def matmul_workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """A zero-headed workspace of at least `nbytes` for the current stream of `device`."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    need = max(nbytes, COUNTER_BYTES)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=torch.device("cuda", idx))
        ws[:COUNTER_BYTES].zero_()       # only the counters have to start at zero (and a capture records only this small fill)
        _workspaces[key] = ws
    return ws


def check_device_status(device: torch.device | None = None) -> None:
    """Synchronise and raise if any kernel on `device` gave up a bounded wait."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    word = status_word(device)
    host = c_int32(0)
    code = load().bi_read_device_status(word.data_ptr(), ctypes.byref(host), stream_ptr(device))
    if code != BI_OK:
        msg = last_error()
        word.zero_()
        _workspaces.clear()          # a kernel that gave up may have left arrival counters behind
        raise KernelError(code, msg)
