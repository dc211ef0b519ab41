"""Python face of the CPU oracle. TEST INFRASTRUCTURE ONLY -- parity unpinned (see bi_oracle.c).

Two tiers:
  * bit-exact: ctypes wrappers over the plain-C restatement of the reference algorithm
    (bi_oracle.c) for RMSNorm, attention, the split fold, dequantization and the CUDA-core
    matmul order. 16-bit values travel as torch tensors and cross as uint16 bit patterns.
  * semantic: float64 numpy versions of each op (``*_f64``) for tolerance checks with the
    reference's metric max|ref - got| / max|ref| (tests/test_batch_invariance.py:28 there).
Also the affine quantizer and the seeded synthetic inputs the configs describe.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int32, c_int64, c_void_p, POINTER

import numpy as np
import torch

from . import build as _build

ORC = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        L = ctypes.CDLL(str(_build.build()))
        L.orc_expf.restype = c_float
        L.orc_expf.argtypes = [c_float]
        L.orc_expf_array.argtypes = [c_void_p, c_void_p, c_int64]
        L.orc_rms_norm.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_int]
        L.orc_attn_decode.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                      c_int64, c_int64, c_float, c_int, c_int]
        L.orc_attn_prefill.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                       c_int64, c_int64, c_float, c_int, c_int, c_int]
        L.orc_matmul_f32order.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                                          c_int64, c_int64, c_int]
        L.orc_combine.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int]
        L.orc_dequant.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int]
        L.orc_layer_norm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_int]
        L.orc_set_threads.restype = c_int
        L.orc_set_threads.argtypes = [c_int]
        _lib = L
    return _lib


def set_threads(n: int) -> int:
    """Use n OpenMP threads in the oracle's loops (returns the count in effect)."""
    return int(lib().orc_set_threads(int(n)))


def _c(t: torch.Tensor) -> torch.Tensor:
    return t.detach().cpu().contiguous()


# ---- bit-exact tier --------------------------------------------------------------------

def expf(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    lib().orc_expf_array(x.ctypes.data, y.ctypes.data, x.size)
    return y


def rms_norm(x: torch.Tensor, w: torch.Tensor | None, eps: float) -> torch.Tensor:
    x = _c(x)
    D = x.shape[-1]
    w = None if w is None else _c(w.to(x.dtype))
    out = torch.empty_like(x)
    lib().orc_rms_norm(x.data_ptr(), None if w is None else w.data_ptr(), out.data_ptr(), x.numel() // D, D,
                       float(eps), ORC[x.dtype])
    return out


def layer_norm(x: torch.Tensor, w: torch.Tensor | None, b: torch.Tensor | None, eps: float) -> torch.Tensor:
    x = _c(x)
    D = x.shape[-1]
    w = None if w is None else _c(w.to(x.dtype))
    b = None if b is None else _c(b.to(x.dtype))
    out = torch.empty_like(x)
    lib().orc_layer_norm(x.data_ptr(), None if w is None else w.data_ptr(), None if b is None else b.data_ptr(),
                         out.data_ptr(), x.numel() // D, D, float(eps), ORC[x.dtype])
    return out


def attn_decode(q, k, v, *, scale: float, split_size: int = 256, kv_lens=None) -> torch.Tensor:
    q, k, v = _c(q), _c(k.to(q.dtype)), _c(v.to(q.dtype))
    B, Hq, Tq, D = q.shape
    _, Hkv, L, _ = k.shape
    assert Tq == 1
    lens = None if kv_lens is None else _c(torch.as_tensor(kv_lens, dtype=torch.int32))
    out = torch.empty_like(q)
    lib().orc_attn_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                          None if lens is None else lens.data_ptr(), B, Hq, Hkv, L, D, float(scale), split_size,
                          ORC[q.dtype])
    return out


def attn_prefill(q, k, v, *, scale: float, causal: bool, split_size: int = 256) -> torch.Tensor:
    q, k, v = _c(q), _c(k.to(q.dtype)), _c(v.to(q.dtype))
    B, Hq, Tq, D = q.shape
    _, Hkv, L, _ = k.shape
    out = torch.empty_like(q)
    lib().orc_attn_prefill(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, Hq, Hkv, Tq, L, D,
                           float(scale), 1 if causal else 0, split_size, ORC[q.dtype])
    return out


def matmul_f32order(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a[M,K] @ b[K,N] in the CUDA-core order (one fp32 fma per k inside a 256 group, left fold)."""
    a, b = _c(a), _c(b)
    M, K = a.shape
    N = b.shape[1]
    out = torch.empty((M, N), dtype=a.dtype)
    lib().orc_matmul_f32order(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, K, 1, N, 1, ORC[a.dtype])
    return out


def combine(part: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    part = _c(part.float())
    G = part.shape[0]
    out = torch.empty(part.shape[1:], dtype=dtype)
    lib().orc_combine(part.data_ptr(), out.data_ptr(), G, out.numel(), ORC[dtype])
    return out


def dequant(w: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, *, group_size: int, bits: int,
            dtype: torch.dtype) -> torch.Tensor:
    """Packed codes -> [N, K] weight in `dtype`: T(fma(float(code), float(scale), float(bias)))."""
    w = _c(w)
    s, b = _c(scales.to(dtype)), _c(biases.to(dtype))
    N = w.shape[0]
    K = w.shape[1] * (32 // bits)
    out = torch.empty((N, K), dtype=dtype)
    lib().orc_dequant(w.data_ptr(), s.data_ptr(), b.data_ptr(), out.data_ptr(), N, K, group_size, bits, ORC[dtype])
    return out


# ---- semantic tier (float64) -----------------------------------------------------------------

def _f64(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().to(torch.float64).numpy()


def matmul_f64(a: torch.Tensor, b: torch.Tensor) -> np.ndarray:
    return _f64(a) @ _f64(b)


def rms_norm_f64(x: torch.Tensor, w: torch.Tensor | None, eps: float) -> np.ndarray:
    xf = _f64(x)
    inv = 1.0 / np.sqrt((xf * xf).mean(-1, keepdims=True) + eps)
    return xf * inv * (1.0 if w is None else _f64(w))


def layer_norm_f64(x: torch.Tensor, w: torch.Tensor | None, b: torch.Tensor | None, eps: float) -> np.ndarray:
    xf = _f64(x)
    y = (xf - xf.mean(-1, keepdims=True)) / np.sqrt(xf.var(-1, keepdims=True) + eps)
    if w is not None:
        y = y * _f64(w)
    if b is not None:
        y = y + _f64(b)
    return y


def unpack_codes(w: torch.Tensor, bits: int) -> np.ndarray:
    wn = w.detach().cpu().numpy().astype(np.uint32)
    per = 32 // bits
    sh = (np.arange(per, dtype=np.uint32) * bits)[None, None, :]
    return ((wn[:, :, None] >> sh) & np.uint32((1 << bits) - 1)).reshape(wn.shape[0], -1)


def dequant_f64(w, scales, biases, *, group_size: int, bits: int) -> np.ndarray:
    codes = unpack_codes(w, bits).astype(np.float64)
    s = np.repeat(_f64(scales), group_size, axis=1)
    b = np.repeat(_f64(biases), group_size, axis=1)
    return codes * s + b


def qmm_f64(x, w, scales, biases, *, group_size: int, bits: int) -> np.ndarray:
    return _f64(x) @ dequant_f64(w, scales, biases, group_size=group_size, bits=bits).T


def attention_f64(q, k, v, *, scale: float, causal: bool, kv_lens=None) -> np.ndarray:
    qf, kf, vf = _f64(q), _f64(k), _f64(v)
    B, Hq, Tq, D = qf.shape
    _, Hkv, L, _ = kf.shape
    G = Hq // Hkv
    out = np.zeros_like(qf)
    for b in range(B):
        Lb = L if kv_lens is None else int(kv_lens[b])
        for h in range(Hq):
            s = (qf[b, h] @ kf[b, h // G, :Lb].T) * scale
            if causal:
                qi = np.arange(Tq)[:, None]
                kj = np.arange(Lb)[None, :]
                s = np.where(kj <= Lb - Tq + qi, s, -np.inf)
            s = s - s.max(-1, keepdims=True)
            p = np.exp(s)
            out[b, h] = (p / p.sum(-1, keepdims=True)) @ vf[b, h // G, :Lb]
    return out


def rel_err(ref: np.ndarray, got: torch.Tensor) -> float:
    """max|ref - got| / max|ref| -- the reference tests' metric."""
    g = _f64(got)
    return float(np.abs(ref - g).max() / (np.abs(ref).max() + 1e-30))


# ---- quantizer and synthetic inputs -----------------------------------------------------

def quantize_affine(W: torch.Tensor, *, group_size: int, bits: int, dtype: torch.dtype):
    """Per-group affine quantization: scale = (max - min) / (2^bits - 1), bias = min,
    code = round((w - bias) / scale) clipped; codes packed low to high in uint32.
    Returns (packed int32-viewable uint32 words [N, K*bits/32], scales [N, K/gs], biases)."""
    Wf = W.detach().cpu().to(torch.float32)
    N, K = Wf.shape
    g = Wf.reshape(N, K // group_size, group_size)
    lo, hi = g.min(-1).values, g.max(-1).values
    levels = float((1 << bits) - 1)
    scale = ((hi - lo) / levels).clamp_min(1e-8).to(dtype)
    bias = lo.to(dtype)
    sf, bf = scale.to(torch.float32), bias.to(torch.float32)
    codes = torch.round((g - bf[..., None]) / sf[..., None]).clamp_(0, levels).to(torch.int64).reshape(N, K)
    per = 32 // bits
    shifts = (torch.arange(per, dtype=torch.int64) * bits)
    words = (codes.reshape(N, K // per, per) << shifts).sum(-1)
    packed = torch.from_numpy(words.numpy().astype(np.uint32).view(np.int32)).contiguous()
    return packed, scale.contiguous(), bias.contiguous()


def bits_of(t: torch.Tensor) -> bytes:
    """Raw bytes of a tensor, for bitwise comparison across dtypes."""
    t = t.detach().cpu().contiguous()
    view = {2: torch.int16, 4: torch.int32, 8: torch.int64}[t.element_size()]
    return t.view(view).numpy().tobytes()
