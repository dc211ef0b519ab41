"""The C-ABI library loads and exports every symbol include/bi_abi.h declares; argument
validation that returns before any CUDA call behaves as documented. No GPU needed."""

import ctypes
import re
from pathlib import Path

import pytest

from mlx_batch_invariant_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "bi_abi.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bi_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for n in ("bi_version", "bi_last_error", "bi_rms_norm", "bi_matmul", "bi_qmm", "bi_attn_decode", "bi_attn_prefill"):
        assert n in names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in bi_abi.h but not exported"


def test_python_binding_covers_every_declared_symbol():
    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_version_and_error_string():
    lib = _lib.load()
    assert lib.bi_version() >= 100
    assert isinstance(_lib.last_error(), str)


@pytest.mark.parametrize("call,code", [
    (lambda L: L.bi_rms_norm(None, None, None, 4, 8, 1e-5, 7, None), _lib.BI_ERR_UNSUPPORTED),
    (lambda L: L.bi_rms_norm(None, None, None, 4, 8, 1e-5, _lib.BI_BF16, None), _lib.BI_ERR_BAD_ARG),
    (lambda L: L.bi_rms_norm(None, None, None, 0, 8, 1e-5, _lib.BI_BF16, None), _lib.BI_OK),
    (lambda L: L.bi_add_rms_norm(None, None, None, None, None, 4, 8, 1e-5, 7, None), _lib.BI_ERR_UNSUPPORTED),
    (lambda L: L.bi_add_rms_norm(None, None, None, None, None, 4, 8, 1e-5, _lib.BI_BF16, None), _lib.BI_ERR_BAD_ARG),
    (lambda L: L.bi_add_rms_norm(None, None, None, None, None, 0, 8, 1e-5, _lib.BI_BF16, None), _lib.BI_OK),
    (lambda L: L.bi_matmul(None, None, None, None, 0, 4, 4, 4, 4, 1, 1, 4, 9, 0, None, None), _lib.BI_ERR_UNSUPPORTED),
    (lambda L: L.bi_matmul(None, None, None, None, 0, 4, 4, 4, 4, 1, 1, 4, _lib.BI_F32, 0, None, None), _lib.BI_ERR_BAD_ARG),
    (lambda L: L.bi_matmul(None, None, None, None, 0, 0, 4, 4, 4, 1, 1, 4, _lib.BI_F32, 0, None, None), _lib.BI_OK),
    (lambda L: L.bi_qmm(None, None, None, None, None, None, 0, 4, 4, 64, 64, 64, 3, _lib.BI_BF16, 0, None, None), _lib.BI_ERR_UNSUPPORTED),
    (lambda L: L.bi_qmm(None, None, None, None, None, None, 0, 4, 4, 64, 64, 48, 4, _lib.BI_BF16, 0, None, None), _lib.BI_ERR_UNSUPPORTED),
    (lambda L: L.bi_attn_decode(None, None, None, None, None, None, 0, 1, 8, 3, 16, 128, 1, 1, 128, 1.0, 256, _lib.BI_BF16, None), _lib.BI_ERR_UNSUPPORTED),
    (lambda L: L.bi_attn_decode(None, None, None, None, None, None, 0, 1, 8, 2, 16, 100, 1, 1, 128, 1.0, 256, _lib.BI_BF16, None), _lib.BI_ERR_UNSUPPORTED),
    (lambda L: L.bi_attn_prefill(None, None, None, None, 1, 8, 2, 4, 16, 128, 1, 1, 128, 1.0, 1, 256, _lib.BI_BF16, None), _lib.BI_ERR_BAD_ARG),
])
def test_validation_status_codes(call, code):
    assert call(_lib.load()) == code
    if code != _lib.BI_OK:
        assert _lib.last_error()


def test_workspace_sizes():
    L = _lib.load()
    assert L.bi_matmul_workspace_bytes(1, 4096, 4096, _lib.BI_BF16) == _lib.COUNTER_BYTES + 16 * 1 * 4096 * 4
    assert L.bi_matmul_workspace_bytes(4096, 4096, 4096, _lib.BI_BF16) == 0   # fused: no scratch
    assert L.bi_matmul_workspace_bytes(8, 4096, 256, _lib.BI_BF16) == 0       # one K group
    assert L.bi_attn_decode_workspace_bytes(2, 32, 257, 128, 256) == 2 * 32 * 2 * (128 + 2) * 4


def test_workspace_sizes_follow_the_auto_launch_shape():
    """bi_matmul_workspace_bytes covers whatever AUTO may pick: the counter block plus ceil(K/256) * M * N * 4
    bytes when the K groups may be spread over CTAs, nothing when the call is sure to fold in place (enough
    tiles at some batch-tile height, or partials too large)."""
    L = _lib.load()
    f = L.bi_matmul_workspace_bytes
    CB = _lib.COUNTER_BYTES
    assert f(1, 4096, 4096, _lib.BI_BF16) == CB + 16 * 1 * 4096 * 4
    assert f(64, 4096, 14336, _lib.BI_BF16) == CB + 56 * 64 * 4096 * 4
    assert f(128, 4096, 4096, _lib.BI_BF16) == 0                            # 32-row batch tiles make 128 tiles: fused
    assert f(96, 4096, 4096, _lib.BI_BF16) == CB + 16 * 96 * 4096 * 4       # 16-row tiles would be needed: split
    assert f(256, 4096, 4096, _lib.BI_BF16) == 0                            # 64-row batch tiles make 128 tiles: fused
    assert f(512, 4096, 4096, _lib.BI_BF16) == 0
    assert f(128, 28672, 4096, _lib.BI_BF16) == 0                           # 224 tiles fill the GPU: fused
    assert f(128, 4096, 14336, _lib.BI_BF16) == 0                           # 117 MB of partials: fused
    assert f(64, 4096, 256, _lib.BI_BF16) == 0                              # one K group: nothing to fold
    assert f(64, 28672, 4096, _lib.BI_BF16) == 0                            # 224 tiles: fused, also at 64 rows
    assert f(16, 4096, 4096, _lib.BI_F32) == CB + 16 * 16 * 4096 * 4        # fp32: the CUDA-core rule (split up to 32 rows)
    assert f(64, 4096, 4096, _lib.BI_F32) == 0
    assert L.bi_qmm_workspace_bytes(16, 14336, 4096, _lib.BI_BF16) == 0     # 112 tiles: fused
    assert L.bi_qmm_workspace_bytes(1, 14336, 4096, _lib.BI_BF16) == CB + 16 * 1 * 14336 * 4   # decode: fewer tiles than SMs -> split
    assert L.bi_qmm_workspace_bytes(1, 28672, 4096, _lib.BI_BF16) == 0      # 224 tiles: fused
    assert L.bi_qmm_workspace_bytes(16, 4096, 4096, _lib.BI_BF16) == CB + 16 * 16 * 4096 * 4
    assert f(0, 4096, 4096, _lib.BI_BF16) == 0
