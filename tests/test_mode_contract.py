"""Mode / dispatch / counter contract, in behaviour the reference's own tests
(tests/test_batch_invariance.py:60-105 there). Runs on CPU tensors: nothing here computes on a
GPU, and because there is no CPU kernel every op is a *counted fallback* -- which is exactly
what these tests need to observe."""

import pytest
import torch
import torch.nn.functional as F

import mlx_batch_invariant_b200 as bi
from mlx_batch_invariant_b200 import ops


def _symbols():
    return (torch.matmul, torch.mm, torch.addmm, F.linear, F.rms_norm, F.scaled_dot_product_attention,
            torch.Tensor.__matmul__, torch.Tensor.matmul)


def test_public_names():
    assert set(bi.__all__) == {
        "set_batch_invariant_mode", "is_batch_invariant_mode_enabled", "stats", "reset_stats",
        "batch_invariant_matmul", "batch_invariant_rms_norm", "batch_invariant_quantized_matmul",
        "batch_invariant_decode_attention", "batch_invariant_prefill_attention", "batch_invariant_attention"}
    assert isinstance(bi.__version__, str)


def test_mode_patches_and_restores():
    orig = _symbols()
    assert not bi.is_batch_invariant_mode_enabled()
    with bi.set_batch_invariant_mode():
        assert bi.is_batch_invariant_mode_enabled()
        assert torch.matmul is not orig[0]
        assert F.scaled_dot_product_attention is not orig[5]
        with bi.set_batch_invariant_mode():  # re-entrant
            assert bi.is_batch_invariant_mode_enabled()
        assert bi.is_batch_invariant_mode_enabled()
        assert torch.matmul is not orig[0]
    assert not bi.is_batch_invariant_mode_enabled()
    assert _symbols() == orig


def test_disabled_mode_is_a_no_op():
    orig = _symbols()
    with bi.set_batch_invariant_mode(enabled=False):
        assert not bi.is_batch_invariant_mode_enabled()
        assert _symbols() == orig


def test_restores_after_exception_and_strict_is_scoped():
    orig = _symbols()
    assert ops.strict is False
    with pytest.raises(ValueError):
        with bi.set_batch_invariant_mode(strict=True):
            assert ops.strict is True
            with bi.set_batch_invariant_mode():      # inner block is non-strict
                assert ops.strict is False
            assert ops.strict is True                # restored to the outer value
            raise ValueError("boom")
    assert ops.strict is False
    assert _symbols() == orig


def test_strict_mode_raises_on_unsupported():
    q = torch.randn(1, 4, 7, 32)
    m = torch.zeros(7, 7, dtype=torch.bool)  # array masks have no kernel
    with bi.set_batch_invariant_mode(strict=True):
        with pytest.raises(RuntimeError, match="no kernel for sdpa"):
            F.scaled_dot_product_attention(q, q, q, attn_mask=m)


def test_non_strict_counts_fallbacks_and_runs_stock():
    q = torch.randn(1, 4, 7, 32)
    m = torch.ones(7, 7, dtype=torch.bool)
    bi.reset_stats()
    with bi.set_batch_invariant_mode():
        out = F.scaled_dot_product_attention(q, q, q, attn_mask=m)
    assert out.shape == q.shape
    assert bi.stats()["fallbacks"].get("sdpa:array-mask") == 1


def test_fallback_reason_strings():
    bi.reset_stats()
    a = torch.randn(2, 3, 4)
    with bi.set_batch_invariant_mode():
        torch.matmul(a, a.transpose(1, 2))                       # batched 3-D rhs
        torch.matmul(torch.ones(2, 2, dtype=torch.int64), torch.ones(2, 2, dtype=torch.int64))
        torch.addmm(torch.zeros(2, 2, dtype=torch.float64), torch.ones(2, 3, dtype=torch.float64), torch.ones(3, 2, dtype=torch.float64))
        F.rms_norm(torch.randn(2, 8, dtype=torch.float64), (8,))
        x = torch.randn(2, 4)          # y = x @ dequant(w) with w stored [K=4, N=64]
        w = torch.zeros(4, 8, dtype=torch.int32)
        ops.quantized_matmul(x, w, torch.ones(4, 1), torch.zeros(4, 1), transpose=False, group_size=64, bits=4)
    fb = bi.stats()["fallbacks"]
    assert fb["matmul:non-2d-rhs-or-non-float"] == 2
    assert fb["addmm:non-2d-rhs-or-non-float"] == 1
    assert fb["rms_norm:non-float"] == 1
    assert fb["quantized_matmul:affine-4bit-g64-N"] == 1
    st = bi.stats()
    assert set(st) == {"handled", "fallbacks"} and isinstance(st["handled"], dict)
    bi.reset_stats()
    assert bi.stats() == {"handled": {}, "fallbacks": {}}


def test_cpu_tensors_are_counted_fallbacks_not_a_cpu_kernel():
    bi.reset_stats()
    lin = torch.nn.Linear(16, 8, bias=True)
    x = torch.randn(3, 16)
    with bi.set_batch_invariant_mode():
        y = lin(x)
        z = x @ lin.weight.T
    assert torch.allclose(y, z + lin.bias)
    fb = bi.stats()["fallbacks"]
    assert fb["addmm:not-cuda"] == 1 and fb["matmul:not-cuda"] == 1
    assert bi.stats()["handled"] == {}
    with bi.set_batch_invariant_mode(strict=True):
        with pytest.raises(RuntimeError, match="not-cuda"):
            lin(x)


def test_direct_kernel_calls_reject_cpu_tensors_and_bad_shapes():
    with pytest.raises(RuntimeError, match="CUDA"):
        bi.batch_invariant_rms_norm(torch.randn(2, 8), None, 1e-5)
    with pytest.raises(ValueError):
        bi.batch_invariant_matmul(torch.randn(2, 8), torch.randn(2, 8, 4))
    with pytest.raises(ValueError):
        bi.batch_invariant_matmul(torch.randn(2, 8), torch.randn(7, 4))
    with pytest.raises(AssertionError):
        q = torch.randn(1, 2, 3, 64)
        bi.batch_invariant_decode_attention(q, q, q, scale=1.0)


def test_mlx_symbols_fall_back_to_the_mlx_stock_ops():
    """With ``mlx.core`` importable the mode patches its six symbols too. Arrays that the kernels cannot take
    (here: host memory) are counted and then handed to the *MLX* stock callable that was installed before --
    never to a torch op, which could not take an mx.array -- and strict mode raises instead."""
    from tests import _fake_mlx

    mx, calls, uninstall = _fake_mlx.install()
    try:
        stock = (mx.matmul, mx.addmm, mx.quantized_matmul, mx.fast.rms_norm, mx.fast.scaled_dot_product_attention,
                 mx.array.__matmul__)
        a, b, c = mx.array(torch.randn(3, 8)), mx.array(torch.randn(8, 4)), mx.array(torch.randn(3, 4))
        q = mx.array(torch.randn(1, 4, 1, 32))
        kv = mx.array(torch.randn(1, 2, 9, 32))
        bi.reset_stats()
        with bi.set_batch_invariant_mode():
            assert mx.matmul is not stock[0] and mx.array.__matmul__ is not stock[5]
            out = mx.matmul(a, b)
            assert isinstance(out, mx.array) and out.shape == (3, 4)
            assert isinstance(a @ b, mx.array)
            mx.addmm(c, a, b, alpha=2.0)
            mx.quantized_matmul(a, mx.array(torch.zeros(4, 1, dtype=torch.int32)), mx.array(torch.ones(4, 1)),
                                mx.array(torch.zeros(4, 1)), group_size=8, bits=4)
            mx.fast.rms_norm(a, None, 1e-5)
            mx.fast.scaled_dot_product_attention(q, kv, kv, scale=0.2)
            with bi.set_batch_invariant_mode(strict=True):
                with pytest.raises(RuntimeError, match="no kernel for matmul"):
                    mx.matmul(a, b)
        assert calls == ["matmul", "array.__matmul__", "addmm", "quantized_matmul", "rms_norm", "sdpa"]
        fb = bi.stats()["fallbacks"]
        assert fb["matmul:not-cuda"] == 3 and fb["addmm:not-cuda"] == 1 and fb["rms_norm:not-cuda"] == 1
        assert fb["quantized_matmul:affine-4bit-g8-T"] == 1 and fb["sdpa:sinks-or-shape"] == 1
        assert (mx.matmul, mx.addmm, mx.quantized_matmul, mx.fast.rms_norm, mx.fast.scaled_dot_product_attention,
                mx.array.__matmul__) == stock
    finally:
        uninstall()
        bi.reset_stats()
