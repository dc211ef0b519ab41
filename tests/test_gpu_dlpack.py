"""The DLPack boundary on the GPU: arrays of a foreign type (anything with ``__dlpack__``; an MLX CUDA-backend
array is the intended guest) go through all six public kernels without a copy and come back in kind, with
the bits the torch path gives; and the MLX half of the mode routes them to the kernels."""

import pytest
import torch

from oracle import reference as R
from tests import _fake_mlx

pytestmark = pytest.mark.gpu


class Foreign:
    """Owns a CUDA tensor, is not a torch.Tensor, exports DLPack."""

    def __init__(self, t):
        self.t = t

    def __dlpack__(self, stream=None):
        return self.t.__dlpack__()

    def __dlpack_device__(self):
        return self.t.__dlpack_device__()

    @property
    def shape(self):
        return tuple(self.t.shape)


def _inputs():
    g = torch.Generator().manual_seed(0)
    dt = torch.bfloat16
    x = torch.randn(5, 512, generator=g).to(dt).cuda()
    w = (torch.randn(256, 512, generator=g) / 16).to(dt).cuda()
    p, s, b = (t.cuda() for t in R.quantize_affine(torch.randn(256, 512, generator=g) * 0.02, group_size=64, bits=4, dtype=dt))
    nw = (1 + 0.1 * torch.randn(512, generator=g)).to(dt).cuda()
    q = torch.randn(2, 8, 1, 128, generator=g).to(dt).cuda()
    qp = torch.randn(2, 8, 7, 128, generator=g).to(dt).cuda()
    k = torch.randn(2, 2, 300, 128, generator=g).to(dt).cuda()
    v = torch.randn(2, 2, 300, 128, generator=g).to(dt).cuda()
    return x, w, p, s, b, nw, q, qp, k, v


def test_foreign_arrays_through_all_six_public_functions(bi):
    x, w, p, s, b, nw, q, qp, k, v = _inputs()
    F_ = Foreign
    sc = 128 ** -0.5
    cases = [
        (lambda f: bi.batch_invariant_matmul(f(x), f(w.T))),
        (lambda f: bi.batch_invariant_quantized_matmul(f(x), f(p), f(s), f(b), group_size=64, bits=4)),
        (lambda f: bi.batch_invariant_rms_norm(f(x), f(nw), 1e-5)),
        (lambda f: bi.batch_invariant_decode_attention(f(q), f(k), f(v), scale=sc)),
        (lambda f: bi.batch_invariant_prefill_attention(f(qp), f(k), f(v), scale=sc, causal=True)),
        (lambda f: bi.batch_invariant_attention(f(qp), f(k), f(v), scale=sc, mask="causal")),
    ]
    for i, case in enumerate(cases):
        want = case(lambda t: t)
        got = case(F_)
        assert isinstance(got, torch.Tensor)                 # an unknown foreign type gets the torch view back
        assert R.bits_of(got) == R.bits_of(want), i


def test_mlx_arrays_reach_the_kernels_through_the_mode(bi):
    """mx.array stand-ins over CUDA memory: the mode's MLX wrappers hand them to the kernels (handled, no
    fallback, strict passes), results come back as mx.array with the bits of the torch path."""
    mx, calls, uninstall = _fake_mlx.install()
    try:
        x, w, p, s, b, nw, q, qp, k, v = _inputs()
        A = mx.array
        sc = 128 ** -0.5
        bi.reset_stats()
        with bi.set_batch_invariant_mode(strict=True):
            outs = [
                mx.matmul(A(x), A(w.T)),
                A(x) @ A(w.T),
                mx.addmm(A(x[:, :256].contiguous()), A(x), A(w.T)),
                mx.quantized_matmul(A(x), A(p), A(s), A(b), group_size=64, bits=4),
                mx.fast.rms_norm(A(x), A(nw), 1e-5),
                mx.fast.scaled_dot_product_attention(A(q), A(k), A(v), scale=sc),
                mx.fast.scaled_dot_product_attention(A(qp), A(k), A(v), scale=sc, mask="causal"),
            ]
        assert calls == [] and bi.stats()["fallbacks"] == {}
        assert bi.stats()["handled"] == {"matmul": 2, "addmm": 1, "quantized_matmul": 1, "rms_norm": 1, "sdpa_decode": 1,
                                         "sdpa_prefill": 1}
        assert all(isinstance(o, A) for o in outs)
        mm = bi.batch_invariant_matmul(x, w.T)
        want = [mm, mm, mm + x[:, :256], bi.batch_invariant_quantized_matmul(x, p, s, b, group_size=64, bits=4),
                bi.batch_invariant_rms_norm(x, nw, 1e-5), bi.batch_invariant_attention(q, k, v, scale=sc),
                bi.batch_invariant_attention(qp, k, v, scale=sc, mask="causal")]
        for i, (o, t) in enumerate(zip(outs, want)):
            assert R.bits_of(o.t) == R.bits_of(t), i
    finally:
        uninstall()
        bi.reset_stats()
