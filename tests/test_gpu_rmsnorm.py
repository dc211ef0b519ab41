"""RMSNorm on the GPU, through the C ABI, bit for bit against the CPU oracle."""

import numpy as np
import pytest
import torch

from oracle import reference as R
from tests.golden import make_golden

pytestmark = pytest.mark.gpu
DTS = [torch.float32, torch.bfloat16, torch.float16]


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("rows,D", [(1, 4096), (3, 4096), (256, 4096), (5, 100), (2, 8192), (4, 264), (2, 50000)])
def test_bit_exact_vs_oracle(bi, dt, rows, D):
    g = torch.Generator().manual_seed(rows * 131 + D)
    x = (3 * torch.randn(rows, D, generator=g)).to(dt)
    w = (1 + 0.1 * torch.randn(D, generator=g)).to(dt)
    got = bi.batch_invariant_rms_norm(x.cuda(), w.cuda(), 1e-5)
    assert R.bits_of(got) == R.bits_of(R.rms_norm(x, w, 1e-5))
    got = bi.batch_invariant_rms_norm(x.cuda(), None, 1e-6)
    assert R.bits_of(got) == R.bits_of(R.rms_norm(x, None, 1e-6))


@pytest.mark.parametrize("dt", DTS)
def test_leading_dims_and_unaligned_views(bi, dt):
    g = torch.Generator().manual_seed(5)
    x = (3 * torch.randn(2, 3, 257, generator=g)).to(dt)   # odd row length: the unstaged path
    w = torch.randn(257, generator=g).to(dt)
    got = bi.batch_invariant_rms_norm(x.cuda(), w.cuda(), 1e-5)
    assert got.shape == x.shape
    assert R.bits_of(got) == R.bits_of(R.rms_norm(x, w, 1e-5))
    base = (3 * torch.randn(4, 4096 + 8, generator=g)).to(dt).cuda()
    view = base[:, 3:4096 + 3]                            # misaligned rows -> wrapper copies
    got = bi.batch_invariant_rms_norm(view, None, 1e-5)
    assert R.bits_of(got) == R.bits_of(R.rms_norm(view.cpu(), None, 1e-5))


@pytest.mark.parametrize("name", ["f32", "bf16", "f16"])
def test_golden_fixture(bi, name):
    gold = np.load(make_golden.OUT)
    i = make_golden.inputs(name)
    got = bi.batch_invariant_rms_norm(i["rms_x"].cuda(), i["rms_w"].cuda(), 1e-5)
    assert make_golden.raw(got).tobytes() == gold[f"{name}_rms"].tobytes()
    ln = bi.batch_invariant_layer_norm(i["rms_x"].cuda(), i["rms_w"].cuda(), (i["rms_w"] - 1).cuda(), 1e-5)
    assert make_golden.raw(ln).tobytes() == gold[f"{name}_ln"].tobytes()


@pytest.mark.parametrize("dt", DTS)
def test_tolerance_vs_float64(bi, dt):
    g = torch.Generator().manual_seed(0)
    x = (3 * torch.randn(64, 4096, generator=g)).to(dt)
    w = (1 + 0.1 * torch.randn(4096, generator=g)).to(dt)
    got = bi.batch_invariant_rms_norm(x.cuda(), w.cuda(), 1e-5)
    assert R.rel_err(R.rms_norm_f64(x, w, 1e-5), got) < (1e-5 if dt == torch.float32 else 2e-2)


def test_empty(bi):
    out = bi.batch_invariant_rms_norm(torch.empty(0, 64, device="cuda"), None, 1e-5)
    assert out.shape == (0, 64)


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("rows,D", [(1, 4096), (64, 4096), (5, 100), (3, 257), (2, 50000)])
def test_add_rms_norm_equals_add_then_norm(bi, dt, rows, D):
    """The fused residual add + norm gives the bits of an elementwise add followed by the norm kernel
    (and of the oracle over that sum), staged and unstaged rows, also with the sum written over x."""
    from mlx_batch_invariant_b200.runner.decoder import KernelBackend
    g = torch.Generator().manual_seed(rows * 7 + D)
    x = (3 * torch.randn(rows, D, generator=g)).to(dt)
    d = torch.randn(rows, D, generator=g).to(dt)
    w = (1 + 0.1 * torch.randn(D, generator=g)).to(dt)
    s_ref = x + d
    s, h = KernelBackend().add_rms_norm(x.cuda(), d.cuda(), w.cuda(), 1e-5)
    assert R.bits_of(s) == R.bits_of(s_ref)
    assert R.bits_of(h) == R.bits_of(R.rms_norm(s_ref, w, 1e-5))
    assert R.bits_of(h) == R.bits_of(bi.batch_invariant_rms_norm(s_ref.cuda(), w.cuda(), 1e-5))
    # in place: sum_out = x
    from mlx_batch_invariant_b200 import _lib
    xg, dg, wg = x.cuda(), d.cuda(), w.cuda()
    out = torch.empty_like(xg)
    _lib.check(_lib.load().bi_add_rms_norm(xg.data_ptr(), dg.data_ptr(), wg.data_ptr(), xg.data_ptr(), out.data_ptr(), rows, D,
                                           1e-5, _lib.DTYPE_CODE[dt], _lib.stream_ptr(xg.device)))
    assert R.bits_of(xg) == R.bits_of(s_ref) and R.bits_of(out) == R.bits_of(h)


# ---- LayerNorm (the reference's roadmap item; same per-row scheme as RMSNorm) ---------------------------------

@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,D", [(1, 4096), (5, 768), (3, 100), (2, 8192), (7, 33)])
def test_layer_norm_bit_exact_vs_oracle(bi, dt, rows, D):
    import mlx_batch_invariant_b200 as m
    g = torch.Generator().manual_seed(rows * 1000 + D)
    x = (3 * torch.randn(rows, D, generator=g) + 0.5).to(dt)
    w = (1 + 0.1 * torch.randn(D, generator=g)).to(dt)
    b = (0.1 * torch.randn(D, generator=g)).to(dt)
    for ww, bb in ((w, b), (w, None), (None, None)):
        got = m.batch_invariant_layer_norm(x.cuda(), None if ww is None else ww.cuda(), None if bb is None else bb.cuda(), 1e-5)
        assert R.bits_of(got) == R.bits_of(R.layer_norm(x, ww, bb, 1e-5))
    tol = 1e-5 if dt == torch.float32 else 2e-2
    assert R.rel_err(R.layer_norm_f64(x, w, b, 1e-5), m.batch_invariant_layer_norm(x.cuda(), w.cuda(), b.cuda(), 1e-5)) < tol


def test_layer_norm_rows_are_batch_invariant_and_routed_by_the_mode(bi):
    import torch.nn.functional as F
    g = torch.Generator().manual_seed(0)
    x = torch.randn(256, 4096, generator=g).to(torch.bfloat16).cuda()
    ln = torch.nn.LayerNorm(4096, device="cuda", dtype=torch.bfloat16)
    bi.reset_stats()
    with bi.set_batch_invariant_mode(strict=True):
        full = ln(x)
        for M in (1, 4, 16, 64):
            assert R.bits_of(ln(x[:M])) == R.bits_of(full[:M])
        assert R.bits_of(F.layer_norm(x[255:], (4096,), ln.weight, ln.bias, ln.eps)) == R.bits_of(full[255:])
    assert bi.stats()["handled"]["layer_norm"] == 6 and bi.stats()["fallbacks"] == {}
    bi.reset_stats()
