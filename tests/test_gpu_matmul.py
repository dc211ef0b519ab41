"""Dense and quantized matmul on the GPU, through the C ABI.

The CUDA-core path (fp32, or weights TMA cannot address) is bit-exact against the CPU oracle.
The tensor-core path cannot be reproduced on a CPU (the MMA's internal order is the hardware's):
it is held to the float64 semantics by tolerance and to itself bit for bit -- split == fused,
every batch size, every row position of the 128-row tile, quantized == dense on the
oracle-dequantized weight."""

import numpy as np
import pytest
import torch

from oracle import reference as R
from tests.golden import make_golden

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-2}


def xw(M, N, K, dt, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(M, K, generator=g).to(dt), (torch.randn(N, K, generator=g) / K ** 0.5).to(dt)


# ---- CUDA-core path -----------------------------------------------------------------------

@pytest.mark.parametrize("M,N,K", [(1, 64, 256), (3, 33, 600), (17, 70, 257), (40, 130, 1000), (5, 8, 16)])
@pytest.mark.parametrize("path", ["auto", "split", "fused"])
def test_fp32_bit_exact_vs_oracle(bi, M, N, K, path):
    x, w = xw(M, N, K, torch.float32, M + N + K)
    got = bi.batch_invariant_matmul(x.cuda(), w.cuda().T, path=path)
    assert R.bits_of(got) == R.bits_of(R.matmul_f32order(x, w.T.contiguous()))


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_16bit_weight_tma_cannot_address_takes_cuda_core_order(bi, dt):
    x, w = xw(6, 40, 300 + 3, dt, 9)         # K % 8 != 0
    got = bi.batch_invariant_matmul(x.cuda(), w.cuda().T)
    assert R.bits_of(got) == R.bits_of(R.matmul_f32order(x, w.T.contiguous()))
    xb, wb = xw(4, 24, 64, dt, 10)           # row-major [K, N] operand (not a W.T view)
    got = bi.batch_invariant_matmul(xb.cuda(), wb.T.contiguous().cuda())
    assert R.bits_of(got) == R.bits_of(R.matmul_f32order(xb, wb.T.contiguous()))


@pytest.mark.parametrize("name", ["f32"])
def test_golden_fixture_fp32(bi, name):
    gold = np.load(make_golden.OUT)
    i = make_golden.inputs(name)
    got = bi.batch_invariant_matmul(i["a"].cuda(), i["w"].cuda().T)
    assert make_golden.raw(got).tobytes() == gold[f"{name}_mm"].tobytes()


def test_fp32_configured_shape_tolerance_and_invariance(bi):
    x, w = xw(256, 4096, 4096, torch.float32, 0)
    xc, wc = x.cuda(), w.cuda()
    full = bi.batch_invariant_matmul(xc, wc.T)
    assert R.rel_err(R.matmul_f64(x[:8], w.T), full[:8]) < 1e-5
    for M in (1, 4, 16, 64):
        assert R.bits_of(bi.batch_invariant_matmul(xc[:M], wc.T)) == R.bits_of(full[:M])
    assert R.bits_of(bi.batch_invariant_matmul(xc[255:], wc.T)) == R.bits_of(full[255:])


# ---- tensor-core path ---------------------------------------------------------------------

@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(1, 128, 256), (1, 4096, 4096), (4, 896, 896), (16, 4864, 896), (64, 4096, 4096),
                                   (256, 4096, 4096), (130, 200, 520), (7, 136, 72), (300, 1000, 264)])
def test_tensor_core_tolerance_and_split_equals_fused(bi, dt, M, N, K):
    x, w = xw(M, N, K, dt, M * 3 + N + K)
    xc, wc = x.cuda(), w.cuda()
    auto = bi.batch_invariant_matmul(xc, wc.T)
    assert R.rel_err(R.matmul_f64(x, w.T), auto) < TOL[dt]
    split = bi.batch_invariant_matmul(xc, wc.T, path="split")
    fused = bi.batch_invariant_matmul(xc, wc.T, path="fused")
    assert R.bits_of(split) == R.bits_of(fused) == R.bits_of(auto)
    bi.check_device_status()


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_row_position_independence(bi, dt):
    """The same activation row gives the same bits at every slot of the 128-row batch tile, in any
    batch tile, next to any neighbours (the premise the whole contract rests on)."""
    N, K = 512, 1024
    x, w = xw(300, N, K, dt, 77)
    wc = w.cuda()
    probe = x[:1].cuda()
    want = R.bits_of(bi.batch_invariant_matmul(probe, wc.T))
    g = torch.Generator().manual_seed(5)
    for pos in list(range(0, 128, 5)) + [127, 128, 129, 255, 256, 299]:
        batch = torch.randn(300, K, generator=g).to(dt).cuda()
        batch[pos] = probe[0]
        for path in ("split", "fused"):
            out = bi.batch_invariant_matmul(batch, wc.T, path=path)
            assert R.bits_of(out[pos:pos + 1]) == want, (pos, path)


# Batch sizes that make the kernel issue every MMA width it can (the instruction's N is the batch rows of a
# tile rounded up to 16: 16, 32, ..., 128) and that sit on either side of every 16-row boundary.
EVERY_WIDTH = [1, 8, 9, 16, 17, 32, 33, 48, 49, 64, 65, 80, 81, 96, 97, 112, 113, 127, 128, 129]


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_every_mma_width_gives_the_batch1_bits(bi, dt):
    """A row's bits at every batch size from 1 to 129, in the first and in the last row of the batch, through
    the split, fused and in-kernel-fold launch shapes, equal its bits alone: an accumulator column depends on
    its own batch row only, whatever width the instruction was issued with."""
    N, K = 384, 1024
    x, w = xw(129, N, K, dt, 5)
    xc, wc = x.cuda(), w.cuda()
    want = R.bits_of(bi.batch_invariant_matmul(xc[:1], wc.T))
    for M in EVERY_WIDTH:
        tail = xc[:M].clone()
        tail[M - 1] = xc[0]
        for path in ("split", "fused", "fold"):
            assert R.bits_of(bi.batch_invariant_matmul(xc[:M], wc.T, path=path)[:1]) == want, (M, path)
            assert R.bits_of(bi.batch_invariant_matmul(tail, wc.T, path=path)[M - 1:M]) == want, (M, path, "last row")
    bi.check_device_status()


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M", [40, 64, 129, 256])
def test_batch_tile_height_moves_no_bit(bi, dt, M):
    """The fused path may cut the batch into tiles of 16, 32, 64 or 128 rows (more tiles to fill the GPU); the
    split path likewise. Every height gives the bits of the default launch."""
    x, w = xw(M, 512, 768, dt, M)
    xc, wc = x.cuda(), w.cuda()
    want = R.bits_of(bi.batch_invariant_matmul(xc, wc.T))
    for bt in (16, 32, 64, 128):
        for path in ("fused", "split", "fold"):
            assert R.bits_of(bi.batch_invariant_matmul(xc, wc.T, path=path, batch_tile=bt)) == want, (bt, path)
    bi.check_device_status()


def test_in_kernel_fold_leaves_its_counters_zero(bi):
    """The fold's arrival counters live at the head of the stream's workspace and must be zero again after
    every call, or the next call would fold early."""
    from mlx_batch_invariant_b200 import _lib
    x, w = xw(16, 4096, 4096, torch.bfloat16, 8)
    xc, wc = x.cuda(), w.cuda()
    want = R.bits_of(bi.batch_invariant_matmul(xc, wc.T, path="split"))
    for _ in range(3):
        assert R.bits_of(bi.batch_invariant_matmul(xc, wc.T, path="fold")) == want
        assert R.bits_of(bi.batch_invariant_matmul(xc, wc.T)) == want          # AUTO folds in the kernel at M <= 16
    torch.cuda.synchronize()
    for ws in _lib._workspaces.values():
        assert int(ws[:_lib.COUNTER_BYTES].view(torch.int32).abs().sum()) == 0
    bi.check_device_status()


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_strided_activation_and_leading_dims(bi, dt):
    x, w = xw(24, 256, 512, dt, 3)
    xc, wc = x.cuda(), w.cuda()
    want = bi.batch_invariant_matmul(xc, wc.T)
    big = torch.zeros(24, 512 + 24, dtype=dt, device="cuda")
    big[:, 8:520] = xc
    assert R.bits_of(bi.batch_invariant_matmul(big[:, 8:520], wc.T)) == R.bits_of(want)       # aligned pitch, in place
    big[:, 3:515] = xc
    assert R.bits_of(bi.batch_invariant_matmul(big[:, 3:515], wc.T)) == R.bits_of(want)       # misaligned -> copied
    assert R.bits_of(bi.batch_invariant_matmul(xc.reshape(2, 3, 4, 512), wc.T).reshape(24, 256)) == R.bits_of(want)
    mixed = bi.batch_invariant_matmul(xc.float(), wc.T)                                        # promoted to fp32
    assert mixed.dtype == torch.float32


# ---- quantized ------------------------------------------------------------------------------

def quant_case(N, K, bits, gs, dt, seed):
    g = torch.Generator().manual_seed(seed)
    W = torch.randn(N, K, generator=g) * 0.02
    return R.quantize_affine(W, group_size=gs, bits=bits, dtype=dt)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("bits,gs", [(4, 32), (4, 64), (4, 128), (8, 32), (8, 64), (8, 128)])
def test_quantized_equals_dense_on_dequantized_weight(bi, dt, bits, gs):
    N, K, M = 200, 1024, 9
    p, s, b = quant_case(N, K, bits, gs, dt, bits * 100 + gs)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(M, K, generator=g).to(dt)
    got = bi.batch_invariant_quantized_matmul(x.cuda(), p.cuda(), s.cuda(), b.cuda(), group_size=gs, bits=bits)
    wd = R.dequant(p, s, b, group_size=gs, bits=bits, dtype=dt)            # oracle dequant, bit-exact spec
    dense = bi.batch_invariant_matmul(x.cuda(), wd.cuda().T)
    assert R.bits_of(got) == R.bits_of(dense)
    assert R.rel_err(R.qmm_f64(x, p, s, b, group_size=gs, bits=bits), got) < TOL[dt]
    for path in ("split", "fused"):
        alt = bi.batch_invariant_quantized_matmul(x.cuda(), p.cuda(), s.cuda(), b.cuda(), group_size=gs, bits=bits, path=path)
        assert R.bits_of(alt) == R.bits_of(got)
    bi.check_device_status()


@pytest.mark.parametrize("bits,gs", [(4, 64), (4, 32), (8, 128), (8, 32)])
def test_quantized_every_width_and_both_stagings(bi, bits, gs):
    """Quantized weights: every MMA width, both ways of staging the dequantized operand (shared memory, the
    tile body; tensor memory, the streaming decode variant), every launch shape -- one set of bits, those of
    the dense kernel on the dequantized weight."""
    dt = torch.bfloat16
    N, K = 264, 896                                     # a partial weight tile and a half-width last K group
    p, s, b = quant_case(N, K, bits, gs, dt, bits + gs)
    g = torch.Generator().manual_seed(6)
    x = torch.randn(129, K, generator=g).to(dt).cuda()
    pc, sc, bc = p.cuda(), s.cuda(), b.cuda()
    wd = R.dequant(p, s, b, group_size=gs, bits=bits, dtype=dt).cuda()
    q = lambda xx, **kw: bi.batch_invariant_quantized_matmul(xx, pc, sc, bc, group_size=gs, bits=bits, **kw)
    want = R.bits_of(bi.batch_invariant_matmul(x[:1], wd.T))
    for M in EVERY_WIDTH:
        dense = bi.batch_invariant_matmul(x[:M], wd.T)
        assert R.bits_of(dense[:1]) == want
        stages = ("smem", "tmem") if M <= 64 else ("smem",)
        for stage in stages:
            for path in ("split", "fused", "fold"):
                assert R.bits_of(q(x[:M], path=path, stage=stage)) == R.bits_of(dense), (M, stage, path)
        assert R.bits_of(q(x[:M])) == R.bits_of(dense), (M, "auto")
    for bt in (16, 32, 64):                             # tall batches cut into short tiles stream as well
        assert R.bits_of(q(x, path="fused", batch_tile=bt, stage="tmem")) == R.bits_of(bi.batch_invariant_matmul(x, wd.T)), bt
    bi.check_device_status()


@pytest.mark.parametrize("K,N", [(896, 896), (896, 4864), (4096, 4096), (4096, 14336)])
def test_quantized_configured_shapes(bi, K, N):
    dt = torch.bfloat16
    p, s, b = quant_case(N, K, 4, 64, dt, K + N)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(64, K, generator=g).to(dt)
    pc, sc, bc, xc = p.cuda(), s.cuda(), b.cuda(), x.cuda()
    full = bi.batch_invariant_quantized_matmul(xc, pc, sc, bc, group_size=64, bits=4)
    assert R.rel_err(R.qmm_f64(x[:4], p, s, b, group_size=64, bits=4), full[:4]) < 2e-2
    for M in (1, 4, 16):
        assert R.bits_of(bi.batch_invariant_quantized_matmul(xc[:M], pc, sc, bc, group_size=64, bits=4)) == R.bits_of(full[:M])
    assert R.bits_of(bi.batch_invariant_quantized_matmul(xc[63:], pc, sc, bc, group_size=64, bits=4)) == R.bits_of(full[63:])
    bi.check_device_status()


def test_quantized_fp32_bit_exact_vs_oracle(bi):
    """fp32 activations stage the dequantized weight in fp32 and take the CUDA-core order."""
    p, s, b = quant_case(40, 256, 4, 64, torch.float32, 4)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(5, 256, generator=g)
    got = bi.batch_invariant_quantized_matmul(x.cuda(), p.cuda(), s.cuda(), b.cuda(), group_size=64, bits=4)
    wd = R.dequant(p, s, b, group_size=64, bits=4, dtype=torch.float32)
    assert R.bits_of(got) == R.bits_of(R.matmul_f32order(x, wd.T.contiguous()))


def test_dequant_golden_fixture(bi):
    """The kernel's dequantization, isolated: x = identity picks out single weight columns."""
    gold = np.load(make_golden.OUT)
    for bits in (4, 8):
        p = torch.from_numpy(gold[f"q{bits}_codes"].copy())
        g = torch.Generator().manual_seed(99)
        W = torch.randn(8, 128, generator=g) * 0.02
        p2, s, b = R.quantize_affine(W, group_size=32, bits=bits, dtype=torch.bfloat16)
        assert torch.equal(p, p2)
        eye = torch.eye(128, dtype=torch.bfloat16)
        got = bi.batch_invariant_quantized_matmul(eye.cuda(), p.cuda(), s.cuda(), b.cuda(), group_size=32, bits=bits)
        want = make_golden.unraw(gold[f"q{bits}_dequant"], torch.bfloat16)
        assert torch.equal(got.cpu().T.contiguous(), want)


# ---- weight-row position independence (what sharding a weight by rows relies on) ----------------

@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_weight_row_position_independence(bi, dt):
    """Rows [o, o+n) of W used as a weight of their own give the same bits as columns [o, o+n) of the
    full product: an output's bits do not depend on which tile, or which row of the 128-row weight
    tile, its weight row sits in. Column-parallel sharding over GPUs changes exactly that."""
    x, w = xw(40, 1024, 768, dt, 21)
    xc, wc = x.cuda(), w.cuda()
    full = bi.batch_invariant_matmul(xc, wc.T)
    for off, n in [(0, 512), (512, 512), (128, 256), (8, 120), (1016, 8), (56, 200)]:
        part = bi.batch_invariant_matmul(xc, wc[off:off + n].T)
        assert R.bits_of(part) == R.bits_of(full[:, off:off + n].contiguous()), (off, n)


def test_quantized_weight_row_position_independence(bi):
    dt = torch.bfloat16
    p, s, b = quant_case(768, 1024, 4, 64, dt, 33)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(12, 1024, generator=g).to(dt).cuda()
    pc, sc, bc = p.cuda(), s.cuda(), b.cuda()
    full = bi.batch_invariant_quantized_matmul(x, pc, sc, bc, group_size=64, bits=4)
    for off, n in [(0, 384), (384, 384), (128, 128), (40, 200)]:
        part = bi.batch_invariant_quantized_matmul(x, pc[off:off + n], sc[off:off + n], bc[off:off + n], group_size=64, bits=4)
        assert R.bits_of(part) == R.bits_of(full[:, off:off + n].contiguous()), (off, n)


# ---- bias in the epilogue ------------------------------------------------------------------------

@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
def test_bias_epilogue_gives_the_bits_of_matmul_then_add(bi, dt):
    """A linear layer's bias added inside the kernel (every launch shape, both matmul paths) equals the unfused
    sequence bit for bit: the product rounded to the output dtype, then an elementwise add."""
    for M, N, K in [(1, 384, 1024), (9, 200, 520), (64, 4096, 4096), (130, 512, 768)]:
        x, w = xw(M, N, K, dt, M + N)
        bias = torch.randn(N, generator=torch.Generator().manual_seed(N)).to(dt).cuda()
        xc, wc = x.cuda(), w.cuda()
        want = bi.batch_invariant_matmul(xc, wc.T) + bias
        for path in ("auto", "split", "fused", "fold"):
            assert R.bits_of(bi.batch_invariant_matmul(xc, wc.T, bias=bias, path=path)) == R.bits_of(want), (M, N, K, path)
    lin = torch.nn.Linear(1024, 384, device="cuda", dtype=dt)
    xin = torch.randn(5, 1024, device="cuda", dtype=dt)
    bi.reset_stats()
    with bi.set_batch_invariant_mode(strict=True):
        y = lin(xin)
    assert bi.stats()["handled"] == {"addmm": 1}
    assert R.bits_of(y) == R.bits_of(bi.batch_invariant_matmul(xin, lin.weight.T) + lin.bias)
    bi.reset_stats()
    bi.check_device_status()
