"""The CPU oracle against what it can be pinned to here: float64 semantics, its own structural
identities (decode == prefill, chunked == one-shot, batch independence) and the committed
golden fixtures. The reference ships no numeric vectors and cannot run off an Apple GPU, so
these fixtures were produced by the oracle itself (tests/golden/make_golden.py): they guard
against drift, they do not pin the oracle to the reference."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import reference as R

GOLD = Path(__file__).resolve().parent / "golden" / "oracle_small.npz"
DTS = [torch.float32, torch.bfloat16, torch.float16]
TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-2}


def test_expf_accuracy_and_special_values():
    x = np.linspace(-86.5, 0, 2_000_001, dtype=np.float32)
    y = R.expf(x)
    ref = np.exp(x.astype(np.float64))
    ulp = np.abs(y - ref) / np.spacing(ref.astype(np.float32))
    assert ulp.max() < 1.1
    sp = R.expf(np.array([0.0, -0.0, -86.6, -1000.0, -np.inf], dtype=np.float32))
    assert sp.tolist() == [1.0, 1.0, 0.0, 0.0, 0.0]


@pytest.mark.parametrize("dt", DTS)
def test_rms_norm_matches_float64(dt):
    g = torch.Generator().manual_seed(0)
    x = (3 * torch.randn(7, 4096, generator=g)).to(dt)
    w = (1 + 0.1 * torch.randn(4096, generator=g)).to(dt)
    assert R.rel_err(R.rms_norm_f64(x, w, 1e-5), R.rms_norm(x, w, 1e-5)) < TOL[dt]
    assert R.rel_err(R.rms_norm_f64(x, None, 1e-5), R.rms_norm(x, None, 1e-5)) < TOL[dt]
    # a row's bits do not depend on its neighbours
    assert R.bits_of(R.rms_norm(x[3:4], w, 1e-5)) == R.bits_of(R.rms_norm(x, w, 1e-5)[3:4])


@pytest.mark.parametrize("dt", DTS)
def test_attention_structure_and_tolerance(dt):
    g = torch.Generator().manual_seed(1)
    B, Hq, Hkv, D, T, T1 = 2, 4, 2, 64, 300, 257
    q = torch.randn(B, Hq, T, D, generator=g).to(dt)
    k = torch.randn(B, Hkv, T, D, generator=g).to(dt)
    v = torch.randn(B, Hkv, T, D, generator=g).to(dt)
    sc = D ** -0.5
    full = R.attn_prefill(q, k, v, scale=sc, causal=True)
    assert R.rel_err(R.attention_f64(q, k, v, scale=sc, causal=True), full) < TOL[dt]
    p1 = R.attn_prefill(q[:, :, :T1], k[:, :, :T1], v[:, :, :T1], scale=sc, causal=True)
    p2 = R.attn_prefill(q[:, :, T1:], k, v, scale=sc, causal=True)
    assert R.bits_of(torch.cat([p1, p2], 2)) == R.bits_of(full)           # chunked == one-shot
    dec = R.attn_decode(q[:, :, -1:], k, v, scale=sc)
    assert R.bits_of(dec) == R.bits_of(full[:, :, -1:])                    # decode == prefill
    assert R.bits_of(R.attn_decode(q[1:, :, -1:], k[1:], v[1:], scale=sc)) == R.bits_of(dec[1:])
    lens = [T, 130]
    mixed = R.attn_decode(q[:, :, -1:], k, v, scale=sc, kv_lens=lens)
    short = R.attn_decode(q[1:, :, -1:], k[1:, :, :130], v[1:, :, :130], scale=sc)
    assert R.bits_of(mixed[1:]) == R.bits_of(short)


@pytest.mark.parametrize("dt", DTS)
def test_matmul_cuda_core_order_matches_float64(dt):
    g = torch.Generator().manual_seed(2)
    a = torch.randn(5, 600, generator=g).to(dt)
    w = (torch.randn(33, 600, generator=g) / 24).to(dt)
    out = R.matmul_f32order(a, w.T.contiguous())
    assert R.rel_err(R.matmul_f64(a, w.T), out) < TOL[dt]
    assert R.bits_of(R.matmul_f32order(a[2:3], w.T.contiguous())) == R.bits_of(out[2:3])


def test_combine_is_a_left_fold():
    part = torch.tensor([[1e8, 1.0], [1.0, 1.0], [-1e8, 1.0]], dtype=torch.float32)
    out = R.combine(part, torch.float32)
    assert out.tolist() == [0.0, 3.0]      # ((0 + 1e8) + 1) - 1e8 == 0 in fp32: order matters


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("gs", [32, 64, 128])
def test_quantizer_and_dequant(bits, gs):
    g = torch.Generator().manual_seed(3)
    W = torch.randn(24, 256, generator=g) * 0.02
    for dt in (torch.bfloat16, torch.float16, torch.float32):
        p, s, b = R.quantize_affine(W, group_size=gs, bits=bits, dtype=dt)
        assert p.shape == (24, 256 * bits // 32) and s.shape == (24, 256 // gs)
        codes = R.unpack_codes(p, bits)
        assert codes.min() >= 0 and codes.max() <= (1 << bits) - 1
        wd = R.dequant(p, s, b, group_size=gs, bits=bits, dtype=dt)
        assert R.rel_err(R.dequant_f64(p, s, b, group_size=gs, bits=bits), wd) < TOL[dt]
        step = float(s.float().max())
        assert float((wd.float() - W).abs().max()) <= 0.6 * step + 1e-3


def test_low_to_high_packing():
    p = torch.tensor([[0x76543210]], dtype=torch.int32)
    assert R.unpack_codes(p, 4).tolist() == [[0, 1, 2, 3, 4, 5, 6, 7]]
    assert R.unpack_codes(p, 8).tolist() == [[0x10, 0x32, 0x54, 0x76]]


def test_golden_fixtures_reproduce():
    from tests.golden import make_golden

    want = np.load(GOLD)
    got = make_golden.compute()
    assert sorted(want.files) == sorted(got)
    for key in want.files:
        assert want[key].tobytes() == got[key].tobytes(), key
