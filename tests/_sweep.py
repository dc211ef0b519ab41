"""Probe-row batch sweep, the acceptance method of the reference (harness/sweep.py:224-242 there):
a fixed probe row is embedded in batches of increasing size, at row 0 and at the last row, and
its output must equal the batch-1 output bit for bit. Fillers are reseeded per (B, position)."""

from __future__ import annotations

import torch

from oracle.reference import bits_of

DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}
BATCHES = [1, 4, 16, 64, 256]


def _gen(seed):
    return torch.Generator().manual_seed(seed)


class RowOp:
    """Ops whose batch axis is axis 0 of one activation tensor."""

    def __init__(self, dt, seed, device):
        self.dt, self.device = dt, device
        self.setup(_gen(seed))

    def filler(self, B, g):
        return torch.randn((B,) + tuple(self.x0.shape[1:]), generator=g).to(self.dt)

    def make_batch(self, B, pos, seed):
        rows = self.filler(B, _gen(seed))
        rows[pos] = self.x0[0]
        return rows.to(self.device)


class Matmul(RowOp):
    name, K, N = "matmul", 4096, 4096

    def setup(self, g):
        self.W = (torch.randn(self.N, self.K, generator=g) / 64).to(self.dt).to(self.device)
        self.x0 = torch.randn(1, self.K, generator=g).to(self.dt)

    def run(self, bi, batch):
        return bi.batch_invariant_matmul(batch, self.W.T)


class QuantizedMatmul(Matmul):
    name, bits, gs = "qmatmul_4b", 4, 64

    def setup(self, g):
        from oracle.reference import quantize_affine

        Wf = torch.randn(self.N, self.K, generator=g) * 0.02
        self.wq, self.sc, self.bs = (t.to(self.device) for t in quantize_affine(Wf, group_size=self.gs, bits=self.bits, dtype=self.dt))
        self.x0 = torch.randn(1, self.K, generator=g).to(self.dt)

    def run(self, bi, batch):
        return bi.batch_invariant_quantized_matmul(batch, self.wq, self.sc, self.bs, group_size=self.gs, bits=self.bits)


class QuantizedMatmul8(QuantizedMatmul):
    name, bits, gs = "qmatmul_8b", 8, 32


class RMSNorm(RowOp):
    name, D = "rms_norm", 4096

    def setup(self, g):
        self.w = (1 + 0.1 * torch.randn(self.D, generator=g)).to(self.dt).to(self.device)
        self.x0 = (3 * torch.randn(1, self.D, generator=g)).to(self.dt)

    def run(self, bi, batch):
        return bi.batch_invariant_rms_norm(batch, self.w, 1e-5)


class SDPADecode:
    name, Hq, Hkv, L, D = "sdpa_decode", 8, 2, 1000, 128

    def __init__(self, dt, seed, device):
        self.dt, self.device = dt, device
        g = _gen(seed)
        self.q0 = torch.randn(1, self.Hq, 1, self.D, generator=g).to(dt)
        self.k0 = torch.randn(1, self.Hkv, self.L, self.D, generator=g).to(dt)
        self.v0 = torch.randn(1, self.Hkv, self.L, self.D, generator=g).to(dt)

    Tq = 1
    mask = None

    def make_batch(self, B, pos, seed):
        g = _gen(seed)
        q = torch.randn(B, self.Hq, self.Tq, self.D, generator=g).to(self.dt)
        k = torch.randn(B, self.Hkv, self.L, self.D, generator=g).to(self.dt)
        v = torch.randn(B, self.Hkv, self.L, self.D, generator=g).to(self.dt)
        q[pos], k[pos], v[pos] = self.q0[0], self.k0[0], self.v0[0]
        return tuple(t.to(self.device) for t in (q, k, v))

    def run(self, bi, batch):
        q, k, v = batch
        return bi.batch_invariant_attention(q, k, v, scale=self.D ** -0.5, mask=self.mask)


class SDPAPrefill(SDPADecode):
    name, Hq, Hkv, Tq, L, D = "sdpa_prefill", 8, 2, 48, 300, 128  # L > Tq: causal against a cache
    mask = "causal"

    def __init__(self, dt, seed, device):
        self.dt, self.device = dt, device
        g = _gen(seed)
        self.q0 = torch.randn(1, self.Hq, self.Tq, self.D, generator=g).to(dt)
        self.k0 = torch.randn(1, self.Hkv, self.L, self.D, generator=g).to(dt)
        self.v0 = torch.randn(1, self.Hkv, self.L, self.D, generator=g).to(dt)


OPS = {c.name: c for c in (Matmul, QuantizedMatmul, QuantizedMatmul8, RMSNorm, SDPADecode, SDPAPrefill)}


def sweep_one(bi, op, batches, seed=0):
    """Returns (passed, first_fail_B, max_abs_diff)."""
    ref = op.run(bi, op.make_batch(1, 0, seed))[0:1]
    ref_bits = bits_of(ref)
    first, worst = None, 0.0
    for B in batches:
        for pos in sorted({0, B - 1}):
            out = op.run(bi, op.make_batch(B, pos, seed + 7 * B + pos))[pos:pos + 1]
            if bits_of(out) != ref_bits:
                first = first or B
                worst = max(worst, float((out.float() - ref.float()).abs().max()))
    return first is None, first, worst
