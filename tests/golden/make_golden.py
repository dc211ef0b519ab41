"""Generate tests/golden/oracle_small.npz: seeded small inputs and the CPU oracle's outputs.

    python -m tests.golden.make_golden

The reference has no numeric vectors and cannot run here (MLX + Apple GPU), so these are
oracle outputs, not reference outputs. 16-bit tensors are stored as int16 bit patterns.
The GPU parity tests check the CUDA kernels against the same arrays.
"""

from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from oracle import reference as R

OUT = Path(__file__).resolve().parent / "oracle_small.npz"
DT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


def raw(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    return t.view({2: torch.int16, 4: torch.int32}[t.element_size()]).numpy()


def unraw(a: np.ndarray, dt: torch.dtype) -> torch.Tensor:
    return torch.from_numpy(a.copy()).view(dt)


def inputs(name: str):
    """Seeded inputs of each case (regenerated, not stored, to keep the fixture small)."""
    g = torch.Generator().manual_seed(1234)
    dt = DT[name]
    return dict(
        rms_x=(3 * torch.randn(3, 512, generator=g)).to(dt),
        rms_w=(1 + 0.1 * torch.randn(512, generator=g)).to(dt),
        q=torch.randn(2, 4, 9, 64, generator=g).to(dt),
        k=torch.randn(2, 2, 265, 64, generator=g).to(dt),
        v=torch.randn(2, 2, 265, 64, generator=g).to(dt),
        a=torch.randn(3, 300, generator=g).to(dt),
        w=(torch.randn(10, 300, generator=g) / 17).to(dt),
    )


def compute() -> dict:
    out = {}
    for name, dt in DT.items():
        i = inputs(name)
        out[f"{name}_rms"] = raw(R.rms_norm(i["rms_x"], i["rms_w"], 1e-5))
        out[f"{name}_ln"] = raw(R.layer_norm(i["rms_x"], i["rms_w"], i["rms_w"] - 1, 1e-5))
        out[f"{name}_prefill"] = raw(R.attn_prefill(i["q"], i["k"], i["v"], scale=0.125, causal=True))
        out[f"{name}_decode"] = raw(R.attn_decode(i["q"][:, :, -1:], i["k"], i["v"], scale=0.125, kv_lens=[265, 100]))
        out[f"{name}_mm"] = raw(R.matmul_f32order(i["a"], i["w"].T.contiguous()))
    g = torch.Generator().manual_seed(99)
    W = torch.randn(8, 128, generator=g) * 0.02
    for bits in (4, 8):
        p, s, b = R.quantize_affine(W, group_size=32, bits=bits, dtype=torch.bfloat16)
        out[f"q{bits}_codes"] = p.numpy()
        out[f"q{bits}_dequant"] = raw(R.dequant(p, s, b, group_size=32, bits=bits, dtype=torch.bfloat16))
    out["expf"] = R.expf(np.linspace(-90, 0, 4097, dtype=np.float32)).view(np.int32)
    return out


if __name__ == "__main__":
    np.savez_compressed(OUT, **compute())
    print(OUT, OUT.stat().st_size, "bytes")
