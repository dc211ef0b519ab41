"""The reference's acceptance sweep (tests/test_batch_invariance.py:11-17 there) on the GPU: a probe
row's bits at batch 1 equal its bits inside batches of 4, 16, 64 and 256, first row and last row,
for every op and dtype; and the mode routes nn modules through the kernels without fallbacks."""

import pytest
import torch
import torch.nn.functional as F

from tests import _sweep

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("op_name", list(_sweep.OPS))
@pytest.mark.parametrize("dt_name", list(_sweep.DTYPES))
def test_invariant_kernels_are_bitwise_batch_invariant(bi, op_name, dt_name):
    if op_name.startswith("sdpa"):
        batches = [1, 4, 16, 64]          # 256 x 1000-key caches adds nothing but time
    else:
        batches = _sweep.BATCHES
    op = _sweep.OPS[op_name](_sweep.DTYPES[dt_name], 0, torch.device("cuda"))
    passed, first, worst = _sweep.sweep_one(bi, op, batches, seed=0)
    assert passed, f"{op_name}/{dt_name} diverged at B={first} (max|diff|={worst})"
    bi.check_device_status()


def test_mode_routes_torch_modules(bi):
    lin = torch.nn.Linear(256, 64, bias=True).cuda().to(torch.bfloat16)
    norm = torch.nn.RMSNorm(256, eps=1e-5).cuda().to(torch.bfloat16)
    x = torch.randn(3, 256, device="cuda", dtype=torch.bfloat16)
    q = torch.randn(2, 8, 5, 64, device="cuda", dtype=torch.bfloat16)
    kv = torch.randn(2, 2, 5, 64, device="cuda", dtype=torch.bfloat16)
    bi.reset_stats()
    with bi.set_batch_invariant_mode(strict=True):
        h = norm(x)
        y = lin(h)
        z = h @ lin.weight.T
        a = F.scaled_dot_product_attention(q, kv, kv, is_causal=True, enable_gqa=True)
        d = F.scaled_dot_product_attention(q[:, :, -1:], kv, kv, enable_gqa=True)
    st = bi.stats()
    assert st["fallbacks"] == {}
    assert st["handled"] == {"rms_norm": 1, "addmm": 1, "matmul": 1, "sdpa_prefill": 1, "sdpa_decode": 1}
    assert torch.equal(y, z + lin.bias)            # addmm adds the bias after the product is rounded
    assert torch.equal(a[:, :, -1:], d)
    ref = F.scaled_dot_product_attention(q, kv, kv, is_causal=True, enable_gqa=True)
    assert (a.float() - ref.float()).abs().max() < 3e-2


def test_quantized_routing_and_strict(bi):
    from oracle.reference import quantize_affine
    from mlx_batch_invariant_b200 import ops

    W = torch.randn(64, 256) * 0.02
    p, s, b = (t.cuda() for t in quantize_affine(W, group_size=64, bits=4, dtype=torch.float16))
    x = torch.randn(3, 256, device="cuda", dtype=torch.float16)
    bi.reset_stats()
    with bi.set_batch_invariant_mode(strict=True):
        y = ops.quantized_matmul(x, p, s, b, transpose=True, group_size=64, bits=4)
        with pytest.raises(RuntimeError):
            ops.quantized_matmul(x, p, s, b, transpose=True, group_size=16, bits=4)
    assert bi.stats()["handled"].get("quantized_matmul") == 1
    assert bi.stats()["fallbacks"] == {"quantized_matmul:affine-4bit-g16-T": 1}
    ref = ops._stock_quantized_matmul(x, p, s, b, True, 64, 4)
    assert (y.float() - ref.float()).abs().max() / ref.float().abs().max() < 2e-2
