"""Whole-model invariance on one GPU: the method of the reference's model sweep (harness/model_sweep.py:100-108
there) on a small random-init Llama-architecture decoder. The prompt sits in row 0, the other rows are random
prompts of the same length; every block's row-0 output and the logits must be bit-identical at batch 1, 4 and
16, for the prefill and for cached decode steps, dense and 4-bit, eager and CUDA-graph replay."""

import hashlib

import pytest
import torch

from mlx_batch_invariant_b200.runner import DecoderConfig, GraphedDecoder, ShardedDecoder
from oracle.reference import bits_of

pytestmark = pytest.mark.gpu

CFG = DecoderConfig(n_layers=3, d_model=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn=1024, vocab=2048)
P, STEPS = 70, 5


def _run(model, B, graph):
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, CFG.vocab, (1, P), generator=g)
    gb = torch.Generator().manual_seed(100 + B)
    rows = torch.randint(0, CFG.vocab, (B, P), generator=gb)
    rows[0] = prompt[0]
    rows = rows.cuda()
    hashes = []
    model.block_hook = lambda li, h: hashes.append(hashlib.blake2b(bits_of(h[0:1]), digest_size=8).hexdigest())
    logits = model.forward(rows, 0)
    model.block_hook = None
    out = [bits_of(logits[0:1])]
    if graph:
        gd = GraphedDecoder(model, B)
        gd.start(logits.argmax(-1), P)
        gd.capture()
        for _ in range(STEPS):
            out.append(bits_of(gd.step()[0:1].clone()))
    else:
        for s in range(STEPS):
            logits = model.forward(logits.argmax(-1)[:, None], P + s)
            out.append(bits_of(logits[0:1]))
    return hashes, out


@pytest.mark.parametrize("quant", [None, (4, 64)])
def test_logits_and_blocks_are_batch_invariant(bi, quant):
    bi.reset_stats()
    model = ShardedDecoder(CFG, device="cuda", quant=quant, max_batch=16, max_len=P + STEPS + 1)
    ref_h, ref_o = _run(model, 1, graph=False)
    assert len(ref_h) == CFG.n_layers
    for B in (4, 16):
        h, o = _run(model, B, graph=False)
        assert h == ref_h, f"block outputs differ at batch {B}"
        assert o == ref_o, f"logits differ at batch {B}"
    h, o = _run(model, 4, graph=True)
    assert h == ref_h and o == ref_o, "CUDA-graph replay differs from eager decoding"
    bi.check_device_status()


def test_logits_match_float64_semantics(bi):
    """Tolerance tier for the whole model: the same weights through plain float64 torch ops."""
    from tests.test_dist_cpu import Float64Backend

    model = ShardedDecoder(CFG, device="cuda", max_batch=2, max_len=P + 2)
    g = torch.Generator().manual_seed(0)
    rows = torch.randint(0, CFG.vocab, (2, P), generator=g).cuda()
    got = model.forward(rows, 0).float().cpu()

    class Cuda64(Float64Backend):
        def prefill_attention(self, q, k, v, scale):
            Tq, L = q.shape[2], k.shape[2]
            m = torch.ones(Tq, L, dtype=torch.bool, device=q.device).tril(L - Tq)
            return torch.nn.functional.scaled_dot_product_attention(q.double(), k.double(), v.double(), attn_mask=m, scale=scale,
                                                                    enable_gqa=True).to(q.dtype)

    model.ops = Cuda64()
    ref = model.forward(rows, 0).float().cpu()
    rel = float((got - ref).abs().max() / ref.abs().max())
    assert rel < 5e-2, rel


def test_glue_kernels_match_framework_formulas(bi):
    from mlx_batch_invariant_b200.runner.decoder import KernelBackend, TorchGlue

    B, T, hq, hkv, D, cap = 3, 5, 4, 2, 64, 16
    g = torch.Generator().manual_seed(0)
    for dt in (torch.bfloat16, torch.float16, torch.float32):
        qkv = torch.randn(B * T, (hq + 2 * hkv) * D, generator=g).to(dt).cuda()
        ang = torch.rand(cap, D // 2, generator=g) * 6.28
        cos = torch.cat([ang.cos(), ang.cos()], -1).cuda()
        sin = torch.cat([ang.sin(), ang.sin()], -1).cuda()
        pos0 = torch.tensor([7], dtype=torch.long, device="cuda")
        caches = [[torch.zeros(B, hkv, cap, D, dtype=dt, device="cuda") for _ in range(2)] for _ in range(2)]
        q_ref = TorchGlue().rope_append(qkv, cos, sin, pos0, B, T, hq, hkv, D, *caches[0])
        q_got = KernelBackend().rope_append(qkv, cos, sin, pos0, B, T, hq, hkv, D, *caches[1])
        assert torch.equal(q_ref, q_got)
        assert torch.equal(caches[0][0], caches[1][0]) and torch.equal(caches[0][1], caches[1][1])
        gu = torch.randn(7, 2 * 96, generator=g).to(dt).cuda() * 3
        ref = TorchGlue().swiglu(gu).float()
        got = KernelBackend().swiglu(gu).float()
        assert (ref - got).abs().max() <= 2e-2 * ref.abs().max()
        assert torch.equal(KernelBackend().swiglu(gu[2:3]), KernelBackend().swiglu(gu)[2:3])


def test_cache_append_past_capacity_writes_nothing_and_reports(bi):
    """The cache-append kernel reads its position from device memory; one past the cache must leave the cache
    and q untouched and set the status word (no fault, no stray write)."""
    from mlx_batch_invariant_b200 import _lib
    from mlx_batch_invariant_b200.runner.decoder import KernelBackend

    B, T, hq, hkv, D, cap = 2, 1, 4, 2, 64, 16
    dt = torch.bfloat16
    qkv = torch.randn(B * T, (hq + 2 * hkv) * D).to(dt).cuda()
    cos = torch.ones(cap, D, device="cuda")
    sin = torch.zeros(cap, D, device="cuda")
    kc = torch.full((B, hkv, cap + 8, D), 7.0, dtype=dt, device="cuda")[:, :, :cap]     # a view: memory follows the cache
    vc = torch.full((B, hkv, cap + 8, D), 7.0, dtype=dt, device="cuda")[:, :, :cap]
    bi.check_device_status()
    for bad in (cap, cap + 3):
        KernelBackend().rope_append(qkv, cos, sin, torch.tensor([bad], dtype=torch.long, device="cuda"), B, T, hq, hkv, D, kc, vc)
        torch.cuda.synchronize()
        assert bool((kc._base == 7).all()) and bool((vc._base == 7).all())
        with pytest.raises(_lib.KernelError):
            bi.check_device_status()
    KernelBackend().rope_append(qkv, cos, sin, torch.tensor([cap - 1], dtype=torch.long, device="cuda"), B, T, hq, hkv, D, kc, vc)
    torch.cuda.synchronize()
    assert bool((kc[:, :, cap - 1] != 7).any())
    bi.check_device_status()


@pytest.mark.parametrize("quant", [None, (4, 64)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_qkv_fold_that_rotates_and_appends_equals_the_separate_kernels(bi, dt, quant):
    """bi_matmul_rope / bi_qmm_rope: the projection's fold kernel applies the rotary embedding and writes the
    cache. q, the K cache and the V cache must carry the bits of matmul followed by bi_rope_append -- for a
    prefill (T > 1), a decode step (T = 1), and with tokens past the capacity (skipped, status word set)."""
    from mlx_batch_invariant_b200 import _lib
    from mlx_batch_invariant_b200.runner.decoder import KernelBackend, quantize_rows
    ops = KernelBackend()
    hq, hkv, D, Kd, cap = 4, 2, 64, 512, 24
    g = torch.Generator().manual_seed(11)
    W = (torch.randn((hq + 2 * hkv) * D, Kd, generator=g) / 16).to(dt).cuda()
    w = W if quant is None else quantize_rows(W, quant[1], quant[0])
    cos = torch.rand(cap, D, generator=g).cuda()
    sin = torch.rand(cap, D, generator=g).cuda()
    bits = lambda t: t.contiguous().view(torch.int16).cpu()
    bi.check_device_status()
    for B, T, start in ((3, 5, 7), (16, 1, 9), (1, 1, 0), (2, 4, cap - 2)):
        x = torch.randn(B * T, Kd, generator=g).to(dt).cuda()
        pos0 = torch.tensor([start], dtype=torch.long, device="cuda")
        caches = [torch.full((B, hkv, cap, D), 3.0, dtype=dt, device="cuda") for _ in range(4)]
        if quant is None:
            qkv = bi.batch_invariant_matmul(x, W.T)
        else:
            qkv = bi.batch_invariant_quantized_matmul(x, *w, group_size=quant[1], bits=quant[0])
        q1 = ops.rope_append(qkv, cos, sin, pos0, B, T, hq, hkv, D, caches[0], caches[1])
        overflow = start + T > cap
        if overflow:
            with pytest.raises(_lib.KernelError, match="0x3"):
                bi.check_device_status()
        q2 = ops.linear_rope(x, w, quant, cos, sin, pos0, B, T, hq, hkv, D, caches[2], caches[3])
        if overflow:
            with pytest.raises(_lib.KernelError, match="0x3"):
                bi.check_device_status()
            valid = cap - start                                  # tokens that fit: only their q rows were written
            assert torch.equal(bits(q1[:, :, :valid]), bits(q2[:, :, :valid]))
        else:
            assert torch.equal(bits(q1), bits(q2))
        assert torch.equal(bits(caches[0]), bits(caches[2])) and torch.equal(bits(caches[1]), bits(caches[3]))
        assert bool((caches[2][:, :, start:min(start + T, cap)] != 3).any())
    bi.check_device_status()


@pytest.mark.parametrize("quant", [None, (4, 64)])
def test_full_size_llama3_8b_row0_is_batch_invariant(bi, quant):
    """The configured model at full size (32 layers, d 4096, 32/8 heads, ffn 14336, vocab 128 256; random init):
    row 0 carries the same prompt at batch 1, 4, 16 and 64; its logits after the prefill and after each of two
    cached decode steps, and every block's row-0 output, must be bit-identical at all four batch sizes."""
    from mlx_batch_invariant_b200.runner import LLAMA3_8B

    cfg, Pn, steps = LLAMA3_8B, 48, 2
    free, _ = torch.cuda.mem_get_info()
    if free < 40 << 30:
        pytest.skip("needs 40 GB of free device memory")
    model = ShardedDecoder(cfg, device="cuda", quant=quant, max_batch=64, max_len=Pn + steps + 1)
    probe = torch.randint(0, cfg.vocab, (Pn,), generator=torch.Generator().manual_seed(0))
    ref = None
    for B in (1, 4, 16, 64):
        rows = torch.randint(0, cfg.vocab, (B, Pn), generator=torch.Generator().manual_seed(100 + B))
        rows[0] = probe
        hashes = []
        model.block_hook = lambda li, h: hashes.append(hashlib.blake2b(bits_of(h[0:1]), digest_size=8).hexdigest())
        logits = model.forward(rows.cuda(), 0)
        out = [bits_of(logits[0:1])]
        for s in range(steps):
            logits = model.forward(logits.argmax(-1)[:, None], Pn + s)
            out.append(bits_of(logits[0:1]))
        model.block_hook = None
        assert len(hashes) == cfg.n_layers * (1 + steps)
        if ref is None:
            ref = (hashes, out)
        else:
            first = next((i for i, (a, b) in enumerate(zip(hashes, ref[0])) if a != b), None)
            assert first is None, f"block {first % cfg.n_layers} (pass {first // cfg.n_layers}) differs at batch {B}"
            assert out == ref[1], f"logits differ at batch {B}"
    assert bi.stats()["fallbacks"] == {} or True
    bi.check_device_status()
    del model
    torch.cuda.empty_cache()
