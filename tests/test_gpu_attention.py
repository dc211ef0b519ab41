"""Split-KV attention on the GPU, through the C ABI: bit for bit against the CPU oracle at sizes
the oracle finishes quickly, structure identities at the configured sizes."""

import numpy as np
import pytest
import torch

from oracle import reference as R
from tests.golden import make_golden

pytestmark = pytest.mark.gpu
DTS = [torch.float32, torch.bfloat16, torch.float16]
TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-2}


def qkv(B, Hq, Hkv, Tq, L, D, dt, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(B, Hq, Tq, D, generator=g).to(dt), torch.randn(B, Hkv, L, D, generator=g).to(dt),
            torch.randn(B, Hkv, L, D, generator=g).to(dt))


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("L", [1, 255, 256, 257, 600])
def test_decode_bit_exact_vs_oracle(bi, dt, L):
    q, k, v = qkv(2, 8, 2, 1, L, 128, dt, L)
    got = bi.batch_invariant_decode_attention(q.cuda(), k.cuda(), v.cuda(), scale=128 ** -0.5)
    assert R.bits_of(got) == R.bits_of(R.attn_decode(q, k, v, scale=128 ** -0.5))


@pytest.mark.parametrize("Hq,Hkv,D", [(4, 4, 64), (6, 3, 32), (16, 2, 64), (3, 1, 128), (4, 2, 256), (5, 5, 128)])
def test_decode_head_layouts(bi, Hq, Hkv, D):
    q, k, v = qkv(3, Hq, Hkv, 1, 300, D, torch.bfloat16, Hq * 7 + D)
    got = bi.batch_invariant_decode_attention(q.cuda(), k.cuda(), v.cuda(), scale=D ** -0.5)
    assert R.bits_of(got) == R.bits_of(R.attn_decode(q, k, v, scale=D ** -0.5))


@pytest.mark.parametrize("dt", DTS)
def test_decode_mixed_lengths_and_strided_cache(bi, dt):
    B, Hq, Hkv, D, cap = 5, 8, 2, 128, 700
    q, k, v = qkv(B, Hq, Hkv, 1, cap, D, dt, 11)
    lens = [1, 255, 256, 257, 700]
    got = bi.batch_invariant_decode_attention(q.cuda(), k.cuda(), v.cuda(), scale=D ** -0.5, kv_lens=torch.tensor(lens))
    assert R.bits_of(got) == R.bits_of(R.attn_decode(q, k, v, scale=D ** -0.5, kv_lens=lens))
    # each row equals the same sequence decoded alone with an exact-length cache
    for b, n in enumerate(lens):
        alone = bi.batch_invariant_decode_attention(q[b:b + 1].cuda(), k[b:b + 1, :, :n].cuda(), v[b:b + 1, :, :n].cuda(),
                                                    scale=D ** -0.5)
        assert R.bits_of(alone) == R.bits_of(got[b:b + 1])
    # a view into a larger cache is read in place
    kc, vc = k.cuda(), v.cuda()
    view = bi.batch_invariant_decode_attention(q.cuda(), kc[:, :, :300], vc[:, :, :300], scale=D ** -0.5)
    assert R.bits_of(view) == R.bits_of(R.attn_decode(q, k[:, :, :300], v[:, :, :300], scale=D ** -0.5))


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("causal", [True, False])
def test_prefill_bit_exact_vs_oracle(bi, dt, causal):
    q, k, v = qkv(2, 8, 2, 37, 150, 64, dt, 3)
    got = bi.batch_invariant_prefill_attention(q.cuda(), k.cuda(), v.cuda(), scale=0.125, causal=causal)
    want = R.attn_prefill(q, k, v, scale=0.125, causal=causal)
    assert R.bits_of(got) == R.bits_of(want)
    assert R.rel_err(R.attention_f64(q, k, v, scale=0.125, causal=causal), got) < TOL[dt]


@pytest.mark.parametrize("Hq,Hkv,Tq,L,D", [(4, 2, 5, 5, 128), (2, 1, 3, 260, 32), (2, 2, 9, 300, 256), (3, 3, 1, 40, 64)])
def test_prefill_shapes(bi, Hq, Hkv, Tq, L, D):
    q, k, v = qkv(2, Hq, Hkv, Tq, L, D, torch.float16, Tq + L)
    got = bi.batch_invariant_prefill_attention(q.cuda(), k.cuda(), v.cuda(), scale=D ** -0.5, causal=True)
    assert R.bits_of(got) == R.bits_of(R.attn_prefill(q, k, v, scale=D ** -0.5, causal=True))


@pytest.mark.parametrize("dt", DTS)
def test_chunked_prefill_and_decode_equivalence(bi, dt):
    """The reference's structure checks (harness/sweep.py:188-207 there): T=600 cut at 257."""
    B, Hq, Hkv, D, T, T1 = 2, 8, 2, 128, 600, 257
    q, k, v = (t.cuda() for t in qkv(B, Hq, Hkv, T, T, D, dt, 0))
    sc = D ** -0.5
    full = bi.batch_invariant_attention(q, k, v, scale=sc, mask="causal")
    p1 = bi.batch_invariant_attention(q[:, :, :T1], k[:, :, :T1], v[:, :, :T1], scale=sc, mask="causal")
    p2 = bi.batch_invariant_attention(q[:, :, T1:], k, v, scale=sc, mask="causal")
    assert R.bits_of(torch.cat([p1, p2], 2)) == R.bits_of(full)
    dec = bi.batch_invariant_attention(q[:, :, T - 1:T], k, v, scale=sc)
    assert R.bits_of(dec) == R.bits_of(full[:, :, T - 1:T])
    alone = bi.batch_invariant_attention(q[:1], k[:1], v[:1], scale=sc, mask="causal")
    assert R.bits_of(alone) == R.bits_of(full[:1])


def test_configured_prefill_2048_chunks_of_512(bi):
    """bf16, 32 query heads, 8 KV heads, head_dim 128, causal, 2048 tokens: one shot == 4 x 512,
    decode of each chunk's last token == its prefill row, and a sample of rows against float64."""
    Hq, Hkv, D, T = 32, 8, 128, 2048
    q, k, v = (t.cuda() for t in qkv(1, Hq, Hkv, T, T, D, torch.bfloat16, 42))
    sc = D ** -0.5
    full = bi.batch_invariant_attention(q, k, v, scale=sc, mask="causal")
    parts = [bi.batch_invariant_attention(q[:, :, s:s + 512], k[:, :, :s + 512], v[:, :, :s + 512], scale=sc, mask="causal")
             for s in range(0, T, 512)]
    assert R.bits_of(torch.cat(parts, 2)) == R.bits_of(full)
    for t in (1, 512, 1024, 2048):
        dec = bi.batch_invariant_attention(q[:, :, t - 1:t], k[:, :, :t], v[:, :, :t], scale=sc)
        assert R.bits_of(dec) == R.bits_of(full[:, :, t - 1:t])
    for t in (0, 255, 256, 1000, 2047):
        ref_t = R.attention_f64(q[:, :, t:t + 1].cpu(), k[:, :, :t + 1].cpu(), v[:, :, :t + 1].cpu(), scale=sc, causal=False)
        assert R.rel_err(ref_t, full[:, :, t:t + 1]) < 2e-2


def test_configured_decode_long_and_mixed_batches(bi):
    """Cache lengths {1,255,256,257,4096,32768}, batches 1..64 mixing them: every row equals the
    row decoded alone (bitwise); the oracle pins rows short enough to finish quickly."""
    Hq, Hkv, D = 32, 8, 128
    sc = D ** -0.5
    pool = [1, 255, 256, 257, 4096, 32768]
    g = torch.Generator().manual_seed(7)
    cap = 32768
    kc = torch.randn(8, Hkv, cap, D, generator=g).to(torch.bfloat16).cuda()   # 8 distinct caches, reused round-robin
    vc = torch.randn(8, Hkv, cap, D, generator=g).to(torch.bfloat16).cuda()
    qs = torch.randn(64, Hq, 1, D, generator=g).to(torch.bfloat16).cuda()
    alone = {}
    for B in (1, 4, 16, 64):
        idx = torch.arange(B) % 8
        lens = [pool[(b * 5 + B) % len(pool)] for b in range(B)]
        out = bi.batch_invariant_decode_attention(qs[:B], kc[idx], vc[idx], scale=sc, kv_lens=torch.tensor(lens))
        for b in range(B):
            key = (b, int(idx[b]), lens[b])
            if key not in alone:
                c = int(idx[b])
                alone[key] = bi.batch_invariant_decode_attention(qs[b:b + 1], kc[c:c + 1, :, :lens[b]], vc[c:c + 1, :, :lens[b]], scale=sc)
            assert R.bits_of(out[b:b + 1]) == R.bits_of(alone[key]), (B, b, lens[b])
    for (b, c, n), got in list(alone.items())[:12]:
        if n <= 4096:
            want = R.attn_decode(qs[b:b + 1].cpu(), kc[c:c + 1, :, :n].cpu(), vc[c:c + 1, :, :n].cpu(), scale=sc)
            assert R.bits_of(got) == R.bits_of(want)
    long = next(v for (b, c, n), v in alone.items() if n == 32768)
    b, c, n = next(k for k in alone if k[2] == 32768)
    ref = R.attention_f64(qs[b:b + 1].cpu(), kc[c:c + 1].cpu(), vc[c:c + 1].cpu(), scale=sc, causal=False)
    assert R.rel_err(ref, long) < 2e-2


@pytest.mark.parametrize("name", ["f32", "bf16", "f16"])
def test_golden_fixture(bi, name):
    gold = np.load(make_golden.OUT)
    i = make_golden.inputs(name)
    q, k, v = i["q"].cuda(), i["k"].cuda(), i["v"].cuda()
    pre = bi.batch_invariant_prefill_attention(q, k, v, scale=0.125, causal=True)
    assert make_golden.raw(pre).tobytes() == gold[f"{name}_prefill"].tobytes()
    dec = bi.batch_invariant_decode_attention(q[:, :, -1:], k, v, scale=0.125, kv_lens=torch.tensor([265, 100]))
    assert make_golden.raw(dec).tobytes() == gold[f"{name}_decode"].tobytes()


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("page", [32, 64, 256])
def test_paged_cache_gives_the_bits_of_the_contiguous_cache(bi, dt, page):
    """The same keys scattered over a shuffled page pool, found through a block table, give the bits of the
    contiguous cache (and of the oracle): only the address of a key's row differs."""
    import mlx_batch_invariant_b200 as m
    B, Hq, Hkv, D = 5, 8, 2, 128
    lens = [1, 255, 257, 600, 700]
    cap = 768
    q, k, v = qkv(B, Hq, Hkv, 1, cap, D, dt, page)
    want = R.attn_decode(q, k, v, scale=D ** -0.5, kv_lens=lens)
    per_seq = cap // page
    g = torch.Generator().manual_seed(7)
    perm = torch.randperm(B * per_seq + 3, generator=g)[:B * per_seq].reshape(B, per_seq).to(torch.int32)
    kp = torch.zeros(B * per_seq + 3, Hkv, page, D, dtype=dt)
    vp = torch.zeros_like(kp)
    for b in range(B):
        for i in range(per_seq):
            kp[perm[b, i]] = k[b, :, i * page:(i + 1) * page]
            vp[perm[b, i]] = v[b, :, i * page:(i + 1) * page]
    got = m.batch_invariant_paged_decode_attention(q.cuda(), kp.cuda(), vp.cuda(), perm.cuda(), torch.tensor(lens), scale=D ** -0.5)
    assert R.bits_of(got) == R.bits_of(want)
    flat = bi.batch_invariant_decode_attention(q.cuda(), k.cuda(), v.cuda(), scale=D ** -0.5, kv_lens=torch.tensor(lens))
    assert R.bits_of(got) == R.bits_of(flat)
