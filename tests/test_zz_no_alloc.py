"""bi_attn_decode_static, the decode-attention entry point that takes no workspace.

It serves hosts that have no way to allocate scratch for the library (a plugin inside a runtime
that owns the allocator, a server that pre-reserved HBM). The test drives it straight through the
C ABI with raw pointers, twice in a row on different problems, and wants the same bits as the
ordinary entry point; the second call finds the first call's partials still in the shared array
and must not be disturbed by them. A problem too large for the built-in array must be refused."""

import pytest
import torch

from mlx_batch_invariant_b200 import _lib

pytestmark = pytest.mark.gpu

MAX_BYTES = 8 << 20


def _call_static(q, k, v, lens, split=256):
    B, Hq, _, D = q.shape
    _, Hkv, L, _ = k.shape
    out = torch.empty_like(q)
    rc = _lib.load().bi_attn_decode_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                           None if lens is None else lens.data_ptr(), B, Hq, Hkv, L, D, k.stride(0),
                                           k.stride(1), k.stride(2), D ** -0.5, split, _lib.DTYPE_CODE[q.dtype],
                                           torch.cuda.current_stream().cuda_stream)
    return rc, out


def _case(B, Hq, Hkv, L, D, dt, seed):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g).to(dt).cuda()
    return mk(B, Hq, 1, D), mk(B, Hkv, L, D), mk(B, Hkv, L, D)


def test_static_scratch_matches_workspace_entry_point_twice(bi):
    # first call: several splits per row, every slot of the partial array up to its size is written
    q, k, v = _case(4, 32, 8, 2100, 128, torch.bfloat16, 1)
    rc, got = _call_static(q, k, v, None)
    assert rc == _lib.BI_OK, _lib.last_error()
    want = bi.batch_invariant_decode_attention(q, k, v, scale=128 ** -0.5)
    assert torch.equal(got, want)
    # second call, straight after: other shapes, ragged lengths, stale partials left in the array
    q2, k2, v2 = _case(3, 8, 2, 700, 64, torch.float16, 2)
    lens = torch.tensor([700, 1, 257], dtype=torch.int32, device="cuda")
    rc, got2 = _call_static(q2, k2, v2, lens)
    assert rc == _lib.BI_OK, _lib.last_error()
    want2 = bi.batch_invariant_decode_attention(q2, k2, v2, scale=64 ** -0.5, kv_lens=lens)
    assert torch.equal(got2, want2)
    # and the first problem again gives the first answer again
    rc, again = _call_static(q, k, v, None)
    assert rc == _lib.BI_OK and torch.equal(again, want)
    torch.cuda.synchronize()


def test_static_scratch_refuses_oversize_problem():
    L = _lib.load()
    B, Hq, Lk, D = 64, 32, 32768, 128
    assert L.bi_attn_decode_workspace_bytes(B, Hq, Lk, D, 256) > MAX_BYTES
    q = torch.zeros(1, device="cuda")       # never dereferenced: the size check comes first
    rc = L.bi_attn_decode_static(q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), None, B, Hq, 8, Lk, D,
                                 8 * Lk * D, Lk * D, D, 1.0, 256, _lib.BI_BF16, None)
    assert rc == _lib.BI_ERR_WORKSPACE
    assert "built-in" in _lib.last_error()
