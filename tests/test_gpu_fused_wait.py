"""The pieces of the fused peer gather that one GPU can check: the gather kernel that computes the SwiGLU gate
on the way (world of one: the destination is local memory), the *_awaiting entry points -- with the peers'
flags already raised they give the bits of the plain entry points; with a flag that nothing raises the bounded
wait runs out, the status word says so, and the context stays usable --, the *_push entry points (matmul,
quantized matmul, decode attention) as one rank of a world of two whose destinations both live on this GPU, and
the kernels launched with programmatic dependent launch. (The exchange between GPUs itself is covered by
tests/test_gpu_multi.py.)"""

import ctypes
import time

import pytest
import torch

from mlx_batch_invariant_b200 import _lib
from oracle import reference as R

pytestmark = pytest.mark.gpu


def _await_args(flags, epoch_word, rank=0, world=2):
    return (flags.data_ptr(), epoch_word.data_ptr(), rank, world)


def test_swiglu_computed_inside_the_gather(bi):
    from mlx_batch_invariant_b200.runner.decoder import KernelBackend
    lib = _lib.load()
    for dt in (torch.bfloat16, torch.float16, torch.float32):
        gu = (3 * torch.randn(7, 2 * 96, generator=torch.Generator().manual_seed(1))).to(dt).cuda()
        want = KernelBackend().swiglu(gu)
        dst = torch.zeros(7, 96, dtype=dt, device="cuda")
        flags = torch.zeros(8, dtype=torch.int32, device="cuda")
        counters = torch.zeros(2, dtype=torch.int32, device="cuda")
        arr = ctypes.c_void_p * 1
        for wait in (1, 0):
            dst.zero_()
            _lib.check(lib.bi_push_gather_swiglu(gu.data_ptr(), arr(dst.data_ptr()), arr(flags.data_ptr()), counters.data_ptr(), 7, 96,
                                                 _lib.DTYPE_CODE[dt], 0, 1, wait, _lib.status_word(gu.device).data_ptr(),
                                                 torch.cuda.current_stream().cuda_stream))
            assert R.bits_of(dst) == R.bits_of(want)
        assert int(counters[1]) == 2 and int(counters[0]) == 0          # two gathers: epoch 2, arrival counter back at 0
    bi.check_device_status()


def test_awaiting_entry_points_with_raised_flags_give_the_plain_bits(bi):
    from mlx_batch_invariant_b200.runner.decoder import KernelBackend, quantize_rows
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(2)
    x = torch.randn(64, 4096, generator=g).to(dt).cuda()
    w = (torch.randn(512, 4096, generator=g) / 64).to(dt).cuda()
    flags = torch.tensor([0, 5, 0, 0, 0, 0, 0, 0], dtype=torch.int32, device="cuda")   # the peer (rank 1) is at epoch 5
    epoch = torch.tensor([5], dtype=torch.int32, device="cuda")
    aw = _await_args(flags, epoch)
    for M in (1, 16, 64):
        for path in ("auto", "split", "fused"):
            assert R.bits_of(bi.batch_invariant_matmul(x[:M], w.T, path=path, awaiting=aw)) == R.bits_of(bi.batch_invariant_matmul(x[:M], w.T, path=path))
        p, s, b = quantize_rows(w, 64, 4)
        plain = bi.batch_invariant_quantized_matmul(x[:M], p, s, b, group_size=64, bits=4)
        assert R.bits_of(bi.batch_invariant_quantized_matmul(x[:M], p, s, b, group_size=64, bits=4, awaiting=aw)) == R.bits_of(plain)
    nw = torch.ones(4096, dtype=dt, device="cuda")
    s0, h0 = KernelBackend().add_rms_norm(x, x.flip(0).contiguous(), nw, 1e-5)
    s1, h1 = KernelBackend().add_rms_norm(x, x.flip(0).contiguous(), nw, 1e-5, awaiting=aw)
    assert R.bits_of(s0) == R.bits_of(s1) and R.bits_of(h0) == R.bits_of(h1)
    bi.check_device_status()


def test_a_flag_that_nothing_raises_runs_the_bounded_wait_out(bi):
    """Failure detection without a fault: the peer never signals, the kernel gives up after its time limit
    (2 s), records which peer and epoch it waited for, and returns; the next call works."""
    dt = torch.bfloat16
    x = torch.randn(8, 1024, device="cuda", dtype=dt)
    w = torch.randn(256, 1024, device="cuda", dtype=dt) / 32
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    epoch = torch.tensor([3], dtype=torch.int32, device="cuda")
    bi.check_device_status()
    t0 = time.perf_counter()
    bi.batch_invariant_matmul(x, w.T, awaiting=_await_args(flags, epoch))
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert 1.5 < waited < 30, waited
    with pytest.raises(_lib.KernelError, match="0x20103"):               # 0x20000 | peer 1 << 8 | epoch 3
        bi.check_device_status()
    assert R.bits_of(bi.batch_invariant_matmul(x, w.T)) == R.bits_of(bi.batch_invariant_matmul(x[:8], w.T, path="fused"))
    bi.check_device_status()


def test_ops_that_push_their_own_output(bi):
    """bi_matmul_push / bi_qmm_push / bi_attn_decode_push as rank 1 of a world of two whose two destinations both
    live on this GPU: the op's bits land in columns [N, 2N) of BOTH destinations, the other columns stay
    untouched, the rank's flag goes up at the peer only, and the epoch advances by one per call."""
    from mlx_batch_invariant_b200.runner.decoder import quantize_rows
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(3)
    x = torch.randn(64, 4096, generator=g).to(dt).cuda()
    w = (torch.randn(512, 4096, generator=g) / 64).to(dt).cuda()
    packed = quantize_rows(w, 64, 4)
    flags = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(2)]
    counters = torch.zeros(2, dtype=torch.int32, device="cuda")
    arr = ctypes.c_void_p * 2
    epoch = 0

    def pushed(rows, cols, run):
        nonlocal epoch
        dst = [torch.zeros(rows, 2 * cols, dtype=dt, device="cuda") for _ in range(2)]
        push = (arr(dst[0].data_ptr(), dst[1].data_ptr()), arr(flags[0].data_ptr(), flags[1].data_ptr()), counters.data_ptr(), 1, 2, 0)
        assert run(push) is None
        epoch += 1
        assert int(counters[1]) == epoch and int(counters[0]) == 0
        assert int(flags[0][1]) == epoch and int(flags[1][1]) == 0 and int(flags[0][0]) == 0
        for d in dst:
            assert int((d[:, :cols] != 0).sum()) == 0
        assert R.bits_of(dst[0][:, cols:]) == R.bits_of(dst[1][:, cols:])
        return dst[0][:, cols:]

    for M in (1, 7, 64):
        want = bi.batch_invariant_matmul(x[:M], w.T)
        assert R.bits_of(pushed(M, 512, lambda push: bi.batch_invariant_matmul(x[:M], w.T, push=push))) == R.bits_of(want)
        want = bi.batch_invariant_quantized_matmul(x[:M], *packed, group_size=64, bits=4)
        got = pushed(M, 512, lambda push: bi.batch_invariant_quantized_matmul(x[:M], *packed, group_size=64, bits=4, push=push))
        assert R.bits_of(got) == R.bits_of(want)
    # the activation itself a gathered buffer that is waited for in the kernel, the output pushed on
    aw = (flags[1].data_ptr(), counters[1:].data_ptr(), 1, 2)
    flags[1][0] = epoch                                            # "rank 0" has delivered the gather before this one
    want = bi.batch_invariant_matmul(x, w.T)
    assert R.bits_of(pushed(64, 512, lambda push: bi.batch_invariant_matmul(x, w.T, push=push, awaiting=aw))) == R.bits_of(want)
    flags[1].zero_()
    for B, L in ((3, 300), (16, 600)):
        q = torch.randn(B, 4, 1, 128, generator=g).to(dt).cuda()
        k = torch.randn(B, 1, L, 128, generator=g).to(dt).cuda()
        v = torch.randn(B, 1, L, 128, generator=g).to(dt).cuda()
        lens = torch.randint(1, L + 1, (B,), generator=g).to(torch.int32).cuda()
        want = bi.batch_invariant_decode_attention(q, k, v, scale=0.09, kv_lens=lens).reshape(B, 4 * 128)
        got = pushed(B, 4 * 128, lambda push: bi.batch_invariant_decode_attention(q, k, v, scale=0.09, kv_lens=lens, push=push))
        assert R.bits_of(got) == R.bits_of(want)
    bi.check_device_status()


def test_programmatic_dependent_launch_gives_the_same_bits(bi, monkeypatch):
    """BI_PDL=1 launches the kernels so that each may start while the one before it drains (every kernel waits
    for its predecessors before it touches global memory). A chain of dependent ops, eagerly and from a replayed
    CUDA graph, must give the bits of the plain launches."""
    from mlx_batch_invariant_b200.runner.decoder import KernelBackend
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(4)
    x = torch.randn(16, 1024, generator=g).to(dt).cuda()
    w1 = (torch.randn(1024, 1024, generator=g) / 32).to(dt).cuda()
    w2 = (torch.randn(2048, 1024, generator=g) / 32).to(dt).cuda()
    nw = torch.ones(1024, dtype=dt, device="cuda")
    q = torch.randn(16, 8, 1, 128, generator=g).to(dt).cuda()
    k = torch.randn(16, 2, 300, 128, generator=g).to(dt).cuda()
    v = torch.randn(16, 2, 300, 128, generator=g).to(dt).cuda()
    ops = KernelBackend()

    def chain():
        h = bi.batch_invariant_matmul(x, w1.T, path="split")
        s, h = ops.add_rms_norm(x, h, nw, 1e-5)
        h = ops.swiglu(bi.batch_invariant_matmul(h, w2.T))
        a = bi.batch_invariant_decode_attention(q, k, v, scale=0.09).reshape(16, 1024)
        return bi.batch_invariant_matmul(h + a, w1.T, path="fused"), s

    want = [R.bits_of(t) for t in chain()]
    monkeypatch.setenv("BI_PDL", "1")
    assert [R.bits_of(t) for t in chain()] == want
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = chain()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert [R.bits_of(t) for t in outs] == want
    bi.check_device_status()
