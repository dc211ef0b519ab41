"""Sharded decoder logic on CPU ranks (gloo, world_size 2): column-parallel linears, KV-head
sharded attention and rank-major all-gather must reproduce the unsharded model. The four ops
are stood in for by float64 torch code (the kernels have no CPU path; this test is about the
index math and the collectives, not the kernels)."""

import os
import socket
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from mlx_batch_invariant_b200.runner import DecoderConfig, ShardedDecoder, greedy_generate  # noqa: E402
from mlx_batch_invariant_b200.runner.decoder import TorchGlue  # noqa: E402

CFG = DecoderConfig(n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn=128, vocab=96)


class Float64Backend(TorchGlue):
    def linear(self, x, w):
        return (x.double() @ w.double().T).to(x.dtype)

    def qlinear(self, x, packed, gs, bits):
        from oracle.reference import dequant_f64
        p, s, b = packed
        wd = torch.from_numpy(dequant_f64(p, s, b, group_size=gs, bits=bits))
        return (x.double() @ wd.T).to(x.dtype)

    def rms_norm(self, x, w, eps):
        xf = x.double()
        return (xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * w.double()).to(x.dtype)

    def prefill_attention(self, q, k, v, scale):
        Tq, L = q.shape[2], k.shape[2]
        m = torch.ones(Tq, L, dtype=torch.bool).tril(L - Tq)
        return torch.nn.functional.scaled_dot_product_attention(q.double(), k.double(), v.double(), attn_mask=m,
                                                                scale=scale, enable_gqa=True).to(q.dtype)

    def decode_attention(self, q, k, v, scale, kv_lens=None):
        return torch.nn.functional.scaled_dot_product_attention(q.double(), k.double(), v.double(), scale=scale,
                                                                enable_gqa=True).to(q.dtype)


def _model(rank, world, quant):
    return ShardedDecoder(CFG, rank=rank, world=world, device="cpu", dtype=torch.float32, backend=Float64Backend(),
                          quant=quant, max_batch=3, max_len=32)


def _worker(rank, world, port, quant, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        prompts = torch.randint(0, CFG.vocab, (3, 7))
        toks, logits = greedy_generate(_model(rank, world, quant), prompts, 4)
        gathered = [torch.empty_like(logits) for _ in range(world)]
        dist.all_gather(gathered, logits)
        assert all(torch.equal(g, logits) for g in gathered), "ranks disagree on the gathered logits"
        if rank == 0:
            torch.save({"toks": toks, "logits": logits}, out_path)
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(quant, tmp_path):
    out = tmp_path / "r0.pt"
    mp.spawn(_worker, args=(2, _free_port(), quant, str(out)), nprocs=2, join=True)
    got = torch.load(out)
    torch.manual_seed(0)
    prompts = torch.randint(0, CFG.vocab, (3, 7))
    toks, logits = greedy_generate(_model(0, 1, quant), prompts, 4)
    assert torch.equal(got["toks"], toks)
    assert torch.allclose(got["logits"], logits, rtol=1e-5, atol=1e-6)


def test_two_rank_sharding_matches_single_rank_dense(tmp_path):
    _run(None, tmp_path)


def test_two_rank_sharding_matches_single_rank_quantized(tmp_path):
    _run((4, 32), tmp_path)


def test_shards_are_slices_of_the_full_weights():
    full = _model(0, 1, None)
    parts = [_model(r, 2, None) for r in range(2)]
    assert torch.equal(torch.cat([p.layers[1]["down"] for p in parts], 0), full.layers[1]["down"])
    for p in parts:                                  # the output projection is replicated, not sliced
        assert torch.equal(p.layers[1]["o"], full.layers[1]["o"])
    assert torch.equal(torch.cat([p.head for p in parts], 0), full.head)
    hq, hkv, D = CFG.n_heads // 2, CFG.n_kv_heads // 2, CFG.head_dim
    fq = full.layers[0]["qkv"]
    for r, p in enumerate(parts):
        q_rows = fq[r * hq * D:(r + 1) * hq * D]
        k_rows = fq[CFG.n_heads * D + r * hkv * D: CFG.n_heads * D + (r + 1) * hkv * D]
        assert torch.equal(p.layers[0]["qkv"][:hq * D], q_rows)
        assert torch.equal(p.layers[0]["qkv"][hq * D:(hq + hkv) * D], k_rows)


def test_quantizing_a_shard_equals_the_shard_of_the_quantized_matrix():
    full = _model(0, 1, (4, 32))
    parts = [_model(r, 2, (4, 32)) for r in range(2)]
    for i in range(3):
        assert torch.equal(torch.cat([p.layers[0]["down"][i] for p in parts], 0), full.layers[0]["down"][i])


def test_world_must_divide_the_sharded_dims():
    import pytest
    with pytest.raises(ValueError):
        ShardedDecoder(CFG, rank=0, world=4, device="cpu", dtype=torch.float32, backend=Float64Backend())


def test_peer_gather_buffer_rotation_never_reuses_a_live_buffer():
    """Replaying a captured sequence of n gathers: consecutive gathers, also across the replay boundary and
    across the switch from the eager warm-up, must land in different destination buffers."""
    from mlx_batch_invariant_b200.runner.peer import NBUF, pick_cycle
    for n in range(2, 400):
        for warm in (0, 1, 2, 3, 7):
            last_eager = (warm - 1) % 3 if warm else None
            mod, calls = pick_cycle(n, 3, warm)
            assert 3 <= mod <= NBUF
            seq = [(calls + i) % mod for i in range(n)]
            if last_eager is not None:
                assert seq[0] != last_eager
            replayed = seq + seq
            assert all(a != b for a, b in zip(replayed, replayed[1:]))
    import pytest
    with pytest.raises(RuntimeError):
        pick_cycle(421, 3, 0)                         # 1 mod 3, 4, 5 and 7: no modulus on offer works


def test_cache_capacity_is_checked_on_the_host_before_any_launch():
    """A prompt or a decode step that would run past the KV cache or the rotary tables raises on the host;
    nothing reaches a kernel (the cache-append kernel takes its position from device memory)."""
    import pytest
    from mlx_batch_invariant_b200.runner import GraphedDecoder

    m = _model(0, 1, None)                                         # max_batch 3, max_len 32
    with pytest.raises(ValueError, match="max_len"):
        m.forward(torch.zeros(2, 33, dtype=torch.long), 0)
    with pytest.raises(ValueError, match="max_len"):
        m.forward(torch.zeros(2, 4, dtype=torch.long), 30)
    with pytest.raises(ValueError, match="max_batch"):
        m.forward(torch.zeros(4, 2, dtype=torch.long), 0)
    m.forward(torch.zeros(3, 32, dtype=torch.long), 0)              # exactly full is fine
    gd = GraphedDecoder(m, 3)
    with pytest.raises(ValueError, match="max_len"):
        gd.start(torch.zeros(3, dtype=torch.long), 32)
    gd.start(torch.zeros(3, dtype=torch.long), 30)
    gd.step()
    gd.step()                                                      # positions 30 and 31: the last two slots
    with pytest.raises(ValueError, match="max_len"):
        gd.step()
    with pytest.raises(ValueError, match="max_batch"):
        GraphedDecoder(m, 4)
