"""Determinism across GPU counts: the small decoder sharded over 2 (and 4, 8 when present) GPUs with NCCL
all-gather must give the logits of the single-GPU run bit for bit, prefill and decode, dense and 4-bit
(one process per GPU; skipped on a single-GPU box)."""

import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

pytestmark = pytest.mark.gpu

P, STEPS, B = 40, 3, 5


def _cfg():
    from mlx_batch_invariant_b200.runner import DecoderConfig
    return DecoderConfig(n_layers=2, d_model=512, n_heads=8, n_kv_heads=8, head_dim=64, ffn=1024, vocab=2048)


def _generate(rank, world, quant):
    from mlx_batch_invariant_b200.runner import GraphedDecoder, ShardedDecoder
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    model = ShardedDecoder(_cfg(), rank=rank, world=world, device=dev, quant=quant, max_batch=B, max_len=P + STEPS + 2)
    g = torch.Generator().manual_seed(3)
    rows = torch.randint(0, 2048, (B, P), generator=g).to(dev)
    logits = model.forward(rows, 0)
    outs = [logits.cpu()]
    for s in range(STEPS):
        logits = model.forward(logits.argmax(-1)[:, None], P + s)
        outs.append(logits.cpu())
    # the same continuation from a captured CUDA graph, replayed (the gathers' buffer rotation repeats)
    model.forward(rows, 0)
    gd = GraphedDecoder(model, B)
    gd.start(outs[0].to(dev).argmax(-1), P)
    gd.capture()
    for s in range(STEPS):
        outs.append(gd.step().clone().cpu())
    return outs


def _worker(rank, world, port, quant, out_path, gather="push"):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0", BI_GATHER=gather)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        outs = _generate(rank, world, quant)
        from mlx_batch_invariant_b200 import check_device_status
        check_device_status(torch.device("cuda", rank))       # no bounded wait of the peer gather ran out
        if rank == 0:
            torch.save(outs, out_path)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("gather", ["push", "nccl"])
@pytest.mark.parametrize("quant", [None, (4, 64)])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_logits_identical_across_gpu_counts(world, quant, gather, tmp_path):
    """gather="push": the peer-memory all-gather of csrc/peer.cu; "nccl": the library collective."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    if gather == "nccl" and quant is not None:
        pytest.skip("the collective's fallback is covered by the dense case")
    ref = _generate(0, 1, quant)
    out = tmp_path / "r0.pt"
    mp.spawn(_worker, args=(world, _free_port(), quant, str(out), gather), nprocs=world, join=True)
    got = torch.load(out)
    assert len(got) == len(ref)
    for i, (a, b) in enumerate(zip(ref, got)):
        assert torch.equal(a, b), f"logits of step {i} differ between 1 and {world} GPUs"
