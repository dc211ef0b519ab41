"""Bit-hash manifest of the kernels' outputs (and a decoder's logits), and a comparer for two manifests.

    python -m mlx_batch_invariant_b200.dump_bits --out bits_a.json [--model small|llama3_8b] [--quant]
    python -m mlx_batch_invariant_b200.dump_bits --compare bits_a.json bits_b.json

The counterpart of the reference's harness/dump_bits.py:32-78: determinism is promised per (library build,
GPU, driver); a manifest records blake2b-8 digests so that two builds, two machines or two GPU counts can be
compared. It covers every op on its probe input in fp16 / bf16 / fp32 -- the stock framework op, the
batch-invariant kernel at batch 1 (``inv``), and the same probe as the LAST row of a batch of 64
(``inv@B64``, which must equal ``inv``) -- and, with ``--model``, row-0 logits of the Llama-architecture
decoder after a prefill and after one cached decode step, at batch 1, 4, 16 and 64 (row 0 is always the same
prompt: all batch sizes must give one digest, the method of harness/model_sweep.py:100-108 there). Under
``torchrun`` the decoder is sharded over the ranks and rank 0 writes the manifest, so manifests taken at 1, 2,
4 and 8 GPUs can be compared with ``--compare``.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys

import torch
import torch.nn.functional as F

import mlx_batch_invariant_b200 as bi
from mlx_batch_invariant_b200 import _lib, ops

DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}
BIG = 64


def digest(t: torch.Tensor) -> str:
    raw = t.detach().contiguous().cpu()
    view = {2: torch.int16, 4: torch.int32}.get(raw.element_size())
    if view is not None:
        raw = raw.view(view)
    return hashlib.blake2b(raw.numpy().tobytes(), digest_size=8).hexdigest()


def _gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


class _Probe:
    """An op with a fixed probe input (row 0 of a batch of one) and seeded filler rows."""

    def batch(self, B: int, pos: int):
        raise NotImplementedError

    def run(self, batch):
        raise NotImplementedError


class _Linear(_Probe):
    K = N = 1024

    def __init__(self, dt, dev):
        g = _gen(0)
        self.dt, self.dev = dt, dev
        self.W = (torch.randn(self.N, self.K, generator=g) / self.K ** 0.5).to(dt).to(dev)
        self.x0 = torch.randn(1, self.K, generator=g).to(dt)

    def batch(self, B, pos):
        rows = torch.randn(B, self.K, generator=_gen(7 * B + pos + 1)).to(self.dt)
        rows[pos] = self.x0[0]
        return rows.to(self.dev)

    def run(self, x):
        return F.linear(x, self.W)


class _QLinear(_Linear):
    bits, gs = 4, 64

    def __init__(self, dt, dev):
        super().__init__(dt, dev)
        from .runner.decoder import quantize_rows
        self.packed = quantize_rows(self.W * 0.5, self.gs, self.bits)

    def run(self, x):
        p, s, b = self.packed
        if not bi.is_batch_invariant_mode_enabled():
            return ops._stock_quantized_matmul(x, p, s, b, True, self.gs, self.bits)
        return ops.quantized_matmul(x, p, s, b, transpose=True, group_size=self.gs, bits=self.bits)


class _QLinear8(_QLinear):
    bits, gs = 8, 32


class _RMSNorm(_Linear):
    def run(self, x):
        return F.rms_norm(x * 3, (self.K,), self.W[0], 1e-5)


class _Decode(_Probe):
    Hq, Hkv, L, D, Tq, causal = 8, 2, 600, 128, 1, False

    def __init__(self, dt, dev):
        g = _gen(0)
        self.dt, self.dev = dt, dev
        self.q0 = torch.randn(1, self.Hq, self.Tq, self.D, generator=g).to(dt)
        self.k0 = torch.randn(1, self.Hkv, self.L, self.D, generator=g).to(dt)
        self.v0 = torch.randn(1, self.Hkv, self.L, self.D, generator=g).to(dt)

    def batch(self, B, pos):
        g = _gen(7 * B + pos + 1)
        q = torch.randn(B, self.Hq, self.Tq, self.D, generator=g).to(self.dt)
        k = torch.randn(B, self.Hkv, self.L, self.D, generator=g).to(self.dt)
        v = torch.randn(B, self.Hkv, self.L, self.D, generator=g).to(self.dt)
        q[pos], k[pos], v[pos] = self.q0[0], self.k0[0], self.v0[0]
        return tuple(t.to(self.dev) for t in (q, k, v))

    def run(self, qkv):
        q, k, v = qkv
        mask = "causal" if self.causal else None
        if not bi.is_batch_invariant_mode_enabled():
            return ops._stock_sdpa(q, k, v, self.D ** -0.5, mask)
        return ops.scaled_dot_product_attention(q, k, v, scale=self.D ** -0.5, mask=mask)


class _Prefill(_Decode):
    Tq, L, causal = 48, 300, True


OPS = {"matmul": _Linear, "qmatmul_4b": _QLinear, "qmatmul_8b": _QLinear8, "rms_norm": _RMSNorm,
       "sdpa_decode": _Decode, "sdpa_prefill": _Prefill}


def dump_ops(dev) -> dict:
    out = {}
    for name, cls in OPS.items():
        for dt_name, dt in DTYPES.items():
            op = cls(dt, dev)
            one = op.batch(1, 0)
            with bi.set_batch_invariant_mode(enabled=False):
                out[f"{name}/{dt_name}/stock"] = digest(op.run(one)[0:1])
            with bi.set_batch_invariant_mode(strict=True):
                out[f"{name}/{dt_name}/inv"] = digest(op.run(one)[0:1])
                out[f"{name}/{dt_name}/inv@B{BIG}"] = digest(op.run(op.batch(BIG, BIG - 1))[BIG - 1:BIG])
    return out


def _decoder_config(name: str):
    from .runner import LLAMA3_8B, DecoderConfig
    if name == "llama3_8b":
        return LLAMA3_8B
    return DecoderConfig(n_layers=4, d_model=1024, n_heads=8, n_kv_heads=8, head_dim=128, ffn=2048, vocab=4096)


def dump_model(name: str, quant, dev, rank: int, world: int, batches, prompt_len: int) -> dict:
    from .runner import ShardedDecoder
    cfg = _decoder_config(name)
    model = ShardedDecoder(cfg, rank=rank, world=world, device=dev, quant=quant, max_batch=max(batches),
                           max_len=prompt_len + 2)
    probe = torch.randint(0, cfg.vocab, (prompt_len,), generator=_gen(0))
    tag = name + ("_q4" if quant else "")
    out = {}
    for B in batches:
        rows = [probe] + [torch.randint(0, cfg.vocab, (prompt_len,), generator=_gen(1000 + 7 * B + r)) for r in range(1, B)]
        toks = torch.stack(rows, 0).to(dev)
        logits = model.forward(toks, 0)
        out[f"{tag}/prefill/B{B}/inv"] = digest(logits[0:1])
        step = model.forward(logits.argmax(-1)[:, None], prompt_len)
        out[f"{tag}/decode/B{B}/inv"] = digest(step[0:1])
    _lib.check_device_status(dev)
    return out


def dump(model_name, quant, batches, prompt_len) -> dict | None:
    if not torch.cuda.is_available():
        raise SystemExit("dump_bits: no CUDA device (the library has no CPU path)")
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    out = {"library": int(lib.bi_version()), "torch": torch.__version__, "cuda": torch.version.cuda,
           "device": torch.cuda.get_device_name(dev), "gpus": world, "ops": {}, "model": {}}
    bi.reset_stats()
    if rank == 0:
        out["ops"] = dump_ops(dev)
    if model_name:
        out["model"] = dump_model(model_name, (4, 64) if quant else None, dev, rank, world, batches, prompt_len)
    out["fallbacks"] = {k: v for k, v in bi.stats()["fallbacks"].items()}
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        torch.cuda.synchronize()
    return out if rank == 0 else None


def compare(a: dict, b: dict) -> int:
    """Print, per section and mode, how many digests the two manifests share; 1 if an invariant digest differs."""
    for tag, d in (("A", a), ("B", b)):
        print(f"{tag}: library {d.get('library')} torch {d.get('torch')} on {d.get('gpus', 1)} x {d.get('device')}")
    print()
    rc = 0
    for section in ("ops", "model"):
        keys = sorted(set(a.get(section, {})) & set(b.get(section, {})))
        if not keys:
            continue
        same = {"stock": [0, 0], "inv": [0, 0]}
        differing = []
        for k in keys:
            mode = "stock" if k.endswith("/stock") else "inv"
            same[mode][1] += 1
            if a[section][k] == b[section][k]:
                same[mode][0] += 1
            else:
                differing.append(k)
                rc |= mode == "inv"
        for mode, (n, tot) in same.items():
            if tot:
                print(f"{section:<6} {mode:<6} identical in both: {n}/{tot}")
        if differing:
            print("  differing: " + ", ".join(differing))
    return int(rc)


def self_check(d: dict) -> list[str]:
    """Invariance inside ONE manifest: inv@B64 equals inv for every op, and every batch size of a model key
    gives one digest. Returns the offending keys."""
    bad = [k for k in d["ops"] if k.endswith("/inv") and d["ops"].get(f"{k}@B{BIG}") not in (None, d["ops"][k])]
    groups: dict[str, set] = {}
    for k, v in d["model"].items():
        name, phase, _, mode = k.split("/")
        groups.setdefault(f"{name}/{phase}/{mode}", set()).add(v)
    return bad + [k for k, v in groups.items() if len(v) != 1]


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--out")
    p.add_argument("--model", choices=["small", "llama3_8b"])
    p.add_argument("--quant", action="store_true", help="4-bit group-64 weights for the decoder")
    p.add_argument("--batches", nargs="+", type=int, default=[1, 4, 16, 64])
    p.add_argument("--prompt-len", type=int, default=64)
    p.add_argument("--compare", nargs=2)
    a = p.parse_args(argv)
    if a.compare:
        return compare(json.load(open(a.compare[0])), json.load(open(a.compare[1])))
    if not a.out:
        p.error("--out or --compare is required")
    d = dump(a.model, a.quant, a.batches, a.prompt_len)
    rc = 0
    if d is not None:
        bad = self_check(d)
        d["self_check"] = "ok" if not bad else bad
        json.dump(d, open(a.out, "w"), indent=1)
        print(f"wrote {a.out}: {len(d['ops'])} op digests, {len(d['model'])} model digests, "
              f"batch invariance inside the manifest: {'ok' if not bad else 'FAILED for ' + ', '.join(bad)}")
        rc = 1 if bad else 0
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        sys.stdout.flush()
        os._exit(rc)
    return rc


if __name__ == "__main__":
    sys.exit(main())
