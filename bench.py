"""Benchmark of the batch-invariant hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one pass of the workload over one batch of seeded synthetic input.
Prints ONE JSON line (rank 0). Workloads:

    llama3_8b_decode   Llama-3-8B-architecture decoder, random init, bf16, batch 64 (--batch 1/4/16/64), 512-token
                       prompts: one step = one greedy decode step of all sequences          -> tok/s (default)
                       sharded column/head-parallel over --gpus N with all-gather (strong scaling). The line
                       also carries `row0_logits_hash` / `tokens_hash` (row 0 is the same probe prompt at every
                       batch size and GPU count: the digests must not change) and, at one GPU, an `ops` block
                       with the op-level components of the metric measured in the same run.
    llama3_8b_decode_q4  the same with 4-bit group-64 weights
    matmul_bf16_m256   dense y = x @ W^T, x[256,4096], W[4096,4096], bf16     -> TFLOP/s
    qmm4_decode        4-bit group-64 quantized matmul, M=1, K=4096 -> N=14336  -> GB/s
    attn_decode        decode attention, bf16, 32/8 heads, D=128, B=64, L=4096  -> GB/s
    attn_decode_short  the same at the decoder workload's shape: 560 keys in a 640-key cache -> GB/s
    rms_norm           RMSNorm [256,4096] bf16                                  -> GB/s

Timing: CUDA events on the launching stream, W >= 3 warm-up steps, inputs rotated over more
distinct buffers than fit in L2 so every step streams from HBM, max over ranks. `value` has
inputs resident in HBM; `e2e` goes through the public API from pinned host buffers and back.
With --gpus N > 1 the op-level workloads run as N independent replicas (no collective: the
op itself does not shard), value = sum over ranks / max time; the decoder workloads shard the
model (every linear by weight rows, attention by KV head) and join slices by all-gather (the library's
peer-memory gather, or NCCL: `config.collective` says which ran).
--impl reference times the CPU restatement of the reference algorithm (the oracle; the
reference itself is Metal-only and cannot run here) on the host cores: for the decoder, every step is
one whole decode step of one sequence (all layers, attention, lm_head).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

L2_BYTES = 126 * 1024 * 1024


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "which": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "which": "fallback"}


# ---------------------------------------------------------------------------------------------
# clocks
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                for n, val in zip(names, f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(n)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out["sm_mhz"] = statistics.median(sm)
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


# ---------------------------------------------------------------------------------------------
# workloads
class Workload:
    """step(i) runs the op on buffer set i % nbuf (device-resident inputs)."""
    name = metric = unit = dtype = ""
    bound = "hbm"
    launches_per_step = 1

    def flops(self): return 0.0
    def algo_bytes(self): return 0.0
    def config(self): return {}


class MatmulBF16(Workload):
    name, metric, unit, dtype = "matmul_bf16_m256", "bf16 TFLOP/s", "TFLOP/s", "bf16"
    M, N, K = 256, 4096, 4096

    def __init__(self, torch, bi, dev):
        self.torch, self.bi, self.dev = torch, bi, dev
        g = torch.Generator().manual_seed(0)
        wbytes = self.N * self.K * 2
        self.nbuf = L2_BYTES * 2 // wbytes + 1           # > 2x L2 of distinct weights
        self.W = [(torch.randn(self.N, self.K, generator=g) / 64).to(torch.bfloat16).to(dev) for _ in range(self.nbuf)]
        self.x_host = torch.randn(self.M, self.K, generator=g).to(torch.bfloat16).pin_memory()
        self.x = self.x_host.to(dev)
        self.y_host = torch.empty(self.M, self.N, dtype=torch.bfloat16).pin_memory()
        self.launches_per_step = 1                        # M = 256 folds in place (64-row batch tiles)

    def step(self, i):
        return self.bi.batch_invariant_matmul(self.x, self.W[i % self.nbuf].T)

    def step_e2e(self, i):
        x = self.x_host.to(self.dev, non_blocking=True)
        y = self.bi.batch_invariant_matmul(x, self.W[i % self.nbuf].T)
        self.y_host.copy_(y, non_blocking=True)
        return self.x_host.numel() * 2, self.y_host.numel() * 2

    def value(self, sec): return self.flops() / sec / 1e12
    def flops(self): return 2.0 * self.M * self.N * self.K
    def algo_bytes(self): return 2.0 * (self.M * self.K + self.K * self.N + self.M * self.N)
    def config(self):
        return {"workload": self.name, "M": self.M, "N": self.N, "K": self.K,
                "l2": f"{self.nbuf} weight buffers rotated ({self.nbuf * self.N * self.K * 2 >> 20} MiB > L2)"}

    def cpu_sample(self, R, threads):
        """Oracle (CUDA-core order of the same K-group algorithm) on the first rows of the workload."""
        torch = self.torch
        rows = 16
        a = self.x_host[:rows].clone()
        b = self.W[0].cpu().T.contiguous()
        t0 = time.perf_counter()
        R.matmul_f32order(a, b)
        dt = time.perf_counter() - t0
        return 2.0 * rows * self.N * self.K / dt / 1e12, f"first {rows} of {self.M} rows, all {self.N} columns, {dt:.1f} s"


class MatmulBF16M1(MatmulBF16):
    name, M = "matmul_bf16_m1", 1

    def __init__(self, torch, bi, dev):
        super().__init__(torch, bi, dev)
        self.launches_per_step = 2                        # split kernel + combine


class MatmulBF16M64(MatmulBF16M1):
    name, M = "matmul_bf16_m64", 64


class QMM4Decode(Workload):
    name, metric, unit, dtype = "qmm4_decode", "4-bit decode HBM GB/s", "GB/s", "bf16"
    M, N, K, gs, bits = 1, 14336, 4096, 64, 4

    def __init__(self, torch, bi, dev):
        from mlx_batch_invariant_b200.runner.decoder import quantize_rows
        self.torch, self.bi, self.dev = torch, bi, dev
        g = torch.Generator().manual_seed(0)
        W = (torch.randn(self.N, self.K, generator=g) * 0.02).to(torch.bfloat16)
        p, s, b = quantize_rows(W.to(dev), self.gs, self.bits)
        wbytes = p.numel() * 4
        self.nbuf = L2_BYTES * 2 // wbytes + 1
        self.p = [p.to(dev).clone() for _ in range(self.nbuf)]
        self.s = [s.to(dev).clone() for _ in range(self.nbuf)]
        self.b = [b.to(dev).clone() for _ in range(self.nbuf)]
        self.x_host = torch.randn(self.M, self.K, generator=g).to(torch.bfloat16).pin_memory()
        self.x = self.x_host.to(dev)
        self.y_host = torch.empty(self.M, self.N, dtype=torch.bfloat16).pin_memory()
        self.launches_per_step = 2                        # split kernel + combine

    def step(self, i):
        j = i % self.nbuf
        return self.bi.batch_invariant_quantized_matmul(self.x, self.p[j], self.s[j], self.b[j], group_size=self.gs, bits=self.bits)

    def step_e2e(self, i):
        j = i % self.nbuf
        x = self.x_host.to(self.dev, non_blocking=True)
        y = self.bi.batch_invariant_quantized_matmul(x, self.p[j], self.s[j], self.b[j], group_size=self.gs, bits=self.bits)
        self.y_host.copy_(y, non_blocking=True)
        return self.x_host.numel() * 2, self.y_host.numel() * 2

    def value(self, sec): return self.algo_bytes() / sec / 1e9
    def flops(self): return 2.0 * self.M * self.N * self.K
    def algo_bytes(self): return self.N * self.K * (self.bits / 8 + 4 / self.gs) + 2.0 * self.M * (self.K + self.N)
    def config(self):
        return {"workload": self.name, "M": self.M, "N": self.N, "K": self.K, "bits": self.bits, "group_size": self.gs,
                "l2": f"{self.nbuf} packed-weight buffers rotated"}

    def cpu_sample(self, R, threads):
        torch = self.torch
        rows = 1024
        p, s, b = self.p[0][:rows].cpu(), self.s[0][:rows].cpu(), self.b[0][:rows].cpu()
        t0 = time.perf_counter()
        wd = R.dequant(p, s, b, group_size=self.gs, bits=self.bits, dtype=torch.bfloat16)
        R.matmul_f32order(self.x_host.clone(), wd.T.contiguous())
        dt = time.perf_counter() - t0
        byts = rows * self.K * (self.bits / 8 + 4 / self.gs)
        return byts / dt / 1e9, f"first {rows} of {self.N} weight rows, {dt:.1f} s"


class AttnDecode(Workload):
    name, metric, unit, dtype = "attn_decode", "decode attention HBM GB/s", "GB/s", "bf16"
    B, Hq, Hkv, L, D = 64, 32, 8, 4096, 128

    def __init__(self, torch, bi, dev):
        self.torch, self.bi, self.dev = torch, bi, dev
        g = torch.Generator(device=dev).manual_seed(0)
        self.nbuf = 2                                       # 2 x 537 MB of K/V >> L2
        self.k = [torch.randn(self.B, self.Hkv, self.L, self.D, generator=g, device=dev, dtype=torch.bfloat16) for _ in range(self.nbuf)]
        self.v = [torch.randn(self.B, self.Hkv, self.L, self.D, generator=g, device=dev, dtype=torch.bfloat16) for _ in range(self.nbuf)]
        self.q_host = torch.randn(self.B, self.Hq, 1, self.D).to(torch.bfloat16).pin_memory()
        self.q = self.q_host.to(dev)
        self.o_host = torch.empty_like(self.q_host).pin_memory()
        self.launches_per_step = 2

    def step(self, i):
        j = i % self.nbuf
        return self.bi.batch_invariant_decode_attention(self.q, self.k[j], self.v[j], scale=self.D ** -0.5)

    def step_e2e(self, i):
        j = i % self.nbuf
        q = self.q_host.to(self.dev, non_blocking=True)
        o = self.bi.batch_invariant_decode_attention(q, self.k[j], self.v[j], scale=self.D ** -0.5)
        self.o_host.copy_(o, non_blocking=True)
        return self.q_host.numel() * 2, self.o_host.numel() * 2

    def value(self, sec): return self.algo_bytes() / sec / 1e9
    def flops(self): return 4.0 * self.B * self.Hq * self.L * self.D
    def algo_bytes(self): return self.B * (2.0 * self.Hkv * self.L * self.D * 2 + 2.0 * self.Hq * self.D * 2)
    def config(self):
        return {"workload": self.name, "B": self.B, "Hq": self.Hq, "Hkv": self.Hkv, "L": self.L, "D": self.D,
                "l2": "two K/V sets of 537 MB alternated"}

    def cpu_sample(self, R, threads):
        nb = 1
        q, k, v = self.q_host[:nb].clone(), self.k[0][:nb].cpu(), self.v[0][:nb].cpu()
        t0 = time.perf_counter()
        R.attn_decode(q, k, v, scale=self.D ** -0.5)
        dt = time.perf_counter() - t0
        return nb * (2.0 * self.Hkv * self.L * self.D * 2) / dt / 1e9, f"{nb} of {self.B} sequences, {dt:.1f} s"


class AttnDecodeShort(AttnDecode):
    """Decode attention at the shape of the decoder workload: 64 sequences of 560 keys in a 640-key cache."""
    name, metric = "attn_decode_short", "decode attention HBM GB/s"
    L, KEYS = 640, 560

    def __init__(self, torch, bi, dev):
        super().__init__(torch, bi, dev)
        self.nbuf = 4                                       # 4 x 168 MB of K/V > L2
        g = torch.Generator(device=dev).manual_seed(1)
        while len(self.k) < self.nbuf:
            self.k.append(torch.randn(self.B, self.Hkv, self.L, self.D, generator=g, device=dev, dtype=torch.bfloat16))
            self.v.append(torch.randn(self.B, self.Hkv, self.L, self.D, generator=g, device=dev, dtype=torch.bfloat16))
        self.lens = torch.full((self.B,), self.KEYS, dtype=torch.int32, device=dev)

    def step(self, i):
        j = i % self.nbuf
        return self.bi.batch_invariant_decode_attention(self.q, self.k[j], self.v[j], scale=self.D ** -0.5, kv_lens=self.lens)

    def step_e2e(self, i):
        j = i % self.nbuf
        q = self.q_host.to(self.dev, non_blocking=True)
        o = self.bi.batch_invariant_decode_attention(q, self.k[j], self.v[j], scale=self.D ** -0.5, kv_lens=self.lens)
        self.o_host.copy_(o, non_blocking=True)
        return self.q_host.numel() * 2, self.o_host.numel() * 2

    def algo_bytes(self): return self.B * (2.0 * self.Hkv * self.KEYS * self.D * 2 + 2.0 * self.Hq * self.D * 2)
    def config(self):
        return {"workload": self.name, "B": self.B, "Hq": self.Hq, "Hkv": self.Hkv, "L": self.L, "keys": self.KEYS, "D": self.D,
                "l2": "four K/V sets of 168 MB rotated"}

    def cpu_sample(self, R, threads):
        q, k, v = self.q_host[:1].clone(), self.k[0][:1, :, :self.KEYS].cpu().contiguous(), self.v[0][:1, :, :self.KEYS].cpu().contiguous()
        t0 = time.perf_counter()
        R.attn_decode(q, k, v, scale=self.D ** -0.5)
        dt = time.perf_counter() - t0
        return (2.0 * self.Hkv * self.KEYS * self.D * 2) / dt / 1e9, f"1 of {self.B} sequences, {dt:.1f} s"


class RMSNormW(Workload):
    name, metric, unit, dtype = "rms_norm", "RMSNorm HBM GB/s", "GB/s", "bf16"
    M, D = 256, 4096

    def __init__(self, torch, bi, dev):
        self.torch, self.bi, self.dev = torch, bi, dev
        g = torch.Generator().manual_seed(0)
        self.nbuf = L2_BYTES * 2 // (self.M * self.D * 2) + 1
        self.x_host = (3 * torch.randn(self.M, self.D, generator=g)).to(torch.bfloat16).pin_memory()
        self.x = [self.x_host.to(dev).clone() for _ in range(self.nbuf)]
        self.w = (1 + 0.1 * torch.randn(self.D, generator=g)).to(torch.bfloat16).to(dev)
        self.y_host = torch.empty_like(self.x_host).pin_memory()

    def step(self, i):
        return self.bi.batch_invariant_rms_norm(self.x[i % self.nbuf], self.w, 1e-5)

    def step_e2e(self, i):
        x = self.x_host.to(self.dev, non_blocking=True)
        y = self.bi.batch_invariant_rms_norm(x, self.w, 1e-5)
        self.y_host.copy_(y, non_blocking=True)
        return self.x_host.numel() * 2, self.y_host.numel() * 2

    def value(self, sec): return self.algo_bytes() / sec / 1e9
    def flops(self): return 4.0 * self.M * self.D
    def algo_bytes(self): return 2.0 * (2 * self.M * self.D + self.D)
    def config(self): return {"workload": self.name, "M": self.M, "D": self.D, "l2": f"{self.nbuf} input buffers rotated"}

    def cpu_sample(self, R, threads):
        reps = 200
        x, w = self.x_host.clone(), self.w.cpu()
        t0 = time.perf_counter()
        for _ in range(reps):
            R.rms_norm(x, w, 1e-5)
        dt = (time.perf_counter() - t0) / reps
        return self.algo_bytes() / dt / 1e9, f"whole [{self.M},{self.D}] input, mean of {reps} passes"


# DRAM bytes (read + write) of one launch of the workload's dominant kernel, from `ncu --set full` captures of
# these workloads on a B200 (dram__bytes_read.sum + dram__bytes_write.sum); None where no capture exists.
NCU_TRAFFIC_BYTES = {
    "matmul_bf16_m64": 34.17e6, "matmul_bf16_m256": 47.3e6, "qmm4_decode": 33.13e6, "attn_decode": 1.0887e9,
}

WORKLOADS = {c.name: c for c in (MatmulBF16, MatmulBF16M1, MatmulBF16M64, QMM4Decode, AttnDecode, AttnDecodeShort, RMSNormW)}


# ---------------------------------------------------------------------------------------------
def timed_region(torch, fn, steps, barrier):
    """K steps between two events on the current stream; barrier + synchronize on both sides."""
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return e0.elapsed_time(e1) / 1e3


def run_ours(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the library has no CPU path)")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    barrier = (lambda: dist.barrier()) if dist else (lambda: None)

    import mlx_batch_invariant_b200 as bi
    from mlx_batch_invariant_b200 import _lib
    _lib.load()                                            # fail loudly if the CUDA library is missing
    wl_cls = WORKLOADS[args.workload]
    if args.shape:                                         # matmul workloads at another weight shape (config says which)
        n, k = (int(v) for v in args.shape.split(","))
        if not hasattr(wl_cls, "N"):
            raise SystemExit(f"--shape applies to the matmul workloads, not to {args.workload}")
        wl_cls = type(wl_cls.__name__, (wl_cls,), {"N": n, "K": k})
    wl = wl_cls(torch, bi, dev)

    for i in range(max(args.warmup, 3)):
        wl.step(i)
    torch.cuda.synchronize()
    # `value`: the op as a serving loop would issue it -- the K timed steps captured in one CUDA graph
    # (step i works on buffer set i % nbuf, so consecutive steps never find their inputs in L2) and
    # replayed once, so the timed region holds the kernels and neither Python call overhead (that is
    # what `e2e` shows) nor one graph launch per step.
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(args.steps):
            wl.step(i)
    graph.replay()                                         # warm-up: the whole step sequence once (>= W steps)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    sec = timed_region(torch, lambda i: graph.replay(), 1, barrier)
    # end to end: pinned host input -> device -> op -> host result, every step
    for i in range(3):
        wl.step_e2e(i)
    h2d = d2h = 0
    def e2e_step(i):
        nonlocal h2d, d2h
        h2d, d2h = wl.step_e2e(i)
    sec_e2e = timed_region(torch, e2e_step, args.steps, barrier)
    clocks = sampler.stop() if rank == 0 else {}
    bi.check_device_status(dev)

    if dist:
        t = torch.tensor([sec, sec_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec, sec_e2e = float(t[0]), float(t[1])
    per = sec / args.steps
    per_e2e = sec_e2e / args.steps
    if rank == 0:
        pk = peaks()
        if wl.bound == "hbm":
            achieved = wl.algo_bytes() / per / 1e9
            roof = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                    "frac": round(achieved / pk["hbm_gbs"], 4), "traffic": NCU_TRAFFIC_BYTES.get(wl.name),
                    "peak_source": f"of {pk['which']}"}
        else:
            achieved = wl.flops() / per / 1e12
            roof = {"bound": "tensor", "achieved": round(achieved, 1), "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": round(achieved / pk["bf16_tflops"], 4), "traffic": NCU_TRAFFIC_BYTES.get(wl.name),
                    "peak_source": f"of {pk['which']}"}
        from oracle import reference as R
        cores = os.cpu_count() or 1
        R.set_threads(cores)                                # a launcher may have pinned OMP_NUM_THREADS to 1
        cv, sample = wl.cpu_sample(R, cores)
        line = {
            "metric": wl.metric, "value": round(wl.value(per) * world, 3), "unit": wl.unit, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(per * 1e3, 5),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": dict(wl.config(), parallelism=("single GPU" if world == 1 else f"{world} independent replicas"),
                           launch="the K timed steps in one CUDA graph, buffer sets rotated inside"),
            "clocks": clocks,
            "e2e": {"value": round(wl.value(per_e2e) * world, 3), "unit": wl.unit, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": round(per_e2e * 1e3, 5)},
            "gpu_launches": wl.launches_per_step * args.steps,
            "roofline": roof,
            "cpu_baseline": {"value": round(cv, 6), "unit": wl.unit, "cores": cores, "kind": "port", "sample": sample},
        }
        print(json.dumps(line), flush=True)
    if dist:
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


# ---------------------------------------------------------------------------------------------
# whole-model workload
MODEL_B, MODEL_P = 64, 512


def _model_bytes_per_step(cfg, quant, B, kv_tokens, world=1):
    """Algorithmic bytes ONE GPU moves in a decode step: its shard of every sharded linear, the whole of the
    replicated output projection, its KV heads' cache (the embedding rows read are negligible)."""
    D = cfg.head_dim
    wb = 2.0 if quant is None else (quant[0] / 8 + 4 / quant[1])
    sharded = cfg.n_layers * ((cfg.n_heads * D + 2 * cfg.n_kv_heads * D) * cfg.d_model + 3 * cfg.ffn * cfg.d_model) + cfg.vocab * cfg.d_model
    replicated = cfg.n_layers * cfg.d_model * cfg.n_heads * D if world > 1 else 0
    if world == 1:
        sharded += cfg.n_layers * cfg.d_model * cfg.n_heads * D
    kv = cfg.n_layers * 2 * cfg.n_kv_heads * D * 2 * kv_tokens * B
    return (sharded / world + replicated) * wb + kv / world


def _cpu_decode_token(R, torch, cfg, keys):
    """One whole greedy decode step of ONE sequence through the oracle port: every layer's RMSNorms, four
    linears (CUDA-core order of the K-group algorithm), the split-KV attention over `keys` cached keys, and the
    lm_head. One layer's random weights are reused for all layers (the work is the same; 15 GB of distinct
    weights would take longer to draw than to use). Returns seconds."""
    g = torch.Generator().manual_seed(0)
    dt = torch.bfloat16
    D, d = cfg.head_dim, cfg.d_model
    mk = lambda n, k: (torch.randn(n, k, generator=g) * cfg.init_std).to(dt).T.contiguous()
    wqkv, wo = mk((cfg.n_heads + 2 * cfg.n_kv_heads) * D, d), mk(d, cfg.n_heads * D)
    wgu, wdown, head = mk(2 * cfg.ffn, d), mk(d, cfg.ffn), mk(cfg.vocab, d)
    nw = torch.ones(d, dtype=dt)
    kc = torch.randn(1, cfg.n_kv_heads, keys, D, generator=g).to(dt)
    vc = torch.randn(1, cfg.n_kv_heads, keys, D, generator=g).to(dt)
    x = torch.randn(1, d, generator=g).to(dt)
    t0 = time.perf_counter()
    for _ in range(cfg.n_layers):
        h = R.rms_norm(x, nw, cfg.eps)
        qkv = R.matmul_f32order(h, wqkv)
        q = qkv[:, :cfg.n_heads * D].reshape(1, cfg.n_heads, 1, D)
        a = R.attn_decode(q, kc, vc, scale=D ** -0.5)
        x = x + R.matmul_f32order(a.reshape(1, cfg.n_heads * D), wo)
        h = R.rms_norm(x, nw, cfg.eps)
        gu = R.matmul_f32order(h, wgu).float()
        act = (torch.nn.functional.silu(gu[:, :cfg.ffn]) * gu[:, cfg.ffn:]).to(dt)
        x = x + R.matmul_f32order(act, wdown)
    logits = R.matmul_f32order(R.rms_norm(x, nw, cfg.eps), head)
    int(logits.float().argmax())
    return time.perf_counter() - t0


def _cpu_tok_per_s(R, torch, cfg, keys=560):
    sec = _cpu_decode_token(R, torch, cfg, keys)
    return 1.0 / sec, (f"one whole decode step of 1 of the {MODEL_B} sequences ({cfg.n_layers} layers: norms, four linears, "
                       f"{keys}-key attention; lm_head), {sec:.1f} s of CPU work")


def _hash8(t):
    """blake2b-8 of a tensor's raw bits (the reference's harness/dump_bits.py:32-40 digest)."""
    import hashlib
    import torch
    raw = t.detach().contiguous().cpu()
    raw = raw.view(torch.int16) if raw.element_size() == 2 else (raw.view(torch.int32) if raw.element_size() == 4 else raw)
    return hashlib.blake2b(raw.numpy().tobytes(), digest_size=8).hexdigest()


def _model_prompts(torch, cfg, B, P):
    """Row 0 is the probe prompt (seed 0, the same for every batch size and GPU count); the other rows are
    fillers reseeded per (B, row), as the reference's model sweep builds its batches (harness/model_sweep.py:100-108)."""
    rows = [torch.randint(0, cfg.vocab, (P,), generator=torch.Generator().manual_seed(0))]
    for r in range(1, B):
        rows.append(torch.randint(0, cfg.vocab, (P,), generator=torch.Generator().manual_seed(1000 + 7 * B + r)))
    return torch.stack(rows, 0)


def _ops_block(torch, bi, dev, pk, steps=20):
    """The op-level components of the headline metric, measured in this same run (each a CUDA-graph replay of
    `steps` calls over rotated buffers): dense bf16 M=256 TFLOP/s beside cuBLAS, 4-bit decode GB/s, decode
    attention GB/s, each with its fraction of the measured peak."""
    out = {}
    def timed(wl, fn):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(steps):
                fn(i)
        g.replay()
        return timed_region(torch, lambda i: g.replay(), 1, lambda: None) / steps
    for cls in (MatmulBF16, QMM4Decode, AttnDecode):
        wl = cls(torch, bi, dev)
        per = timed(wl, wl.step)
        ent = {"value": round(wl.value(per), 1), "unit": wl.unit, "us": round(per * 1e6, 2)}
        if cls is MatmulBF16:
            lib_per = timed(wl, lambda i: torch.matmul(wl.x, wl.W[i % wl.nbuf].T))
            ent.update(frac=round(wl.value(per) / pk["bf16_tflops"], 4), frac_of="measured bf16 burst",
                       cublas_us=round(lib_per * 1e6, 2), vs_cublas=round(lib_per / per, 3))
        else:
            ent.update(frac=round(wl.value(per) / pk["hbm_gbs"], 4), frac_of="measured HBM copy")
        out[wl.name] = ent
        del wl
        torch.cuda.empty_cache()
    return out


def run_model(args, quant):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the library has no CPU path)")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    barrier = (lambda: dist.barrier()) if dist else (lambda: None)

    import mlx_batch_invariant_b200 as bi
    from mlx_batch_invariant_b200 import _lib
    from mlx_batch_invariant_b200.runner import LLAMA3_8B, GraphedDecoder, ShardedDecoder
    _lib.load()
    cfg = LLAMA3_8B
    B, P = args.batch, MODEL_P
    warm = max(args.warmup, 3)
    pk = peaks()
    # op-level components of the headline metric, in the same run (single GPU only: the ops do not shard)
    ops_block = _ops_block(torch, bi, dev, pk) if (world == 1 and not args.no_ops) else None
    total_steps = warm + args.steps * 2 + 8
    model = ShardedDecoder(cfg, rank=rank, world=world, device=dev, quant=quant, max_batch=B, max_len=P + total_steps + 1)
    prompts = _model_prompts(torch, cfg, B, P).to(dev)
    logits = model.forward(prompts, 0)
    # Bit evidence: row 0 is the same probe prompt at every batch size and GPU count, so these digests must be
    # the same in every run of this workload (prefill logits, then the logits and tokens of decode steps 1-3).
    row0_bits = [logits[0].clone()]
    row0_tokens = [logits[0].argmax().reshape(1).clone()]
    gd = GraphedDecoder(model, B)
    gd.start(logits.argmax(-1), P)
    lib = _lib.load()
    graphed = True
    c0 = lib.bi_launch_count()
    try:
        gd.capture()
        launches_per_step = (lib.bi_launch_count() - c0) // 2          # capture() runs the step twice: eagerly, then recorded
    except Exception as e:                                  # a step that cannot be captured still runs eagerly
        graphed = False
        gd.graph = None
        gd.start(logits.argmax(-1), P)
        launches_per_step = None
        if rank == 0:
            print(f"bench.py: CUDA-graph capture failed ({type(e).__name__}: {e}); timing eager steps", file=sys.stderr)
    for i in range(warm):
        c1 = lib.bi_launch_count()
        lg = gd.step()
        if launches_per_step is None:
            launches_per_step = lib.bi_launch_count() - c1
        if i < 3:
            row0_bits.append(lg[0].clone())
            row0_tokens.append(gd.tokens[0].reshape(1).clone())
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    sec = timed_region(torch, lambda i: gd.step(), args.steps, barrier)
    # end to end: this step's token ids from pinned host memory, next token ids back to the host, every step
    tok_host = torch.zeros(B, 1, dtype=torch.long).pin_memory()
    nxt_host = torch.zeros(B, 1, dtype=torch.long).pin_memory()
    nxt_host.copy_(gd.tokens)
    torch.cuda.synchronize()
    def e2e_step(i):
        tok_host.copy_(nxt_host)
        gd.tokens.copy_(tok_host, non_blocking=True)
        gd.step()
        nxt_host.copy_(gd.tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    sec_e2e = timed_region(torch, e2e_step, args.steps, barrier)
    clocks = sampler.stop() if rank == 0 else {}
    bi.check_device_status(dev)
    fallbacks = bi.stats()["fallbacks"]
    if dist:
        t = torch.tensor([sec, sec_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec, sec_e2e = float(t[0]), float(t[1])
    per, per_e2e = sec / args.steps, sec_e2e / args.steps
    if rank == 0:
        kv_tokens = P + warm + args.steps // 2
        bytes_step = _model_bytes_per_step(cfg, quant, B, kv_tokens, world)       # per GPU
        achieved = bytes_step / per / 1e9
        gather = "none (single GPU)"
        if world > 1:
            if model._pg is None:
                gather = "NCCL all_gather_into_tensor, 97 per step"
            elif model._fused_push():
                gather = ("peer-memory push over NVLink, 97 per step: 96 fused into the producing kernels (attention merge, "
                          "SwiGLU, down-projection fold) with the wait in the consumer, 1 stand-alone (logits)")
            else:
                gather = "peer-memory push all-gather (bi_push_gather), 97 per step"
        from oracle import reference as R
        cores = os.cpu_count() or 1
        R.set_threads(cores)                                # torchrun pins OMP_NUM_THREADS to 1; the baseline uses every core
        cv, sample = _cpu_tok_per_s(R, torch, cfg)
        name = "llama3_8b_decode" + ("" if quant is None else "_q4")
        line = {
            "metric": "model tok/s", "value": round(B / per, 1), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": round(per * 1e3, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16" if quant is None else "bf16 activations, 4-bit group-64 weights",
            "data": "synthetic",
            "config": {"workload": name, "architecture": "Llama-3-8B (32 layers, d 4096, 32/8 heads, head_dim 128, ffn 14336, vocab 128256), random init",
                       "global_batch": B, "prompt_len": P, "decode": "greedy, KV cache, CUDA graph replay" if graphed else "greedy, KV cache, eager",
                       "parallelism": "single GPU" if world == 1 else f"tp{world}: weight-row / KV-head shards, output projection replicated",
                       "collective": gather,
                       "l2": "15 GB of weights streamed per step (>> L2)"},
            "clocks": clocks,
            "e2e": {"value": round(B / per_e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * 8,
                    "ms_per_step": round(per_e2e * 1e3, 4)},
            "gpu_launches": int(launches_per_step or 0) * args.steps,
            "gpu_launches_per_step": int(launches_per_step or 0),
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4), "traffic": None,
                         "traffic_note": "no whole-step capture (a step is ~300 launches; ncu captures are kept to one kernel): "
                                         "per-kernel DRAM traffic is in profiles/ and in the op workloads' lines",
                         "peak_source": f"of {pk['which']}",
                         "kernel": "whole decode step per GPU: its weight shards + replicated output projection + its KV heads' cache, / step time"},
            "cpu_baseline": {"value": round(cv, 4), "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
            "fallbacks": fallbacks,
            "row0_logits_hash": _hash8(torch.stack(row0_bits, 0)),
            "tokens_hash": _hash8(torch.cat(row0_tokens, 0)),
            "hash_of": "row 0 (the probe prompt): logits of the prefill and of decode steps 1-3; its first 4 greedy tokens",
        }
        if ops_block is not None:
            line["ops"] = ops_block
        print(json.dumps(line), flush=True)
    _shutdown(torch, dist, [gd])


def _shutdown(torch, dist, holders):
    """Leave a multi-rank run without hanging: drop CUDA graphs that captured NCCL kernels, meet at a
    barrier, then exit the process directly (tearing the NCCL communicator down while graphs that used
    it were alive has been seen to block in the watchdog)."""
    for h in holders:
        h.graph = None
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def run_reference(args):
    """The reference's algorithm on the host cores. The reference itself is Metal source strings
    behind MLX and cannot execute off an Apple GPU, so this arm times the CPU restatement."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)      # torchrun pins it to 1; the baseline uses every core
    import torch
    from oracle import reference as R
    cores = os.cpu_count() or 1

    class _NoDev:                                          # build the workload's host-side inputs only
        pass
    # CPU-only construction of the same seeded inputs
    R.set_threads(cores)
    if args.workload.startswith("llama3_8b_decode"):
        from mlx_batch_invariant_b200.runner import LLAMA3_8B
        vals = []
        sample = ""
        for i in range(args.warmup + args.steps):
            v, sample = _cpu_tok_per_s(R, torch, LLAMA3_8B)             # every step really runs one whole token
            if i >= args.warmup:
                vals.append(v)
        v = statistics.mean(vals)
        line = {"impl": "reference", "metric": "model tok/s", "value": round(v, 4), "unit": "tok/s",
                "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(1e3 / v, 1),
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": args.workload, "global_batch": MODEL_B, "prompt_len": MODEL_P,
                           "note": "the reference is Metal-only; this arm is its algorithm restated in C (oracle port) on the host cores, "
                                   "one sequence per step (a bounded sample of the 64-sequence step)"},
                "cpu_baseline": {"value": round(v, 4), "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
                "e2e": {"value": round(v, 4), "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return
    wl_cls = WORKLOADS[args.workload]
    vals = []
    sample = ""
    g = torch.Generator().manual_seed(0)
    if wl_cls is MatmulBF16:
        W = (torch.randn(wl_cls.N, wl_cls.K, generator=g) / 64).to(torch.bfloat16)
        x = torch.randn(wl_cls.M, wl_cls.K, generator=g).to(torch.bfloat16)
        rows = 16
        b = W.T.contiguous()
        for i in range(args.warmup + args.steps):
            t0 = time.perf_counter()
            R.matmul_f32order(x[:rows].clone(), b)
            dt = time.perf_counter() - t0
            if i >= args.warmup:
                vals.append(2.0 * rows * wl_cls.N * wl_cls.K / dt / 1e12)
        sample = f"first {rows} of {wl_cls.M} rows per step"
        cfg = {"workload": wl_cls.name, "M": wl_cls.M, "N": wl_cls.N, "K": wl_cls.K}
    else:
        # the contract's fallback line: this workload's CPU leg is its `cpu_baseline` only
        print(json.dumps({"impl": "reference", "unavailable": f"no reference arm for workload {args.workload}: its CPU "
                                                              f"restatement is timed as cpu_baseline in the default arm"}))
        return
    v = statistics.mean(vals)
    line = {"impl": "reference", "metric": wl_cls.metric, "value": round(v, 6), "unit": wl_cls.unit,
            "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl_cls.dtype,
            "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": round(v, 6), "unit": wl_cls.unit, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": round(v, 6), "unit": wl_cls.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--workload", default="llama3_8b_decode", choices=["llama3_8b_decode", "llama3_8b_decode_q4"] + list(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=MODEL_B, choices=[1, 4, 16, 64], help="decoder workloads: sequences per step")
    ap.add_argument("--shape", default=None, metavar="N,K", help="matmul workloads: weight rows and row length instead of the workload's own")
    ap.add_argument("--no-ops", action="store_true", help="decoder workloads: skip the op-level block of the line")
    args = ap.parse_args()
    model = args.workload.startswith("llama3_8b_decode")
    if args.steps is None:
        args.steps = 64 if model else 200
    if args.warmup is None:
        args.warmup = 5 if model else 10
    if args.impl == "reference":
        if args.steps > 3 and model:
            args.steps, args.warmup = min(args.steps, 3), min(args.warmup, 1)     # each CPU step is seconds long
        run_reference(args)
    elif model:
        run_model(args, (4, 64) if args.workload.endswith("_q4") else None)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
