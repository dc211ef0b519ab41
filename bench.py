"""Benchmark of the batch-invariant hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one pass of the workload's op over one batch of seeded synthetic input.
Prints ONE JSON line (rank 0). Workloads:

    matmul_bf16_m256   dense y = x @ W^T, x[256,4096], W[4096,4096], bf16     -> TFLOP/s   (default)
    qmm4_decode        4-bit group-64 quantized matmul, M=1, K=4096 -> N=14336  -> GB/s
    attn_decode        decode attention, bf16, 32/8 heads, D=128, B=64, L=4096  -> GB/s
    rms_norm           RMSNorm [256,4096] bf16                                  -> GB/s

Timing: CUDA events on the launching stream, W >= 3 warm-up steps, inputs rotated over more
distinct buffers than fit in L2 so every step streams from HBM, max over ranks. `value` has
inputs resident in HBM; `e2e` goes through the public API from pinned host buffers and back.
With --gpus N > 1 the op-level workloads run as N independent replicas (no collective: the
op itself does not shard), value = sum over ranks / max time.
--impl reference times the CPU restatement of the reference algorithm (the oracle; the
reference itself is Metal-only and cannot run here) on the host cores.
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
        self.launches_per_step = 1                        # fused path at M=256

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
        from oracle.reference import quantize_affine
        self.torch, self.bi, self.dev = torch, bi, dev
        g = torch.Generator().manual_seed(0)
        W = torch.randn(self.N, self.K, generator=g) * 0.02
        p, s, b = quantize_affine(W, group_size=self.gs, bits=self.bits, dtype=torch.bfloat16)
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


WORKLOADS = {c.name: c for c in (MatmulBF16, MatmulBF16M1, MatmulBF16M64, QMM4Decode, AttnDecode, RMSNormW)}


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
    wl = WORKLOADS[args.workload](torch, bi, dev)

    for i in range(max(args.warmup, 3)):
        wl.step(i)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    sec = timed_region(torch, wl.step, args.steps, barrier)
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
                    "frac": round(achieved / pk["hbm_gbs"], 4), "traffic": None, "peak_source": f"of {pk['which']}"}
        else:
            achieved = wl.flops() / per / 1e12
            roof = {"bound": "tensor", "achieved": round(achieved, 1), "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": round(achieved / pk["bf16_tflops"], 4), "traffic": None, "peak_source": f"of {pk['which']}"}
        from oracle import reference as R
        cores = os.cpu_count() or 1
        cv, sample = wl.cpu_sample(R, cores) if world == 1 or True else (None, "")
        line = {
            "metric": wl.metric, "value": round(wl.value(per) * world, 3), "unit": wl.unit, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(per * 1e3, 5),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": dict(wl.config(), parallelism=("single GPU" if world == 1 else f"{world} independent replicas")),
            "clocks": clocks,
            "e2e": {"value": round(wl.value(per_e2e) * world, 3), "unit": wl.unit, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": round(per_e2e * 1e3, 5)},
            "gpu_launches": wl.launches_per_step * args.steps,
            "roofline": roof,
            "cpu_baseline": {"value": round(cv, 6), "unit": wl.unit, "cores": cores, "kind": "port", "sample": sample},
        }
        print(json.dumps(line), flush=True)
    if dist:
        dist.destroy_process_group()


def run_reference(args):
    """The reference's algorithm on the host cores. The reference itself is Metal source strings
    behind MLX and cannot execute off an Apple GPU, so this arm times the CPU restatement."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from oracle import reference as R
    cores = os.cpu_count() or 1

    class _NoDev:                                          # build the workload's host-side inputs only
        pass
    # CPU-only construction of the same seeded inputs
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
        raise SystemExit(f"--impl reference: workload {args.workload} not wired")
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
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="matmul_bf16_m256", choices=list(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
