"""The parts of bench.py that run without a GPU: the byte accounting of a decode step, the bit digest, the probe
prompts, and the reference arm's line for a workload it has no arm for."""

import importlib.util
import json
import subprocess
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_bytes_of_a_decode_step_count_every_weight_once_and_the_replicated_projection_per_gpu():
    b = _bench()
    from mlx_batch_invariant_b200.runner import LLAMA3_8B as cfg
    D = cfg.head_dim
    weights = cfg.n_layers * ((cfg.n_heads + 2 * cfg.n_kv_heads) * D * cfg.d_model + cfg.d_model * cfg.n_heads * D
                              + 3 * cfg.ffn * cfg.d_model) + cfg.vocab * cfg.d_model
    kv = cfg.n_layers * 2 * cfg.n_kv_heads * D * 2 * 560 * 64
    assert b._model_bytes_per_step(cfg, None, 64, 560, 1) == weights * 2.0 + kv
    o_proj = cfg.n_layers * cfg.d_model * cfg.n_heads * D
    two = b._model_bytes_per_step(cfg, None, 64, 560, 2)
    assert two == ((weights - o_proj) / 2 + o_proj) * 2.0 + kv / 2          # the output projection is not sharded
    q4 = b._model_bytes_per_step(cfg, (4, 64), 64, 560, 1)
    assert q4 == weights * (0.5 + 4 / 64) + kv


def test_digest_is_of_the_raw_bits():
    b = _bench()
    x = torch.tensor([1.0, -0.0, 3.5], dtype=torch.bfloat16)
    y = torch.tensor([1.0, 0.0, 3.5], dtype=torch.bfloat16)
    assert b._hash8(x) == b._hash8(x.clone()) and len(b._hash8(x)) == 16
    assert b._hash8(x) != b._hash8(y)                                         # -0.0 and 0.0 differ in bits


def test_row_zero_is_the_same_probe_prompt_at_every_batch_size():
    b = _bench()
    from mlx_batch_invariant_b200.runner import LLAMA3_8B as cfg
    p1, p4, p64 = (b._model_prompts(torch, cfg, B, 32) for B in (1, 4, 64))
    assert torch.equal(p1[0], p4[0]) and torch.equal(p1[0], p64[0])
    assert not torch.equal(p4[1], p64[1])


def test_reference_arm_without_an_arm_prints_the_unavailable_line():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "rms_norm", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-500:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line
