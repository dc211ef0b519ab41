"""The bit-hash manifest tool (the counterpart of the reference's harness/dump_bits.py): comparing and
self-checking manifests needs no GPU; producing one does."""

import json

import pytest
import torch

from mlx_batch_invariant_b200 import dump_bits as D


def _manifest(**over):
    d = {"library": 100, "torch": "x", "cuda": "y", "device": "gpu", "gpus": 1,
         "ops": {"matmul/bf16/stock": "aa", "matmul/bf16/inv": "bb", "matmul/bf16/inv@B64": "bb"},
         "model": {"small/prefill/B1/inv": "cc", "small/prefill/B4/inv": "cc", "small/decode/B1/inv": "dd",
                   "small/decode/B4/inv": "dd"}}
    d.update(over)
    return d


def test_compare_and_self_check(capsys):
    a, b = _manifest(), _manifest()
    assert D.self_check(a) == []
    assert D.compare(a, b) == 0
    b["ops"]["matmul/bf16/stock"] = "zz"                       # the stock op may differ between builds: reported, not an error
    assert D.compare(a, b) == 0
    assert "differing: matmul/bf16/stock" in capsys.readouterr().out
    b["model"]["small/decode/B4/inv"] = "ee"
    assert D.compare(a, b) == 1
    assert D.self_check(b) == ["small/decode/inv"]
    c = _manifest()
    c["ops"]["matmul/bf16/inv@B64"] = "qq"
    assert D.self_check(c) == ["matmul/bf16/inv"]


def test_digest_is_blake2b_8_of_the_raw_bits():
    import hashlib
    t = torch.tensor([1.0, -2.5], dtype=torch.bfloat16)
    assert D.digest(t) == hashlib.blake2b(t.view(torch.int16).numpy().tobytes(), digest_size=8).hexdigest()
    assert D.digest(t) != D.digest(t.float())


@pytest.mark.gpu
def test_dump_twice_identical_and_internally_invariant(tmp_path):
    """Two dumps in a row agree digest for digest (run-to-run reproducibility, the check of the reference's
    harness/generate_bench.py:24-33), every op's batch-64 probe equals its batch-1 probe, and the small decoder
    gives one digest at batch 1, 4, 16 and 64, dense and 4-bit; nothing fell back."""
    outs = []
    for i, quant in enumerate((False, False, True)):
        path = tmp_path / f"bits{i}.json"
        assert D.main(["--out", str(path), "--model", "small"] + (["--quant"] if quant else [])) == 0
        outs.append(json.load(open(path)))
    a, b, q = outs
    assert a["self_check"] == "ok" and q["self_check"] == "ok"
    assert a["fallbacks"] == {} and q["fallbacks"] == {}
    assert len(a["ops"]) == 6 * 3 * 3 and len(a["model"]) == 8
    assert D.compare(a, b) == 0 and a["ops"] == b["ops"] and a["model"] == b["model"]
    assert set(q["model"]) != set(a["model"])
