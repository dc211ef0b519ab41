"""Batch-invariant kernels for NVIDIA B200 behind the mlx_batch_invariant API.

    import mlx_batch_invariant_b200 as bi
    with bi.set_batch_invariant_mode():
        logits = model(tokens)          # same bits at batch 1 and batch 256
    print(bi.stats())                   # which ops were handled / fell back

The public names are those of the reference package (mlx_batch_invariant/__init__.py:20-32).
"""

from ._mode import is_batch_invariant_mode_enabled, set_batch_invariant_mode
from .ops import reset_stats, stats
from .kernels import (
    batch_invariant_attention,
    batch_invariant_decode_attention,
    batch_invariant_prefill_attention,
    batch_invariant_matmul,
    batch_invariant_quantized_matmul,
    batch_invariant_rms_norm,
)
from .kernels import batch_invariant_paged_decode_attention  # extension (paged KV cache)
from .kernels import batch_invariant_layer_norm  # extension (the reference's roadmap item); __all__ stays the reference's
from ._lib import KernelError, check_device_status

__all__ = [
    "set_batch_invariant_mode",
    "is_batch_invariant_mode_enabled",
    "stats",
    "reset_stats",
    "batch_invariant_matmul",
    "batch_invariant_rms_norm",
    "batch_invariant_quantized_matmul",
    "batch_invariant_decode_attention",
    "batch_invariant_prefill_attention",
    "batch_invariant_attention",
]
__version__ = "0.1.0"
