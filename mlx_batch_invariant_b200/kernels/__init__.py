"""Batch-invariant kernels for B200 (host wrappers over the C ABI).

One rule, as in the reference (mlx_batch_invariant/kernels/__init__.py:3-10): the
floating-point reduction order of an output element never depends on how many
other rows or sequences share the launch.
"""

from .matmul import batch_invariant_matmul
from .rmsnorm import batch_invariant_rms_norm
from .layernorm import batch_invariant_layer_norm  # beyond the reference's six kernels: not in __all__
from .quantized import batch_invariant_quantized_matmul
from .attention import batch_invariant_paged_decode_attention  # beyond the reference's six kernels: not in __all__
from .attention import (
    batch_invariant_attention,
    batch_invariant_decode_attention,
    batch_invariant_prefill_attention,
)

__all__ = [
    "batch_invariant_matmul",
    "batch_invariant_rms_norm",
    "batch_invariant_quantized_matmul",
    "batch_invariant_decode_attention",
    "batch_invariant_prefill_attention",
    "batch_invariant_attention",
]
