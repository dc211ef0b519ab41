"""Decoder runner: the whole-model caller of the batch-invariant ops (Llama-3 architecture,
random init), single GPU or sharded over 2/4/8 GPUs along reduction-free dimensions only."""

from .decoder import DecoderConfig, GraphedDecoder, KernelBackend, ShardedDecoder, LLAMA3_8B, greedy_generate

__all__ = ["DecoderConfig", "GraphedDecoder", "KernelBackend", "ShardedDecoder", "LLAMA3_8B", "greedy_generate"]
