"""CPU oracle for the batch-invariant hot path. Test infrastructure only: nothing in
mlx_batch_invariant_b200 imports this package."""
