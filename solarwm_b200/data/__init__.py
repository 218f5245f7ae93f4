"""Data plane: index rows, deterministic sample plans, tar shard reader, camera conventions,
shard transport / prefetch, synthetic sources for benchmarks."""
