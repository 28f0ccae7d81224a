"""CPU oracle, workload generators, timing and profiling helpers."""
