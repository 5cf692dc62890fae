"""Multi-GPU execution: peer-mapped memory, tensor parallelism, expert parallelism."""
