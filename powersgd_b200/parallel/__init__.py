"""Multi-GPU plumbing: symmetric memory, in-kernel collective channels, collective benchmarks."""
