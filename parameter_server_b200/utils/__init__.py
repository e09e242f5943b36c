"""Utilities: status helpers, timers / NVTX ranges, metrics, config parsing."""
