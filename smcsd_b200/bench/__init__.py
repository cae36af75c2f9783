"""User-facing harnesses: offline throughput, sweeps, GSM8K accuracy (offline and HTTP), quality check, profiler."""
