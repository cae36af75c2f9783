"""Debug records, profiling helpers and synthetic workload generators."""
