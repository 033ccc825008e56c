"""CPU oracle of the sparse-aggregation path.  Test infrastructure: only tests/,
the smoke check and the CPU-baseline leg of bench.py may import this package."""
