"""CPU oracle (test infrastructure).  Only the tests, the smoke run and the
CPU-baseline leg of the benchmark may import this package; the product path never does."""
