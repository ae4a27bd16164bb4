"""TEST INFRASTRUCTURE ONLY: CPU checker for the CUDA MatMulNBits path. Imported by tests,
the smoke check and the CPU-baseline leg of the benchmark; never by the product path."""
