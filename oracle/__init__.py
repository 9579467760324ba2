"""CPU oracle for the GGUF quantised-matmul path.  Test infrastructure only: tests, the smoke
check and the benchmark's CPU-baseline legs import it; the CUDA product path never does."""
