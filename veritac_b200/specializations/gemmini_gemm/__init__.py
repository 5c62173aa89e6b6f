"""gemmini_gemm specialization (B200 back end); implementations are loaded explicitly."""
