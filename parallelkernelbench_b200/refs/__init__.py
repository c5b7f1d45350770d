"""PyTorch + NCCL (+cuBLAS) reference implementations: the correctness oracle and the timed baseline."""
