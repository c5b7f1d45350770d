"""parallelkernelbench_b200: Blackwell-native fused communication + compute kernels and the harness
that evaluates them (per-rank output compare against PyTorch+NCCL references, device timing as the
max over ranks, roofline fractions).

Sub-packages
------------
``ops``       thin wrappers over the hand-written sm_100a kernels
``parallel``  process groups / meshes, the symmetric heap (GPU) and its CPU twin
``models``    composite blocks built from the ops (tensor-parallel MLP, MoE layer, Llama decoder)
``refs``      the PyTorch + NCCL (+cuBLAS) reference implementation of every op
``workloads`` the op registry: inputs, reference, ours, tolerances, FLOP/byte model per op
``harness``   launcher, per-rank worker, compare, timing, roofline, reports
``utils``     seeding, clocks sampling, environment helpers
"""
__version__ = "0.1.0"
