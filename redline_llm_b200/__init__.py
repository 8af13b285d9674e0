"""B200-native (sm_100a) non-GEMM decode kernels behind the launch contract of
Kasamix/redline-llm's src/kernels/kernels.cuh, plus a thin host mirror."""
__version__ = "0.1.0"
