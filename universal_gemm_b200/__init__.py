"""B200-native universal distributed GEMM."""
__version__ = "0.1.0"
