"""B200-native backend for Tessera's dense-contraction hot path (GEMM, flash attention, MoE)."""
__version__ = "0.1.0"
