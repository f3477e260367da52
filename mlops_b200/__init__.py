"""FBLA compressed-KV attention for NVIDIA B200 (sm_100a): the `mlops.attention` interface over hand-written CUDA kernels."""
__version__ = "0.4.0"
