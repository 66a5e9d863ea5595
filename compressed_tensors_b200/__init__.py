"""B200-native tensor codec behind the compressed-tensors API (hand-written sm_100a CUDA through a C ABI)."""
__version__ = "0.1.0"
