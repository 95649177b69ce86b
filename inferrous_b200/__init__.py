"""B200-native W8A8 linear layer for the inferrous Qwen3-8B engine.

The product is the C-ABI CUDA library `inferrous_b200/lib/libw8a8.so` (include/w8a8.h).
This package is the thin Python face of it: `capi` binds the exported symbols with ctypes,
`ops` mirrors the reference host's operator methods on torch device tensors (torch is used
for device memory and streams only).  There is no CPU or PyTorch fallback: importing `ops`
without the built library, or calling it without a CUDA device, raises.
"""
__version__ = "0.1.0"
