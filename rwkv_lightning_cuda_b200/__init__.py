"""rwkv_lightning_cuda_b200 -- sm_100a RWKV-7 forward (decode + chunked prefill) behind a C ABI.

The compute lives in ``librwkv7_b200.so`` (hand-written CUDA + a C++ engine, built in-tree by
``rwkv_lightning_cuda_b200.build``); this package is the thin ctypes binding and a Python mirror
of the reference's ``ModelBackend`` interface.  There is no CPU or PyTorch fallback: if the
library cannot be loaded, importing :mod:`rwkv_lightning_cuda_b200.backend` raises.
"""
from .lib import load_library, library_path, Rwkv7B200Error  # noqa: F401

__all__ = ["load_library", "library_path", "Rwkv7B200Error"]
