"""mojolearn's identical-mode matrix product, rebuilt for NVIDIA B200 (sm_100a).

`linalg` and `lowbit` keep the reference's Python operator surface on host
buffers; `torch_ops` takes device-resident tensors on the caller's stream. All
arithmetic runs in hand-written CUDA behind the C ABI of include/b200i.h; there
is no CPU fallback.
"""
from . import linalg, lowbit  # noqa: F401

__all__ = ["linalg", "lowbit"]
