"""B200 (sm_100a) implementation of lemonade-burn's packed ternary x int8 matmul path.

`pack`     host-side layout and ternariser (crates/lb-ternary/src/pack.rs)
`ternary`  lb-ternary's public API over the CUDA C ABI, numpy host buffers
`ops`      lb-model's op boundary on torch CUDA tensors (device resident)
The arithmetic lives in liblbk.so (csrc/, C ABI in include/lbk.h); importing this package
does not load it, using any op does, and a missing library is an error, never a fallback.
"""
from . import pack  # noqa: F401
from .pack import BLOCK, BLOCK_BYTES, PackedTernary, TernaryView  # noqa: F401

__all__ = ["pack", "PackedTernary", "TernaryView", "BLOCK", "BLOCK_BYTES"]
