"""CPU sampling of the serve surface: crates/ksearch_gemma/src/sample.rs:9-81 over the library's host code."""
from __future__ import annotations

import numpy as np

from . import _lib


def sample_softcap_min_p(logits, cap: float, temperature: float, min_p: float, seed: int) -> int:
    """logits: uint16 array of f16 bit patterns (the reference's form) or a float32 array."""
    lib = _lib.load()
    a = np.ascontiguousarray(logits)
    if a.dtype == np.uint16:
        return int(lib.ks_sample_softcap_min_p(a.ctypes.data, a.size, cap, temperature, min_p, seed & 0xFFFFFFFF))
    a = np.ascontiguousarray(a, dtype=np.float32)
    return int(lib.ks_sample_softcap_min_p_f32(a.ctypes.data, a.size, cap, temperature, min_p, seed & 0xFFFFFFFF))
