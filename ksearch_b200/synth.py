"""Seeded synthetic tensors in the GGUF block layouts the decode path reads.

No GGUF file or tokenizer exists where this runs, so every weight, cache row
and activation comes from one 64-bit seed.  Each tensor has its own stream:
``splitmix64`` over a counter, started at ``seed XOR fnv1a64(name)``; packed
bytes are taken eight per draw, little endian.  Block layouts follow
``crates/ksearch_ir/src/lib.rs:52-74`` of the reference (Q4_0 18 B / 32,
Q4_K 144 B / 256, Q6_K 210 B / 256).
"""
from __future__ import annotations

import numpy as np

F32, F16, Q4K, Q6K, Q40 = 0, 1, 2, 3, 4
BLOCK_BYTES = {Q4K: 144, Q6K: 210, Q40: 18}
BLOCK_ELEMS = {Q4K: 256, Q6K: 256, Q40: 32}

_GOLD = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def fnv1a64(name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def stream_seed(seed: int, name: str) -> int:
    return (seed ^ fnv1a64(name)) & 0xFFFFFFFFFFFFFFFF


def draws(seed: int, name: str, n: int, offset: int = 0) -> np.ndarray:
    """n consecutive splitmix64 outputs of the tensor's stream (uint64)."""
    with np.errstate(over="ignore"):
        i = np.arange(offset + 1, offset + n + 1, dtype=np.uint64)
        z = np.uint64(stream_seed(seed, name)) + i * _GOLD
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def rand_bytes(seed: int, name: str, n: int) -> np.ndarray:
    d = draws(seed, name, (n + 7) // 8)
    return d.view(np.uint8)[:n].copy()


def uniform01(seed: int, name: str, n: int, offset: int = 0) -> np.ndarray:
    """53-bit uniforms in (0, 1)."""
    d = draws(seed, name, n, offset)
    return ((d >> np.uint64(11)).astype(np.float64) + 0.5) * (1.0 / 9007199254740992.0)


def normals(seed: int, name: str, n: int, sigma: float = 1.0) -> np.ndarray:
    """Box-Muller in f64 from two uniforms per value, cast to f32."""
    u1 = uniform01(seed, name, n, 0)
    u2 = uniform01(seed, name, n, n)
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (z * sigma).astype(np.float32)


def _abs_half_bits(seed: int, name: str, n: int, sigma: float) -> np.ndarray:
    """fp16 bit patterns of |N(0, sigma)| (round to nearest even, never inf/nan)."""
    v = np.abs(normals(seed, name, n, sigma))
    return v.astype(np.float16).view(np.uint16)


def q4k_matrix(seed: int, name: str, rows: int, cols: int, sigma: float = 0.01) -> np.ndarray:
    """[rows, cols] in Q4_K: nibbles uniform 0..15, 6-bit scales/mins uniform
    0..63 (uniform bytes in the 12-byte field make every packed 6-bit value
    uniform), d and dmin = fp16(|N(0, sigma)|).  Returns uint8 [rows*cols/256*144]."""
    assert cols % 256 == 0
    nb = rows * cols // 256
    buf = rand_bytes(seed, name, nb * 144).reshape(nb, 144)
    dd = _abs_half_bits(seed, name + "/d", nb * 2, sigma).reshape(nb, 2)
    buf[:, 0:4] = dd.view(np.uint8).reshape(nb, 4)
    return buf.reshape(-1)


def q5k_matrix(seed: int, name: str, rows: int, cols: int, sigma: float = 0.01) -> np.ndarray:
    """[rows, cols] in Q5_K (176 bytes per 256): qs nibbles and qh bits uniform, 6-bit scales / mins uniform,
    d and dmin = fp16(|N(0, sigma)|)."""
    assert cols % 256 == 0
    nb = rows * cols // 256
    buf = rand_bytes(seed, name, nb * 176).reshape(nb, 176)
    dd = _abs_half_bits(seed, name + "/d", nb * 2, sigma).reshape(nb, 2)
    buf[:, 0:4] = dd.view(np.uint8).reshape(nb, 4)
    return buf.reshape(-1)


def q6k_matrix(seed: int, name: str, rows: int, cols: int, sigma: float = 0.01,
               signed_scales: bool = False) -> np.ndarray:
    """[rows, cols] in Q6_K: ql/qh bytes uniform, 16 int8 scales uniform 0..63
    (or -64..63 with signed_scales), d = fp16(|N(0, sigma)|)."""
    assert cols % 256 == 0
    nb = rows * cols // 256
    buf = rand_bytes(seed, name, nb * 210).reshape(nb, 210)
    if signed_scales:
        sc = (buf[:, 192:208] & 0x7F).astype(np.int16) - 64
        buf[:, 192:208] = sc.astype(np.int8).view(np.uint8)
    else:
        buf[:, 192:208] &= 0x3F
    d = _abs_half_bits(seed, name + "/d", nb, sigma)
    buf[:, 208:210] = d.view(np.uint8).reshape(nb, 2)
    return buf.reshape(-1)


def q40_rows(seed: int, name: str, n_elems: int, sigma: float = 0.05) -> np.ndarray:
    """n_elems values in Q4_0: nibble bytes uniform, scale = fp16(|N(0, sigma)|)."""
    assert n_elems % 32 == 0
    nb = n_elems // 32
    buf = rand_bytes(seed, name, nb * 18).reshape(nb, 18)
    d = _abs_half_bits(seed, name + "/d", nb, sigma)
    buf[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
    return buf.reshape(-1)


def norm_weight(seed: int, name: str, n: int) -> np.ndarray:
    """RMSNorm weight: 1 + 0.1*N(0,1), stored as f32 values that are exact in fp16."""
    w = 1.0 + 0.1 * normals(seed, name, n)
    return w.astype(np.float16).astype(np.float32)


def token_ids(seed: int, name: str, n: int, vocab: int) -> np.ndarray:
    return (draws(seed, name, n) % np.uint64(vocab)).astype(np.int32)
