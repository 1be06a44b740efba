"""Writes the committed fixtures of tests/golden/.

The reference is a Rust workspace and no Rust toolchain exists where this
project is built, so these fixtures come from the CPU oracle (oracle/ks_oracle.c)
after it was cross-checked against tests/np_ref.py and the reference's own CPU
test.  They pin the oracle, the synthetic generator and the packed layouts
against drift, and give the GPU tests stored inputs with stored expected outputs.

    python -m tests.golden.make_golden        # rewrites digests.json and cases.npz
"""
import hashlib
import json
import os

import numpy as np

from ksearch_b200 import synth

HERE = os.path.dirname(os.path.abspath(__file__))
Q4K, Q6K, Q40 = synth.Q4K, synth.Q6K, synth.Q40
SEED = 20240607


def _d(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()[:32]


def _ref_signal():
    i = np.arange(1024, dtype=np.float32)
    t = (np.sin((i * np.float32(0.017) + np.float32(0.3)).astype(np.float32)) * np.float32(1.7)
         + np.cos((i * np.float32(0.041)).astype(np.float32)) * np.float32(0.4) - np.float32(0.15)).astype(np.float32)
    t[256:512] = 0.0
    t[512:768] = -0.25
    return t


def cases(oracle):
    """Small stored cases: name -> dict of arrays."""
    out = {}
    for name, dt, rows, cols in (("q4k_64x512", Q4K, 64, 512), ("q4k_24x1536", Q4K, 24, 1536), ("q6k_32x1536", Q6K, 32, 1536)):
        W = (synth.q4k_matrix if dt == Q4K else synth.q6k_matrix)(SEED, name, rows, cols)
        x = synth.normals(SEED, name + "/x", cols)
        y32, y64 = oracle.matvec(dt, W, rows, cols, x)
        out[name] = dict(W=W, x=x, y32=y32, y64=y64)
    v = synth.normals(SEED, "pack", 32 * 16, sigma=0.7)
    out["pack_q40"] = dict(v=v, packed=oracle.pack_q40(v))
    return out


def compute(oracle):
    """Digests of bit-exact quantities only (no libm-dependent values)."""
    g = {}
    g["synth.q4k"] = _d(synth.q4k_matrix(SEED, "a", 4, 512))
    g["synth.q6k"] = _d(synth.q6k_matrix(SEED, "b", 4, 512))
    g["synth.q6k_signed"] = _d(synth.q6k_matrix(SEED, "b", 4, 512, signed_scales=True))
    g["synth.q40"] = _d(synth.q40_rows(SEED, "c", 1024))
    g["synth.normals"] = _d(synth.normals(SEED, "x", 777))
    g["synth.tokens"] = _d(synth.token_ids(SEED, "p", 64, 262144))
    W4 = synth.q4k_matrix(SEED, "w4", 16, 1024)
    W6 = synth.q6k_matrix(SEED, "w6", 16, 1024, signed_scales=True)
    KV = synth.q40_rows(SEED, "kv", 4096)
    g["dequant.q4k"] = _d(oracle.dequant(Q4K, W4, 16 * 1024))
    g["dequant.q6k"] = _d(oracle.dequant(Q6K, W6, 16 * 1024))
    g["dequant.q40"] = _d(oracle.dequant(Q40, KV, 4096))
    x = synth.normals(SEED, "xv", 1024)
    g["matvec.q4k.y32"] = _d(oracle.matvec(Q4K, W4, 16, 1024, x)[0])
    g["matvec.q6k.y32"] = _d(oracle.matvec(Q6K, W6, 16, 1024, x)[0])
    g["quantize.q4k.ref_signal"] = _d(oracle.quantize_q4k(_ref_signal()))
    r = np.arange(64)[:, None]
    c = np.arange(256)[None, :]
    w = ((((r * 17 + c * 13) % 200).astype(np.float32) - 100.0) * np.float32(0.02)).astype(np.float32)
    g["quantize.q4k.mulmm_64x256"] = _d(oracle.quantize_q4k(w.ravel()))
    g["pack.q40"] = _d(oracle.pack_q40(synth.normals(SEED, "pack", 512, sigma=0.7)))
    g["pack.q40.through_half"] = _d(oracle.pack_q40(synth.normals(SEED, "pack", 512, sigma=0.7), through_half=True))
    g["f32_to_f16_ref"] = _d(oracle.f32_to_f16_ref(synth.normals(SEED, "h", 4096, sigma=3.0)))
    W5 = synth.q5k_matrix(SEED, "w5", 16, 1024)
    g["synth.q5k"] = _d(synth.q5k_matrix(SEED, "e", 4, 512))
    g["dequant.q5k"] = _d(oracle.dequant(5, W5, 16 * 1024))
    # the load-time requantisation of the reference's loader: dequantise, then quantize_f32_to_q4k
    g["requant.q6k_to_q4k"] = _d(oracle.quantize_q4k(oracle.dequant(Q6K, W6, 16 * 1024)))
    g["requant.q5k_to_q4k"] = _d(oracle.quantize_q4k(oracle.dequant(5, W5, 16 * 1024)))
    return g


def main():
    from oracle import ks_oracle
    with open(os.path.join(HERE, "digests.json"), "w") as f:
        json.dump(compute(ks_oracle), f, indent=1, sort_keys=True)
    flat = {}
    for name, d in cases(ks_oracle).items():
        for k, v in d.items():
            flat[f"{name}.{k}"] = v
    np.savez_compressed(os.path.join(HERE, "cases.npz"), **flat)
    print("wrote", len(flat), "arrays")


if __name__ == "__main__":
    main()
