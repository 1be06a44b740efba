"""ctypes front end of the CPU oracle (``ks_oracle.c``).

Test infrastructure only: imported by ``tests/``, by ``__graft_entry__.smoke``
and by the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.  The
shipped package never imports it.

Two builds of the same C file exist: the parity build (``-O2
-ffp-contract=off``) and a timed build (``-O3 -march=native``) that is compiled
on the machine it runs on, keyed by the CPU's flag set, so a library built on
one host is never executed on another.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "ks_oracle.c")

F32, F16, Q4K, Q6K, Q40 = 0, 1, 2, 3, 4
BLOCK_BYTES = {Q4K: 144, Q6K: 210, Q40: 18}
BLOCK_ELEMS = {Q4K: 256, Q6K: 256, Q40: 32}


def _cpu_tag() -> str:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return hashlib.sha1(line.encode()).hexdigest()[:10]
    except OSError:
        pass
    return "generic"


def _build(out: str, flags: list[str]) -> None:
    cmd = ["gcc", *flags, "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared", "-o", out, _SRC, "-lm"]
    subprocess.run(cmd, check=True, capture_output=True)


def build(fast: bool = False) -> str:
    """Compile (if stale) and return the path of the requested oracle build."""
    if fast:
        out = os.path.join(_HERE, f"libks_oracle_fast_{_cpu_tag()}.so")
        flags = ["-O3", "-march=native"]
    else:
        out = os.path.join(_HERE, "libks_oracle.so")
        flags = ["-O2"]
    if not os.path.exists(out) or os.path.getmtime(out) < os.path.getmtime(_SRC):
        _build(out, flags)
    return out


_libs: dict[bool, C.CDLL] = {}

_u8p = C.POINTER(C.c_uint8)
_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)


def _ptr(a, ty):
    if a is None:
        return None
    return a.ctypes.data_as(ty)


def lib(fast: bool = False) -> C.CDLL:
    if fast not in _libs:
        L = C.CDLL(build(fast))
        L.kso_f16_to_f32.restype = C.c_float
        L.kso_f16_to_f32.argtypes = [C.c_uint16]
        L.kso_f32_to_f16_ref.restype = C.c_uint16
        L.kso_f32_to_f16_ref.argtypes = [C.c_float]
        L.kso_f32_to_f16_rne.restype = C.c_uint16
        L.kso_f32_to_f16_rne.argtypes = [C.c_float]
        L.kso_gelu_mul.restype = C.c_float
        L.kso_gelu_mul.argtypes = [C.c_float, C.c_float]
        L.kso_softcap_argmax.restype = C.c_float
        L.kso_softcap_argmax.argtypes = [_f32p, C.c_size_t, C.c_float, _f32p]
        L.kso_dequant.argtypes = [C.c_int, _u8p, C.c_size_t, _f32p]
        L.kso_quantize_q4k.argtypes = [_f32p, C.c_size_t, _u8p]
        L.kso_matvec.argtypes = [C.c_int, _u8p, C.c_size_t, C.c_size_t, _f32p, C.c_size_t, _f32p, _f64p]
        L.kso_matvec_two_pass.argtypes = [C.c_int, _u8p, C.c_size_t, C.c_size_t, _f32p, _f32p, _f32p]
        L.kso_gelu_mul_n.argtypes = [_f32p, _f32p, _f32p, C.c_size_t]
        L.kso_rmsnorm.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_float, C.c_size_t, C.c_size_t, C.c_float, _f32p]
        L.kso_rmsnorm_add_then_rmsnorm.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_size_t, C.c_size_t, C.c_float, _f32p, _f32p]
        L.kso_pack_q40.argtypes = [_f32p, C.c_size_t, C.c_int, _u8p]
        L.kso_rope_table.argtypes = [C.c_size_t, C.c_size_t, C.c_float, C.c_size_t, _f32p]
        L.kso_rmsnorm_per_head_qkv_q40.argtypes = [C.c_size_t] * 4 + [C.c_float] + [_f32p] * 6 + [_f32p, _u8p, _u8p, C.c_size_t]
        L.kso_sdpa_decode.argtypes = [C.c_size_t] * 3 + [_f32p, _u8p, _u8p, C.c_size_t, C.c_size_t, C.c_float, C.c_size_t, _f32p]
        L.kso_copy_scale_indexed.argtypes = [C.c_int, _u8p, C.c_size_t, _f32p, C.c_size_t, C.c_float, _f32p]
        L.kso_f16_to_f32_n.argtypes = [C.POINTER(C.c_uint16), _f32p, C.c_size_t]
        L.kso_f32_to_f16_rne_n.argtypes = [_f32p, C.POINTER(C.c_uint16), C.c_size_t]
        L.kso_f32_to_f16_ref_n.argtypes = [_f32p, C.POINTER(C.c_uint16), C.c_size_t]
        L.kso_state_new.restype = C.c_void_p
        L.kso_state_new.argtypes = [C.c_void_p]
        L.kso_state_free.argtypes = [C.c_void_p]
        L.kso_state_reset.argtypes = [C.c_void_p]
        L.kso_state_logits.restype = _f32p
        L.kso_state_logits.argtypes = [C.c_void_p]
        L.kso_state_hidden.restype = _f32p
        L.kso_state_hidden.argtypes = [C.c_void_p]
        L.kso_state_kv.restype = _u8p
        L.kso_state_kv.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.kso_forward_token.restype = C.c_int
        L.kso_forward_token.argtypes = [C.c_void_p, C.c_int, C.c_int]
        _libs[fast] = L
    return _libs[fast]


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


# ---- scalar / vector conversions -------------------------------------------

def f16_to_f32(h) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16)
    out = np.empty(h.shape, np.float32)
    lib().kso_f16_to_f32_n(h.ctypes.data_as(C.POINTER(C.c_uint16)), _ptr(out, _f32p), h.size)
    return out


def f32_to_f16_rne(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, np.uint16)
    lib().kso_f32_to_f16_rne_n(_ptr(x, _f32p), out.ctypes.data_as(C.POINTER(C.c_uint16)), x.size)
    return out


def f32_to_f16_ref(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, np.uint16)
    lib().kso_f32_to_f16_ref_n(_ptr(x, _f32p), out.ctypes.data_as(C.POINTER(C.c_uint16)), x.size)
    return out


# ---- dequant / quant --------------------------------------------------------

def dequant(dtype: int, data, nelem: int) -> np.ndarray:
    data = _u8(data)
    out = np.empty(nelem, np.float32)
    if lib().kso_dequant(dtype, _ptr(data, _u8p), nelem, _ptr(out, _f32p)):
        raise ValueError("dequant: bad dtype or length")
    return out


def quantize_q4k(x) -> np.ndarray:
    x = _f32(x).ravel()
    out = np.empty(x.size // 256 * 144, np.uint8)
    if lib().kso_quantize_q4k(_ptr(x, _f32p), x.size, _ptr(out, _u8p)):
        raise ValueError("quantize_q4k: length not a multiple of 256")
    return out


def matvec(dtype: int, W, rows: int, cols: int, x, want64: bool = True, fast: bool = False):
    """Returns (y32, y64): f32-sequential sums as the reference's check computes
    them, and the same products summed in f64.  x may be [cols] or [n_tok, cols]."""
    W = _u8(W)
    x = _f32(x)
    n_tok = 1 if x.ndim == 1 else x.shape[0]
    y32 = np.empty((n_tok, rows), np.float32)
    y64 = np.empty((n_tok, rows), np.float64) if want64 else None
    rc = lib(fast).kso_matvec(dtype, _ptr(W, _u8p), rows, cols, _ptr(x, _f32p), n_tok, _ptr(y32, _f32p), _ptr(y64, _f64p))
    if rc:
        raise ValueError("matvec: bad shape")
    if x.ndim == 1:
        return y32[0], (y64[0] if want64 else None)
    return y32, y64


def matvec_two_pass(dtype: int, W, rows: int, cols: int, x, wd_scratch=None, fast: bool = True):
    W = _u8(W)
    x = _f32(x)
    wd = wd_scratch if wd_scratch is not None else np.empty(rows * cols, np.float32)
    y = np.empty(rows, np.float32)
    lib(fast).kso_matvec_two_pass(dtype, _ptr(W, _u8p), rows, cols, _ptr(x, _f32p), _ptr(wd, _f32p), _ptr(y, _f32p))
    return y


# ---- shader-math ops --------------------------------------------------------

def gelu_mul(g, u) -> np.ndarray:
    g, u = _f32(g), _f32(u)
    out = np.empty_like(g)
    lib().kso_gelu_mul_n(_ptr(g, _f32p), _ptr(u, _f32p), _ptr(out, _f32p), g.size)
    return out


def rmsnorm(x, w, eps: float, res=None, scale=None, rows: int = 1) -> np.ndarray:
    x = _f32(x)
    n = x.size // rows
    w = None if w is None else _f32(w)
    res = None if res is None else _f32(res)
    y = np.empty_like(x)
    lib().kso_rmsnorm(_ptr(x, _f32p), _ptr(w, _f32p), _ptr(res, _f32p), int(scale is not None),
                      float(scale or 0.0), n, rows, eps, _ptr(y, _f32p))
    return y


def rmsnorm_add_then_rmsnorm(y, w_post, res, w_ffn, eps: float, rows: int = 1):
    y, w_post, res, w_ffn = _f32(y), _f32(w_post), _f32(res), _f32(w_ffn)
    n = y.size // rows
    ox, ox2 = np.empty_like(y), np.empty_like(y)
    lib().kso_rmsnorm_add_then_rmsnorm(_ptr(y, _f32p), _ptr(w_post, _f32p), _ptr(res, _f32p), _ptr(w_ffn, _f32p),
                                       n, rows, eps, _ptr(ox, _f32p), _ptr(ox2, _f32p))
    return ox, ox2


def pack_q40(x, through_half: bool = False) -> np.ndarray:
    x = _f32(x).ravel()
    out = np.empty(x.size // 32 * 18, np.uint8)
    lib().kso_pack_q40(_ptr(x, _f32p), x.size, int(through_half), _ptr(out, _u8p))
    return out


def rope_table(max_seq: int, hd: int, theta: float, rope_angles: int | None = None) -> np.ndarray:
    out = np.empty((max_seq, hd), np.float32)
    lib().kso_rope_table(max_seq, hd, theta, hd // 2 if rope_angles is None else rope_angles, _ptr(out, _f32p))
    return out


def rmsnorm_per_head_qkv_q40(n_q, n_kv, hd, n_tok, eps, q, qw, rope, k, kw, v, kv_k, kv_v, kv_byte_off):
    """kv_k / kv_v are uint8 arrays updated in place; returns q_out."""
    q, qw, rope, k, kw, v = map(_f32, (q, qw, rope, k, kw, v))
    q_out = np.empty_like(q)
    lib().kso_rmsnorm_per_head_qkv_q40(n_q, n_kv, hd, n_tok, eps, _ptr(q, _f32p), _ptr(qw, _f32p), _ptr(rope, _f32p),
                                       _ptr(k, _f32p), _ptr(kw, _f32p), _ptr(v, _f32p), _ptr(q_out, _f32p),
                                       _ptr(kv_k, _u8p), _ptr(kv_v, _u8p), kv_byte_off)
    return q_out


def sdpa_decode(n_q, n_kv, hd, q, K, V, tlen, start=0, scale=1.0, nwg=0) -> np.ndarray:
    q, K, V = _f32(q), _u8(K), _u8(V)
    out = np.empty(n_q * hd, np.float32)
    lib().kso_sdpa_decode(n_q, n_kv, hd, _ptr(q, _f32p), _ptr(K, _u8p), _ptr(V, _u8p), tlen, start, scale, nwg,
                          _ptr(out, _f32p))
    return out


def copy_scale_indexed(dtype, src, n, idx, scale) -> np.ndarray:
    src = np.ascontiguousarray(src)
    idx = _f32(np.atleast_1d(idx))
    out = np.empty((idx.size, n), np.float32)
    rc = lib().kso_copy_scale_indexed(dtype, C.cast(src.ctypes.data, _u8p), n, _ptr(idx, _f32p), idx.size, scale,
                                      _ptr(out, _f32p))
    if rc:
        raise ValueError("copy_scale_indexed: bad shape")
    return out


def softcap_argmax(x, cap: float):
    x = _f32(x)
    bv = C.c_float()
    i = lib().kso_softcap_argmax(_ptr(x, _f32p), x.size, cap, C.byref(bv))
    return int(i), float(bv.value)


# ---- CPU decoder ------------------------------------------------------------

class _Model(C.Structure):
    _fields_ = [
        ("n_layers", C.c_int), ("hidden", C.c_int), ("ffn", C.c_int), ("n_q", C.c_int), ("n_kv", C.c_int),
        ("hd", C.c_int), ("vocab", C.c_int), ("max_seq", C.c_int),
        ("eps", C.c_float), ("rope_theta", C.c_float), ("softcap", C.c_float), ("attn_scale", C.c_float),
        ("embd_dtype", C.c_int),
        ("token_embd", C.c_void_p), ("output_norm", C.c_void_p),
        ("wq", C.c_void_p), ("wk", C.c_void_p), ("wv", C.c_void_p), ("wo", C.c_void_p),
        ("wgate", C.c_void_p), ("wup", C.c_void_p), ("wdown", C.c_void_p),
        ("attn_norm", C.c_void_p), ("q_norm", C.c_void_p), ("k_norm", C.c_void_p),
        ("post_attn_norm", C.c_void_p), ("ffn_norm", C.c_void_p), ("post_ffw_norm", C.c_void_p),
        ("sliding_window", C.c_int), ("swa_layers", C.c_ulonglong),
    ]


# struct field -> GGUF tensor suffix (crates/ksearch_gemma/src/gemma_prim.rs:174-181, 356-357)
_LAYER_FIELDS = {"wq": "attn_q.weight", "wk": "attn_k.weight", "wv": "attn_v.weight", "wo": "attn_output.weight",
                 "wgate": "ffn_gate.weight", "wup": "ffn_up.weight", "wdown": "ffn_down.weight",
                 "attn_norm": "attn_norm.weight", "q_norm": "attn_q_norm.weight", "k_norm": "attn_k_norm.weight",
                 "post_attn_norm": "post_attention_norm.weight", "ffn_norm": "ffn_norm.weight",
                 "post_ffw_norm": "post_ffw_norm.weight"}


class CpuDecoder:
    """CPU fp32 decoder over the same packed tensors the CUDA model is given.

    ``cfg``: dict with n_layers, hidden, ffn, n_q, n_kv, hd, vocab, max_seq, eps,
    rope_theta, softcap, attn_scale, embd_dtype.  ``tensors``: GGUF tensor name ->
    ndarray (``token_embd.weight``, ``output_norm.weight``, ``blk.N.attn_q.weight`` ...);
    packed weights uint8, norm weights float32.
    """

    def __init__(self, cfg: dict, tensors: dict, fast: bool = False):
        self._L = lib(fast)
        self._keep = []
        m = _Model()
        for k in ("n_layers", "hidden", "ffn", "n_q", "n_kv", "hd", "vocab", "max_seq", "embd_dtype"):
            setattr(m, k, int(cfg[k]))
        for k in ("eps", "rope_theta", "softcap", "attn_scale"):
            setattr(m, k, float(cfg[k]))
        m.sliding_window = int(cfg.get("sliding_window", 0))
        m.swa_layers = int(cfg.get("swa_layers", 0))

        def hold(a, dt):
            a = np.ascontiguousarray(a, dtype=dt)
            self._keep.append(a)
            return a.ctypes.data

        m.token_embd = hold(tensors["token_embd.weight"], np.uint8)
        m.output_norm = hold(tensors["output_norm.weight"], np.float32)
        for f, suffix in _LAYER_FIELDS.items():
            dt = np.uint8 if f.startswith("w") else np.float32
            arr = (C.c_void_p * m.n_layers)(*[hold(tensors[f"blk.{l}.{suffix}"], dt) for l in range(m.n_layers)])
            self._keep.append(arr)
            setattr(m, f, C.cast(arr, C.c_void_p))
        self._m = m
        self.cfg = dict(cfg)
        self._s = self._L.kso_state_new(C.addressof(m))

    def reset(self):
        self._L.kso_state_reset(self._s)

    def forward_token(self, token: int, want_logits: bool = True) -> int:
        r = self._L.kso_forward_token(self._s, int(token), int(want_logits))
        if r < 0:
            raise RuntimeError("max_seq exceeded")
        return r

    def logits(self) -> np.ndarray:
        return np.ctypeslib.as_array(self._L.kso_state_logits(self._s), shape=(self.cfg["vocab"],)).copy()

    def hidden(self) -> np.ndarray:
        return np.ctypeslib.as_array(self._L.kso_state_hidden(self._s), shape=(self.cfg["hidden"],)).copy()

    def kv(self, layer: int, which: int) -> np.ndarray:
        """A view (not a copy) of one layer's cache rows, [max_seq * n_kv * hd/32 * 18] bytes; which: 0 = K, 1 = V."""
        c = self.cfg
        n = c["max_seq"] * c["n_kv"] * (c["hd"] // 32) * 18
        return np.ctypeslib.as_array(self._L.kso_state_kv(self._s, layer, which), shape=(n,))

    def generate(self, prompt, n_new: int):
        """gemma_prim.rs:1658-1768: prompt[:-1] without logits, then n_new greedy steps from prompt[-1]."""
        self.reset()
        for t in prompt[:-1]:
            self.forward_token(int(t), want_logits=False)
        tok = int(prompt[-1])
        out = []
        for _ in range(n_new):
            tok = self.forward_token(tok, True)
            out.append(tok)
        return out

    def close(self):
        if self._s:
            self._L.kso_state_free(self._s)
            self._s = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_CFG_KEYS = ("n_layers", "hidden", "ffn", "n_q", "n_kv", "hd", "vocab", "max_seq", "eps", "rope_theta",
             "softcap", "attn_scale", "embd_dtype")


def decoder_cfg(cfg) -> dict:
    """The CpuDecoder's config dict from a model-config object (attributes of the same names)."""
    d = {k: getattr(cfg, k) for k in _CFG_KEYS}
    d["sliding_window"] = int(getattr(cfg, "sliding_window", 0))
    d["swa_layers"] = int(getattr(cfg, "swa_layers", 0))
    return d


def compare_streams(cuda_tokens, cpu_decoder, prompt, logit_tol: float = 2e-3):
    """Greedy streams must be identical; the one allowed exception is a near-tie: where the CUDA
    token differs, the CPU logits of the two candidates must differ by less than logit_tol
    (relative to the logit scale), and the comparison continues on the CUDA token.
    Returns (n_equal, n_near_tie)."""
    cpu_decoder.reset()
    for t in prompt[:-1]:
        cpu_decoder.forward_token(int(t), False)
    tok = int(prompt[-1])
    equal = ties = 0
    for got in cuda_tokens:
        want = cpu_decoder.forward_token(tok, True)
        if want == got:
            equal += 1
        else:
            lg = cpu_decoder.logits()
            gap = abs(float(lg[want]) - float(lg[got]))
            if gap > logit_tol * max(1.0, float(np.abs(lg).max())):
                raise AssertionError(f"token stream diverged: cuda {got} vs cpu {want}, logit gap {gap}")
            ties += 1
        tok = got
    return equal, ties
