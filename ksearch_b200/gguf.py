"""GGUF files on the load side of the decode path: a thin mirror of the reference's `Gguf`
(crates/ksearch_gguf/src/gguf_impl.rs:122-417) over the library's reader, and of `GemmaConfig::from_gguf`
(crates/ksearch_gemma/src/lib.rs:38-122)."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import _lib
from .eng import KsError

# ggml type ids of the file (gguf_impl.rs:20-31)
GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q4_K, GGML_Q5_K, GGML_Q6_K, GGML_BF16 = 0, 1, 2, 12, 13, 14, 30
GGML_NAMES = {0: "F32", 1: "F16", 2: "Q4_0", 3: "Q4_1", 7: "Q5_1", 8: "Q8_0", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K", 30: "BF16"}


@dataclass
class TensorInfo:
    name: str
    ggml_type: int
    dims: tuple          # ne0 first, as in the file
    file_offset: int     # absolute (tensor_file_offset)
    nbytes: int

    def n_rows(self) -> int:
        return int(np.prod(self.dims[1:])) if len(self.dims) > 1 else 1


class Gguf:
    """Gguf::open: maps the file, parses header, metadata and tensor infos."""

    def __init__(self, path: str):
        self.lib = _lib.load()
        err = C.create_string_buffer(256)
        self.h = self.lib.ks_gguf_open(str(path).encode(), err, 256)
        if not self.h:
            raise KsError(_lib.ERR_INVALID, err.value.decode(errors="replace"))

    def close(self):
        if self.h:
            self.lib.ks_gguf_close(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    @property
    def version(self) -> int:
        return self.lib.ks_gguf_version(self.h)

    @property
    def data_offset(self) -> int:
        return self.lib.ks_gguf_data_offset(self.h)

    def n_kv(self) -> int:
        return self.lib.ks_gguf_n_kv(self.h)

    def tensor_names(self) -> list:
        return [self.lib.ks_gguf_tensor_name(self.h, i).decode(errors="replace") for i in range(self.lib.ks_gguf_n_tensors(self.h))]

    def has_tensor(self, name: str) -> bool:
        return self.lib.ks_gguf_tensor(self.h, name.encode(), None, None, None, None, None) == 0

    def tensor(self, name: str) -> TensorInfo:
        t, nd, off, nb = C.c_uint32(), C.c_uint32(), C.c_uint64(), C.c_uint64()
        dims = (C.c_uint64 * 4)()
        if self.lib.ks_gguf_tensor(self.h, name.encode(), C.byref(t), C.byref(nd), dims, C.byref(off), C.byref(nb)):
            raise KsError(_lib.ERR_INVALID, f"tensor not found: {name}")
        return TensorInfo(name, t.value, tuple(int(d) for d in dims[:min(nd.value, 4)]), off.value, nb.value)

    def tensor_raw(self, name: str) -> np.ndarray:
        """The tensor's on-disk bytes (a copy of the mapped range)."""
        info = self.tensor(name)
        ptr = self.lib.ks_gguf_tensor_raw(self.h, name.encode())
        if not ptr:
            raise KsError(_lib.ERR_UNSUPPORTED, f"unsupported ggml type id {info.ggml_type}")
        return np.ctypeslib.as_array((C.c_uint8 * info.nbytes).from_address(ptr)).copy()

    # -- metadata (get_u32 / get_f32 / ... with the reference's coercions; None when absent or of another type)
    def has_key(self, key: str) -> bool:
        return bool(self.lib.ks_gguf_has_key(self.h, key.encode()))

    def _scalar(self, fn, ctype, key):
        v = ctype()
        return v.value if fn(self.h, key.encode(), C.byref(v)) else None

    def get_u32(self, key):
        return self._scalar(self.lib.ks_gguf_get_u32, C.c_uint32, key)

    def get_u64(self, key):
        return self._scalar(self.lib.ks_gguf_get_u64, C.c_uint64, key)

    def get_f32(self, key):
        return self._scalar(self.lib.ks_gguf_get_f32, C.c_float, key)

    def get_bool(self, key):
        v = self._scalar(self.lib.ks_gguf_get_bool, C.c_int, key)
        return None if v is None else bool(v)

    def get_str(self, key):
        s = self.lib.ks_gguf_get_str(self.h, key.encode())
        return None if s is None else s.decode(errors="replace")

    def arr_len(self, key):
        """(length, element type id) of an array value, or None."""
        et = C.c_uint32()
        n = self.lib.ks_gguf_arr_len(self.h, key.encode(), C.byref(et))
        return None if n < 0 else (int(n), et.value)

    def _arr(self, fn, ctype, key):
        n = fn(self.h, key.encode(), None, 0)
        if n < 0:
            return None
        out = (ctype * max(int(n), 1))()
        fn(self.h, key.encode(), out, int(n))
        return [out[i] for i in range(int(n))]

    def get_arr_u32(self, key):
        return self._arr(self.lib.ks_gguf_get_arr_u32, C.c_uint32, key)

    def get_arr_i32(self, key):
        return self._arr(self.lib.ks_gguf_get_arr_i32, C.c_int32, key)

    def get_arr_f32(self, key):
        return self._arr(self.lib.ks_gguf_get_arr_f32, C.c_float, key)

    def get_arr_bool(self, key):
        v = self._arr(self.lib.ks_gguf_get_arr_bool, C.c_uint8, key)
        return None if v is None else [bool(b) for b in v]

    def get_arr_str(self, key):
        ln = self.arr_len(key)
        if ln is None or ln[1] != 8:
            return None
        return [self.lib.ks_gguf_get_arr_str(self.h, key.encode(), i).decode(errors="replace") for i in range(ln[0])]

    def get_usize_list(self, key):
        """gguf_impl.rs:394-404: a u32 or i32 array, or a single U32 / I32 / U64, as a list."""
        v = self.get_arr_u32(key)
        if v is None:
            v = self.get_arr_i32(key)
        if v is None:
            s = self.get_u64(key)
            return None if s is None else [int(s)]
        return [int(x) for x in v]


@dataclass
class GemmaConfig:
    """GemmaConfig (crates/ksearch_gemma/src/lib.rs:14-36), filled as from_gguf fills it (lib.rs:38-122)."""
    n_layers: int
    hidden: int
    n_heads: int
    n_kv: int
    head_dim_swa: int
    head_dim_full: int
    sliding_window: int
    shared_kv_layers: int
    ffn: list
    swa_pattern: list
    rms_eps: float
    softcap: float
    vocab: int
    ple_dim: int
    rope_theta_full: float
    rope_theta_swa: float
    partial_rotary: float = 0.25
    context_length: int = 131072
    notes: list = field(default_factory=list)

    @classmethod
    def from_gguf(cls, g: Gguf) -> "GemmaConfig":
        arch = g.get_str("general.architecture")
        if arch is not None and arch != "gemma4":
            raise KsError(_lib.ERR_UNSUPPORTED, f"unsupported GGUF architecture `{arch}` (expected gemma4)")
        if (g.get_u32("gemma4.expert_count") or 0) > 0:
            raise KsError(_lib.ERR_UNSUPPORTED, "Gemma 4 MoE (A4B) is not supported")
        n_layers = g.get_u32("gemma4.block_count")
        if n_layers is None:
            raise KsError(_lib.ERR_INVALID, "block_count")
        hidden = g.get_u32("gemma4.embedding_length")
        n_heads = g.get_u32("gemma4.attention.head_count")
        if hidden is None or n_heads is None:
            raise KsError(_lib.ERR_INVALID, "embedding_length / attention.head_count")
        n_kv_list = g.get_usize_list("gemma4.attention.head_count_kv") or [1]
        if len(n_kv_list) > 1:
            raise KsError(_lib.ERR_UNSUPPORTED, "per-layer head_count_kv is not supported (A4B/MoE)")
        n_kv = max(n_kv_list[0] if n_kv_list else 1, 1)
        if n_heads % n_kv:
            raise KsError(_lib.ERR_INVALID, f"head_count {n_heads} not divisible by head_count_kv {n_kv}")
        ffn = g.get_usize_list("gemma4.feed_forward_length") or [6144]
        ffn = ffn * n_layers if len(ffn) == 1 else ffn if len(ffn) == n_layers else [6144] * n_layers
        pattern = g.get_arr_bool("gemma4.attention.sliding_window_pattern")
        if pattern is None:
            pattern = [(i + 1) % 6 != 0 for i in range(n_layers)]
        vocab = g.tensor("token_embd.weight").n_rows() if g.has_tensor("token_embd.weight") else 262144
        dflt = lambda v, d: d if v is None else v
        return cls(
            n_layers=n_layers, hidden=hidden, n_heads=n_heads, n_kv=n_kv,
            head_dim_swa=dflt(g.get_u32("gemma4.attention.key_length_swa"), 256),
            head_dim_full=dflt(g.get_u32("gemma4.attention.key_length"), 512),
            sliding_window=dflt(g.get_u32("gemma4.attention.sliding_window"), 512),
            shared_kv_layers=dflt(g.get_u32("gemma4.attention.shared_kv_layers"), 0),
            ffn=ffn, swa_pattern=pattern,
            rms_eps=dflt(g.get_f32("gemma4.attention.layer_norm_rms_epsilon"), 1e-6),
            softcap=dflt(g.get_f32("gemma4.final_logit_softcapping"), 30.0),
            vocab=vocab,
            ple_dim=dflt(g.get_u32("gemma4.embedding_length_per_layer_input"), 256),
            rope_theta_full=dflt(g.get_f32("gemma4.rope.freq_base"), 1_000_000.0),
            rope_theta_swa=dflt(g.get_f32("gemma4.rope.freq_base_swa"), 10_000.0),
            context_length=dflt(g.get_u32("gemma4.context_length"), 131072),
        )
