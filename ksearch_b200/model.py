"""Host-side mirror of ``GemmaPrimModel`` (crates/ksearch_gemma/src/gemma_prim.rs) for the
dense synthetic decoders, over the C ABI's decode driver, plus the seeded model builder.

No checkpoint or tokenizer exists where this runs: weights are random-init from a seed with the
distributions of the benchmark configs (Q4_K attention/FFN matrices, Q6_K tied embedding /
lm_head, Q4_0 KV cache, norm weights 1 + 0.1*N(0,1)).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib, synth
from ._lib import F16, F32, Q4K, Q6K
from .eng import CudaContext, KsError


@dataclass
class ModelConfig:
    """The GemmaConfig fields the dense path uses (crates/ksearch_gemma/src/lib.rs:14-36)."""
    n_layers: int
    hidden: int
    ffn: int
    n_q: int
    n_kv: int
    hd: int
    vocab: int
    max_seq: int
    n_slots: int = 1
    eps: float = 1e-6
    rope_theta: float = 1e6
    softcap: float = 30.0
    attn_scale: float = 1.0 / 16.0
    embd_dtype: int = Q6K
    act: int = F32
    sliding_window: int = 0       # positions a sliding-window layer attends to (0: every layer is full attention)
    swa_layers: int = 0           # bit l set: layer l is a sliding-window layer
    # synthetic-weight scales: fp16 |N(0, sigma)| super-block scales
    sigma_w: float = 0.01
    sigma_embd: float = 1e-4


def e2b_config(max_seq: int = 256, n_slots: int = 1) -> ModelConfig:
    """E2B-shaped: 35 layers, hidden 1536, GeGLU 6144, 8 q / 1 kv heads of 256, vocab 262144."""
    return ModelConfig(35, 1536, 6144, 8, 1, 256, 262144, max_seq, n_slots)


def e4b_config(max_seq: int = 16384, n_slots: int = 8) -> ModelConfig:
    """E4B-shaped: 42 layers, hidden 2560, GeGLU 10240, 8 q / 2 kv heads of 256, vocab 262144."""
    return ModelConfig(42, 2560, 10240, 8, 2, 256, 262144, max_seq, n_slots)


def tiny_config(max_seq: int = 64, n_slots: int = 1, n_kv: int = 1, act: int = F32) -> ModelConfig:
    return ModelConfig(3, 512, 1024, 4, n_kv, 128, 2048, max_seq, n_slots, act=act, sigma_w=0.01, sigma_embd=5e-5)


def tensor_specs(cfg: ModelConfig):
    """(name, kind, rows, cols) for every tensor, in upload order."""
    H, F, qn, kvn = cfg.hidden, cfg.ffn, cfg.n_q * cfg.hd, cfg.n_kv * cfg.hd
    yield "token_embd.weight", "embd", cfg.vocab, H
    yield "output_norm.weight", "norm", 1, H
    for l in range(cfg.n_layers):
        p = f"blk.{l}."
        yield p + "attn_q.weight", "q4k", qn, H
        yield p + "attn_k.weight", "q4k", kvn, H
        yield p + "attn_v.weight", "q4k", kvn, H
        yield p + "attn_output.weight", "q4k", H, qn
        yield p + "ffn_gate.weight", "q4k", cfg.ffn, H
        yield p + "ffn_up.weight", "q4k", cfg.ffn, H
        yield p + "ffn_down.weight", "q4k", H, F
        yield p + "attn_norm.weight", "norm", 1, H
        yield p + "attn_q_norm.weight", "norm", 1, cfg.hd
        yield p + "attn_k_norm.weight", "norm", 1, cfg.hd
        yield p + "post_attention_norm.weight", "norm", 1, H
        yield p + "ffn_norm.weight", "norm", 1, H
        yield p + "post_ffw_norm.weight", "norm", 1, H


def synth_tensor(cfg: ModelConfig, seed: int, name: str, kind: str, rows: int, cols: int) -> np.ndarray:
    """Packed weights as uint8; norm weights as float32 (values exact in fp16)."""
    if kind == "q4k":
        return synth.q4k_matrix(seed, name, rows, cols, cfg.sigma_w)
    if kind == "embd":
        gen = synth.q6k_matrix if cfg.embd_dtype == Q6K else synth.q4k_matrix
        kw = dict(signed_scales=True) if cfg.embd_dtype == Q6K else {}
        # generated in row slabs so a 262144-row table never needs more than ~100 MB of scratch
        slab = 16384
        if rows <= slab:
            return gen(seed, name, rows, cols, cfg.sigma_embd, **kw)
        return np.concatenate([gen(seed, f"{name}/{r0}", min(slab, rows - r0), cols, cfg.sigma_embd, **kw)
                               for r0 in range(0, rows, slab)])
    return synth.norm_weight(seed, name, cols)


def synth_tensors(cfg: ModelConfig, seed: int) -> dict:
    return {n: synth_tensor(cfg, seed, n, k, r, c) for n, k, r, c in tensor_specs(cfg)}


def weight_bytes_per_token(cfg: ModelConfig) -> int:
    """Packed weight bytes one decode step must stream (layers + tied lm_head)."""
    H, F, qn, kvn = cfg.hidden, cfg.ffn, cfg.n_q * cfg.hd, cfg.n_kv * cfg.hd
    per_layer = (qn * H + 2 * kvn * H + H * qn + 2 * F * H + H * F) // 256 * 144
    head = cfg.vocab * H // 256 * (210 if cfg.embd_dtype == Q6K else 144)
    return cfg.n_layers * per_layer + head


class _Cfg(C.Structure):
    _fields_ = [(k, C.c_int) for k in ("n_layers", "hidden", "ffn", "n_q", "n_kv", "hd", "vocab", "max_seq", "n_slots")] + \
               [(k, C.c_float) for k in ("eps", "rope_theta", "softcap", "attn_scale")] + \
               [("embd_dtype", C.c_int), ("act", C.c_int), ("sliding_window", C.c_int), ("swa_layers", C.c_ulonglong)]


class GenStats(C.Structure):
    _fields_ = [("prefill_tokens", C.c_int), ("decode_tokens", C.c_int),
                ("prefill_ms_device", C.c_float), ("decode_ms_device", C.c_float)]


class GemmaCudaModel:
    """load / bind_slot / decode_token / generate_timed over libksearch_cuda.so."""

    def __init__(self, ctx: CudaContext, cfg: ModelConfig):
        self.ctx, self.cfg, self.lib = ctx, cfg, ctx.lib
        c = _Cfg(**{k: getattr(cfg, k) for k, _ in _Cfg._fields_})
        self.h = self.lib.ks_model_create(ctx.h, C.byref(c))
        if not self.h:
            raise KsError(_lib.ERR_INVALID, self.lib.ks_last_error(ctx.h).decode(errors="replace"))

    @classmethod
    def synthetic(cls, ctx: CudaContext, cfg: ModelConfig, seed: int, keep: bool = False):
        """Random-init model from a seed; with keep=True also returns the host tensors."""
        m = cls(ctx, cfg)
        kept = {}
        for name, kind, rows, cols in tensor_specs(cfg):
            t = synth_tensor(cfg, seed, name, kind, rows, cols)
            m.upload_tensor(name, t)
            if keep:
                kept[name] = t
        return (m, kept) if keep else m

    def upload_tensor(self, name: str, data: np.ndarray, dtype: int | None = None):
        """ensure_weight (crates/ksearch_gemma/src/gemma_prim.rs:415-451).  dtype: the tensor's type in the file when
        it differs from the resident one (Q6_K / F16 / F32 matrices are requantised to Q4_K on the device)."""
        a = np.ascontiguousarray(data)
        if a.dtype == np.float32 and self.cfg.act == F16 and "norm" in name:
            a = a.astype(np.float16)
        if dtype is None:
            self.ctx.check(self.lib.ks_model_upload_tensor(self.h, name.encode(), a.ctypes.data, a.nbytes))
        else:
            self.ctx.check(self.lib.ks_model_upload_tensor_as(self.h, name.encode(), dtype, a.ctypes.data, a.nbytes))

    def warm_plans(self, n_tok: int = 1) -> int:
        """Load-time BEAM warm (gemma_prim.rs:254-290): search or load the launch plan of every matvec shape."""
        return self.lib.ks_model_warm_plans(self.h, n_tok)

    def weight_bytes(self) -> int:
        return self.lib.ks_model_weight_bytes(self.h)

    # -- slots (KvPool)
    def slot_alloc(self) -> int:
        s = self.lib.ks_model_slot_alloc(self.h)
        if s < 0:
            raise KsError(s, self.lib.ks_last_error(self.ctx.h).decode(errors="replace"))
        return s

    def slot_free(self, slot: int):
        self.ctx.check(self.lib.ks_model_slot_free(self.h, slot))

    def slot_reset(self, slot: int):
        self.ctx.check(self.lib.ks_model_slot_reset(self.h, slot))

    def seq_len(self, slot: int) -> int:
        n = self.lib.ks_model_slot_seq_len(self.h, slot)
        if n < 0:
            raise KsError(n, "bad SlotId")
        return n

    def active_batch(self) -> int:
        return self.lib.ks_model_slot_active(self.h)

    # -- forward
    def forward(self, first: int, n: int, tokens, want_logits: bool):
        arr = None if tokens is None else (C.c_int * n)(*[int(t) for t in tokens])
        self.ctx.check(self.lib.ks_model_forward(self.h, first, n, arr, int(want_logits)))

    def prefill(self, slot: int, tokens):
        """Prompt tokens without logits, eight per pass over the weights (prefill_chunk, gemma_prim.rs:1305-1315)."""
        toks = [int(t) for t in tokens]
        arr = (C.c_int * max(1, len(toks)))(*toks)
        self.ctx.check(self.lib.ks_model_prefill(self.h, slot, arr, len(toks)))

    def decode_token(self, tokens, first: int = 0):
        toks = [int(t) for t in np.atleast_1d(tokens)]
        n = len(toks)
        out = (C.c_int * n)()
        self.ctx.check(self.lib.ks_model_decode_token(self.h, first, n, (C.c_int * n)(*toks), out))
        return list(out)

    def generate_timed(self, prompt, n_new: int, slot: int = 0, max_inflight: int = 1):
        p = (C.c_int * len(prompt))(*[int(t) for t in prompt])
        out = (C.c_int * max(1, n_new))()
        st = GenStats()
        self.ctx.check(self.lib.ks_model_generate(self.h, slot, p, len(prompt), n_new, max_inflight, out, C.byref(st)))
        return list(out)[:n_new], st

    def read_debug(self, which: int, slot: int = 0) -> np.ndarray:
        n = self.cfg.hidden if which == 0 else self.cfg.vocab
        ptr = self.lib.ks_model_debug_ptr(self.h, which, slot)
        nb = n * (4 if self.cfg.act == F32 else 2)
        buf = self.lib.ks_buf_wrap(self.ctx.h, ptr, nb)
        out = np.empty(nb, np.uint8)
        self.ctx.check(self.lib.ks_buf_download(self.ctx.h, buf, 0, out.ctypes.data, nb))
        self.lib.ks_buf_free(self.ctx.h, buf)
        return out.view(np.float32 if self.cfg.act == F32 else np.float16).astype(np.float32)

    def load_gguf(self, g):
        """Every tensor of the model out of an open Gguf (ks_model_load_gguf): uploads by GGUF name, requantises
        Q6_K / F16 / F32 matrices to Q4_K on the device as the reference's loader does on the host."""
        self.ctx.check(self.lib.ks_model_load_gguf(self.h, g.h))

    def read_tensor(self, name: str) -> np.ndarray:
        """The resident bytes of a tensor (after any load-time requantisation)."""
        nb = self.lib.ks_model_tensor_bytes(self.h, name.encode())
        ptr = self.lib.ks_model_tensor_ptr(self.h, name.encode())
        if not ptr or not nb:
            raise KsError(-1, f"missing tensor {name}")
        buf = self.lib.ks_buf_wrap(self.ctx.h, ptr, nb)
        out = np.empty(nb, np.uint8)
        self.ctx.check(self.lib.ks_buf_download(self.ctx.h, buf, 0, out.ctypes.data, nb))
        self.lib.ks_buf_free(self.ctx.h, buf)
        return out

    POLL_LIMIT, STALL, SPLIT_FROM, PHASE_CLOCKS = 0, 1, 2, 3

    def debug_set(self, what: int, value: int, slot: int = 0):
        """Knobs of the slot's persistent decode kernel (ks_model_debug_set)."""
        self.ctx.check(self.lib.ks_model_debug_set(self.h, slot, what, value))

    def phase_clocks(self, slot: int = 0) -> np.ndarray:
        """SM clock stamps of the last token, int64 [2 (first, last block)][n_layers][5 (qkv, attention, o-proj,
        gate-up, down)][8]; matvec phases: entered, inputs arrived, x staged, tasks done, block joined, row stored
        (6 used); attention: entered, q arrived, q/k/v built, positions done, folded, -,
        stored, left.  Recorded only after debug_set(PHASE_CLOCKS, 1) or with KSEARCH_PROFILE set
        (gemma_prim.rs:885)."""
        ptr = self.lib.ks_model_debug_ptr(self.h, 2, slot)
        if not ptr:
            raise KsError(_lib.ERR_STATE, "the persistent decode kernel has not run for this slot")
        n = 2 * self.cfg.n_layers * 5 * 8
        buf = self.lib.ks_buf_wrap(self.ctx.h, ptr, n * 8)
        out = np.empty(n, np.int64)
        self.ctx.check(self.lib.ks_buf_download(self.ctx.h, buf, 0, out.ctypes.data, n * 8))
        self.lib.ks_buf_free(self.ctx.h, buf)
        return out.reshape(2, self.cfg.n_layers, 5, 8)

    def _kv_buf(self, layer: int, which: int, slot: int):
        ptr = self.lib.ks_model_kv_ptr(self.h, layer, which, slot)
        if not ptr:
            raise KsError(_lib.ERR_STATE, "bad layer / slot")
        return self.lib.ks_buf_wrap(self.ctx.h, ptr, self.lib.ks_model_kv_slot_bytes(self.h))

    def read_kv(self, layer: int, which: int, slot: int = 0, nbytes: int | None = None) -> np.ndarray:
        """One slot's rows of a layer's K (which=0) or V (which=1) cache, packed Q4_0 bytes."""
        nb = self.lib.ks_model_kv_slot_bytes(self.h) if nbytes is None else nbytes
        buf = self._kv_buf(layer, which, slot)
        out = np.empty(nb, np.uint8)
        self.ctx.check(self.lib.ks_buf_download(self.ctx.h, buf, 0, out.ctypes.data, nb))
        self.lib.ks_buf_free(self.ctx.h, buf)
        return out

    def write_kv(self, layer: int, which: int, data: np.ndarray, slot: int = 0):
        """Overwrite the first len(data) bytes of one slot's K or V rows of a layer (restoring a snapshot)."""
        a = np.ascontiguousarray(data, dtype=np.uint8)
        buf = self._kv_buf(layer, which, slot)
        self.ctx.check(self.lib.ks_buf_upload(self.ctx.h, buf, 0, a.ctypes.data, a.nbytes))
        self.lib.ks_buf_free(self.ctx.h, buf)

    def close(self):
        if self.h:
            self.lib.ks_model_destroy(self.h)
            self.h = None
