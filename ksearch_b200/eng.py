"""Host-side mirror of the reference's device runtime and op interface.

``CudaContext`` stands in for ``MetalContext`` (crates/ksearch_metal/src/lib.rs)
and ``Eng`` for ``ksearch_kernels::Eng`` (crates/ksearch_kernels/src/lib.rs):
same method names, argument order and meaning, errors raised where the
reference returns ``Err``.  Every call goes through the C ABI of
libksearch_cuda.so; nothing here computes.

Differences from the reference, all deliberate:
  * activations may be f32 (``Eng(ctx, act=F32)``, the default) or f16 (the
    reference's only mode);
  * the attention ops take a ``scale`` (the reference hard-wires 1);
  * ``matvec_batch`` accepts 1..8 tokens and streams the weights once.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import F16, F32, Q4K, Q6K, Q40  # noqa: F401  (re-exported)

ACT_NP = {F32: np.float32, F16: np.float16}


class KsError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"[{code}] {msg}")
        self.code = code
        self.msg = msg


def q40_row_bytes(hd: int) -> int:
    """crates/ksearch_ir/src/lib.rs:52-59"""
    return hd // 32 * 18


def q40_nbytes(rows: int, hd: int) -> int:
    return rows * q40_row_bytes(hd)


def q4k_nbytes(rows: int, cols: int) -> int:
    """crates/ksearch_ir/src/lib.rs:61-64"""
    return rows * (cols // 256) * 144


def q6k_nbytes(rows: int, cols: int) -> int:
    """crates/ksearch_ir/src/lib.rs:71-74"""
    return rows * (cols // 256) * 210


class Buffer:
    """Device memory handle (``metal::Buffer`` in the reference)."""

    def __init__(self, ctx: "CudaContext", handle: int, nbytes: int):
        self.ctx = ctx
        self.h = handle
        self.nbytes = nbytes

    @property
    def ptr(self) -> int:
        return self.ctx.lib.ks_buf_device_ptr(self.h)

    def free(self):
        if self.h:
            self.ctx.lib.ks_buf_free(self.ctx.h, self.h)
            self.h = None

    def __del__(self):
        try:
            if self.h and self.ctx.h:
                self.free()
        except Exception:
            pass


class CudaContext:
    """One GPU, one stream; enqueue-only ops, explicit flush / wait / synchronize."""

    def __init__(self, device: int = 0, flags: int = 0):
        self.lib = _lib.load()
        self.h = self.lib.ks_ctx_create(device, flags)
        if not self.h:
            raise KsError(_lib.ERR_UNSUPPORTED, self.lib.ks_last_error(None).decode(errors="replace"))

    # -- errors
    def check(self, rc: int):
        if rc != 0:
            raise KsError(rc, self.lib.ks_last_error(self.h).decode(errors="replace"))

    def device_name(self) -> str:
        return self.lib.ks_chip_name(self.h).decode()

    @property
    def sm_count(self) -> int:
        return self.lib.ks_ctx_sm_count(self.h)

    @property
    def stream(self) -> int:
        return self.lib.ks_ctx_stream(self.h)

    def launch_count(self) -> int:
        return self.lib.ks_ctx_launch_count(self.h)

    # -- buffers (M:63-135)
    def buffer_empty_bytes(self, nbytes: int) -> Buffer:
        h = self.lib.ks_buf_alloc(self.h, nbytes)
        if not h:
            raise KsError(_lib.ERR_OOM, self.lib.ks_last_error(self.h).decode(errors="replace"))
        return Buffer(self, h, nbytes)

    def buffer_empty_f32(self, n: int) -> Buffer:
        return self.buffer_empty_bytes(n * 4)

    def buffer_empty_f16(self, n: int) -> Buffer:
        return self.buffer_empty_bytes(n * 2)

    def buffer_bytes(self, data) -> Buffer:
        a = np.ascontiguousarray(data)
        b = self.buffer_empty_bytes(a.nbytes)
        self.write_buffer(b, a)
        return b

    def write_buffer(self, buf: Buffer, data, byte_off: int = 0):
        a = np.ascontiguousarray(data)
        self.check(self.lib.ks_buf_upload(self.h, buf.h, byte_off, a.ctypes.data, a.nbytes))

    def read_bytes(self, buf: Buffer, nbytes: int | None = None, byte_off: int = 0) -> np.ndarray:
        n = buf.nbytes - byte_off if nbytes is None else nbytes
        out = np.empty(n, np.uint8)
        self.check(self.lib.ks_buf_download(self.h, buf.h, byte_off, out.ctypes.data, n))
        return out

    def read_f32(self, buf: Buffer, n: int, off: int = 0) -> np.ndarray:
        return self.read_bytes(buf, n * 4, off * 4).view(np.float32)

    def read_f16(self, buf: Buffer, n: int, off: int = 0) -> np.ndarray:
        return self.read_bytes(buf, n * 2, off * 2).view(np.float16)

    def read_act(self, buf: Buffer, n: int, act: int, off: int = 0) -> np.ndarray:
        return (self.read_f32(buf, n, off) if act == F32 else self.read_f16(buf, n, off).astype(np.float32))

    def buffer_act(self, data, act: int) -> Buffer:
        return self.buffer_bytes(np.asarray(data, dtype=ACT_NP[act]))

    # -- ordering (M:157-218)
    def flush_async(self):
        self.check(self.lib.ks_flush(self.h))

    def wait_inflight_at_most(self, n: int):
        self.check(self.lib.ks_wait_inflight_at_most(self.h, n))

    def synchronize(self):
        self.check(self.lib.ks_synchronize(self.h))

    def has_gpu_work(self) -> bool:
        return bool(self.lib.ks_has_gpu_work(self.h))

    # -- device stopwatch and plan override
    def timer_begin(self):
        self.check(self.lib.ks_timer_begin(self.h))

    def timer_end_ms(self) -> float:
        ms = C.c_float()
        self.check(self.lib.ks_timer_end_ms(self.h, C.byref(ms)))
        return float(ms.value)

    def plan_override(self, plan: "_lib.Plan | None"):
        self.check(self.lib.ks_plan_override(self.h, C.byref(plan) if plan is not None else None))

    # -- whole-token replay
    def graph_begin(self):
        self.check(self.lib.ks_graph_begin(self.h))

    def graph_end(self) -> int:
        g = self.lib.ks_graph_end(self.h)
        if not g:
            raise KsError(_lib.ERR_CUDA, self.lib.ks_last_error(self.h).decode(errors="replace"))
        return g

    def graph_launch(self, g: int):
        self.check(self.lib.ks_graph_launch(self.h, g))

    def graph_free(self, g: int):
        self.lib.ks_graph_free(self.h, g)

    def close(self):
        if self.h:
            self.lib.ks_ctx_destroy(self.h)
            self.h = None


class Eng:
    """The op interface of the decode path (crates/ksearch_kernels/src/lib.rs)."""

    SDPA_MWG_NWG = 16          # K:1114
    SDPA_MWG_THRESHOLD = 128   # K:1115

    def __init__(self, act: int = F32):
        if act not in (F32, F16):
            raise ValueError("activation dtype must be F32 or F16")
        self.act = act

    # ---- matvec family ----------------------------------------------------
    def matvec_wd(self, ctx, rows, cols, weight_dtype, a, x, y):
        """K:137"""
        ctx.check(ctx.lib.ks_matvec(ctx.h, rows, cols, weight_dtype, a.h, 0, self.act, x.h, 0, y.h, 0, 1))

    def matvec_wd_at(self, ctx, rows, cols, weight_dtype, a, x, x_off_elems, y, y_off_elems):
        """K:1446"""
        ctx.check(ctx.lib.ks_matvec(ctx.h, rows, cols, weight_dtype, a.h, 0, self.act, x.h, x_off_elems, y.h, y_off_elems, 1))

    def matvec_batch(self, ctx, rows, cols, batch, weight_dtype, a, x, y):
        """K:1414 (batch <= 8: token-looped GEMV family; 9..256 rows: the tensor-core GEMM, the reference's mul_mm route)"""
        ctx.check(ctx.lib.ks_matvec(ctx.h, rows, cols, weight_dtype, a.h, 0, self.act, x.h, 0, y.h, 0, batch))

    def matvec_qkv_wds(self, ctx, q_rows, kv_rows, cols, wq_dtype, wk_dtype, wv_dtype, wq, wk, wv, x, q, k, v):
        """K:227"""
        ctx.check(ctx.lib.ks_matvec_qkv(ctx.h, q_rows, kv_rows, cols, wq_dtype, wk_dtype, wv_dtype, wq.h, wk.h, wv.h,
                                        self.act, x.h, q.h, k.h, v.h))

    def matvec_qkv_wd(self, ctx, q_rows, kv_rows, cols, weight_dtype, wq, wk, wv, x, q, k, v):
        """K:193"""
        self.matvec_qkv_wds(ctx, q_rows, kv_rows, cols, weight_dtype, weight_dtype, weight_dtype, wq, wk, wv, x, q, k, v)

    def matvec_gate_up_gelu_wd(self, ctx, rows, cols, weight_dtype, w_gate, w_up, x, y):
        """K:953"""
        ctx.check(ctx.lib.ks_matvec_gate_up_gelu(ctx.h, rows, cols, weight_dtype, w_gate.h, w_up.h, self.act, x.h, y.h))

    # ---- RMSNorm fused into the following matvec (optionally with the residual update in front)
    @staticmethod
    def _h(b):
        return None if b is None else b.h

    def rmsnorm_matvec_wd(self, ctx, rows, cols, eps, weight_dtype, x, w_norm, a, y, y_prev=None, w_post=None, out_x=None):
        """K:278"""
        ctx.check(ctx.lib.ks_rmsnorm_matvec(ctx.h, rows, cols, eps, weight_dtype, self.act, x.h, w_norm.h, a.h, y.h,
                                            self._h(y_prev), self._h(w_post), self._h(out_x)))

    def rmsnorm_matvec_qkv_wd(self, ctx, q_rows, kv_rows, cols, eps, weight_dtype, x, w_norm, wq, wk, wv, q, k, v,
                              y_prev=None, w_post=None, out_x=None):
        """K:341"""
        ctx.check(ctx.lib.ks_rmsnorm_matvec_qkv(ctx.h, q_rows, kv_rows, cols, eps, weight_dtype, self.act, x.h, w_norm.h,
                                                wq.h, wk.h, wv.h, q.h, k.h, v.h, self._h(y_prev), self._h(w_post),
                                                self._h(out_x)))

    def rmsnorm_matvec_gate_up_gelu_wd(self, ctx, rows, cols, eps, weight_dtype, x, w_norm, w_gate, w_up, y,
                                       y_prev=None, w_post=None, out_x=None):
        """K:1004"""
        ctx.check(ctx.lib.ks_rmsnorm_matvec_gate_up_gelu(ctx.h, rows, cols, eps, weight_dtype, self.act, x.h, w_norm.h,
                                                         w_gate.h, w_up.h, y.h, self._h(y_prev), self._h(w_post),
                                                         self._h(out_x)))

    # ---- RMSNorm family ---------------------------------------------------
    def rmsnorm(self, ctx, n, eps, x, w, y):
        """K:456"""
        self.rmsnorm_at(ctx, n, eps, x, 0, w, y, 0)

    def rmsnorm_at(self, ctx, n, eps, x, x_off_elems, w, y, y_off_elems):
        """K:468"""
        ctx.check(ctx.lib.ks_rmsnorm(ctx.h, n, 1, eps, self.act, x.h, x_off_elems, w.h, None, 0, 0, 0.0, y.h, y_off_elems))

    def rmsnorm_add(self, ctx, n, eps, x, w, residual, y):
        """K:492"""
        ctx.check(ctx.lib.ks_rmsnorm(ctx.h, n, 1, eps, self.act, x.h, 0, w.h, residual.h, 0, 0, 0.0, y.h, 0))

    def rmsnorm_add_scale(self, ctx, n, eps, scale, x, w, residual, y):
        """K:514"""
        ctx.check(ctx.lib.ks_rmsnorm(ctx.h, n, 1, eps, self.act, x.h, 0, w.h, residual.h, 0, 1, scale, y.h, 0))

    def rmsnorm_rows(self, ctx, n, rows, eps, x, w, y):
        """K:1478"""
        ctx.check(ctx.lib.ks_rmsnorm(ctx.h, n, rows, eps, self.act, x.h, 0, w.h, None, 0, 0, 0.0, y.h, 0))

    def rmsnorm_add_rows(self, ctx, n, rows, eps, x, w, residual, y):
        """K:1502"""
        ctx.check(ctx.lib.ks_rmsnorm(ctx.h, n, rows, eps, self.act, x.h, 0, w.h, residual.h, 0, 0, 0.0, y.h, 0))

    def rmsnorm_add_then_rmsnorm(self, ctx, n, eps, y, w_post, residual, w_ffn, out_x, out_x2):
        """K:539"""
        ctx.check(ctx.lib.ks_rmsnorm_add_then_rmsnorm(ctx.h, n, 1, eps, self.act, y.h, w_post.h, residual.h, w_ffn.h,
                                                      out_x.h, out_x2.h))

    def rmsnorm_add_then_rmsnorm_rows(self, ctx, n, rows, eps, y, w_post, residual, w_ffn, out_x, out_x2):
        """K:1561"""
        ctx.check(ctx.lib.ks_rmsnorm_add_then_rmsnorm(ctx.h, n, rows, eps, self.act, y.h, w_post.h, residual.h, w_ffn.h,
                                                      out_x.h, out_x2.h))

    def rmsnorm_per_head_qkv_q40_off(self, ctx, n_q, n_kv, hd, eps, q, qw, cos_sin, cos_sin_off_elems, k, kw, v,
                                     q_out, kv_k, kv_v, kv_byte_off):
        """K:1257"""
        ctx.check(ctx.lib.ks_rmsnorm_per_head_qkv_q40(ctx.h, n_q, n_kv, hd, 1, eps, self.act, q.h, qw.h, cos_sin.h,
                                                      cos_sin_off_elems, k.h, kw.h, v.h, q_out.h, kv_k.h, kv_v.h,
                                                      kv_byte_off))

    def rmsnorm_per_head_qkv_q40_batch(self, ctx, n_q, n_kv, hd, n_tok, eps, q, qw, cos_sin, cos_sin_off_elems, k, kw,
                                       v, q_out, kv_k, kv_v, kv_byte_off):
        """K:1750"""
        ctx.check(ctx.lib.ks_rmsnorm_per_head_qkv_q40(ctx.h, n_q, n_kv, hd, n_tok, eps, self.act, q.h, qw.h, cos_sin.h,
                                                      cos_sin_off_elems, k.h, kw.h, v.h, q_out.h, kv_k.h, kv_v.h,
                                                      kv_byte_off))

    # ---- attention --------------------------------------------------------
    def sdpa_tmp_floats(self, n_q, hd, n_splits, n_slots=1) -> int:
        return _lib.load().ks_sdpa_tmp_floats(n_slots, n_q, hd, n_splits)

    def sdpa_decode(self, ctx, n_slots, n_q, n_kv, hd, max_t, q, k, v, meta, tmp, out, scale=1.0, n_splits=0,
                    kv_byte_off=0, slot_stride_bytes=0, kv_dtype=Q40):
        ctx.check(ctx.lib.ks_sdpa_decode(ctx.h, n_slots, n_q, n_kv, hd, max_t, kv_dtype, scale, self.act, q.h, k.h, v.h,
                                         kv_byte_off, slot_stride_bytes, meta.h, tmp.h if tmp is not None else None,
                                         out.h, n_splits))

    def sdpa_naive_kv(self, ctx, n_q, n_kv, hd, max_t, kv_dtype, q, k, v, meta, out, scale=1.0):
        """K:1086: single pass, no partitions."""
        self.sdpa_decode(ctx, 1, n_q, n_kv, hd, max_t, q, k, v, meta, None, out, scale, 1, kv_dtype=kv_dtype)

    def sdpa_mwg_kv(self, ctx, n_q, n_kv, hd, max_t, kv_dtype, q, k, v, meta, tmp, out, scale=1.0):
        """K:1118: SDPA_MWG_NWG partitions + merge; tmp is f32 [n_q * NWG * (hd + 2)]."""
        self.sdpa_decode(ctx, 1, n_q, n_kv, hd, max_t, q, k, v, meta, tmp, out, scale, self.SDPA_MWG_NWG, kv_dtype=kv_dtype)

    def sdpa_hybrid_kv(self, ctx, n_q, n_kv, hd, max_t, attn_t, kv_dtype, q, k, v, meta, tmp, out, scale=1.0):
        """K:1157"""
        if attn_t >= self.SDPA_MWG_THRESHOLD:
            self.sdpa_mwg_kv(ctx, n_q, n_kv, hd, max_t, kv_dtype, q, k, v, meta, tmp, out, scale)
        else:
            self.sdpa_naive_kv(ctx, n_q, n_kv, hd, max_t, kv_dtype, q, k, v, meta, out, scale)

    # ---- small ops --------------------------------------------------------
    def quantize_q40(self, ctx, n, src, dst, dst_byte_off):
        """K:1181"""
        ctx.check(ctx.lib.ks_quantize_q40(ctx.h, n, self.act, src.h, 0, dst.h, dst_byte_off))

    def copy_scale_indexed_wd(self, ctx, n, scale, dtype, src, idx, dst):
        """K:1364"""
        ctx.check(ctx.lib.ks_copy_scale_indexed(ctx.h, n, 1, scale, dtype, src.h, idx.h, 0, self.act, dst.h))

    def copy_scale_indexed_batch_wd(self, ctx, n, batch, scale, dtype, src, idx, dst):
        """K:1387"""
        ctx.check(ctx.lib.ks_copy_scale_indexed(ctx.h, n, batch, scale, dtype, src.h, idx.h, 0, self.act, dst.h))

    def softcap_argmax(self, ctx, n, cap, logits, out_idx):
        """K:1966"""
        ctx.check(ctx.lib.ks_softcap_argmax(ctx.h, n, cap, self.act, logits.h, out_idx.h, 0))

    def gelu_mul(self, ctx, n, g, u, y):
        """K:695"""
        ctx.check(ctx.lib.ks_gelu_mul(ctx.h, n, self.act, g.h, u.h, y.h))

    # ---- test hook ----------------------------------------------------------
    def dequant(self, ctx, dtype, src, nelem, dst, src_byte_off=0, dst_off=0):
        """crates/ksearch_gguf/src/gguf_impl.rs:577-794 (Q4_0, Q4_K, Q6_K, F16)"""
        ctx.check(ctx.lib.ks_dequant(ctx.h, dtype, src.h, src_byte_off, nelem, dst.h, dst_off))


    # ---- load-time requantisation ---------------------------------------------
    def quantize_q4k(self, ctx, src_dtype, src, nelem, dst, src_byte_off=0, dst_byte_off=0):
        """crates/ksearch_gguf/src/gguf_impl.rs:803-1016 quantize_f32_to_q4k over the dequantised source, as
        crates/ksearch_gemma/src/gemma_prim.rs:415-440 applies it to Q6_K ffn_down / attn_v tensors at load."""
        ctx.check(ctx.lib.ks_quantize_q4k(ctx.h, src_dtype, src.h, src_byte_off, nelem, dst.h, dst_byte_off))


def write_meta(ctx: CudaContext, meta: Buffer, tlen: int, start: int = 0, win: int = 0, slot: int = 0):
    """Host write of (tlen, start, win) as f32 (crates/ksearch_gemma/src/gemma_prim.rs:636-644)."""
    ctx.write_buffer(meta, np.array([tlen, start, win, 0], np.float32), slot * 16)
