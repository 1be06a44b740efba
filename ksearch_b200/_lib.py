"""Loads libksearch_cuda.so and declares the C ABI of include/ksearch_cuda.h.

There is no fallback: if the library is missing this raises, and creating a
context on a machine without an sm_100 GPU fails with the library's message.
"""
from __future__ import annotations

import ctypes as C
import os
import re

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libksearch_cuda.so")
HEADER = os.path.join(os.path.dirname(PKG), "include", "ksearch_cuda.h")

F32, F16, Q4K, Q6K, Q40, Q5K = 0, 1, 2, 3, 4, 5
OK, ERR_INVALID, ERR_CUDA, ERR_OOM, ERR_UNSUPPORTED, ERR_STATE, ERR_TIMEOUT = 0, -1, -2, -3, -4, -5, -6

_sz, _i, _f, _vp, _u64 = C.c_size_t, C.c_int, C.c_float, C.c_void_p, C.c_uint64

# name -> (restype, argtypes)
SIGNATURES = {
    "ks_ctx_create": (_vp, [_i, _u64]),
    "ks_ctx_destroy": (None, [_vp]),
    "ks_last_error": (C.c_char_p, [_vp]),
    "ks_chip_name": (C.c_char_p, [_vp]),
    "ks_ctx_device": (_i, [_vp]),
    "ks_ctx_sm_count": (_i, [_vp]),
    "ks_ctx_stream": (_vp, [_vp]),
    "ks_ctx_launch_count": (_u64, [_vp]),
    "ks_buf_alloc": (_vp, [_vp, _sz]),
    "ks_buf_free": (None, [_vp, _vp]),
    "ks_buf_size": (_sz, [_vp]),
    "ks_buf_device_ptr": (_vp, [_vp]),
    "ks_buf_wrap": (_vp, [_vp, _vp, _sz]),
    "ks_buf_upload": (_i, [_vp, _vp, _sz, _vp, _sz]),
    "ks_buf_download": (_i, [_vp, _vp, _sz, _vp, _sz]),
    "ks_buf_upload_async": (_i, [_vp, _vp, _sz, _vp, _sz]),
    "ks_buf_download_async": (_i, [_vp, _vp, _sz, _vp, _sz]),
    "ks_buf_zero": (_i, [_vp, _vp, _sz, _sz]),
    "ks_host_alloc_pinned": (_vp, [_sz]),
    "ks_host_free_pinned": (None, [_vp]),
    "ks_flush": (_i, [_vp]),
    "ks_wait_inflight_at_most": (_i, [_vp, _i]),
    "ks_synchronize": (_i, [_vp]),
    "ks_has_gpu_work": (_i, [_vp]),
    "ks_timer_begin": (_i, [_vp]),
    "ks_timer_end_ms": (_i, [_vp, C.POINTER(C.c_float)]),
    "ks_graph_begin": (_i, [_vp]),
    "ks_graph_end": (_vp, [_vp]),
    "ks_graph_launch": (_i, [_vp, _vp]),
    "ks_graph_free": (None, [_vp, _vp]),
    "ks_plan_override": (_i, [_vp, _vp]),
    "ks_plan_set": (_i, [_vp, C.c_char_p, _sz, _sz, _i, _vp]),
    "ks_plan_get": (_i, [_vp, C.c_char_p, _sz, _sz, _i, _vp]),
    "ks_plan_search": (_i, [_vp, C.c_char_p, _sz, _sz, _sz, _i, _vp]),
    "ks_plan_candidates": (_i, [C.c_char_p, _vp, _i]),
    "ks_plan_file_name": (_i, [C.c_char_p, C.c_char_p, C.c_char_p, _sz]),
    "ks_plan_file_save": (_i, [C.c_char_p, C.c_char_p, C.c_char_p, _vp]),
    "ks_plan_file_load": (_i, [C.c_char_p, C.c_char_p, C.c_char_p, _vp]),
    "ks_dequant": (_i, [_vp, _i, _vp, _sz, _sz, _vp, _sz]),
    "ks_quantize_q4k": (_i, [_vp, _i, _vp, _sz, _sz, _vp, _sz]),
    "ks_matvec": (_i, [_vp, _sz, _sz, _i, _vp, _sz, _i, _vp, _sz, _vp, _sz, _i]),
    "ks_matvec_qkv": (_i, [_vp, _sz, _sz, _sz, _i, _i, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp]),
    "ks_matvec_gate_up_gelu": (_i, [_vp, _sz, _sz, _i, _vp, _vp, _i, _vp, _vp]),
    "ks_rmsnorm_matvec": (_i, [_vp, _sz, _sz, _f, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "ks_rmsnorm_matvec_qkv": (_i, [_vp, _sz, _sz, _sz, _f, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "ks_rmsnorm_matvec_gate_up_gelu": (_i, [_vp, _sz, _sz, _f, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "ks_matvec_host": (_i, [_vp, _sz, _sz, _i, _vp, _sz, _vp, _vp, _i]),
    "ks_rmsnorm": (_i, [_vp, _sz, _sz, _f, _i, _vp, _sz, _vp, _vp, _sz, _i, _f, _vp, _sz]),
    "ks_rmsnorm_add_then_rmsnorm": (_i, [_vp, _sz, _sz, _f, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "ks_rmsnorm_per_head_qkv_q40": (_i, [_vp, _sz, _sz, _sz, _sz, _f, _i, _vp, _vp, _vp, _sz, _vp, _vp, _vp, _vp, _vp, _vp, _sz]),
    "ks_sdpa_tmp_floats": (_sz, [_sz, _sz, _sz, _i]),
    "ks_sdpa_pick_splits": (_i, [_vp, _sz, _sz, _sz]),
    "ks_sdpa_decode": (_i, [_vp, _sz, _sz, _sz, _sz, _sz, _i, _f, _i, _vp, _vp, _vp, _sz, _sz, _vp, _vp, _vp, _i]),
    "ks_quantize_q40": (_i, [_vp, _sz, _i, _vp, _sz, _vp, _sz]),
    "ks_copy_scale_indexed": (_i, [_vp, _sz, _sz, _f, _i, _vp, _vp, _sz, _i, _vp]),
    "ks_softcap_argmax": (_i, [_vp, _sz, _f, _i, _vp, _vp, _sz]),
    "ks_softcap_argmax_noalloc": (_i, [_i, _vp, _sz, _f, _vp, _vp]),
    "ks_gelu_mul": (_i, [_vp, _sz, _i, _vp, _vp, _vp]),
    "ks_model_create": (_vp, [_vp, _vp]),
    "ks_model_destroy": (None, [_vp]),
    "ks_model_warm_plans": (_i, [_vp, _i]),
    "ks_model_tensor_bytes": (_sz, [_vp, C.c_char_p]),
    "ks_model_upload_tensor": (_i, [_vp, C.c_char_p, _vp, _sz]),
    "ks_model_upload_tensor_as": (_i, [_vp, C.c_char_p, _i, _vp, _sz]),
    "ks_model_load_gguf": (_i, [_vp, _vp]),
    "ks_sample_softcap_min_p": (C.c_uint32, [_vp, _sz, _f, _f, _f, C.c_uint32]),
    "ks_sample_softcap_min_p_f32": (C.c_uint32, [_vp, _sz, _f, _f, _f, C.c_uint32]),
    "ks_gguf_open": (_vp, [C.c_char_p, C.c_char_p, _sz]),
    "ks_gguf_close": (None, [_vp]),
    "ks_gguf_version": (_i, [_vp]),
    "ks_gguf_n_tensors": (_sz, [_vp]),
    "ks_gguf_n_kv": (_sz, [_vp]),
    "ks_gguf_data_offset": (C.c_uint64, [_vp]),
    "ks_gguf_tensor_name": (C.c_char_p, [_vp, _sz]),
    "ks_gguf_tensor": (_i, [_vp, C.c_char_p, _vp, _vp, _vp, _vp, _vp]),
    "ks_gguf_tensor_raw": (_vp, [_vp, C.c_char_p]),
    "ks_gguf_has_key": (_i, [_vp, C.c_char_p]),
    "ks_gguf_get_u32": (_i, [_vp, C.c_char_p, _vp]),
    "ks_gguf_get_u64": (_i, [_vp, C.c_char_p, _vp]),
    "ks_gguf_get_f32": (_i, [_vp, C.c_char_p, _vp]),
    "ks_gguf_get_bool": (_i, [_vp, C.c_char_p, _vp]),
    "ks_gguf_get_str": (C.c_char_p, [_vp, C.c_char_p]),
    "ks_gguf_arr_len": (C.c_longlong, [_vp, C.c_char_p, _vp]),
    "ks_gguf_get_arr_u32": (C.c_longlong, [_vp, C.c_char_p, _vp, _sz]),
    "ks_gguf_get_arr_i32": (C.c_longlong, [_vp, C.c_char_p, _vp, _sz]),
    "ks_gguf_get_arr_f32": (C.c_longlong, [_vp, C.c_char_p, _vp, _sz]),
    "ks_gguf_get_arr_bool": (C.c_longlong, [_vp, C.c_char_p, _vp, _sz]),
    "ks_gguf_get_arr_str": (C.c_char_p, [_vp, C.c_char_p, _sz]),
    "ks_model_tensor_ptr": (_vp, [_vp, C.c_char_p]),
    "ks_model_weight_bytes": (_sz, [_vp]),
    "ks_model_slot_alloc": (_i, [_vp]),
    "ks_model_slot_free": (_i, [_vp, _i]),
    "ks_model_slot_reset": (_i, [_vp, _i]),
    "ks_model_slot_seq_len": (_i, [_vp, _i]),
    "ks_model_slot_active": (_i, [_vp]),
    "ks_model_forward": (_i, [_vp, _i, _i, _vp, _i]),
    "ks_model_prefill": (_i, [_vp, _i, _vp, _i]),
    "ks_model_decode_token": (_i, [_vp, _i, _i, _vp, _vp]),
    "ks_model_generate": (_i, [_vp, _i, _vp, _i, _i, _i, _vp, _vp]),
    "ks_model_debug_ptr": (_vp, [_vp, _i, _i]),
    "ks_model_debug_set": (_i, [_vp, _i, _i, C.c_uint]),
    "ks_comm_unique_id": (_i, [_vp]),
    "ks_comm_init": (_vp, [_vp, _i, _i, _vp]),
    "ks_comm_destroy": (None, [_vp]),
    "ks_comm_p2p_handle": (_i, [_vp, _vp]),
    "ks_comm_p2p_open": (_i, [_vp, _vp]),
    "ks_comm_set": (_i, [_vp, _i, C.c_uint]),
    "ks_comm_rank": (_i, [_vp]),
    "ks_comm_size": (_i, [_vp]),
    "ks_comm_all_gather_f32": (_i, [_vp, _vp, _sz, _sz]),
    "ks_matvec_sharded": (_i, [_vp, _sz, _sz, _sz, _i, _vp, _sz, _vp, _sz, _vp, _sz, _i]),
    "ks_argmax_sharded": (_i, [_vp, _sz, _sz, _f, _vp, _sz, _vp, _sz]),
    "ks_model_kv_ptr": (_vp, [_vp, _i, _i, _i]),
    "ks_model_kv_slot_bytes": (_sz, [_vp]),
}



class Plan(C.Structure):
    """ks_plan of include/ksearch_cuda.h"""
    _fields_ = [("variant", _i), ("nr", _i), ("nwarps", _i), ("ctas_per_sm", _i), ("ms", _f)]


_lib = None


def header_symbols() -> list[str]:
    """Every function the public header declares."""
    with open(HEADER) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ks_[a-z0-9_]+)\s*\(", text)))


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m ksearch_b200.build` "
                "(there is no CPU fallback for this backend)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
