"""The GGUF reader (crates/ksearch_gguf/src/gguf_impl.rs:130-417) against files written by tests/gguf_writer.py:
header, every metadata value type with the reference's coercions, tensor infos, alignment, raw tensor bytes, and
the errors the reference raises as panics.  Host code: runs without a GPU."""
import struct

import numpy as np
import pytest

from ksearch_b200 import KsError, synth
from ksearch_b200.gguf import GGML_F16, GGML_F32, GGML_Q4_K, GGML_Q6_K, GemmaConfig, Gguf
from tests import gguf_writer as W


def _file(tmp_path, **kw):
    md = [
        ("general.architecture", W.STR, "gemma4"),
        ("gemma4.block_count", W.U32, 3),
        ("gemma4.embedding_length", W.U64, 512),            # U64 where a U32 is asked for
        ("gemma4.attention.head_count", W.I32, 4),           # I32 where a U32 is asked for
        ("gemma4.attention.head_count_kv", W.ARR, (W.I32, [2])),
        ("gemma4.attention.layer_norm_rms_epsilon", W.F64, 1e-5),   # F64 where an F32 is asked for
        ("gemma4.feed_forward_length", W.ARR, (W.U32, [1024, 1024, 2048])),
        ("gemma4.attention.sliding_window_pattern", W.ARR, (W.BOOL, [1, 1, 0])),
        ("small.u8", W.U8, 200), ("small.i8", W.I8, -5), ("small.u16", W.U16, 65000), ("small.i16", W.I16, -300),
        ("small.bool", W.BOOL, 1), ("big.i64", W.I64, -(1 << 40)), ("f.f32", W.F32, 0.25),
        ("tokenizer.ggml.tokens", W.ARR, (W.STR, ["<pad>", "a", "bé"])),
        ("tokenizer.ggml.scores", W.ARR, (W.F32, [0.0, -1.5, 2.0])),
        ("other.u16s", W.ARR, (W.U16, [1, 2, 3, 4, 5])),    # an array type the reader only counts
    ]
    q4 = synth.q4k_matrix(5, "a", 8, 512)
    q6 = synth.q6k_matrix(5, "b", 4, 256, signed_scales=True)
    f32 = synth.normals(5, "n", 512).astype(np.float32)
    f16 = synth.normals(5, "h", 96).astype(np.float16)
    tensors = [("blk.0.attn_q.weight", GGML_Q4_K, (512, 8), q4), ("token_embd.weight", GGML_Q6_K, (256, 4), q6),
               ("output_norm.weight", GGML_F32, (512,), f32), ("odd.f16", GGML_F16, (32, 3), f16)]
    path = tmp_path / "m.gguf"
    offs = W.write_gguf(path, md, tensors, **kw)
    return path, tensors, offs


@pytest.mark.parametrize("version,alignment", [(3, None), (2, None), (3, 64), (3, 4096)])
def test_open_and_read_everything(tmp_path, version, alignment):
    path, tensors, offs = _file(tmp_path, version=version, alignment=alignment)
    with Gguf(path) as g:
        assert g.version == version
        assert g.data_offset % (alignment or 32) == 0
        assert g.tensor_names() == [t[0] for t in tensors]            # file order
        for name, gt, dims, data in tensors:
            info = g.tensor(name)
            raw = np.ascontiguousarray(data).view(np.uint8).ravel()
            assert (info.ggml_type, info.dims, info.nbytes, info.file_offset) == (gt, tuple(dims), raw.size, offs[name])
            assert info.file_offset % (alignment or 32) == 0
            assert np.array_equal(g.tensor_raw(name), raw)
        assert g.tensor("token_embd.weight").n_rows() == 4
        # scalars and the coercions of get_u32 / get_u64 / get_f32
        assert g.get_str("general.architecture") == "gemma4"
        assert g.get_u32("gemma4.block_count") == 3 and g.get_u64("gemma4.block_count") == 3
        assert g.get_u32("gemma4.embedding_length") == 512 and g.get_u32("gemma4.attention.head_count") == 4
        assert g.get_u32("small.u16") == 65000 and g.get_u64("small.u16") is None
        assert g.get_u32("small.u8") is None and g.get_u32("f.f32") is None and g.get_u32("absent") is None
        assert g.get_f32("f.f32") == 0.25 and abs(g.get_f32("gemma4.attention.layer_norm_rms_epsilon") - 1e-5) < 1e-12
        assert g.get_f32("gemma4.block_count") is None
        assert g.get_bool("small.bool") is True and g.get_bool("small.u8") is None
        assert g.has_key("big.i64") and not g.has_key("nope")
        # arrays
        assert g.get_arr_u32("gemma4.feed_forward_length") == [1024, 1024, 2048]
        assert g.get_arr_i32("gemma4.attention.head_count_kv") == [2] and g.get_arr_u32("gemma4.attention.head_count_kv") is None
        assert g.get_usize_list("gemma4.attention.head_count_kv") == [2] and g.get_usize_list("gemma4.block_count") == [3]
        assert g.get_usize_list("f.f32") is None
        assert g.get_arr_bool("gemma4.attention.sliding_window_pattern") == [True, True, False]
        assert g.get_arr_str("tokenizer.ggml.tokens") == ["<pad>", "a", "bé"]
        assert g.get_arr_f32("tokenizer.ggml.scores") == [0.0, -1.5, 2.0]
        assert g.arr_len("other.u16s") == (5, W.U16) and g.get_arr_u32("other.u16s") is None
        assert g.arr_len("f.f32") is None
        assert g.n_kv() == 18 + (alignment is not None)
        with pytest.raises(KsError, match="tensor not found: nope"):
            g.tensor("nope")
        assert not g.has_tensor("nope") and g.has_tensor("odd.f16")


def test_config_from_gguf(tmp_path):
    path, _, _ = _file(tmp_path)
    with Gguf(path) as g:
        c = GemmaConfig.from_gguf(g)
    assert (c.n_layers, c.hidden, c.n_heads, c.n_kv, c.vocab) == (3, 512, 4, 2, 4)
    assert c.ffn == [1024, 1024, 2048] and c.swa_pattern == [True, True, False]
    assert abs(c.rms_eps - 1e-5) < 1e-12 and c.softcap == 30.0                       # a key in the file, a default
    assert (c.head_dim_swa, c.head_dim_full, c.sliding_window, c.shared_kv_layers, c.ple_dim) == (256, 512, 512, 0, 256)
    assert (c.rope_theta_full, c.rope_theta_swa, c.context_length) == (1_000_000.0, 10_000.0, 131072)
    # the refusals of from_gguf
    for md, msg in (([("general.architecture", W.STR, "llama")], "unsupported GGUF architecture"),
                    ([("gemma4.expert_count", W.U32, 8)], "MoE"),
                    ([("general.architecture", W.STR, "gemma4")], "block_count"),
                    ([("gemma4.block_count", W.U32, 2), ("gemma4.embedding_length", W.U32, 64),
                      ("gemma4.attention.head_count", W.U32, 4),
                      ("gemma4.attention.head_count_kv", W.ARR, (W.U32, [1, 2]))], "per-layer head_count_kv"),
                    ([("gemma4.block_count", W.U32, 2), ("gemma4.embedding_length", W.U32, 64),
                      ("gemma4.attention.head_count", W.U32, 4),
                      ("gemma4.attention.head_count_kv", W.U32, 3)], "not divisible")):
        p = tmp_path / "bad.gguf"
        W.write_gguf(p, md, [])
        with Gguf(p) as g, pytest.raises(KsError, match=msg):
            GemmaConfig.from_gguf(g)
    # defaults: one ffn width for every layer, the 5-local-1-global pattern
    p = tmp_path / "dflt.gguf"
    W.write_gguf(p, [("gemma4.block_count", W.U32, 7), ("gemma4.embedding_length", W.U32, 64),
                     ("gemma4.attention.head_count", W.U32, 4), ("gemma4.feed_forward_length", W.U32, 128)], [])
    with Gguf(p) as g:
        c = GemmaConfig.from_gguf(g)
    assert c.ffn == [128] * 7 and c.swa_pattern == [True] * 5 + [False, True] and c.n_kv == 1 and c.vocab == 262144


def test_open_errors(tmp_path):
    with pytest.raises(KsError, match="failed to open"):
        Gguf(tmp_path / "absent.gguf")
    p = tmp_path / "x.gguf"
    W.write_gguf(p, [], [], magic=0x46554746)
    with pytest.raises(KsError, match="bad magic"):
        Gguf(p)
    W.write_gguf(p, [], [], version=1)
    with pytest.raises(KsError, match="unsupported GGUF version 1"):
        Gguf(p)
    path, _, _ = _file(tmp_path)
    whole = path.read_bytes()
    for cut in (3, 12, 40, 300, 700):                     # inside the magic, the counts, a key, the metadata, the tensor infos
        p.write_bytes(whole[:cut])
        with pytest.raises(KsError, match="truncated|bad magic"):
            Gguf(p)
    with Gguf(path) as g:
        data_off = g.data_offset
    p.write_bytes(whole[:data_off + 64])                  # header intact, tensor data cut off
    with pytest.raises(KsError, match="lies outside the file"):
        Gguf(p)
    W.write_gguf(p, [], [("t", GGML_Q4_K, (100,), np.zeros(144, np.uint8))])
    with pytest.raises(KsError, match="not divisible by block 256"):
        Gguf(p)
    W.write_gguf(p, [("k", 99, 0)] if False else [], [("t", 5, (32,), np.zeros(64, np.uint8))])   # a ggml type the reader does not know
    with Gguf(p) as g:
        assert g.tensor("t").ggml_type == 5 and g.tensor("t").nbytes == 0
        with pytest.raises(KsError, match="unsupported ggml type id 5"):
            g.tensor_raw("t")
    # a metadata value type that does not exist
    head = struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + struct.pack("<Q", 1) + b"k" + struct.pack("<I", 77) + b"\0" * 64
    p.write_bytes(head)
    with pytest.raises(KsError, match="unexpected scalar value type 77"):
        Gguf(p)


def test_damaged_headers_are_refused_or_read_never_trusted(tmp_path):
    """Every truncation of the header and a few hundred random byte changes in it: the reader either refuses the file
    with an error or opens it and answers every query from inside the mapping (counts, lengths and offsets in the
    file are bounds-checked before use).  Strings that are no longer UTF-8 come back with replacement characters,
    as the reference's lossy conversion gives them (gguf_impl.rs:172)."""
    path, _, _ = _file(tmp_path)
    whole = path.read_bytes()
    with Gguf(path) as g:
        data_off = g.data_offset
    p = tmp_path / "d.gguf"
    for cut in range(0, data_off + 1, 5):
        p.write_bytes(whole[:cut])
        with pytest.raises(KsError):
            Gguf(p)
    rng = np.random.default_rng(7)
    opened = 0
    for _ in range(300):
        b = bytearray(whole)
        for _ in range(int(rng.integers(1, 4))):
            b[int(rng.integers(0, data_off))] = int(rng.integers(0, 256))
        p.write_bytes(bytes(b))
        try:
            g = Gguf(p)
        except KsError:
            continue
        with g:
            opened += 1
            for name in g.tensor_names():
                info = g.tensor(name) if g.has_tensor(name) else None
                if info is not None and info.nbytes:
                    assert info.file_offset + info.nbytes <= len(whole)
                    assert g.tensor_raw(name).size == info.nbytes
            for key in ("tokenizer.ggml.tokens", "gemma4.feed_forward_length", "general.architecture"):
                g.get_arr_str(key), g.get_usize_list(key), g.get_str(key)
            try:
                GemmaConfig.from_gguf(g)
            except KsError:
                pass
    assert 0 < opened < 300
