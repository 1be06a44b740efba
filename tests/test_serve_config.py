"""dense_model_config: which GGUF files this build can run, and what it says about the others.  CPU only."""
import numpy as np
import pytest

from ksearch_b200 import KsError, Q4K, Q6K
from ksearch_b200.gguf import GGML_F16, GGML_Q4_K, GGML_Q6_K, GemmaConfig, Gguf
from ksearch_b200.serve import dense_model_config
from tests import gguf_writer as W


def _md(**over):
    md = {"general.architecture": (W.STR, "gemma4"), "gemma4.block_count": (W.U32, 3), "gemma4.embedding_length": (W.U32, 512),
          "gemma4.attention.head_count": (W.U32, 4), "gemma4.attention.head_count_kv": (W.U32, 1),
          "gemma4.attention.key_length": (W.U32, 128), "gemma4.attention.key_length_swa": (W.U32, 128),
          "gemma4.feed_forward_length": (W.U32, 1024), "gemma4.attention.sliding_window": (W.U32, 16),
          "gemma4.attention.sliding_window_pattern": (W.ARR, (W.BOOL, [1, 0, 1])), "gemma4.context_length": (W.U32, 256)}
    md.update(over)
    return [(k, v[0], v[1]) for k, v in md.items() if v is not None]


def _cfg(tmp_path, md, tensors=None, max_seq=64):
    tensors = tensors if tensors is not None else [("token_embd.weight", GGML_Q6_K, (512, 8), np.zeros(8 * 2 * 210, np.uint8))]
    p = tmp_path / "c.gguf"
    W.write_gguf(p, md, tensors)
    with Gguf(p) as g:
        return dense_model_config(g, GemmaConfig.from_gguf(g), max_seq, 2)


def test_a_file_this_build_runs(tmp_path):
    c = _cfg(tmp_path, _md())
    assert (c.n_layers, c.hidden, c.ffn, c.n_q, c.n_kv, c.hd, c.vocab, c.max_seq, c.n_slots) == (3, 512, 1024, 4, 1, 128, 8, 64, 2)
    assert (c.sliding_window, c.swa_layers, c.embd_dtype, c.attn_scale, c.softcap) == (16, 0b101, Q6K, 1.0, 30.0)
    assert c.rope_theta == 10_000.0                                         # the sliding-window layers' base
    wide = _cfg(tmp_path, _md(**{"gemma4.attention.sliding_window": (W.U32, 512)}))
    assert (wide.sliding_window, wide.swa_layers) == (0, 0)                 # a window longer than the cache is no window
    q4 = _cfg(tmp_path, _md(), [("token_embd.weight", GGML_Q4_K, (512, 8), np.zeros(8 * 2 * 144, np.uint8))])
    assert q4.embd_dtype == Q4K


def test_files_that_need_more(tmp_path):
    cases = [
        (_md(**{"gemma4.attention.key_length": (W.U32, 512)}), None, "own head dim"),
        (_md(**{"gemma4.attention.shared_kv_layers": (W.U32, 2)}), None, "shared-KV"),
        (_md(**{"gemma4.feed_forward_length": (W.ARR, (W.U32, [1024, 2048, 1024]))}), None, "feed-forward widths"),
        (_md(), [("token_embd.weight", GGML_Q6_K, (512, 8), np.zeros(8 * 2 * 210, np.uint8)),
                 ("per_layer_token_embd.weight", GGML_F16, (256, 8), np.zeros(256 * 8, np.float16))], "per-layer embeddings"),
        (_md(), [("token_embd.weight", GGML_F16, (512, 8), np.zeros(512 * 8, np.float16))], "Q4_K or Q6_K expected"),
    ]
    for md, tensors, msg in cases:
        with pytest.raises(KsError, match=msg):
            _cfg(tmp_path, md, tensors)
    # the real E2B shape of the reference's table (two head dims, shared KV, per-layer embeddings) names all of it at once
    md = _md(**{"gemma4.attention.key_length": (W.U32, 512), "gemma4.attention.shared_kv_layers": (W.U32, 1)})
    with pytest.raises(KsError) as ei:
        _cfg(tmp_path, md)
    assert "own head dim" in str(ei.value) and "shared-KV" in str(ei.value)
