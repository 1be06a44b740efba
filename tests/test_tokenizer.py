"""build_tokenizer_from_gguf (crates/ksearch_gguf/src/tokenizer.rs:11-94) over a small vocabulary written into a GGUF
file: pieces, merges, byte fallback, special tokens, the BOS template and the Metaspace round trip.  CPU only."""
import pytest

from ksearch_b200 import KsError
from ksearch_b200.chat import gemma4_chat_prompt
from ksearch_b200.gguf import Gguf
from ksearch_b200.tokenizer import TOKEN_BYTE, TOKEN_CONTROL, TOKEN_NORMAL, TOKEN_USER_DEFINED, build_tokenizer_from_gguf, encode_prompt
from tests import gguf_writer as W

SP = "▁"


def _vocab():
    toks = ["<pad>", "<eos>", "<bos>", "<unk>", "<|turn>", "<turn|>"]
    types = [TOKEN_CONTROL, TOKEN_CONTROL, TOKEN_CONTROL, 2, TOKEN_USER_DEFINED, TOKEN_USER_DEFINED]
    toks += [f"<0x{b:02X}>" for b in range(256)]
    types += [TOKEN_BYTE] * 256
    pieces = [SP, "h", "i", "e", "l", "o", "w", "r", "d", "u", "s", "m", "\n", "hi", "he", "ll", "hell", "hello", SP + "w", "or", "ld",
              SP + "wor", SP + "world", "us", "er", "user", "mo", "de", "mode", "model"]
    toks += pieces
    types += [TOKEN_NORMAL] * len(pieces)
    merges = ["h i", "h e", "l l", "he ll", "hell o", SP + " w", "o r", "l d", SP + "w or", SP + "wor ld", "u s", "e r", "us er",
              "m o", "d e", "mo de", "mode l"]
    return toks, types, merges


def _write(tmp_path, extra=(), drop=()):
    toks, types, merges = _vocab()
    md = [("tokenizer.ggml.model", W.STR, "gemma4"), ("tokenizer.ggml.tokens", W.ARR, (W.STR, toks)),
          ("tokenizer.ggml.merges", W.ARR, (W.STR, merges)), ("tokenizer.ggml.token_type", W.ARR, (W.I32, types)),
          ("tokenizer.ggml.unknown_token_id", W.U32, 3), ("tokenizer.ggml.bos_token_id", W.U32, 2)]
    md = [m for m in md if m[0] not in drop] + list(extra)
    p = tmp_path / "tok.gguf"
    W.write_gguf(p, md, [])
    return p, toks


def test_encode_decode_specials_and_bos(tmp_path):
    p, toks = _write(tmp_path)
    with Gguf(p) as g:
        tok = build_tokenizer_from_gguf(g)
    ids = encode_prompt(tok, "hello world")
    assert [toks[i] for i in ids] == ["<bos>", "hello", SP + "world"]          # BOS template, merges, the space as a metaspace
    assert tok.decode(ids, skip_special_tokens=True) == "hello world"
    assert encode_prompt(tok, "hello world", add_special=False) == ids[1:]
    # a character outside the vocabulary falls back to its UTF-8 bytes; the reference installs only a Metaspace decoder
    # (tokenizer.rs:63), so byte tokens decode as their literal names, and so do they here
    ids = encode_prompt(tok, "hi é", add_special=False)
    assert [toks[i] for i in ids] == ["hi", SP, "<0xC3>", "<0xA9>"]
    assert tok.decode(ids) == "hi <0xC3><0xA9>"
    # the chat template's turn markers are single (user-defined) tokens, never split into pieces
    ids = encode_prompt(tok, gemma4_chat_prompt("hi"))
    names = [toks[i] for i in ids]
    assert names[:2] == ["<bos>", "<|turn>"] and names.count("<|turn>") == 2 and names.count("<turn|>") == 1
    assert "user" in names and "model" in names and "hi" in names


def test_options_and_refusals(tmp_path):
    p, toks = _write(tmp_path, extra=[("tokenizer.ggml.add_bos_token", W.BOOL, 0), ("tokenizer.ggml.add_space_prefix", W.BOOL, 1)])
    with Gguf(p) as g:
        tok = build_tokenizer_from_gguf(g)
    ids = encode_prompt(tok, "world")
    assert [toks[i] for i in ids] == [SP + "world"]                           # no BOS; a space is put in front of the first word
    assert tok.decode(ids) == "world"
    for drop, extra, msg in ((("tokenizer.ggml.tokens",), (), "tokens missing"), (("tokenizer.ggml.merges",), (), "merges missing"),
                             (("tokenizer.ggml.model",), (("tokenizer.ggml.model", W.STR, "gpt2"),), "unexpected tokenizer.ggml.model 'gpt2'")):
        p, _ = _write(tmp_path, extra=extra, drop=drop)
        with Gguf(p) as g, pytest.raises(KsError, match=msg):
            build_tokenizer_from_gguf(g)
