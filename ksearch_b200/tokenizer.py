"""The tokenizer of the serve surface, built from the `tokenizer.ggml.*` metadata of a GGUF file as
crates/ksearch_gguf/src/tokenizer.rs:11-94 builds it — with the same HuggingFace `tokenizers` library the reference
links (its Python binding here): byte-fallback BPE over the file's vocabulary and merges, Metaspace pre-tokenizer and
decoder, control / user-defined tokens registered as special, a BOS template when the file asks for one."""
from __future__ import annotations

from .eng import KsError
from . import _lib

TOKEN_NORMAL, TOKEN_UNKNOWN, TOKEN_CONTROL, TOKEN_USER_DEFINED, TOKEN_UNUSED, TOKEN_BYTE = 1, 2, 3, 4, 5, 6   # gguf_impl.rs:492-499
MODELS = ("gemma4", "llama", "gemma", "gemma3")


def build_tokenizer_from_gguf(g):
    """g: ksearch_b200.gguf.Gguf.  Returns a tokenizers.Tokenizer."""
    from tokenizers import AddedToken, Tokenizer, decoders, pre_tokenizers, processors
    from tokenizers.models import BPE
    model = g.get_str("tokenizer.ggml.model") or ""
    if model not in MODELS:
        raise KsError(_lib.ERR_UNSUPPORTED, f"unexpected tokenizer.ggml.model '{model}'")
    tokens = g.get_arr_str("tokenizer.ggml.tokens")
    if tokens is None:
        raise KsError(_lib.ERR_INVALID, "tokenizer.ggml.tokens missing")
    merges = g.get_arr_str("tokenizer.ggml.merges")
    if merges is None:
        raise KsError(_lib.ERR_INVALID, "tokenizer.ggml.merges missing")
    types = g.get_arr_i32("tokenizer.ggml.token_type")
    vocab = {t: i for i, t in enumerate(tokens)}                                   # a repeated piece keeps its last id
    pairs = [tuple(m.split(" ", 1)) for m in merges if " " in m]
    unk_id = g.get_u32("tokenizer.ggml.unknown_token_id")
    unk = tokens[unk_id] if unk_id is not None and unk_id < len(tokens) else "<unk>"
    try:
        tok = Tokenizer(BPE(vocab=vocab, merges=pairs, unk_token=unk, byte_fallback=True, fuse_unk=True))
    except Exception as e:
        raise KsError(_lib.ERR_INVALID, f"BPE build failed: {e}")
    scheme = "first" if g.get_bool("tokenizer.ggml.add_space_prefix") else "never"
    tok.pre_tokenizer = pre_tokenizers.Metaspace(replacement="▁", prepend_scheme=scheme, split=True)
    tok.decoder = decoders.Metaspace(replacement="▁", prepend_scheme=scheme, split=True)
    if types is not None:
        specials = [AddedToken(t, special=True) for i, t in enumerate(tokens)
                    if i < len(types) and types[i] in (TOKEN_CONTROL, TOKEN_USER_DEFINED)]
        tok.add_special_tokens(specials)
    add_bos = g.get_bool("tokenizer.ggml.add_bos_token")
    if add_bos is None or add_bos:
        bos_id = g.get_u32("tokenizer.ggml.bos_token_id")
        if bos_id is not None and bos_id < len(tokens):
            bos = tokens[bos_id]
            tok.post_processor = processors.TemplateProcessing(single=f"{bos} $A", special_tokens=[(bos, bos_id)])
    return tok


def encode_prompt(tok, text: str, add_special: bool = True) -> list:
    """tokenizer.rs:136-141"""
    return list(tok.encode(text, add_special_tokens=add_special).ids)
