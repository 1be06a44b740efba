"""From a GGUF file to served tokens: the load and request path of the reference's `serve` command
(crates/ksearch_cli/src/serve.rs:224-249 builds model, pool and scheduler; gemma_prim.rs:149-183 the model) over
this library — GGUF reader, config, device model, tokenizer, chat template, scheduler.  No HTTP here.

`dense_model_config` maps the file's GemmaConfig onto the model this build runs and says which of the file's
features are not built yet instead of loading something that would compute the wrong thing."""
from __future__ import annotations

from . import _lib
from .chat import gemma4_chat_from_messages
from .eng import CudaContext, KsError
from .gguf import GGML_Q4_K, GGML_Q6_K, GemmaConfig, Gguf
from .model import GemmaCudaModel, ModelConfig
from .scheduler import InferenceRequest, Scheduler, SchedulerConfig
from .tokenizer import build_tokenizer_from_gguf, encode_prompt


def dense_model_config(g: Gguf, gc: GemmaConfig, max_seq: int, n_slots: int, attn_scale: float = 1.0) -> ModelConfig:
    """The ModelConfig of a file whose layers this build can run: one head dim, one FFN width, every layer with its
    own KV, no per-layer embeddings.  attn_scale: the reference's attention uses 1 (its q is scaled by the norm weights)."""
    missing = []
    full = [l for l in range(gc.n_layers) if not gc.swa_pattern[l]]
    if full and gc.head_dim_full != gc.head_dim_swa:
        missing.append(f"full-attention layers with their own head dim ({gc.head_dim_full} vs {gc.head_dim_swa}) and RoPE table")
    if gc.shared_kv_layers:
        missing.append(f"{gc.shared_kv_layers} shared-KV layers")
    if len(set(gc.ffn)) != 1:
        missing.append("per-layer feed-forward widths")
    if g.has_tensor("per_layer_token_embd.weight") or g.has_tensor("per_layer_model_proj.weight"):
        missing.append("per-layer embeddings")
    if gc.n_layers > 64 and any(gc.swa_pattern):
        missing.append("more than 64 layers with a sliding-window pattern")
    if missing:
        raise KsError(_lib.ERR_UNSUPPORTED, "this file needs what is not built yet: " + "; ".join(missing))
    embd = g.tensor("token_embd.weight").ggml_type
    if embd not in (GGML_Q4_K, GGML_Q6_K):
        raise KsError(_lib.ERR_UNSUPPORTED, f"token_embd.weight of ggml type {embd}: Q4_K or Q6_K expected")
    swa = sum(1 << l for l in range(gc.n_layers) if gc.swa_pattern[l])
    window = gc.sliding_window if swa and gc.sliding_window < max_seq else 0
    return ModelConfig(gc.n_layers, gc.hidden, gc.ffn[0], gc.n_heads, gc.n_kv, gc.head_dim_swa, gc.vocab, max_seq, n_slots,
                       eps=gc.rms_eps, rope_theta=gc.rope_theta_swa if swa else gc.rope_theta_full, softcap=gc.softcap,
                       attn_scale=attn_scale, embd_dtype=_lib.Q4K if embd == GGML_Q4_K else _lib.Q6K,
                       sliding_window=window, swa_layers=swa if window else 0)


class Server:
    """Model, tokenizer and scheduler of one GGUF file on one GPU."""

    def __init__(self, path: str, ctx: CudaContext | None = None, max_seq: int = 4096, slots: int = 4, attn_scale: float = 1.0):
        self.ctx = ctx or CudaContext(0, flags=1)
        with Gguf(path) as g:
            self.gemma = GemmaConfig.from_gguf(g)
            self.cfg = dense_model_config(g, self.gemma, min(max_seq, self.gemma.context_length), slots, attn_scale)
            self.tokenizer = build_tokenizer_from_gguf(g)
            self.model = GemmaCudaModel(self.ctx, self.cfg)
            self.model.load_gguf(g)
        self.scheduler = Scheduler(self.model, SchedulerConfig(slots=slots), detokenize=lambda t: self.tokenizer.decode([t], skip_special_tokens=False))

    def submit(self, messages, max_tokens: int = 64, temperature: float = 0.0, min_p: float = 0.05, seed: int = 1, stop=()):
        """messages: (role, content) pairs; returns the request (its `events` fill as the scheduler runs)."""
        ids = encode_prompt(self.tokenizer, gemma4_chat_from_messages(messages), True)
        req = InferenceRequest(ids, max_tokens=max_tokens, stop=list(stop), temperature=temperature, min_p=min_p, seed=seed)
        self.scheduler.submit(req)
        return req

    def complete(self, messages, **kw) -> str:
        req = self.submit(messages, **kw)
        self.scheduler.run()
        err = [e for e in req.events if e[0] == "error"]
        if err:
            raise KsError(_lib.ERR_STATE, err[0][1])
        return self.tokenizer.decode([e[1] for e in req.events if e[0] == "token"], skip_special_tokens=True)

    def close(self):
        self.model.close()
