"""CPU decoder of the oracle: deterministic, honours max_seq, matches a NumPy restatement
of one layer stack on a tiny model."""
import numpy as np
import pytest

from ksearch_b200 import model as ksm
from ksearch_b200 import synth
from tests import np_ref


def _np_forward(cfg, T, oracle, tokens):
    """Straight NumPy f64 transformer over the same packed tensors (full recompute per token)."""
    H, hd, nq, nkv = cfg.hidden, cfg.hd, cfg.n_q, cfg.n_kv
    deq = lambda name, dt, r, c: oracle.dequant(dt, T[name], r * c).reshape(r, c).astype(np.float64)
    emb = deq("token_embd.weight", cfg.embd_dtype, cfg.vocab, H)
    rope = oracle.rope_table(cfg.max_seq, hd, cfg.rope_theta).astype(np.float64)
    half = hd // 2
    Ks = [[] for _ in range(cfg.n_layers)]
    Vs = [[] for _ in range(cfg.n_layers)]
    logits = None
    for pos, tok in enumerate(tokens):
        x = np.sqrt(np.float32(H)).astype(np.float64) * emb[tok]
        for l in range(cfg.n_layers):
            p = f"blk.{l}."
            h = np_ref.rmsnorm(x, T[p + "attn_norm.weight"], cfg.eps)
            q = deq(p + "attn_q.weight", synth.Q4K, nq * hd, H) @ h
            k = deq(p + "attn_k.weight", synth.Q4K, nkv * hd, H) @ h
            v = deq(p + "attn_v.weight", synth.Q4K, nkv * hd, H) @ h
            c, s = rope[pos, :half], rope[pos, half:]

            def rot(vec, w):
                y = np_ref.rmsnorm(vec, w, cfg.eps)
                return np.concatenate([y[:half] * c - y[half:] * s, y[:half] * s + y[half:] * c])

            qh = np.stack([rot(q[i * hd:(i + 1) * hd], T[p + "attn_q_norm.weight"]) for i in range(nq)])
            kh = np.stack([rot(k[i * hd:(i + 1) * hd], T[p + "attn_k_norm.weight"]) for i in range(nkv)])
            vh = np.stack([np_ref.rmsnorm(v[i * hd:(i + 1) * hd], None, cfg.eps) for i in range(nkv)])
            # the cache holds Q4_0-rounded rows
            kq = oracle.dequant(synth.Q40, oracle.pack_q40(kh.astype(np.float32), True), nkv * hd).reshape(nkv, hd)
            vq = oracle.dequant(synth.Q40, oracle.pack_q40(vh.astype(np.float32), True), nkv * hd).reshape(nkv, hd)
            Ks[l].append(kq)
            Vs[l].append(vq)
            # a sliding-window layer attends to the last `sliding_window` positions (gemma_prim.rs:1009-1016)
            lo = max(0, len(Ks[l]) - cfg.sliding_window) if cfg.sliding_window and (cfg.swa_layers >> l) & 1 else 0
            o = np_ref.attention(qh, np.stack(Ks[l][lo:]), np.stack(Vs[l][lo:]), nq, nkv, hd, cfg.attn_scale)
            a = deq(p + "attn_output.weight", synth.Q4K, H, nq * hd) @ o
            x = x + np_ref.rmsnorm(a, T[p + "post_attention_norm.weight"], cfg.eps)
            h2 = np_ref.rmsnorm(x, T[p + "ffn_norm.weight"], cfg.eps)
            g = deq(p + "ffn_gate.weight", synth.Q4K, cfg.ffn, H) @ h2
            u = deq(p + "ffn_up.weight", synth.Q4K, cfg.ffn, H) @ h2
            gc = np.clip(g, -20, 20)
            ff = 0.5 * gc * (1 + np.tanh(0.79788456 * (gc + 0.044715 * gc ** 3))) * u
            d = deq(p + "ffn_down.weight", synth.Q4K, H, cfg.ffn) @ ff
            x = x + np_ref.rmsnorm(d, T[p + "post_ffw_norm.weight"], cfg.eps)
        logits = emb @ np_ref.rmsnorm(x, T["output_norm.weight"], cfg.eps)
    return logits


def test_cpu_decoder_matches_numpy_and_is_deterministic(oracle):
    cfg = ksm.tiny_config(max_seq=8)
    cfg.n_layers = 2
    T = ksm.synth_tensors(cfg, 3)
    dec = oracle.CpuDecoder(oracle.decoder_cfg(cfg), T)
    toks = [5, 77, 1024]
    for i, t in enumerate(toks):
        nxt = dec.forward_token(t, i == len(toks) - 1)
    got = dec.logits().astype(np.float64)
    want = _np_forward(cfg, T, oracle, toks)
    scale = np.abs(want).max()
    # the two differ only through Q4_0 rounding decisions on values that sit on a boundary
    assert np.abs(got - want).max() < 2e-2 * scale
    assert nxt == int(np.argmax(got))
    a = dec.generate([1, 2, 3], 4)
    b = dec.generate([1, 2, 3], 4)
    assert a == b and len(a) == 4
    dec.close()


def test_cpu_decoder_sliding_window_layers(oracle):
    """Layers flagged in swa_layers attend to the last sliding_window positions only (gemma_prim.rs:1009-1016):
    against the NumPy restatement, and against the full-attention decoder (equal while the context fits the
    window, different beyond)."""
    cfg = ksm.tiny_config(max_seq=12)
    cfg.n_layers = 2
    T = ksm.synth_tensors(cfg, 6)
    toks = [9, 300, 41, 1500, 7, 7, 88, 1023]
    full = oracle.CpuDecoder(oracle.decoder_cfg(cfg), T)
    cfg.sliding_window, cfg.swa_layers = 3, 0b01          # layer 0 slides, layer 1 is full
    win = oracle.CpuDecoder(oracle.decoder_cfg(cfg), T)
    for i, t in enumerate(toks):
        full.forward_token(t, True)
        win.forward_token(t, True)
        same = np.array_equal(full.logits(), win.logits())
        assert same == (i < 3), i
    got = win.logits().astype(np.float64)
    want = _np_forward(cfg, T, oracle, toks)
    assert np.abs(got - want).max() < 2e-2 * np.abs(want).max()
    cfg.sliding_window = 64                                # a window longer than the cache changes nothing
    wide = oracle.CpuDecoder(oracle.decoder_cfg(cfg), T)
    for t in toks:
        wide.forward_token(t, True)
    assert np.array_equal(wide.logits(), full.logits())
    for d in (full, win, wide):
        d.close()


def test_cpu_decoder_max_seq(oracle):
    cfg = ksm.tiny_config(max_seq=3)
    cfg.n_layers = 1
    dec = oracle.CpuDecoder(oracle.decoder_cfg(cfg), ksm.synth_tensors(cfg, 4))
    for t in (1, 2, 3):
        dec.forward_token(t, False)
    with pytest.raises(RuntimeError, match="max_seq exceeded"):
        dec.forward_token(4, False)
    dec.close()


def test_model_byte_accounting():
    """1,027,031,040 B per token for the E2B shape, 2,718,105,600 B for the E4B shape."""
    assert ksm.weight_bytes_per_token(ksm.e2b_config()) == 1_027_031_040
    assert ksm.weight_bytes_per_token(ksm.e4b_config()) == 2_718_105_600
