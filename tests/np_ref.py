"""Independent NumPy statements of the block formats, written from the format
definitions (GGUF Q4_0 / Q4_K / Q6_K), not from the C oracle.  The tests use
them to cross-check the oracle: two implementations that agree bit for bit.
"""
import numpy as np


def half_to_f32(bits):
    return np.asarray(bits, np.uint16).view(np.float16).astype(np.float32)


def scale_min_k4(q):
    """q: [nb, 12] uint8 -> (sc [nb, 8], m [nb, 8]) as uint8."""
    q = q.astype(np.uint8)
    sc = np.empty(q.shape[:-1] + (8,), np.uint8)
    m = np.empty_like(sc)
    for j in range(8):
        if j < 4:
            sc[..., j] = q[..., j] & 63
            m[..., j] = q[..., j + 4] & 63
        else:
            sc[..., j] = (q[..., j + 4] & 0x0F) | ((q[..., j - 4] >> 6) << 4)
            m[..., j] = (q[..., j + 4] >> 4) | ((q[..., j] >> 6) << 4)
    return sc, m


def dequant_q4k(data, nelem):
    nb = nelem // 256
    blk = np.asarray(data, np.uint8)[: nb * 144].reshape(nb, 144)
    d = half_to_f32(blk[:, 0:2].copy().view(np.uint16)[:, 0])
    dmin = half_to_f32(blk[:, 2:4].copy().view(np.uint16)[:, 0])
    sc, m = scale_min_k4(blk[:, 4:16])
    qs = blk[:, 16:144].reshape(nb, 4, 32)
    out = np.empty((nb, 4, 2, 32), np.float32)
    for g in range(4):
        for hi in range(2):
            j = 2 * g + hi
            dj = (d * sc[:, j].astype(np.float32)).astype(np.float32)
            mj = (dmin * m[:, j].astype(np.float32)).astype(np.float32)
            nib = (qs[:, g, :] >> 4) if hi else (qs[:, g, :] & 0x0F)
            prod = (dj[:, None] * nib.astype(np.float32)).astype(np.float32)
            out[:, g, hi, :] = (prod - mj[:, None]).astype(np.float32)
    return out.reshape(-1)


def dequant_q5k(data, nelem):
    """crates/ksearch_gguf/src/gguf_impl.rs:722-760, vectorised over blocks."""
    nb = nelem // 256
    blk = np.asarray(data, np.uint8)[: nb * 176].reshape(nb, 176)
    d = half_to_f32(blk[:, 0:2].copy().view(np.uint16)[:, 0])
    dmin = half_to_f32(blk[:, 2:4].copy().view(np.uint16)[:, 0])
    sc, m = scale_min_k4(blk[:, 4:16])
    qh = blk[:, 16:48]
    qs = blk[:, 48:176].reshape(nb, 4, 32)
    out = np.empty((nb, 4, 2, 32), np.float32)
    for g in range(4):
        for hi in range(2):
            j = 2 * g + hi
            dj = (d * sc[:, j].astype(np.float32)).astype(np.float32)
            mj = (dmin * m[:, j].astype(np.float32)).astype(np.float32)
            nib = (qs[:, g, :] >> 4) if hi else (qs[:, g, :] & 0x0F)
            q = nib.astype(np.float32) + np.where((qh >> j) & 1, np.float32(16.0), np.float32(0.0))
            out[:, g, hi, :] = ((dj[:, None] * q).astype(np.float32) - mj[:, None]).astype(np.float32)
    return out.reshape(-1)


def dequant_q6k(data, nelem):
    nb = nelem // 256
    blk = np.asarray(data, np.uint8)[: nb * 210].reshape(nb, 210)
    ql = blk[:, 0:128].reshape(nb, 2, 64)
    qh = blk[:, 128:192].reshape(nb, 2, 32)
    sc = blk[:, 192:208].view(np.int8).reshape(nb, 2, 8)
    d = half_to_f32(blk[:, 208:210].copy().view(np.uint16)[:, 0])
    out = np.empty((nb, 2, 4, 32), np.float32)
    l = np.arange(32)
    isx = l // 16
    for h in range(2):
        for k in range(4):
            qlb = ql[:, h, (k & 1) * 32:(k & 1) * 32 + 32]
            lo4 = (qlb >> 4) if (k & 2) else (qlb & 0x0F)
            hi2 = (qh[:, h, :] >> (2 * k)) & 3
            q = (lo4 | (hi2 << 4)).astype(np.int32) - 32
            s = sc[:, h, isx + 2 * k].astype(np.float32)
            ds = (d[:, None] * s).astype(np.float32)
            out[:, h, k, :] = (ds * q.astype(np.float32)).astype(np.float32)
    return out.reshape(-1)


def dequant_q40(data, nelem):
    nb = nelem // 32
    blk = np.asarray(data, np.uint8)[: nb * 18].reshape(nb, 18)
    d = half_to_f32(blk[:, 0:2].copy().view(np.uint16)[:, 0])
    qs = blk[:, 2:18]
    lo = (qs & 0x0F).astype(np.int32) - 8
    hi = (qs >> 4).astype(np.int32) - 8
    out = np.concatenate([lo, hi], axis=1).astype(np.float32) * d[:, None]
    return out.astype(np.float32).reshape(-1)


def attention(q, Kf, Vf, n_q, n_kv, hd, scale):
    """softmax(scale * q K^T) V in f64. Kf, Vf: [t, n_kv, hd] dequantised."""
    g = n_q // n_kv
    out = np.empty((n_q, hd))
    for h in range(n_q):
        kh = h // g
        s = (Kf[:, kh, :].astype(np.float64) @ q[h].astype(np.float64)) * scale
        p = np.exp(s - s.max())
        p /= p.sum()
        out[h] = p @ Vf[:, kh, :].astype(np.float64)
    return out.reshape(-1)


def rmsnorm(x, w, eps):
    x = x.astype(np.float64)
    return x / np.sqrt((x * x).mean() + eps) * (1.0 if w is None else w.astype(np.float64))
