"""CPU tests of the oracle: against an independent NumPy statement of the block
formats, against the reference's own CPU test (q4k_roundtrip_approx), on the
reference's check_mul_mm input patterns, and against committed fixtures."""
import hashlib
import json
import os

import numpy as np
import pytest

from ksearch_b200 import synth
from tests import np_ref

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
Q4K, Q6K, Q40 = synth.Q4K, synth.Q6K, synth.Q40


def test_f16_to_f32_all_bit_patterns(oracle):
    bits = np.arange(65536, dtype=np.uint16)
    got = oracle.f16_to_f32(bits)
    want = bits.view(np.float16).astype(np.float32)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))


def test_f32_to_f16_rne_matches_ieee(oracle):
    rng = np.random.default_rng(1)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32) * np.float32(10.0) ** rng.integers(-8, 5, 200000).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 5.96e-8, 2.98e-8, 2.99e-8, 6.1e-5, np.inf, -np.inf], np.float32),
        bits_halfway(),
    ])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    got = oracle.f32_to_f16_rne(x)
    assert np.array_equal(got, want)


def bits_halfway():
    # exact ties between adjacent halves (normal and subnormal), both parities
    h = np.arange(0, 0x7BFF, 37, dtype=np.uint16)
    a = h.view(np.float16).astype(np.float64)
    b = (h + 1).astype(np.uint16).view(np.float16).astype(np.float64)
    return ((a + b) / 2).astype(np.float32)


def test_f32_to_f16_ref_rounds_half_up(oracle):
    """The reference's own converter adds 0x1000 (lib.rs:69): a tie goes UP even when
    ties-to-even would go down, and it agrees with RNE away from ties."""
    one_tie = np.array([1.0 + 2.0 ** -11], np.float32)   # halfway between 1.0 and next half; RNE -> 1.0 (even)
    assert oracle.f32_to_f16_rne(one_tie)[0] == 0x3C00
    assert oracle.f32_to_f16_ref(one_tie)[0] == 0x3C01
    rng = np.random.default_rng(2)
    x = (rng.standard_normal(50000) * 3).astype(np.float32)
    r, e = oracle.f32_to_f16_ref(x), oracle.f32_to_f16_rne(x)
    assert np.abs(r.astype(np.int32) - e.astype(np.int32)).max() <= 1
    assert (r != e).mean() < 1e-3
    assert oracle.f32_to_f16_ref(np.array([70000.0], np.float32))[0] == 0x7C00
    assert oracle.f32_to_f16_ref(np.array([-0.0], np.float32))[0] == 0x8000


def test_scale_min_k4_matches_numpy(oracle):
    import ctypes as C
    rng = np.random.default_rng(3)
    q = rng.integers(0, 256, (64, 12), dtype=np.uint8)
    sc, m = np_ref.scale_min_k4(q)
    L = oracle.lib()
    for b in range(64):
        for j in range(8):
            d, mm = C.c_uint8(), C.c_uint8()
            L.kso_scale_min_k4(j, q[b].ctypes.data_as(C.POINTER(C.c_uint8)), C.byref(d), C.byref(mm))
            assert (d.value, mm.value) == (sc[b, j], m[b, j])


@pytest.mark.parametrize("dtype,fn,gen", [
    (Q4K, np_ref.dequant_q4k, lambda: synth.q4k_matrix(7, "w", 8, 1024)),
    (Q6K, np_ref.dequant_q6k, lambda: synth.q6k_matrix(7, "w", 8, 1024)),
    (Q6K, np_ref.dequant_q6k, lambda: synth.q6k_matrix(7, "ws", 8, 1024, signed_scales=True)),
    (Q40, np_ref.dequant_q40, lambda: synth.q40_rows(7, "kv", 8 * 1024)),
    (5, np_ref.dequant_q5k, lambda: synth.q5k_matrix(7, "w5", 8, 1024)),
])
def test_dequant_bit_exact_vs_numpy(oracle, dtype, fn, gen):
    data = gen()
    got = oracle.dequant(dtype, data, 8 * 1024)
    want = fn(data, 8 * 1024)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_dequant_rejects_ragged(oracle):
    with pytest.raises(ValueError):
        oracle.dequant(Q4K, np.zeros(144, np.uint8), 100)
    assert oracle.dequant(Q4K, np.zeros(0, np.uint8), 0).size == 0


def test_q4k_hand_block(oracle):
    """One block worked by hand: d=2, dmin=0.5, sub-block j has scale j+1 and min 2j,
    nibbles lo=3, hi=12 -> value = 2*(j+1)*nib - 0.5*2j."""
    blk = np.zeros(144, np.uint8)
    blk[0:2] = np.array([0x4000], np.uint16).view(np.uint8)  # 2.0
    blk[2:4] = np.array([0x3800], np.uint16).view(np.uint8)  # 0.5
    sc = [j + 1 for j in range(8)]
    mn = [2 * j for j in range(8)]
    q = np.zeros(12, np.uint8)
    for j in range(8):
        if j < 4:
            q[j] = sc[j]
            q[j + 4] = mn[j]
        else:
            q[j + 4] = (sc[j] & 0xF) | ((mn[j] & 0xF) << 4)
            q[j - 4] |= (sc[j] >> 4) << 6
            q[j] |= (mn[j] >> 4) << 6
    blk[4:16] = q
    blk[16:144] = 3 | (12 << 4)
    got = oracle.dequant(Q4K, blk, 256)
    want = np.empty(256, np.float32)
    for g in range(4):
        want[64 * g:64 * g + 32] = 2.0 * sc[2 * g] * 3 - 0.5 * mn[2 * g]
        want[64 * g + 32:64 * g + 64] = 2.0 * sc[2 * g + 1] * 12 - 0.5 * mn[2 * g + 1]
    assert np.array_equal(got, want)


def _ref_signal():
    """The deterministic signal of q4k_roundtrip_approx (gguf_impl.rs:1024-1038)."""
    i = np.arange(256 * 4, dtype=np.float32)
    t = (np.sin((i * np.float32(0.017) + np.float32(0.3)).astype(np.float32)) * np.float32(1.7)
         + np.cos((i * np.float32(0.041)).astype(np.float32)) * np.float32(0.4) - np.float32(0.15)).astype(np.float32)
    t[256:512] = 0.0
    t[512:768] = -0.25
    return t


def test_q4k_roundtrip_approx(oracle):
    """The reference's own CPU test of the Q4_K quantizer/dequantizer pair, same thresholds."""
    elems = _ref_signal()
    q = oracle.quantize_q4k(elems)
    assert q.size == elems.size // 256 * 144
    back = oracle.dequant(Q4K, q, elems.size)
    assert back.size == elems.size
    e = np.abs(elems - back)
    assert float((e.astype(np.float64) ** 2).mean()) < 0.01
    assert float(e.max()) < 0.35
    assert np.all(back[256:512] == 0.0)
    # the quantizer's output decodes identically in the NumPy statement of the format
    assert np.array_equal(np_ref.dequant_q4k(q, elems.size), back)


def _mulmm_inputs(rows, cols, batch):
    """check_mul_mm.rs:48-59 integer patterns."""
    r = np.arange(rows)[:, None]
    c = np.arange(cols)[None, :]
    w = (((r * 17 + c * 13) % 200).astype(np.float32) - 100.0) * np.float32(0.02)
    t = np.arange(batch)[:, None]
    x = (((t * 11 + c * 7) % 50).astype(np.float32) - 25.0) * np.float32(0.04)
    return w.astype(np.float32), x.astype(np.float32)


@pytest.mark.parametrize("rows,cols,batch", [(64, 256, 16), (128, 256, 9), (256, 1536, 4)])
def test_matvec_on_reference_patterns(oracle, rows, cols, batch):
    """quantize -> dequant -> f32 dot, as check_mul_mm.rs:60-71; the f32 sums stay within
    f32 summation noise of the f64 sums, and the quantised matrix stays close to the input."""
    w, x = _mulmm_inputs(rows, cols, batch)
    wq = oracle.quantize_q4k(w.ravel())
    wd = oracle.dequant(Q4K, wq, rows * cols).reshape(rows, cols)
    assert np.abs(wd - w).max() < 0.15
    y32, y64 = oracle.matvec(Q4K, wq, rows, cols, x)
    want = x.astype(np.float64) @ wd.astype(np.float64).T
    assert np.allclose(y64, want, rtol=1e-12, atol=1e-9)
    scale = np.abs(want).max()
    assert np.abs(y32 - want).max() <= 1e-5 * scale * np.sqrt(cols)


def test_matvec_q6k_matches_numpy(oracle):
    W = synth.q6k_matrix(11, "lm", 64, 1536, signed_scales=True)
    x = synth.normals(11, "x", 1536)
    y32, y64 = oracle.matvec(Q6K, W, 64, 1536, x)
    wd = np_ref.dequant_q6k(W, 64 * 1536).reshape(64, 1536).astype(np.float64)
    assert np.allclose(y64, wd @ x.astype(np.float64), rtol=1e-12, atol=1e-9)
    two = oracle.matvec_two_pass(Q6K, W, 64, 1536, x, fast=False)
    assert np.array_equal(two, y32)


def test_pack_q40(oracle):
    rng = np.random.default_rng(5)
    v = (rng.standard_normal(32 * 50) * 0.7).astype(np.float32)
    v[0:32] = 0.0                      # all-zero block: scale 1, nibbles 8
    v[32:64] = np.linspace(-7, 7, 32)  # exact grid
    p = oracle.pack_q40(v).reshape(-1, 18)
    assert p[0, 0:2].view(np.uint16)[0] == 0x3C00 and np.all(p[0, 2:] == 0x88)
    back = oracle.dequant(Q40, p.reshape(-1), v.size)
    amax = np.abs(v.reshape(-1, 32)).max(axis=1)
    step = np.where(amax > 0, amax / 7, 1.0)
    # within half a step plus the fp16 rounding of the stored scale
    assert np.all(np.abs(back - v).reshape(-1, 32) <= (0.5 * step * 1.002 + 1e-7)[:, None] + 8 * step[:, None] * 2 ** -11)
    # independent restatement of the pack
    scale = np.where(amax > 0, (amax / np.float32(7.0)).astype(np.float32), np.float32(1.0)).astype(np.float32)
    inv = (np.float32(1.0) / scale).astype(np.float32)
    t = (v.reshape(-1, 32) * inv[:, None]).astype(np.float32)
    q = np.clip((np.sign(t) * np.floor(np.abs(t) + np.float32(0.5))).astype(np.int32) + 8, 0, 15)
    want = (q[:, :16] | (q[:, 16:] << 4)).astype(np.uint8)
    assert np.array_equal(p[:, 2:], want)
    assert np.array_equal(p[:, 0:2].copy().view(np.uint16)[:, 0], scale.astype(np.float16).view(np.uint16))
    # the through-half variant equals packing the f16-rounded values
    assert np.array_equal(oracle.pack_q40(v, through_half=True), oracle.pack_q40(v.astype(np.float16).astype(np.float32)))


def test_rmsnorm_family_vs_numpy(oracle):
    rng = np.random.default_rng(6)
    n = 1536
    x = rng.standard_normal(n).astype(np.float32) * 3
    w = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    res = rng.standard_normal(n).astype(np.float32)
    eps = 1e-6
    base = np_ref.rmsnorm(x, w, eps)
    assert np.allclose(oracle.rmsnorm(x, w, eps), base, rtol=1e-5, atol=1e-6)
    assert np.allclose(oracle.rmsnorm(x, w, eps, res=res), base + res, rtol=1e-5, atol=1e-6)
    assert np.allclose(oracle.rmsnorm(x, w, eps, res=res, scale=0.5), 0.5 * (base + res), rtol=1e-5, atol=1e-6)
    w2 = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    ox, ox2 = oracle.rmsnorm_add_then_rmsnorm(x, w, res, w2, eps)
    assert np.allclose(ox, base + res, rtol=1e-5, atol=1e-6)
    assert np.allclose(ox2, np_ref.rmsnorm(ox, w2, eps), rtol=1e-5, atol=1e-6)
    rows = oracle.rmsnorm(np.stack([x, 2 * x]), w, eps, rows=2)
    assert np.allclose(rows[0], base, rtol=1e-5, atol=1e-6) and np.allclose(rows[1], rows[0], rtol=1e-4, atol=1e-5)


def test_rope_table(oracle):
    t = oracle.rope_table(16, 64, 1e6)
    assert np.all(t[0, :32] == 1.0) and np.all(t[0, 32:] == 0.0)
    i = np.arange(32)
    freq = (1.0 / np.power(1e6, 2 * i / 64)).astype(np.float32)
    ang = (np.float32(5) * freq).astype(np.float32)
    assert np.allclose(t[5, :32], np.cos(ang), atol=1e-6) and np.allclose(t[5, 32:], np.sin(ang), atol=1e-6)
    part = oracle.rope_table(4, 64, 1e4, rope_angles=8)
    assert np.all(part[:, 8:32] == 1.0) and np.all(part[:, 40:] == 0.0)


def test_per_head_qkv_q40(oracle):
    rng = np.random.default_rng(8)
    n_q, n_kv, hd, eps = 4, 2, 64, 1e-6
    q = rng.standard_normal(n_q * hd).astype(np.float32)
    k = rng.standard_normal(n_kv * hd).astype(np.float32)
    v = rng.standard_normal(n_kv * hd).astype(np.float32)
    qw = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    kw = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    rope = oracle.rope_table(8, hd, 1e4)
    rowb = hd // 32 * 18
    kk = np.zeros(8 * n_kv * rowb, np.uint8)
    vv = np.zeros_like(kk)
    pos = 3
    qo = oracle.rmsnorm_per_head_qkv_q40(n_q, n_kv, hd, 1, eps, q, qw, rope[pos], k, kw, v, kk, vv, pos * n_kv * rowb)
    half = hd // 2
    c, s = rope[pos, :half].astype(np.float64), rope[pos, half:].astype(np.float64)

    def rot(xh, w):
        y = np_ref.rmsnorm(xh, w, eps)
        return np.concatenate([y[:half] * c - y[half:] * s, y[:half] * s + y[half:] * c])

    for h in range(n_q):
        assert np.allclose(qo[h * hd:(h + 1) * hd], rot(q[h * hd:(h + 1) * hd], qw), rtol=1e-5, atol=1e-6)
    # rows other than `pos` untouched; the written rows decode to the rotated K / normalised V within one step
    assert not kk[: pos * n_kv * rowb].any() and not kk[(pos + 1) * n_kv * rowb:].any()
    kd = oracle.dequant(Q40, kk[pos * n_kv * rowb:(pos + 1) * n_kv * rowb], n_kv * hd)
    vd = oracle.dequant(Q40, vv[pos * n_kv * rowb:(pos + 1) * n_kv * rowb], n_kv * hd)
    for h in range(n_kv):
        want_k = rot(k[h * hd:(h + 1) * hd], kw)
        want_v = np_ref.rmsnorm(v[h * hd:(h + 1) * hd], None, eps)
        for got, want in ((kd[h * hd:(h + 1) * hd], want_k), (vd[h * hd:(h + 1) * hd], want_v)):
            step = np.abs(want.reshape(-1, 32)).max(axis=1) / 7
            assert np.all(np.abs(got - want).reshape(-1, 32) <= 0.51 * step[:, None] + 1e-3)


@pytest.mark.parametrize("n_q,n_kv,tlen,start,nwg", [(8, 1, 1, 0, 0), (8, 1, 100, 0, 0), (8, 2, 300, 5, 16), (4, 4, 17, 0, 16), (8, 1, 129, 0, 16)])
def test_sdpa_vs_numpy_softmax(oracle, n_q, n_kv, tlen, start, nwg):
    hd = 64
    max_t = start + tlen + 3
    K = synth.q40_rows(21, "k", max_t * n_kv * hd, sigma=0.05)
    V = synth.q40_rows(21, "v", max_t * n_kv * hd, sigma=0.05)
    q = synth.normals(21, "q", n_q * hd)
    scale = 1.0 / np.sqrt(hd)
    got = oracle.sdpa_decode(n_q, n_kv, hd, q, K, V, tlen, start, scale, nwg)
    Kf = oracle.dequant(Q40, K, max_t * n_kv * hd).reshape(max_t, n_kv, hd)[start:start + tlen]
    Vf = oracle.dequant(Q40, V, max_t * n_kv * hd).reshape(max_t, n_kv, hd)[start:start + tlen]
    want = np_ref.attention(q.reshape(n_q, hd), Kf, Vf, n_q, n_kv, hd, scale)
    assert np.allclose(got, want, rtol=1e-4, atol=1e-6)


def test_sdpa_needle(oracle):
    """check_mul_mm.rs:249-294: K[0]=q, V[0]=1, everything else 0 -> the output stays at
    V[0]'s weight; with scale 1 and q=1 (score 256 vs 0) it is 1 to rounding."""
    n_q, hd, tlen = 8, 256, 512
    k = np.zeros((tlen, hd), np.float32)
    v = np.zeros((tlen, hd), np.float32)
    k[0] = 1.0
    v[0] = 1.0
    K, V = oracle.pack_q40(k), oracle.pack_q40(v)
    for nwg in (0, 16):
        out = oracle.sdpa_decode(n_q, 1, hd, np.ones(n_q * hd, np.float32), K, V, tlen, 0, 1.0, nwg)
        assert np.allclose(out, 1.0, atol=1e-3)


def test_softcap_argmax_and_gelu(oracle):
    x = np.array([0.1, 5.0, 5.0, -3.0, 4.999], np.float32)
    assert oracle.softcap_argmax(x, 30.0)[0] == 1          # tie -> lower index
    big = np.array([400.0, 1000.0, 500.0], np.float32)     # all saturate to cap -> first
    assert oracle.softcap_argmax(big, 30.0)[0] == 0
    rng = np.random.default_rng(9)
    z = rng.standard_normal(10000).astype(np.float32) * 10
    assert oracle.softcap_argmax(z, 30.0)[0] == int(np.argmax(z))
    g = np.array([-30.0, -1.0, 0.0, 0.5, 3.0, 25.0], np.float32)
    u = np.full(6, 2.0, np.float32)
    gc = np.clip(g.astype(np.float64), -20, 20)
    want = 0.5 * gc * (1 + np.tanh(0.79788456 * (gc + 0.044715 * gc ** 3))) * 2.0
    assert np.allclose(oracle.gelu_mul(g, u), want, rtol=1e-5, atol=1e-6)


def test_copy_scale_indexed(oracle):
    W = synth.q6k_matrix(13, "embd", 16, 512)
    out = oracle.copy_scale_indexed(Q6K, W, 512, np.array([3.0, 15.0], np.float32), 2.5)
    wd = oracle.dequant(Q6K, W, 16 * 512).reshape(16, 512)
    assert np.array_equal(out[0], np.float32(2.5) * wd[3]) and np.array_equal(out[1], np.float32(2.5) * wd[15])


def _digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_golden_fixtures(oracle):
    """Fixtures written by tests/golden/make_golden.py from the oracle itself (the reference
    is Rust and cannot run here).  They pin the oracle and the generator against drift."""
    with open(os.path.join(GOLDEN, "digests.json")) as f:
        gold = json.load(f)
    from tests.golden import make_golden
    now = make_golden.compute(oracle)
    assert now == gold
