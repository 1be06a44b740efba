"""GPU parity tests of the small ops, through the C ABI, against the CPU oracle."""
import numpy as np
import pytest

from ksearch_b200 import F16, F32, Q4K, Q6K, Q40, Eng, KsError, synth, write_meta
from tests.conftest import assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,gen,n", [
    (Q4K, lambda n: synth.q4k_matrix(31, "w", n // 1024, 1024), 64 * 1024),
    (Q6K, lambda n: synth.q6k_matrix(31, "w", n // 1024, 1024, signed_scales=True), 64 * 1024),
    (Q40, lambda n: synth.q40_rows(31, "kv", n), 64 * 1024),
    (Q4K, lambda n: synth.q4k_matrix(32, "w", 1, 256), 256),
    (5, lambda n: synth.q5k_matrix(31, "w5", n // 1024, 1024), 64 * 1024),      # Q5_K
])
def test_dequant_bit_exact(ctx, oracle, dtype, gen, n):
    data = gen(n)
    src = ctx.buffer_bytes(data)
    dst = ctx.buffer_empty_f32(n)
    Eng().dequant(ctx, dtype, src, n, dst)
    got = ctx.read_f32(dst, n)
    want = oracle.dequant(dtype, data, n)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_dequant_edge_cases(ctx):
    e = Eng()
    src = ctx.buffer_bytes(np.zeros(144, np.uint8))
    dst = ctx.buffer_empty_f32(256)
    e.dequant(ctx, Q4K, src, 0, dst)             # empty input is a no-op
    with pytest.raises(KsError):
        e.dequant(ctx, Q4K, src, 100, dst)        # ragged
    with pytest.raises(KsError):
        e.dequant(ctx, Q4K, src, 512, dst)        # source too small
    with pytest.raises(KsError):
        e.dequant(ctx, 17, src, 256, dst)         # unsupported ggml type


def _q4k_sources(n):
    """Source tensors for the load-time requantisation: the reference applies it to Q6_K tensors (signed scales as
    real files have them) and to f32 ones; the f32 case carries the shapes a quantizer trips over."""
    q6 = synth.q6k_matrix(51, "down", n // 1024, 1024, signed_scales=True)
    f = (synth.normals(52, "w", n) * 0.05).astype(np.float32)
    f[:256] = 0.0                                   # an all-zero super-block: zero scales, zero levels
    f[256:288] = 0.37                               # a constant positive sub-block (its minimum clamps to 0)
    f[288:320] = -0.37                              # a constant negative sub-block (max == min)
    f[512:768] = np.abs(f[512:768])                 # a super-block without negative values: every minimum is 0
    f[768:1024] *= 1e-6                             # tiny values: scales near the f16 subnormal range
    f[1024:1280] *= 300.0                           # large values
    return [(Q6K, q6), (F32, f), (F16, f.astype(np.float16)), (5, synth.q5k_matrix(53, "ple", n // 1024, 1024))]


@pytest.mark.parametrize("which", [0, 1, 2, 3])
def test_quantize_q4k_matches_reference_quantizer(ctx, oracle, which):
    """ks_quantize_q4k: gguf_impl.rs:803-1016 on the GPU, byte for byte against the CPU restatement fed with the
    dequantised source (gemma_prim.rs:415-440: dequant_to_f32, then quantize_f32_to_q4k)."""
    n = 96 * 1024
    dtype, data = _q4k_sources(n)[which]
    src = ctx.buffer_bytes(data)
    dst = ctx.buffer_empty_bytes(n // 256 * 144)
    Eng().quantize_q4k(ctx, dtype, src, n, dst)
    got = ctx.read_bytes(dst, n // 256 * 144)
    flat = oracle.dequant(dtype, data, n) if dtype in (Q6K, 5) else np.asarray(data, np.float32)
    want = oracle.quantize_q4k(flat)
    bad = np.flatnonzero(got != want)
    assert bad.size == 0, f"{bad.size} differing bytes, first at {bad[:8]} (block {bad[0] // 144}, byte {bad[0] % 144})"
    # and the result is a usable Q4_K tensor: it dequantises close to the source
    back = oracle.dequant(Q4K, got, n)
    scale = np.abs(flat).reshape(-1, 256).max(axis=1).repeat(256) + 1e-30
    assert np.abs(back - flat).max() <= 0.12 * scale.max() and np.median(np.abs(back - flat) / scale) < 0.03


def test_quantize_q4k_edge_cases(ctx):
    e = Eng()
    src = ctx.buffer_bytes(np.zeros(256, np.float32))
    dst = ctx.buffer_empty_bytes(144)
    e.quantize_q4k(ctx, F32, src, 0, dst)            # empty input is a no-op
    e.quantize_q4k(ctx, F32, src, 256, dst)
    assert not ctx.read_bytes(dst, 144).any()        # zeros quantise to an all-zero block
    with pytest.raises(KsError):
        e.quantize_q4k(ctx, F32, src, 100, dst)      # ragged
    with pytest.raises(KsError):
        e.quantize_q4k(ctx, F32, src, 512, dst)      # source too small
    with pytest.raises(KsError):
        e.quantize_q4k(ctx, Q40, src, 256, dst)      # unsupported source type


@pytest.mark.parametrize("act", [F32, F16])
@pytest.mark.parametrize("n,rows", [(1536, 1), (2560, 1), (256, 5), (4096, 3), (100, 2)])
def test_rmsnorm_family(ctx, oracle, act, n, rows):
    e = Eng(act)
    npdt = np.float32 if act == F32 else np.float16
    x = (synth.normals(41, "x", n * rows) * 3).astype(npdt)
    w = synth.norm_weight(41, "w", n).astype(npdt)
    res = synth.normals(41, "r", n * rows).astype(npdt)
    bx, bw, br = ctx.buffer_bytes(x), ctx.buffer_bytes(w), ctx.buffer_bytes(res)
    by = ctx.buffer_empty_bytes(n * rows * x.itemsize)
    tol = dict(rtol=1e-3, atol=1e-4) if act == F32 else dict(rtol=2e-3, atol=2e-3)
    xf, wf, rf = x.astype(np.float32), w.astype(np.float32), res.astype(np.float32)

    e.rmsnorm_rows(ctx, n, rows, 1e-6, bx, bw, by)
    assert_close(ctx.read_act(by, n * rows, act), oracle.rmsnorm(xf, wf, 1e-6, rows=rows), what="rmsnorm", **tol)
    e.rmsnorm_add_rows(ctx, n, rows, 1e-6, bx, bw, br, by)
    assert_close(ctx.read_act(by, n * rows, act), oracle.rmsnorm(xf, wf, 1e-6, res=rf, rows=rows), what="rmsnorm_add", **tol)
    if rows == 1:
        e.rmsnorm_add_scale(ctx, n, 1e-6, 0.25, bx, bw, br, by)
        assert_close(ctx.read_act(by, n, act), oracle.rmsnorm(xf, wf, 1e-6, res=rf, scale=0.25), what="rmsnorm_add_scale", **tol)
        # in-place residual update, as the decode loop uses it (y aliases the residual)
        e.rmsnorm_add(ctx, n, 1e-6, bx, bw, br, br)
        assert_close(ctx.read_act(br, n, act), oracle.rmsnorm(xf, wf, 1e-6, res=rf), what="rmsnorm_add in place", **tol)


@pytest.mark.parametrize("act", [F32, F16])
def test_rmsnorm_add_then_rmsnorm(ctx, oracle, act):
    e = Eng(act)
    n, rows = 1536, 2
    npdt = np.float32 if act == F32 else np.float16
    y = (synth.normals(42, "y", n * rows) * 2).astype(npdt)
    res = synth.normals(42, "r", n * rows).astype(npdt)
    wp = synth.norm_weight(42, "wp", n).astype(npdt)
    wf = synth.norm_weight(42, "wf", n).astype(npdt)
    by, br, bwp, bwf = map(ctx.buffer_bytes, (y, res, wp, wf))
    ox, ox2 = ctx.buffer_empty_bytes(y.nbytes), ctx.buffer_empty_bytes(y.nbytes)
    e.rmsnorm_add_then_rmsnorm_rows(ctx, n, rows, 1e-6, by, bwp, br, bwf, ox, ox2)
    wx, wx2 = oracle.rmsnorm_add_then_rmsnorm(y.astype(np.float32), wp.astype(np.float32), res.astype(np.float32),
                                              wf.astype(np.float32), 1e-6, rows=rows)
    tol = dict(rtol=1e-3, atol=1e-4) if act == F32 else dict(rtol=3e-3, atol=3e-3)
    assert_close(ctx.read_act(ox, n * rows, act), wx, what="out_x", **tol)
    assert_close(ctx.read_act(ox2, n * rows, act), wx2, what="out_x2", **tol)
    # aliasing used by the decode loop: residual in/out and y in / x2 out share buffers
    e.rmsnorm_add_then_rmsnorm_rows(ctx, n, rows, 1e-6, by, bwp, br, bwf, br, by)
    assert_close(ctx.read_act(br, n * rows, act), wx, what="out_x aliased", **tol)
    assert_close(ctx.read_act(by, n * rows, act), wx2, what="out_x2 aliased", **tol)
    with pytest.raises(KsError, match="LOCAL staging"):
        e.rmsnorm_add_then_rmsnorm(ctx, 1 << 20, 1e-6, by, bwp, br, bwf, ox, ox2)


def test_quantize_q40_bit_exact(ctx, oracle, golden_cases):
    e = Eng(F32)
    v = golden_cases["pack_q40.v"]
    dst = ctx.buffer_empty_bytes(v.size // 32 * 18 + 36)
    e.quantize_q40(ctx, v.size, ctx.buffer_bytes(v), dst, 36)
    got = ctx.read_bytes(dst)
    assert not got[:36].any()
    assert np.array_equal(got[36:], golden_cases["pack_q40.packed"])
    # zero block and a larger random case against the oracle
    big = synth.normals(43, "v", 32 * 4096, sigma=0.3)
    big[:32] = 0
    d2 = ctx.buffer_empty_bytes(big.size // 32 * 18)
    e.quantize_q40(ctx, big.size, ctx.buffer_bytes(big), d2, 0)
    assert np.array_equal(ctx.read_bytes(d2), oracle.pack_q40(big))
    with pytest.raises(KsError):
        e.quantize_q40(ctx, 33, ctx.buffer_bytes(big), d2, 0)


@pytest.mark.parametrize("act", [F32, F16])
@pytest.mark.parametrize("n_q,n_kv,hd,n_tok", [(8, 1, 256, 1), (8, 2, 256, 1), (8, 1, 256, 5), (4, 2, 64, 3)])
def test_per_head_qkv_q40(ctx, oracle, act, n_q, n_kv, hd, n_tok):
    e = Eng(act)
    npdt = np.float32 if act == F32 else np.float16
    eps, max_seq, pos0 = 1e-6, 16, 4
    q = synth.normals(44, "q", n_tok * n_q * hd).astype(npdt)
    k = synth.normals(44, "k", n_tok * n_kv * hd).astype(npdt)
    v = synth.normals(44, "v", n_tok * n_kv * hd).astype(npdt)
    qw = synth.norm_weight(44, "qw", hd).astype(npdt)
    kw = synth.norm_weight(44, "kw", hd).astype(npdt)
    rope = oracle.rope_table(max_seq, hd, 1e6)
    rowb = hd // 32 * 18
    bq, bk, bv, bqw, bkw, brope = map(ctx.buffer_bytes, (q, k, v, qw, kw, rope))
    kvk = ctx.buffer_empty_bytes(max_seq * n_kv * rowb)
    kvv = ctx.buffer_empty_bytes(max_seq * n_kv * rowb)
    off = pos0 * n_kv * rowb
    e.rmsnorm_per_head_qkv_q40_batch(ctx, n_q, n_kv, hd, n_tok, eps, bq, bqw, brope, pos0 * hd, bk, bkw, bv, bq, kvk, kvv, off)
    got_q = ctx.read_act(bq, q.size, act)
    gk, gv = ctx.read_bytes(kvk), ctx.read_bytes(kvv)
    ok_ = np.zeros(max_seq * n_kv * rowb, np.uint8)
    ov_ = np.zeros_like(ok_)
    want_q = oracle.rmsnorm_per_head_qkv_q40(n_q, n_kv, hd, n_tok, eps, q.astype(np.float32), qw.astype(np.float32),
                                             rope[pos0:pos0 + n_tok], k.astype(np.float32), kw.astype(np.float32),
                                             v.astype(np.float32), ok_, ov_, off)
    tol = dict(rtol=1e-3, atol=1e-4) if act == F32 else dict(rtol=3e-3, atol=3e-3)
    assert_close(got_q, want_q, what="q_out", **tol)
    # untouched rows stay zero; written rows: scales within 1 fp16 ulp, nibbles within 1 step for a
    # handful of values that sit on a rounding boundary, identical otherwise
    span = slice(off, off + n_tok * n_kv * rowb)
    for g, o in ((gk, ok_), (gv, ov_)):
        assert not g[:off].any() and not g[off + n_tok * n_kv * rowb:].any()
        gb, ob = g[span].reshape(-1, 18), o[span].reshape(-1, 18)
        ds = gb[:, :2].copy().view(np.uint16).astype(np.int32) - ob[:, :2].copy().view(np.uint16).astype(np.int32)
        assert np.abs(ds).max() <= 1
        dn = np.abs(np.concatenate([gb[:, 2:] & 15, gb[:, 2:] >> 4], 1).astype(np.int32) -
                    np.concatenate([ob[:, 2:] & 15, ob[:, 2:] >> 4], 1).astype(np.int32))
        assert dn.max() <= 1 and (dn != 0).mean() < 0.01
    with pytest.raises(KsError, match="max_seq exceeded"):
        e.rmsnorm_per_head_qkv_q40_off(ctx, n_q, n_kv, hd, eps, bq, bqw, brope, 0, bk, bkw, bv, bq, kvk, kvv, max_seq * n_kv * rowb)
    with pytest.raises(KsError):
        e.rmsnorm_per_head_qkv_q40_off(ctx, n_q, n_kv, 48, eps, bq, bqw, brope, 0, bk, bkw, bv, bq, kvk, kvv, 0)


@pytest.mark.parametrize("dtype", [Q6K, Q4K, 5, F16, F32])     # 5: Q5_K, the per-layer-embedding table's type (render.rs:695-724)
def test_copy_scale_indexed(ctx, oracle, dtype):
    e = Eng(F32)
    n, vocab = 1536, 64
    if dtype == 5:
        src = synth.q5k_matrix(45, "e", vocab, n)
    elif dtype == Q6K:
        src = synth.q6k_matrix(45, "e", vocab, n, signed_scales=True)
    elif dtype == Q4K:
        src = synth.q4k_matrix(45, "e", vocab, n)
    elif dtype == F16:
        src = synth.normals(45, "e", vocab * n).astype(np.float16)
    else:
        src = synth.normals(45, "e", vocab * n)
    ids = np.array([0, 63, 17], np.float32)
    dst = ctx.buffer_empty_f32(3 * n)
    scale = float(np.sqrt(np.float32(n)))
    e.copy_scale_indexed_batch_wd(ctx, n, 3, scale, dtype, ctx.buffer_bytes(src), ctx.buffer_bytes(ids), dst)
    want = oracle.copy_scale_indexed(dtype, src, n, ids, scale)
    assert np.array_equal(ctx.read_f32(dst, 3 * n).view(np.uint32), want.ravel().view(np.uint32))
    one = ctx.buffer_empty_f32(n)
    e.copy_scale_indexed_wd(ctx, n, scale, dtype, ctx.buffer_bytes(src), ctx.buffer_bytes(ids[1:2]), one)
    assert np.array_equal(ctx.read_f32(one, n), want[1])
    with pytest.raises(KsError, match="not wired"):
        e.copy_scale_indexed_wd(ctx, n, scale, Q40, ctx.buffer_bytes(src), ctx.buffer_bytes(ids), one)


def test_softcap_argmax(ctx, oracle):
    e = Eng(F32)
    out = ctx.buffer_empty_f32(1)
    for seed, n in ((1, 262144), (2, 1000), (3, 1), (4, 4097)):
        x = synth.normals(seed, "logits", n, sigma=8.0)
        e.softcap_argmax(ctx, n, 30.0, ctx.buffer_bytes(x), out)
        got = int(ctx.read_f32(out, 1)[0])
        want, _ = oracle.softcap_argmax(x, 30.0)
        assert got == want == int(np.argmax(x))
    # ties go to the lower index; saturated values all tie at cap
    x = np.zeros(5000, np.float32)
    x[[4000, 77, 2500]] = 5.0
    e.softcap_argmax(ctx, x.size, 30.0, ctx.buffer_bytes(x), out)
    assert int(ctx.read_f32(out, 1)[0]) == 77
    x = np.full(3000, 1000.0, np.float32)
    x[:10] = 1.0
    e.softcap_argmax(ctx, x.size, 30.0, ctx.buffer_bytes(x), out)
    assert int(ctx.read_f32(out, 1)[0]) == 10 == oracle.softcap_argmax(x, 30.0)[0]
    # repeated launches reuse the cross-block counter
    for _ in range(3):
        e.softcap_argmax(ctx, x.size, 30.0, ctx.buffer_bytes(x), out)
        assert int(ctx.read_f32(out, 1)[0]) == 10


def test_gelu_mul(ctx, oracle):
    e = Eng(F32)
    g = synth.normals(46, "g", 6144, sigma=6.0)
    g[:4] = [-30, 30, 0, 20]
    u = synth.normals(46, "u", 6144)
    y = ctx.buffer_empty_f32(6144)
    e.gelu_mul(ctx, 6144, ctx.buffer_bytes(g), ctx.buffer_bytes(u), y)
    assert_close(ctx.read_f32(y, 6144), oracle.gelu_mul(g, u), what="gelu_mul")


def _attn_case(ctx, oracle, e, n_slots, n_q, n_kv, hd, max_t, tlens, starts, scale, n_splits, act=F32):
    npdt = np.float32 if act == F32 else np.float16
    rowb = hd // 32 * 18
    slot_bytes = max_t * n_kv * rowb
    K = synth.q40_rows(51, "K", n_slots * max_t * n_kv * hd, sigma=0.05)
    V = synth.q40_rows(51, "V", n_slots * max_t * n_kv * hd, sigma=0.05)
    q = synth.normals(51, "q", n_slots * n_q * hd).astype(npdt)
    bK, bV, bq = ctx.buffer_bytes(K), ctx.buffer_bytes(V), ctx.buffer_bytes(q)
    meta = ctx.buffer_empty_f32(4 * n_slots)
    for s in range(n_slots):
        write_meta(ctx, meta, tlens[s], starts[s], 0, slot=s)
    ns = n_splits if n_splits else ctx.lib.ks_sdpa_pick_splits(ctx.h, n_slots, n_kv, max_t)
    tmp = ctx.buffer_empty_f32(max(1, e.sdpa_tmp_floats(n_q, hd, ns, n_slots)))
    out = ctx.buffer_empty_bytes(q.nbytes)
    e.sdpa_decode(ctx, n_slots, n_q, n_kv, hd, max_t, bq, bK, bV, meta, tmp, out, scale=scale, n_splits=n_splits,
                  slot_stride_bytes=slot_bytes)
    got = ctx.read_act(out, q.size, act).reshape(n_slots, -1)
    for s in range(n_slots):
        want = oracle.sdpa_decode(n_q, n_kv, hd, q.astype(np.float32).reshape(n_slots, -1)[s],
                                  K[s * slot_bytes:(s + 1) * slot_bytes], V[s * slot_bytes:(s + 1) * slot_bytes],
                                  tlens[s], starts[s], scale, 0)
        tol = dict(rtol=1e-3, atol=1e-4) if act == F32 else dict(rtol=3e-3, atol=1e-3)
        assert_close(got[s], want, what=f"sdpa slot {s} tlen {tlens[s]}", **tol)


@pytest.mark.parametrize("n_q,n_kv", [(8, 1), (8, 2)])
@pytest.mark.parametrize("tlen,n_splits", [(1, 1), (1, 16), (17, 16), (127, 1), (128, 16), (1024, 0), (1000, 64), (1000, 128), (300, 2)])
def test_sdpa_single_slot(ctx, oracle, n_q, n_kv, tlen, n_splits):
    _attn_case(ctx, oracle, Eng(F32), 1, n_q, n_kv, 256, 1024, [tlen], [0], 1.0 / 16.0, n_splits)


def test_sdpa_window_start_and_scale_one(ctx, oracle):
    """Sliding-window form: positions start..start+tlen-1 (GP:1010-1017); reference scale 1."""
    _attn_case(ctx, oracle, Eng(F32), 1, 8, 1, 256, 600, [300], [211], 1.0, 16)


@pytest.mark.parametrize("n_q,n_kv", [(8, 1), (8, 2)])
def test_sdpa_four_slots_independent_lengths(ctx, oracle, n_q, n_kv):
    _attn_case(ctx, oracle, Eng(F32), 4, n_q, n_kv, 256, 4096, [1024, 4096, 77, 2048], [0, 0, 3, 100], 1.0 / 16.0, 0)


@pytest.mark.parametrize("n_q,n_kv", [(8, 1), (8, 2)])
def test_sdpa_context_16384_and_slot_mix(ctx, oracle, n_q, n_kv):
    """The attention benchmark shape as written: contexts of 1024 / 4096 / 16384 positions, one slot at the
    full 16384, and four slots of independent lengths {1024, 4096, 16384, 16384} in one launch."""
    _attn_case(ctx, oracle, Eng(F32), 1, n_q, n_kv, 256, 16384, [16384], [0], 1.0 / 16.0, 0)
    _attn_case(ctx, oracle, Eng(F32), 4, n_q, n_kv, 256, 16384, [1024, 4096, 16384, 16384], [0, 0, 0, 0], 1.0 / 16.0, 0)


def test_sdpa_f16_and_hd128(ctx, oracle):
    _attn_case(ctx, oracle, Eng(F16), 2, 8, 2, 256, 512, [512, 200], [0, 0], 1.0 / 16.0, 8, act=F16)
    _attn_case(ctx, oracle, Eng(F32), 1, 4, 1, 128, 256, [250], [0], 0.1, 4)


def test_sdpa_hybrid_and_needle(ctx, oracle):
    """The reference's dispatch (online below 128 positions, 16 partitions from 128) and its
    'needle' check: K[0]=q, V[0]=1, rest 0 -> output 1 (check_mul_mm.rs:249-294)."""
    e = Eng(F32)
    n_q, hd = 8, 256
    for tlen in (64, 512, 8192, 16384):
        k = np.zeros((tlen, hd), np.float32)
        v = np.zeros((tlen, hd), np.float32)
        k[0] = 1.0
        v[0] = 1.0
        bk_f, bv_f = ctx.buffer_bytes(k), ctx.buffer_bytes(v)
        bk, bv = ctx.buffer_empty_bytes(tlen * hd // 32 * 18), ctx.buffer_empty_bytes(tlen * hd // 32 * 18)
        e.quantize_q40(ctx, tlen * hd, bk_f, bk, 0)
        e.quantize_q40(ctx, tlen * hd, bv_f, bv, 0)
        meta = ctx.buffer_empty_f32(4)
        write_meta(ctx, meta, tlen, 0, tlen)
        tmp = ctx.buffer_empty_f32(n_q * Eng.SDPA_MWG_NWG * (hd + 2))
        o = ctx.buffer_empty_f32(n_q * hd)
        e.sdpa_hybrid_kv(ctx, n_q, 1, hd, tlen, tlen, Q40, ctx.buffer_bytes(np.ones(n_q * hd, np.float32)), bk, bv, meta, tmp, o)
        out = ctx.read_f32(o, n_q * hd)
        assert np.allclose(out, 1.0, atol=1e-3), (tlen, out.min(), out.max())


def test_sdpa_errors(ctx):
    e = Eng(F32)
    b = ctx.buffer_empty_bytes(1024 * 144)
    q = ctx.buffer_empty_f32(8 * 256)
    meta = ctx.buffer_empty_f32(4)
    with pytest.raises(KsError, match="too small"):
        e.sdpa_decode(ctx, 1, 8, 1, 256, 2048, q, b, b, meta, None, q, n_splits=1)
    with pytest.raises(KsError, match="multiple of 32"):
        e.sdpa_decode(ctx, 1, 8, 1, 100, 16, q, b, b, meta, None, q, n_splits=1)
    with pytest.raises(KsError):
        e.sdpa_decode(ctx, 1, 8, 3, 256, 16, q, b, b, meta, None, q, n_splits=1)
    with pytest.raises(KsError, match="tmp"):
        e.sdpa_decode(ctx, 1, 8, 1, 256, 1024, q, b, b, meta, ctx.buffer_empty_f32(16), q, n_splits=16)


def test_runtime_ordering_calls(ctx):
    """flush / wait_inflight_at_most / synchronize / has_gpu_work (M:157-218)."""
    e = Eng(F32)
    x = synth.normals(47, "x", 1536)
    w = synth.norm_weight(47, "w", 1536)
    bx, bw, by = ctx.buffer_bytes(x), ctx.buffer_bytes(w), ctx.buffer_empty_f32(1536)
    n0 = ctx.launch_count()
    for _ in range(4):
        e.rmsnorm(ctx, 1536, 1e-6, bx, bw, by)
        ctx.flush_async()
    assert ctx.launch_count() == n0 + 4
    ctx.wait_inflight_at_most(1)
    ctx.synchronize()
    assert not ctx.has_gpu_work()
    with pytest.raises(KsError):
        ctx.write_buffer(by, np.zeros(4096, np.float32))   # larger than the buffer
