"""GPU parity tests of the dequant-fused matvec family, through the C ABI.

Tolerance (the path's contract): |y - ref| <= 1e-4 + 1e-3*|ref| element-wise against the
f64-accumulated CPU result, plus a norm-wise bound against the reference-style f32
sequential sum (whose own rounding noise exceeds the element-wise bound on rows that
cancel to ~0, so it cannot be the element-wise yardstick)."""
import numpy as np
import pytest

from ksearch_b200 import F16, F32, Q4K, Q6K, Eng, KsError, synth
from tests.conftest import assert_close

pytestmark = pytest.mark.gpu


def _gen(dtype, seed, name, rows, cols, **kw):
    return (synth.q4k_matrix if dtype == Q4K else synth.q6k_matrix)(seed, name, rows, cols, **kw)


def _check(y, y32, y64, what):
    assert_close(y, y64, what=what)
    scale = np.abs(y64).max()
    assert np.abs(y - y32).max() <= 1e-5 * scale + 1e-4, what


@pytest.mark.parametrize("name", ["q4k_64x512", "q4k_24x1536", "q6k_32x1536"])
def test_matvec_golden_cases(ctx, golden_cases, name):
    W, x = golden_cases[name + ".W"], golden_cases[name + ".x"]
    dtype = Q4K if name.startswith("q4k") else Q6K
    rows, cols = (int(v) for v in name.split("_")[1].split("x"))
    y = ctx.buffer_empty_f32(rows)
    Eng().matvec_wd(ctx, rows, cols, dtype, ctx.buffer_bytes(W), ctx.buffer_bytes(x), y)
    _check(ctx.read_f32(y, rows), golden_cases[name + ".y32"], golden_cases[name + ".y64"], name)


@pytest.mark.parametrize("dtype,rows,cols", [
    (Q4K, 256, 4096),    # config 0 columns
    (Q4K, 128, 1536), (Q4K, 96, 6144), (Q4K, 64, 10240), (Q4K, 130, 2048), (Q4K, 33, 2560),
    (Q4K, 1, 256), (Q4K, 7, 768), (Q4K, 5, 512), (Q4K, 3, 1280),
    (Q6K, 512, 1536), (Q6K, 100, 2560), (Q6K, 1, 256), (Q6K, 9, 768), (Q6K, 31, 4096),
])
def test_matvec_vs_oracle(ctx, oracle, dtype, rows, cols):
    W = _gen(dtype, 61, f"W{rows}x{cols}", rows, cols)
    x = synth.normals(61, "x", cols)
    y = ctx.buffer_empty_f32(rows + 8)
    Eng().matvec_wd_at(ctx, rows, cols, dtype, ctx.buffer_bytes(W), ctx.buffer_bytes(np.concatenate([np.zeros(3, np.float32), x])), 3, y, 4)
    got = ctx.read_f32(y, rows + 8)
    assert not got[:4].any() and not got[rows + 4:].any()      # nothing written outside [y_off, y_off+rows)
    y32, y64 = oracle.matvec(dtype, W, rows, cols, x)
    _check(got[4:rows + 4], y32, y64, f"matvec {dtype} {rows}x{cols}")


def test_matvec_q6k_signed_scales(ctx, oracle):
    W = synth.q6k_matrix(62, "W", 200, 1536, signed_scales=True)
    x = synth.normals(62, "x", 1536)
    y = ctx.buffer_empty_f32(200)
    Eng().matvec_wd(ctx, 200, 1536, Q6K, ctx.buffer_bytes(W), ctx.buffer_bytes(x), y)
    y32, y64 = oracle.matvec(Q6K, W, 200, 1536, x)
    _check(ctx.read_f32(y, 200), y32, y64, "q6k signed scales")


@pytest.mark.parametrize("rows,cols,nr", [(512, 1536, 1), (203, 1536, 2), (100, 2560, 2), (9, 768, 1), (31, 4096, 2), (1, 256, 1)])
def test_matvec_q6k_fixed_point_variant(ctx, oracle, rows, cols, nr):
    """Plan variant 2: x as 24-bit block fixed point, 6-bit weights x x as byte dot products (the lm_head kernel).
    Odd row counts and odd block counts per row put blocks on both 2-byte alignments."""
    from ksearch_b200 import _lib
    W = synth.q6k_matrix(63, f"W{rows}x{cols}", rows, cols, signed_scales=True)
    x = synth.normals(63, "x", cols)
    y = ctx.buffer_empty_f32(rows + 8)
    ctx.plan_override(_lib.Plan(2, nr, 8, 4, 0.0))
    try:
        launches = ctx.launch_count()
        Eng().matvec_wd_at(ctx, rows, cols, Q6K, ctx.buffer_bytes(W), ctx.buffer_bytes(x), 0, y, 4)
        assert ctx.launch_count() == launches + 1
    finally:
        ctx.plan_override(None)
    got = ctx.read_f32(y, rows + 8)
    assert not got[:4].any() and not got[rows + 4:].any()
    y32, y64 = oracle.matvec(Q6K, W, rows, cols, x)
    _check(got[4:rows + 4], y32, y64, f"q6k fixed-point {rows}x{cols}")


def test_matvec_reference_patterns(ctx, oracle):
    """check_mul_mm.rs:47-109 inputs: integer-pattern W quantised by the reference quantizer,
    pattern x; GEMV vs CPU dequant + f32 dot.  The reference prints max|err| against a 0.05
    threshold; here the path's own tolerance applies."""
    for rows, cols, batch in ((64, 256, 8), (128, 256, 8), (512, 1536, 4)):
        r, c, t = np.arange(rows)[:, None], np.arange(cols)[None, :], np.arange(batch)[:, None]
        w = ((((r * 17 + c * 13) % 200).astype(np.float32) - 100.0) * np.float32(0.02)).astype(np.float32)
        x = ((((t * 11 + c * 7) % 50).astype(np.float32) - 25.0) * np.float32(0.04)).astype(np.float32)
        wq = oracle.quantize_q4k(w.ravel())
        y32, y64 = oracle.matvec(Q4K, wq, rows, cols, x)
        by = ctx.buffer_empty_f32(batch * rows)
        Eng().matvec_batch(ctx, rows, cols, batch, Q4K, ctx.buffer_bytes(wq), ctx.buffer_bytes(x), by)
        got = ctx.read_f32(by, batch * rows).reshape(batch, rows)
        _check(got, y32, y64, f"pattern {rows}x{cols}x{batch}")


@pytest.mark.parametrize("dtype", [Q4K, Q6K])
@pytest.mark.parametrize("batch", [1, 2, 3, 4, 5, 8])
def test_matvec_batch(ctx, oracle, dtype, batch):
    rows, cols = 96, 1536
    W = _gen(dtype, 63, "W", rows, cols)
    x = synth.normals(63, "x", batch * cols).reshape(batch, cols)
    y = ctx.buffer_empty_f32(batch * rows)
    Eng().matvec_batch(ctx, rows, cols, batch, dtype, ctx.buffer_bytes(W), ctx.buffer_bytes(x), y)
    y32, y64 = oracle.matvec(dtype, W, rows, cols, x)
    _check(ctx.read_f32(y, batch * rows).reshape(batch, rows), np.atleast_2d(y32), np.atleast_2d(y64), f"batch {batch}")


@pytest.mark.parametrize("q_rows,kv_rows,cols", [(2048, 256, 1536), (2048, 512, 2560), (40, 8, 512)])
def test_matvec_qkv(ctx, oracle, q_rows, kv_rows, cols):
    Wq, Wk, Wv = (_gen(Q4K, 64, n, r, cols) for n, r in (("q", q_rows), ("k", kv_rows), ("v", kv_rows)))
    x = synth.normals(64, "x", cols)
    q, k, v = ctx.buffer_empty_f32(q_rows), ctx.buffer_empty_f32(kv_rows), ctx.buffer_empty_f32(kv_rows)
    Eng().matvec_qkv_wd(ctx, q_rows, kv_rows, cols, Q4K, *map(ctx.buffer_bytes, (Wq, Wk, Wv)), ctx.buffer_bytes(x), q, k, v)
    for buf, W, r, nm in ((q, Wq, q_rows, "q"), (k, Wk, kv_rows, "k"), (v, Wv, kv_rows, "v")):
        y32, y64 = oracle.matvec(Q4K, W, r, cols, x)
        _check(ctx.read_f32(buf, r), y32, y64, "qkv " + nm)


def test_matvec_qkv_mixed_dtypes(ctx, oracle):
    """Q4K / Q4K / Q6K packings in one call (K:226 'per-buffer weight dtypes')."""
    cols = 1536
    Wq, Wk, Wv = _gen(Q4K, 65, "q", 64, cols), _gen(Q4K, 65, "k", 16, cols), _gen(Q6K, 65, "v", 16, cols)
    x = synth.normals(65, "x", cols)
    q, k, v = ctx.buffer_empty_f32(64), ctx.buffer_empty_f32(16), ctx.buffer_empty_f32(16)
    Eng().matvec_qkv_wds(ctx, 64, 16, cols, Q4K, Q4K, Q6K, *map(ctx.buffer_bytes, (Wq, Wk, Wv)), ctx.buffer_bytes(x), q, k, v)
    y32, y64 = oracle.matvec(Q6K, Wv, 16, cols, x)
    _check(ctx.read_f32(v, 16), y32, y64, "mixed v")
    y32, y64 = oracle.matvec(Q4K, Wq, 64, cols, x)
    _check(ctx.read_f32(q, 64), y32, y64, "mixed q")


@pytest.mark.parametrize("rows,cols", [(6144, 1536), (1000, 2560), (6, 512)])
def test_matvec_gate_up_gelu(ctx, oracle, rows, cols):
    # d scaled down so the gate lands in GELU's curved range rather than saturating
    Wg, Wu = _gen(Q4K, 66, "g", rows, cols, sigma=0.0005), _gen(Q4K, 66, "u", rows, cols, sigma=0.0005)
    x = synth.normals(66, "x", cols)
    y = ctx.buffer_empty_f32(rows)
    Eng().matvec_gate_up_gelu_wd(ctx, rows, cols, Q4K, ctx.buffer_bytes(Wg), ctx.buffer_bytes(Wu), ctx.buffer_bytes(x), y)
    _, g64 = oracle.matvec(Q4K, Wg, rows, cols, x)
    _, u64 = oracle.matvec(Q4K, Wu, rows, cols, x)
    want = oracle.gelu_mul(g64.astype(np.float32), u64.astype(np.float32))
    # the product of two rounded dot products: allow each factor its own tolerance
    got = ctx.read_f32(y, rows)
    tol = 1e-4 + 2e-3 * np.abs(want) + 1e-4 * (np.abs(g64) + np.abs(u64))
    assert np.all(np.abs(got - want) <= tol)


def test_matvec_f16_activations(ctx, oracle):
    """The reference's own mode: f16 x in, f16 y out, f32 accumulation (RE:2263-2274)."""
    rows, cols = 256, 1536
    W = _gen(Q4K, 67, "W", rows, cols, sigma=0.001)
    x = synth.normals(67, "x", cols).astype(np.float16)
    y = ctx.buffer_empty_f16(rows)
    Eng(F16).matvec_wd(ctx, rows, cols, Q4K, ctx.buffer_bytes(W), ctx.buffer_bytes(x), y)
    _, y64 = oracle.matvec(Q4K, W, rows, cols, x.astype(np.float32))
    got = ctx.read_f16(y, rows).astype(np.float64)
    assert np.all(np.abs(got - y64) <= 1e-3 + 1.5e-3 * np.abs(y64))


def test_matvec_linearity_full_size(ctx):
    """Size-independent property at the full 4096x4096 shape: W(a*x1 + x2) = a*W x1 + W x2."""
    rows = cols = 4096
    W = ctx.buffer_bytes(synth.q4k_matrix(68, "W", rows, cols))
    x1, x2 = synth.normals(68, "x1", cols), synth.normals(68, "x2", cols)
    e = Eng()
    ys = []
    for x in (x1, x2, (np.float32(0.5) * x1 + x2).astype(np.float32)):
        y = ctx.buffer_empty_f32(rows)
        e.matvec_wd(ctx, rows, cols, Q4K, W, ctx.buffer_bytes(x), y)
        ys.append(ctx.read_f32(y, rows).astype(np.float64))
    scale = np.abs(ys[2]).max()
    assert np.abs(0.5 * ys[0] + ys[1] - ys[2]).max() <= 2e-5 * scale


def test_matvec_full_config_shapes_row_checksums(ctx, oracle):
    """Full-size shapes of the sweep; the oracle checks a strided sample of rows exactly and the
    rest through the sum of outputs (y . 1 = (W^T 1) . x is linear in the rows)."""
    for dtype, rows, cols in ((Q4K, 4096, 4096), (Q4K, 6144, 1536), (Q4K, 1536, 6144), (Q4K, 2560, 10240), (Q6K, 32768, 1536)):
        W = _gen(dtype, 69, f"W{rows}x{cols}", rows, cols)
        x = synth.normals(69, "x", cols)
        y = ctx.buffer_empty_f32(rows)
        Eng().matvec_wd(ctx, rows, cols, dtype, ctx.buffer_bytes(W), ctx.buffer_bytes(x), y)
        got = ctx.read_f32(y, rows)
        rb = cols // 256 * (144 if dtype == Q4K else 210)
        sel = np.arange(0, rows, max(1, rows // 256))
        Wsel = np.concatenate([W[r * rb:(r + 1) * rb] for r in sel])
        y32, y64 = oracle.matvec(dtype, Wsel, sel.size, cols, x)
        _check(got[sel], y32, y64, f"sample {rows}x{cols}")
        assert np.isfinite(got).all()


def test_q6k_lm_head_all_rows(ctx, oracle):
    """The tied lm_head at its full size, 262144 x 1536 Q6_K with signed scales: every row against the oracle."""
    from ksearch_b200 import model as ksm
    rows, cols = 262144, 1536
    cfg = ksm.e2b_config()
    W = ksm.synth_tensor(cfg, 77, "token_embd.weight", "embd", rows, cols)
    x = synth.normals(77, "x", cols)
    y = ctx.buffer_empty_f32(rows)
    bw = ctx.buffer_bytes(W)
    Eng().matvec_wd(ctx, rows, cols, Q6K, bw, ctx.buffer_bytes(x), y)
    got = ctx.read_f32(y, rows)
    y32, y64 = oracle.matvec(Q6K, W, rows, cols, x)
    _check(got, y32, y64, "lm_head 262144x1536")
    bw.free()


def test_matvec_host_entry(ctx, oracle):
    rows, cols = 512, 1536
    W = _gen(Q4K, 70, "W", rows, cols)
    x = synth.normals(70, "x", 2 * cols)
    y = np.empty(2 * rows, np.float32)
    bw = ctx.buffer_bytes(W)
    ctx.check(ctx.lib.ks_matvec_host(ctx.h, rows, cols, Q4K, bw.h, 0, x.ctypes.data, y.ctypes.data, 2))
    y32, y64 = oracle.matvec(Q4K, W, rows, cols, x.reshape(2, cols))
    _check(y.reshape(2, rows), y32, y64, "matvec_host")


def test_matvec_errors(ctx):
    e = Eng()
    W = ctx.buffer_bytes(synth.q4k_matrix(71, "W", 8, 512))
    x, y = ctx.buffer_empty_f32(512), ctx.buffer_empty_f32(8)
    with pytest.raises(KsError, match="multiple of 256"):
        e.matvec_wd(ctx, 8, 500, Q4K, W, x, y)
    with pytest.raises(KsError, match="too small"):
        e.matvec_wd(ctx, 16, 512, Q4K, W, x, y)
    with pytest.raises(KsError, match="not supported"):
        e.matvec_wd(ctx, 8, 512, F16, W, x, y)
    with pytest.raises(KsError, match="n_tok"):
        e.matvec_batch(ctx, 8, 512, 0, Q4K, W, x, y)
    with pytest.raises(KsError, match="y buffer"):
        e.matvec_wd_at(ctx, 8, 512, Q4K, W, x, 0, y, 4)
    with pytest.raises(KsError):
        e.matvec_gate_up_gelu_wd(ctx, 8, 512, Q6K, W, W, x, y)


@pytest.mark.parametrize("act", [F32, F16])
def test_rmsnorm_fused_into_matvec(ctx, oracle, act):
    """K:278 / K:379 / K:1004 and the fused residual update: same numbers as norm kernel + matvec."""
    e = Eng(act)
    npdt = np.float32 if act == F32 else np.float16
    cols, rows, kv_rows, eps = 1536, 512, 256, 1e-6
    sig = 0.01 if act == F32 else 0.0005
    W, Wk, Wv = (_gen(Q4K, 72, n, r, cols, sigma=sig) for n, r in (("q", rows), ("k", kv_rows), ("v", kv_rows)))
    x = (synth.normals(72, "x", cols) * 2).astype(npdt)
    yp = synth.normals(72, "yp", cols).astype(npdt)
    wn = synth.norm_weight(72, "wn", cols).astype(npdt)
    wp = synth.norm_weight(72, "wp", cols).astype(npdt)
    bx, byp, bwn, bwp = map(ctx.buffer_bytes, (x, yp, wn, wp))
    f = lambda a: a.astype(np.float32)
    tol = dict(rtol=1e-3, atol=1e-4) if act == F32 else dict(rtol=4e-3, atol=4e-3)

    # plain norm + matvec
    x2 = oracle.rmsnorm(f(x), f(wn), eps)
    if act == F16:
        x2 = x2.astype(np.float16).astype(np.float32)
    y = ctx.buffer_empty_bytes(rows * x.itemsize)
    e.rmsnorm_matvec_wd(ctx, rows, cols, eps, Q4K, bx, bwn, ctx.buffer_bytes(W), y)
    _, y64 = oracle.matvec(Q4K, W, rows, cols, x2)
    assert_close(ctx.read_act(y, rows, act), y64, what="rmsnorm_matvec", **tol)

    # residual update + norm + fused QKV
    ox, ox2 = oracle.rmsnorm_add_then_rmsnorm(f(yp), f(wp), f(x), f(wn), eps)
    if act == F16:
        ox2 = oracle.rmsnorm(ox.astype(np.float16).astype(np.float32), f(wn), eps).astype(np.float16).astype(np.float32)
    q, k, v = (ctx.buffer_empty_bytes(r * x.itemsize) for r in (rows, kv_rows, kv_rows))
    out_x = ctx.buffer_empty_bytes(x.nbytes)
    e.rmsnorm_matvec_qkv_wd(ctx, rows, kv_rows, cols, eps, Q4K, bx, bwn, *map(ctx.buffer_bytes, (W, Wk, Wv)), q, k, v,
                            y_prev=byp, w_post=bwp, out_x=out_x)
    assert_close(ctx.read_act(out_x, cols, act), ox, what="out_x", **(dict(rtol=1e-3, atol=1e-4) if act == F32 else dict(rtol=2e-3, atol=2e-3)))
    for buf, Wm, r in ((q, W, rows), (k, Wk, kv_rows), (v, Wv, kv_rows)):
        _, y64 = oracle.matvec(Q4K, Wm, r, cols, ox2)
        assert_close(ctx.read_act(buf, r, act), y64, what="fused qkv", **tol)

    # gate/up with the norm fused
    Wg, Wu = _gen(Q4K, 72, "g", rows, cols, sigma=0.0005), _gen(Q4K, 72, "u", rows, cols, sigma=0.0005)
    yy = ctx.buffer_empty_bytes(rows * x.itemsize)
    e.rmsnorm_matvec_gate_up_gelu_wd(ctx, rows, cols, eps, Q4K, bx, bwn, ctx.buffer_bytes(Wg), ctx.buffer_bytes(Wu), yy)
    _, g64 = oracle.matvec(Q4K, Wg, rows, cols, x2)
    _, u64 = oracle.matvec(Q4K, Wu, rows, cols, x2)
    want = oracle.gelu_mul(g64.astype(np.float32), u64.astype(np.float32))
    got = ctx.read_act(yy, rows, act)
    k_ = 1.0 if act == F32 else 4.0
    assert np.all(np.abs(got - want) <= k_ * (1e-4 + 2e-3 * np.abs(want) + 1e-4 * (np.abs(g64) + np.abs(u64))))

    with pytest.raises(KsError, match="alias"):
        e.rmsnorm_matvec_wd(ctx, rows, cols, eps, Q4K, bx, bwn, ctx.buffer_bytes(W), y, y_prev=byp, w_post=bwp, out_x=bx)
    with pytest.raises(KsError, match="go together"):
        e.rmsnorm_matvec_wd(ctx, rows, cols, eps, Q4K, bx, bwn, ctx.buffer_bytes(W), y, y_prev=byp)
    with pytest.raises(KsError):   # 6144 columns: no fused norm
        e.rmsnorm_matvec_wd(ctx, 8, 6144, eps, Q4K, bx, bwn, ctx.buffer_bytes(W), y)


@pytest.mark.parametrize("rows,cols", [(4096, 4096), (6144, 1536), (1536, 6144), (2560, 10240), (10240, 2560), (130, 2048), (7, 768), (64, 512)])
def test_matvec_q4k_fixed_point_variant(ctx, oracle, rows, cols):
    """Planner variant 3: rows out of a shared-memory ring against a block fixed-point x (exact integer
    products); the same bounds as the f32 kernels."""
    from ksearch_b200 import _lib
    W = _gen(Q4K, 73, f"W{rows}x{cols}", rows, cols)
    x = synth.normals(73, "x", cols)
    y = ctx.buffer_empty_f32(rows)
    bw = ctx.buffer_bytes(W)
    for cps in (1, 2):
        ctx.plan_override(_lib.Plan(3, 0, 8, cps, 0.0))
        try:
            n0 = ctx.launch_count()
            Eng().matvec_wd(ctx, rows, cols, Q4K, bw, ctx.buffer_bytes(x), y)
            got = ctx.read_f32(y, rows)
        finally:
            ctx.plan_override(None)
        assert ctx.launch_count() == n0 + 1
        y32, y64 = oracle.matvec(Q4K, W, rows, cols, x)
        _check(got, y32, y64, f"fx {rows}x{cols} cps={cps}")
    bw.free()


@pytest.mark.parametrize("rows,cols", [(512, 1536), (4096, 1536), (1024, 2560), (8, 256), (264, 768)])
def test_matvec_q6k_ring_variant(ctx, oracle, rows, cols):
    """Planner variant 4: the Q6_K rows streamed through per-warp shared-memory rings (one bulk copy per 8 rows),
    the arithmetic of variant 2; signed scales; two and three stages."""
    from ksearch_b200 import _lib
    W = synth.q6k_matrix(74, f"W{rows}x{cols}", rows, cols, signed_scales=True)
    x = synth.normals(74, "x", cols)
    y = ctx.buffer_empty_f32(rows)
    bw = ctx.buffer_bytes(W)
    y32, y64 = oracle.matvec(Q6K, W, rows, cols, x)
    for stages, nw in ((2, 8), (3, 6)):
        ctx.plan_override(_lib.Plan(4 | (stages << 8), 2, nw, 1, 0.0))
        try:
            Eng().matvec_wd(ctx, rows, cols, Q6K, bw, ctx.buffer_bytes(x), y)
            got = ctx.read_f32(y, rows)
        finally:
            ctx.plan_override(None)
        _check(got, y32, y64, f"q6k ring {rows}x{cols} stages={stages}")
    bw.free()
