"""Batches of more than 8 token rows: the tensor-core GEMM behind matvec_batch (crates/ksearch_kernels/src/lib.rs:1414
routes them to mul_mm, crates/ksearch_codegen/src/render.rs:1073-1291).  Checked against the CPU dequant + dot of
check_mul_mm.rs:60-71 (f32 sequential and f64) on the same inputs, with the single-token tolerance: the kernel
splits both operands into two f16 terms, so it is held to f32 accuracy, not to the reference's 0.05."""
import numpy as np
import pytest

from ksearch_b200 import Q4K, Q6K, Eng, KsError, synth
from tests.test_gpu_matvec import _gen


def _check(y, y32, y64, what):
    y, y64 = np.asarray(y, np.float64), np.asarray(y64, np.float64)
    scale = np.abs(y64).max()
    err = np.abs(y - y64)
    bad = err > 1e-3 * np.abs(y64) + 1e-5 * scale
    assert not bad.any(), f"{what}: {int(bad.sum())}/{y.size} outside tolerance, worst {err.max() / scale:.2e} of the output scale"
    assert np.abs(y - np.asarray(y32, np.float64)).max() <= 2e-5 * scale + 1e-4, what

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [Q4K, Q6K])
@pytest.mark.parametrize("rows,cols,batch", [
    (128, 256, 9), (64, 256, 16), (96, 1536, 17), (300, 768, 33), (128, 2560, 64), (257, 1536, 100),
    (256, 1024, 128), (130, 512, 255), (128, 512, 256),
])
def test_gemm_vs_oracle(ctx, oracle, dtype, rows, cols, batch):
    """Row counts off the 128-row tile, token counts off the 16-column granule, 1..40 k-steps."""
    W = _gen(dtype, 81, f"W{rows}x{cols}", rows, cols)
    x = synth.normals(81, f"x{batch}", batch * cols).reshape(batch, cols)
    y = ctx.buffer_empty_f32(batch * rows + 16)
    launches = ctx.launch_count()
    bw, bx = ctx.buffer_bytes(W), ctx.buffer_bytes(x)
    ctx.check(ctx.lib.ks_matvec(ctx.h, rows, cols, dtype, bw.h, 0, 0, bx.h, 0, y.h, 8, batch))
    assert ctx.launch_count() in (launches + 2, launches + 3)   # operand split + GEMM (+ sum of k-split partials)
    got = ctx.read_f32(y, batch * rows + 16)
    assert not got[:8].any() and not got[8 + batch * rows:].any()
    y32, y64 = oracle.matvec(dtype, W, rows, cols, x)
    _check(got[8:8 + batch * rows].reshape(batch, rows), np.atleast_2d(y32), np.atleast_2d(y64), f"gemm {rows}x{cols}x{batch}")


def test_gemm_reference_patterns(ctx, oracle):
    """check_mul_mm.rs:47-109,300-304: integer-pattern W through the reference quantizer, pattern x, the example's
    own shapes (rows x cols x batch)."""
    for rows, cols, batch in ((64, 256, 16), (128, 256, 9), (2048, 1536, 256), (4096, 1536, 256), (4096, 1536, 55)):
        r, c, t = np.arange(rows)[:, None], np.arange(cols)[None, :], np.arange(batch)[:, None]
        w = ((((r * 17 + c * 13) % 200).astype(np.float32) - 100.0) * np.float32(0.02)).astype(np.float32)
        x = ((((t * 11 + c * 7) % 50).astype(np.float32) - 25.0) * np.float32(0.04)).astype(np.float32)
        wq = oracle.quantize_q4k(w.ravel())
        y32, y64 = oracle.matvec(Q4K, wq, rows, cols, x)
        by = ctx.buffer_empty_f32(batch * rows)
        Eng().matvec_batch(ctx, rows, cols, batch, Q4K, ctx.buffer_bytes(wq), ctx.buffer_bytes(x), by)
        got = ctx.read_f32(by, batch * rows).reshape(batch, rows)
        _check(got, y32, y64, f"pattern {rows}x{cols}x{batch}")


def test_gemm_same_as_single_rows(ctx, oracle):
    """Every row of a batch equals the single-token matvec of that row within the shared tolerance, and a batch
    that repeats one row gives identical outputs for every copy."""
    rows, cols, batch = 384, 1536, 40
    W = _gen(Q4K, 82, "W", rows, cols)
    x1 = synth.normals(82, "x", cols)
    x = np.tile(x1, (batch, 1))
    y = ctx.buffer_empty_f32(batch * rows)
    Eng().matvec_batch(ctx, rows, cols, batch, Q4K, ctx.buffer_bytes(W), ctx.buffer_bytes(x), y)
    got = ctx.read_f32(y, batch * rows).reshape(batch, rows)
    assert (got == got[0]).all()
    y1 = ctx.buffer_empty_f32(rows)
    Eng().matvec_wd(ctx, rows, cols, Q4K, ctx.buffer_bytes(W), ctx.buffer_bytes(x1), y1)
    one = ctx.read_f32(y1, rows)
    assert np.abs(got[0] - one).max() <= 1e-5 * np.abs(one).max() + 1e-5
    y64 = oracle.matvec(Q4K, W, rows, cols, x1)[1]
    print(f"[gemm vs f64] worst {np.abs(got[0] - y64).max() / np.abs(y64).max():.2e} of the output scale; "
          f"single-token kernel {np.abs(one - y64).max() / np.abs(y64).max():.2e}")


def test_gemm_errors(ctx):
    e = Eng()
    W = ctx.buffer_bytes(synth.q4k_matrix(71, "W", 8, 512))
    x, y = ctx.buffer_empty_f32(512 * 300), ctx.buffer_empty_f32(8 * 300)
    with pytest.raises(KsError, match="n_tok"):
        e.matvec_batch(ctx, 8, 512, 257, Q4K, W, x, y)
    with pytest.raises(KsError, match="x buffer"):
        e.matvec_batch(ctx, 8, 512, 16, Q4K, W, ctx.buffer_empty_f32(512 * 15), y)


@pytest.mark.parametrize("batch,stall", [(16, 1), (128, 1), (200, 1)])
def test_gemm_wait_gives_up_and_recovers(oracle, monkeypatch, batch, stall):
    """A bounded wait of the GEMM kernel that runs out, without a fault or a hang: with KSEARCH_GEMM_TEST_STALL=k the
    warp that requests the token rows withholds the copy of k-step k - 1 in every CTA and every wait gives up after
    4000 polls.  The MMA warp stops waiting for the operand, the dequantising warps for their stage, the CTA awaits
    what it has in flight, frees its tensor memory and leaves; the next synchronize reports KS_ERR_TIMEOUT, and
    the same call without the hook is correct again."""
    from ksearch_b200 import CudaContext, _lib
    c = CudaContext(0, flags=1)
    rows, cols = 512, 1536
    W = _gen(Q4K, 91, "Wstall", rows, cols)
    x = synth.normals(91, "xstall", batch * cols).reshape(batch, cols)
    bw, bx, y = c.buffer_bytes(W), c.buffer_bytes(x), c.buffer_empty_f32(batch * rows)
    monkeypatch.setenv("KSEARCH_GEMM_TEST_STALL", str(stall))
    c.check(c.lib.ks_matvec(c.h, rows, cols, Q4K, bw.h, 0, 0, bx.h, 0, y.h, 0, batch))   # enqueues fine
    with pytest.raises(KsError) as ei:
        c.synchronize()
    assert ei.value.code == _lib.ERR_TIMEOUT
    c.synchronize()                                                                       # the status word was cleared
    monkeypatch.delenv("KSEARCH_GEMM_TEST_STALL")
    c.check(c.lib.ks_matvec(c.h, rows, cols, Q4K, bw.h, 0, 0, bx.h, 0, y.h, 0, batch))
    c.synchronize()
    y32, y64 = oracle.matvec(Q4K, W, rows, cols, x)
    _check(c.read_f32(y, batch * rows).reshape(batch, rows), np.atleast_2d(y32), np.atleast_2d(y64), "gemm after a give-up")
    c.close()


@pytest.mark.parametrize("dtype", [Q4K, Q6K])
def test_gemm_token_rows_beyond_the_f16_range(ctx, oracle, dtype):
    """Token rows whose values leave the f16 range (65504): the operand image stores such a row scaled by a power
    of two and the kernel scales its outputs back, so the result still matches the f64 CPU result.  Rows of small,
    ordinary and huge magnitude side by side in one batch."""
    rows, cols, batch = 256, 1024, 12
    W = _gen(dtype, 83, "Wrange", rows, cols)
    x = synth.normals(83, "xrange", batch * cols).reshape(batch, cols).astype(np.float32)
    x[1] *= 1e-4
    x[2] *= 3.0e4        # peaks near 1e5: past the f16 range
    x[5] *= 1.0e9
    x[7, 100] = 7.0e5    # one outlier in an ordinary row
    x[9] *= 2.5e30
    y = ctx.buffer_empty_f32(batch * rows)
    bw, bx = ctx.buffer_bytes(W), ctx.buffer_bytes(x)
    ctx.check(ctx.lib.ks_matvec(ctx.h, rows, cols, dtype, bw.h, 0, 0, bx.h, 0, y.h, 0, batch))
    got = ctx.read_f32(y, batch * rows).reshape(batch, rows).astype(np.float64)
    assert np.isfinite(got).all()
    _, y64 = oracle.matvec(dtype, W, rows, cols, x)
    y64 = np.atleast_2d(y64).astype(np.float64)
    for t in range(batch):                     # each row against its own scale
        scale = np.abs(y64[t]).max()
        err = np.abs(got[t] - y64[t])
        assert (err <= 1e-3 * np.abs(y64[t]) + 1e-5 * scale).all(), (t, err.max() / scale)
