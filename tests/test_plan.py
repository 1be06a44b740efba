"""Planner: the on-disk plan cache needs no GPU; the timing search does."""
import ctypes as C
import os

import pytest

from ksearch_b200 import _lib


def test_plan_file_round_trip(tmp_path):
    lib = _lib.load()
    p = _lib.Plan((3 << 8) | (6 << 16), 2, 6, 2, 0.004321)
    d = str(tmp_path / "cache" / "beam").encode()
    assert lib.ks_plan_file_save(d, b"mv_q4k_4096x4096", b"NVIDIA B200", C.byref(p)) == 0
    name = C.create_string_buffer(256)
    assert lib.ks_plan_file_name(b"mv_q4k_4096x4096", b"NVIDIA B200", name, 256) == 0
    path = os.path.join(d.decode(), name.value.decode())
    text = open(path).read()
    assert "nr0=2" in text and "nsg=6" in text and "stages=3" in text and "chip=NVIDIA B200" in text
    q = _lib.Plan()
    assert lib.ks_plan_file_load(d, b"mv_q4k_4096x4096", b"NVIDIA B200", C.byref(q)) == 0
    assert (q.variant, q.nr, q.nwarps, q.ctas_per_sm) == (p.variant, 2, 6, 2) and abs(q.ms - p.ms) < 1e-6
    # the chip is part of the key: another chip does not see this plan (CG:63-66)
    assert lib.ks_plan_file_load(d, b"mv_q4k_4096x4096", b"Some Other GPU", C.byref(q)) != 0
    assert lib.ks_plan_file_load(d, b"mv_q4k_1x256", b"NVIDIA B200", C.byref(q)) != 0
    # a truncated file is not a plan
    open(path, "w").write("nr0=2\n")
    assert lib.ks_plan_file_load(d, b"mv_q4k_4096x4096", b"NVIDIA B200", C.byref(q)) != 0


def test_plan_candidates():
    lib = _lib.load()
    arr = (_lib.Plan * 64)()
    n = lib.ks_plan_candidates(b"mv_q4k", arr, 64)
    assert 16 <= n <= 64
    assert {(arr[i].variant & 0xFF) for i in range(n)} == {0, 1, 3}
    m = lib.ks_plan_candidates(b"gu_q4k", arr, 64)
    assert 0 < m < n and all(arr[i].nr in (1, 2, 4) for i in range(m))


@pytest.mark.gpu
def test_plan_search_caches_and_is_used(tmp_path, monkeypatch, oracle):
    import numpy as np
    from ksearch_b200 import CudaContext, Eng, Q4K, synth
    monkeypatch.setenv("KSEARCH_BEAM_CACHE", str(tmp_path))
    ctx = CudaContext(0)
    best = _lib.Plan()
    ctx.check(ctx.lib.ks_plan_search(ctx.h, b"mv_q4k", 2048, 0, 1536, 1, C.byref(best)))
    assert best.ms > 0 and len(os.listdir(tmp_path)) == 1
    got = _lib.Plan()
    assert ctx.lib.ks_plan_get(ctx.h, b"mv_q4k", 2048, 1536, 1, C.byref(got)) == 0
    assert (got.variant, got.nr, got.nwarps, got.ctas_per_sm) == (best.variant, best.nr, best.nwarps, best.ctas_per_sm)
    # a second context finds the file instead of searching (same plan, no new file)
    ctx2 = CudaContext(0)
    again = _lib.Plan()
    ctx2.check(ctx2.lib.ks_plan_search(ctx2.h, b"mv_q4k", 2048, 0, 1536, 1, C.byref(again)))
    assert (again.variant, again.nr, again.nwarps) == (best.variant, best.nr, best.nwarps) and len(os.listdir(tmp_path)) == 1
    # KSEARCH_SKIP_BEAM: no search for an unknown shape
    monkeypatch.setenv("KSEARCH_SKIP_BEAM", "1")
    assert ctx2.lib.ks_plan_search(ctx2.h, b"mv_q4k", 512, 0, 1536, 1, C.byref(again)) != 0
    # results do not depend on the plan in force
    W = synth.q4k_matrix(81, "W", 2048, 1536)
    x = synth.normals(81, "x", 1536)
    y = ctx.buffer_empty_f32(2048)
    Eng().matvec_wd(ctx, 2048, 1536, Q4K, ctx.buffer_bytes(W), ctx.buffer_bytes(x), y)
    _, y64 = oracle.matvec(Q4K, W, 2048, 1536, x)
    got_y = ctx.read_f32(y, 2048)
    assert np.all(np.abs(got_y - y64) <= 1e-4 + 1e-3 * np.abs(y64))
    ctx2.close()
    ctx.close()
