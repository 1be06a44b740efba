"""The allocation-free arg-max entry point against the ordinary one, through the C ABI.

Collected last on purpose (file name): if it fails, a run that stops at the first failure has
already run everything else.  The entry point is for hosts that hold device pointers but may not
allocate device memory themselves; the TEST allocates its inputs and outputs through a context
(the entry point must not), then calls it twice in a row: the scratch array inside the library
keeps the first call's contents, so the second call checks that nothing stale leaks through.
"""
import ctypes as C

import numpy as np
import pytest

from ksearch_b200 import CudaContext, Eng, F32, synth

pytestmark = pytest.mark.gpu


def test_noalloc_argmax_matches_context_version_twice():
    ctx = CudaContext(0)
    lib = ctx.lib
    eng = Eng(F32)
    dev = lib.ks_ctx_device(ctx.h)
    out_ref = ctx.buffer_empty_f32(1)
    out_new = ctx.buffer_empty_f32(1)
    cases = [(262144, 7), (5000, 8)]          # second call is shorter: fewer blocks than the first left behind
    for n, seed in cases:
        x = synth.normals(seed, "logits", n, sigma=6.0)
        if seed == 8:
            x[[4000, 77, 2500]] = 40.0        # ties: the lower index must win in both versions
        bx = ctx.buffer_bytes(x)
        eng.softcap_argmax(ctx, n, 30.0, bx, out_ref)
        ctx.synchronize()
        rc = lib.ks_softcap_argmax_noalloc(dev, ctx.stream, n, 30.0, bx.ptr, out_new.ptr)
        assert rc == 0, lib.ks_last_error(None).decode()
        ctx.synchronize()
        a, b = ctx.read_f32(out_ref, 1)[0], ctx.read_f32(out_new, 1)[0]
        assert a == b, (n, a, b)              # an index: exact, no tolerance
        assert int(b) == (77 if seed == 8 else int(np.argmax(x)))
    # sizes beyond the fixed scratch are refused with a message, nothing is launched
    rc = lib.ks_softcap_argmax_noalloc(dev, ctx.stream, (1 << 22) + 1, 30.0, out_ref.ptr, out_new.ptr)
    assert rc != 0 and "limit" in lib.ks_last_error(None).decode()
    assert lib.ks_softcap_argmax_noalloc(dev, ctx.stream, 16, 30.0, None, out_new.ptr) != 0
    ctx.close()
