"""Row-sharded matvec through the C ABI: ks_comm_*, ks_matvec_sharded (in-place NCCL all-gather on the
context's stream) and ks_argmax_sharded (one (value, index) pair per rank).  The 2-rank cases need 2 GPUs
and are skipped on a 1-GPU box; the 1-rank case runs everywhere."""
import os

import numpy as np
import pytest

from ksearch_b200 import shard, synth

pytestmark = pytest.mark.gpu
Q4K, Q6K = 2, 3


def _case(dtype, rows, cols):
    gen = synth.q6k_matrix if dtype == Q6K else synth.q4k_matrix
    kw = dict(signed_scales=True) if dtype == Q6K else {}
    return gen(92, "W", rows, cols, **kw), synth.normals(92, "x", cols)


def test_sharded_entry_points_one_rank(ctx, oracle):
    """n_ranks == 1 needs no NCCL: the same entry points, the whole matrix local."""
    rows, cols, cap = 4096, 1536, 30.0
    W, x = _case(Q6K, rows, cols)
    comm = shard.Comm(ctx, 1, 0, None)
    sm = shard.ShardedMatvec(ctx, comm, Q6K, rows, cols, W)
    y = sm.forward(x)
    _, y64 = oracle.matvec(Q6K, W, rows, cols, x)
    assert np.all(np.abs(y - y64) <= 1e-4 + 1e-3 * np.abs(y64))
    tok = sm.argmax(x, cap)
    want, _ = oracle.softcap_argmax(y.astype(np.float32), cap)
    assert tok == want
    comm.close()


def _gpu_rank(rank, world, uid_q, out_q, dtype, rows, cols, cap):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from ksearch_b200 import CudaContext
    ctx = CudaContext(rank, flags=1)
    if rank == 0:
        uid = shard.Comm.unique_id(ctx.lib)
        for _ in range(world - 1):
            uid_q.put(uid)
    else:
        uid = uid_q.get(timeout=120)
    comm = shard.Comm(ctx, world, rank, uid)
    W, x = _case(dtype, rows, cols)
    off, nb = shard.shard_byte_range(dtype, rows, cols, world, rank)
    sm = shard.ShardedMatvec(ctx, comm, dtype, rows, cols, W[off:off + nb])
    y = sm.forward(x)
    tok = sm.argmax(x, cap)
    # the same two steps captured in one graph and replayed: nothing in them synchronises or allocates
    ctx.graph_begin()
    sm.enqueue(True)
    g = ctx.graph_end()
    ctx.graph_launch(g)
    y2 = shard.gather_rows(list(ctx.read_f32(sm.y_all, world * sm.per).reshape(world, sm.per)), rows, world)
    ctx.graph_free(g)
    out_q.put((rank, y, tok, bool(np.array_equal(y, y2))))
    comm.close()
    ctx.close()


@pytest.mark.parametrize("dtype,rows,cols", [(Q6K, 4096, 1536), (Q4K, 6144, 1536)])
def test_sharded_matvec_two_gpus(oracle, dtype, rows, cols):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    world, cap = 2, 30.0
    c = mp.get_context("spawn")
    uid_q, out_q = c.Queue(), c.Queue()
    procs = [c.Process(target=_gpu_rank, args=(r, world, uid_q, out_q, dtype, rows, cols, cap)) for r in range(world)]
    for p in procs:
        p.start()
    res = [out_q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    W, x = _case(dtype, rows, cols)
    _, y64 = oracle.matvec(dtype, W, rows, cols, x)
    for rank, y, tok, same in res:
        assert np.all(np.abs(y - y64) <= 1e-4 + 1e-3 * np.abs(y64)), rank   # every rank holds the whole gathered vector
        want, _ = oracle.softcap_argmax(y.astype(np.float32), cap)
        assert tok == want and same
