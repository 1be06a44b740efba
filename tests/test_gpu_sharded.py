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


def _p2p_rank(rank, world, uid_q, h_qs, out_q, rows, cols, cap):
    """Peer-memory arg-max exchange: several steps with different x, against the NCCL path on the same inputs; then
    the bounded wait: rank 1 sits one step out, rank 0's wait runs out after 2000 polls (a status, not a hang),
    both ranks clear their mailboxes and the next step agrees again."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from ksearch_b200 import CudaContext, KsError, _lib
    ctx = CudaContext(rank, flags=1)
    if rank == 0:
        uid = shard.Comm.unique_id(ctx.lib)
        for _ in range(world - 1):
            uid_q.put(uid)
    else:
        uid = uid_q.get(timeout=120)
    comm = shard.Comm(ctx, world, rank, uid)
    mine = comm.p2p_handle()
    for r in range(world):                       # every rank's handle to every other rank (host queues)
        if r != rank:
            h_qs[r].put((rank, mine))
    handles = {rank: mine}
    while len(handles) < world:
        r, h = h_qs[rank].get(timeout=120)
        handles[r] = h
    comm.p2p_open(b"".join(handles[r] for r in range(world)))
    W = synth.q6k_matrix(92, "W", rows, cols, signed_scales=True)
    off, nb = shard.shard_byte_range(Q6K, rows, cols, world, rank)
    sm = shard.ShardedMatvec(ctx, comm, Q6K, rows, cols, W[off:off + nb])
    toks_p2p, toks_nccl = [], []
    for step in range(5):
        x = synth.normals(92, f"x{step}", cols)
        toks_p2p.append(sm.argmax(x, cap))
    comm.set(comm.USE_P2P, 0)
    for step in range(5):
        x = synth.normals(92, f"x{step}", cols)
        toks_nccl.append(sm.argmax(x, cap))
    comm.set(comm.USE_P2P, 1)
    # a graph of three exchanges replays like three calls
    x = synth.normals(92, "x0", cols)
    sm.set_x(x)
    ctx.graph_begin()
    for _ in range(3):
        sm.enqueue(False)
        sm.enqueue_argmax(cap)
    g = ctx.graph_end()
    ctx.graph_launch(g)
    tok_graph = int(ctx.read_f32(sm.tok, 1)[0])
    ctx.graph_free(g)
    # the give-up path, made on the host: rank 1 does not take part in one step
    timed_out = None
    if rank == 0:
        comm.set(comm.POLL_LIMIT, 2000)
        sm.enqueue(False)
        sm.enqueue_argmax(cap)
        try:
            ctx.synchronize()
            timed_out = False
        except KsError as e:
            timed_out = e.code == _lib.ERR_TIMEOUT
        comm.set(comm.POLL_LIMIT, 1 << 23)
    out_q.put(("phase1", rank))                  # both ranks idle from here: clear the mailboxes, then go on
    h_qs[rank].get(timeout=120)                  # the parent's go-ahead
    comm.set(comm.RESET, 0)
    out_q.put(("reset", rank))
    h_qs[rank].get(timeout=120)
    tok_after = sm.argmax(synth.normals(92, "x1", cols), cap)
    out_q.put(("done", rank, toks_p2p, toks_nccl, tok_graph, timed_out, tok_after))
    comm.close()
    ctx.close()


def test_sharded_argmax_over_peer_memory_two_gpus(oracle):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    world, cap, rows, cols = 2, 30.0, 4096, 1536
    c = mp.get_context("spawn")
    uid_q, out_q = c.Queue(), c.Queue()
    h_qs = [c.Queue() for _ in range(world)]
    procs = [c.Process(target=_p2p_rank, args=(r, world, uid_q, h_qs, out_q, rows, cols, cap)) for r in range(world)]
    for p in procs:
        p.start()
    for tag in ("phase1", "reset"):              # two host-side barriers: every rank reports, then every rank may go on
        got = [out_q.get(timeout=300) for _ in range(world)]
        assert all(g[0] == tag for g in got)
        for q in h_qs:
            q.put("go")
    res = [out_q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    W = synth.q6k_matrix(92, "W", rows, cols, signed_scales=True)
    want = []
    for step in range(5):
        _, y64 = oracle.matvec(Q6K, W, rows, cols, synth.normals(92, f"x{step}", cols))
        want.append(oracle.softcap_argmax(y64.astype(np.float32), cap)[0])
    for _, rank, toks_p2p, toks_nccl, tok_graph, timed_out, tok_after in res:
        assert toks_p2p == want and toks_nccl == want, rank
        assert tok_graph == want[0] and tok_after == want[1], rank
        if rank == 0:
            assert timed_out is True
