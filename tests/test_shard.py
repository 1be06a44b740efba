"""Row-sharding arithmetic and the gather layout, with 2 gloo ranks on CPU (the local matvec of each
rank is the CPU oracle); the NCCL path of the same code is a GPU test."""
import os
import socket

import numpy as np
import pytest

from ksearch_b200 import shard, synth

Q4K, Q6K = 2, 3


def test_row_shard_covers_rows_exactly():
    for rows in (1, 7, 8, 64, 1536, 2560, 6144, 262144, 1000):
        for world in (1, 2, 3, 4, 8):
            got = [shard.row_shard(rows, world, r) for r in range(world)]
            assert got[0][0] == 0 and sum(n for _, n in got) == rows
            for (a0, an), (b0, bn) in zip(got, got[1:]):
                assert a0 + an == b0
            assert all(n % 8 == 0 for _, n in got[:-1] if n and _ + n < rows)
            per = shard.padded_rows(rows, world)
            assert all(n <= per for _, n in got)
    with pytest.raises(ValueError):
        shard.row_shard(8, 2, 2)


def test_shard_byte_ranges_tile_the_matrix():
    for dt, bb in ((Q4K, 144), (Q6K, 210)):
        rows, cols = 262144, 1536
        total = rows * cols // 256 * bb
        pos = 0
        for r in range(8):
            off, n = shard.shard_byte_range(dt, rows, cols, 8, r)
            assert off == pos and off % 16 == 0
            pos += n
        assert pos == total
    with pytest.raises(ValueError):
        shard.shard_byte_range(Q4K, 8, 100, 2, 0)


def test_merge_argmax_prefers_lower_global_index():
    assert shard.merge_argmax([(1.0, 5), (3.0, 2), (3.0, 0)], [0, 100, 200]) == 102
    assert shard.merge_argmax([(3.0, 7), (3.0, 0)], [0, 8]) == 7


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, rows, cols, q):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import ks_oracle
    W = synth.q4k_matrix(91, "W", rows, cols)
    x = synth.normals(91, "x", cols)
    off, nb = shard.shard_byte_range(Q4K, rows, cols, world, rank)
    r0, n = shard.row_shard(rows, world, rank)
    per = shard.padded_rows(rows, world)
    mine = np.zeros(per, np.float32)
    if n:
        mine[:n] = ks_oracle.matvec(Q4K, W[off:off + nb], n, cols, x)[0]
    out = torch.empty(world * per)
    dist.all_gather_into_tensor(out, torch.from_numpy(mine))
    y = shard.gather_rows(list(out.numpy().reshape(world, per)), rows, world)
    # the 8-byte exchange: local arg-max + gather of (value, index)
    pair = torch.tensor([mine[:n].max() if n else -np.inf, float(mine[:n].argmax()) if n else 0.0])
    pairs = torch.empty(world * 2)
    dist.all_gather_into_tensor(pairs, pair)
    am = shard.merge_argmax(pairs.numpy().reshape(world, 2), [shard.row_shard(rows, world, k)[0] for k in range(world)])
    if rank == 0:
        q.put((y, am))
    dist.destroy_process_group()


@pytest.mark.parametrize("rows", [1000, 64])
def test_sharded_matvec_two_gloo_ranks(oracle, rows):
    import torch.multiprocessing as mp
    cols, world = 512, 2
    ctxm = mp.get_context("spawn")
    q = ctxm.Queue()
    port = _free_port()
    procs = [ctxm.Process(target=_rank_main, args=(r, world, port, rows, cols, q)) for r in range(world)]
    for p in procs:
        p.start()
    y, am = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    W = synth.q4k_matrix(91, "W", rows, cols)
    x = synth.normals(91, "x", cols)
    want = oracle.matvec(Q4K, W, rows, cols, x)[0]
    assert np.array_equal(y, want)             # sharding changes nothing, bit for bit
    assert am == int(np.argmax(want))
