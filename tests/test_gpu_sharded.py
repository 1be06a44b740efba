"""Row-sharded lm_head-style matvec over 2 GPUs with an NCCL all-gather (skipped on a 1-GPU box)."""
import os

import numpy as np
import pytest

from ksearch_b200 import shard, synth

pytestmark = pytest.mark.gpu
Q6K = 3


def _gpu_rank(rank, world, port, rows, cols, q):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from ksearch_b200 import CudaContext
    ctx = CudaContext(rank)
    W = synth.q6k_matrix(92, "W", rows, cols, signed_scales=True)
    x = synth.normals(92, "x", cols)
    off, nb = shard.shard_byte_range(Q6K, rows, cols, world, rank)
    sm = shard.ShardedMatvec(ctx, Q6K, rows, cols, W[off:off + nb], world, rank)
    y = sm.forward(x)
    if rank == 0:
        q.put(y)
    dist.barrier()
    dist.destroy_process_group()
    ctx.close()


def test_sharded_matvec_two_gpus(oracle):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    from tests.test_shard import _free_port
    rows, cols, world = 4096, 1536, 2
    c = mp.get_context("spawn")
    q = c.Queue()
    port = _free_port()
    procs = [c.Process(target=_gpu_rank, args=(r, world, port, rows, cols, q)) for r in range(world)]
    for p in procs:
        p.start()
    y = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    W = synth.q6k_matrix(92, "W", rows, cols, signed_scales=True)
    x = synth.normals(92, "x", cols)
    _, y64 = oracle.matvec(Q6K, W, rows, cols, x)
    assert np.all(np.abs(y - y64) <= 1e-4 + 1e-3 * np.abs(y64))
