"""Row-sharded matvec across the GPUs of one box.

A K-quant matrix is row-major over blocks, so the rows [r0, r0+n) of rank k are one contiguous
byte range: sharding by output row needs no repacking.  x (a few KB) is replicated, every rank
computes its slice of y, and ONE exchange follows: an all-gather of the y slices (NCCL over
NVLink on GPUs, gloo in the CPU tests).  Where only the arg-max of y is wanted (the lm_head in
greedy decode), each rank reduces its own slice and 8 bytes per rank are gathered instead.

The reference has no multi-device code (crates/ksearch_metal/src/lib.rs:33 uses the system default
device); this module is new.  torch.distributed is plumbing here: process group, all-gather.
"""
from __future__ import annotations

import numpy as np

BLOCK_BYTES = {2: 144, 3: 210}  # Q4K, Q6K


def row_shard(rows: int, world: int, rank: int, align: int = 8) -> tuple[int, int]:
    """(first row, row count) of `rank`: contiguous, multiples of `align` except the last shard."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad world/rank")
    per = -(-rows // world)
    per = -(-per // align) * align
    r0 = min(rows, rank * per)
    return r0, min(rows, r0 + per) - r0


def shard_byte_range(dtype: int, rows: int, cols: int, world: int, rank: int, align: int = 8) -> tuple[int, int]:
    """(byte offset, byte count) of the rank's rows inside the packed matrix."""
    if cols % 256:
        raise ValueError("cols must be a multiple of 256")
    rb = cols // 256 * BLOCK_BYTES[dtype]
    r0, n = row_shard(rows, world, rank, align)
    return r0 * rb, n * rb


def padded_rows(rows: int, world: int, align: int = 8) -> int:
    """Rows per rank in the gathered buffer (all-gather wants equal counts)."""
    per = -(-rows // world)
    return -(-per // align) * align


def gather_rows(parts, rows: int, world: int, align: int = 8) -> np.ndarray:
    """Undo the padding of an all-gather: parts[k] holds padded_rows() values of rank k."""
    per = padded_rows(rows, world, align)
    out = np.empty(rows, dtype=np.asarray(parts[0]).dtype)
    for k in range(world):
        r0, n = row_shard(rows, world, k, align)
        out[r0:r0 + n] = np.asarray(parts[k])[:n]
        assert len(parts[k]) == per
    return out


def merge_argmax(pairs, row0s) -> int:
    """pairs[k] = (best value, local index) of rank k; the global arg-max, ties to the LOWER global
    index (crates/ksearch_codegen/src/render.rs:2355)."""
    best_v, best_i = -np.inf, -1
    for (v, i), r0 in zip(pairs, row0s):
        gi = int(i) + r0
        if v > best_v or (v == best_v and gi < best_i):
            best_v, best_i = float(v), gi
    return best_i


class ShardedMatvec:
    """One rank's share of y = W x and the exchange that follows.

    ctx: a CudaContext of this rank's GPU; W_local: the rank's packed rows (uint8).  all_gather runs on
    torch.distributed's default group (NCCL on GPUs).  The context's stream is synchronised before
    the collective, which is issued on torch's current stream.
    """

    def __init__(self, ctx, dtype: int, rows: int, cols: int, W_local: np.ndarray, world: int, rank: int):
        import torch  # noqa: F401  (plumbing only)
        self.ctx, self.dtype, self.rows, self.cols, self.world, self.rank = ctx, dtype, rows, cols, world, rank
        self.r0, self.n = row_shard(rows, world, rank)
        self.per = padded_rows(rows, world)
        off, nb = shard_byte_range(dtype, rows, cols, world, rank)
        assert W_local.nbytes == nb, "W_local must be exactly this rank's rows"
        self.W = ctx.buffer_bytes(W_local) if nb else None
        self.y_local = ctx.buffer_empty_f32(self.per)
        self.x = ctx.buffer_empty_f32(cols)

    def _as_tensor(self, buf, n):
        import torch

        class _Arr:
            __cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (buf.ptr, False), "version": 3}
        return torch.as_tensor(_Arr(), device=f"cuda:{self.ctx.lib.ks_ctx_device(self.ctx.h)}")

    def local(self, x_host: np.ndarray):
        self.ctx.write_buffer(self.x, np.asarray(x_host, np.float32))
        if self.n:
            self.ctx.check(self.ctx.lib.ks_matvec(self.ctx.h, self.n, self.cols, self.dtype, self.W.h, 0, 0,
                                                  self.x.h, 0, self.y_local.h, 0, 1))

    def all_gather(self):
        """Returns a torch tensor [world * per] with every rank's slice (padded)."""
        import torch
        import torch.distributed as dist
        self.ctx.synchronize()
        mine = self._as_tensor(self.y_local, self.per)
        out = torch.empty(self.world * self.per, dtype=torch.float32, device=mine.device)
        dist.all_gather_into_tensor(out, mine)
        return out

    def forward(self, x_host: np.ndarray) -> np.ndarray:
        self.local(x_host)
        g = self.all_gather().cpu().numpy().reshape(self.world, self.per)
        return gather_rows(list(g), self.rows, self.world)
