"""Row-sharded matvec across the GPUs of one box.

A K-quant matrix is row-major over blocks, so the rows [r0, r0+n) of rank k are one contiguous
byte range: sharding by output row needs no repacking.  x (a few KB) is replicated, every rank
computes its slice of y, and ONE exchange follows: an all-gather of the y slices (NCCL over
NVLink on GPUs, gloo in the CPU tests).  Where only the arg-max of y is wanted (the lm_head in
greedy decode), each rank reduces its own slice and 8 bytes per rank are gathered instead.

The reference has no multi-device code (crates/ksearch_metal/src/lib.rs:33 uses the system default
device); this module is new.  The GPU path goes through the C ABI (ks_comm_*, ks_matvec_sharded,
ks_argmax_sharded: NCCL on the context's stream); the row arithmetic below is shared with the CPU tests.
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


class Comm:
    """ks_comm of include/ksearch_cuda.h: one rank of the NCCL group the sharded ops exchange over."""

    ID_BYTES = 128

    def __init__(self, ctx, world: int, rank: int, unique_id: bytes | None):
        import ctypes as C
        self.ctx, self.world, self.rank = ctx, world, rank
        buf = C.create_string_buffer(unique_id, self.ID_BYTES) if unique_id is not None else None
        self.h = ctx.lib.ks_comm_init(ctx.h, world, rank, buf)
        if not self.h:
            from .eng import KsError
            raise KsError(-2, ctx.lib.ks_last_error(ctx.h).decode(errors="replace"))

    @staticmethod
    def unique_id(lib) -> bytes:
        """Rank 0 makes the rendezvous id; the other ranks get the bytes over any host channel."""
        import ctypes as C
        buf = C.create_string_buffer(Comm.ID_BYTES)
        rc = lib.ks_comm_unique_id(buf)
        if rc:
            from .eng import KsError
            raise KsError(rc, lib.ks_last_error(None).decode(errors="replace"))
        return buf.raw

    P2P_HANDLE_BYTES = 64
    USE_P2P, POLL_LIMIT, RESET = 0, 1, 2

    def p2p_handle(self) -> bytes:
        """This rank's mailbox for the peer-memory exchange, as the 64 bytes the other ranks open."""
        import ctypes as C
        buf = C.create_string_buffer(self.P2P_HANDLE_BYTES)
        self.ctx.check(self.ctx.lib.ks_comm_p2p_handle(self.h, buf))
        return buf.raw

    def p2p_open(self, all_handles: bytes):
        """all_handles: the handles of every rank, rank r's at r * 64 (gathered over any host channel)."""
        import ctypes as C
        assert len(all_handles) == self.world * self.P2P_HANDLE_BYTES
        self.ctx.check(self.ctx.lib.ks_comm_p2p_open(self.h, C.create_string_buffer(all_handles, len(all_handles))))

    def set(self, what: int, value: int):
        self.ctx.check(self.ctx.lib.ks_comm_set(self.h, what, value))

    def close(self):
        if self.h:
            self.ctx.lib.ks_comm_destroy(self.h)
            self.h = None


class ShardedMatvec:
    """One rank's share of y = W x and the exchange that follows, through the C ABI: x and the
    gathered y stay on the device, everything is enqueued on the context's stream.

    ctx: a CudaContext of this rank's GPU; comm: this rank's Comm; W_local: the rank's packed rows (uint8).
    """

    def __init__(self, ctx, comm: Comm, dtype: int, rows: int, cols: int, W_local: np.ndarray):
        self.ctx, self.comm, self.dtype, self.rows, self.cols = ctx, comm, dtype, rows, cols
        self.world, self.rank = comm.world, comm.rank
        self.r0, self.n = row_shard(rows, self.world, self.rank)
        self.per = padded_rows(rows, self.world)
        off, nb = shard_byte_range(dtype, rows, cols, self.world, self.rank)
        assert W_local.nbytes == nb, "W_local must be exactly this rank's rows"
        self.W = ctx.buffer_bytes(W_local) if nb else ctx.buffer_empty_bytes(16)
        self.y_all = ctx.buffer_empty_f32(self.world * self.per)
        self.x = ctx.buffer_empty_f32(cols)
        self.tok = ctx.buffer_empty_f32(1)

    def set_x(self, x_host: np.ndarray):
        self.ctx.write_buffer(self.x, np.asarray(x_host, np.float32))

    def enqueue(self, gather: bool = True):
        """Local rows into this rank's slot of y_all, then (gather) the in-place all-gather."""
        self.ctx.check(self.ctx.lib.ks_matvec_sharded(self.comm.h, self.n, self.per, self.cols, self.dtype, self.W.h, 0,
                                                      self.x.h, 0, self.y_all.h, 0, 1 if gather else 0))

    def enqueue_argmax(self, cap: float):
        """Greedy token from the local logits: one (value, index) pair per rank is gathered instead of the vector."""
        self.ctx.check(self.ctx.lib.ks_argmax_sharded(self.comm.h, self.n, self.r0, cap, self.y_all.h, self.rank * self.per,
                                                      self.tok.h, 0))

    def forward(self, x_host: np.ndarray) -> np.ndarray:
        self.set_x(x_host)
        self.enqueue(True)
        g = self.ctx.read_f32(self.y_all, self.world * self.per).reshape(self.world, self.per)
        return gather_rows(list(g), self.rows, self.world)

    def argmax(self, x_host: np.ndarray, cap: float) -> int:
        self.set_x(x_host)
        self.enqueue(False)
        self.enqueue_argmax(cap)
        return int(self.ctx.read_f32(self.tok, 1)[0])
