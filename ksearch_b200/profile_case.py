"""Runs one op of the decode path a few times on seeded inputs: the small, self-ending case that
profiler captures are taken on.

    python -m ksearch_b200.profile_case matvec --dtype q4k --rows 4096 --cols 4096 --copies 16 --iters 2
    python -m ksearch_b200.profile_case gate_up --rows 6144 --cols 1536 --copies 16 --iters 2
    python -m ksearch_b200.profile_case matvec --dtype q4k --rows 20480 --cols 2560 --copies 6 --iters 2 --batch 128
    python -m ksearch_b200.profile_case decode --layers 4 --tokens 4
    python -m ksearch_b200.profile_case attn --kv 1 --ctx 16384 --slots 4 --copies 8 --iters 2

`--copies` distinct weight copies are cycled so that a launch never finds its weights in L2
(copies * matrix bytes should exceed the 126 MB L2).  Prints the CUDA-event time per launch.
"""
from __future__ import annotations

import argparse

import numpy as np

from . import Q4K, Q6K, CudaContext, Eng, synth
from . import model as ksm


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["matvec", "gate_up", "decode", "attn"])
    ap.add_argument("--dtype", default="q4k", choices=["q4k", "q6k"])
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--copies", type=int, default=16)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--tokens", type=int, default=4)
    ap.add_argument("--pdl", type=int, default=0)
    ap.add_argument("--kv", type=int, default=1, help="attn: KV heads (8 query heads)")
    ap.add_argument("--ctx", type=int, default=16384, help="attn: positions per slot")
    ap.add_argument("--slots", type=int, default=4, help="attn: slots")
    ap.add_argument("--batch", type=int, default=1, help="token rows per matvec call (more than 8: the tensor-core GEMM)")
    args = ap.parse_args()
    ctx = CudaContext(0, flags=args.pdl)
    eng = Eng()
    if args.op == "decode":
        cfg = ksm.e2b_config(max_seq=64)
        cfg.n_layers = args.layers
        cfg.vocab = 32768
        m = ksm.GemmaCudaModel.synthetic(ctx, cfg, 7)
        m.slot_alloc()
        m.forward(0, 1, [3], True)
        ctx.synchronize()
        ctx.timer_begin()
        for _ in range(args.tokens):
            m.forward(0, 1, None, True)
        ms = ctx.timer_end_ms()
        print(f"decode: {ms / args.tokens * 1e3:.1f} us/token over {args.tokens} tokens ({args.layers} layers, vocab {cfg.vocab})")
        return
    if args.op == "attn":
        from .eng import write_meta
        n_q, hd, rowb = 8, 256, 144
        slot_bytes = args.ctx * args.kv * rowb
        one = args.slots * slot_bytes
        K = synth.q40_rows(1, "K", one // 18 * 32, sigma=0.05)
        bK = ctx.buffer_empty_bytes(one * args.copies)
        bV = ctx.buffer_empty_bytes(one * args.copies)
        for c in range(args.copies):
            ctx.write_buffer(bK, K, c * one)
            ctx.write_buffer(bV, K, c * one)
        q = ctx.buffer_bytes(synth.normals(1, "q", args.slots * n_q * hd))
        o = ctx.buffer_empty_f32(args.slots * n_q * hd)
        meta = ctx.buffer_empty_f32(4 * args.slots)
        for s_ in range(args.slots):
            write_meta(ctx, meta, args.ctx, 0, 0, slot=s_)
        ns = ctx.lib.ks_sdpa_pick_splits(ctx.h, args.slots, args.kv, args.ctx)
        tmp = ctx.buffer_empty_f32(max(1, eng.sdpa_tmp_floats(n_q, hd, ns, args.slots)))
        ctx.synchronize()
        ctx.timer_begin()
        n = 0
        for _ in range(args.iters):
            for c in range(args.copies):
                ctx.check(ctx.lib.ks_sdpa_decode(ctx.h, args.slots, n_q, args.kv, hd, args.ctx, 4, 1.0 / 16.0, 0, q.h, bK.h, bV.h,
                                                 c * one, slot_bytes, meta.h, tmp.h, o.h, ns))
                n += 1
        ms = ctx.timer_end_ms()
        print(f"attn: {args.slots} slots x {args.ctx} positions, {args.kv} KV heads, {ns} splits: {ms / n * 1e3:.1f} us/call (host-paced)")
        return
    dt = Q4K if args.dtype == "q4k" else Q6K
    gen = synth.q4k_matrix if dt == Q4K else synth.q6k_matrix
    one = gen(1, "w", args.rows, args.cols)
    n_mat = 2 if args.op == "gate_up" else 1
    big = ctx.buffer_empty_bytes(one.nbytes * args.copies * n_mat)
    for c in range(args.copies * n_mat):
        ctx.write_buffer(big, one, c * one.nbytes)
    x = ctx.buffer_bytes(synth.normals(1, "x", args.cols * args.batch))
    y = ctx.buffer_empty_f32(args.rows * args.batch)
    lib = ctx.lib
    bufs = [lib.ks_buf_wrap(ctx.h, big.ptr + c * one.nbytes, one.nbytes) for c in range(args.copies * n_mat)]

    def launch(c):
        if args.op == "gate_up":
            ctx.check(lib.ks_matvec_gate_up_gelu(ctx.h, args.rows, args.cols, dt, bufs[2 * c], bufs[2 * c + 1], 0, x.h, y.h))
        else:
            ctx.check(lib.ks_matvec(ctx.h, args.rows, args.cols, dt, bufs[c], 0, 0, x.h, 0, y.h, 0, args.batch))

    for c in range(args.copies):   # first touch
        launch(c)
    ctx.synchronize()
    ctx.timer_begin()
    n = 0
    for _ in range(args.iters):
        for c in range(args.copies):
            launch(c)
            n += 1
    ms = ctx.timer_end_ms()
    nbytes = one.nbytes * n_mat + 4 * (args.rows + args.cols)
    print(f"{args.op} {args.dtype} {args.rows}x{args.cols}: {ms / n * 1e3:.2f} us/launch (host-paced), "
          f"{nbytes / (ms / n) / 1e6:.0f} GB/s algorithmic")


if __name__ == "__main__":
    main()
