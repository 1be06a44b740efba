#!/usr/bin/env python
"""Decode benchmark of the B200 backend on the E2B-shaped synthetic model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one greedy decode token: the whole forward pass (35 layers + Q6_K lm_head +
softcap argmax) for one slot.  Rank 0 prints ONE JSON line.

  value     decode tok/s with everything resident on the device: K graph replays back to
            back, the token id chained on the device, timed with CUDA events on the
            context's stream.
  e2e       the same through the blocking C-ABI call ks_model_decode_token with HOST token
            ids in and out every step (4 B up, 4 B down), host wall clock.
  roofline  the dominant kernel, timed alone with CUDA events over the model's own 35 layers
            of weights (371 MB of gate/up matrices, or the 330 MB lm_head: larger than L2, so
            every launch streams from HBM), against MEASURED_PEAKS.json's copy bandwidth.
  cpu_baseline  the CPU restatement of the reference's dequant + f32 dot decoder, timed on
            this host's cores on a bounded sample (N=1, rank 0).

With --gpus N > 1 (under torchrun) every rank owns a full model replica and one slot:
independent serve slots, no collective on the data path; value is the sum over ranks
("scaling": "weak").  --impl reference times the CPU decoder instead (rank 0 only).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEED = 1234
PROMPT_LEN = 64
FALLBACK_HBM_GBS = 6650.0


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons during the timed region."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.lines, self.proc = device, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.device)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._pump, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def run_reference(args, rank, world):
    """The reference's CPU path (dequant + f32 dot decoder restated in C), all host threads."""
    if rank != 0:
        return
    from ksearch_b200 import model as ksm
    from ksearch_b200 import synth
    from oracle import ks_oracle
    full = ksm.e2b_config(max_seq=PROMPT_LEN + 8)
    cores = os.cpu_count() or 1
    # Bounded sample: a model cut to `ls` layers and the same fraction of lm_head rows; per-token time
    # scales with streamed bytes, so tok/s(full) = tok/s(sample) * bytes(sample) / bytes(full).
    budget_s = 150.0
    ls = 2
    cfg = ksm.e2b_config(max_seq=args.steps + args.warmup + 8)
    cfg.n_layers = ls
    cfg.vocab = max(256, full.vocab * ls // full.n_layers // 256 * 256)
    T = ksm.synth_tensors(cfg, SEED)
    dec = ks_oracle.CpuDecoder(ks_oracle.decoder_cfg(cfg), T, fast=True)
    tok = 17
    t0 = time.perf_counter()
    tok = dec.forward_token(tok, True)
    t_one = time.perf_counter() - t0
    total = args.steps + args.warmup
    if t_one * total > budget_s and ls > 1:
        pass  # already the smallest sample that keeps every op of the layer loop
    frac = ksm.weight_bytes_per_token(cfg) / ksm.weight_bytes_per_token(full)
    for _ in range(args.warmup):
        tok = dec.forward_token(tok % cfg.vocab, True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        tok = dec.forward_token(tok % cfg.vocab, True)
    dt = time.perf_counter() - t0
    ms_sample = dt / max(1, args.steps) * 1e3
    ms_full = ms_sample / frac
    value = 1000.0 / ms_full
    sample = (f"{ls} of {full.n_layers} layers + {cfg.vocab} of {full.vocab} lm_head rows per step "
              f"({frac:.4f} of a token's weight bytes), scaled to a full token by bytes")
    line = {
        "impl": "reference", "metric": "decode_tok_s_e2b_q4k", "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_full, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(full, args.gpus),
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(cfg, n_gpus):
    return {"workload": "E2B-shaped synthetic decoder: 35 layers, hidden 1536, GeGLU 6144, 8 q / 1 kv heads x 256, "
                        "vocab 262144, Q4_K layers, Q6_K tied lm_head, Q4_0 KV; 64-token prompt then greedy decode, "
                        "one slot per GPU",
            "weight_bytes_per_token": 1027031040, "prompt_len": PROMPT_LEN, "slots_per_gpu": 1,
            "parallelism": f"replicas x{n_gpus}, no collective on the data path",
            "l2": "weights (1.03 GB/token) are 8x the 126 MB L2, so every step streams them from HBM",
            "arithmetic": "f32 activations and accumulation; inside the persistent decode kernel and the lm_head the input vector "
                          "is 24-bit block fixed point (three int8 planes per 32 elements) and weight x input products are exact "
                          "dp4a integer sums, scaled back in f32"}


# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the persistent decode kernel on this
# workload (697.9 MB read + 1.0 MB written), from the ncu capture summarised in profiles/decode_layers_e2b.md.
DECODE_KERNEL_DRAM_TRAFFIC = 698972160


def time_kernel_alone(ctx, model, slot, lib, cfg, peak, steps):
    """CUDA-event timing of the heavy kernels alone, over the model's own weights."""
    from ksearch_b200 import Q4K, Q6K
    from ksearch_b200 import model as ksm
    model_h = model.h
    out = {}
    # The persistent decode kernel: steps without the head are embed + that kernel + a one-thread
    # position update, so their device time is the kernel's (the two small launches add ~2 us).
    n = max(4, min(steps, 32))
    for rep in range(2):
        ctx.timer_begin()
        for i in range(n):
            model.forward(slot, 1, [1 + i], False)
        ms = ctx.timer_end_ms() / n
    head = cfg.vocab * cfg.hidden // 256 * (210 if cfg.embd_dtype == Q6K else 144)
    nbytes = ksm.weight_bytes_per_token(cfg) - head
    out["decode_layers"] = {"kernel": "mega_kernel (all 35 layers of a token in one persistent launch: qkv | attention | "
                                      "o-proj | gate-up+GELU | down per layer, grid barriers between)",
                            "us": ms * 1e3, "bytes": nbytes, "gbs": nbytes / ms / 1e6, "launches_per_token": 1}
    x = ctx.buffer_bytes(np.random.default_rng(0).standard_normal(cfg.hidden).astype(np.float32))
    # gate/up: 35 distinct layer pairs, 10.6 MB each
    y = ctx.buffer_empty_f32(cfg.ffn)
    tb = lambda name: lib.ks_model_tensor_bytes(model_h, name.encode())
    bufs = []
    for l in range(cfg.n_layers):
        g = lib.ks_model_tensor_ptr(model_h, f"blk.{l}.ffn_gate.weight".encode())
        u = lib.ks_model_tensor_ptr(model_h, f"blk.{l}.ffn_up.weight".encode())
        bufs.append((lib.ks_buf_wrap(ctx.h, g, tb(f"blk.{l}.ffn_gate.weight")), lib.ks_buf_wrap(ctx.h, u, tb(f"blk.{l}.ffn_up.weight"))))
    ctx.graph_begin()   # one graph of 35 launches: device time, not host launch rate
    for g, u in bufs:
        ctx.check(lib.ks_matvec_gate_up_gelu(ctx.h, cfg.ffn, cfg.hidden, Q4K, g, u, 0, x.h, y.h))
    gr = ctx.graph_end()
    for rep in range(3):  # first passes warm
        ctx.timer_begin()
        ctx.graph_launch(gr)
        ms = ctx.timer_end_ms() / len(bufs)
    ctx.graph_free(gr)
    nbytes = 2 * cfg.ffn * cfg.hidden // 256 * 144 + 4 * cfg.hidden + 4 * cfg.ffn
    out["q4k_gate_up"] = {"kernel": "mvs_q4k_kernel (stand-alone gate||up+GELU, 2x6144x1536; the multi-slot path)",
                          "us": ms * 1e3, "bytes": nbytes, "gbs": nbytes / ms / 1e6, "launches_per_token": 0}
    for g, u in bufs:
        lib.ks_buf_free(ctx.h, g)
        lib.ks_buf_free(ctx.h, u)
    # lm_head: one 330 MB matrix (larger than L2 on its own)
    e = lib.ks_buf_wrap(ctx.h, lib.ks_model_tensor_ptr(model_h, b"token_embd.weight"), tb("token_embd.weight"))
    lg = ctx.buffer_empty_f32(cfg.vocab)
    for rep in range(2):
        ctx.timer_begin()
        for _ in range(4):
            ctx.check(lib.ks_matvec(ctx.h, cfg.vocab, cfg.hidden, Q6K, e, 0, 0, x.h, 0, lg.h, 0, 1))
        ms = ctx.timer_end_ms() / 4
    nbytes = cfg.vocab * cfg.hidden // 256 * 210 + 4 * cfg.hidden + 4 * cfg.vocab
    out["q6k_lm_head"] = {"kernel": "mv_q6k_fx_kernel (lm_head 262144x1536, planner-chosen variant)", "us": ms * 1e3, "bytes": nbytes,
                          "gbs": nbytes / ms / 1e6, "launches_per_token": 1}
    lib.ks_buf_free(ctx.h, e)
    return out


def gemv_config0(ctx, peak):
    """Config 0: Q4_K 4096x4096 matvec, fp32 x/y, over 48 distinct weight copies (453 MB > 2x L2),
    launches captured in one CUDA graph so the figure is device time, not host launch rate."""
    from ksearch_b200 import Q4K, synth
    rows = cols = 4096
    one = synth.q4k_matrix(SEED, "cfg0", rows, cols)
    ncopy = 48
    big = ctx.buffer_empty_bytes(one.nbytes * ncopy)
    for c in range(ncopy):
        ctx.write_buffer(big, one, c * one.nbytes)
    x = ctx.buffer_bytes(synth.normals(SEED, "cfg0/x", cols))
    y = ctx.buffer_empty_f32(rows)
    lib = ctx.lib
    lib.ks_plan_search(ctx.h, b"mv_q4k", rows, 0, cols, 1, None)   # load-time plan search for this shape, untimed
    ctx.graph_begin()
    for c in range(ncopy):
        ctx.check(lib.ks_matvec(ctx.h, rows, cols, Q4K, big.h, c * one.nbytes, 0, x.h, 0, y.h, 0, 1))
    g = ctx.graph_end()
    for _ in range(3):
        ctx.graph_launch(g)
    ctx.timer_begin()
    reps = 4
    for _ in range(reps):
        ctx.graph_launch(g)
    ms = ctx.timer_end_ms() / (reps * ncopy)
    ctx.graph_free(g)
    big.free()
    nbytes = one.nbytes + 4 * (rows + cols)
    return {"shape": "Q4_K 4096x4096, fp32 x/y", "us": ms * 1e3, "bytes": nbytes, "gbs": nbytes / ms / 1e6,
            "frac_of_measured_peak": nbytes / ms / 1e6 / peak, "frac_of_8000": nbytes / ms / 1e6 / 8000.0,
            "launches_timed": reps * ncopy, "cold_l2": f"{ncopy} rotating weight copies ({ncopy * one.nbytes / 1e6:.0f} MB)"}


def cpu_baseline(cfg_full):
    """Oracle CPU decoder on a bounded sample of the same workload."""
    from ksearch_b200 import model as ksm
    from oracle import ks_oracle
    cfg = ksm.e2b_config(max_seq=80)
    ls = 2
    cfg.n_layers = ls
    cfg.vocab = cfg_full.vocab * ls // cfg_full.n_layers // 256 * 256
    T = ksm.synth_tensors(cfg, SEED)
    dec = ks_oracle.CpuDecoder(ks_oracle.decoder_cfg(cfg), T, fast=True)
    frac = ksm.weight_bytes_per_token(cfg) / ksm.weight_bytes_per_token(cfg_full)
    tok = dec.forward_token(3, True)
    n, t0 = 0, time.perf_counter()
    while n < 3 or (time.perf_counter() - t0 < 10.0 and n < 64):
        tok = dec.forward_token(tok % cfg.vocab, True)
        n += 1
    dt = (time.perf_counter() - t0) / n
    dec.close()
    return {"value": frac / dt, "unit": "tok/s", "cores": os.cpu_count() or 1, "kind": "port",
            "sample": f"{n} tokens through {ls} of {cfg_full.n_layers} layers + {cfg.vocab} of {cfg_full.vocab} lm_head rows "
                      f"({frac:.4f} of a token's weight bytes), scaled to a full token by bytes; OpenMP over all host cores"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank, world, local = dist_env()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import ctypes as C
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from ksearch_b200 import CudaContext
    from ksearch_b200 import model as ksm
    from ksearch_b200 import synth
    peak, peak_kind = measured_peak()
    ctx = CudaContext(local, flags=1)  # bit 0: programmatic dependent launch
    lib = ctx.lib
    cfg = ksm.e2b_config(max_seq=PROMPT_LEN + args.steps * 2 + args.warmup * 2 + 16 + 64)
    model = ksm.GemmaCudaModel.synthetic(ctx, cfg, SEED + rank)
    plans_found = model.warm_plans(1)   # load-time plan search / per-chip cache, outside every timed region
    slot = model.slot_alloc()
    prompt = synth.token_ids(SEED + rank, "prompt", PROMPT_LEN, cfg.vocab)

    def barrier():
        ctx.synchronize()
        if dist is not None:
            import torch
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-resident decode: prompt, W warm-up steps, then exactly K timed steps
    for t in prompt[:-1]:
        model.forward(slot, 1, [int(t)], False)
    model.forward(slot, 1, [int(prompt[-1])], True)
    for _ in range(args.warmup - 1):
        model.forward(slot, 1, None, True)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    n0 = ctx.launch_count()
    ctx.timer_begin()
    for _ in range(args.steps):
        model.forward(slot, 1, None, True)
    ms = ctx.timer_end_ms()
    launches = ctx.launch_count() - n0
    barrier()

    # ---- end to end: host token ids in and out of every step through the blocking C-ABI call
    tok = 1
    for _ in range(args.warmup):
        tok = model.decode_token([tok], slot)[0]
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        tok = model.decode_token([tok], slot)[0]
    ctx.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop() if rank == 0 else None
    barrier()

    if dist is not None:
        import torch
        t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
        ln = torch.tensor([launches], device="cuda", dtype=torch.int64)
        dist.all_reduce(ln)
        launches = int(ln[0])

    if rank == 0:
        value = world * args.steps / (ms / 1e3)
        e2e = world * args.steps / (e2e_ms / 1e3)
        wb = ksm.weight_bytes_per_token(cfg)
        line = {
            "metric": "decode_tok_s_e2b_q4k", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(cfg, world),
            "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4,
                    "api": "ks_model_decode_token (blocking, host token ids in and out)"},
            "gpu_launches": launches, "clocks": clocks,
            "weight_stream": {"bytes_per_token": wb, "gbs_per_gpu": wb / (ms / args.steps) / 1e6,
                              "frac_of_peak": wb / (ms / args.steps) / 1e6 / peak, "peak_gbs": peak, "peak_kind": peak_kind},
        }
        if world == 1:
            alone = time_kernel_alone(ctx, model, slot, lib, cfg, peak, args.steps)
            share = {k: v["us"] * v["launches_per_token"] for k, v in alone.items()}
            dom = max(share, key=share.get)
            d = alone[dom]
            line["roofline"] = {"bound": "hbm", "kernel": d["kernel"], "achieved": d["gbs"], "peak": peak, "unit": "GB/s",
                                "frac": d["gbs"] / peak, "of": peak_kind,
                                "traffic": DECODE_KERNEL_DRAM_TRAFFIC if dom == "decode_layers" else None, "us_per_launch": d["us"],
                                "bytes_per_launch": d["bytes"]}
            line["kernels_alone"] = alone
            line["gemv_config0"] = gemv_config0(ctx, peak)
            if not args.no_cpu_baseline:
                line["cpu_baseline"] = cpu_baseline(cfg)
        print(json.dumps(line), flush=True)
    model.close()
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
