#!/usr/bin/env python
"""Decode benchmark of the B200 backend on the E2B-shaped synthetic model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one greedy decode token: the whole forward pass (35 layers + Q6_K lm_head +
softcap argmax) for one slot.  Rank 0 prints ONE JSON line.

  value     decode tok/s with everything resident on the device: K graph replays back to
            back, the token id chained on the device, timed with CUDA events on the
            context's stream.
  e2e       the same through the blocking C-ABI call ks_model_decode_token with HOST token
            ids in and out every step (4 B up, 8 B down), host wall clock.
  roofline  the dominant kernel (the persistent decode kernel: all 35 layers of a token),
            timed alone with CUDA events, against MEASURED_PEAKS.json's copy bandwidth.
  parity    the first greedy tokens of this very model and prompt against the CPU decoder.
  cpu_baseline  the CPU restatement of the reference's dequant + f32 dot decoder on the full
            model, timed on this host's cores (N=1, rank 0).
  kernels_alone, gemv_config0, matvec_shapes, attention   the other benchmark configurations'
            kernels, timed alone (medians of 5), weights rotated so every launch streams from HBM.
  serve_e4b the E4B-shaped serve workload: 8 slots spread over the GPUs, 512-token prompts,
            256 decoded tokens per slot.
  sharded   (N > 1) the row-sharded lm_head and FFN matvecs with their NCCL exchange.

With --gpus N > 1 (under torchrun) every rank owns a full model replica and one slot:
independent serve slots, no collective on the decode path; value is the sum over ranks
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
PARITY_TOKENS = 16
FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126 << 20

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the persistent decode kernel on the full 35-layer
# E2B shape, divided by 35 (ncu capture of this bench's own command at the last change of ks_mega.cu, commit bf56ad6:
# 698.50 MB read + 0.54 MB written per launch, median of three launches).
DECODE_KERNEL_DRAM_TRAFFIC_PER_LAYER = 19_973_000


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


def cpu_threads() -> int:
    """All host cores for the CPU decoder.  torchrun exports OMP_NUM_THREADS=1 to its workers, so the
    count is set explicitly, before the oracle's OpenMP runtime is loaded."""
    n = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(n)
    return n


def workload_config(n_gpus):
    return {"workload": "E2B-shaped synthetic decoder: 35 layers, hidden 1536, GeGLU 6144, 8 q / 1 kv heads x 256, "
                        "vocab 262144, Q4_K layers, Q6_K tied lm_head, Q4_0 KV; 64-token prompt then greedy decode, "
                        "one slot per GPU",
            "weight_bytes_per_token": 1027031040, "prompt_len": PROMPT_LEN, "slots_per_gpu": 1,
            "parallelism": f"replicas x{n_gpus}, no collective on the decode path",
            "l2": "weights (1.03 GB/token) are 8x the 126 MB L2, so every step streams them from HBM",
            "positions": "value and e2e are timed over the same positions: prompt, W warm-up tokens, then K tokens "
                         "(the slot is rewound and the prompt replayed before the e2e leg)",
            "arithmetic": "f32 activations and accumulation; inside the persistent decode kernel and the lm_head the input vector "
                          "is 24-bit block fixed point (three int8 planes per 32 elements) and weight x input products are exact "
                          "dp4a integer sums, scaled back in f32"}


def run_reference(args, rank, world, emit):
    """The reference's CPU path (dequant + f32 dot decoder restated in C) on the full model, all host threads:
    the benchmark's prompt, W warm-up tokens, then K timed greedy tokens."""
    if rank != 0:
        return
    threads = cpu_threads()
    from ksearch_b200 import model as ksm
    from ksearch_b200 import synth
    from oracle import ks_oracle
    cfg = ksm.e2b_config(max_seq=PROMPT_LEN + args.steps + args.warmup + 8)
    T = ksm.synth_tensors(cfg, SEED)
    dec = ks_oracle.CpuDecoder(ks_oracle.decoder_cfg(cfg), T, fast=True)
    prompt = synth.token_ids(SEED, "prompt", PROMPT_LEN, cfg.vocab)
    for t in prompt[:-1]:
        dec.forward_token(int(t), False)
    tok = int(prompt[-1])
    for _ in range(args.warmup):
        tok = dec.forward_token(tok, True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        tok = dec.forward_token(tok, True)
    dt = time.perf_counter() - t0
    value = args.steps / dt
    sample = (f"the full model (no scaling): {PROMPT_LEN}-token prompt, {args.warmup} warm-up tokens, then {args.steps} timed greedy "
              f"tokens; OpenMP over {threads} threads")
    line = {
        "impl": "reference", "metric": "decode_tok_s_e2b_q4k", "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": os.cpu_count() or 1, "threads": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def cpu_baseline_and_parity(cfg, T, prompt, gpu_tokens):
    """The CPU decoder on the full model and the benchmark's prompt: the first greedy tokens must be the GPU's
    (a differing token counts as a near-tie only if the CPU logits of the two candidates are within 2e-3 of the
    logit scale); the decode steps are timed."""
    threads = cpu_threads()
    from oracle import ks_oracle
    dec = ks_oracle.CpuDecoder(ks_oracle.decoder_cfg(cfg), T, fast=True)
    for t in prompt[:-1]:
        dec.forward_token(int(t), False)
    tok = int(prompt[-1])
    equal = ties = 0
    diverged = None
    t0 = time.perf_counter()
    for i, got in enumerate(gpu_tokens):
        want = dec.forward_token(tok, True)
        if want == got:
            equal += 1
        else:
            lg = dec.logits()
            gap = abs(float(lg[want]) - float(lg[got]))
            if gap <= 2e-3 * max(1.0, float(np.abs(lg).max())):
                ties += 1
            elif diverged is None:
                diverged = i
        tok = int(got)
    dt = time.perf_counter() - t0
    dec.close()
    n = len(gpu_tokens)
    base = {"value": n / dt, "unit": "tok/s", "cores": os.cpu_count() or 1, "threads": threads, "kind": "port",
            "sample": f"{n} greedy tokens of the full model after the {len(prompt)}-token prompt (no scaling), OpenMP over {threads} threads"}
    par = {"tokens_checked": n, "equal": equal, "near_ties": ties, "first_divergence": diverged,
           "against": "CPU decoder (oracle) on the same weights and prompt"}
    return base, par


def median_ms(ctx, fn, reps=5, warm=1):
    for _ in range(warm):
        fn()
    ctx.synchronize()
    out = []
    for _ in range(reps):
        ctx.timer_begin()
        fn()
        out.append(ctx.timer_end_ms())
    return float(np.median(out))


def graph_of(ctx, launches):
    ctx.graph_begin()
    for f in launches:
        f()
    return ctx.graph_end()


def time_kernels_alone(ctx, model, slot, cfg, peak, steps):
    """CUDA-event timing of the heavy kernels alone, over the model's own weights (medians of 5)."""
    from ksearch_b200 import Q4K, Q6K
    from ksearch_b200 import model as ksm
    lib, model_h = ctx.lib, model.h
    out = {}
    # The persistent decode kernel: steps without the head are embed + that kernel + a one-thread
    # position update, so their device time is the kernel's (the two small launches add ~2 us).
    n = max(8, min(steps, 32))
    model.slot_reset(slot)
    for i in range(PROMPT_LEN):   # the benchmark's context length, then 6 x n more positions
        model.forward(slot, 1, [1 + i], False)

    def layers_only():
        for i in range(n):
            model.forward(slot, 1, [1 + i], False)
    ms = median_ms(ctx, layers_only) / n
    head = cfg.vocab * cfg.hidden // 256 * (210 if cfg.embd_dtype == Q6K else 144)
    nbytes = ksm.weight_bytes_per_token(cfg) - head
    out["decode_layers"] = {"kernel": "mega_kernel (all 35 layers of a token in one persistent launch; q/k/v, attention, o-proj, "
                                      "gate/up + GELU, down per layer, a grid barrier between phases)",
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
    gr = graph_of(ctx, [lambda g=g, u=u: ctx.check(lib.ks_matvec_gate_up_gelu(ctx.h, cfg.ffn, cfg.hidden, Q4K, g, u, 0, x.h, y.h))
                        for g, u in bufs])
    ms = median_ms(ctx, lambda: ctx.graph_launch(gr)) / len(bufs)
    ctx.graph_free(gr)
    nbytes = 2 * cfg.ffn * cfg.hidden // 256 * 144 + 4 * cfg.hidden + 4 * cfg.ffn
    out["q4k_gate_up"] = {"kernel": "stand-alone gate||up+GELU, 2x6144x1536 (the multi-slot path)",
                          "us": ms * 1e3, "bytes": nbytes, "gbs": nbytes / ms / 1e6, "launches_per_token": 0}
    for g, u in bufs:
        lib.ks_buf_free(ctx.h, g)
        lib.ks_buf_free(ctx.h, u)
    # lm_head: one 330 MB matrix (larger than L2 on its own)
    e = lib.ks_buf_wrap(ctx.h, lib.ks_model_tensor_ptr(model_h, b"token_embd.weight"), tb("token_embd.weight"))
    lg = ctx.buffer_empty_f32(cfg.vocab)

    def head4():
        for _ in range(4):
            ctx.check(lib.ks_matvec(ctx.h, cfg.vocab, cfg.hidden, Q6K, e, 0, 0, x.h, 0, lg.h, 0, 1))
    ms = median_ms(ctx, head4) / 4
    nbytes = cfg.vocab * cfg.hidden // 256 * 210 + 4 * cfg.hidden + 4 * cfg.vocab
    out["q6k_lm_head"] = {"kernel": "Q6_K lm_head 262144x1536 (planner-chosen variant)", "us": ms * 1e3, "bytes": nbytes,
                          "gbs": nbytes / ms / 1e6, "frac_of_measured_peak": nbytes / ms / 1e6 / peak, "launches_per_token": 1}
    lib.ks_buf_free(ctx.h, e)
    return out


def matvec_shape(ctx, peak, dtype, rows, cols, tag):
    """One matvec shape over enough distinct weight copies to exceed twice the L2, the launches captured in one
    CUDA graph (device time, not host launch rate); median of 5 replays."""
    from ksearch_b200 import Q4K, synth
    lib = ctx.lib
    one = (synth.q4k_matrix if dtype == Q4K else synth.q6k_matrix)(SEED, tag, rows, cols)
    ncopy = int(max(8, -(-2 * L2_BYTES // one.nbytes) + 1))
    big = ctx.buffer_empty_bytes(one.nbytes * ncopy)
    for c in range(ncopy):
        ctx.write_buffer(big, one, c * one.nbytes)
    x = ctx.buffer_bytes(synth.normals(SEED, tag + "/x", cols))
    y = ctx.buffer_empty_f32(rows)
    lib.ks_plan_search(ctx.h, b"mv_q4k" if dtype == Q4K else b"mv_q6k", rows, 0, cols, 1, None)   # load-time plan search, untimed
    g = graph_of(ctx, [lambda c=c: ctx.check(lib.ks_matvec(ctx.h, rows, cols, dtype, big.h, c * one.nbytes, 0, x.h, 0, y.h, 0, 1))
                       for c in range(ncopy)])
    ms = median_ms(ctx, lambda: ctx.graph_launch(g), warm=2) / ncopy
    ctx.graph_free(g)
    big.free()
    nbytes = one.nbytes + 4 * (rows + cols)
    return {"shape": f"{'Q4_K' if dtype == Q4K else 'Q6_K'} {rows}x{cols}, fp32 x/y", "us": ms * 1e3, "bytes": nbytes,
            "gbs": nbytes / ms / 1e6, "frac_of_measured_peak": nbytes / ms / 1e6 / peak, "frac_of_8000": nbytes / ms / 1e6 / 8000.0,
            "launches_timed": 5 * ncopy, "cold_l2": f"{ncopy} rotating weight copies ({ncopy * one.nbytes / 1e6:.0f} MB)"}


def gemm_shape(ctx, dtype, rows, cols, n_tok, tag):
    """The tensor-core GEMM behind batches of more than 8 rows (prompt chunks, many slots): rows x cols weights
    against n_tok token rows, over rotating weight copies larger than L2, one CUDA graph; median of 5.  Each call is
    the operand split, the GEMM and (when the k range was split) the ordered sum of the partials."""
    from ksearch_b200 import Q4K, synth
    lib = ctx.lib
    one = (synth.q4k_matrix if dtype == Q4K else synth.q6k_matrix)(SEED, tag, rows, cols)
    ncopy = int(max(3, -(-2 * L2_BYTES // one.nbytes) + 1))
    big = ctx.buffer_empty_bytes(one.nbytes * ncopy)
    for c in range(ncopy):
        ctx.write_buffer(big, one, c * one.nbytes)
    x = ctx.buffer_bytes(synth.normals(SEED, tag + "/x", cols * n_tok))
    y = ctx.buffer_empty_f32(rows * n_tok)
    ctx.check(lib.ks_matvec(ctx.h, rows, cols, dtype, big.h, 0, 0, x.h, 0, y.h, 0, n_tok))   # sizes the scratch, untimed
    g = graph_of(ctx, [lambda c=c: ctx.check(lib.ks_matvec(ctx.h, rows, cols, dtype, big.h, c * one.nbytes, 0, x.h, 0, y.h, 0, n_tok))
                       for c in range(ncopy)])
    ms = median_ms(ctx, lambda: ctx.graph_launch(g), warm=2) / ncopy
    ctx.graph_free(g)
    big.free()
    flops = 2.0 * rows * cols * n_tok
    return {"shape": f"{'Q4_K' if dtype == Q4K else 'Q6_K'} {rows}x{cols} x {n_tok} rows, fp32 x/y", "us": ms * 1e3,
            "weight_gbs": one.nbytes / ms / 1e6, "tflops_useful": flops / ms / 1e9,
            "tflops_issued": 3.0 * flops / ms / 1e9,
            "note": "three f16 products per weight and x (hi.hi + hi.lo + lo.hi) keep f32 accuracy; bound by the CUDA-core dequantisation and instruction issue"}


def attention_shapes(ctx, peak):
    """Decode attention over a Q4_0 cache: 8 query heads on 1 (MQA) and 2 (GQA) KV heads of 256, 4 slots, contexts
    1024 / 4096 / 16384 and the mixed batch; caches rotated so every launch reads its rows from HBM."""
    from ksearch_b200 import Eng, synth
    from ksearch_b200.eng import write_meta
    e = Eng()
    n_q, hd, n_slots, rowb = 8, 256, 4, 144
    out = []
    for n_kv in (1, 2):
        for name, lens in (("1024", [1024] * 4), ("4096", [4096] * 4), ("16384", [16384] * 4),
                           ("1024/4096/16384/16384", [1024, 4096, 16384, 16384])):
            max_t = max(lens)
            slot_bytes = max_t * n_kv * rowb
            one = n_slots * slot_bytes
            ncopy = int(max(2, -(-2 * L2_BYTES // (2 * one)) + 1))
            K = synth.q40_rows(SEED, "attK", one // 18 * 32, sigma=0.05)
            V = synth.q40_rows(SEED, "attV", one // 18 * 32, sigma=0.05)
            bK = ctx.buffer_empty_bytes(one * ncopy)
            bV = ctx.buffer_empty_bytes(one * ncopy)
            for c in range(ncopy):
                ctx.write_buffer(bK, K, c * one)
                ctx.write_buffer(bV, V, c * one)
            q = ctx.buffer_bytes(synth.normals(SEED, "attq", n_slots * n_q * hd))
            o = ctx.buffer_empty_f32(n_slots * n_q * hd)
            meta = ctx.buffer_empty_f32(4 * n_slots)
            for s in range(n_slots):
                write_meta(ctx, meta, lens[s], 0, 0, slot=s)
            ns = ctx.lib.ks_sdpa_pick_splits(ctx.h, n_slots, n_kv, max_t)
            tmp = ctx.buffer_empty_f32(max(1, e.sdpa_tmp_floats(n_q, hd, ns, n_slots)))
            g = graph_of(ctx, [lambda c=c: ctx.check(ctx.lib.ks_sdpa_decode(
                ctx.h, n_slots, n_q, n_kv, hd, max_t, 4, 1.0 / 16.0, 0, q.h, bK.h, bV.h, c * one, slot_bytes, meta.h, tmp.h, o.h, ns))
                for c in range(ncopy)])
            ms = median_ms(ctx, lambda: ctx.graph_launch(g), warm=2) / ncopy
            ctx.graph_free(g)
            nbytes = sum(lens) * n_kv * 2 * rowb + 2 * n_slots * n_q * hd * 4
            out.append({"kv_heads": n_kv, "contexts": name, "splits": ns, "us": ms * 1e3, "bytes": nbytes, "gbs": nbytes / ms / 1e6,
                        "frac_of_measured_peak": nbytes / ms / 1e6 / peak})
            for b in (bK, bV, q, o, meta, tmp):
                b.free()
    return out


def serve_e4b(ctx, rank, world, dist, peak, prompt_len=512, n_new=256):
    """The E4B-shaped serve workload: 8 slots spread over the GPUs (8 / N each, one model replica per GPU, no
    collective), every slot a random 512-token prompt (ks_model_prefill) and 256 greedy tokens; the slots of one
    GPU advance together through one pass over the weights (slot scheduler decode_round, scheduler.rs:163-231)."""
    from ksearch_b200 import model as ksm
    from ksearch_b200 import synth
    n_local = max(1, 8 // world)
    cfg = ksm.e4b_config(max_seq=16384, n_slots=n_local)
    model = ksm.GemmaCudaModel.synthetic(ctx, cfg, SEED + 100 + rank)
    model.warm_plans(n_local)
    slots = [model.slot_alloc() for _ in range(n_local)]
    prompts = [synth.token_ids(SEED + rank, f"serve/{s}", prompt_len, cfg.vocab) for s in slots]
    ctx.synchronize()
    t0 = time.perf_counter()
    for s in slots:
        model.prefill(s, prompts[s][:-1])
    ctx.synchronize()
    prefill_s = time.perf_counter() - t0
    model.forward(0, n_local, [int(p[-1]) for p in prompts], True)
    for _ in range(3):
        model.forward(0, n_local, None, True)
    ctx.synchronize()
    ctx.timer_begin()
    for _ in range(n_new - 4):
        model.forward(0, n_local, None, True)
    ms = ctx.timer_end_ms()
    steps = n_new - 4
    if dist is not None:
        import torch
        t = torch.tensor([ms, prefill_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, prefill_s = float(t[0]), float(t[1])
    wb = ksm.weight_bytes_per_token(cfg)
    pos = prompt_len + n_new // 2
    kv_bytes = n_local * pos * cfg.n_layers * cfg.n_kv * 288
    per_step = wb + kv_bytes
    res = {"workload": "E4B-shaped: 42 layers, hidden 2560, GeGLU 10240, 8 q / 2 kv heads x 256, vocab 262144; 8 slots, max-seq 16384, "
                       f"{prompt_len}-token prompts, {n_new} decoded tokens per slot",
           "slots_total": n_local * world, "slots_per_gpu": n_local, "decode_tok_s_total": n_local * world * steps / (ms / 1e3),
           "decode_tok_s_per_slot": steps / (ms / 1e3), "ms_per_round": ms / steps,
           "prefill_tok_s_total": n_local * world * (prompt_len - 1) / prefill_s,
           "bytes_required_per_round_per_gpu": per_step, "gbs_per_gpu": per_step / (ms / steps) / 1e6,
           "frac_of_measured_peak": per_step / (ms / steps) / 1e6 / peak,
           "path": "persistent decode kernel" if n_local == 1 else "two persistent-kernel passes per round" if n_local == 2 else "one launch per op; the slots share one pass through the tensor-core GEMM, "
                                                                   "prompts run in 256-row GEMM chunks"}
    model.close()
    return res


def sharded_matvecs(ctx, rank, world, dist, peak):
    """(N > 1) The tied lm_head (Q6_K 262144x1536) and the stacked gate||up matrix (Q4_K 20480x2560) row-sharded over
    the ranks: local rows, NCCL all-gather of the slices, all on the context's stream; for the lm_head also the
    arg-max form (one pair per rank).  Device time, max over ranks; checked against the 1-GPU result on rank 0."""
    import torch
    from ksearch_b200 import Q4K, Q6K, shard, synth
    from ksearch_b200 import model as ksm
    lib = ctx.lib
    uid = torch.zeros(shard.Comm.ID_BYTES, dtype=torch.uint8, device="cuda")
    if rank == 0:
        uid = torch.frombuffer(bytearray(shard.Comm.unique_id(lib)), dtype=torch.uint8).cuda()
    dist.broadcast(uid, 0)
    comm = shard.Comm(ctx, world, rank, uid.cpu().numpy().tobytes())
    # mailboxes for the arg-max exchange over peer memory: every rank's 64-byte handle to every rank
    mine = torch.frombuffer(bytearray(comm.p2p_handle()), dtype=torch.uint8).cuda()
    allh = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(allh, mine)
    comm.p2p_open(b"".join(h.cpu().numpy().tobytes() for h in allh))
    out = {}
    cfg = ksm.e2b_config()
    for name, dtype, rows, cols in (("q6k_lm_head_262144x1536", Q6K, 262144, 1536), ("q4k_gate_up_20480x2560", Q4K, 20480, 2560)):
        if dtype == Q6K:
            W = ksm.synth_tensor(cfg, SEED, "token_embd.weight", "embd", rows, cols)
        else:
            W = synth.q4k_matrix(SEED, "shard/gu", rows, cols)
        x = synth.normals(SEED, "shard/x", cols)
        off, nb = shard.shard_byte_range(dtype, rows, cols, world, rank)
        sm = shard.ShardedMatvec(ctx, comm, dtype, rows, cols, W[off:off + nb])
        sm.set_x(x)
        reps = 20
        # load-time plan search for the local and the whole shape (untimed), as a model's warm_plans does
        for r_ in (sm.n, rows):
            lib.ks_plan_search(ctx.h, b"mv_q4k" if dtype == Q4K else b"mv_q6k", r_, 0, cols, 1, None)

        def t(fn):
            g = graph_of(ctx, [fn] * reps)
            ms = median_ms(ctx, lambda: ctx.graph_launch(g), warm=2) / reps
            ctx.graph_free(g)
            tt = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            return float(tt[0]) * 1e3
        local_us = t(lambda: sm.enqueue(False))
        gather_us = t(lambda: ctx.check(lib.ks_comm_all_gather_f32(comm.h, sm.y_all.h, 0, sm.per)))
        both_us = t(lambda: sm.enqueue(True))
        res = {"rows": rows, "cols": cols, "local_matvec_us": local_us, "all_gather_us": gather_us, "sharded_us": both_us,
               "all_gather_bytes": 4 * sm.per * world}
        if dtype == Q6K:   # local rows + arg-max + exchange of one (value, index) word per rank: peer memory, then NCCL
            res["sharded_argmax_us"] = t(lambda: (sm.enqueue(False), sm.enqueue_argmax(30.0)))
            comm.set(comm.USE_P2P, 0)
            res["sharded_argmax_nccl_us"] = t(lambda: (sm.enqueue(False), sm.enqueue_argmax(30.0)))
            comm.set(comm.USE_P2P, 1)
            res["argmax_exchange"] = "one kernel: 8-byte stores into the peers' mailboxes over NVLink, bounded poll, merge"
        # parity and the 1-GPU time, on rank 0 (it holds the whole matrix for this)
        y = sm.forward(x)
        tok = sm.argmax(x, 30.0) if dtype == Q6K else None
        ok = torch.ones(1, device="cuda")
        if rank == 0:
            Wb = ctx.buffer_bytes(W)
            y1 = ctx.buffer_empty_f32(rows)
            ctx.check(lib.ks_matvec(ctx.h, rows, cols, dtype, Wb.h, 0, 0, sm.x.h, 0, y1.h, 0, 1))
            ref = ctx.read_f32(y1, rows)
            good = bool(np.all(np.abs(y - ref) <= 1e-4 + 1e-3 * np.abs(ref)))
            if tok is not None:
                good = good and tok == int(np.argmax(np.tanh(ref / 30.0)))
            g = graph_of(ctx, [lambda: ctx.check(lib.ks_matvec(ctx.h, rows, cols, dtype, Wb.h, 0, 0, sm.x.h, 0, y1.h, 0, 1))] * 4)
            res["one_gpu_us"] = median_ms(ctx, lambda: ctx.graph_launch(g), warm=2) / 4 * 1e3
            ctx.graph_free(g)
            Wb.free()
            ok[0] = 1.0 if good else 0.0
        dist.broadcast(ok, 0)
        res["parity_ok"] = bool(ok[0] > 0)
        if rank == 0:
            res["speedup_over_one_gpu"] = res["one_gpu_us"] / both_us
            if "sharded_argmax_us" in res:   # the one-GPU figure is the matvec alone, without its arg-max
                res["argmax_speedup_over_one_gpu_matvec"] = res["one_gpu_us"] / res["sharded_argmax_us"]
            res["bound_by"] = "the all-gather" if gather_us > local_us else "the local rows"
        out[name] = res
    comm.close()
    return out


def main():
    # Libraries (NCCL's version banner, for one) print to stdout; the one JSON line must be alone there, so everything
    # else goes to stderr and the line is written to the saved descriptor at the end.
    sys.stdout.flush()
    out_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(obj):
        os.write(out_fd, (json.dumps(obj) + "\n").encode())

    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-serve", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the other configurations' kernels (N = 1)")
    args = ap.parse_args()
    rank, world, local = dist_env()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args, rank, world, emit)
        return

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from ksearch_b200 import Q4K, CudaContext
    from ksearch_b200 import model as ksm
    from ksearch_b200 import synth
    peak, peak_kind = measured_peak()
    ctx = CudaContext(local, flags=1)  # bit 0: programmatic dependent launch
    cfg = ksm.e2b_config(max_seq=PROMPT_LEN + args.steps * 2 + args.warmup * 2 + 16 + 64 + 256)
    want_cpu = world == 1 and not args.no_cpu_baseline
    if want_cpu:
        model, T = ksm.GemmaCudaModel.synthetic(ctx, cfg, SEED + rank, keep=True)
    else:
        model, T = ksm.GemmaCudaModel.synthetic(ctx, cfg, SEED + rank), None
    model.warm_plans(1)   # load-time plan search / per-chip cache, outside every timed region
    slot = model.slot_alloc()
    prompt = synth.token_ids(SEED + rank, "prompt", PROMPT_LEN, cfg.vocab)

    def barrier():
        ctx.synchronize()
        if dist is not None:
            import torch
            dist.barrier()
            torch.cuda.synchronize()

    # ---- untimed: the first greedy tokens of this prompt, for the parity check against the CPU decoder
    gpu_first = model.generate_timed(prompt, PARITY_TOKENS)[0] if want_cpu else []

    # ---- device-resident decode: prompt, W warm-up steps, then exactly K timed steps
    model.slot_reset(slot)
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

    # ---- end to end: host token ids in and out of every step through the blocking C-ABI call, over the SAME
    # positions as the device-resident leg (the slot is rewound and the prompt replayed, untimed; decode time grows
    # with the context, so timing this leg further down the sequence would measure a different workload)
    model.slot_reset(slot)
    for t in prompt[:-1]:
        model.forward(slot, 1, [int(t)], False)
    tok = int(prompt[-1])
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

    line = None
    if rank == 0:
        value = world * args.steps / (ms / 1e3)
        e2e = world * args.steps / (e2e_ms / 1e3)
        wb = ksm.weight_bytes_per_token(cfg)
        line = {
            "metric": "decode_tok_s_e2b_q4k", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(world),
            "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 8,
                    "api": "ks_model_decode_token (blocking, host token id in; next id and a status flag out)"},
            "gpu_launches": launches, "clocks": clocks,
            "weight_stream": {"bytes_per_token": wb, "gbs_per_gpu": wb / (ms / args.steps) / 1e6,
                              "frac_of_peak": wb / (ms / args.steps) / 1e6 / peak, "peak_gbs": peak, "peak_kind": peak_kind},
        }
    if world == 1:
        alone = time_kernels_alone(ctx, model, slot, cfg, peak, args.steps)
        share = {k: v["us"] * v["launches_per_token"] for k, v in alone.items()}
        dom = max(share, key=share.get)
        d = alone[dom]
        traffic = None
        if dom == "decode_layers" and DECODE_KERNEL_DRAM_TRAFFIC_PER_LAYER:
            traffic = DECODE_KERNEL_DRAM_TRAFFIC_PER_LAYER * cfg.n_layers
        line["roofline"] = {"bound": "hbm", "kernel": d["kernel"], "achieved": d["gbs"], "peak": peak, "unit": "GB/s",
                            "frac": d["gbs"] / peak, "of": peak_kind, "traffic": traffic, "us_per_launch": d["us"],
                            "bytes_per_launch": d["bytes"]}
        line["kernels_alone"] = alone
        line["gemv_config0"] = matvec_shape(ctx, peak, Q4K, 4096, 4096, "cfg0")
        if not args.no_extras:
            line["matvec_shapes"] = [matvec_shape(ctx, peak, Q4K, r, c, f"cfg1/{r}x{c}")
                                     for r, c in ((1536, 6144), (6144, 1536), (2560, 10240), (10240, 2560))]
            line["attention"] = attention_shapes(ctx, peak)
            # the reference's own mul_mm check shapes (check_mul_mm.rs:300-304) and one E4B FFN shape at a full chunk
            line["gemm_shapes"] = [gemm_shape(ctx, Q4K, r, c, t, f"gemm/{r}x{c}x{t}")
                                   for r, c, t in ((2048, 1536, 256), (4096, 1536, 256), (4096, 1536, 55), (20480, 2560, 128))]
    model.close()
    if want_cpu:
        line["cpu_baseline"], line["parity"] = cpu_baseline_and_parity(cfg, T, prompt, gpu_first)
    T = None
    if world > 1:
        sh = sharded_matvecs(ctx, rank, world, dist, peak)
        if rank == 0:
            line["sharded"] = sh
    if not args.no_serve:
        sv = serve_e4b(ctx, rank, world, dist, peak)
        if rank == 0:
            line["serve_e4b"] = sv
    if rank == 0:
        emit(line)
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
