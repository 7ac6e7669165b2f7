#!/usr/bin/env python
"""Decode benchmark for the RWKV-7 quantised-weight hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload decode_bsz1_int8|decode_bsz320_nvfp4|decode_bsz1_nvfp4|pipeline_bsz320_nvfp4|gemv_*|gemm_*]
                    [--model 7.2b|0.1b|tiny]

One "step" is one decode step of the whole model (every matrix product of the 32 blocks, the WKV-7
state update between them and the vocabulary head) for the workload's batch. Weights are random
(seeded, reference checkpoint schema), since trained checkpoints are not available offline.

Prints ONE JSON line. The default workload is the batch-1 int8 decode of the 7.2B shapes; its line also carries,
under `also`, the second configuration of the metric (NVFP4, 320 sequences per GPU: a full record with its own `e2e`,
`roofline` and `clocks`) and the single int8 matrix-vector product of baseline config 1 with its HBM GB/s, measured in
the same process at every N. `value` is device-timed (CUDA events, inputs resident in HBM, CUDA-graph
replay of the library's launches); `e2e` is a decode loop through the public calls: `RWKV_x070.forward[_batch]`
on host token ids (pinned host -> device), greedy sampling on the device, next ids read back to the host, every step.
`--impl reference` times the CPU restatement of the reference's PyTorch path (oracle/) on the host
cores on a bounded sample of the same workload.
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
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "decode_bsz1_int8": dict(batch=1, quant="int8"),
    "decode_bsz320_nvfp4": dict(batch=320, quant="nvfp4"),
    "decode_bsz1_nvfp4": dict(batch=1, quant="nvfp4"),
    "pipeline_bsz320_nvfp4": dict(batch=320, quant="nvfp4"),   # layer pipeline: one stage per rank (torchrun, N >= 2)
    "gemv_int8": dict(batch=1, quant="int8"),
    "gemv_nvfp4": dict(batch=1, quant="nvfp4"),
    "gemm_int8": dict(batch=320, quant="int8"),
    "gemm_nvfp4": dict(batch=320, quant="nvfp4"),
}
METRIC = "rwkv7_decode_tokens_per_s"


def measured_peaks(burst: bool = False):
    """(HBM GB/s, dense bf16 TFLOP/s, source). The tensor figure is the burst one for a kernel timed alone and the
    sustained one for a kernel timed inside a long step."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        tf = d.get("bf16_tflops") if burst else d.get("bf16_tflops_sustained", d.get("bf16_tflops"))
        return float(d["hbm_gbs"]), float(tf or 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "25", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=lambda: [self.lines.append(l) for l in self.proc.stdout], daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.t.join(timeout=2)
        sm, mx, reasons = [], [], set()
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def profiled_traffic() -> dict:
    """DRAM bytes (read + write) per launch of the profiled kernels, read from the table in
    profiles/dram_traffic.md (one row per ncu capture: kernel | workload key | DRAM bytes | algorithmic bytes).
    A kernel whose capture is missing gets `traffic: null`."""
    out = {}
    path = os.path.join(ROOT, "profiles", "dram_traffic.md")
    if not os.path.exists(path):
        return out
    for line in open(path):
        f = [x.strip() for x in line.strip().strip("|").split("|")]
        if len(f) >= 4 and f[0] and not set(f[0]) <= set("-: ") and f[0] != "kernel":
            try:
                out[(f[0], f[1])] = (float(f[2]), float(f[3]))
            except ValueError:
                continue
    return out


def decode_traffic(algorithmic_total: int, quant: str, n_embd: int):
    """decode_kernel was captured on a model with the same block shapes and 4 blocks; the kernel walks the same
    phase list per block, so the captured traffic / algorithmic ratio carries over to 32 blocks."""
    t = profiled_traffic().get(("decode_kernel", f"{quant}_d{n_embd}"))
    return algorithmic_total * t[0] / t[1] if t else None


def gemm_traffic(quant: str, n_out: int, k: int, rows: int):
    t = profiled_traffic().get(("gemm_tc_kernel", f"{quant}_{n_out}x{k}x{rows}"))
    return t[0] if t else None


def workload_config(a, workload: str, batch: int) -> dict:
    """The `config` object of a JSON line: a function of the command line only, so both arms print the same one."""
    from albatross_b200 import synth
    L, D, V, _ = synth.CONFIGS[a.model]
    return {"workload": workload, "shapes": a.model, "batch_per_gpu": batch, "n_layer": L, "n_embd": D, "vocab": V,
            "sharding": "independent sequences per GPU, no collective in the step",
            "l2": "inputs larger than L2: every step streams all weights of the model (GBs) from HBM"}


def time_gemm_alone(model, B: int, dev: int, steps: int) -> dict:
    """CUDA-event time of ab_gemm on the channel-mix key matrices of the model, one block after the other
    (32 different matrices: 1.2 GB of NVFP4, so every launch streams its weights from HBM)."""
    import ctypes as C
    from albatross_b200 import _lib
    mats = model.packed_matrices("ffn.key.weight")
    n_out, k = mats[0].n_out, mats[0].k
    cm = [m.as_mat() for m in mats]
    x = torch.randn(B, k, device=f"cuda:{dev}").half()
    y = torch.empty(B, n_out, dtype=torch.float16, device=f"cuda:{dev}")
    scratch = torch.zeros(_lib.lib.ab_gemm_scratch_bytes(C.byref(cm[0]), B) + 256, dtype=torch.uint8, device=f"cuda:{dev}")
    st = torch.cuda.current_stream().cuda_stream
    n = max(steps, 32)
    call = lambda i: _lib.check(_lib.lib.ab_gemm(C.byref(cm[i % len(cm)]), B, x.data_ptr(), y.data_ptr(), 3, None,
                                                 scratch.data_ptr(), st))
    for i in range(len(cm)):
        call(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
        call(i)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / n
    flops = 2.0 * B * n_out * k
    return {"us": us, "flops": flops, "tflops": flops / (us * 1e-6) / 1e12, "launches": n}


def algorithmic_bytes(model, batch: int) -> dict:
    """Bytes one decode step must move: every weight once, the kv state read + written, the WKV vectors."""
    L, D = model.n_layer, model.n_embd
    H = D // 64
    weights = model.weight_bytes()
    kv = batch * L * H * (2 * 64 * 64 * 4 + 7 * 64 * 2)
    return {"weights": weights, "kv_state": kv, "total": weights + kv}


# ----------------------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------------------
def run_ours(a, rank, world, dev, workload=None, batch=None):
    from albatross_b200 import RWKV_x070, synth
    workload = workload or a.workload
    wl = WORKLOADS[workload]
    B = batch or wl["batch"]
    args = synth.make_args(a.model)
    torch.cuda.set_device(dev)
    model = RWKV_x070(args, quant=wl["quant"], state_dict=synth.iter_checkpoint(a.model, seed=0, device=f"cuda:{dev}"),
                      device=f"cuda:{dev}", use_graph=not a.no_graph, decode_mode=a.decode_mode)
    if a.stages:
        model.set_option("stages", a.stages)
    if a.no_pdl:
        model.set_option("pdl", 0)
    V = args.vocab_size
    g = torch.Generator().manual_seed(1000 + rank)
    n_tok = a.warmup + a.steps + 8
    toks = torch.randint(0, V, (n_tok, B), generator=g)
    if B > 1:      # gather + per block (2 LN+lerp, 2 grouped + 3 single matrix products, WKV) + final LN + head
        launches_per_step = 1 + 8 * args.n_layer + 2
    else:
        launches_per_step = 1 if model.decode_mode == "persistent" else 5 * args.n_layer + 1

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=f"cuda:{dev}")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return float(t.item())

    # ---- e2e: the public calls of a decode loop, every step: host token ids in (pinned -> device), forward, greedy
    # sampling on the device (the library's replacement for the reference's argsort sampler), ids back on the host
    from albatross_b200 import sampler_simple_batch
    pinned_ids = torch.empty((B, 1), dtype=torch.int64).pin_memory()
    state = model.new_state(B if B > 1 else None)

    tok_lists = toks.tolist()       # host token ids as the Python lists the reference's API takes

    def e2e_step(i):
        nonlocal state
        if B == 1:
            logits, state = model.forward(tok_lists[i][0], state)
            logits = logits.unsqueeze(0)
        else:
            logits, state = model.forward_batch([[t] for t in tok_lists[i]], state)
        sampler_simple_batch(logits, noise=0.0, out=pinned_ids)     # the kernel stores the ids to pinned host memory
        torch.cuda.current_stream().synchronize()

    for i in range(a.warmup):
        e2e_step(i)
    sync_all()
    sampler = ClockSampler(dev)     # runs across both timed regions (the GPU is under load from here to the end)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.warmup, a.warmup + a.steps):
        e2e_step(i)
    e1.record()
    sync_all()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1))
    e2e_val = world * B * a.steps / (e2e_ms * 1e-3)

    # ---- device-timed: token ids resident, one CUDA graph replay per step, events on the launch stream
    state = model.new_state(B if B > 1 else None)
    tok_dev = toks.to(torch.int32).to(f"cuda:{dev}")
    if B == 1 and not model.use_graph:
        cur = torch.zeros(1, dtype=torch.int32, device=f"cuda:{dev}")
        logits_buf = torch.empty(V, dtype=torch.float16, device=f"cuda:{dev}")
        step_fn = lambda i: (cur.copy_(tok_dev[i]), model._run(1, 1, cur, state, logits_buf, False))
    elif B == 1 and model.decode_mode == "persistent":
        _, prog_ptr, tok_buf, logits_buf = model._program_for(state)
        from albatross_b200 import _lib as _l
        st_ = torch.cuda.current_stream().cuda_stream
        step_fn = lambda i: (tok_buf.copy_(tok_dev[i]), _l.check(_l.lib.ab_decode_run(model._handle, prog_ptr, st_)))
    elif B == 1:
        model.forward(0, state)                     # captures the graph for this state
        graph, tok_buf, logits_buf = model._graphs[tuple(t.data_ptr() for t in state)]
        step_fn = lambda i: (tok_buf.copy_(tok_dev[i]), graph.replay())
    elif model.use_graph:
        model.forward_batch([[0]] * B, state)       # records the graph of one batched step for this state
        graph, tok_buf, logits_buf = model._graphs[(B,) + tuple(t.data_ptr() for t in state)][:3]
        step_fn = lambda i: (tok_buf.copy_(tok_dev[i]), graph.replay())
    else:
        cur = torch.zeros(B, dtype=torch.int32, device=f"cuda:{dev}")
        logits_buf = torch.empty(B, V, dtype=torch.float16, device=f"cuda:{dev}")
        step_fn = lambda i: (cur.copy_(tok_dev[i]), model._run(B, 1, cur, state, logits_buf, False))
    for i in range(a.warmup):
        step_fn(i)
    sync_all()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(a.steps + 1)]
    ev[0].record()
    for i in range(a.steps):
        step_fn(a.warmup + i)
        ev[i + 1].record()
    sync_all()
    clocks = sampler.stop()
    per_step = np.array([ev[i].elapsed_time(ev[i + 1]) for i in range(a.steps)])
    total_ms = max_over_ranks(ev[0].elapsed_time(ev[-1]))
    value = world * B * a.steps / (total_ms * 1e-3)

    from albatross_b200 import _lib
    hbm, tf, which = measured_peaks()
    ab = algorithmic_bytes(model, B)
    ms_step = total_ms / a.steps
    if B == 1:
        # One persistent kernel per token (or a graph of matrix-vector launches): the step IS the dominant kernel.
        achieved = ab["total"] / (ms_step * 1e-3) / 1e9
        kernel = "decode_kernel (one launch per token)" if model.decode_mode == "persistent" else "gemv_stream_kernel"
        roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                    "traffic": decode_traffic(ab["total"], wl["quant"], args.n_embd) if model.decode_mode == "persistent" else None,
                    "peak_source": which, "kernel": kernel, "algorithmic_bytes_per_launch": ab}
    else:
        # The tensor-core products take the largest share of the step; the largest of them (channel-mix key,
        # n_out = 4 * n_embd) is timed alone, live, on the model's own packed weights of every block in turn.
        gm = time_gemm_alone(model, B, dev, a.steps)
        flops_step = 2.0 * B * model.matrix_params()
        _, tf_burst, _ = measured_peaks(burst=True)
        roofline = {"bound": "tensor", "achieved": gm["tflops"], "peak": tf_burst, "unit": "TFLOP/s", "frac": gm["tflops"] / tf_burst,
                    "frac_of_sustained_peak": gm["tflops"] / tf,
                    "traffic": gemm_traffic(wl["quant"], 4 * args.n_embd, args.n_embd, B),
                    "peak_source": which + " (dense bf16 cuBLAS; burst figure, the kernel is timed alone)",
                    "kernel": "gemm_tc_kernel on ffn.key [%d x %d] x batch %d" % (4 * args.n_embd, args.n_embd, B),
                    "algorithmic_flops_per_launch": gm["flops"], "us_per_launch": gm["us"],
                    "whole_step": {"matrix_tflops": flops_step / (ms_step * 1e-3) / 1e12,
                                   "hbm_gbs": ab["total"] / (ms_step * 1e-3) / 1e9, "algorithmic_bytes": ab,
                                   "algorithmic_flops": flops_step}}
    status = _lib.device_status()
    out = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": ms_step, "ms_per_step_p10": float(np.percentile(per_step, 10)),
        "ms_per_step_p50": float(np.percentile(per_step, 50)),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 weights (dp4a, exact int32 sums), fp16 activations, fp32 WKV state" if wl["quant"] == "int8"
        else "nvfp4 weights de-quantised to fp16 in registers, fp16 activations, fp32 accumulate and WKV state",
        "data": "synthetic (seeded random weights in the reference checkpoint schema, random token ids)",
        "config": workload_config(a, workload, B),
        "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 8 * B,
                "ms_per_step": e2e_ms / a.steps,
                "what": "RWKV_x070.forward[_batch] on host token ids + sampler_simple_batch on the device + ids to the host"},
        "gpu_launches": launches_per_step * a.steps,
        "roofline": roofline,
        "clocks": clocks, "device_status": status,
    }
    return out


# ----------------------------------------------------------------------------------------------
# layer pipeline: rank s holds blocks [s*L/S, (s+1)*L/S); x and v_first ([b, D] fp16) cross each boundary
# ----------------------------------------------------------------------------------------------
def run_pipeline(a, rank, world, dev):
    from albatross_b200 import RWKV_x070, synth, dist as adist
    import torch.distributed as td
    wl = WORKLOADS[a.workload]
    B, M = a.batch or wl["batch"], a.micro
    assert world >= 2 and B % M == 0, "the pipeline workload needs torchrun with >= 2 ranks and batch % micro == 0"
    b = B // M
    args = synth.make_args(a.model)
    D, V = args.n_embd, args.vocab_size
    lo, hi = adist.stage_layers(args.n_layer, world, rank)
    device = f"cuda:{dev}"
    model = RWKV_x070(args, quant=wl["quant"], state_dict=synth.iter_checkpoint(a.model, seed=0, device=device),
                      device=device, layer_range=(lo, hi))
    states = [model.new_state(b) for _ in range(M)]
    xout = [torch.empty(b, D, dtype=torch.float16, device=device) for _ in range(M)]
    vbuf = [torch.empty(b, D, dtype=torch.float16, device=device) for _ in range(M)]
    rbuf = [[torch.empty(b, D, dtype=torch.float16, device=device) for _ in range(2)] for _ in range(M)]
    turn = [0] * M

    def make_buffer(mb):   # called twice per micro-batch and step: x_in, then v_first
        t = rbuf[mb][turn[mb] & 1]
        turn[mb] += 1
        return t

    def stage_fn(mb, inp, v_first):
        if model.is_first:
            model.forward_stage(states[mb], vbuf[mb], tokens=inp.to(torch.int32), x_out=xout[mb])
            return xout[mb], vbuf[mb]
        if model.is_last:
            return model.forward_stage(states[mb], v_first, x_in=inp).argmax(-1)
        model.forward_stage(states[mb], v_first, x_in=inp, x_out=xout[mb])
        return xout[mb], v_first

    dec = adist.PipelineDecoder(stage_fn, M, make_buffer, lambda mb: torch.empty(b, dtype=torch.int64, device=device))
    g = torch.Generator().manual_seed(7)
    tokens = [torch.randint(0, V, (b,), generator=g).to(device) for _ in range(M)] if model.is_first else None

    def sync_all():
        torch.cuda.synchronize(); td.barrier(); torch.cuda.synchronize()

    tokens = dec.run(tokens, a.warmup)
    sync_all()
    sampler = ClockSampler(dev)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    # all steps in one call: a micro-batch starts its next step as soon as its token ids are back on the first stage,
    # so with at least as many micro-batches as stages the stages do not idle between steps
    tokens = dec.run(tokens, a.steps)
    e1.record()
    sync_all()
    clocks = sampler.stop()
    t = torch.tensor([e0.elapsed_time(e1)], device=device)
    td.all_reduce(t, op=td.ReduceOp.MAX)
    total_ms = float(t.item())
    from albatross_b200 import _lib
    return {"metric": METRIC, "value": B * a.steps / (total_ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": total_ms / a.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "nvfp4 weights de-quantised to fp16 in registers, fp16 activations, fp32 accumulate and WKV state",
            "data": "synthetic (seeded random weights in the reference checkpoint schema, random token ids)",
            "config": {"workload": a.workload, "shapes": a.model, "global_batch": B, "micro_batches": M, "stages": world,
                       "blocks_per_stage": hi - lo, "exchange": "x and v_first, [%d, %d] fp16 each, NCCL send/recv per micro-batch and stage boundary; "
                       "token ids int64 [%d] back to stage 0" % (b, D, b)},
            "e2e": None, "gpu_launches": (8 * (hi - lo) + 2) * M * a.steps, "roofline": None, "clocks": clocks,
            "device_status": _lib.device_status()}


# ----------------------------------------------------------------------------------------------
# single-kernel workload: one quantised matrix-vector product (baseline config 1 and its larger shapes)
# ----------------------------------------------------------------------------------------------
def run_gemv(a, dev, workload=None, n=None, k=None):
    """Times ab_gemv alone. Each launch streams a different matrix (enough of them to exceed the L2),
    so every launch reads its weights from HBM."""
    import ctypes as C
    from albatross_b200 import _lib, quant
    torch.cuda.set_device(dev)
    workload = workload or a.workload
    fmt = "nvfp4" if "nvfp4" in workload else "int8"
    n, k = n or a.n_out, k or a.k
    per = n * k * (1.0 if fmt == "int8" else 0.5625)
    n_mats = max(4, int(400e6 // per) + 1)
    torch.manual_seed(0)
    mats = [quant.quantize((torch.randn(n, k, device=f"cuda:{dev}") * 0.02).half(), fmt) for _ in range(n_mats)]
    cm = [m.as_mat() for m in mats]
    x = torch.randn(k, device=f"cuda:{dev}").half()
    y = torch.empty(n, dtype=torch.float16, device=f"cuda:{dev}")
    st = torch.cuda.current_stream().cuda_stream
    call = lambda i: _lib.check(_lib.lib.ab_gemv(C.byref(cm[i % n_mats]), x.data_ptr(), y.data_ptr(), st))
    for i in range(max(a.warmup, n_mats)):
        call(i)
    torch.cuda.synchronize()
    sampler = ClockSampler(dev)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        call(i)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / a.steps
    alg = mats[0].nbytes() + 2 * (n + k)
    hbm, _, which = measured_peaks()
    gbs = alg / (ms * 1e-3) / 1e9
    return {"metric": "gemv_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": fmt + " weights, fp16 activations", "data": "synthetic",
            "config": {"workload": workload, "n_out": n, "k": k, "matrices_cycled": n_mats,
                       "l2": "each launch reads a different matrix; the set is larger than L2"},
            "gpu_launches": a.steps,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm, "traffic": None,
                         "peak_source": which, "kernel": "gemv_stream_kernel", "algorithmic_bytes_per_launch": alg},
            "clocks": clocks, "device_status": _lib.device_status()}


def run_gemm(a, dev):
    """Times ab_gemm alone (tensor-core path). Each launch uses a different weight matrix."""
    import ctypes as C
    from albatross_b200 import _lib, quant
    torch.cuda.set_device(dev)
    fmt = "nvfp4" if "nvfp4" in a.workload else "int8"
    n, k, rows = a.n_out, a.k, (a.batch or 320)
    per = n * k * (1.0 if fmt == "int8" else 0.5625)
    n_mats = max(2, int(300e6 // per) + 1)
    torch.manual_seed(0)
    mats = [quant.quantize((torch.randn(n, k, device=f"cuda:{dev}") * 0.02).half(), fmt) for _ in range(n_mats)]
    cm = [m.as_mat() for m in mats]
    x = torch.randn(rows, k, device=f"cuda:{dev}").half()
    y = torch.empty(rows, n, dtype=torch.float16, device=f"cuda:{dev}")
    scratch = torch.zeros(_lib.lib.ab_gemm_scratch_bytes(C.byref(cm[0]), rows) + 256, dtype=torch.uint8, device=f"cuda:{dev}")
    st = torch.cuda.current_stream().cuda_stream
    call = lambda i: _lib.check(_lib.lib.ab_gemm(C.byref(cm[i % n_mats]), rows, x.data_ptr(), y.data_ptr(), 0, None,
                                                 scratch.data_ptr(), st))
    for i in range(max(a.warmup, n_mats)):
        call(i)
    torch.cuda.synchronize()
    sampler = ClockSampler(dev)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        call(i)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / a.steps
    flops = 2.0 * rows * n * k
    _, tf, which = measured_peaks(burst=True)
    tfs = flops / (ms * 1e-3) / 1e12
    return {"metric": "gemm_tflops", "value": tfs, "unit": "TFLOP/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": fmt + " weights de-quantised to fp16 in registers, fp16 activations, fp32 accumulate (tcgen05 kind::f16)",
            "data": "synthetic", "config": {"workload": a.workload, "n_out": n, "k": k, "batch": rows, "matrices_cycled": n_mats},
            "gpu_launches": a.steps,
            "roofline": {"bound": "tensor", "achieved": tfs, "peak": tf, "unit": "TFLOP/s", "frac": tfs / tf, "traffic": None,
                         "peak_source": which + " (dense bf16 cuBLAS; burst figure, the kernel is timed alone)", "kernel": "gemm_tc_kernel",
                         "algorithmic_flops_per_launch": flops},
            "clocks": clocks, "device_status": _lib.device_status()}


# ----------------------------------------------------------------------------------------------
# CPU arm: the oracle's restatement of the reference's PyTorch path on the host cores
# ----------------------------------------------------------------------------------------------
def run_cpu(a, n_layers_sample: int = 4, steps: int = 0):
    """Times the single-token path (the only one that is pure torch in the reference) in fp32.

    A 7.2B fp32 checkpoint is 28 GB, so the sample is `n_layers_sample` blocks plus the vocabulary head
    at the workload's shapes; per-block time is extrapolated to the full depth."""
    from albatross_b200 import synth
    from oracle.rwkv7_oracle import Oracle, new_state, prepare
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    steps = steps or max(6, min(a.steps, 32))
    L, D, V, ranks = synth.CONFIGS[a.model]
    Ls = min(L, n_layers_sample)
    raw = synth.make_checkpoint((Ls, D, V, ranks), seed=0)
    z = prepare(raw, D, torch.float32)
    o = Oracle(z, Ls, D)
    st = new_state(Ls, D)
    toks = torch.randint(0, V, (steps + 2,), generator=torch.Generator().manual_seed(0)).tolist()
    # head-only time: a zero-block model
    o0 = Oracle(z, 0, D)
    ts_full, ts_head = [], []
    for i, t in enumerate(toks):
        t0 = time.perf_counter(); o.step(t, st); t1 = time.perf_counter()
        o0.step(t, []); t2 = time.perf_counter()
        if i >= 2:
            ts_full.append(t1 - t0); ts_head.append(t2 - t1)
    t_head = float(np.percentile(ts_head, 10))
    t_block = (float(np.percentile(ts_full, 10)) - t_head) / Ls
    t_token = t_block * L + t_head
    B = a.batch or WORKLOADS[a.workload]["batch"]
    return {"value": 1.0 / t_token, "unit": "tokens/s", "cores": cores, "kind": "port", "ms_per_token": 1e3 * t_token,
            "sample": f"{Ls} of {L} blocks + head at {a.model} shapes, fp32 torch single-token path, {steps} steps, p10, "
                      f"extrapolated to {L} blocks; bsz {B} on the CPU = this rate (sequences run one after another)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode_bsz1_int8", choices=sorted(WORKLOADS))
    ap.add_argument("--model", default="7.2b")
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--stages", type=int, default=0)
    ap.add_argument("--micro", type=int, default=4, help="pipeline workload: micro-batches in flight")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from the host (profiling)")
    ap.add_argument("--decode-mode", default=None, choices=["persistent", "graph", "eager"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="default workload only: skip the bsz-320 NVFP4 and single-product records")
    ap.add_argument("--n-out", type=int, default=4096, help="gemv_* workloads: output rows")
    ap.add_argument("--k", type=int, default=4096, help="gemv_* workloads: input length")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    default_line = a.workload == "decode_bsz1_int8" and not a.batch and not a.no_also
    if a.impl == "reference":
        if rank != 0:
            return
        cb = run_cpu(a)
        B = a.batch or WORKLOADS[a.workload]["batch"]
        line = {
            "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "tokens/s", "n_gpus": a.gpus,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": 1e3 / cb["value"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp32 (CPU)", "data": "synthetic",
            "config": workload_config(a, a.workload, B),
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        if default_line:
            # the host cores run sequences one after another: 320 resident sequences decode at the single-sequence rate
            line["also"] = {"decode_bsz320_nvfp4": {"value": cb["value"], "unit": "tokens/s",
                                                    "config": workload_config(a, "decode_bsz320_nvfp4", 320),
                                                    "note": "same CPU port; a batch on the host cores is a loop over sequences"}}
        print(json.dumps(line))
        return

    if a.workload.startswith("gemm_"):
        if rank == 0:
            print(json.dumps(run_gemm(a, local)))
        return
    if a.workload.startswith("gemv_"):
        if rank == 0:
            print(json.dumps(run_gemv(a, local)))
        return
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        torch.distributed.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    out = run_pipeline(a, rank, world, local) if a.workload.startswith("pipeline_") else run_ours(a, rank, world, local)
    if default_line:
        # The metric names two decode configurations and the matrix-vector bandwidth: the second configuration
        # (7.2B NVFP4, 320 sequences per GPU) and the single int8 product are measured in the same process, at every N.
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        second = run_ours(a, rank, world, local, workload="decode_bsz320_nvfp4")
        out["also"] = {"decode_bsz320_nvfp4": second}
        gc.collect()
        torch.cuda.empty_cache()
        if rank == 0:
            gv = run_gemv(a, local, workload="gemv_int8", n=4096, k=4096)
            out["also"]["gemv_int8_4096x4096"] = {k_: gv[k_] for k_ in ("metric", "value", "unit", "ms_per_step", "config", "roofline")}
            # ... and the same kernel on the largest matrix of the model (the vocabulary head), where a launch is long
            # enough to show the streaming rate itself
            gh = run_gemv(a, local, workload="gemv_int8", n=65536, k=4096)
            out["also"]["gemv_int8_65536x4096"] = {k_: gh[k_] for k_ in ("metric", "value", "unit", "ms_per_step", "config", "roofline")}
            out["gpu_launches"] += second["gpu_launches"] + gv["gpu_launches"] + gh["gpu_launches"]
    if rank == 0:
        if world == 1 and not a.no_cpu_baseline and not a.workload.startswith("pipeline_"):
            out["cpu_baseline"] = run_cpu(a)
        print(json.dumps(out))
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
