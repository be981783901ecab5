#!/usr/bin/env python3
"""Benchmark of the decode hot path: packed-KV bytes scanned per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (``config.workload``): one decode step = one pass of the hot path over every layer
of a stack with independent, seeded synthetic KV per layer.  Default = the configuration the headline
metric is quoted on: Llama-3.1-8B layer geometry (32 query heads, 8 KV heads,
head_dim 128), mode K4V4 (group 128), batch 4, context 32768, top-k 256, 32 layers.
Other workloads: ``--workload c1|c3|c4`` or explicit ``--mode/--batch/--ctx/--layers/...``.

What is timed
  value  device-resident: per layer the fused scan + top-k + finish kernels and the
         correction merge (o_new resident), all layers of a step replayed as one CUDA
         graph; CUDA events on the launching stream, max over ranks.
  e2e    the same step through the public ops with HOST buffers: q copied host->device,
         selected slots device->host, the host correction (C++ worker pool over the
         full-precision mirror in host DRAM), o_new host->device, merge, output
         device->host; layers are pipelined (the GPU runs ahead while the host corrects).
  roofline  the scan kernel alone: algorithmic bytes per launch / mean launch time.
  cpu_baseline  the CPU restatement of the scan (oracle/jf_oracle_c.c, OpenMP) plus the
         host correction, timed on one layer of the same workload.

Multi-GPU: one process per GPU (torchrun); every rank owns the KV heads of its shard
(per-GPU work fixed: weak scaling) and the per-head outputs of all layers are gathered
into the TP layout with one NCCL all-gather per step.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (mode, H_q, H_kv, batch, ctx, top_k, layers, description)
    "c1": ("k3v2", 32, 8, 1, 32768, 256, 1, "Llama-3.1-8B layer, K3V2, B1, ctx 32768, top-k 256, 1 layer"),
    "c2": ("k4v4", 32, 8, 4, 32768, 256, 32, "Llama-3.1-8B layer, K4V4, B4, ctx 32768, top-k 256, 32 layers"),
    "c3": ("k3v2", 64, 8, 4, 65536, 512, 80, "Llama-3.3-70B layer, K3V2, B4, ctx 65536, top-k 512, 80 layers"),
    "c4": ("k3v2", 32, 4, 8, 32768, 256, 48, "Qwen3-30B-A3B layer, K3V2, B8, ctx 32768, top-k 256, 48 layers"),
}
BYTES_PER_TOKEN_HEAD = {"k3v2": 88, "k4v4": 132}
MODE_BITS = {"k3v2": (3, 2, 64), "k4v4": (4, 4, 128)}
DRAM_BYTES_PER_TOKEN_HEAD = {"k3v2": 91.2, "k4v4": 137.3}   # dram__bytes_read.sum + dram__bytes_write.sum, one ncu capture


def parse_args():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--mode", choices=["k3v2", "k4v4"])
    ap.add_argument("--batch", type=int)
    ap.add_argument("--ctx", type=int)
    ap.add_argument("--layers", type=int)
    ap.add_argument("--top-k", type=int)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-in-the-loop measurement")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-threads", type=int, default=0, help="host correction threads (0 = cores / ranks)")
    return ap.parse_args()


def resolve_workload(args):
    mode, h_q, h_kv, batch, ctx, top_k, layers, desc = WORKLOADS[args.workload]
    custom = any(v is not None for v in (args.mode, args.batch, args.ctx, args.layers, args.top_k))
    mode = args.mode or mode
    batch = args.batch or batch
    ctx = args.ctx or ctx
    layers = args.layers or layers
    top_k = args.top_k or top_k
    if custom:
        desc = f"custom: {mode}, H_q {h_q}, H_kv {h_kv}, B{batch}, ctx {ctx}, top-k {top_k}, {layers} layers"
    return dict(mode=mode, H_q=h_q, H_kv=h_kv, batch=batch, ctx=ctx, top_k=top_k, layers=layers, desc=desc)


# ---------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while a region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                try:
                    r = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# ---------------------------------------------------------------------------------------
# synthetic workload
# ---------------------------------------------------------------------------------------

def make_layer_kv(torch, w, layer, rank, device, dtype):
    """Seeded N(0,1) K/V (K scaled per channel by log-normal(0, 0.75)) for one layer,
    in token-major layout (T, H_kv, 128), T = batch * ctx."""
    g = torch.Generator(device=device)
    g.manual_seed(1_000_003 * 2 + 7919 * rank + layer)
    t = w["batch"] * w["ctx"]
    ch = torch.exp(0.75 * torch.randn(1, w["H_kv"], 128, generator=g, device=device))
    k = (torch.randn(t, w["H_kv"], 128, generator=g, device=device) * ch).to(dtype)
    v = torch.randn(t, w["H_kv"], 128, generator=g, device=device).to(dtype)
    return k, v


class Layer:
    pass


def build_stack(torch, ops, w, rank, device, dtype, mirror_layers):
    kb, vb, gs = MODE_BITS[w["mode"]]
    ng = 128 // gs
    t = w["batch"] * w["ctx"]
    blocks_per_seq = w["ctx"] // 16
    block_table = torch.arange(w["batch"] * blocks_per_seq, dtype=torch.int64, device=device).reshape(
        w["batch"], blocks_per_seq)                      # identity paging for timing
    seq_lens = torch.full((w["batch"],), w["ctx"], dtype=torch.int32, device=device)
    slots = torch.arange(t, dtype=torch.int64, device=device)
    gq = torch.Generator().manual_seed(4242 + rank)
    layers = []
    stage = None
    for li in range(w["layers"]):
        L = Layer()
        k, v = make_layer_kv(torch, w, li, rank, device, dtype)
        L.k_data = torch.empty(w["H_kv"], t, 16 * kb, dtype=torch.uint8, device=device)
        L.v_data = torch.empty(w["H_kv"], t, 16 * vb, dtype=torch.uint8, device=device)
        L.k_scales = torch.empty(w["H_kv"], t, ng, dtype=torch.bfloat16, device=device)
        L.v_scales = torch.empty(w["H_kv"], t, ng, dtype=torch.bfloat16, device=device)
        ops.fused_quant_write_kv(k, v, slots, L.k_data, L.k_scales, L.v_data, L.v_scales, gs, kb, vb)
        with_mirror = li < mirror_layers
        if with_mirror:  # full-precision mirror in host DRAM, (H_kv, num_slots, 128)
            L.k_shadow = torch.empty(w["H_kv"], t, 128, dtype=dtype)
            L.v_shadow = torch.empty(w["H_kv"], t, 128, dtype=dtype)
            if stage is None:
                stage = torch.empty(w["H_kv"], t, 128, dtype=dtype, pin_memory=True)
            for src, dst in ((k, L.k_shadow), (v, L.v_shadow)):
                stage.copy_(src.transpose(0, 1), non_blocking=False)
                dst.copy_(stage)
        del k, v
        L.q_host = torch.randn(w["batch"], w["H_q"], 128, generator=gq).to(dtype).pin_memory()
        L.q = L.q_host.to(device)
        L.call = ops.DecodeCall(w["mode"], L.q, L.k_data, L.k_scales, L.v_data, L.v_scales, block_table, seq_lens,
                                w["ctx"], w["H_q"], w["H_kv"], 16, w["top_k"], 128 ** -0.5)
        L.o_new = torch.zeros(w["batch"], w["H_q"], 128, dtype=dtype, device=device)
        L.o_new_host = torch.zeros(w["batch"], w["H_q"], 128, dtype=dtype).pin_memory()
        L.slots_host = torch.empty(w["batch"], w["H_q"], w["top_k"], dtype=torch.int64).pin_memory()
        L.out = torch.empty(w["batch"], w["H_q"], 128, dtype=dtype, device=device)
        L.out_host = torch.empty(w["batch"], w["H_q"], 128, dtype=dtype).pin_memory()
        L.event = torch.cuda.Event()
        if with_mirror:
            L.host_call = ops.HostCorrectionCall(L.q_host, L.k_shadow, L.v_shadow, None, L.slots_host, L.o_new_host,
                                                 128 ** -0.5)
        layers.append(L)
    torch.cuda.synchronize()
    return layers


def layer_bytes(w):
    return w["batch"] * w["H_kv"] * w["ctx"] * BYTES_PER_TOKEN_HEAD[w["mode"]]


# ---------------------------------------------------------------------------------------
# CPU arm (cpu_baseline of the b200 line, and the whole --impl reference line)
# ---------------------------------------------------------------------------------------

def cpu_layer_inputs(w, dtype_name, seed=99):
    """One layer of the workload built on the host (numpy): packed cache through the oracle's
    quantiser, 16-bit mirror, query."""
    import numpy as np
    import torch
    from oracle import jf_oracle as O
    kb, vb, gs = MODE_BITS[w["mode"]]
    dtype = torch.bfloat16 if dtype_name == "bf16" else torch.float16
    g = torch.Generator().manual_seed(seed)
    t = w["batch"] * w["ctx"]
    ch = torch.exp(0.75 * torch.randn(w["H_kv"], 1, 128, generator=g))
    k = (torch.randn(w["H_kv"], t, 128, generator=g) * ch).to(dtype)
    v = torch.randn(w["H_kv"], t, 128, generator=g).to(dtype)
    q = torch.randn(w["batch"], w["H_q"], 128, generator=g).to(dtype)
    kd, ks = O.quantize_and_pack(k.float().numpy(), gs, kb)
    vd, vs = O.quantize_and_pack(v.float().numpy(), gs, vb)
    bt = np.arange(w["batch"] * (w["ctx"] // 16), dtype=np.int64).reshape(w["batch"], -1)
    lens = np.full(w["batch"], w["ctx"], np.int32)
    return dict(k=k, v=v, q=q, kd=kd, ks=ks, vd=vd, vs=vs, bt=bt, lens=lens)


def cpu_step(w, inp, threads, correction):
    """One CPU pass over one layer: scan restatement + host correction.  Returns seconds."""
    import torch
    from oracle import native
    t0 = time.perf_counter()
    r = native.c_decode(w["mode"], inp["q"].float().numpy(), inp["kd"], inp["ks"], inp["vd"], inp["vs"], inp["bt"],
                        inp["lens"], w["ctx"], w["top_k"], 128 ** -0.5, n_threads=threads)
    slots = torch.from_numpy(r["topk_slots"])
    o_new = torch.empty_like(inp["q"])
    correction(inp["q"], inp["k"], inp["v"], slots, o_new)
    return time.perf_counter() - t0


def pick_correction(dtype_name, threads, w):
    """The reference's own cpu_topk_attn when it was built and the mirror is bf16, else the
    product's host code.  Returns (callable, label)."""
    import torch
    from oracle import native, jf_oracle as O
    mod = native.ref_cpu_topk_attn_module() if dtype_name == "bf16" else None
    hm = torch.from_numpy(O.head_map(w["batch"], w["H_q"], w["H_q"] // w["H_kv"], w["top_k"]))
    if mod is not None:
        mod.set_cpu_attn_threads(threads)
        return (lambda q, k, v, s, o: mod.cpu_topk_attn(q, k, v, hm, s, o, 128 ** -0.5, None)), \
            "scan: C restatement (the reference has no CPU scan); correction: reference cpu_topk_attn.cpp unmodified"
    from jetfire_b200 import ops
    ops.set_cpu_attn_threads(threads)
    return (lambda q, k, v, s, o: ops.cpu_topk_attn(q, k, v, None, s, o, 128 ** -0.5)), \
        "scan: C restatement (the reference has no CPU scan); correction: this library's host code"


def run_cpu_baseline(w, dtype_name, repeats=3):
    threads = os.cpu_count() or 1
    inp = cpu_layer_inputs(w, dtype_name)
    corr, label = pick_correction(dtype_name, threads, w)
    cpu_step(w, inp, threads, corr)  # warm-up
    ts = [cpu_step(w, inp, threads, corr) for _ in range(repeats)]
    best = min(ts)
    return {"value": layer_bytes(w) / best / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"1 of {w['layers']} layers of the workload (all {w['batch']} sequences, all heads), "
                      f"best of {repeats}; {label}", "ms_per_layer": best * 1e3}


def run_reference_arm(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    inp = cpu_layer_inputs(w, args.dtype)
    corr, label = pick_correction(args.dtype, threads, w)
    for _ in range(max(args.warmup, 1)):
        cpu_step(w, inp, threads, corr)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(w, inp, threads, corr)
    dt = (time.perf_counter() - t0) / args.steps
    val = layer_bytes(w) / dt / 1e9
    sample = f"each step = 1 of {w['layers']} layers of the workload on the host cores; {label}"
    line = {"impl": "reference", "metric": "decode_attn_packed_kv_GBps", "value": val, "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": args.dtype,
            "data": "synthetic", "config": {"workload": w["desc"], "mode": w["mode"], "batch": w["batch"],
                                            "ctx": w["ctx"], "top_k": w["top_k"], "layers": w["layers"]},
            "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "tokens_per_s": w["batch"] / (dt * w["layers"]), "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------

def main():
    args = parse_args()
    w = resolve_workload(args)
    if args.impl == "reference":
        run_reference_arm(args, w)
        return 0

    import torch
    import torch.distributed as dist
    from jetfire_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    cores = os.cpu_count() or 1
    # one core per rank stays with the thread that drives the GPU: with a worker on every core the
    # driving thread is preempted and every layer waits for it (16 workers: 7.2 ms per step, 15: 5.5)
    cpu_threads = args.cpu_threads or max(1, cores // world - 1)
    ops.set_cpu_attn_threads(cpu_threads)

    do_e2e = not args.no_e2e
    # The end-to-end leg needs the full-precision mirror of every layer in host DRAM (17 GB per
    # rank at the default workload).  If all ranks' mirrors would take more than 40 % of the free
    # host memory, the leg runs over the first layers only (its throughput is per layer anyway).
    mirror_layers = w["layers"] if do_e2e else 0
    if do_e2e:
        import psutil
        per_layer = 2 * w["H_kv"] * w["batch"] * w["ctx"] * 128 * 2
        need = per_layer * w["layers"] * world
        budget = 0.4 * psutil.virtual_memory().available
        if need > budget:
            mirror_layers = max(2, min(w["layers"], int(w["layers"] * budget / need)))
        if world > 1:   # rank 0 decides for everyone
            ml = torch.tensor([mirror_layers], dtype=torch.int64, device=device)
            dist.broadcast(ml, 0)
            mirror_layers = int(ml.item())
    layers = build_stack(torch, ops, w, rank, device, dtype, mirror_layers)
    n_layers = len(layers)
    step_bytes = layer_bytes(w) * n_layers

    gathered = None
    if world > 1:
        my_out = torch.empty(n_layers, w["batch"], w["H_q"] * 128, dtype=dtype, device=device)
        gathered = torch.empty(world, n_layers, w["batch"], w["H_q"] * 128, dtype=dtype, device=device)
        for i, L in enumerate(layers):   # the merge kernel writes straight into the gather's send buffer
            L.out = my_out[i].view(w["batch"], w["H_q"], 128)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-resident step as one CUDA graph (per rank; the gather stays outside it) ----
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for L in layers:      # eager warm-up (also sets kernel attributes before capture)
            L.call.fused()
            ops.blend_unnorm_into(L.call.out["o_hat"], L.call.out["o_old_unnorm"], L.call.out["W"], L.o_new, L.out)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    for L in layers:
        L.call.status()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for L in layers:
            L.call.fused()
            ops.blend_unnorm_into(L.call.out["o_hat"], L.call.out["o_old_unnorm"], L.call.out["W"], L.o_new, L.out)

    def graph_step():
        graph.replay()
        if world > 1:
            dist.all_gather_into_tensor(gathered, my_out)

    for _ in range(max(args.warmup, 3)):
        graph_step()
    barrier()
    sampler = ClockSampler(local_rank)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with sampler:
        ev0.record()
        for _ in range(args.steps):
            graph_step()
        ev1.record()
        barrier()
        # keep the region long enough for a few clock samples
        t_end = time.time() + 0.3
        while time.time() < t_end:
            graph_step()
        torch.cuda.synchronize()
    ms_total = ev0.elapsed_time(ev1)
    t = torch.tensor([ms_total], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    value = step_bytes * world / (ms_step * 1e-3) / 1e9

    # diagnostic (outside the timed region): each rank's step without the gather, so that a slow
    # GPU can be told from the coupling of the ranks through the collective
    per_rank_ms = None
    if world > 1:
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        c0.record()
        for _ in range(args.steps):
            graph.replay()
        c1.record()
        torch.cuda.synchronize()
        mine = torch.tensor([c0.elapsed_time(c1) / args.steps], dtype=torch.float64, device=device)
        every = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        per_rank_ms = [round(float(x.item()), 4) for x in every]

    # ---- roofline of the scan kernel alone ----
    for L in layers:
        L.call.scan()
    torch.cuda.synchronize()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(1, min(args.steps, 200 // max(n_layers, 1) + 1))
    s0.record()
    for _ in range(reps):
        for L in layers:
            L.call.scan()
    s1.record()
    torch.cuda.synchronize()
    scan_ms = s0.elapsed_time(s1) / (reps * n_layers)
    # restore a consistent state (select/finish after the last scan)
    for L in layers:
        L.call.select(); L.call.finish()
    torch.cuda.synchronize()
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = layer_bytes(w) / (scan_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": f"scan_{w['mode']}_kernel", "achieved": achieved, "peak": peak,
                "peak_source": "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "fallback 6650 GB/s",
                "unit": "GB/s", "frac": achieved / peak, "us_per_launch": scan_ms * 1e3,
                "algorithmic_bytes_per_launch": layer_bytes(w), "traffic": None}
    # dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of the scan kernel, per
    # (token, KV head), scaled to this launch by the units it processes (traffic grows in
    # proportion)
    roofline["traffic"] = DRAM_BYTES_PER_TOKEN_HEAD[w["mode"]] * w["batch"] * w["H_kv"] * w["ctx"]
    # the same fraction for the whole layer (scan + select+finish + merge, from `value`)
    roofline["layer_frac"] = value / world / peak

    # ---- end to end with the host in the loop ----
    e2e = None
    if do_e2e:
        copy_stream = torch.cuda.Stream()
        e2e_layers = layers[:mirror_layers]

        def e2e_step():
            main_s = torch.cuda.current_stream()
            for L in e2e_layers:
                L.q.copy_(L.q_host, non_blocking=True)
                L.call.fused()
                L.slots_host.copy_(L.call.out["topk_slots"], non_blocking=True)
                L.event.record(main_s)

            def merge(L):  # o_new host -> device, merge, result device -> host; on the copy stream
                with torch.cuda.stream(copy_stream):
                    L.o_new.copy_(L.o_new_host, non_blocking=True)
                    ops.blend_unnorm_into(L.call.out["o_hat"], L.call.out["o_old_unnorm"], L.call.out["W"],
                                          L.o_new, L.out)
                    L.out_host.copy_(L.out, non_blocking=True)

            # The next layer's correction is queued before the previous one is waited for, so the
            # workers flow from one job into the next; merges are launched as jobs complete.
            prev = None
            for L in e2e_layers:
                L.event.synchronize()
                ticket = L.host_call.submit()
                if prev is not None:
                    L.host_call.wait_ticket(prev[1])
                    merge(prev[0])
                prev = (L, ticket)
            prev[0].host_call.wait_ticket(prev[1])
            merge(prev[0])
            copy_stream.synchronize()
            if world > 1:
                dist.all_gather_into_tensor(gathered, my_out)

        e2e_steps = max(3, min(args.steps, 10))
        for _ in range(2):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        barrier()
        dt = (time.perf_counter() - t0) / e2e_steps
        tt = torch.tensor([dt], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt = float(tt.item())
        esz = 2
        n_e2e = len(e2e_layers)
        h2d = n_e2e * 2 * w["batch"] * w["H_q"] * 128 * esz
        d2h = n_e2e * (w["batch"] * w["H_q"] * w["top_k"] * 8 + w["batch"] * w["H_q"] * 128 * esz)
        # dt covers n_e2e layers; ms_per_step and tokens/s are scaled to the workload's layer count
        dt_full = dt * n_layers / n_e2e
        e2e = {"value": layer_bytes(w) * n_e2e * world / dt / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d * world,
               "d2h_bytes_per_step": d2h * world, "ms_per_step": dt_full * 1e3, "steps": e2e_steps,
               "layers_measured": n_e2e,
               "tokens_per_s": w["batch"] * world / dt_full, "host_threads_per_rank": cpu_threads,
               "timing": "host wall clock around barrier + synchronize (host work is inside the region)"}
        if n_e2e < n_layers:
            e2e["note"] = (f"host memory: mirrors of {n_e2e} of {n_layers} layers; the copies above are per measured "
                           "step, ms_per_step and tokens_per_s are scaled to all layers")
        for L in layers:
            L.call.status()

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_baseline = run_cpu_baseline(w, args.dtype)

    # clocks of every rank's GPU during the timed region: the slowest one decides the step
    clocks = sampler.summary()
    if world > 1:
        every_clock = [None] * world
        dist.all_gather_object(every_clock, clocks)
        known = [c["sm_mhz"] for c in every_clock if c["sm_mhz"] is not None]
        clocks = {"sm_mhz": min(known) if known else None, "sm_max_mhz": clocks["sm_max_mhz"],
                  "reasons": sorted({r for c in every_clock for r in c["reasons"]}),
                  "samples": min(c["samples"] for c in every_clock),
                  "per_rank_sm_mhz": [c["sm_mhz"] for c in every_clock],
                  "per_rank_reasons": [c["reasons"] for c in every_clock]}
    if rank == 0:
        line = {
            "metric": "decode_attn_packed_kv_GBps", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": args.dtype,
            "data": "synthetic",
            "config": {"workload": w["desc"], "mode": w["mode"], "batch_per_gpu": w["batch"], "ctx": w["ctx"],
                       "top_k": w["top_k"], "layers": w["layers"], "H_q_per_gpu": w["H_q"], "H_kv_per_gpu": w["H_kv"],
                       "sharding": "KV heads per GPU fixed; outputs all-gathered (NCCL) once per step" if world > 1
                       else "single GPU",
                       "l2": f"inputs larger than L2: {step_bytes / 1e6:.0f} MB of packed KV per step, each byte read once"},
            "tokens_per_s": w["batch"] * world / (ms_step * 1e-3),
            "us_per_layer": ms_step * 1e3 / n_layers,
            "gpu_launches": 3 * n_layers * args.steps,  # per layer: scan, select+finish, merge
            "per_rank_ms_without_gather": per_rank_ms,
            "roofline": roofline, "e2e": e2e, "cpu_baseline": cpu_baseline, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
