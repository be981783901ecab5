#!/usr/bin/env python3
"""Benchmark of the decode hot path: packed-KV bytes scanned per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c1|c2|c3|c4|c5]

Workload (``config.workload``): one decode step = one pass of the hot path over every layer of
a stack with independent, seeded synthetic KV per layer.  The default is the K3V2 configuration
of the Llama-3.3-70B attention geometry (64 query heads, 8 KV heads, head_dim 128, GQA group 8),
80 layers, batch 4, context 65536, top-k 512 -- the mode and context range the headline metric is
quoted on; it fits one GPU (14.8 GB of packed KV), and at ``--gpus N`` the SAME workload is
sharded: KV heads over the GPUs first, then the batch (``jetfire_b200.adapter.sharding``), so the
total work is fixed ("strong" scaling).  ``--workload c1|c2|c4`` select the other configurations
(c2 = Llama-3.1-8B geometry, K4V4, B 4, ctx 32768, 32 layers; c4 = Qwen3-30B-A3B geometry, K3V2,
B 8, ctx 32768, 48 layers), ``--workload c5`` the append + decode sweep; ``--mode/--batch/--ctx/
--layers/--top-k`` override single fields.

Synthetic data: every K/V element is a pure function of (layer, tensor, KV head, sequence,
position, channel) through a 64-bit counter hash -- twelve 16-bit uniforms summed (an
Irwin-Hall stand-in for N(0,1): mean 0, variance 1, integer arithmetic only) -- K scaled per
channel by a log-normal(0, 0.75) factor.  The GPU (torch integer ops) and the CPU (numpy)
evaluate the same function bit for bit, so any rank can build any shard, and any timed row can
be replayed through the CPU oracle (done for one (layer, sequence, KV head) outside the timed
region; ``run.oracle_check``).

What is timed
  value     device-resident: per layer the scan, the select+finish kernel and the correction
            merge (o_new resident), all layers of a step replayed as one CUDA graph, plus (N > 1)
            the NCCL gather of the per-head outputs into the (B, H_q * 128) layout, captured as a
            graph of its own; CUDA events on the launching stream, max over ranks.
  e2e       the same step through the public ops with HOST buffers: q host->device, selected
            slots device->host, the host correction (C++ worker pool over the full-precision
            mirror in host DRAM), o_new host->device, merge, output device->host.  Layers are
            pipelined (the GPU runs ahead while the host corrects; the synthetic layers are
            independent); ``e2e.serial_layers`` is the same with layer l+1 starting after layer
            l's merge, as a real decoder must.
  roofline  over the span scan + select+finish + merge of a layer (frac), with every kernel --
            and the quantise-on-append kernel -- timed on its own beside it (per_kernel).
  cpu_baseline  a bounded sample of the workload on the host cores: the C restatement of the scan
            (the reference has no CPU scan) plus the reference's own host correction.
  reference_gpu_kernels  the reference's own GPU kernels compiled from their unmodified sources for
            sm_100 (when they were built), on one layer of the same inputs.
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
DEFAULT_WORKLOAD = "c3"
BYTES_PER_TOKEN_HEAD = {"k3v2": 88, "k4v4": 132}
MODE_BITS = {"k3v2": (3, 2, 64), "k4v4": (4, 4, 128)}
# dram__bytes_read.sum + dram__bytes_write.sum of the scan kernel per (token, KV head), from the ncu
# captures summarised under profiles/ (scaled to a launch by the units it processes)
DRAM_BYTES_PER_TOKEN_HEAD = {"k3v2": 94.9, "k4v4": 137.3}
METRIC = "decode_attn_packed_kv_GBps"


def parse_args():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS) + ["c5"])
    ap.add_argument("--mode", choices=["k3v2", "k4v4"])
    ap.add_argument("--batch", type=int)
    ap.add_argument("--ctx", type=int)
    ap.add_argument("--layers", type=int)
    ap.add_argument("--top-k", type=int)
    ap.add_argument("--stage-b", choices=["fp32", "int8p"], help="K4V4 weights (default: int8p when batch > 1, "
                    "the reference's release plan)")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-in-the-loop measurement")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU and reference-kernel baselines")
    ap.add_argument("--no-extra", action="store_true", help="skip the extra single-GPU configurations")
    ap.add_argument("--no-check", action="store_true", help="skip the oracle replay of one timed row")
    ap.add_argument("--cpu-threads", type=int, default=0, help="host correction threads (0 = cores / ranks - 1)")
    ap.add_argument("--no-huge-pages", action="store_true", help="host mirrors on the system's default pages")
    ap.add_argument("--gpu-correction-share", default="auto", metavar="auto|F",
                    help="end-to-end leg: fraction of the correction's rows the GPU computes straight from the host "
                         "mirror over the host link while the workers do the rest (auto: from the two measured rates; "
                         "0: the workers do all of it)")
    ap.add_argument("--no-numa", action="store_true",
                    help="leave the host mirrors and the correction workers where the system puts them")
    ap.add_argument("--as-shard", metavar="R/N", help="single GPU only: run the shard that rank R of an N-GPU run owns "
                    "(same seeded data, no gather); every figure then counts that shard's bytes")
    return ap.parse_args()


def resolve_workload(args, name=None):
    mode, h_q, h_kv, batch, ctx, top_k, layers, desc = WORKLOADS[name or args.workload]
    custom = name is None and any(v is not None for v in (args.mode, args.batch, args.ctx, args.layers, args.top_k))
    if name is None:
        mode, batch, ctx = args.mode or mode, args.batch or batch, args.ctx or ctx
        layers, top_k = args.layers or layers, args.top_k or top_k
    if custom:
        desc = f"custom: {mode}, H_q {h_q}, H_kv {h_kv}, B{batch}, ctx {ctx}, top-k {top_k}, {layers} layers"
    # the reference's release plan: K4V4 with a configured batch above 1 rounds the weights per tile
    stage_b = "fp32"
    if mode == "k4v4":
        stage_b = (args.stage_b if name is None and args.stage_b else ("int8p" if batch > 1 else "fp32"))
    return dict(mode=mode, H_q=h_q, H_kv=h_kv, batch=batch, ctx=ctx, top_k=top_k, layers=layers, desc=desc,
                stage_b=stage_b, name=name or args.workload)


def config_dict(w, world, dtype):
    """The same for both arms, so that their lines can be matched."""
    per_gpu = w["batch"] * w["H_kv"] * w["ctx"] * BYTES_PER_TOKEN_HEAD[w["mode"]] * w["layers"] / max(world, 1)
    return {"workload": w["desc"], "mode": w["mode"], "H_q": w["H_q"], "H_kv": w["H_kv"], "batch": w["batch"],
            "ctx": w["ctx"], "top_k": w["top_k"], "layers": w["layers"], "stage_b": w["stage_b"], "dtype": dtype,
            "n_gpus": world,
            "l2": f"inputs larger than L2: {per_gpu / 1e6:.0f} MB of packed KV per GPU and step, each byte read once"}


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
# synthetic data: a counter hash that torch (GPU) and numpy (CPU) evaluate identically
# ---------------------------------------------------------------------------------------

_GOLD = 0x9E3779B97F4A7C15
_MUL1, _MUL2 = 0xBF58476D1CE4E5B9, 0x94D049BB133111EB
_LANES = 0x0000FFFF0000FFFF
T_K, T_V, T_Q, T_C = 0, 1, 2, 3     # tensor ids


def _s64(x: int) -> int:
    """A 64-bit pattern as the signed Python int torch's int64 arithmetic wants."""
    x &= (1 << 64) - 1
    return x - (1 << 64) if x >= (1 << 63) else x


def _unit_normal_np(idx, seed):
    """idx: uint64 array of element counters -> float32 values, mean 0, variance 1."""
    import numpy as np
    u = np.uint64
    total = np.zeros(idx.shape, np.uint64)
    with np.errstate(over="ignore"):
        for j in range(3):
            z = (idx * u(4) + u(j)) * u(_GOLD) + u(seed)
            z = (z ^ (z >> u(30))) * u(_MUL1)
            z = (z ^ (z >> u(27))) * u(_MUL2)
            z = z ^ (z >> u(31))
            a = (z & u(_LANES)) + ((z >> u(16)) & u(_LANES))
            total += (a & u(0xFFFFFFFF)) + (a >> u(32))
    return ((2.0 * total.astype(np.float64) - 12.0 * 65535.0) * 2.0 ** -17).astype(np.float32)


def _unit_normal_torch(idx, seed):
    """The same function on an int64 tensor (two's-complement arithmetic wraps like uint64)."""
    import torch

    def lsr(x, k):
        return (x >> k) & ((1 << (64 - k)) - 1)

    total = torch.zeros_like(idx)
    for j in range(3):
        z = (idx * 4 + j) * _s64(_GOLD) + _s64(seed)
        z = (z ^ lsr(z, 30)) * _s64(_MUL1)
        z = (z ^ lsr(z, 27)) * _s64(_MUL2)
        z = z ^ lsr(z, 31)
        a = (z & _LANES) + (lsr(z, 16) & _LANES)
        total += (a & 0xFFFFFFFF) + lsr(a, 32)
    return ((2.0 * total.to(torch.float64) - 12.0 * 65535.0) * 2.0 ** -17).to(torch.float32)


def _counter(xp, w, layer, tensor, head, seq, pos, chan):
    """Element counter; all arguments broadcastable integer arrays / scalars."""
    return ((((layer * 4 + tensor) * w["H_kv"] + head) * w["batch"] + seq) * w["ctx"] + pos) * 128 + chan


def data_seed(w):
    """One seed per configuration (1_000_003 * its index; the sweep has its own)."""
    names = sorted(WORKLOADS)
    return 1_000_003 * ((1 + names.index(w["name"])) if w["name"] in names else 99)


def channel_scale_np(w, layer):
    """(H_kv, 128) float32 log-normal(0, 0.75) K channel factors of a layer (computed on the host, shipped)."""
    import numpy as np
    h = np.arange(w["H_kv"], dtype=np.uint64)[:, None]
    d = np.arange(128, dtype=np.uint64)[None, :]
    n = _unit_normal_np(_counter(np, w, np.uint64(layer), np.uint64(T_C), h, np.uint64(0), np.uint64(0), d), data_seed(w))
    return np.exp(0.75 * n.astype(np.float64)).astype(np.float32)


def query_np(w, layer):
    """(B, H_q, 128) float32 N(0,1)-like query of a layer (H_q takes the head slot of the counter)."""
    import numpy as np
    wq = dict(w, H_kv=w["H_q"])
    b = np.arange(w["batch"], dtype=np.uint64)[:, None, None]
    h = np.arange(w["H_q"], dtype=np.uint64)[None, :, None]
    d = np.arange(128, dtype=np.uint64)[None, None, :]
    return _unit_normal_np(_counter(np, wq, np.uint64(layer), np.uint64(T_Q), h, b, np.uint64(0), d), data_seed(w))


def kv_rows_np(w, layer, tensor, head, seq, c_scale=None):
    """(ctx, 128) float32 rows of one (layer, KV head, sequence) on the host."""
    import numpy as np
    p = np.arange(w["ctx"], dtype=np.uint64)[:, None]
    d = np.arange(128, dtype=np.uint64)[None, :]
    x = _unit_normal_np(_counter(np, w, np.uint64(layer), np.uint64(tensor), np.uint64(head), np.uint64(seq), p, d),
                        data_seed(w))
    return x * c_scale[head][None, :] if (tensor == T_K and c_scale is not None) else x


def kv_rows_torch(torch, w, layer, tensor, kv_start, kv_count, b_start, b_count, device, dtype, c_scale=None,
                  chunk_tokens=8192):
    """(b_count * ctx, kv_count, 128) rows of a shard in token-major order, in `dtype`."""
    out = torch.empty(b_count * w["ctx"], kv_count, 128, dtype=dtype, device=device)
    h = torch.arange(kv_start, kv_start + kv_count, dtype=torch.int64, device=device)[None, :, None]
    d = torch.arange(128, dtype=torch.int64, device=device)[None, None, :]
    cs = None
    if tensor == T_K and c_scale is not None:
        cs = torch.from_numpy(c_scale[kv_start:kv_start + kv_count]).to(device)[None]
    for b in range(b_count):
        for p0 in range(0, w["ctx"], chunk_tokens):
            p1 = min(p0 + chunk_tokens, w["ctx"])
            p = torch.arange(p0, p1, dtype=torch.int64, device=device)[:, None, None]
            x = _unit_normal_torch(_counter(torch, w, layer, tensor, h, b_start + b, p, d), data_seed(w))
            if cs is not None:
                x = x * cs
            out[b * w["ctx"] + p0:b * w["ctx"] + p1] = x.to(dtype)
    return out


# ---------------------------------------------------------------------------------------
# the stack of layers of one rank's shard
# ---------------------------------------------------------------------------------------

class Layer:
    pass


def build_stack(torch, ops, w, shard, device, dtype, mirror_layers, n_layers=None, layer0=0, huge_pages=True,
                numa_node=-1):
    """Packed caches (through the product's append kernel), queries, decode calls and -- for the
    first `mirror_layers` layers -- the full-precision host mirror of this shard."""
    kb, vb, gs = MODE_BITS[w["mode"]]
    ng = 128 // gs
    B, H_kv, H_q = shard.b_count, shard.kv_count, shard.q_count
    t = B * w["ctx"]
    blocks_per_seq = w["ctx"] // 16
    block_table = torch.arange(B * blocks_per_seq, dtype=torch.int64, device=device).reshape(B, blocks_per_seq)
    seq_lens = torch.full((B,), w["ctx"], dtype=torch.int32, device=device)
    slots = torch.arange(t, dtype=torch.int64, device=device)
    layers, stage = [], None
    for li in range(layer0, layer0 + (n_layers if n_layers is not None else w["layers"])):
        L = Layer()
        L.index = li
        cs = channel_scale_np(w, li)
        k = kv_rows_torch(torch, w, li, T_K, shard.kv_start, H_kv, shard.b_start, B, device, dtype, cs)
        v = kv_rows_torch(torch, w, li, T_V, shard.kv_start, H_kv, shard.b_start, B, device, dtype)
        L.k_data = torch.empty(H_kv, t, 16 * kb, dtype=torch.uint8, device=device)
        L.v_data = torch.empty(H_kv, t, 16 * vb, dtype=torch.uint8, device=device)
        L.k_scales = torch.empty(H_kv, t, ng, dtype=torch.bfloat16, device=device)
        L.v_scales = torch.empty(H_kv, t, ng, dtype=torch.bfloat16, device=device)
        ops.fused_quant_write_kv(k, v, slots, L.k_data, L.k_scales, L.v_data, L.v_scales, gs, kb, vb)
        with_mirror = (li - layer0) < mirror_layers
        if with_mirror:  # full-precision mirror in host DRAM, (H_kv, num_slots, 128)
            L.k_shadow = torch.empty(H_kv, t, 128, dtype=dtype)
            L.v_shadow = torch.empty(H_kv, t, 128, dtype=dtype)
            if huge_pages:   # before the first write: the random row gathers of the correction miss the TLB less
                ops.advise_huge_pages(L.k_shadow)
                ops.advise_huge_pages(L.v_shadow)
            if numa_node >= 0:   # likewise before the first write
                ops.bind_memory_to_node(L.k_shadow, numa_node)
                ops.bind_memory_to_node(L.v_shadow, numa_node)
            if stage is None:
                stage = torch.empty(H_kv, t, 128, dtype=dtype, pin_memory=True)
            for src, dst in ((k, L.k_shadow), (v, L.v_shadow)):
                stage.copy_(src.transpose(0, 1), non_blocking=False)
                dst.copy_(stage)
        L.kv_tokens = (k, v) if (li == layer0) else None     # kept for the append timing
        del k, v
        q_full = torch.from_numpy(query_np(w, li)).to(dtype)
        L.q_host = q_full[shard.b_start:shard.b_start + B, shard.q_start:shard.q_start + H_q].contiguous().pin_memory()
        L.q = L.q_host.to(device)
        L.call = ops.DecodeCall(w["mode"], L.q, L.k_data, L.k_scales, L.v_data, L.v_scales, block_table, seq_lens,
                                w["ctx"], H_q, H_kv, 16, w["top_k"], 128 ** -0.5, stage_b=w["stage_b"], slots_i32=True)
        L.o_new = torch.zeros(B, H_q, 128, dtype=dtype, device=device)
        L.o_new_host = torch.zeros(B, H_q, 128, dtype=dtype).pin_memory()
        L.slots_host = torch.empty(B, H_q, w["top_k"], dtype=torch.int32).pin_memory()   # 32-bit slot lists: half the D2H
        L.out = torch.empty(B, H_q, 128, dtype=dtype, device=device)
        L.out_host = torch.empty(B, H_q, 128, dtype=dtype).pin_memory()
        L.event = torch.cuda.Event()
        if with_mirror:
            L.host_call = ops.HostCorrectionCall(L.q_host, L.k_shadow, L.v_shadow, None, L.slots_host, L.o_new_host,
                                                 128 ** -0.5)
        layers.append(L)
    torch.cuda.synchronize()
    return layers, (block_table, seq_lens, slots)


def layer_bytes(w, b=None, h_kv=None):
    return (b if b is not None else w["batch"]) * (h_kv if h_kv is not None else w["H_kv"]) * w["ctx"] * \
        BYTES_PER_TOKEN_HEAD[w["mode"]]


def merge(ops, L):
    ops.blend_unnorm_into(L.call.out["o_hat"], L.call.out["o_old_unnorm"], L.call.out["W"], L.o_new, L.out)


def time_loop(torch, fn, reps):
    """Mean device time of fn() in microseconds (CUDA events on the current stream)."""
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def time_graph(torch, fn, reps):
    """The same for a sequence of launches replayed as one CUDA graph, so that short kernels are
    timed on the device and not by how fast the host can launch them."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return time_loop(torch, g.replay, reps)


def per_kernel_times(torch, ops, w, layers, reps):
    """Each kernel of a layer replayed on its own over all layers (inputs larger than L2 in total)."""
    n = len(layers)

    def scans():
        for L in layers:
            L.call.scan()

    def selects():
        for L in layers:
            L.call.select_finish()

    def merges():
        for L in layers:
            merge(ops, L)

    t_scan = time_graph(torch, scans, reps) / n
    t_sel = time_graph(torch, selects, reps) / n
    t_mrg = time_graph(torch, merges, reps) / n
    return {"scan_us": t_scan, "select_finish_us": t_sel, "merge_us": t_mrg}


# ---------------------------------------------------------------------------------------
# CPU arm (cpu_baseline of the b200 line, and the whole --impl reference line)
# ---------------------------------------------------------------------------------------

def cpu_sample(w):
    """The bounded sample of the workload a CPU step runs: one layer, as many whole sequences as
    keep it near 128 (sequence, query head) rows."""
    b = max(1, min(w["batch"], 128 // w["H_q"]))
    return dict(w, batch=b, layers=1), f"1 of {w['layers']} layers, {b} of {w['batch']} sequences, all heads"


def cpu_layer_inputs(ws, dtype_name, seed=99):
    """The sample built on the host: packed cache through the oracle's quantiser, 16-bit mirror, query."""
    import numpy as np
    import torch
    from oracle import jf_oracle as O
    kb, vb, gs = MODE_BITS[ws["mode"]]
    dtype = torch.bfloat16 if dtype_name == "bf16" else torch.float16
    g = torch.Generator().manual_seed(seed)
    t = ws["batch"] * ws["ctx"]
    ch = torch.exp(0.75 * torch.randn(ws["H_kv"], 1, 128, generator=g))
    k = (torch.randn(ws["H_kv"], t, 128, generator=g) * ch).to(dtype)
    v = torch.randn(ws["H_kv"], t, 128, generator=g).to(dtype)
    q = torch.randn(ws["batch"], ws["H_q"], 128, generator=g).to(dtype)
    kd = np.empty((ws["H_kv"], t, 16 * kb), np.uint8)
    vd = np.empty((ws["H_kv"], t, 16 * vb), np.uint8)
    ks = np.empty((ws["H_kv"], t, 128 // gs), np.uint16)
    vs = np.empty((ws["H_kv"], t, 128 // gs), np.uint16)
    for h in range(ws["H_kv"]):       # head by head: bounds the host memory of the numpy quantiser
        kd[h], ks[h] = O.quantize_and_pack(k[h].float().numpy(), gs, kb)
        vd[h], vs[h] = O.quantize_and_pack(v[h].float().numpy(), gs, vb)
    bt = np.arange(ws["batch"] * (ws["ctx"] // 16), dtype=np.int64).reshape(ws["batch"], -1)
    lens = np.full(ws["batch"], ws["ctx"], np.int32)
    return dict(k=k, v=v, q=q, kd=kd, ks=ks, vd=vd, vs=vs, bt=bt, lens=lens)


def cpu_step(ws, inp, threads, correction):
    """One CPU pass over the sample: scan restatement + host correction.  Returns seconds."""
    import torch
    from oracle import native
    t0 = time.perf_counter()
    r = native.c_decode(ws["mode"], inp["q"].float().numpy(), inp["kd"], inp["ks"], inp["vd"], inp["vs"], inp["bt"],
                        inp["lens"], ws["ctx"], ws["top_k"], 128 ** -0.5, n_threads=threads, stage_b=ws["stage_b"])
    slots = torch.from_numpy(r["topk_slots"])
    o_new = torch.empty_like(inp["q"])
    correction(inp["q"], inp["k"], inp["v"], slots, o_new)
    return time.perf_counter() - t0


def pick_correction(dtype_name, threads, ws):
    """The reference's own cpu_topk_attn when it was built and the mirror is bf16, else the
    product's host code.  Returns (callable, label, kind)."""
    import torch
    from oracle import native, jf_oracle as O
    mod = native.ref_cpu_topk_attn_module() if dtype_name == "bf16" else None
    hm = torch.from_numpy(O.head_map(ws["batch"], ws["H_q"], ws["H_q"] // ws["H_kv"], ws["top_k"]))
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
    ws, what = cpu_sample(w)
    inp = cpu_layer_inputs(ws, dtype_name)
    corr, label = pick_correction(dtype_name, threads, ws)
    cpu_step(ws, inp, threads, corr)  # warm-up
    ts = [cpu_step(ws, inp, threads, corr) for _ in range(repeats)]
    best = min(ts)
    return {"value": layer_bytes(ws) / best / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{what}, best of {repeats}; {label}", "ms_per_sample": best * 1e3}


def run_reference_arm(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    ws, what = cpu_sample(w)
    inp = cpu_layer_inputs(ws, args.dtype)
    corr, label = pick_correction(args.dtype, threads, ws)
    for _ in range(max(args.warmup, 1)):
        cpu_step(ws, inp, threads, corr)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(ws, inp, threads, corr)
    dt = (time.perf_counter() - t0) / args.steps
    val = layer_bytes(ws) / dt / 1e9
    sample = f"each step = {what} of the workload on the host cores; {label}"
    scale = (w["batch"] * w["layers"]) / ws["batch"]      # samples per whole-workload step
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": args.dtype,
            "data": "synthetic", "config": config_dict(w, args.gpus, args.dtype),
            "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "tokens_per_s": w["batch"] / (dt * scale), "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_reference_gpu_kernels(torch, w, L, tables, dtype):
    """The reference's own GPU kernels (unmodified sources built for sm_100; the int8tc_* pair with
    only the architecture flag of their loader changed) on one layer of the same inputs: Stage A,
    Stage B and the blend, timed with CUDA events.  None when they were not built or the query is
    not bf16 (the reference accepts nothing else)."""
    from oracle import native
    if dtype != torch.bfloat16:
        return None
    k3 = w["mode"] == "k3v2"
    names = ("int3_qk_scores", "int2_softmax_v", "blend") if k3 else \
        ("int8tc_qk_scores", "int8tc_softmax_v_fused" if w["stage_b"] == "int8p" else "int4_softmax_v", "blend")
    mods = [native.ref_gpu_module(n) for n in names]
    if any(m is None for m in mods):
        return None
    qk, sv, bl = mods
    bt, sl, _ = tables
    B, H_q, H_kv = L.q.shape[0], L.q.shape[1], L.k_data.shape[0]
    geom = (w["ctx"], H_q, H_kv, 16)
    out = torch.empty_like(L.out)

    def step():
        if k3:
            scores, idx, _slots = qk.int3_qk_scores_topk(L.q, L.k_data, L.k_scales, bt, sl, *geom, 128 ** -0.5, w["top_k"])
            o_hat, o_old, W = sv.int2_softmax_v_with_pre_corr_wvs2(scores, L.v_data, L.v_scales, bt, sl, idx, *geom, w["top_k"])
        else:
            scores, idx, _slots, m, iz = qk.int8tc_qk_scores_topk_stats(L.q, L.k_data, L.k_scales, bt, sl, *geom,
                                                                         128 ** -0.5, w["top_k"])
            if w["stage_b"] == "int8p":
                o_hat, o_old, W = sv.int8tc_softmax_v_with_pre_corr_reg_stats(scores, m, iz, L.v_data, L.v_scales, bt, sl,
                                                                              idx, *geom, w["top_k"])
            else:
                o_hat, o_old, W = sv.int4_softmax_v_with_pre_corr_wvs2_scores(scores, L.v_data, L.v_scales, bt, sl, idx,
                                                                              *geom, w["top_k"])
        bl.blend_unnorm_into(o_hat, o_old, W, L.o_new, out)

    us = time_loop(torch, step, 5)
    nbytes = layer_bytes(w, B, H_kv)
    return {"value": nbytes / us / 1e3, "unit": "GB/s", "us_per_layer": us,
            "what": "reference Stage A + Stage B + blend kernels, " + ", ".join(names) +
                    (" (unmodified sources, sm_100)" if k3 else " (unmodified sources; loader flag sm_90 -> sm_100)") +
                    ", one layer of this rank's shard, eager launches, L2 not flushed"}


# ---------------------------------------------------------------------------------------
# oracle replay of one timed row group (outside the timed region)
# ---------------------------------------------------------------------------------------

def oracle_check(torch, w, shard, L, seq_local=0, head_local=0):
    """Rebuild one (layer, sequence, KV head) of the timed data on the host with numpy, run the CPU
    oracle over it and compare with what the GPU produced for the same rows: top-k lists must be
    identical, o_hat within the output gate."""
    import numpy as np
    from oracle import jf_oracle as O, native
    kb, vb, gs = MODE_BITS[w["mode"]]
    G = w["H_q"] // w["H_kv"]
    head, seq = shard.kv_start + head_local, shard.b_start + seq_local
    cs = channel_scale_np(w, L.index)
    to16 = (lambda a: O.bf16_bits_to_f32(O.f32_to_bf16_bits(a))) if L.q.dtype == torch.bfloat16 else \
        (lambda a: a.astype(np.float16).astype(np.float32))
    k = to16(kv_rows_np(w, L.index, T_K, head, seq, cs))
    v = to16(kv_rows_np(w, L.index, T_V, head, seq))
    kd, ks = O.quantize_and_pack(k[None], gs, kb)
    vd, vs = O.quantize_and_pack(v[None], gs, vb)
    same_cache = bool(np.array_equal(kd[0], L.k_data[head_local, seq_local * w["ctx"]:(seq_local + 1) * w["ctx"]].cpu().numpy()))
    q = to16(query_np(w, L.index)[seq:seq + 1, head * G:(head + 1) * G])
    bt = np.arange(w["ctx"] // 16, dtype=np.int64)[None]
    ref = native.c_decode(w["mode"], q, kd, ks, vd, vs, bt, np.array([w["ctx"]], np.int32), w["ctx"], w["top_k"],
                          128 ** -0.5, stage_b=w["stage_b"])
    rows = slice(head_local * G, (head_local + 1) * G)
    idx = L.call.out["topk_idx"][seq_local, rows].cpu().numpy()
    o_hat = L.call.out["o_hat"][seq_local, rows].cpu().numpy()
    err = float(np.abs(o_hat - ref["o_hat"][0]).max())
    ok = same_cache and bool(np.array_equal(idx, ref["topk_idx"][0])) and \
        bool((np.abs(o_hat - ref["o_hat"][0]) <= 2e-3 + 1e-3 * np.abs(ref["o_hat"][0])).all())
    return {"layer": L.index, "sequence": seq, "kv_head": head, "packed_bytes_equal": same_cache,
            "topk_equal": bool(np.array_equal(idx, ref["topk_idx"][0])), "o_hat_max_abs_err": err, "ok": ok}


# ---------------------------------------------------------------------------------------
# c5: append + decode sweep
# ---------------------------------------------------------------------------------------

def run_c5(torch, ops, args, device, dtype):
    """Llama-3.1-8B layer geometry, context 8k/32k/128k x batch 1/4/16 x both modes: the timed
    quantise-on-append of a 32768-token chunk (packed cache + host-mirror rows written by the same
    kernel into mapped memory), then 128 decode steps, each appending one token per sequence and
    scanning the grown context.  One layer; every step is a replay of one captured graph."""
    peak = measured_peak()
    rows = []
    H_q, H_kv, top_k, steps = 32, 8, 256, 128
    for mode in ("k3v2", "k4v4"):
        kb, vb, gs = MODE_BITS[mode]
        ng = 128 // gs
        # -- append of a 32768-token chunk --
        T = 32768
        w = dict(mode=mode, H_q=H_q, H_kv=H_kv, batch=1, ctx=T, top_k=top_k, layers=1, name="c5", stage_b="fp32")
        cs = channel_scale_np(w, 0)
        k = kv_rows_torch(torch, w, 0, T_K, 0, H_kv, 0, 1, device, dtype, cs)
        v = kv_rows_torch(torch, w, 0, T_V, 0, H_kv, 0, 1, device, dtype)
        kd = torch.empty(H_kv, T, 16 * kb, dtype=torch.uint8, device=device)
        vd = torch.empty(H_kv, T, 16 * vb, dtype=torch.uint8, device=device)
        ks = torch.empty(H_kv, T, ng, dtype=torch.bfloat16, device=device)
        vs = torch.empty(H_kv, T, ng, dtype=torch.bfloat16, device=device)
        sl = torch.arange(T, dtype=torch.int64, device=device)
        us = time_loop(torch, lambda: ops.fused_quant_write_kv(k, v, sl, kd, ks, vd, vs, gs, kb, vb), 20)
        kh, kdv = ops.alloc_mapped_pinned_pair((H_kv, T, 128), dtype)
        vh, vdv = ops.alloc_mapped_pinned_pair((H_kv, T, 128), dtype)
        us_m = time_loop(torch, lambda: ops.fused_quant_write_kv_mirror(k, v, sl, kd, ks, vd, vs, gs, kb, vb, kdv, vdv), 5)
        a_bytes = 2 * T * H_kv * 256 + T * H_kv * BYTES_PER_TOKEN_HEAD[mode]
        append = {"tokens": T, "algorithmic_bytes": a_bytes, "us": us, "GBps": a_bytes / us / 1e3,
                  "frac_of_hbm_peak": a_bytes / us / 1e3 / peak,
                  "with_host_mirror_us": us_m, "host_link_GBps": 2 * T * H_kv * 256 / us_m / 1e3}
        del k, v, kd, vd, ks, vs, kh, kdv, vh, vdv
        for ctx in (8192, 32768, 131072):
            for B in (1, 4, 16):
                cap = ctx + steps + 16 - (ctx + steps) % 16          # slots per sequence
                wd = dict(mode=mode, H_q=H_q, H_kv=H_kv, batch=B, ctx=cap, top_k=top_k, layers=1, name="c5",
                          stage_b=("int8p" if (mode == "k4v4" and B > 1) else "fp32"))
                cs = channel_scale_np(wd, 0)
                k = kv_rows_torch(torch, wd, 0, T_K, 0, H_kv, 0, B, device, dtype, cs)    # (B * cap, H_kv, 128)
                v = kv_rows_torch(torch, wd, 0, T_V, 0, H_kv, 0, B, device, dtype)
                kd = torch.zeros(H_kv, B * cap, 16 * kb, dtype=torch.uint8, device=device)
                vd = torch.zeros(H_kv, B * cap, 16 * vb, dtype=torch.uint8, device=device)
                ks = torch.zeros(H_kv, B * cap, ng, dtype=torch.bfloat16, device=device)
                vs = torch.zeros(H_kv, B * cap, ng, dtype=torch.bfloat16, device=device)
                pos = torch.arange(B * cap, dtype=torch.int64, device=device)
                prefix = torch.where(pos % cap < ctx, pos, torch.full_like(pos, -1))   # the first ctx tokens of every sequence
                ops.fused_quant_write_kv(k, v, prefix, kd, ks, vd, vs, gs, kb, vb)
                bt = torch.arange(B * cap // 16, dtype=torch.int64, device=device).reshape(B, -1)
                lens0 = torch.full((B,), ctx, dtype=torch.int32, device=device)
                lens = lens0.clone()
                q = torch.from_numpy(query_np(wd, 0)).to(dtype).to(device)
                call = ops.DecodeCall(mode, q, kd, ks, vd, vs, bt, lens, cap, H_q, H_kv, 16, top_k, 128 ** -0.5,
                                      stage_b=wd["stage_b"])
                o_new = torch.zeros(B, H_q, 128, dtype=dtype, device=device)
                out = torch.empty(B, H_q, 128, dtype=dtype, device=device)
                base = torch.arange(B, dtype=torch.int64, device=device) * cap

                def step():
                    new_slots = base + lens.to(torch.int64)                       # the token at position len of every sequence
                    ops.fused_quant_write_kv(k.index_select(0, new_slots), v.index_select(0, new_slots), new_slots,
                                             kd, ks, vd, vs, gs, kb, vb)
                    lens.add_(1)
                    call.fused()
                    ops.blend_unnorm_into(call.out["o_hat"], call.out["o_old_unnorm"], call.out["W"], o_new, out)

                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    step()
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                lens.copy_(lens0)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    step()
                lens.copy_(lens0)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(steps):
                    g.replay()
                e1.record()
                torch.cuda.synchronize()
                call.status()
                assert int(lens[0]) == ctx + steps
                us_step = e0.elapsed_time(e1) * 1e3 / steps
                nbytes = B * H_kv * (ctx + steps / 2) * BYTES_PER_TOKEN_HEAD[mode]
                rows.append({"mode": mode, "ctx": ctx, "batch": B, "stage_b": wd["stage_b"], "decode_steps": steps,
                             "us_per_step": us_step, "GBps": nbytes / us_step / 1e3,
                             "frac_of_hbm_peak": nbytes / us_step / 1e3 / peak, "tokens_per_s": B / (us_step * 1e-6)})
                del k, v, kd, vd, ks, vs, call, g
                torch.cuda.empty_cache()
        rows.append({"mode": mode, "append_32768_tokens": append})
    return rows


def to_tp_layout(gathered, full_out, head_shards):
    """gathered (world, layers, b_loc, q_loc * 128), rank r = (batch shard r // head_shards, head shard
    r % head_shards) -> full_out (layers, B, H_q * 128): every layer's outputs in the order the next
    operator of a tensor-parallel model expects."""
    world, n_layers, b_loc, qd = gathered.shape
    batch_shards = world // head_shards
    g5 = gathered.view(batch_shards, head_shards, n_layers, b_loc, qd)
    full_out.view(n_layers, batch_shards, b_loc, head_shards, qd).copy_(g5.permute(2, 0, 3, 1, 4))


def measured_peak():
    try:
        return float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text()).get("hbm_gbs", 6650.0))
    except Exception:
        return 6650.0


def peak_source():
    return "measured (MEASURED_PEAKS.json hbm_gbs)" if (ROOT / "MEASURED_PEAKS.json").exists() else "fallback 6650 GB/s"


# ---------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------

def quick_config(torch, ops, args, name, shard_cls, device, dtype, n_layers=4):
    """A few layers of another configuration on this GPU: device-resident layer time and the
    per-kernel split (extra keys of the line, single GPU only)."""
    w = resolve_workload(args, name)
    shard = shard_cls(0, 0, w["H_kv"], 0, w["H_q"], 0, w["batch"])
    layers, _ = build_stack(torch, ops, w, shard, device, dtype, 0, n_layers=min(n_layers, w["layers"]))

    def step():
        for L in layers:
            L.call.fused()
            merge(ops, L)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    us_layer = time_loop(torch, g.replay, 20) / len(layers)
    pk = per_kernel_times(torch, ops, w, layers, 10)
    for L in layers:
        L.call.status()
    peak = measured_peak()
    nb = layer_bytes(w)
    return {"workload": w["desc"], "stage_b": w["stage_b"], "layers_measured": len(layers), "us_per_layer": us_layer,
            "GBps": nb / us_layer / 1e3, "frac": nb / us_layer / 1e3 / peak,
            "scan_us": pk["scan_us"], "scan_frac": nb / pk["scan_us"] / 1e3 / peak,
            "select_finish_us": pk["select_finish_us"], "merge_us": pk["merge_us"]}


def main():
    args = parse_args()
    if args.workload == "c5" and args.impl == "reference":
        args.workload = "c1"
    w = resolve_workload(args) if args.workload != "c5" else None
    if args.impl == "reference":
        run_reference_arm(args, w)
        return 0

    import torch
    import torch.distributed as dist
    from jetfire_b200 import ops
    from jetfire_b200.adapter.sharding import Shard, shard_plan

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16

    if args.workload == "c5":
        if rank == 0:
            rows = run_c5(torch, ops, args, device, dtype)
            print(json.dumps({"metric": METRIC, "workload": "c5: append of a 32768-token chunk, then 128 decode steps "
                              "each appending one token per sequence; Llama-3.1-8B layer geometry, one layer",
                              "unit": "GB/s", "peak": measured_peak(), "peak_source": peak_source(), "sweep": rows}), flush=True)
        return 0

    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    cores = os.cpu_count() or 1
    # one core per rank stays with the thread that drives the GPU: with a worker on every core the
    # driving thread is preempted and every layer waits for it
    cpu_threads = args.cpu_threads or max(1, cores // world - 1)
    # On a host with several memory nodes the mirrors of this rank and the workers that gather
    # from them go to the node its GPU is attached to (nothing happens on a single-node host, or
    # where the system does not say where the GPU sits).
    from jetfire_b200.adapter.sharding import resolve_numa_node, workers_on_node
    numa_nodes = ops.numa_node_count()
    numa_node = -1 if args.no_numa else resolve_numa_node(-2, ops.numa_node_of_device(device.index or 0), numa_nodes)
    if numa_node >= 0:
        try:
            node_cpus = len(ops.numa_node_cpus(numa_node))
            if not args.cpu_threads:
                cpu_threads = workers_on_node(cpu_threads, node_cpus - 1, (world + numa_nodes - 1) // numa_nodes)
            ops.set_cpu_attn_node(numa_node)
        except RuntimeError:
            numa_node = -1
    ops.set_cpu_attn_threads(cpu_threads)

    # a few layers of the other single-GPU configurations first (their memory is released again)
    extra = None
    if rank == 0 and world == 1 and not args.no_extra:
        extra = {name: quick_config(torch, ops, args, name, Shard, device, dtype)
                 for name in ("c4", "c2", "c1") if name != w["name"]}
        torch.cuda.empty_cache()

    plan = shard_plan(w["H_q"], w["H_kv"], w["batch"], world)
    shard = plan[rank]
    head_shards = min(world, w["H_kv"])
    as_shard = None
    if args.as_shard:
        if world != 1:
            raise SystemExit("--as-shard is a single-GPU diagnostic")
        r_s, n_s = (int(x) for x in args.as_shard.split("/"))
        if not (0 <= r_s < n_s):
            raise SystemExit("--as-shard R/N needs 0 <= R < N")
        shard = shard_plan(w["H_q"], w["H_kv"], w["batch"], n_s)[r_s]
        as_shard = f"{r_s}/{n_s}"
    # bytes of one layer of the whole job (of the one shard, in the --as-shard diagnostic)
    job_layer_bytes = layer_bytes(w, shard.b_count, shard.kv_count) if as_shard else layer_bytes(w)

    do_e2e = not args.no_e2e
    # The end-to-end leg needs the full-precision mirror of every layer of the shard in host DRAM.
    # If all ranks' mirrors would take more than 40 % of the free host memory, the leg runs over
    # the first layers only (its throughput is per layer anyway).
    mirror_layers = w["layers"] if do_e2e else 0
    if do_e2e:
        import psutil
        per_layer = 2 * shard.kv_count * shard.b_count * w["ctx"] * 128 * 2
        need = per_layer * w["layers"] * world
        budget = 0.4 * psutil.virtual_memory().available
        if need > budget:
            mirror_layers = max(2, min(w["layers"], int(w["layers"] * budget / need)))
        if world > 1:   # rank 0 decides for everyone
            ml = torch.tensor([mirror_layers], dtype=torch.int64, device=device)
            dist.broadcast(ml, 0)
            mirror_layers = int(ml.item())
    t_build = time.perf_counter()
    layers, tables = build_stack(torch, ops, w, shard, device, dtype, mirror_layers, huge_pages=not args.no_huge_pages,
                                 numa_node=numa_node)
    t_build = time.perf_counter() - t_build
    n_layers = len(layers)
    step_bytes_total = job_layer_bytes * n_layers

    # outputs of all layers in one buffer (the gather's send buffer); gathered: TP layout per layer
    my_out = torch.empty(n_layers, shard.b_count, shard.q_count * 128, dtype=dtype, device=device)
    for i, L in enumerate(layers):
        L.out = my_out[i].view(shard.b_count, shard.q_count, 128)
    gathered = full_out = None
    if world > 1:
        gathered = torch.empty(world, n_layers, shard.b_count, shard.q_count * 128, dtype=dtype, device=device)
        full_out = torch.empty(n_layers, w["batch"], w["H_q"] * 128, dtype=dtype, device=device)

    def gather_step():
        """One all-gather of every layer's per-head outputs, then the (B, H_q * 128) layout:
        rank r = (batch shard r // head_shards, head shard r % head_shards)."""
        dist.all_gather_into_tensor(gathered, my_out)
        to_tp_layout(gathered, full_out, head_shards)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-resident step as one CUDA graph; the gather as a graph of its own ----
    def compute_step():
        for L in layers:
            L.call.fused()
            merge(ops, L)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        compute_step()      # eager warm-up (also sets kernel attributes before capture)
        if world > 1:
            gather_step()   # brings the communicator up before any capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    for L in layers:
        L.call.status()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        compute_step()
    ggraph, gather_in_graph = None, False
    if world > 1:
        try:
            ggraph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(ggraph):
                gather_step()
            gather_in_graph = True
        except Exception:
            ggraph = None
            torch.cuda.synchronize()

    def graph_step():
        graph.replay()
        if world > 1:
            if ggraph is not None:
                ggraph.replay()
            else:
                gather_step()

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
    value = step_bytes_total / (ms_step * 1e-3) / 1e9

    # ---- multi-GPU correctness (outside the timed region): layer 0 run unsharded on rank 0's GPU.
    #      The selected positions of rank 0's own rows must be identical.  The gathered outputs are
    #      held to the output gate (2e-3 + 1e-3 relative), not to bit equality: a GPU that holds fewer
    #      (sequence, KV head) pairs cuts every row into more splits, so its fp32 sums run in a
    #      different order (the largest difference and the share of equal values are reported). ----
    gather_check = None
    if world > 1 and rank == 0 and not args.no_check:
        whole = Shard(0, 0, w["H_kv"], 0, w["H_q"], 0, w["batch"])
        ref_layers, _ = build_stack(torch, ops, w, whole, device, dtype, 0, n_layers=1)
        R = ref_layers[0]
        R.call.fused()
        merge(ops, R)
        torch.cuda.synchronize()
        got = full_out[0].view(w["batch"], w["H_q"], 128).float()
        want = R.out.float()
        diff = (got - want).abs()
        mine_idx = layers[0].call.out["topk_idx"]
        ref_idx = R.call.out["topk_idx"][shard.b_start:shard.b_start + shard.b_count,
                                         shard.q_start:shard.q_start + shard.q_count]
        gather_check = {"layer": 0, "topk_lists_equal_to_single_gpu": bool(torch.equal(mine_idx, ref_idx)),
                        "out_max_abs_diff": float(diff.max()),
                        "out_within_output_gate": bool((diff <= 2e-3 + 1e-3 * want.abs()).all()),
                        "out_bit_equal_fraction": float((got == want).float().mean())}
        del ref_layers, R
        torch.cuda.empty_cache()

    # ---- per-kernel times (every rank: a slow GPU or a slow row shows here) ----
    reps = max(2, min(args.steps, 200 // max(n_layers, 1) + 1))
    pk = per_kernel_times(torch, ops, w, layers, reps)
    rank_ms = time_loop(torch, graph.replay, max(3, min(args.steps, 10))) / 1e3   # this rank's step without the gather
    for L in layers:    # restore a consistent state (select/finish after the last scan)
        L.call.fused()
    torch.cuda.synchronize()
    per_rank = None
    if world > 1:
        mine = {"rank": rank, "ms_without_gather": round(rank_ms, 4), **{k: round(v, 2) for k, v in pk.items()}}
        per_rank = [None] * world
        dist.all_gather_object(per_rank, mine)
    # quantise-on-append: the kernel that built the caches, timed on layer 0's tokens
    kb, vb, gs = MODE_BITS[w["mode"]]
    k_tok, v_tok = layers[0].kv_tokens
    L0 = layers[0]
    pack_us = time_loop(torch, lambda: ops.fused_quant_write_kv(k_tok, v_tok, tables[2], L0.k_data, L0.k_scales,
                                                                L0.v_data, L0.v_scales, gs, kb, vb), 10)
    pack_bytes = k_tok.shape[0] * shard.kv_count * (512 + BYTES_PER_TOKEN_HEAD[w["mode"]])
    layers[0].kv_tokens = None
    del k_tok, v_tok

    peak = measured_peak()
    lb_rank = layer_bytes(w, shard.b_count, shard.kv_count)
    us_layer = ms_step * 1e3 / n_layers
    span_us = pk["scan_us"] + pk["select_finish_us"] + pk["merge_us"]
    achieved = lb_rank / (rank_ms * 1e3 / n_layers) / 1e3     # this rank's layer span inside the captured step
    roofline = {
        "bound": "hbm", "kernel": f"scan_{w['mode']}_kernel + topk_select_kernel (select+finish) + merge_correct_kernel",
        "span": "one layer of rank 0's shard inside the captured step (CUDA events over the whole step / layers)",
        "achieved": achieved, "peak": peak, "peak_source": peak_source(), "unit": "GB/s", "frac": achieved / peak,
        "us_per_layer": rank_ms * 1e3 / n_layers, "algorithmic_bytes_per_launch": lb_rank,
        # dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of the scan kernel, per
        # (token, KV head), scaled to this launch by the units it processes
        "traffic": DRAM_BYTES_PER_TOKEN_HEAD[w["mode"]] * shard.b_count * shard.kv_count * w["ctx"],
        "per_kernel": {
            f"scan_{w['mode']}_kernel": {"us": pk["scan_us"], "achieved": lb_rank / pk["scan_us"] / 1e3,
                                         "frac": lb_rank / pk["scan_us"] / 1e3 / peak},
            "topk_select_kernel (select+finish)": {"us": pk["select_finish_us"], "share_of_span": pk["select_finish_us"] / span_us},
            "merge_correct_kernel": {"us": pk["merge_us"], "share_of_span": pk["merge_us"] / span_us},
            "pack_append_kernel": {"us": pack_us, "algorithmic_bytes": pack_bytes, "achieved": pack_bytes / pack_us / 1e3,
                                   "frac": pack_bytes / pack_us / 1e3 / peak,
                                   "what": "quantise-on-append of one layer of the shard (K and V in one launch)"},
        },
    }
    roofline["scan_frac"] = roofline["per_kernel"][f"scan_{w['mode']}_kernel"]["frac"]

    # ---- end to end with the host in the loop ----
    e2e = None
    if do_e2e:
        copy_stream = torch.cuda.Stream()
        e2e_layers = layers[:mirror_layers]

        # ---- the correction shared with the GPU ----
        # The step is bounded by the workers' scattered reads of the cold mirror while the GPU and its
        # host link idle: the GPU computes the last rows of every layer's correction itself, reading the
        # selected mirror rows over the link (jf_gpu_topk_attn_rows), the workers the first ones.  The
        # share follows from the two rates, measured here on the first layers.
        n_rows = shard.b_count * shard.q_count
        plan = {"cut": n_rows, "calls": None}      # workers only, until the shared plan has proved faster
        share_info = {"share": 0.0}
        gpu_full_us = None
        side_stream = torch.cuda.Stream()
        want_share = args.gpu_correction_share
        if want_share != "0":
            try:
                t0 = time.perf_counter()
                for li, L in enumerate(e2e_layers):   # the mirrors become visible to the GPU (page-locked where they lie)
                    L.k_mirror_dev = ops.map_host_tensor(L.k_shadow)
                    L.v_mirror_dev = ops.map_host_tensor(L.v_shadow)
                    if li == 0 and (time.perf_counter() - t0) * len(e2e_layers) > 90.0:
                        ops.unmap_host_tensor(L.k_shadow)
                        ops.unmap_host_tensor(L.v_shadow)
                        raise RuntimeError(f"page-locking the mirrors would take {(time.perf_counter() - t0) * len(e2e_layers):.0f} s")
                share_info["map_s"] = round(time.perf_counter() - t0, 2)
                probe = e2e_layers[:min(4, len(e2e_layers))]
                for L in probe:             # slot lists for the probe
                    L.q.copy_(L.q_host)
                    L.call.fused()
                    L.slots_host.copy_(L.call.out["topk_slots_i32"])
                torch.cuda.synchronize()
                sample = max(1, n_rows // 8)
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                gpu_us = []
                for L in probe:             # the GPU's rate over the link: the last eighth of the rows, alone
                    ev0.record()
                    ops.gpu_topk_attn_rows(L.q, L.k_mirror_dev, L.v_mirror_dev, L.call.out["topk_slots_i32"], L.o_new,
                                           128 ** -0.5, (n_rows - sample, n_rows))
                    ev1.record()
                    torch.cuda.synchronize()
                    gpu_us.append(ev0.elapsed_time(ev1) * 1e3 * n_rows / sample)
                # the check of the GPU's rows against the workers' (rounding of the 16-bit result apart)
                Lc = probe[-1]
                Lc.host_call.run()
                ref_rows = Lc.o_new_host.view(n_rows, 128)[n_rows - sample:].float()
                got_rows = Lc.o_new.view(n_rows, 128)[n_rows - sample:].float().cpu()
                agree = bool(((got_rows - ref_rows).abs() <= 1e-3 + 2.0 ** -7 * ref_rows.abs()).all())
                share_info["rows_agree_with_host"] = agree
                if agree:
                    gpu_full_us = sorted(gpu_us)[len(gpu_us) // 2]
                    share_info["gpu_us_per_layer_alone"] = gpu_full_us
                    share_info["gpu_link_GBps"] = n_rows * w["top_k"] * 512 / gpu_full_us / 1e3
            except Exception as exc:        # the mirrors could not be page-locked, or the probe failed: workers only
                gpu_full_us, share_info = None, {"share": 0.0, "why": f"{type(exc).__name__}: {exc}"[:200]}

        def shared_plan(host_us):
            """Rows for the GPU from the two rates: the workers' per layer inside the pipelined loop and
            the GPU's alone; a little less than the balance point, since the two slow each other."""
            f = 0.9 * host_us / (host_us + gpu_full_us) if want_share == "auto" else float(want_share)
            cut = n_rows - int(round(min(max(f, 0.0), 0.5) * n_rows))      # at most a half: the workers always have rows
            if cut >= n_rows:
                return None
            for L in e2e_layers:
                L.gpu_event = torch.cuda.Event()
            return {"cut": cut, "calls": [ops.HostCorrectionCall(L.q_host, L.k_shadow, L.v_shadow, None, L.slots_host,
                                                                 L.o_new_host, 128 ** -0.5, rows=(0, cut)) for L in e2e_layers]}

        def merge_e2e(L):  # o_new host -> device, merge, result device -> host; on the copy stream
            cut = plan["cut"]
            with torch.cuda.stream(copy_stream):
                if cut < n_rows:            # the workers' rows come from the host, the GPU's are in place
                    copy_stream.wait_event(L.gpu_event)
                    L.o_new.view(n_rows, 128)[:cut].copy_(L.o_new_host.view(n_rows, 128)[:cut], non_blocking=True)
                else:
                    L.o_new.copy_(L.o_new_host, non_blocking=True)
                merge(ops, L)
                L.out_host.copy_(L.out, non_blocking=True)

        def e2e_step():
            main_s = torch.cuda.current_stream()
            cut, shared_calls = plan["cut"], plan["calls"]
            for L in e2e_layers:
                L.q.copy_(L.q_host, non_blocking=True)
                L.call.fused()
                L.slots_host.copy_(L.call.out["topk_slots_i32"], non_blocking=True)
                L.event.record(main_s)
                if cut < n_rows:            # the GPU's rows of this layer, beside the next layers' kernels
                    side_stream.wait_event(L.event)
                    with torch.cuda.stream(side_stream):
                        ops.gpu_topk_attn_rows(L.q, L.k_mirror_dev, L.v_mirror_dev, L.call.out["topk_slots_i32"], L.o_new,
                                               128 ** -0.5, (cut, n_rows))
                        L.gpu_event.record(side_stream)
            # The next layer's correction is queued before the previous one is waited for, so the
            # workers flow from one job into the next; merges are launched as jobs complete.
            prev = None
            for li, L in enumerate(e2e_layers):
                L.event.synchronize()
                ticket = shared_calls[li].submit() if shared_calls else L.host_call.submit()
                if prev is not None:
                    L.host_call.wait_ticket(prev[1])
                    merge_e2e(prev[0])
                prev = (L, ticket)
            prev[0].host_call.wait_ticket(prev[1])
            merge_e2e(prev[0])
            copy_stream.synchronize()
            if world > 1:
                gather_step()
                torch.cuda.current_stream().synchronize()

        def e2e_serial_step():
            """Layer l + 1 starts after layer l's merge, as in a real decoder."""
            for L in e2e_layers:
                L.q.copy_(L.q_host, non_blocking=True)
                L.call.fused()
                L.slots_host.copy_(L.call.out["topk_slots_i32"], non_blocking=True)
                torch.cuda.current_stream().synchronize()
                L.host_call.run()
                L.o_new.copy_(L.o_new_host, non_blocking=True)
                merge(ops, L)
            for L in e2e_layers:
                L.out_host.copy_(L.out, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            if world > 1:
                gather_step()
                torch.cuda.current_stream().synchronize()

        # The same serial chain with nothing waiting on the host inside a step: a kernel raises a word in
        # mapped memory when a layer's slots are on the host, a dispatcher thread queues the correction,
        # a kernel polls the word the last worker sets, and the merge reads o_new where the workers
        # wrote it (the adapter's stream-ordered decode step).  One core goes to the dispatcher.
        sig = []
        for L in e2e_layers:
            S = Layer()
            S.words_host, S.words_dev = ops.alloc_mapped_pinned_pair((16,), torch.int64)
            S.words_host.zero_()
            S.o_new_host, S.o_new = ops.alloc_mapped_pinned_pair((shard.b_count, shard.q_count, 128), dtype)
            S.o_new_host.zero_()
            S.host_call = ops.HostCorrectionCall(L.q_host, L.k_shadow, L.v_shadow, None, L.slots_host, S.o_new_host,
                                                 128 ** -0.5, done_flag=S.words_host[8:9])
            sig.append(S)
        watched = [False]

        def e2e_serial_stream_step():
            if not watched[0]:
                for S in sig:
                    S.host_call.watch(S.words_host[0:1])
                watched[0] = True
            for L, S in zip(e2e_layers, sig):
                L.q.copy_(L.q_host, non_blocking=True)
                L.call.fused()
                L.slots_host.copy_(L.call.out["topk_slots_i32"], non_blocking=True)
                ops.stream_signal_host(S.words_dev[8:9], S.words_dev[0:1])
                ops.stream_wait_host_flag(S.words_dev[8:9], 5000, L.call.status_record())
                res = L.call.out
                ops.blend_unnorm_into(res["o_hat"], res["o_old_unnorm"], res["W"], S.o_new, L.out)
            for L in e2e_layers:
                L.out_host.copy_(L.out, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            if world > 1:
                gather_step()
                torch.cuda.current_stream().synchronize()

        def timed(fn, n):
            for _ in range(2):
                fn()
            barrier()
            t0 = time.perf_counter()
            for _ in range(n):
                fn()
            barrier()
            dt = (time.perf_counter() - t0) / n
            tt = torch.tensor([dt], dtype=torch.float64, device=device)
            if world > 1:
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            return float(tt.item())

        e2e_steps = max(3, min(args.steps, 10))
        dt = timed(e2e_step, e2e_steps)            # the workers do every row
        # The shared plan is kept only if it is faster, measured the same way.  Under several ranks every
        # rank takes the second measurement if any rank has a plan (the timing is a collective).
        mine = shared_plan(dt / len(e2e_layers) * 1e6) if gpu_full_us is not None else None
        anyone = torch.tensor([1 if mine is not None else 0], dtype=torch.int32, device=device)
        if world > 1:
            dist.all_reduce(anyone, op=dist.ReduceOp.MAX)
        if int(anyone.item()):
            if mine is not None:
                plan.update(mine)
            dt_shared = timed(e2e_step, e2e_steps)
            rate = lambda t: job_layer_bytes * len(e2e_layers) / t / 1e9
            share_info.update({"workers_only_GBps": rate(dt), "shared_GBps": rate(dt_shared), "kept": dt_shared < dt})
            if mine is not None:
                share_info.update({"share": (n_rows - mine["cut"]) / n_rows, "rows_gpu": n_rows - mine["cut"],
                                   "rows_host": mine["cut"]})
            if dt_shared < dt:
                dt = dt_shared
            else:
                plan.update({"cut": n_rows, "calls": None})
                share_info["share"] = 0.0
        pipelined_out = e2e_layers[-1].out_host.clone()
        dt_serial_wait = timed(e2e_serial_step, max(2, e2e_steps // 2))
        check_out = e2e_layers[-1].out_host.clone()
        # the pipelined leg's output (some rows corrected by the GPU) against the workers-only chain
        d_out = (pipelined_out.float() - check_out.float()).abs()
        share_info["outputs_agree"] = bool((d_out <= 2e-3 + 2.0 ** -7 * check_out.float().abs()).all())
        share_info["outputs_max_abs_diff"] = float(d_out.max())
        ops.set_cpu_attn_threads(max(1, cpu_threads - 1))
        dt_serial_stream = timed(e2e_serial_stream_step, max(2, e2e_steps // 2))
        ops.set_cpu_attn_threads(cpu_threads)
        for S in sig:
            S.host_call.stream_status()
            S.host_call.close()
        serial_forms_agree = bool(torch.equal(check_out, e2e_layers[-1].out_host))
        dt_serial = min(dt_serial_wait, dt_serial_stream)
        # the host's share alone: the corrections of all measured layers back to back over the slot
        # lists the last step left on the host, nothing else running (each layer's mirror is cold)
        for L in e2e_layers[:2]:
            L.host_call.run()
        t0 = time.perf_counter()
        for L in e2e_layers:
            L.host_call.run()
        host_only_us = (time.perf_counter() - t0) / len(e2e_layers) * 1e6
        esz = 2
        n_e2e = len(e2e_layers)
        h2d = n_e2e * 2 * shard.b_count * shard.q_count * 128 * esz
        d2h = n_e2e * (shard.b_count * shard.q_count * w["top_k"] * 4 + shard.b_count * shard.q_count * 128 * esz)
        # dt covers n_e2e layers; ms_per_step and tokens/s are scaled to the workload's layer count
        dt_full, dts_full = dt * n_layers / n_e2e, dt_serial * n_layers / n_e2e
        e2e = {"value": job_layer_bytes * n_e2e / dt / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d * world,
               "d2h_bytes_per_step": d2h * world, "ms_per_step": dt_full * 1e3, "steps": e2e_steps,
               "layers_measured": n_e2e, "tokens_per_s": w["batch"] / dt_full, "host_threads_per_rank": cpu_threads,
               "us_per_layer": dt / n_e2e * 1e6, "host_correction_alone_us_per_layer": host_only_us,
               "gpu_correction": dict(share_info, mirror_bytes_read_by_gpu_per_step=(n_rows - plan["cut"]) * w["top_k"] * 512 * n_e2e * world,
                                      what="rows of the correction the GPU computes from the host mirror over the host link "
                                           "(jf_gpu_topk_attn_rows) while the workers do the others; pipelined leg only"),
               "serial_layers": {"value": job_layer_bytes * n_e2e / dt_serial / 1e9, "unit": "GB/s",
                                 "ms_per_step": dts_full * 1e3, "tokens_per_s": w["batch"] / dts_full,
                                 "what": "layer l + 1 starts after layer l's merge (host correction on the critical path)",
                                 "how": ("stream-ordered: correction started and joined by kernels through words in mapped memory"
                                         if dt_serial_stream <= dt_serial_wait else
                                         "host waits for the slots, runs the correction, queues the merge"),
                                 "host_wait_form": job_layer_bytes * n_e2e / dt_serial_wait / 1e9,
                                 "stream_ordered_form": job_layer_bytes * n_e2e / dt_serial_stream / 1e9,
                                 "forms_agree_bitwise": serial_forms_agree},
               "timing": "host wall clock around barrier + synchronize (host work is inside the region)"}
        if n_e2e < n_layers:
            e2e["note"] = (f"host memory: mirrors of {n_e2e} of {n_layers} layers; the copies above are per measured "
                           "step, ms_per_step and tokens_per_s are scaled to all layers")
        for L in layers:
            L.call.status()

    # ---- oracle replay of one timed row group; baselines (rank 0, single GPU) ----
    check = None
    if rank == 0 and not args.no_check:
        L = layers[min(1, n_layers - 1)]
        L.call.fused()
        torch.cuda.synchronize()
        check = oracle_check(torch, w, shard, L, seq_local=shard.b_count - 1, head_local=shard.kv_count - 1)
    cpu_baseline = ref_gpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        ref_gpu = run_reference_gpu_kernels(torch, w, layers[0], tables, dtype)
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
        cfg = config_dict(w, world, args.dtype)
        run = {
            "sharding": (f"{head_shards} KV-head shard(s) x {world // head_shards} batch shard(s): {shard.kv_count} KV heads, "
                         f"{shard.q_count} query heads, {shard.b_count} sequences per GPU; one NCCL all-gather of the per-head "
                         f"outputs per step into (B, H_q * 128)" + (", captured as a CUDA graph" if gather_in_graph else ""))
            if world > 1 else (f"single GPU running the shard of rank {as_shard} ({shard.kv_count} KV heads, {shard.q_count} "
                               f"query heads, {shard.b_count} sequences)" if as_shard else "single GPU"),
            "data_generator": "counter hash (Irwin-Hall of twelve 16-bit uniforms per element), identical on GPU and CPU",
            "host": {"cores": cores, "correction_workers": cpu_threads, "memory_nodes": numa_nodes,
                     "mirror_node": numa_node},
            "build_s": round(t_build, 1), "oracle_check": check, "gather_check": gather_check}
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": args.dtype,
            "data": "synthetic", "config": cfg, "run": run,
            "tokens_per_s": w["batch"] / (ms_step * 1e-3),
            "us_per_layer": us_layer,
            "gpu_launches": 3 * n_layers * args.steps * world,  # per layer and rank: scan, select+finish, merge
            "per_rank": per_rank,
            "roofline": roofline, "e2e": e2e, "cpu_baseline": cpu_baseline, "reference_gpu_kernels": ref_gpu,
            "other_configs_single_gpu": extra, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # graphs that captured a collective go before the communicator they refer to; a shutdown
        # that does not come back within 20 s ends the process instead of holding the GPUs
        ggraph = graph = None
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        watchdog = threading.Timer(20.0, lambda: os._exit(0))
        watchdog.daemon = True
        watchdog.start()
        dist.destroy_process_group()
        watchdog.cancel()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
