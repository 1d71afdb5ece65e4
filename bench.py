"""Benchmark of the MoE-layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c5] [--impl ours|reference]

One step = one MoE layer call (expert sort, gather, grouped fc1 + SwiGLU + re-quantisation, grouped fc2 +
scatter) over one batch of synthetic, seeded inputs. Prints ONE JSON line: whole-job FP8 TFLOP/s (`value`), the
same through the drop-in `moe_test` call with host buffers (`e2e`), the roofline of the dominant kernel (the fc1
grouped GEMM), a parity figure for the very buffers that were timed, a sustained figure over at least a second
of back-to-back steps, and the CPU oracle timed on a bounded sample (`cpu_baseline`). The default workload (c2)
also carries short records of the other configurations (`c3`, `c4`, `c5`, `c2_mx`, `moe_block`).

With --gpus N > 1 (launched by torch.distributed.run) the layer runs expert-parallel: every rank keeps T tokens
(weak scaling) and E/N experts, rows travel through peer memory; the line then also has the per-phase times of
a call and, for c3, the strong-scaling case (T tokens in all).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "dqmoe_b200", "dropin")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

WORKLOADS = {
    # name: T, H, I, E, k, quant mode, scoring
    "c1": dict(T=64, H=1024, I=2048, E=8, k=2, mode=256, scoring="softmax",
               desc="CPU-size layer, per-tensor FP8"),
    "c2": dict(T=4096, H=4096, I=14336, E=8, k=2, mode=1024, scoring="softmax",
               desc="Mixtral-8x7B-shape prefill layer, 1x128/128x128 block FP8"),
    "c3": dict(T=8192, H=7168, I=2048, E=256, k=8, mode=1024, scoring="sigmoid",
               desc="DeepSeek-V3-shape routed-expert layer, block FP8"),
    "c4": dict(T=16384, H=2048, I=768, E=128, k=8, mode=512, scoring="softmax",
               desc="Qwen-MoE-shape channel-wise layer, Zipf(1.1) expert bias"),
    # the Mixtral shape of c2 in the added MXFP8 mode (1x32 UE8M0 scales on the block-scaled tensor-core instruction)
    "c2-mx": dict(T=4096, H=4096, I=14336, E=8, k=2, mode=2048, scoring="softmax",
                  desc="Mixtral-8x7B-shape prefill layer, MXFP8 (1x32 power-of-two scales)"),
    "c3-mx": dict(T=8192, H=7168, I=2048, E=256, k=8, mode=2048, scoring="sigmoid",
                  desc="DeepSeek-V3-shape routed-expert layer, MXFP8 (1x32 power-of-two scales)"),
}
# dram__bytes_read.sum + dram__bytes_write.sum of one fc1 launch divided by the launch's algorithmic bytes, from
# ncu captures of the same kernel (ncu cannot run inside a timed bench; the ratio scales the algorithmic bytes
# that are computed here for the workload at hand)
NCU_FC1_TRAFFIC_RATIO = {1024: 1.004, 512: 1.0, 256: 1.0, 0: 1.0, 2048: 1.0}
MODE_NAME = {0: "bf16", 256: "fp8-tensor", 512: "fp8-channel", 1024: "fp8-block", 2048: "mxfp8"}
COS_MIN, REL_MAX = 0.999, 2e-2  # layer tolerance against the oracle: cosine and max|x - ref| / max|ref|


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and clock-event reasons while a timed region runs.

    Reads only (NVML queries every 2 ms from a thread; the nvidia-smi command line every 100 ms as a
    fallback): nothing here changes a GPU setting."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []
        self.samples = []       # (sm MHz, reasons bit mask) from NVML
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if self.index < len(ids) and ids[self.index].isdigit():
                return int(ids[self.index])
        return self.index

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml

            def poll():
                while not self._stop.is_set():
                    try:
                        mhz = float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                        mask = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h))
                        self.samples.append((mhz, mask))
                    except pynvml.NVMLError:
                        pass
                    time.sleep(0.002)
            self._thread = threading.Thread(target=poll, daemon=True)
            self._thread.start()
            return
        except Exception:  # no NVML binding or no permission: fall back to the command line
            self._nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self, histogram: bool = False):
        if self._nvml is not None:
            self._stop.set()
            self._thread.join(timeout=2)
            nv = self._nvml
            bits = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown,
                    "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                    "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown,
                    "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
            mhz = [m for m, _ in self.samples]
            reasons = sorted(n for n, b in bits.items() if any(mask & b for _, mask in self.samples))
            try:
                nv.nvmlShutdown()
            except Exception:
                pass
            out = {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_min_mhz": min(mhz) if mhz else None,
                   "sm_max_mhz": self.max_mhz, "samples": len(mhz), "source": "nvml, 2 ms", "reasons": reasons}
            if histogram and mhz:
                hist = {}
                for m in mhz:
                    b = int(m // 100) * 100
                    hist[b] = hist.get(b, 0) + 1
                out["sm_mhz_histogram_100"] = {str(b): c for b, c in sorted(hist.items())}
            return out
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], [], set()
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(self.NAMES, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(mhz), "source": "nvidia-smi, 100 ms", "reasons": sorted(reasons)}


def bind_to_gpu_numa_node(local_rank: int):
    """Run this process on the CPUs of the NUMA node its GPU hangs off, so that the pinned host buffers
    allocated afterwards land in that node's memory (first touch). Read-only queries of sysfs and an affinity
    call on this process only; returns a short note for the JSON line (None when the topology is not visible)."""
    try:
        pr = torch.cuda.get_device_properties(local_rank)
        bus = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
    except Exception:
        return None
    try:
        dom_bus = bus.lower()
        if len(dom_bus.split(":")[0]) == 8:  # NVML prints an 8-digit domain, sysfs a 4-digit one
            dom_bus = dom_bus[4:]
        with open(f"/sys/bus/pci/devices/{dom_bus}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0) & cpus
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return f"numa node {node}, {len(allowed)} cpus"
    except Exception:
        return None


def synth_inputs(wl, seed, device, T=None):
    """Seeded synthetic inputs of a workload on `device` (bf16 activations N(0,1), router logits N(0,1))."""
    T = wl["T"] if T is None else T
    g = torch.Generator(device=device).manual_seed(seed)
    H, E = wl["H"], wl["E"]
    x = torch.randn(T, H, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device=device, dtype=torch.float32)
    if wl.get("desc", "").find("Zipf") >= 0:
        perm = torch.randperm(E, generator=g, device=device)
        bias = -1.1 * torch.log(torch.arange(1, E + 1, device=device, dtype=torch.float32))
        logits = logits + bias[perm]
    return x, logits


def synth_weights(wl, seed, device, experts=None):
    """bf16 weights N(0, 0.02) of the experts `experts` (default: all), one generator per global expert so
    that every rank of every world size builds the same model."""
    H, I = wl["H"], wl["I"]
    experts = list(range(wl["E"])) if experts is None else list(experts)
    b = torch.empty(len(experts), 2 * I, H, device=device, dtype=torch.bfloat16)
    b1 = torch.empty(len(experts), H, I, device=device, dtype=torch.bfloat16)
    for i, e in enumerate(experts):
        g = torch.Generator(device=device).manual_seed(seed * 100003 + e)
        b[i] = (torch.randn(2 * I, H, generator=g, device=device) * 0.02).to(torch.bfloat16)
        b1[i] = (torch.randn(H, I, generator=g, device=device) * 0.02).to(torch.bfloat16)
    return b, b1


def quantize_weights_gpu(ops, b, b1, mode):
    E = b.shape[0]
    if mode == 1024:
        return (*ops.per_block_cast_to_fp8(b), *ops.per_block_cast_to_fp8(b1))
    if mode == 512:
        bq, bs = ops.per_channel_cast_to_fp8(b)
        b1q, b1s = ops.per_channel_cast_to_fp8(b1)
        return bq, bs.view(E, -1), b1q, b1s.view(E, -1)
    if mode == 256:
        return (*ops.per_tensor_cast_to_fp8(b, per_expert=True), *ops.per_tensor_cast_to_fp8(b1, per_expert=True))
    if mode == 2048:
        return (*ops.mx_cast_weights_to_fp8(b), *ops.mx_cast_weights_to_fp8(b1))
    return b, None, b1, None


def build_model(ops, wl, seed, device, experts=None, chunk=16):
    """Quantised weights (fc1, fc1 scales, fc2, fc2 scales) of the given experts, built in chunks of experts to
    bound the bf16 temporaries."""
    experts = list(range(wl["E"])) if experts is None else list(experts)
    parts = []
    for i in range(0, len(experts), chunk):
        b, b1 = synth_weights(wl, seed, device, experts[i:i + chunk])
        parts.append(quantize_weights_gpu(ops, b, b1, wl["mode"]))
        del b, b1
    if len(parts) == 1:
        return parts[0]
    return tuple(None if parts[0][j] is None else torch.cat([p[j] for p in parts]) for j in range(4))


def quantize_activations_gpu(ops, x, mode):
    if mode == 1024:
        return ops.per_token_block_cast_to_fp8(x)
    if mode == 512:
        q, s = ops.per_token_cast_to_fp8(x)
        return q, s.view(-1)
    if mode == 256:
        return ops.per_tensor_cast_to_fp8(x)
    if mode == 2048:
        return ops.mx_cast_to_fp8(x)
    return x, None


def launches_per_step(n, mode):
    sort = 1 if n <= 2048 else 3
    # sort, gather, fc1, [re-quantisation pass | scale tiling of the MXFP8 mode], fc2
    return sort + 1 + 1 + (1 if mode in (256, 512, 2048) else 0) + 1


def config_of(name, wl, world, T=None):
    mode = wl["mode"]
    return {"workload": f"{name}: {wl['desc']}", "T_per_gpu": wl["T"] if T is None else T, "H": wl["H"], "I": wl["I"],
            "E": wl["E"], "k": wl["k"], "quant": MODE_NAME[mode], "parallelism": f"ep{world}" if world > 1 else "single",
            "l2": "operands larger than L2 (weights %.2f GB); no flush" % (3.0 * wl["E"] * wl["H"] * wl["I"] * (1 if mode else 2) / 1e9)}


def fc1_algorithmic_bytes(n, H, I, E, mode):
    """HBM bytes one fc1 launch has to move: every expert's weights once, the expert-sorted activations once,
    the intermediate (+ scales) once."""
    esz = 1 if mode else 2
    g = lambda v: (v + 127) // 128
    w = E * 2 * I * H * esz
    a = n * H * esz
    out = n * I * (1 if mode == 1024 else 2)
    scales = 0
    if mode == 1024:
        scales = n * g(H) * 4 + E * g(2 * I) * g(H) * 4 + n * g(I) * 4
    elif mode == 512:
        scales = n * 4 * 2 + E * 2 * I * 4
    elif mode == 2048:
        out = n * I
        scales = n * H // 32 + E * 2 * I * H // 32 + n * I // 32
    return w + a + out + scales


# --------------------------------------------------------------------------------------- CPU arm

def cpu_baseline(wl, sample_tokens, seed=0, steps=1, warmup=0, ops=None, device=None):
    """The oracle (torch on the host cores) on a bounded sample of the workload: `sample_tokens` tokens and, for
    workloads with many experts, the first 16 experts only (weights for all 256 would take minutes to generate on
    the host). Inputs are prepared once, the layer call is timed. With `ops` and `device` the same sample also
    runs through the CUDA layer and the two outputs are compared (returned as the second value)."""
    from oracle import moe_oracle as orc
    T = min(sample_tokens, wl["T"])
    H, I, k, mode = wl["H"], wl["I"], wl["k"], wl["mode"]
    E = min(wl["E"], 16)
    sub = dict(wl, E=E)
    x, logits = synth_inputs(sub, seed, "cpu", T=T)
    idx, _ = orc.route_topk(logits, k, wl["scoring"])
    b, b1 = synth_weights(sub, seed, "cpu")
    qs = orc.quantize_inputs(x, b, b1, mode) if mode else None
    times = []
    ref = None
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        if mode:
            ref = orc.moe_layer_fp8(*qs, idx, E, mode)
        else:
            ref = orc.moe_layer_bf16(x, b, b1, idx, E)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
        if dt > 30 and times:  # keep the whole run within minutes
            break
    dt = statistics.mean(times)
    flops = 6.0 * T * k * H * I
    base = dict(value=flops / dt / 1e12, unit="TFLOP/s", cores=torch.get_num_threads(), kind="port",
                sample=f"{T} of {wl['T']} tokens, {E} of {wl['E']} experts, {len(times)} layer call(s) of {dt:.2f} s",
                tokens_per_s=T / dt, steps=len(times))
    parity = None
    if ops is not None:
        dev_in = [t.to(device).contiguous() for t in qs] if mode else [x.to(device), None, b.to(device), None, b1.to(device), None]
        if mode == 2048:  # the layer takes the weights' scale bytes in the tiled layout
            dev_in[3], dev_in[5] = ops.mx_tile_scales(dev_in[3], H), ops.mx_tile_scales(dev_in[5], I)
        if mode == 512:
            dev_in[1], dev_in[3], dev_in[5] = dev_in[1].view(-1), dev_in[3].view(E, -1), dev_in[5].view(E, -1)
        ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, mode) + 256, dtype=torch.uint8, device=device)
        d = torch.zeros(T, k, H, dtype=torch.bfloat16, device=device)
        ops.moe_forward(*dev_in, d, idx.to(device), ws, mode)
        got = d.cpu()
        parity = {"against": "the CPU oracle on the cpu_baseline sample (same bytes in, CUDA layer vs oracle)",
                  "rows": T * k, "cosine": orc.cosine(got, ref), "max_rel_err": orc.max_rel_err(got, ref),
                  "tolerance": {"cosine_min": COS_MIN, "max_rel_err_max": REL_MAX}}
        parity["ok"] = bool(parity["cosine"] >= COS_MIN and parity["max_rel_err"] <= REL_MAX)
    return base, parity


def run_reference(args, wl, rank):
    """--impl reference: the reference's CPU implementation of the path (the oracle port of its torch code;
    the reference's CUDA path cannot be built here), all host cores, a bounded sample per step. Under torchrun
    the launcher sets one OpenMP thread per rank; this arm runs on rank 0 alone and takes every core back, so
    that its figure is the same at every N."""
    if rank != 0:
        return
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(max(cores, 1))
    base, _ = cpu_baseline(wl, 2048, steps=args.steps, warmup=min(args.warmup, 1))
    val = base["value"]
    out = {"impl": "reference", "metric": "moe_layer_fp8_tflops" if wl["mode"] else "moe_layer_bf16_tflops",
           "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
           "steps": base["steps"], "warmup": min(args.warmup, 1), "ms_per_step": None, "higher_is_better": True,
           "scaling": "weak", "vs_baseline": None, "dtype": "f32 (dequantised e4m3)", "data": "synthetic",
           "config": config_of(args.workload, wl, max(args.gpus, 1)),
           "cpu_baseline": base,
           "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(out))


# --------------------------------------------------------------------------------------- decode sweep (c5)

def decode_sweep(args, dev, ops, with_cpu=True):
    """Decode-shape latency sweep (Mixtral shape, memory-bound): p50 layer latency and weight-streaming bandwidth
    for T in {1,16,64,256}, bf16 and per-tensor FP8, an L2 flush before every timed call, CUDA-graph replay
    beside it. Returns the JSON record."""
    H, I, E, k = 4096, 14336, 8, 2
    wl = dict(H=H, I=I, E=E, k=k, mode=0)
    b, b1 = synth_weights(wl, 0, dev)
    bq, bs = ops.per_tensor_cast_to_fp8(b, per_expert=True)
    b1q, b1s = ops.per_tensor_cast_to_fp8(b1, per_expert=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # larger than the 126 MB L2
    pk = peaks()
    rows = []
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    steps, warm = args.steps, max(args.warmup, 3)
    for mode in (0, 256):
        for T in (1, 16, 64, 256):
            g = torch.Generator(device=dev).manual_seed(T)
            x = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
            idx, _ = ops.route_topk(torch.randn(T, E, generator=g, device=dev), k, "softmax")
            active = int(torch.unique(idx).numel())
            ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, mode), dtype=torch.uint8, device=dev)
            d = torch.empty(T, k, H, dtype=torch.bfloat16, device=dev)
            if mode:
                aq, as_ = ops.per_tensor_cast_to_fp8(x)
                call = (aq, as_, bq, bs, b1q, b1s)
            else:
                call = (x, None, b, None, b1, None)
            times = []
            for i in range(warm + steps):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                ops.moe_forward(*call, d, idx, ws, mode)
                e1.record()
                torch.cuda.synchronize()
                if i >= warm:
                    times.append(e0.elapsed_time(e1))
            p50 = statistics.median(times)
            # the same with L2 flushed by READING the buffer: the flush by writing leaves 126 MB of dirty lines whose
            # write-back shares HBM with the timed call's reads
            ctimes = []
            for i in range(steps + 3):
                flush.sum()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                ops.moe_forward(*call, d, idx, ws, mode)
                e1.record()
                torch.cuda.synchronize()
                if i >= 3:
                    ctimes.append(e0.elapsed_time(e1))
            p50c = statistics.median(ctimes)
            # the same call replayed from a CUDA graph (what a decode loop does): launch gaps removed
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                ops.moe_forward(*call, d, idx, ws, mode)
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    ops.moe_forward(*call, d, idx, ws, mode)
            gtimes = []
            for i in range(steps + 3):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                graph.replay()
                e1.record()
                torch.cuda.synchronize()
                if i >= 3:
                    gtimes.append(e0.elapsed_time(e1))
            p50g = statistics.median(gtimes)
            del graph
            # algorithmic bytes: weights of the experts hit + activations in and out
            nbytes = active * 3 * H * I * (1 if mode else 2) + T * H * (1 if mode else 2) + T * k * H * 2
            rows.append({"quant": MODE_NAME[mode], "T": T, "active_experts": active, "p50_us": p50 * 1e3,
                         "p50_us_cuda_graph": p50g * 1e3, "gbs_cuda_graph": nbytes / (p50g * 1e-3) / 1e9,
                         "p50_us_l2_flushed_by_read": p50c * 1e3,
                         "frac_of_measured_hbm_l2_flushed_by_read": nbytes / (p50c * 1e-3) / 1e9 / pk["hbm_gbs"],
                         "bytes": nbytes, "gbs": nbytes / (p50 * 1e-3) / 1e9,
                         "frac_of_measured_hbm": nbytes / (p50 * 1e-3) / 1e9 / pk["hbm_gbs"],
                         "frac_of_8000_gbs": nbytes / (p50 * 1e-3) / 1e9 / 8000.0})
    clocks = sampler.stop()
    if ops.device_status() != 0:
        raise SystemExit("device status non-zero: a kernel's bounded wait gave up; no number reported")
    head = next(r for r in rows if r["quant"] == "fp8-tensor" and r["T"] == 64)

    # the headline point end to end: quantised activations, scale and expert ids come from pinned host memory,
    # the [T, k, H] result goes back to pinned host memory, every call
    T = 64
    g = torch.Generator(device=dev).manual_seed(T)
    x = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    idx, _ = ops.route_topk(torch.randn(T, E, generator=g, device=dev), k, "softmax")
    aq, as_ = ops.per_tensor_cast_to_fp8(x)
    h_aq, h_as, h_idx = aq.cpu().pin_memory(), as_.cpu().pin_memory(), idx.cpu().pin_memory()
    d_aq, d_as, d_idx = torch.empty_like(aq), torch.empty_like(as_), torch.empty_like(idx)
    d = torch.empty(T, k, H, dtype=torch.bfloat16, device=dev)
    h_d = torch.empty(T, k, H, dtype=torch.bfloat16).pin_memory()
    ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, 256), dtype=torch.uint8, device=dev)
    etimes = []
    for i in range(steps + 3):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        d_aq.copy_(h_aq, non_blocking=True)
        d_as.copy_(h_as, non_blocking=True)
        d_idx.copy_(h_idx, non_blocking=True)
        ops.moe_forward(d_aq, d_as, bq, bs, b1q, b1s, d, d_idx, ws, 256)
        h_d.copy_(d, non_blocking=True)
        e1.record()
        torch.cuda.synchronize()
        if i >= 3:
            etimes.append(e0.elapsed_time(e1))
    e2e = {"value": statistics.median(etimes) * 1e3, "unit": "us",
           "h2d_bytes_per_step": h_aq.numel() + 4 * h_as.numel() + 4 * h_idx.numel(),
           "d2h_bytes_per_step": h_d.numel() * 2}

    base = None
    if with_cpu:
        # the oracle on the host cores for the smallest point of the sweep: one token, its two experts, bf16
        from oracle import moe_oracle as orc
        gc = torch.Generator().manual_seed(0)
        xb = torch.randn(1, H, generator=gc).to(torch.bfloat16)
        bb = (torch.randn(2, 2 * I, H, generator=gc) * 0.02).to(torch.bfloat16)
        bb1 = (torch.randn(2, H, I, generator=gc) * 0.02).to(torch.bfloat16)
        ids = torch.tensor([[0, 1]], dtype=torch.int32)
        ct = []
        for _ in range(3):
            t0 = time.perf_counter()
            orc.moe_layer_bf16(xb, bb, bb1, ids, 2)
            ct.append(time.perf_counter() - t0)
        base = {"value": statistics.median(ct) * 1e6, "unit": "us", "cores": torch.get_num_threads(), "kind": "port",
                "sample": "bf16 layer, T=1, its 2 active experts (the sweep's smallest point), median of 3 calls"}
    return {
        "metric": "moe_layer_decode_p50_latency_us", "value": head["p50_us"], "unit": "us", "n_gpus": 1,
        "steps": steps, "warmup": warm, "ms_per_step": head["p50_us"] / 1e3,
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32", "data": "synthetic",
        "config": {"workload": "c5: decode-shape sweep, Mixtral shape, T in {1,16,64,256}; headline = fp8-tensor T=64",
                   "H": H, "I": I, "E": E, "k": k, "l2": "256 MB flush write before every timed call"},
        "clocks": clocks, "sweep": rows, "e2e": e2e, "cpu_baseline": base,
        "gpu_launches": launches_per_step(64 * k, 256) * steps,
        "roofline": {"bound": "hbm", "achieved": head["gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": head["gbs"] / pk["hbm_gbs"], "traffic": None,
                     "peak_note": f"of {pk['source']} copy bandwidth; nominal 8000 GB/s"}}


# --------------------------------------------------------------------------------------- prefill workloads

class EPModel:
    """Synthetic model of one workload sharded by expert for the expert-parallel bench: this rank's quantised
    experts and the layer object that exchanges rows over peer memory (DQMOE_EP_IMPL=nccl: collectives)."""

    def __init__(self, wl, T, device, seed, ops, ep, dist, out_buffers=1):
        world, rank = dist.get_world_size(), dist.get_rank()
        self.ops, self.mode = ops, wl["mode"]
        lo, hi = ep.expert_range(rank, world, wl["E"])
        self.lo, self.hi = lo, hi
        self.wq = build_model(ops, wl, seed, device, range(lo, hi))
        use_peer = os.environ.get("DQMOE_EP_IMPL", "peer") == "peer" and world <= 8 and wl["mode"] in (0, 512, 1024, 2048)
        if use_peer:
            self.layer = ep.PeerExpertParallelLayer(T, wl["H"], wl["I"], wl["E"], wl["k"], wl["mode"], self.wq, ops,
                                                    out_buffers=out_buffers)
        else:
            self.layer = ep.ExpertParallelLayer(wl["E"], wl["k"], wl["mode"], self.wq, ep.CudaBackend(ops))
        self.impl = "peer" if use_peer else "nccl"

    def forward(self, aq, a_scale, idx, weights=None, **kw):
        return self.layer.forward(aq, a_scale, idx, weights, **kw)


def time_steps(step, steps, barrier, dist=None, dev=None):
    """EXACTLY `steps` calls between two events, a barrier + synchronize on both sides; max over ranks."""
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(steps):
        step()
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def sustained_run(step, steps, local_rank, barrier, flops_step, pk, mode, is_rank0, dist=None, dev=None):
    """Back-to-back blocks of `steps` calls for at least a second of GPU time (and at least 30 blocks), each
    block between its own event pair, clocks sampled throughout: the figure the kernel holds under the power
    cap, beside the burst figure of the contract's K-step region."""
    probe = time_steps(step, steps, barrier, dist, dev)
    blocks = int(min(400, max(30, math.ceil(1000.0 / max(probe, 1e-3)))))
    sampler = ClockSampler(local_rank)
    if is_rank0:
        sampler.start()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(blocks + 1)]
    barrier()
    evs[0].record()
    for b in range(blocks):
        for _ in range(steps):
            step()
        evs[b + 1].record()
    barrier()
    per_block = [evs[b].elapsed_time(evs[b + 1]) / steps for b in range(blocks)]
    clocks = sampler.stop(histogram=True) if is_rank0 else None
    if dist is not None:  # the slowest rank sets the pace of every block
        t = torch.tensor(per_block, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        per_block = t.tolist()
    per_block_sorted = sorted(per_block)
    med = statistics.median(per_block)
    q = lambda f: per_block_sorted[min(len(per_block_sorted) - 1, int(f * len(per_block_sorted)))]
    tail = per_block[len(per_block) // 2:]  # the second half: after the clocks have settled
    out = {"blocks": blocks, "steps_per_block": steps, "seconds": sum(per_block) * steps / 1e3,
           "ms_per_step_median": med, "ms_per_step_p10": q(0.1), "ms_per_step_p90": q(0.9),
           "ms_per_step_first_block": per_block[0], "ms_per_step_second_half_median": statistics.median(tail),
           "value": flops_step / (med * 1e-3) / 1e12, "unit": "TFLOP/s",
           "value_second_half": flops_step / (statistics.median(tail) * 1e-3) / 1e12,
           "clocks": clocks}
    if clocks and clocks.get("sm_mhz"):
        out["ms_x_mhz_median"] = med * clocks["sm_mhz"]
    peak = pk["bf16_sustained"] * (2.0 if mode else 1.0)
    world = dist.get_world_size() if dist is not None else 1
    out["frac_of_sustained_peak"] = out["value"] / world / peak
    out["sustained_peak_note"] = ("2 x " if mode else "") + f"{pk['source']} bf16 sustained ({pk['bf16_sustained']} TFLOP/s) per GPU"
    return out


def run_prefill(args, name, wl, ops, dev, rank, world, local_rank, dist=None, ep=None, T=None, headline=True,
                scaling="weak", keep_full_model=None):
    """One prefill workload at this world size: device-timed steps, parity of what was timed, the fc1 roofline,
    and for the headline also sustained, end-to-end and (N > 1) per-phase figures. Returns a dict (rank 0's is
    printed); raises SystemExit when parity or the device status fails."""
    import moe_test
    T = wl["T"] if T is None else T
    H, I, E, k, mode = wl["H"], wl["I"], wl["E"], wl["k"], wl["mode"]
    n = T * k
    pk = peaks()
    steps, warm = args.steps, max(args.warmup, 3)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- inputs resident in HBM
    x, logits = synth_inputs(wl, 1234 + rank, dev, T=T)
    idx, weights = ops.route_topk(logits, k, wl["scoring"])
    aq, as_ = quantize_activations_gpu(ops, x, mode)
    full = keep_full_model
    layer = None
    if world == 1:
        if full is None:
            full = build_model(ops, wl, 0, dev)
        bq, bs, b1q, b1s = full
        ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, mode), dtype=torch.uint8, device=dev)
        d = torch.empty(T, k, H, dtype=torch.bfloat16, device=dev)

        def step():
            ops.moe_forward(aq, as_, bq, bs, b1q, b1s, d, idx, ws, mode)
        per_step_launches = launches_per_step(n, mode)
    else:
        layer = EPModel(wl, T, dev, 0, ops, ep, dist, out_buffers=2 if headline else 1)
        sort_l = 1 if n <= 2048 else 3
        # peer exchange per rank and step: sort + publish/plan, dispatch, wait + row addresses, fc1, [requant | scale
        # tiling], fc2, signal/wait; collective exchange: sort, gather, segment ids, the layer on the received rows, scatter
        per_step_launches = (sort_l + 6 + (1 if mode in (512, 2048) else 0)) * world if layer.impl == "peer" else \
            (sort_l + 2 + (3 + 3 + (1 if mode in (256, 512) else 0)) + 1) * world

        def step():
            layer.forward(aq, as_, idx, None)  # d[T, k, H] like the single-GPU step
    torch.cuda.synchronize()
    for _ in range(warm):
        step()
    barrier()

    # ---- parity of the configuration that is about to be timed
    parity = None
    if world > 1:
        # every rank checks a sample of its own tokens against the single-GPU layer holding all experts
        # (any rank can rebuild any expert: weights are seeded per global expert)
        if full is None:
            full = build_model(ops, wl, 0, dev)
        S = min(T, 256)
        rows = torch.arange(0, T, max(T // S, 1), device=dev)[:S]
        got = layer.forward(aq, as_, idx, None)[rows].clone()
        ws1 = torch.empty(ops.moe_workspace_bytes(rows.numel(), H, I, E, k, mode) + 256, dtype=torch.uint8, device=dev)
        want = torch.zeros(rows.numel(), k, H, dtype=torch.bfloat16, device=dev)
        ops.moe_forward(aq[rows].contiguous(), None if as_ is None else as_[rows].contiguous(), full[0], full[1], full[2],
                        full[3], want, idx[rows].contiguous(), ws1, mode)
        torch.cuda.synchronize()
        gf, wf = got.double().flatten(), want.double().flatten()
        cos = float((gf @ wf) / (gf.norm() * wf.norm()).clamp(min=1e-300))
        rel = float((gf - wf).abs().max() / wf.abs().max().clamp(min=1e-300))
        stats = torch.tensor([1.0 if torch.equal(got, want) else 0.0, cos, -rel], device=dev, dtype=torch.float64)
        dist.all_reduce(stats, op=dist.ReduceOp.MIN)
        parity = {"against": "the single-GPU layer holding all experts, on a sample of every rank's own tokens",
                  "rows": int(rows.numel() * k * world), "bit_equal": bool(stats[0].item() == 1.0),
                  "cosine": float(stats[1].item()), "max_rel_err": float(-stats[2].item()), "ranks": world}
        parity["ok"] = bool(parity["bit_equal"] or (parity["cosine"] >= 0.99999 and parity["max_rel_err"] <= 1e-3))
        del ws1, want, got
        if keep_full_model is None and not (rank == 0 and scaling == "strong"):
            full = None
        torch.cuda.empty_cache()
        if not parity["ok"]:
            raise SystemExit(f"parity check failed at {world} GPUs for {name}: {parity}; no number reported")

    # ---- device-timed region: inputs in HBM, EXACTLY `steps` steps
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_total = time_steps(step, steps, barrier, dist if world > 1 else None, dev)
    clocks = sampler.stop() if rank == 0 else None
    code = ops.device_status()
    if code != 0:
        raise SystemExit(f"device status {code}: a kernel's bounded wait gave up; no number reported")
    ms_step = ms_total / steps
    flops_step = 6.0 * T * k * H * I * world
    value = flops_step / (ms_step * 1e-3) / 1e12
    rec = {
        "metric": "moe_layer_fp8_tflops" if mode else "moe_layer_bf16_tflops",
        "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps, "warmup": warm,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
        "dtype": "e4m3 x e4m3 -> f32" if mode else "bf16 x bf16 -> f32", "data": "synthetic",
        "tokens_per_s": T * world / (ms_step * 1e-3),
        "config": dict(config_of(name, wl, world, T), **({"exchange": layer.impl} if world > 1 else {})),
        "gpu_launches": per_step_launches * steps, "clocks": clocks, "parity": parity,
    }

    # ---- roofline of the dominant kernel: the fc1 grouped GEMM timed alone
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fc1 = None
    if world == 1:
        import ctypes
        from dqmoe_b200 import _lib
        lib = _lib.load()

        def wptr(which):
            return lib.dqmoe_moe_workspace_ptr(ctypes.c_void_p(ws.data_ptr()), which, T, H, I, E, k, mode)
        p_off, p_perm, p_perm_s, p_act_s, p_mt = wptr(0), wptr(2), wptr(3), wptr(5), wptr(7)
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        scratch_amax = torch.zeros(max(n, 1), dtype=torch.float32, device=dev)
        gated_out = torch.empty(n * I * 2, dtype=torch.uint8, device=dev)
        sa1 = as_.data_ptr() if mode == 256 else p_perm_s

        def fc1_mx():
            _lib.check(lib.dqmoe_grouped_gemm_mx(p_perm, p_perm_s, bq.data_ptr(), bs.data_ptr(), p_off, p_mt, n, I, H, E, 1,
                                                 gated_out.data_ptr(), p_act_s, None, stream))

        def fc1():  # on the step's own expert-sorted (ragged) rows, as left in the workspace by the last step
            if mode == 2048:
                return fc1_mx()
            _lib.check(lib.dqmoe_grouped_gemm(p_perm, sa1, bq.data_ptr(), bs.data_ptr() if bs is not None else None,
                                              p_off, p_mt, n, I, H, E, mode, 1, gated_out.data_ptr(), p_act_s,
                                              scratch_amax.data_ptr(), None, stream))
        fc1_n, fc1_e, fc1_what = n, E, "the step's own expert-sorted rows"
    elif mode in (0, 1024, 2048) and layer.impl == "peer":
        # Expert parallel: the same kernel alone on this rank's expert shard, with this rank's rows repeated k
        # times and split evenly over its experts (the received rows of a step have this size on average).
        e_loc = layer.wq[0].shape[0]
        rows_ = aq.repeat_interleave(k, dim=0)
        rows_s = as_.repeat_interleave(k, dim=0) if as_ is not None else None
        cuts = [(n * i) // e_loc for i in range(e_loc + 1)]
        offs = torch.tensor(cuts, dtype=torch.int32, device=dev)
        mt = ops.mtile_prefix(offs)
        out1 = torch.empty((n, I), dtype=torch.uint8 if mode else torch.bfloat16, device=dev)
        out1_s = torch.empty((n, (I + 127) // 128), dtype=torch.float32, device=dev)

        if mode == 2048:
            rows_s = ops.mx_tile_scales(rows_s, H, offsets=offs, mtile_pref=mt)
            out1_t = torch.empty(rows_s.numel() // H * I + 512, dtype=torch.uint8, device=dev)

        def fc1():
            if mode == 2048:
                return ops.grouped_gemm_mx(rows_, rows_s, layer.wq[0], layer.wq[1], offs, mt, I, True, out1, out1_t)
            ops.grouped_gemm(rows_, rows_s, layer.wq[0], layer.wq[1], offs, mt, I, mode, True, out1, out_scale=out1_s)
        fc1_n, fc1_e, fc1_what = n, e_loc, "rank 0's expert shard, its rows split evenly"
    if fc1 is not None:
        for _ in range(3):
            fc1()
        torch.cuda.synchronize()
        ev0.record()
        for _ in range(steps):
            fc1()
        ev1.record()
        torch.cuda.synchronize()
        fc1_ms = ev0.elapsed_time(ev1) / steps
        achieved = 2.0 * fc1_n * (2 * I) * H / (fc1_ms * 1e-3) / 1e12
        peak = pk["bf16"] * (2.0 if mode else 1.0)
        algo = fc1_algorithmic_bytes(fc1_n, H, I, fc1_e, mode)
        rec["roofline"] = {
            "bound": "tensor", "kernel": f"moe_GemmGrouped_GemmUniversal_tcgen05 (fc1, gated) on {fc1_what}",
            "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
            "frac_of_nominal": achieved / (4500.0 if mode else 2250.0),
            "peak_note": ("2 x measured bf16 burst (no FP8 peak was measured); " if mode else "") +
                         f"of {pk['source']}; nominal dense {'FP8 4500' if mode else 'BF16 2250'} TFLOP/s",
            "ms_per_launch": fc1_ms, "algorithmic_bytes": algo,
            "traffic": algo * NCU_FC1_TRAFFIC_RATIO[mode],
            "traffic_note": "algorithmic bytes of this launch x the dram-bytes / algorithmic-bytes ratio of the ncu capture "
                            "of the same kernel"}
    else:
        rec["roofline"] = None

    if not headline:
        del layer
        torch.cuda.empty_cache()
        return rec, full

    # ---- sustained: at least a second of back-to-back steps
    rec["sustained"] = sustained_run(step, steps, local_rank, barrier, flops_step, pk, mode, rank == 0,
                                     dist if world > 1 else None, dev)

    # ---- per-phase times of an expert-parallel call
    if world > 1 and layer.impl == "peer":
        acc, calls = {}, 10
        barrier()
        for _ in range(calls):
            tl = []
            layer.forward(aq, as_, idx, None, timeline=tl)
            torch.cuda.synchronize()
            for (_, e_a), (nm, e_b) in zip(tl[:-1], tl[1:]):
                acc[nm] = acc.get(nm, 0.0) + e_a.elapsed_time(e_b) / calls
        names = list(acc)
        t = torch.tensor([acc[nm] for nm in names], device=dev)
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        # rows that leave this GPU: all kept rows minus those routed to its own experts
        own = int(((idx >= layer.lo) & (idx < layer.hi)).sum().item())
        kept = int(((idx >= 0) & (idx < E)).sum().item())
        scale_cols = (H + 127) // 128 if mode == 1024 else (1 if mode == 512 else 0)
        rec["phases"] = {
            "ms_rank0": {nm: float(v) for nm, v in zip(names, t.tolist())},
            "ms_max_over_ranks": {nm: float(v) for nm, v in zip(names, tmax.tolist())},
            "note": "CUDA events between the launches of one call, mean of 10 calls; a wait phase includes the skew between ranks",
            "nvlink_bytes_out_rank0": {"dispatch": (kept - own) * (H * (1 if mode else 2) + scale_cols * 4 + 4),
                                       "combine (fc2 epilogue stores)": (kept - own) * H * 2}}

    # ---- end to end through the public call with host buffers (rank-local copies inside the timed region):
    # every step copies its own inputs from pinned host memory and reads its result back. Steps are
    # double-buffered over three streams (copy-in, compute, copy-out) as a serving loop would do, so a step's
    # PCIe copies overlap other steps' compute.
    numa = bind_to_gpu_numa_node(local_rank)
    h_aq = aq.cpu().pin_memory()
    h_as = as_.cpu().pin_memory() if as_ is not None else None
    h_idx = idx.cpu().pin_memory()
    h_w = weights.cpu().pin_memory()
    dummy = torch.ones(1, device=dev)
    comp, s_in, s_out = torch.cuda.current_stream(), torch.cuda.Stream(), torch.cuda.Stream()
    bufs = []
    for _ in range(2):
        bufs.append(dict(aq=torch.empty_like(aq), as_=torch.empty_like(as_) if as_ is not None else None,
                         idx=torch.empty_like(idx), w=torch.empty_like(weights),
                         d=torch.empty((T, k, H), dtype=torch.bfloat16, device=dev) if world == 1 else None,
                         h_d=torch.empty((T, k, H), dtype=torch.bfloat16).pin_memory(),
                         h_o=torch.empty((T, H), dtype=torch.bfloat16).pin_memory(),
                         ev_in=torch.cuda.Event(), ev_comp=torch.cuda.Event(), ev_out=torch.cuda.Event()))
    if world == 1:
        fn = moe_test.m_grouped_moe_nt_contiguous_fp8_bf16 if mode else moe_test.m_grouped_moe_nt_contiguous_bf16

        def e2e_forward(bf):
            fn((bf["aq"], bf["as_"] if mode else dummy), (bq, bs if mode else dummy), (b1q, b1s if mode else dummy),
               bf["d"], bf["idx"], ws, mode)
            return bf["d"]
    else:
        def e2e_forward(bf):  # the result stays in the exchange buffer (two alternate), copied out from there
            return layer.forward(bf["aq"], bf["as_"], bf["idx"], None)

    def make_e2e_step(weighted):
        def e2e_step(i):
            bf = bufs[i % 2]
            with torch.cuda.stream(s_in):
                s_in.wait_event(bf["ev_comp"])  # the step that last read these input buffers is done
                bf["aq"].copy_(h_aq, non_blocking=True)
                if h_as is not None:
                    bf["as_"].copy_(h_as, non_blocking=True)
                bf["idx"].copy_(h_idx, non_blocking=True)
                if weighted:
                    bf["w"].copy_(h_w, non_blocking=True)
                bf["ev_in"].record(s_in)
            comp.wait_event(bf["ev_in"])
            comp.wait_event(bf["ev_out"])       # the previous result in this output buffer has been read back
            out = e2e_forward(bf)
            if weighted:
                out = ops.finalize_weighted(out, bf["w"])
            bf["ev_comp"].record(comp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(bf["ev_comp"])
                (bf["h_o"] if weighted else bf["h_d"]).copy_(out, non_blocking=True)
                out.record_stream(s_out)
                bf["ev_out"].record(s_out)
        return e2e_step

    def time_e2e(e2e_step):
        for i in range(4):
            e2e_step(i)
        comp.wait_stream(s_out)
        barrier()
        ev0.record()
        s_in.wait_event(ev0)
        for i in range(steps):
            e2e_step(i)
        comp.wait_stream(s_out)
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1) / steps
        if world > 1:
            tmax = torch.tensor([ms], device=dev)
            dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
            ms = float(tmax.item())
        return ms

    e2e_ms = time_e2e(make_e2e_step(False))
    e2e_w_ms = time_e2e(make_e2e_step(True))
    h2d = h_aq.numel() * h_aq.element_size() + (h_as.numel() * 4 if h_as is not None else 0) + h_idx.numel() * 4
    rec["e2e"] = {"value": flops_step / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                  "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": T * k * H * 2 * world,
                  "pipelining": "double-buffered: copy-in, compute and copy-out streams", "host_numa_binding": numa}
    rec["e2e_weighted_output"] = {
        "value": flops_step / (e2e_w_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_w_ms,
        "h2d_bytes_per_step": (h2d + h_w.numel() * 4) * world, "d2h_bytes_per_step": T * H * 2 * world,
        "note": "the k slots are combined with the router weights on the device (dqmoe_finalize_weighted) and "
                "[T, H] goes back to the host instead of the reference contract's [T, k, H]"}
    if world > 1:
        # the same copies with no compute in between: what the host side of this box can move per rank while
        # every rank copies at once
        def copy_only(i):
            bf = bufs[i % 2]
            with torch.cuda.stream(s_in):
                bf["aq"].copy_(h_aq, non_blocking=True)
                if h_as is not None:
                    bf["as_"].copy_(h_as, non_blocking=True)
                bf["idx"].copy_(h_idx, non_blocking=True)
            with torch.cuda.stream(s_out):
                bf["h_d"].copy_(layer.layer.d_outs[i % 2], non_blocking=True)
        if layer.impl == "peer":
            for i in range(2):
                copy_only(i)
            barrier()
            ev0.record()
            s_in.wait_event(ev0)
            s_out.wait_event(ev0)
            for i in range(steps):
                copy_only(i)
            comp.wait_stream(s_in)
            comp.wait_stream(s_out)
            ev1.record()
            barrier()
            cms = ev0.elapsed_time(ev1) / steps
            tmax = torch.tensor([cms], device=dev)
            dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
            cms = float(tmax.item())
            rec["e2e"]["copy_only_ms_per_step"] = cms
            rec["e2e"]["copy_only_gbs_per_gpu"] = (h2d + T * k * H * 2) / (cms * 1e-3) / 1e9
    code = ops.device_status()
    if code != 0:
        raise SystemExit(f"device status {code}: a kernel's bounded wait gave up; no number reported")
    return rec, full


def time_moe_block(args, name, wl, ops, dev, full):
    """dqmoe_moe_block: router -> gather fused with the 1x128 activation quantisation -> layer -> weighted combine,
    from bf16 activations and fp32 logits to [T, H]."""
    T, H, I, E, k, mode = wl["T"], wl["H"], wl["I"], wl["E"], wl["k"], wl["mode"]
    x, logits = synth_inputs(wl, 1234, dev)
    ws = torch.empty(_block_ws(ops, T, H, I, E, k, mode), dtype=torch.uint8, device=dev)

    def call():
        return ops.moe_block(x, logits, full[0], full[1], full[2], full[3], k, wl["scoring"], mode, workspace=ws)
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        call()
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / args.steps
    return {"workload": name, "ms_per_call": ms, "value": 6.0 * T * k * H * I / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "tokens_per_s": T / (ms * 1e-3),
            "what": "router + quantise-in-gather + fc1 + fc2 + weighted combine, bf16 [T,H] and fp32 logits in, bf16 [T,H] out"}


def _block_ws(ops, T, H, I, E, k, mode):
    from dqmoe_b200 import _lib
    return max(int(_lib.load().dqmoe_moe_block_workspace_bytes(T, H, I, E, k, mode)), 256)


def run_nvfp4(args, ops, dev, name="c2"):
    """The added NVFP4 mode on a prefill shape, single GPU: layer time with inputs resident in HBM, the fc1 grouped
    GEMM timed alone on the step's own expert-sorted rows, and parity of a sample of tokens against the CPU oracle
    (same packed bytes in). Fractions are of 4 x the measured bf16 peak (no FP4 peak was measured; nominal dense
    FP4 is 9 000 TFLOP/s)."""
    from dqmoe_b200 import _lib
    wl = dict(WORKLOADS[name])
    T, H, I, E, k = wl["T"], wl["H"], wl["I"], wl["E"], wl["k"]
    x, logits = synth_inputs(wl, 1, dev)
    idx, _ = ops.route_topk(logits, k, wl["scoring"])
    parts = []
    for i in range(0, E, 16):
        b, b1 = synth_weights(wl, 0, dev, range(i, min(E, i + 16)))
        parts.append((*ops.nvfp4_cast_weights(b), *ops.nvfp4_cast_weights(b1), b.shape[0]))
        del b, b1
    bq, b1q = torch.cat([p_[0] for p_ in parts]), torch.cat([p_[3] for p_ in parts])
    bg, b1g = torch.cat([p_[2] for p_ in parts]), torch.cat([p_[5] for p_ in parts])
    bs, b1s = torch.cat([p_[1] for p_ in parts]), torch.cat([p_[4] for p_ in parts])  # whole 128-row blocks per expert
    del parts
    a_g = ops.nvfp4_global_scale(x)
    aq, a_sf = ops.nvfp4_cast(x, a_g)
    # the global scale of the intermediate is a calibration constant of the layer: here amax 64, above what
    # silu(gate) * value reaches on these inputs
    act_g = torch.tensor([64.0 / (448.0 * 6.0)], dtype=torch.float32, device=dev)
    ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, 4096), dtype=torch.uint8, device=dev)
    d = torch.empty(T, k, H, dtype=torch.bfloat16, device=dev)
    call = (aq, a_sf, a_g, bq, bs, bg, b1q, b1s, b1g, act_g)
    step = lambda: ops.moe_forward_nvfp4(*call, d, idx, ws)
    barrier = torch.cuda.synchronize
    sampler = ClockSampler(dev.index or 0)
    for _ in range(max(args.warmup, 3)):
        step()
    sampler.start()
    ms = time_steps(step, args.steps, barrier) / args.steps
    clocks = sampler.stop()
    if ops.device_status() != 0:
        raise SystemExit("device status non-zero: a kernel's bounded wait gave up; no number reported")
    flops = 6.0 * T * k * H * I
    pk = peaks()
    peak = 4.0 * pk["bf16"]
    # fc1 alone on the step's own sorted rows (the workspace still holds them)
    lib = _lib.load()
    n = T * k
    wp = lambda which: lib.dqmoe_moe_workspace_ptr(ws.data_ptr(), which, T, H, I, E, k, 4096)
    stream = torch.cuda.current_stream().cuda_stream
    def fc1():
        _lib.check(lib.dqmoe_grouped_gemm_nvfp4(wp(2), wp(3), a_g.data_ptr(), bq.data_ptr(), bs.data_ptr(), bg.data_ptr(), wp(0),
                                                wp(7), n, I, H, E, 1, wp(4), wp(5), act_g.data_ptr(), None, stream))
    for _ in range(3):
        fc1()
    ms1 = time_steps(fc1, args.steps, barrier) / args.steps
    step()  # leave the workspace as a layer call leaves it
    fl1 = 4.0 * n * I * H
    # parity on a sample of tokens: the oracle on the same packed bytes
    par = None
    if not args.no_cpu_baseline:
        from oracle import moe_oracle as orc
        sample = 64
        c = lambda t: t.cpu()
        untile = lambda tiled, rows, cols: tiled.cpu().numpy().reshape(-1, rows // 128, cols // 64, 32, 4, 4).transpose(
            0, 1, 4, 3, 2, 5).reshape(-1, rows, cols // 16)
        bs_rm = torch.from_numpy(untile(bs, 2 * I, H).copy())
        b1s_rm = torch.from_numpy(untile(b1s, H, I).copy())
        ref = orc.moe_layer_nvfp4(c(aq[:sample]), c(a_sf[:sample]), c(a_g), c(bq), bs_rm, c(bg), c(b1q), b1s_rm, c(b1g), c(act_g),
                                  c(idx[:sample]), E)
        ds = torch.empty(sample, k, H, dtype=torch.bfloat16, device=dev)
        wss = torch.empty(ops.moe_workspace_bytes(sample, H, I, E, k, 4096), dtype=torch.uint8, device=dev)
        ops.moe_forward_nvfp4(aq[:sample].contiguous(), a_sf[:sample].contiguous(), a_g, bq, bs, bg, b1q, b1s, b1g, act_g, ds,
                              idx[:sample].contiguous(), wss)
        torch.cuda.synchronize()
        par = {"against": "cpu oracle (same packed bytes in)", "tokens": sample, "cosine": orc.cosine(ds.cpu(), ref),
               "max_rel_err": orc.max_rel_err(ds.cpu(), ref)}
        par["ok"] = par["cosine"] >= 0.999 and par["max_rel_err"] <= 2e-2
        if not par["ok"]:
            raise SystemExit(f"parity of the NVFP4 layer against the CPU oracle failed: {par}; no number reported")
    return {"metric": "moe_layer_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "e2m1 x e2m1 -> f32 (ue4m3 scales per 16)",
            "data": "synthetic", "parity": par, "clocks": clocks, "gpu_launches": args.steps * (launches_per_step(n, 2048)),
            "roofline": {"bound": "tensor", "kernel": "fc1 grouped GEMM (gated, NVFP4 re-quantisation)", "achieved": fl1 / (ms1 * 1e-3) / 1e12,
                         "peak": peak, "unit": "TFLOP/s", "frac": fl1 / (ms1 * 1e-3) / 1e12 / peak,
                         "peak_note": "4 x measured bf16 burst (no FP4 peak measured; nominal dense FP4 9 000)",
                         "ms_per_launch": ms1, "traffic": None},
            "config": {"workload": f"{name} shape in the added NVFP4 mode", "T_per_gpu": T, "H": H, "I": I, "E": E, "k": k,
                       "quant": "nvfp4", "parallelism": "single", "l2": "operands larger than L2; no flush"}}


def short(rec, keys=("value", "unit", "ms_per_step", "tokens_per_s", "scaling", "parity", "roofline", "config", "n_gpus")):
    return {k_: rec.get(k_) for k_ in keys}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + ["c5", "c2-nvfp4", "c3-nvfp4"],
                    help="c2 (default, the headline), c3, c4, c5 (decode sweep), c1 (CPU-size), c2-mx / c3-mx (added MXFP8 mode)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="headline workload only: no c3/c4/c5/moe_block records")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        # the CPU path is timed on the CPU-size layer for the decode sweep, and on the fp32-scaled shape for the NVFP4 records
        name = "c1" if args.workload == "c5" else args.workload.replace("-nvfp4", "")
        args.workload = name
        run_reference(args, WORKLOADS[name], rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: dqmoe_b200 has no CPU path "
                         "(use --impl reference for the CPU oracle)")
    from dqmoe_b200 import ops

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if args.workload == "c5":
        if rank == 0:
            print(json.dumps(decode_sweep(args, dev, ops, with_cpu=not args.no_cpu_baseline)))
        return
    if args.workload.endswith("-nvfp4"):  # single-GPU record of the added NVFP4 mode
        if rank == 0:
            print(json.dumps(run_nvfp4(args, ops, dev, args.workload.split("-")[0])))
        return
    dist = ep = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        from dqmoe_b200 import ep
    wl = WORKLOADS[args.workload]
    rec, full = run_prefill(args, args.workload, wl, ops, dev, rank, world, local_rank, dist, ep)

    extras = args.workload == "c2" and not args.no_extras

    def settle():
        """The extra records are burst measurements like the headline (20 calls, tens of ms): let the board leave the
        power-capped state the headline's one-second sustained loop put it in before each of them starts."""
        torch.cuda.synchronize()
        time.sleep(2.0)

    if extras:
        rec["extras_note"] = "every extra record starts after a 2 s pause (burst conditions, as for the headline value)"
    if extras and world == 1:
        rec["moe_block"] = [time_moe_block(args, "c2", wl, ops, dev, full)]
    del full
    torch.cuda.empty_cache()
    if extras:
        c3 = WORKLOADS["c3"]
        if world == 1:
            settle()
            r3, full3 = run_prefill(args, "c3", c3, ops, dev, rank, world, local_rank, headline=False)
            rec["c3"] = short(r3)
            rec["moe_block"].append(time_moe_block(args, "c3", c3, ops, dev, full3))
            del full3
            torch.cuda.empty_cache()
            settle()
            r4, full4 = run_prefill(args, "c4", WORKLOADS["c4"], ops, dev, rank, world, local_rank, headline=False)
            rec["c4"] = short(r4)
            del full4
            torch.cuda.empty_cache()
            # the headline shape in the added MXFP8 mode (scales applied inside the tensor-core instruction)
            settle()
            rmx, fullmx = run_prefill(args, "c2-mx", WORKLOADS["c2-mx"], ops, dev, rank, world, local_rank, headline=False)
            rec["c2_mx"] = short(rmx)
            del fullmx
            torch.cuda.empty_cache()
            settle()
            rec["c2_nvfp4"] = short(run_nvfp4(args, ops, dev))
            torch.cuda.empty_cache()
            settle()
            r5 = decode_sweep(args, dev, ops, with_cpu=False)
            rec["c5"] = {k_: r5[k_] for k_ in ("metric", "value", "unit", "sweep", "roofline", "e2e", "config")}
        else:
            # weak: T tokens per GPU (what the headline does for c2); strong: T tokens in all, the configuration as
            # stated (256 / W experts per GPU); rank 0 also times the whole problem alone for the strong efficiency
            r3w, _ = run_prefill(args, "c3", c3, ops, dev, rank, world, local_rank, dist, ep, headline=False)
            r3s, full3 = run_prefill(args, "c3", c3, ops, dev, rank, world, local_rank, dist, ep, T=c3["T"] // world,
                                     headline=False, scaling="strong")
            strong = short(r3s)
            if rank == 0:
                r1, _ = run_prefill(args, "c3", c3, ops, dev, 0, 1, local_rank, headline=False, keep_full_model=full3)
                strong["single_gpu_ms_per_step_same_run"] = r1["ms_per_step"]
                strong["efficiency"] = r1["ms_per_step"] / (world * r3s["ms_per_step"])
                strong["efficiency_note"] = "t(1 GPU, whole problem, rank 0 in this run) / (W x t(W GPUs))"
            del full3
            torch.cuda.empty_cache()
            dist.barrier()
            rec["c3"] = {"weak": short(r3w), "strong": strong}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    # the CPU baseline (and, with it, the oracle parity of the CUDA layer on the same sample) at N=1 only
    base = par = None
    if not args.no_cpu_baseline and world == 1:
        base, par = cpu_baseline(wl, 2048, ops=ops, device=dev)
        if par is not None and not par["ok"]:
            raise SystemExit(f"parity against the CPU oracle failed: {par}; no number reported")
        rec["parity"] = par
    rec["cpu_baseline"] = base
    print(json.dumps(rec))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
