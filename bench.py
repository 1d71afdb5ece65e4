"""Benchmark of the MoE-layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c5] [--impl ours|reference]

One step = one MoE layer call (expert sort, gather, grouped fc1 + SwiGLU +
re-quantisation, grouped fc2 + scatter) over one batch of synthetic, seeded
inputs. Prints ONE JSON line: whole-job FP8 TFLOP/s (`value`), the same through
the drop-in `moe_test` call with host buffers (`e2e`), the roofline of the
dominant kernel (the fc1 grouped GEMM) and the CPU oracle timed on a bounded
sample (`cpu_baseline`).

With --gpus N > 1 (launched by torch.distributed.run) the layer runs
expert-parallel: every rank keeps T tokens (weak scaling) and E/N experts, rows
travel by all-to-all.
"""
from __future__ import annotations

import argparse
import json
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
}
# dram__bytes_read.sum + dram__bytes_write.sum of one fc1 launch, from the ncu capture summarised in
# profiles/c2_block_fp8_grouped_gemm.md (ncu cannot run inside a timed bench, so the figure is recorded here)
NCU_FC1_DRAM_BYTES = {"c2": 977.622272e6 + 119.235328e6}
MODE_NAME = {0: "bf16", 256: "fp8-tensor", 512: "fp8-channel", 1024: "fp8-block"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and clock-event reasons while the timed region runs.

    Reads only (NVML queries every 2 ms from a thread; the nvidia-smi command line every 100 ms as a
    fallback): nothing here changes a GPU setting. The timed regions last tens of milliseconds, far
    shorter than nvidia-smi's start-up, which is why NVML is polled in-process."""

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

    def stop(self):
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
            return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_min_mhz": min(mhz) if mhz else None,
                    "sm_max_mhz": self.max_mhz, "samples": len(mhz), "source": "nvml, 2 ms", "reasons": reasons}
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


def synth_inputs(wl, seed, device, T=None):
    """Seeded synthetic inputs of a workload on `device` (bf16 activations N(0,1), weights N(0,0.02))."""
    T = wl["T"] if T is None else T
    g = torch.Generator(device=device).manual_seed(seed)
    H, I, E, k = wl["H"], wl["I"], wl["E"], wl["k"]
    x = torch.randn(T, H, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device=device, dtype=torch.float32)
    if wl.get("desc", "").find("Zipf") >= 0:
        perm = torch.randperm(E, generator=g, device=device)
        bias = -1.1 * torch.log(torch.arange(1, E + 1, device=device, dtype=torch.float32))
        logits = logits + bias[perm]
    return x, logits


def synth_weights(wl, seed, device, experts=None):
    g = torch.Generator(device=device).manual_seed(seed + 1000)
    H, I = wl["H"], wl["I"]
    E = wl["E"] if experts is None else experts
    b = torch.empty(E, 2 * I, H, device=device, dtype=torch.bfloat16)
    b1 = torch.empty(E, H, I, device=device, dtype=torch.bfloat16)
    for e in range(E):  # per expert to bound the fp32 temporaries
        b[e] = (torch.randn(2 * I, H, generator=g, device=device) * 0.02).to(torch.bfloat16)
        b1[e] = (torch.randn(H, I, generator=g, device=device) * 0.02).to(torch.bfloat16)
    return b, b1


def quantize_gpu(ops, x, b, b1, mode):
    if mode == 1024:
        return (*ops.per_token_block_cast_to_fp8(x), *ops.per_block_cast_to_fp8(b), *ops.per_block_cast_to_fp8(b1))
    if mode == 512:
        aq, as_ = ops.per_token_cast_to_fp8(x)
        bq, bs = ops.per_channel_cast_to_fp8(b)
        b1q, b1s = ops.per_channel_cast_to_fp8(b1)
        return aq, as_.view(-1), bq, bs.view(b.shape[0], -1), b1q, b1s.view(b1.shape[0], -1)
    if mode == 256:
        return (*ops.per_tensor_cast_to_fp8(x), *ops.per_tensor_cast_to_fp8(b, per_expert=True),
                *ops.per_tensor_cast_to_fp8(b1, per_expert=True))
    return x, None, b, None, b1, None


def launches_per_step(n, mode):
    sort = 1 if n <= 2048 else 3
    return sort + 1 + 1 + (1 if mode in (256, 512) else 0) + 1


def config_of(name, wl, world):
    mode = wl["mode"]
    return {"workload": f"{name}: {wl['desc']}", "T_per_gpu": wl["T"], "H": wl["H"], "I": wl["I"], "E": wl["E"],
            "k": wl["k"], "quant": MODE_NAME[mode], "parallelism": f"ep{world}" if world > 1 else "single",
            "l2": "operands larger than L2 (weights %.2f GB); no flush" % (3.0 * wl["E"] * wl["H"] * wl["I"] * (1 if mode else 2) / 1e9)}


def cpu_baseline(wl, sample_tokens, seed=0, steps=1, warmup=0):
    """The oracle (torch on the host cores) on a bounded sample of the workload: `sample_tokens`
    tokens and, for workloads with many experts, the first 16 experts only (weights for all 256
    would take minutes to generate on the host). Inputs are prepared once, the layer call is timed."""
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
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        if mode:
            orc.moe_layer_fp8(*qs, idx, E, mode)
        else:
            orc.moe_layer_bf16(x, b, b1, idx, E)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
        if dt > 30 and times:  # keep the whole run within minutes
            break
    dt = statistics.mean(times)
    flops = 6.0 * T * k * H * I
    return dict(value=flops / dt / 1e12, unit="TFLOP/s", cores=torch.get_num_threads(), kind="port",
                sample=f"{T} of {wl['T']} tokens, {E} of {wl['E']} experts, {len(times)} layer call(s) of {dt:.2f} s",
                tokens_per_s=T / dt, steps=len(times))


def run_reference(args, wl, rank):
    """--impl reference: the reference's CPU implementation of the path (the oracle port of its torch code;
    the reference's CUDA path cannot be built here), all host threads, a bounded sample per step."""
    if rank != 0:
        return
    base = cpu_baseline(wl, 2048, steps=args.steps, warmup=min(args.warmup, 1))
    val = base["value"]
    out = {"impl": "reference", "metric": "moe_layer_fp8_tflops" if wl["mode"] else "moe_layer_bf16_tflops",
           "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
           "steps": base["steps"], "warmup": min(args.warmup, 1), "ms_per_step": None, "higher_is_better": True,
           "scaling": "weak", "vs_baseline": None, "dtype": "f32 (dequantised e4m3)", "data": "synthetic",
           "config": config_of(args.workload, wl, max(args.gpus, 1)),
           "cpu_baseline": base,
           "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(out))


def run_decode(args, rank):
    """--workload c5: decode-shape latency sweep (Mixtral shape, memory-bound). One JSON line with the
    p50 layer latency and the weight-streaming bandwidth for T in {1,16,64,256}, bf16 and per-tensor FP8."""
    if rank != 0:
        return
    from dqmoe_b200 import ops
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    H, I, E, k = 4096, 14336, 8, 2
    wl = dict(H=H, I=I, E=E, k=k)
    b, b1 = synth_weights(wl, 0, dev)
    bq, bs = ops.per_tensor_cast_to_fp8(b, per_expert=True)
    b1q, b1s = ops.per_tensor_cast_to_fp8(b1, per_expert=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # larger than the 126 MB L2
    pk = peaks()
    rows = []
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
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
            for i in range(max(args.warmup, 3) + args.steps):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                ops.moe_forward(*call, d, idx, ws, mode)
                e1.record()
                torch.cuda.synchronize()
                if i >= max(args.warmup, 3):
                    times.append(e0.elapsed_time(e1))
            p50 = statistics.median(times)
            # the same call replayed from a CUDA graph (what a decode loop does): launch gaps removed
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                ops.moe_forward(*call, d, idx, ws, mode)
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    ops.moe_forward(*call, d, idx, ws, mode)
            gtimes = []
            for i in range(args.steps + 3):
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
                         "bytes": nbytes, "gbs": nbytes / (p50 * 1e-3) / 1e9,
                         "frac_of_measured_hbm": nbytes / (p50 * 1e-3) / 1e9 / pk["hbm_gbs"]})
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
    for i in range(args.steps + 3):
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
    if not args.no_cpu_baseline:
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
    print(json.dumps({
        "metric": "moe_layer_decode_p50_latency_us", "value": head["p50_us"], "unit": "us", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": head["p50_us"] / 1e3,
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32", "data": "synthetic",
        "config": {"workload": "c5: decode-shape sweep, Mixtral shape, T in {1,16,64,256}; headline = fp8-tensor T=64",
                   "H": H, "I": I, "E": E, "k": k, "l2": "256 MB flush write before every timed call"},
        "clocks": clocks, "sweep": rows, "e2e": e2e, "cpu_baseline": base,
        "gpu_launches": launches_per_step(64 * k, 256) * args.steps,
        "roofline": {"bound": "hbm", "achieved": head["gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": head["gbs"] / pk["hbm_gbs"], "traffic": None,
                     "peak_note": f"of {pk['source']} copy bandwidth; nominal 8000 GB/s"}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + ["c5"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    if args.workload == "c5":
        if args.impl == "reference":
            args.workload = "c1"  # the CPU path is timed on the CPU-size layer for the decode sweep
        else:
            return run_decode(args, rank)
    wl = WORKLOADS[args.workload]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, wl, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: dqmoe_b200 has no CPU path "
                         "(use --impl reference for the CPU oracle)")
    from dqmoe_b200 import ops
    import moe_test

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        from dqmoe_b200 import ep
    T, H, I, E, k, mode = wl["T"], wl["H"], wl["I"], wl["E"], wl["k"], wl["mode"]
    n = T * k
    pk = peaks()

    # ---- inputs resident in HBM
    x, logits = synth_inputs(wl, 1234 + rank, dev)
    idx, weights = ops.route_topk(logits, k, wl["scoring"])
    if world == 1:
        b, b1 = synth_weights(wl, 0, dev)
        aq, as_, bq, bs, b1q, b1s = quantize_gpu(ops, x, b, b1, mode)
        del b, b1
        ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, mode), dtype=torch.uint8, device=dev)
        d = torch.empty(T, k, H, dtype=torch.bfloat16, device=dev)

        def step():
            ops.moe_forward(aq, as_, bq, bs, b1q, b1s, d, idx, ws, mode)
    else:
        layer = ep.ExpertParallelMoE(wl, dev, seed=0, ops=ops)
        # per rank and step: sort (1 or 3) + publish, plan, dispatch, wait, row_ptrs, fc1, [requant], fc2, signal, wait (peer exchange)
        sort_l = 1 if n <= 2048 else 3
        # collective exchange: sort, gather, segment ids, then the layer on the received rows, then scatter
        ep_launches = (sort_l + 9 + (1 if mode == 512 else 0)) * world if layer.impl == "peer" else \
            (sort_l + 2 + (3 + 3 + (1 if mode in (256, 512) else 0)) + 1) * world
        aq, as_ = layer.quantize_activations(x)

        def step():
            layer.forward(aq, as_, idx, None)  # d[T, k, H] like the single-GPU step
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed region: inputs in HBM
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if rank == 0 else None
    code = ops.device_status()
    if code != 0:
        raise SystemExit(f"device status {code}: a kernel's bounded wait gave up; no number reported")
    if world > 1:
        tmax = torch.tensor([ms_total], device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        ms_total = float(tmax.item())
    ms_step = ms_total / args.steps
    flops_step = 6.0 * T * k * H * I * world
    value = flops_step / (ms_step * 1e-3) / 1e12

    # ---- end to end through the drop-in call with host buffers (rank-local copies inside the timed region)
    # End to end through the public call with host buffers: every step copies its own inputs from pinned
    # host memory and reads its result back. Steps are double-buffered over three streams (copy-in,
    # compute, copy-out) as a serving loop would do, so a step's PCIe copies overlap other steps' compute.
    h_aq = aq.cpu().pin_memory()
    h_as = as_.cpu().pin_memory() if as_ is not None else None
    h_idx = idx.cpu().pin_memory()
    dummy = torch.ones(1, device=dev)
    comp, s_in, s_out = torch.cuda.current_stream(), torch.cuda.Stream(), torch.cuda.Stream()
    bufs = []
    for _ in range(2):
        bufs.append(dict(aq=torch.empty_like(aq), as_=torch.empty_like(as_) if as_ is not None else None,
                         idx=torch.empty_like(idx), d=torch.empty((T, k, H), dtype=torch.bfloat16, device=dev),
                         h_d=torch.empty((T, k, H), dtype=torch.bfloat16).pin_memory(),
                         ev_in=torch.cuda.Event(), ev_comp=torch.cuda.Event(), ev_out=torch.cuda.Event()))
    if world == 1:
        fn = moe_test.m_grouped_moe_nt_contiguous_fp8_bf16 if mode else moe_test.m_grouped_moe_nt_contiguous_bf16

        def e2e_forward(bf):
            fn((bf["aq"], bf["as_"] if mode else dummy), (bq, bs if mode else dummy), (b1q, b1s if mode else dummy),
               bf["d"], bf["idx"], ws, mode)
    else:
        def e2e_forward(bf):
            bf["d"].copy_(layer.forward(bf["aq"], bf["as_"], bf["idx"], None))  # out of the exchange buffer

    def e2e_step(i):
        bf = bufs[i % 2]
        with torch.cuda.stream(s_in):
            s_in.wait_event(bf["ev_comp"])  # the step that last read these input buffers is done
            bf["aq"].copy_(h_aq, non_blocking=True)
            if h_as is not None:
                bf["as_"].copy_(h_as, non_blocking=True)
            bf["idx"].copy_(h_idx, non_blocking=True)
            bf["ev_in"].record(s_in)
        comp.wait_event(bf["ev_in"])
        comp.wait_event(bf["ev_out"])       # the previous result in this output buffer has been read back
        e2e_forward(bf)
        bf["ev_comp"].record(comp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(bf["ev_comp"])
            bf["h_d"].copy_(bf["d"], non_blocking=True)
            bf["ev_out"].record(s_out)

    for i in range(4):
        e2e_step(i)
    comp.wait_stream(s_out)
    barrier()
    ev0.record()
    s_in.wait_event(ev0)
    for i in range(args.steps):
        e2e_step(i)
    comp.wait_stream(s_out)
    ev1.record()
    barrier()
    e2e_ms = ev0.elapsed_time(ev1) / args.steps
    if world > 1:
        tmax = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        e2e_ms = float(tmax.item())
    h2d = h_aq.numel() * h_aq.element_size() + (h_as.numel() * 4 if h_as is not None else 0) + h_idx.numel() * 4
    e2e = {"value": flops_step / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": T * k * H * 2 * world,
           "pipelining": "double-buffered: copy-in, compute and copy-out streams"}

    # ---- roofline of the dominant kernel: the fc1 grouped GEMM timed alone on this step's own operands
    roofline = None
    if world == 1:
        import ctypes
        from dqmoe_b200 import _lib
        lib = _lib.load()

        def wptr(which):
            return lib.dqmoe_moe_workspace_ptr(ctypes.c_void_p(ws.data_ptr()), which, T, H, I, E, k, mode)
        p_off, p_perm, p_perm_s, p_act, p_act_s, p_mt = wptr(0), wptr(2), wptr(3), wptr(4), wptr(5), wptr(7)
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        scratch_amax = torch.zeros(max(n, 1), dtype=torch.float32, device=dev)
        gated_out = torch.empty(n * I * 2, dtype=torch.uint8, device=dev)
        sa1 = as_.data_ptr() if mode == 256 else p_perm_s

        def fc1():
            _lib.check(lib.dqmoe_grouped_gemm(p_perm, sa1, bq.data_ptr(), bs.data_ptr() if bs is not None else None,
                                              p_off, p_mt, n, I, H, E, mode, 1, gated_out.data_ptr(), p_act_s,
                                              scratch_amax.data_ptr(), None, stream))
        for _ in range(3):
            fc1()
        torch.cuda.synchronize()
        ev0.record()
        for _ in range(args.steps):
            fc1()
        ev1.record()
        torch.cuda.synchronize()
        fc1_ms = ev0.elapsed_time(ev1) / args.steps
        fc1_flops = 2.0 * n * (2 * I) * H
        achieved = fc1_flops / (fc1_ms * 1e-3) / 1e12
        peak = pk["bf16"] * (2.0 if mode else 1.0)
        roofline = {"bound": "tensor", "kernel": "moe_GemmGrouped_GemmUniversal_tcgen05 (fc1, gated)",
                    "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "peak_note": ("2 x measured bf16 burst (no FP8 peak was measured); " if mode else "") +
                                 f"of {pk['source']}; nominal dense {'FP8 4500' if mode else 'BF16 2250'} TFLOP/s",
                    "ms_per_launch": fc1_ms, "traffic": None}
        roofline["traffic"] = NCU_FC1_DRAM_BYTES.get(args.workload)
    elif mode in (0, 1024) and layer.impl == "peer":
        # Expert parallel: the same kernel timed alone on rank 0's expert shard, with this rank's rows repeated k
        # times and split evenly over its experts (the received rows of a step have this size on average).
        e_loc = layer.wq[0].shape[0]
        rows = aq.repeat_interleave(k, dim=0)
        rows_s = as_.repeat_interleave(k, dim=0) if as_ is not None else None
        cuts = [(n * i) // e_loc for i in range(e_loc + 1)]
        offs = torch.tensor(cuts, dtype=torch.int32, device=dev)
        mt = ops.mtile_prefix(offs)
        out1 = torch.empty((n, I), dtype=torch.uint8 if mode else torch.bfloat16, device=dev)
        out1_s = torch.empty((n, (I + 127) // 128), dtype=torch.float32, device=dev)

        def fc1():
            ops.grouped_gemm(rows, rows_s, layer.wq[0], layer.wq[1], offs, mt, I, mode, True, out1, out_scale=out1_s)
        for _ in range(3):
            fc1()
        torch.cuda.synchronize()
        ev0.record()
        for _ in range(args.steps):
            fc1()
        ev1.record()
        torch.cuda.synchronize()
        fc1_ms = ev0.elapsed_time(ev1) / args.steps
        achieved = 2.0 * n * (2 * I) * H / (fc1_ms * 1e-3) / 1e12
        peak = pk["bf16"] * (2.0 if mode else 1.0)
        roofline = {"bound": "tensor", "kernel": "moe_GemmGrouped_GemmUniversal_tcgen05 (fc1, gated), rank 0's shard",
                    "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "peak_note": ("2 x measured bf16 burst (no FP8 peak was measured); " if mode else "") +
                                 f"of {pk['source']}; nominal dense {'FP8 4500' if mode else 'BF16 2250'} TFLOP/s",
                    "ms_per_launch": fc1_ms, "traffic": None}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    # the CPU baseline is timed at N=1 only (torchrun also pins the host threads to one per rank)
    base = None if args.no_cpu_baseline or world > 1 else cpu_baseline(wl, 2048)
    out = {
        "metric": "moe_layer_fp8_tflops" if mode else "moe_layer_bf16_tflops",
        "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "e4m3 x e4m3 -> f32" if mode else "bf16 x bf16 -> f32", "data": "synthetic",
        "tokens_per_s": T * world / (ms_step * 1e-3),
        "config": dict(config_of(args.workload, wl, world), **({"exchange": layer.impl} if world > 1 else {})),
        "gpu_launches": (launches_per_step(n, mode) if world == 1 else ep_launches) * args.steps,
        "clocks": clocks, "e2e": e2e, "roofline": roofline, "cpu_baseline": base,
    }
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
