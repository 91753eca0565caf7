"""Benchmark of the quantized linear-layer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (BASELINE.json configs[1]): NVFP4 batched decode, 8 lanes, one 27B-style dense layer with
hidden 5120 -- q 5120->6144, k and v 5120->1024, o 6144->5120, gate and up 5120->17408,
down 17408->5120 -- repeated over 64 layers of distinct synthetic weights (12.27 GB, far larger than
L2, so no timed iteration finds its weights cached). A step is one pass over all layers. The
metric is the weight-stream rate: algorithmic bytes (codes + scales + divisors + activations in
and out) per second, whole job.

At N > 1 (launched under torch.distributed.run) every matrix is sharded column-wise over N and each
rank streams its own rows: strong scaling, no collective in the timed region (outputs stay
sharded). Rank 0 prints one JSON line.

`--impl reference` times the reference's CPU implementation of the same path (its host
dequantizer compiled in place when available, else the oracle port, plus the fp64 product) on
the host cores, each step a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# (name, n, k, input): the seven matrices of one layer and which activation buffer each reads
LAYER = [("q", 6144, 5120, "h"), ("k", 1024, 5120, "h"), ("v", 1024, 5120, "h"), ("o", 5120, 6144, "a"),
         ("gate", 17408, 5120, "h"), ("up", 17408, 5120, "h"), ("down", 5120, 17408, "m")]
INPUT_WIDTH = {"h": 5120, "a": 6144, "m": 17408}
GROUPS = [["q", "k", "v"], ["o"], ["gate", "up"], ["down"]]  # calls that share one activation read
METRIC = "nvfp4_gemv_hbm_gbs"
UNIT = "GB/s"


def weight_bytes(n: int, k: int) -> int:
    return n * k // 2 + n * k // 16 + 4


def layer_algorithmic_bytes(tokens: int, world: int = 1) -> int:
    """Bytes one rank must move for one layer: its shard of every payload, each activation read
    once per call that uses it, each output written once."""
    total = 0
    for _, n, k, _ in LAYER:
        total += weight_bytes(n // world, k) + tokens * k * 2 + tokens * (n // world) * 2
    return total


def measured_peak() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int) -> None:
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:  # NVML missing: the bench still runs, clocks are reported as unknown
            self._nvml = None

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                self.samples.append(self._nvml.nvmlDeviceGetClockInfo(self._handle, self._nvml.NVML_CLOCK_SM))
                mask = self._nvml.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ---- the CPU arm --------------------------------------------------------------------------------

def cpu_sample(seconds_target: float = 12.0):
    """Times the reference's CPU path on a bounded sample: rows of the q matrix (K = 5120) at
    8 tokens -- dequantize to the logical FP32 weight, then the threaded fp64 product -- and
    returns (GB/s of algorithmic bytes, description dict)."""
    import numpy as np
    import torch

    from ignis_b200 import nvfp4
    from oracle.oracle import Oracle, default_threads

    orc = Oracle()
    kind, dequant = "port", orc.nvfp4_dequant
    try:
        from oracle.oracle import Reference

        dequant = Reference().nvfp4_dequant
        kind = "reference"
    except (FileNotFoundError, OSError):
        pass
    threads = default_threads()
    k, tokens = 5120, 8
    rng = np.random.default_rng(20261126)
    x = torch.randn(tokens, k, generator=torch.Generator().manual_seed(20261126)).to(torch.bfloat16).float().numpy()

    def run(rows: int) -> float:
        codes = rng.integers(0, 256, (rows, k // 2)).astype(np.uint8)
        natural = torch.from_numpy((np.abs(rng.standard_normal((rows, k // 16))) + 0.1).astype(np.float32))
        scales = nvfp4.swizzle_scales(natural.to(torch.float8_e4m3fn).view(torch.uint8).numpy())
        t0 = time.perf_counter()
        w = dequant(codes, scales, rows, k, 448.0)
        orc.gemm_f64(w, x, threads)
        return time.perf_counter() - t0

    probe_rows = 256
    t = run(probe_rows)
    rows = int(min(6144, max(256, seconds_target / max(t, 1e-6) * probe_rows))) // 128 * 128
    # whole q-sized pieces (fresh random rows each) until about `seconds_target` of CPU work is done
    elapsed, pieces = 0.0, 0
    while pieces == 0 or (elapsed < seconds_target and pieces < 64):
        elapsed += run(rows)
        pieces += 1
    nbytes = pieces * (weight_bytes(rows, k) + tokens * k * 2 + tokens * rows * 2)
    desc = {"kind": kind, "cores": threads,
            "sample": f"{pieces} x {rows} rows of q (K=5120) at 8 tokens: host dequantize ({kind}, 1 thread) + fp64 product "
                      f"({threads} threads), {elapsed:.2f} s"}
    return nbytes / elapsed / 1e9, desc


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    values = []
    desc = {}
    for _ in range(args.warmup):
        cpu_sample(2.0)
    t0 = time.perf_counter()
    for _ in range(max(1, args.steps)):
        v, desc = cpu_sample(6.0)
        values.append(v)
    total = time.perf_counter() - t0
    value = sum(values) / len(values)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total / max(1, args.steps) * 1e3, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": "configs[1]: NVFP4 decode, 8 lanes, 27B-style dense layer (CPU: a bounded row sample per step)"},
            "cpu_baseline": {"value": value, "unit": UNIT, **desc},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ---- the CUDA arm -------------------------------------------------------------------------------

def build_workload(layers: int, rank: int, world: int, tokens: int, device):
    import torch

    from ignis_b200 import nvfp4

    gen = torch.Generator(device=device)
    weights = []
    for layer in range(layers):
        entry = {}
        for idx, (name, n, k, _) in enumerate(LAYER):
            rows = n // world
            gen.manual_seed(20261126 + (layer * 16 + idx) * 64 + rank)
            codes = torch.randint(0, 256, (rows, k // 2), dtype=torch.uint8, device=device, generator=gen)
            natural = (torch.randn((rows, k // 16), device=device, generator=gen).abs() + 0.1).to(torch.float8_e4m3fn)
            natural = natural.view(torch.uint8)
            stored = natural.reshape(rows // 128, 4, 32, k // 64, 4).permute(0, 3, 2, 1, 4).contiguous().reshape(-1)
            entry[name] = nvfp4.Weight(codes, stored, rows, k, 448.0, 448.0)
        weights.append(entry)
    cpu_gen = torch.Generator().manual_seed(20261126)
    host_inputs = {key: torch.randn(tokens, width, generator=cpu_gen).to(torch.bfloat16).pin_memory()
                   for key, width in INPUT_WIDTH.items()}
    inputs = {key: t.to(device) for key, t in host_inputs.items()}
    outputs = {name: torch.empty(tokens, n // world, dtype=torch.bfloat16, device=device) for name, n, _, _ in LAYER}
    return weights, host_inputs, inputs, outputs


TRELLIS_LAYER = [("q", 5120, 6144), ("k", 5120, 1024), ("v", 5120, 1024), ("o", 6144, 5120), ("gate", 5120, 17408),
                 ("up", 5120, 17408), ("down", 17408, 5120)]  # (name, in, out), configs[3]


def build_trellis_workload(layers: int, rank: int, world: int, tokens: int, device):
    """configs[3]: the layer's seven shapes at 3 bits per weight (k2 = 6), random words (every bit
    pattern is a valid encoding), suh / svh = +-(0.5..2) x {0.05, 0.03}."""
    import torch

    from ignis_b200 import trellis

    gen = torch.Generator(device=device)
    weights = []
    total = 0
    for layer in range(layers):
        entry = {}
        for idx, (name, in_, out) in enumerate(TRELLIS_LAYER):
            cols = out // world
            gen.manual_seed(20261127 + (layer * 16 + idx) * 64 + rank)
            words = torch.randint(-32768, 32767, ((in_ // 16) * (cols // 16) * 48,), dtype=torch.int16, device=device,
                                  generator=gen)
            suh = ((torch.rand(in_, device=device, generator=gen) * 1.5 + 0.5) * 0.05).to(torch.float16)
            svh = ((torch.rand(cols, device=device, generator=gen) * 1.5 + 0.5) * 0.03).to(torch.float16)
            entry[name] = trellis.Weight(words, suh, svh, 6, in_, cols)
            if layer == 0:
                total += trellis.weight_bytes(in_, cols, 6) + tokens * in_ * 2 + tokens * cols * 2
        weights.append(entry)
    cpu_gen = torch.Generator().manual_seed(20261127)
    inputs = {w: torch.randn(tokens, w, generator=cpu_gen).to(torch.bfloat16).to(device) for w in (5120, 6144, 17408)}
    outputs = {name: torch.empty(tokens, out // world, dtype=torch.bfloat16, device=device) for name, _, out in TRELLIS_LAYER}
    return weights, inputs, outputs, total * layers


def build_moe_workload(tokens: int, device, rank=0, world=1, hidden=2048, inter=768, experts=512, top_k=10, k2=5):
    """configs[4]: 512 experts of (hidden 2048, intermediate 768) at 2.5 bits per weight, every record
    distinct (random words: every bit pattern is a valid encoding), Zipf(1.1) expert popularity over a
    seeded permutation, 10 distinct experts per token drawn in proportion to popularity, routing
    weights = BF16(softmax of 10 normal logits). The shared expert is the FP8 row-scale one."""
    import numpy as np
    import torch

    from ignis_b200 import moe

    local_experts = experts // world
    moe.set_geometry(hidden, inter, local_experts, top_k)
    moe.prepare()
    gen = torch.Generator(device=device).manual_seed(20261129 + rank)
    gu_bytes, dn_bytes = moe.record_bytes(moe.PROJ_GATE_UP, k2), moe.record_bytes(moe.PROJ_DOWN, k2)
    buffer = torch.empty(local_experts * (gu_bytes + dn_bytes), dtype=torch.uint8, device=device)
    offsets, k2s, assign = [], [], []

    def fill(at: int, in_: int, out: int, amp_in: float, amp_out: float) -> None:
        words = in_ * out * k2 // 16
        buffer[at: at + words] = torch.randint(0, 256, (words,), dtype=torch.uint8, device=device, generator=gen)
        for base, n, amp in ((at + words, in_, amp_in), (at + words + 2 * in_, out, amp_out)):
            v = (torch.rand(n, device=device, generator=gen) * 1.5 + 0.5) * amp
            v = v * (torch.randint(0, 2, (n,), device=device, generator=gen) * 2 - 1)
            buffer[base: base + 2 * n] = v.to(torch.float16).view(torch.uint8)

    at = 0
    for e in range(local_experts):
        fill(at, hidden, 2 * inter, 0.05, 0.03)
        offsets.append(at); k2s.append(k2); at += gu_bytes
        fill(at, inter, hidden, 0.25, 0.06)
        offsets.append(at); k2s.append(k2); at += dn_bytes
        assign.append((2 * e, 2 * e + 1))
    table = moe.SlotTable.from_device_records(buffer, offsets, k2s, assign)

    cpu = torch.Generator().manual_seed(20261129)
    perm = torch.randperm(experts, generator=cpu)
    popularity = torch.empty(experts)
    popularity[perm] = 1.0 / torch.arange(1, experts + 1, dtype=torch.float32) ** 1.1
    ids = torch.multinomial(popularity.expand(tokens, experts), top_k, replacement=False, generator=cpu).to(torch.int32)
    weights = torch.softmax(torch.randn(tokens, top_k, generator=cpu), dim=1).to(torch.bfloat16).float()
    x = (torch.randn(tokens, hidden, generator=cpu) * 0.5).to(torch.bfloat16)
    shared = [torch.from_numpy(moe.fp8_row_scale_payload(torch.randn(r, c, generator=cpu) * 0.02)).to(device)
              for r, c in ((inter, hidden), (inter, hidden), (hidden, inter))]
    w_gate = (torch.randn(hidden, generator=cpu) * 0.02).to(torch.bfloat16).to(device)
    hit = int(torch.unique(ids).numel())
    flops = tokens * top_k * (2.0 * hidden * 2 * inter + 2.0 * inter * hidden) + tokens * (2.0 * hidden * 2 * inter + 2.0 * inter * hidden)
    if world == 1:
        ws = moe.Workspace(min(8, tokens), tokens, device)
    else:   # a rank may be sent every token of the job
        ws = moe.Workspace(8, tokens, device)
        lo, hi = rank * tokens // world, (rank + 1) * tokens // world
        ids, weights, x = ids[lo:hi], weights[lo:hi], x[lo:hi]
    host = {"x": x.pin_memory(), "ids": ids.pin_memory(), "weights": weights.pin_memory()}
    return {"table": table, "ids": ids.to(device), "weights": weights.to(device), "x": x.to(device), "shared": shared,
            "w_gate": w_gate, "ws": ws, "flops": flops, "weight_bytes": hit * (gu_bytes + dn_bytes), "hit": hit,
            "host": host, "experts": experts}


def run_moe_workload(args) -> None:
    """`--workload moe` (configs[4]): routed experts + shared expert + combine, TFLOP/s. One GPU: the
    step is one CUDA graph. N GPUs: expert-parallel, tokens split over the ranks, one all-to-all
    each way per step (NCCL), timed on the device, max over ranks."""
    import torch
    import torch.distributed as dist

    from ignis_b200 import moe, moe_ep

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    tokens = args.moe_tokens
    m = build_moe_workload(tokens, device, rank, world)
    out_host = torch.empty((m["x"].shape[0], 2048), dtype=torch.bfloat16).pin_memory()
    stream = torch.cuda.Stream()

    side = torch.cuda.Stream()   # the shared expert needs no exchange: it runs beside it

    def one_step():
        if world == 1:
            moe.experts_prefill(m["x"], m["ids"], m["weights"], m["table"], m["ws"])
            shared, _ = moe.shared_expert(m["shared"][0], m["shared"][1], m["shared"][2], m["x"])
            return moe.combine(m["ws"], shared, m["x"], m["w_gate"])
        main = torch.cuda.current_stream()
        side.wait_stream(main)
        with torch.cuda.stream(side):
            shared, _ = moe.shared_expert(m["shared"][0], m["shared"][1], m["shared"][2], m["x"])
        acc = moe_ep.routed_experts(m["x"], m["ids"], m["weights"], m["experts"],
                                    lambda rows, local, w: moe.experts_tokens(rows, local, w, m["table"], m["ws"]))
        main.wait_stream(side)
        shared.record_stream(main)
        return moe.combine(m["ws"], shared, m["x"], m["w_gate"], acc=acc)

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(stream):
        out = one_step()
        stream.synchronize()
        step = one_step
        graphed = bool(args.graph) and world == 1   # the exchange sizes its buffers on the host
        if graphed:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                out = one_step()
            step = graph.replay
        for _ in range(args.warmup):
            step()
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as clocks:
            start.record(stream)
            for _ in range(args.steps):
                step()
            stop.record(stream)
            barrier()
        device_ms = start.elapsed_time(stop)
        # end to end: the step's tokens and routing from pinned host memory in, its output back
        e2e_start, e2e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2e_start.record(stream)
        for _ in range(args.steps):
            for key in ("x", "ids", "weights"):
                m[key].copy_(m["host"][key], non_blocking=True)
            got = step()
            out_host.copy_(out if graphed else got, non_blocking=True)
        e2e_stop.record(stream)
        barrier()
        e2e_ms = e2e_start.elapsed_time(e2e_stop)

    status = m["ws"].status()
    times = torch.tensor([device_ms, e2e_ms, float(status)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.destroy_process_group()
    device_ms, e2e_ms, status = times.tolist()
    if rank != 0:
        return
    ms = device_ms / args.steps
    value = m["flops"] / 1e12 / (ms * 1e-3)
    peak = 1403.2 * world
    h2d = sum(t.numel() * t.element_size() for t in m["host"].values())
    print(json.dumps({
        "metric": "moe_expert_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16xf16->f32", "data": "synthetic",
        "config": {"workload": f"configs[4]: MoE routed experts + shared expert + combine, {tokens} tokens x top-10 of 512 experts, "
                               f"hidden 2048, intermediate 768, 2.5 bpw trellis records, Zipf(1.1) routing; {m['hit']} experts hit, "
                               f"{m['weight_bytes'] / 1e6:.0f} MB of expert records",
                   "cuda_graph": graphed, "l2": "inputs larger than L2",
                   "parallelism": "one GPU" if world == 1 else f"expert-parallel over {world} ranks, tokens split, NCCL all-to-all each way"},
        "e2e": {"value": m["flops"] / 1e12 / (e2e_ms / args.steps * 1e-3), "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": out_host.numel() * 2},
        "gpu_launches": 8 * args.steps, "clocks": clocks.summary(),
        "roofline": {"bound": "tensor", "achieved": value, "peak": peak, "unit": "TFLOP/s", "frac": value / peak,
                     "peak_source": "measured sustained BF16 cuBLAS rate per GPU (the experts multiply in FP16 with FP32 accumulation)",
                     "kernel": "moe_experts_kernel", "traffic": None, "device_status": int(status),
                     "record_gbs": m["weight_bytes"] / (ms * 1e-3) / 1e9}}))


def run_side_workload(args) -> None:
    """The other measured configs, one JSON line each, same timing rules as the headline:
    `--workload prefill` (configs[2], W4A4 tensor-core GEMM, TFLOP/s) and `--workload trellis`
    (configs[3], 3-bit trellis decode, GB/s). One GPU."""
    import torch

    from ignis_b200 import nvfp4, trellis

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    nvfp4.prepare()
    trellis.prepare()
    stream = torch.cuda.Stream()
    peak_hbm, peak_kind = measured_peak()
    with torch.cuda.stream(stream):
        if args.workload == "prefill":
            tokens = args.tokens if args.tokens > 8 else 8192
            shapes = [("up", 17408, 5120), ("down", 5120, 17408)]
            gen = torch.Generator(device=device)
            ws_bytes = max(nvfp4.workspace_bytes(n, k, nvfp4.ALLOW_A4, tokens) for _, n, k in shapes)
            ws = nvfp4.Workspace(ws_bytes, device)
            items = []
            for idx, (name, n, k) in enumerate(shapes):
                gen.manual_seed(20261128 + idx)
                codes = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=device, generator=gen)
                natural = (torch.randn((n, k // 16), device=device, generator=gen).abs() + 0.1).to(torch.float8_e4m3fn).view(torch.uint8)
                stored = natural.reshape(n // 128, 4, 32, k // 64, 4).permute(0, 3, 2, 1, 4).contiguous().reshape(-1)
                w = nvfp4.Weight(codes, stored, n, k, 448.0, 448.0)
                x = torch.randn(tokens, k, device=device, generator=gen).to(torch.bfloat16)
                y = torch.empty(tokens, n, dtype=torch.bfloat16, device=device)
                items.append((w, x, y))
            flops = sum(2.0 * tokens * w.n * w.k for w, _, _ in items)

            def one_step() -> None:
                for w, x, y in items:
                    if args.a16:
                        nvfp4.linear(x, w, out=y)   # A16: BF16 activations as they are, weights decoded into the MMA
                    else:
                        nvfp4.linear(x, w, out=y, policy=nvfp4.ALLOW_A4, workspace=ws)

            launches = (1 if args.a16 else 2) * len(items)
            if args.mlp:
                # the layers' MLP through one entry: gate|up with the SwiGLU + re-quantizing epilogue, then down
                gen.manual_seed(20261130)
                n_gu, k_gu = 2 * 17408, 5120
                codes = torch.randint(0, 256, (n_gu, k_gu // 2), dtype=torch.uint8, device=device, generator=gen)
                natural = (torch.randn((n_gu, k_gu // 16), device=device, generator=gen).abs() + 0.1).to(torch.float8_e4m3fn).view(torch.uint8)
                stored = natural.reshape(n_gu // 128, 4, 32, k_gu // 64, 4).permute(0, 3, 2, 1, 4).contiguous().reshape(-1)
                gate_up = nvfp4.Weight(codes, stored, n_gu, k_gu, 448.0, 448.0)
                down_w, _, y_down = items[1]
                x_in = items[0][1]
                mlp_ws = nvfp4.Workspace(nvfp4.mlp_workspace_bytes(n_gu, k_gu, nvfp4.ALLOW_A4, tokens), device)
                flops = 2.0 * tokens * (n_gu * k_gu + down_w.n * down_w.k)

                def one_step() -> None:
                    nvfp4.mlp(x_in, gate_up, down_w, mlp_ws, out=y_down, policy=nvfp4.ALLOW_A4)

                ws = mlp_ws
                launches = 3
            metric, unit, work = "nvfp4_prefill_gemm_tflops", "TFLOP/s", flops / 1e12
            workload = f"configs[2]: NVFP4 W4A4 prefill GEMM, M={tokens}, up 5120->17408 and down 17408->5120, fused-layout activation quantizer + tcgen05 block-scaled MMA"
            if args.a16:
                workload = (f"configs[2]'s shapes under the A16 policy, M={tokens}: weights decoded to BF16 in shared memory, "
                            "tcgen05 kind::f16 MMA, no activation quantization")
            if args.mlp:
                workload = (f"configs[2] as the layer's MLP, M={tokens}: gate|up 5120->34816 with SwiGLU and the down product's "
                            "quantizer in its epilogue, then down 17408->5120; one activation quantizer launch")
        elif args.workload == "head":
            # the output head: 5120 -> 248320 at 4 bits per weight, the largest product of a decode step
            in_, out, k2 = 5120, 248320, 8
            gen = torch.Generator(device=device).manual_seed(20261131)
            heads = []
            for _ in range(2):   # two copies: 2 x 636 MB streams past the L2
                words = torch.randint(-32768, 32767, ((in_ // 16) * (out // 16) * 64,), dtype=torch.int16, device=device, generator=gen)
                suh = ((torch.rand(in_, device=device, generator=gen) * 1.5 + 0.5) * 0.05).to(torch.float16)
                svh = ((torch.rand(out, device=device, generator=gen) * 1.5 + 0.5) * 0.03).to(torch.float16)
                heads.append(trellis.Weight(words, suh, svh, k2, in_, out))
            xh = torch.randn(args.tokens, in_, device=device, generator=gen).to(torch.bfloat16)
            yh = torch.empty(args.tokens, out, dtype=torch.bfloat16, device=device)
            nbytes = 2 * (trellis.weight_bytes(in_, out, k2) + args.tokens * in_ * 2 + args.tokens * out * 2)

            def one_step() -> None:
                for w in heads:
                    trellis.linear(w, xh, out=yh)

            launches = 2
            metric, unit, work = "trellis_gemv_gbs", "GB/s", nbytes / 1e9
            workload = f"output head: trellis 4 bpw, 5120 -> 248320, M={args.tokens}, two distinct copies per step"
        else:
            weights, inputs, outputs, nbytes = build_trellis_workload(args.layers, 0, 1, args.tokens, device)
            by = {name: (in_, out) for name, in_, out in TRELLIS_LAYER}

            # q | k | v share one launch (narrow weights alone cannot fill the device); the wide ones run alone
            groups = [["q", "k", "v"], ["o"], ["gate"], ["up"], ["down"]] if args.group else [[n] for n, *_ in TRELLIS_LAYER]

            def one_step() -> None:
                for layer in weights:
                    for names in groups:
                        src = inputs[by[names[0]][0]]
                        if len(names) == 1:
                            trellis.linear(layer[names[0]], src, out=outputs[names[0]])
                        else:
                            trellis.linear_group([layer[n] for n in names], src, outs=[outputs[n] for n in names])

            launches = len(groups) * args.layers
            metric, unit, work = "trellis_gemv_gbs", "GB/s", nbytes / 1e9
            workload = f"configs[3]: trellis 3 bpw decode, M={args.tokens}, 27B-style layer x {args.layers} layers of distinct weights"
        one_step()
        stream.synchronize()
        step = one_step
        if args.graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                one_step()
            step = graph.replay
        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(0) as clocks:
            start.record(stream)
            for _ in range(args.steps):
                step()
            stop.record(stream)
            torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / args.steps
    value = work / (ms * 1e-3)
    if args.workload == "prefill" and args.a16:
        peak = 1403.2
        roof = {"bound": "tensor", "achieved": value, "peak": peak, "unit": "TFLOP/s", "frac": value / peak,
                "peak_source": "measured sustained BF16 cuBLAS rate", "frac_of_nominal_2250": value / 2250.0,
                "kernel": "nvfp4_a16_mma_kernel", "traffic": None, "device_status": nvfp4.device_status()}
    elif args.workload == "prefill":
        status = ws.status()
        peak = 4.0 * 1403.2
        roof = {"bound": "tensor", "achieved": value, "peak": peak, "unit": "TFLOP/s", "frac": value / peak,
                "peak_source": "4 x the measured sustained BF16 cuBLAS rate (FP4 dense is 4 x BF16 dense on this part)",
                "frac_of_nominal_9000": value / 9000.0, "kernel": "w4a4_gemm_pair_kernel", "traffic": None,
                "device_status": status}
    else:
        roof = {"bound": "hbm", "achieved": value, "peak": peak_hbm, "unit": "GB/s", "frac": value / peak_hbm,
                "peak_source": f"{peak_kind} copy bandwidth; the kernel is instruction-issue bound (about 5 integer operations per weight)",
                "kernel": "trellis_linear_kernel", "traffic": None}  # also the head workload
    print(json.dumps({"metric": metric, "value": value, "unit": unit, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
                      "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                      "dtype": ("bf16xbf16->f32" if args.a16 else "e2m1xe2m1->f32") if args.workload == "prefill" else "f16xf16->f32", "data": "synthetic",
                      "config": {"workload": workload, "cuda_graph": bool(args.graph), "l2": "inputs larger than L2"},
                      "gpu_launches": launches * args.steps, "clocks": clocks.summary(), "roofline": roof}))


def run_cuda_arm(args) -> None:
    import torch
    import torch.distributed as dist

    from ignis_b200 import nvfp4

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    nvfp4.prepare()
    tokens = args.tokens
    # How the matrices shard over N ranks: always column-wise (output rows) with no exchange inside
    # a product. "weak" (default): every rank holds a full configs[1] layer set - the shard of a
    # layer N times as wide - so per-GPU work is fixed. "strong": configs[1] itself is cut in N.
    split = world if args.scaling == "strong" else 1
    weights, host_inputs, inputs, outputs = build_workload(args.layers, rank, split, tokens, device)
    by_name = {name: (n, k, src) for name, n, k, src in LAYER}
    calls = GROUPS if args.group else [[name] for name, *_ in LAYER]

    gather = args.gather == 1 and world > 1
    fused = args.gather == 2 and world > 1
    # "a16" (the headline): BF16 activations as they are. "a4": the reference engine's default AllowA4
    # policy, under which these calls quantize their activations from 4 / 5 / 8 tokens (W4A4).
    policy = nvfp4.ALLOW_A4 if args.policy == "a4" and not fused else nvfp4.A16_ONLY
    if gather:
        from ignis_b200 import shard

        full = {name: torch.empty(tokens, outputs[name].shape[1] * world, dtype=torch.bfloat16, device=device) for name in outputs}
    if fused:
        from ignis_b200 import shard

        peer = shard.PeerOutputs({name: (tokens, outputs[name].shape[1] * world) for name in outputs})

    def one_step(policy: int = policy) -> None:
        for layer in weights:
            for names in calls:
                src = inputs[by_name[names[0]][2]]
                if fused:
                    # every rank's epilogue stores its columns into all ranks' full-width buffers; the
                    # device barrier behind it is all that is left of the all-gather
                    ws = [layer[nm] for nm in names]
                    nvfp4.linear_group_scatter(src, ws, [peer.pointers(nm) for nm in names], [w.n * world for w in ws],
                                               [w.n * rank for w in ws])
                    peer.barrier()
                elif len(names) == 1:
                    nvfp4.linear(src, layer[names[0]], out=outputs[names[0]], policy=policy)
                else:
                    nvfp4.linear_group(src, [layer[nm] for nm in names], outs=[outputs[nm] for nm in names], policy=policy)
                if gather:   # rejoin the column shards where a consumer would need the full width
                    for nm in names:
                        shard.gather_columns(outputs[nm], out=full[nm])

    launches_per_step = len(calls) * args.layers * (2 if fused else 1)   # the fused form adds a barrier launch per call
    stream = torch.cuda.Stream()
    graph = None
    with torch.cuda.stream(stream):
        one_step()  # untimed: first-launch costs
        stream.synchronize()
        if args.graph and not gather:   # the collectives run outside a graph
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                one_step()
        step = graph.replay if graph is not None else one_step

        def barrier() -> None:
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        for _ in range(args.warmup):
            step()
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as clocks:
            start.record(stream)
            for _ in range(args.steps):
                step()
            stop.record(stream)
            barrier()
        device_ms = start.elapsed_time(stop)

        # end to end: host activations in, last output back, every step
        result_host = torch.empty_like(outputs["down"], device="cpu").pin_memory()
        for _ in range(2):
            for key in inputs:
                inputs[key].copy_(host_inputs[key], non_blocking=True)
            step()
            result_host.copy_(outputs["down"], non_blocking=True)
        barrier()
        e2e_start, e2e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2e_start.record(stream)
        for _ in range(args.steps):
            for key in inputs:
                inputs[key].copy_(host_inputs[key], non_blocking=True)
            step()
            result_host.copy_(outputs["down"], non_blocking=True)
        e2e_stop.record(stream)
        barrier()
        e2e_ms = e2e_start.elapsed_time(e2e_stop)

        # the same step under the reference engine's default policy, timed the same way, reported beside
        # the headline (never instead of it)
        a4_ms = None
        if policy == nvfp4.A16_ONLY and world == 1 and args.graph and tokens >= 4:
            one_step(nvfp4.ALLOW_A4)
            stream.synchronize()
            a4_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(a4_graph, stream=stream):
                one_step(nvfp4.ALLOW_A4)
            for _ in range(args.warmup):
                a4_graph.replay()
            a4_start, a4_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a4_start.record(stream)
            for _ in range(args.steps):
                a4_graph.replay()
            a4_stop.record(stream)
            torch.cuda.synchronize()
            a4_ms = a4_start.elapsed_time(a4_stop) / args.steps

    times = torch.tensor([device_ms, e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    device_ms, e2e_ms = times.tolist()
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return

    per_rank_bytes = layer_algorithmic_bytes(tokens, split) * args.layers
    job_bytes = per_rank_bytes * world
    ms_per_step = device_ms / args.steps
    value = job_bytes / (ms_per_step * 1e-3) / 1e9
    e2e_value = job_bytes / (e2e_ms / args.steps * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    per_gpu = value / world
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f16xf16->f32",
        "data": "synthetic",
        "config": {"workload": "configs[1]: NVFP4 decode, 8 lanes (M=8), 27B-style dense layer (q,k,v,o,gate,up,down), hidden 5120",
                   "layers": args.layers, "tokens": tokens,
                   "policy": "AllowA4 (activations quantized to NVFP4 inside the product, W4A4 on tcgen05)" if policy == nvfp4.ALLOW_A4 else "A16",
                   "device_status": nvfp4.device_status(), "sharding": (f"column-wise over N, {world} rank(s); " +
                                ("every rank holds configs[1]-sized shards of a layer N times as wide (per-GPU work fixed)"
                                 if args.scaling == "weak" else "configs[1] itself cut in N (total work fixed)")),
                   "calls_per_layer": len(calls), "cuda_graph": bool(args.graph) and not gather,
                   "l2": "inputs larger than L2: %.2f GB of distinct weights per rank per step" % (per_rank_bytes / 1e9),
                   "collective": ("NCCL all-gather of every output (%d per layer)" % len(LAYER)) if gather else
                                 ("fused: epilogues store into every rank's buffer over NVLink, one device barrier per call" if fused
                                  else "none (outputs stay sharded)"),
                   **({"barrier_timeouts": peer.missing()} if fused else {})},
        "e2e": {"value": e2e_value, "unit": UNIT,
                "h2d_bytes_per_step": sum(t.numel() * 2 for t in host_inputs.values()),
                "d2h_bytes_per_step": outputs["down"].numel() * 2},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                     "peak_source": f"{peak_kind} copy bandwidth", "frac_of_nominal_8000": per_gpu / 8000.0,
                     "kernel": "nvfp4_gemv_kernel<1>", "bytes_per_launch": per_rank_bytes / launches_per_step,
                     "us_per_launch": ms_per_step * 1e3 / launches_per_step, "traffic": TRAFFIC_PER_LAUNCH / split},
    }
    if a4_ms is not None:
        a4_value = job_bytes / (a4_ms * 1e-3) / 1e9
        line["allow_a4"] = {"policy": "the reference engine's default AllowA4: activations quantized to NVFP4 inside each product "
                                      "(from 4 / 5 / 8 tokens by problem), W4A4 on tcgen05, weights from HBM to the tensor cores by TMA",
                            "value": a4_value, "unit": UNIT, "ms_per_step": a4_ms, "frac": a4_value / peak,
                            "kernel": "w4a4_decode_kernel", "us_per_launch": a4_ms * 1e3 / launches_per_step}
    if world == 1 and not args.no_cpu_baseline:
        v, desc = cpu_sample()
        line["cpu_baseline"] = {"value": v, "unit": UNIT, **desc}
    print(json.dumps(line))


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel: the mean over the
# four launches of one layer in the ncu capture summarised in profiles/nvfp4_gemv_decode_m8.md
# (196.97 MB per layer; the algorithmic bytes of the same four launches are 193.3 MB).
TRAFFIC_PER_LAUNCH = 49.24e6


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200q", choices=["b200q", "reference"])
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--group", type=int, default=1, help="1: q|k|v and gate|up share one launch each; 0: seven launches per layer")
    ap.add_argument("--graph", type=int, default=1, help="replay the step as one CUDA graph")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="decode workload under torchrun: weak = per-GPU work fixed (default), strong = configs[1] cut in N")
    ap.add_argument("--gather", type=int, default=0, help="decode workload under torchrun: 1 all-gathers every output after its product (NCCL); 2 the fused form (peer stores + device barrier)")
    ap.add_argument("--moe-tokens", type=int, default=4096, help="tokens of the --workload moe step (configs[4]: 4096; up to 8 takes the decode entry's item size)")
    ap.add_argument("--policy", choices=["a16", "a4"], default="a16",
                    help="decode workload: a16 (headline) or a4, the reference's AllowA4 policy (W4A4 from 4 / 5 / 8 tokens)")
    ap.add_argument("--a16", type=int, default=0, help="with --workload prefill: 1 runs the two products under the A16 policy")
    ap.add_argument("--mlp", type=int, default=0, help="with --workload prefill: 1 runs the fused MLP entry instead of two plain products")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "trellis", "moe", "head"],
                    help="decode: configs[1] (the headline); prefill: configs[2]; trellis: configs[3]; moe: configs[4]")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "moe":
        run_moe_workload(args)
    elif args.workload != "decode":
        run_side_workload(args)
    else:
        run_cuda_arm(args)


if __name__ == "__main__":
    main()
