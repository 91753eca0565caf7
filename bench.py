"""Benchmark of the quantized linear-layer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline (BASELINE.json configs[1]): NVFP4 batched decode, 8 lanes, one 27B-style dense layer with
hidden 5120 -- q 5120->6144, k and v 5120->1024, o 6144->5120, gate and up 5120->17408,
down 17408->5120 -- repeated over 64 layers of distinct synthetic weights (12.27 GB, far larger than
L2, so no timed iteration finds its weights cached). A step is one pass over all layers, replayed as
one CUDA graph. The metric is the weight-stream rate: algorithmic bytes (codes + scales + divisors
+ activations in and out) per second, whole job.

On one GPU the line also carries one object per other config of BASELINE.json, each timed the same
way: `config0` (M = 1 GEMV), `config2` (W4A4 prefill GEMM, TFLOP/s, against the measured FP4 tensor
rate in `fp4_peak`), `config3` (trellis 3 bpw, M = 1 and 8), `config4` (MoE experts), and `allow_a4`
(the headline under the reference engine's default AllowA4 policy).

At N > 1 (launched under torch.distributed.run) configs[1] itself is cut in N: every matrix is
sharded column-wise (output rows) over the ranks, total work fixed ("scaling": "strong"), and the
outputs are rejoined where the next op needs the full width -- after `o`, after gate|up (down's
K = 17408 input), after `down` -- by the products themselves: their epilogues store into every
rank's buffer over NVLink and the barrier between the ranks rides in the first instructions of the
consuming product (`--gather 3`, the default; 0 none, 1 NCCL all-gather, 2 a barrier launch per product;
`--scaling weak` gives every rank a full layer set instead). The N > 1 line carries `config2`
(the prefill GEMM N-sharded, both ways of sharing the quantized operand) and `config4` (MoE,
expert-parallel with an NCCL all-to-all each way). Rank 0 prints one JSON line.

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
DTYPE = "e2m1 (ue4m3 block scale) x bf16 -> f32"


_RESULT_STREAM = None


def claim_stdout() -> None:
    """Under torchrun, libraries write to file descriptor 1 on their own (NCCL prints its version
    there): keep a private copy of stdout for the result line and point descriptor 1 at stderr."""
    global _RESULT_STREAM
    if _RESULT_STREAM is None and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        sys.stdout.flush()
        _RESULT_STREAM = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(line: dict) -> None:
    """The run's one JSON line, on the process's original stdout."""
    out = _RESULT_STREAM or sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def weight_bytes(n: int, k: int) -> int:
    return n * k // 2 + n * k // 16 + 4


def layer_algorithmic_bytes(tokens: int, world: int = 1) -> int:
    """Bytes one rank must move for one layer: its shard of every payload, each activation read
    once per call that uses it, each output written once."""
    total = 0
    for _, n, k, _ in LAYER:
        total += weight_bytes(n // world, k) + tokens * k * 2 + tokens * (n // world) * 2
    return total


def measured_peaks() -> dict:
    """The driver-measured denominators (HBM copy GB/s, BF16 cuBLAS TFLOP/s burst and sustained),
    else the fallback measured earlier on this pool."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d["bf16_tflops_sustained"]), "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "kind": "fallback"}


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
    emit(line)


# ---- synthetic weights ----------------------------------------------------------------------------

def random_nvfp4(n: int, k: int, gen, device, d_w: float = 448.0, d_in: float = 448.0):
    """configs[0]'s distribution on the device: codes uniform over 16 values, scales = E4M3(|N(0,1)| + 0.1)
    in the stored (swizzled) order, tensor scale 1 / 448."""
    import torch

    from ignis_b200 import nvfp4

    codes = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=device, generator=gen)
    natural = (torch.randn((n, k // 16), device=device, generator=gen).abs() + 0.1).to(torch.float8_e4m3fn).view(torch.uint8)
    stored = natural.reshape(n // 128, 4, 32, k // 64, 4).permute(0, 3, 2, 1, 4).contiguous().reshape(-1)
    return nvfp4.Weight(codes, stored, n, k, d_w, d_in)


def build_workload(layers: int, rank: int, world: int, tokens: int, device):
    import torch

    gen = torch.Generator(device=device)
    weights = []
    for layer in range(layers):
        entry = {}
        for idx, (name, n, k, _) in enumerate(LAYER):
            gen.manual_seed(20261126 + (layer * 16 + idx) * 64 + rank)
            entry[name] = random_nvfp4(n // world, k, gen, device)
        weights.append(entry)
    cpu_gen = torch.Generator().manual_seed(20261126)
    host_inputs = {key: torch.randn(tokens, width, generator=cpu_gen).to(torch.bfloat16).pin_memory()
                   for key, width in INPUT_WIDTH.items()}
    inputs = {key: t.to(device) for key, t in host_inputs.items()}
    outputs = {name: torch.empty(tokens, n // world, dtype=torch.bfloat16, device=device) for name, n, _, _ in LAYER}
    return weights, host_inputs, inputs, outputs


TRELLIS_LAYER = [("q", 5120, 6144), ("k", 5120, 1024), ("v", 5120, 1024), ("o", 6144, 5120), ("gate", 5120, 17408),
                 ("up", 5120, 17408), ("down", 17408, 5120)]  # (name, in, out), configs[3]


def build_trellis_workload(layers: int, tokens: int, device):
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
            gen.manual_seed(20261127 + (layer * 16 + idx) * 64)
            words = torch.randint(-32768, 32767, ((in_ // 16) * (out // 16) * 48,), dtype=torch.int16, device=device,
                                  generator=gen)
            suh = ((torch.rand(in_, device=device, generator=gen) * 1.5 + 0.5) * 0.05).to(torch.float16)
            svh = ((torch.rand(out, device=device, generator=gen) * 1.5 + 0.5) * 0.03).to(torch.float16)
            entry[name] = trellis.Weight(words, suh, svh, 6, in_, out)
            if layer == 0:
                total += trellis.weight_bytes(in_, out, 6) + tokens * in_ * 2 + tokens * out * 2
        weights.append(entry)
    cpu_gen = torch.Generator().manual_seed(20261127)
    inputs = {w: torch.randn(tokens, w, generator=cpu_gen).to(torch.bfloat16).to(device) for w in (5120, 6144, 17408)}
    outputs = {name: torch.empty(tokens, out, dtype=torch.bfloat16, device=device) for name, _, out in TRELLIS_LAYER}
    return weights, inputs, outputs, total * layers


def build_moe_workload(tokens: int, device, rank=0, world=1, hidden=2048, inter=768, experts=512, top_k=10, k2=5):
    """configs[4]: 512 experts of (hidden 2048, intermediate 768) at 2.5 bits per weight, every record
    distinct (random words: every bit pattern is a valid encoding), Zipf(1.1) expert popularity over a
    seeded permutation, 10 distinct experts per token drawn in proportion to popularity, routing
    weights = BF16(softmax of 10 normal logits). The shared expert is the FP8 row-scale one."""
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
            "host": host, "experts": experts, "hidden": hidden}


# ---- timing -----------------------------------------------------------------------------------------

def time_region(stream, step, steps: int, warmup: int, barrier=None, sampler: ClockSampler | None = None) -> float:
    """`warmup` untimed steps, then exactly `steps` timed with CUDA events on `stream`, a barrier and
    a device synchronize on both sides. Returns milliseconds for all `steps`."""
    import torch

    def sync() -> None:
        if barrier is not None:
            barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    sync()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if sampler is not None:
        sampler.__enter__()
    try:
        start.record(stream)
        for _ in range(steps):
            step()
        stop.record(stream)
        sync()
    finally:
        if sampler is not None:
            sampler.__exit__(None, None, None)
    return start.elapsed_time(stop)


def graphed(stream, one_step, enable: bool = True):
    """Runs `one_step` once (first-launch costs), then returns a replay of it as one CUDA graph."""
    import torch

    one_step()
    stream.synchronize()
    if not enable:
        return one_step
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        one_step()
    return graph.replay


# ---- the side configs, each a dict for the headline line or a line of its own ---------------------------

def measure_fp4_peak(stream, device, seconds: float = 2.5) -> dict:
    """The tensor cores' block-scaled FP4 rate (tcgen05.mma kind::mxf4nvf4 over resident operands): a
    burst (the best of the first launches, the part cold and at full clock) and the rate sustained
    over `seconds` of back-to-back launches, the SM clock sampled beside it; both issue forms."""
    import torch

    from ignis_b200 import nvfp4

    sink = torch.zeros(256, dtype=torch.float32, device=device)
    out = {}
    for name, pair in (("one_cta", False), ("cta_pair", True)):
        iters = 4096                                    # about 1.2 ms a launch at the nominal rate
        nvfp4.mma_peak(64, pair, sink)                  # module load, first launch
        stream.synchronize()
        evs = []
        sampler = ClockSampler(device.index or 0)
        with sampler:
            t_end = time.perf_counter() + seconds / 2
            flops = 0.0
            while time.perf_counter() < t_end:
                batch = []
                for _ in range(20):
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(stream)
                    flops = nvfp4.mma_peak(iters, pair, sink)
                    b.record(stream)
                    batch.append((a, b))
                stream.synchronize()
                evs += [a.elapsed_time(b) for a, b in batch]
        burst = flops / 1e12 / (min(evs[:20]) * 1e-3)
        tail = evs[len(evs) // 2:]
        sustained = flops / 1e12 / (sum(tail) / len(tail) * 1e-3)
        out[name] = {"burst_tflops": burst, "sustained_tflops": sustained, "launches": len(evs), "clocks": sampler.summary()}
    out["status"] = nvfp4.mma_peak_status()
    best = max(out["one_cta"]["burst_tflops"], out["cta_pair"]["burst_tflops"])
    best_sustained = max(out["one_cta"]["sustained_tflops"], out["cta_pair"]["sustained_tflops"])
    out.update({"burst_tflops": best, "sustained_tflops": best_sustained, "nominal_tflops": 9000.0,
                "how": "tcgen05.mma kind::mxf4nvf4 block_scale scale_vec::4X over operands resident in shared and tensor memory, "
                       "every SM, no global traffic (b200q_nvfp4_mma_peak); burst = best of the first 20 launches, sustained = mean of "
                       "the second half of back-to-back launches"})
    return out


def prefill_roofline(value: float, ms: float, fp4: dict | None, peaks: dict, kernel: str, status: int) -> dict:
    """configs[2] against the measured FP4 rate: the burst figure for a region of a few milliseconds,
    beside 4 x the measured BF16 burst rate and the nominal 9 PFLOP/s."""
    roof = {"bound": "tensor", "achieved": value, "unit": "TFLOP/s", "kernel": kernel, "traffic": None, "device_status": status,
            "frac_of_4x_bf16_burst": value / (4.0 * peaks["bf16_tflops"]), "frac_of_nominal_9000": value / 9000.0}
    if fp4 is not None:
        roof.update({"peak": fp4["burst_tflops"], "frac": value / fp4["burst_tflops"],
                     "peak_source": "measured: tcgen05 kind::mxf4nvf4 loop over resident operands, burst (this run)",
                     "frac_of_sustained_fp4": value / fp4["sustained_tflops"]})
    else:
        roof.update({"peak": 4.0 * peaks["bf16_tflops"], "frac": value / (4.0 * peaks["bf16_tflops"]),
                     "peak_source": f"4 x the {peaks['kind']} BF16 cuBLAS burst rate (no FP4 loop in this run)"})
    return roof


def measure_prefill(stream, device, steps: int, warmup: int, peaks: dict, fp4: dict | None, tokens: int = 8192, form: str = "linear",
                    graph: bool = True) -> dict:
    """configs[2]: up 5120 -> 17408 and down 17408 -> 5120 at `tokens` tokens. form "linear": two
    b200q_nvfp4_linear calls under AllowA4 (activation quantizer + tensor-core GEMM each, both inside
    the timed region); "mlp": the layer's MLP through b200q_nvfp4_mlp (gate|up with SwiGLU and the
    down product's quantizer in its epilogue); "a16": the two products under A16."""
    import torch

    from ignis_b200 import nvfp4

    gen = torch.Generator(device=device)
    shapes = [("up", 17408, 5120), ("down", 5120, 17408)]
    items = []
    for idx, (_, n, k) in enumerate(shapes):
        gen.manual_seed(20261128 + idx)
        w = random_nvfp4(n, k, gen, device)
        x = torch.randn(tokens, k, device=device, generator=gen).to(torch.bfloat16)
        items.append((w, x, torch.empty(tokens, n, dtype=torch.bfloat16, device=device)))
    flops = sum(2.0 * tokens * w.n * w.k for w, _, _ in items)
    if form == "mlp":
        gen.manual_seed(20261130)
        gate_up = random_nvfp4(2 * 17408, 5120, gen, device)
        down_w, _, y_down = items[1]
        x_in = items[0][1]
        ws = nvfp4.Workspace(nvfp4.mlp_workspace_bytes(gate_up.n, gate_up.k, nvfp4.ALLOW_A4, tokens), device)
        flops = 2.0 * tokens * (gate_up.n * gate_up.k + down_w.n * down_w.k)

        def one_step() -> None:
            nvfp4.mlp(x_in, gate_up, down_w, ws, out=y_down, policy=nvfp4.ALLOW_A4)

        launches, kernel = 3, "w4a4_gemm_pair_kernel"
        what = (f"configs[2] as the layer's MLP, M={tokens}: gate|up 5120->34816 with SwiGLU and the down product's quantizer in its "
                "epilogue, then down 17408->5120; one activation quantizer launch")
    elif form == "a16":
        ws = None

        def one_step() -> None:
            for w, x, y in items:
                nvfp4.linear(x, w, out=y)

        launches, kernel = 2, "nvfp4_a16_mma_kernel"
        what = (f"configs[2]'s shapes under the A16 policy, M={tokens}: weights decoded to BF16 in shared memory, tcgen05 kind::f16, "
                "no activation quantization")
    else:
        ws = nvfp4.Workspace(max(nvfp4.workspace_bytes(w.n, w.k, nvfp4.ALLOW_A4, tokens) for w, _, _ in items), device)

        def one_step() -> None:
            for w, x, y in items:
                nvfp4.linear(x, w, out=y, policy=nvfp4.ALLOW_A4, workspace=ws)

        launches, kernel = 4, "w4a4_gemm_pair_kernel"
        what = (f"configs[2]: NVFP4 W4A4 prefill GEMM, M={tokens}, up 5120->17408 and down 17408->5120, activation quantizer "
                "(inside the timed region) + tcgen05 block-scaled MMA")
    step = graphed(stream, one_step, graph)
    sampler = ClockSampler(device.index or 0)
    ms = time_region(stream, step, steps, warmup, sampler=sampler) / steps
    value = flops / 1e12 / (ms * 1e-3)
    status = ws.status() if ws is not None else nvfp4.device_status()
    if form == "a16":
        roof = {"bound": "tensor", "achieved": value, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": value / peaks["bf16_tflops"],
                "peak_source": f"{peaks['kind']} BF16 cuBLAS burst rate", "kernel": kernel, "traffic": None, "device_status": status}
    else:
        roof = prefill_roofline(value, ms, fp4, peaks, kernel, status)
    return {"metric": "nvfp4_prefill_gemm_tflops", "value": value, "unit": "TFLOP/s", "ms_per_step": ms, "steps": steps, "warmup": warmup,
            "dtype": "bf16 x bf16 -> f32" if form == "a16" else "e2m1 x e2m1 (ue4m3 block scales) -> f32",
            "config": {"workload": what, "cuda_graph": graph, "l2": "inputs larger than L2"}, "gpu_launches": launches * steps,
            "clocks": sampler.summary(), "roofline": roof}


def measure_config0(stream, device, weights, steps: int, warmup: int, peaks: dict, graph: bool = True) -> dict:
    """configs[0]: the M = 1 GEMV over one MLP up-projection (17408 x 5120). One matrix (50 MB) would
    sit in the L2, so a step walks the gate and up matrices of every layer of the headline's weight
    set: 2 x layers distinct copies of the configs[0] shape."""
    import torch

    from ignis_b200 import nvfp4

    cpu_gen = torch.Generator().manual_seed(20261125)
    x = torch.randn(1, 5120, generator=cpu_gen).to(torch.bfloat16).to(device)
    y = torch.empty(1, 17408, dtype=torch.bfloat16, device=device)
    mats = [layer[name] for layer in weights for name in ("gate", "up")]

    def one_step() -> None:
        for w in mats:
            nvfp4.linear(x, w, out=y)

    step = graphed(stream, one_step, graph)
    ms = time_region(stream, step, steps, warmup) / steps
    per = weight_bytes(17408, 5120) + 2 * 5120 + 2 * 17408
    value = per * len(mats) / (ms * 1e-3) / 1e9
    return {"metric": METRIC, "value": value, "unit": UNIT, "ms_per_step": ms, "steps": steps, "warmup": warmup, "dtype": DTYPE,
            "config": {"workload": f"configs[0]: NVFP4 GEMV M=1, K=5120, N=17408, {len(mats)} distinct matrices per step "
                                   f"({per * len(mats) / 1e9:.2f} GB: larger than L2)", "cuda_graph": graph},
            "gpu_launches": len(mats) * steps, "us_per_launch": ms * 1e3 / len(mats),
            "roofline": {"bound": "hbm", "achieved": value, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": value / peaks["hbm_gbs"],
                         "peak_source": f"{peaks['kind']} copy bandwidth", "frac_of_nominal_8000": value / 8000.0,
                         "kernel": "nvfp4_gemv_kernel<1>", "bytes_per_launch": per, "traffic": None}}


def measure_trellis(stream, device, steps: int, warmup: int, peaks: dict, layers: int = 64, tokens: int = 8, group: bool = True,
                    graph: bool = True) -> dict:
    """configs[3]: the 27B layer's seven shapes at 3 bits per weight, `layers` distinct copies, M = `tokens`."""
    from ignis_b200 import trellis

    weights, inputs, outputs, nbytes = build_trellis_workload(layers, tokens, device)
    by = {name: (in_, out) for name, in_, out in TRELLIS_LAYER}
    # q | k | v share one launch (narrow weights alone cannot fill the device); the wide ones run alone
    groups = [["q", "k", "v"], ["o"], ["gate"], ["up"], ["down"]] if group else [[n] for n, *_ in TRELLIS_LAYER]

    def one_step() -> None:
        for layer in weights:
            for names in groups:
                src = inputs[by[names[0]][0]]
                if len(names) == 1:
                    trellis.linear(layer[names[0]], src, out=outputs[names[0]])
                else:
                    trellis.linear_group([layer[n] for n in names], src, outs=[outputs[n] for n in names])

    step = graphed(stream, one_step, graph)
    sampler = ClockSampler(device.index or 0)
    ms = time_region(stream, step, steps, warmup, sampler=sampler) / steps
    value = nbytes / 1e9 / (ms * 1e-3)
    return {"metric": "trellis_gemv_gbs", "value": value, "unit": "GB/s", "ms_per_step": ms, "steps": steps, "warmup": warmup,
            "dtype": "trellis 3 bpw -> f16 x f16 -> f32",
            "config": {"workload": f"configs[3]: trellis 3 bpw decode, M={tokens}, 27B-style layer x {layers} layers of distinct weights "
                                   f"({nbytes / 1e9:.2f} GB per step)", "cuda_graph": graph, "l2": "inputs larger than L2"},
            "gpu_launches": len(groups) * layers * steps, "clocks": sampler.summary(),
            "roofline": {"bound": "hbm", "achieved": value, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": value / peaks["hbm_gbs"],
                         "peak_source": f"{peaks['kind']} copy bandwidth; the kernel is instruction-issue bound (about 5 integer operations per weight)",
                         "kernel": "trellis_linear_kernel", "traffic": None, "device_status": 0}}


def measure_trellis_prefill(stream, device, steps: int, warmup: int, peaks: dict, layers: int = 4, tokens: int = 1024, graph: bool = True) -> dict:
    """The dense trellis linear beyond 64 tokens (the tensor-core route): configs[3]'s seven shapes at
    `tokens` tokens over `layers` distinct layers, TFLOP/s of 2 x tokens x in x out."""
    from ignis_b200 import trellis

    weights, inputs, outputs, _ = build_trellis_workload(layers, tokens, device)
    by = {name: (in_, out) for name, in_, out in TRELLIS_LAYER}
    ws = trellis.WorkspaceBuffer(max(trellis.workspace_bytes(in_, out, 1, tokens) for _, in_, out in TRELLIS_LAYER), device)
    flops = layers * sum(2.0 * tokens * in_ * out for _, in_, out in TRELLIS_LAYER)

    def one_step() -> None:
        for layer in weights:
            for name, (in_, _) in by.items():
                trellis.linear(layer[name], inputs[in_], out=outputs[name], workspace=ws)

    step = graphed(stream, one_step, graph)
    sampler = ClockSampler(device.index or 0)
    ms = time_region(stream, step, steps, warmup, sampler=sampler) / steps
    value = flops / 1e12 / (ms * 1e-3)
    return {"metric": "trellis_prefill_gemm_tflops", "value": value, "unit": "TFLOP/s", "ms_per_step": ms, "steps": steps, "warmup": warmup,
            "dtype": "trellis 3 bpw -> f16 x f16 -> f32",
            "config": {"workload": f"configs[3]'s shapes at M={tokens}: rotation + tcgen05 product per weight, {layers} layers of distinct weights",
                       "cuda_graph": graph},
            "gpu_launches": 2 * len(TRELLIS_LAYER) * layers * steps, "clocks": sampler.summary(),
            "roofline": {"bound": "tensor", "achieved": value, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": value / peaks["bf16_tflops"],
                         "peak_source": f"{peaks['kind']} BF16 cuBLAS burst rate (fp16 operands run at the same rate)",
                         "kernel": "trellis_tc_dense_kernel", "traffic": None, "device_status": trellis.device_status()}}


def measure_head(stream, device, steps: int, warmup: int, peaks: dict, tokens: int, graph: bool = True) -> dict:
    """The output head: 5120 -> 248320 at 4 bits per weight, the largest product of a decode step."""
    import torch

    from ignis_b200 import trellis

    in_, out, k2 = 5120, 248320, 8
    gen = torch.Generator(device=device).manual_seed(20261131)
    heads = []
    for _ in range(2):   # two copies: 2 x 636 MB streams past the L2
        words = torch.randint(-32768, 32767, ((in_ // 16) * (out // 16) * 64,), dtype=torch.int16, device=device, generator=gen)
        suh = ((torch.rand(in_, device=device, generator=gen) * 1.5 + 0.5) * 0.05).to(torch.float16)
        svh = ((torch.rand(out, device=device, generator=gen) * 1.5 + 0.5) * 0.03).to(torch.float16)
        heads.append(trellis.Weight(words, suh, svh, k2, in_, out))
    xh = torch.randn(tokens, in_, device=device, generator=gen).to(torch.bfloat16)
    yh = torch.empty(tokens, out, dtype=torch.bfloat16, device=device)
    nbytes = 2 * (trellis.weight_bytes(in_, out, k2) + tokens * in_ * 2 + tokens * out * 2)

    def one_step() -> None:
        for w in heads:
            trellis.linear(w, xh, out=yh)

    step = graphed(stream, one_step, graph)
    ms = time_region(stream, step, steps, warmup) / steps
    value = nbytes / 1e9 / (ms * 1e-3)
    return {"metric": "trellis_gemv_gbs", "value": value, "unit": "GB/s", "ms_per_step": ms, "steps": steps, "warmup": warmup,
            "dtype": "trellis 4 bpw -> f16 x f16 -> f32",
            "config": {"workload": f"output head: trellis 4 bpw, 5120 -> 248320, M={tokens}, two distinct copies per step", "cuda_graph": graph},
            "gpu_launches": 2 * steps,
            "roofline": {"bound": "hbm", "achieved": value, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": value / peaks["hbm_gbs"],
                         "peak_source": f"{peaks['kind']} copy bandwidth", "kernel": "trellis_linear_kernel", "traffic": None}}


def measure_moe(stream, device, steps: int, warmup: int, peaks: dict, tokens: int = 4096, rank: int = 0, world: int = 1,
                graph: bool = True, barrier=None, exchange: str = "gathered") -> dict:
    """configs[4]: routed experts + shared expert + combine, TFLOP/s. One GPU: the step is one CUDA
    graph. N GPUs: expert-parallel, tokens split over the ranks. `exchange` "gathered": all-gather
    of the tokens, every rank runs its experts over all of them, one reduce-scatter of the integer
    sums (fixed sizes, no host synchronisation, the step is one CUDA graph); "compact": the
    counted all-to-all each way (sizes known on the host, eager). Timed on the device (the caller
    takes the max over ranks)."""
    import torch

    from ignis_b200 import moe, moe_ep

    m = build_moe_workload(tokens, device, rank, world)
    out_host = torch.empty((m["x"].shape[0], m["hidden"]), dtype=torch.bfloat16).pin_memory()
    side = torch.cuda.Stream()   # the shared expert needs no exchange: it runs beside it
    phases = {}

    def one_step():
        if world == 1:
            moe.experts_prefill(m["x"], m["ids"], m["weights"], m["table"], m["ws"])
            shared, _ = moe.shared_expert(m["shared"][0], m["shared"][1], m["shared"][2], m["x"])
            return moe.combine(m["ws"], shared, m["x"], m["w_gate"])
        main = torch.cuda.current_stream()
        side.wait_stream(main)
        with torch.cuda.stream(side):
            shared, _ = moe.shared_expert(m["shared"][0], m["shared"][1], m["shared"][2], m["x"])
        run = lambda rows, local, w: moe.experts_tokens(rows, local, w, m["table"], m["ws"])
        if exchange == "gathered":
            acc = moe_ep.routed_experts_gathered(m["x"], m["ids"], m["weights"], m["experts"], run, buffers=buffers, phases=phases)
        else:
            acc = moe_ep.routed_experts(m["x"], m["ids"], m["weights"], m["experts"], run, phases=phases)
        main.wait_stream(side)
        shared.record_stream(main)
        return moe.combine(m["ws"], shared, m["x"], m["w_gate"], acc=acc)

    buffers = None
    if world > 1 and exchange == "gathered":
        moe_ep.check_shard_table(m["experts"], m["hidden"], m["ids"].shape[1])
        buffers = moe_ep.GatheredExchange(m["x"].shape[0], m["hidden"], m["ids"].shape[1], m["x"].dtype, device)
    use_graph = graph and (world == 1 or exchange == "gathered")   # the counted exchange sizes its buffers on the host
    out = one_step()
    stream.synchronize()
    step = one_step
    if use_graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            out = one_step()
        step = g.replay
    sampler = ClockSampler(device.index or 0)
    device_ms = time_region(stream, step, steps, warmup, barrier=barrier, sampler=sampler)

    def e2e_step():
        for key in ("x", "ids", "weights"):
            m[key].copy_(m["host"][key], non_blocking=True)
        got = step()
        out_host.copy_(out if use_graph else got, non_blocking=True)

    e2e_ms = time_region(stream, e2e_step, steps, 1, barrier=barrier)
    # where a step's time goes on this rank (expert-parallel runs): events around the three parts of one more step
    split = None
    if world > 1:
        phases["events"] = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        one_step()
        torch.cuda.synchronize()
        ev = phases.pop("events")
        split = {"dispatch_ms": ev[0].elapsed_time(ev[1]), "experts_ms": ev[1].elapsed_time(ev[2]), "combine_ms": ev[2].elapsed_time(ev[3])}
    status = m["ws"].status()
    h2d = sum(t.numel() * t.element_size() for t in m["host"].values())
    return {"device_ms": device_ms, "e2e_ms": e2e_ms, "status": status, "flops": m["flops"], "hit": m["hit"], "weight_bytes": m["weight_bytes"],
            "h2d": h2d, "d2h": out_host.numel() * 2, "clocks": sampler.summary(), "graph": use_graph, "tokens": tokens, "split": split,
            "exchange": exchange}


def moe_line(r: dict, steps: int, warmup: int, world: int, peaks: dict) -> dict:
    ms = r["device_ms"] / steps
    value = r["flops"] / 1e12 / (ms * 1e-3)
    peak = peaks["bf16_tflops_sustained"] * world
    return {"metric": "moe_expert_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "trellis 2.5 bpw -> f16 x f16 -> f32", "data": "synthetic",
            "config": {"workload": f"configs[4]: MoE routed experts + shared expert + combine, {r['tokens']} tokens x top-10 of 512 experts, "
                                   f"hidden 2048, intermediate 768, 2.5 bpw trellis records, Zipf(1.1) routing; {r['hit']} experts hit, "
                                   f"{r['weight_bytes'] / 1e6:.0f} MB of expert records",
                       "cuda_graph": r["graph"], "l2": "inputs larger than L2",
                       "parallelism": "one GPU" if world == 1 else (
                           f"expert-parallel over {world} ranks, tokens split; NCCL all-gather of tokens, reduce-scatter of the integer sums, no host synchronisation"
                           if r.get("exchange") == "gathered" else
                           f"expert-parallel over {world} ranks, tokens split, counted NCCL all-to-all each way"),
                       **({"rank0_step_split": r["split"]} if r["split"] else {})},
            "e2e": {"value": r["flops"] / 1e12 / (r["e2e_ms"] / steps * 1e-3), "unit": "TFLOP/s", "h2d_bytes_per_step": r["h2d"],
                    "d2h_bytes_per_step": r["d2h"]},
            "gpu_launches": (11 if r["tokens"] > 8 else 10) * steps, "clocks": r["clocks"],   # count, scan, scatter, 2 rotations, 2 expert products, the fold (wide calls), 2 shared-expert products, combine
            "roofline": {"bound": "tensor", "achieved": value, "peak": peak, "unit": "TFLOP/s", "frac": value / peak,
                         "peak_source": f"{peaks['kind']} sustained BF16 cuBLAS rate per GPU (the experts multiply in FP16 with FP32 accumulation)",
                         "kernel": "moe_tc_gemm_kernel" if r["tokens"] > 64 else "moe_experts_kernel", "traffic": None,
                         "device_status": int(r["status"]),
                         "record_gbs": r["weight_bytes"] / (ms * 1e-3) / 1e9}}


def measure_prefill_sharded(stream, device, steps: int, warmup: int, rank: int, world: int, barrier, tokens: int = 8192) -> dict:
    """configs[2] N-sharded (column-wise over the weight rows, outputs stay sharded), two ways of
    getting the quantized operand to every rank: "replicated" - every rank quantizes all of x itself
    (no traffic, N times the quantizer work); "token_sharded" - every rank quantizes tokens / N rows
    and the ranks all-gather the operand's bytes (codes and scale tiles: 9/16 of a byte per value)
    over NCCL. Returns milliseconds per step of both, this rank's."""
    import torch
    import torch.distributed as dist

    from ignis_b200 import nvfp4

    gen = torch.Generator(device=device)
    items = []
    for idx, (n, k) in enumerate(((17408, 5120), (5120, 17408))):
        gen.manual_seed(20261128 + idx)                # the same x on every rank, this rank's rows of the weight
        x = torch.randn(tokens, k, device=device, generator=gen).to(torch.bfloat16)
        gen.manual_seed(20261228 + idx * 8 + rank)
        w = random_nvfp4(n // world, k, gen, device)
        ws = nvfp4.Workspace(nvfp4.workspace_bytes(w.n, k, nvfp4.ALLOW_A4, tokens), device)
        items.append((w, x, torch.empty(tokens, w.n, dtype=torch.bfloat16, device=device), ws))
    flops = sum(2.0 * tokens * w.n * w.k for w, _, _, _ in items) * world
    per = tokens // world

    def replicated() -> None:
        for w, x, y, ws in items:
            nvfp4.linear(x, w, out=y, policy=nvfp4.ALLOW_A4, workspace=ws)

    def token_sharded() -> None:
        for w, x, y, ws in items:
            nvfp4.quantize_operand(x[rank * per:(rank + 1) * per], tokens, rank * per, w.k, w.input_scale_divisor, ws)
            (c0, cb), (s0, sb) = nvfp4.operand_ranges(w.k, tokens, 0, per)
            dist.all_gather_into_tensor(ws.buffer[c0: c0 + cb * world], ws.buffer[c0 + rank * cb: c0 + (rank + 1) * cb])
            dist.all_gather_into_tensor(ws.buffer[s0: s0 + sb * world], ws.buffer[s0 + rank * sb: s0 + (rank + 1) * sb])
            nvfp4.linear_prequantized(w, tokens, ws, out=y)

    out = {"flops": flops, "tokens": tokens}
    for name, fn in (("replicated", replicated), ("token_sharded", token_sharded)):
        fn()
        stream.synchronize()
        if name == "token_sharded":   # same operand bytes either way: the second form must reproduce the first form's outputs
            replicated()
            want = [y.clone() for _, _, y, _ in items]
            fn()
            stream.synchronize()
            out["forms_agree"] = all(torch.equal(a, y) for a, (_, _, y, _) in zip(want, items))
        out[name] = time_region(stream, fn, steps, warmup, barrier=barrier) / steps
    out["status"] = max(ws.status() for _, _, _, ws in items)
    return out


# ---- the headline ----------------------------------------------------------------------------------------

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
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")   # plain peer stores beside NCCL: no multicast objects on the buffers
        dist.init_process_group("nccl", device_id=device)
    nvfp4.prepare()
    peaks = measured_peaks()
    tokens = args.tokens
    # How the matrices shard over N ranks: always column-wise (output rows) with no exchange inside a
    # product. "strong" (default): configs[1] itself is cut in N. "weak": every rank holds a full
    # configs[1] layer set - the shard of a layer N times as wide - so per-GPU work is fixed.
    split = world if args.scaling == "strong" else 1
    weights, host_inputs, inputs, outputs = build_workload(args.layers, rank, split, tokens, device)
    by_name = {name: (n, k, src) for name, n, k, src in LAYER}
    calls = GROUPS if args.group else [[name] for name, *_ in LAYER]
    mode = args.gather if world > 1 else 0
    # "a16" (the headline): BF16 activations as they are. "a4": the reference engine's default AllowA4
    # policy, under which these calls quantize their activations from 4 / 5 / 8 tokens (W4A4).
    policy = nvfp4.ALLOW_A4 if args.policy == "a4" and mode < 2 else nvfp4.A16_ONLY
    peer = None
    if mode == 1:
        from ignis_b200 import shard

        full = {name: torch.empty(tokens, outputs[name].shape[1] * world, dtype=torch.bfloat16, device=device) for name in outputs}
    if mode >= 2:
        from ignis_b200 import shard

        rejoined = ["o", "gate", "up", "down"]   # q | k | v feed attention heads that stay with their rank
        peer = shard.PeerOutputs({name: (tokens, outputs[name].shape[1] * world) for name in rejoined}, sets=2,
                                 points=["o", "gate_up", "down"])
    # the rejoin point a call's input comes from: its first instructions are that point's barrier
    rejoin_of = {"q": "down", "o": None, "gate": "o", "down": "gate_up"}

    def one_step(policy: int = policy) -> None:
        for li, layer in enumerate(weights):
            which = li & 1                       # a point's two buffers alternate by layer: see the reuse rule of the gather entry
            for names in calls:
                src = inputs[by_name[names[0]][2]]
                ws = [layer[nm] for nm in names]
                if mode == 3:
                    # the barrier rides in the product that reads a gathered buffer (no barrier launch)
                    point = rejoin_of[names[0]]
                    sync = peer.sync(point) if point else None
                    if names[0] == "q":
                        nvfp4.linear_group_gather(src, ws, [[outputs[nm].data_ptr()] for nm in names], [w.n for w in ws], [0] * len(ws), rejoin=sync)
                    else:
                        nvfp4.linear_group_gather(src, ws, [peer.pointers(nm, which) for nm in names], [w.n * world for w in ws],
                                                  [w.n * rank for w in ws], rejoin=sync)
                elif mode == 2 and names[0] != "q":
                    # every rank's epilogue stores its columns into all ranks' full-width buffers; a
                    # barrier launch behind it is all that is left of the all-gather
                    nvfp4.linear_group_scatter(src, ws, [peer.pointers(nm, which) for nm in names], [w.n * world for w in ws],
                                               [w.n * rank for w in ws])
                    peer.barrier()
                elif len(names) == 1:
                    nvfp4.linear(src, ws[0], out=outputs[names[0]], policy=policy)
                else:
                    nvfp4.linear_group(src, ws, outs=[outputs[nm] for nm in names], policy=policy)
                if mode == 1 and names[0] != "q":   # rejoin the column shards where a consumer needs the full width
                    for nm in names:
                        shard.gather_columns(outputs[nm], out=full[nm])

    if mode == 3 and not args.group:
        raise SystemExit("--gather 3 needs --group 1 (the rejoin points are those of the grouped call list)")
    rejoin_calls = sum(1 for names in calls if names[0] != "q")
    launches_per_step = len(calls) * args.layers + (rejoin_calls * args.layers if mode == 2 else 0)
    stream = torch.cuda.Stream()
    extras = {}
    with torch.cuda.stream(stream):
        use_graph = bool(args.graph) and mode != 1   # NCCL collectives run outside a graph here
        step = graphed(stream, one_step, use_graph)

        def barrier() -> None:
            if world > 1:
                dist.barrier()

        clocks = ClockSampler(local_rank)
        device_ms = time_region(stream, step, args.steps, args.warmup, barrier=barrier, sampler=clocks)

        # end to end: host activations in, last output back, every step
        result_src = peer.views[("down", (args.layers - 1) & 1)] if mode >= 2 else outputs["down"]
        result_host = torch.empty_like(result_src, device="cpu").pin_memory()

        def e2e_step() -> None:
            for key in inputs:
                inputs[key].copy_(host_inputs[key], non_blocking=True)
            step()
            result_host.copy_(result_src, non_blocking=True)

        e2e_ms = time_region(stream, e2e_step, args.steps, 2, barrier=barrier)
        missing = peer.missing() if peer is not None else 0

        if world == 1 and args.extras:
            # the same step under the reference engine's default policy, timed the same way, reported beside
            # the headline (never instead of it)
            if policy == nvfp4.A16_ONLY and args.graph and tokens >= 4:
                a4_step = graphed(stream, lambda: one_step(nvfp4.ALLOW_A4))
                a4_ms = time_region(stream, a4_step, args.steps, args.warmup) / args.steps
                extras["allow_a4_ms"] = a4_ms
            side_steps, side_warmup = max(3, min(args.steps, 10)), 3
            extras["config0"] = measure_config0(stream, device, weights, side_steps, side_warmup, peaks)
            del weights, step
            torch.cuda.empty_cache()
            fp4 = measure_fp4_peak(stream, device)
            extras["fp4_peak"] = fp4
            extras["config2"] = measure_prefill(stream, device, side_steps, side_warmup, peaks, fp4)
            extras["config2"]["mlp"] = {k: v for k, v in measure_prefill(stream, device, side_steps, side_warmup, peaks, fp4, form="mlp").items()
                                        if k in ("value", "unit", "ms_per_step", "roofline", "config", "gpu_launches")}
            torch.cuda.empty_cache()
            extras["config3"] = measure_trellis(stream, device, side_steps, side_warmup, peaks, tokens=8)
            m1 = measure_trellis(stream, device, side_steps, side_warmup, peaks, tokens=1)
            extras["config3"]["m1"] = {k: m1[k] for k in ("value", "unit", "ms_per_step", "roofline", "gpu_launches")}
            torch.cuda.empty_cache()
            pf = measure_trellis_prefill(stream, device, side_steps, side_warmup, peaks)
            extras["config3"]["prefill_m1024"] = {k: pf[k] for k in ("metric", "value", "unit", "ms_per_step", "roofline", "config", "gpu_launches")}
            torch.cuda.empty_cache()
            extras["config4"] = moe_line(measure_moe(stream, device, side_steps, side_warmup, peaks), side_steps, side_warmup, 1, peaks)
        elif world > 1 and args.extras:
            del weights, step
            torch.cuda.empty_cache()
            side_steps, side_warmup = max(3, min(args.steps, 10)), 3
            extras["prefill"] = measure_prefill_sharded(stream, device, side_steps, side_warmup, rank, world, barrier)
            torch.cuda.empty_cache()
            extras["moe"] = measure_moe(stream, device, side_steps, side_warmup, peaks, rank=rank, world=world, barrier=barrier)

    # max over ranks of every device time
    names, values = ["device_ms", "e2e_ms", "missing"], [device_ms, e2e_ms, float(missing)]
    if world > 1 and args.extras:
        names += ["pf_replicated", "pf_token_sharded", "pf_status", "moe_device_ms", "moe_e2e_ms", "moe_status"]
        values += [extras["prefill"]["replicated"], extras["prefill"]["token_sharded"], float(extras["prefill"]["status"]),
                   extras["moe"]["device_ms"], extras["moe"]["e2e_ms"], float(extras["moe"]["status"])]
    times = torch.tensor(values, dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.destroy_process_group()
    got = dict(zip(names, times.tolist()))
    if rank != 0:
        return

    per_rank_bytes = layer_algorithmic_bytes(tokens, split) * args.layers
    job_bytes = per_rank_bytes * world
    ms_per_step = got["device_ms"] / args.steps
    value = job_bytes / (ms_per_step * 1e-3) / 1e9
    e2e_value = job_bytes / (got["e2e_ms"] / args.steps * 1e-3) / 1e9
    per_gpu = value / world
    collective = {0: "none (outputs stay sharded)",
                  1: "NCCL all-gather of every rejoined output (o, gate, up, down)",
                  2: "fused: epilogues store into every rank's buffer over NVLink, one device barrier launch per rejoined call",
                  3: "fused, no barrier launch: epilogues store into every rank's buffer over NVLink (plain peer stores); the barrier "
                     "between the ranks rides in the first instructions of the product that reads the gathered buffer; rejoined after o, "
                     "gate|up and down, two buffers per point alternating by layer"}[mode]
    # dram bytes per launch of the dominant kernel, from the ncu capture of this exact configuration
    # (8 tokens, A16, grouped calls, one GPU): 196.97 MB per layer of four launches
    profiled = world == 1 and tokens == 8 and args.group == 1 and policy == nvfp4.A16_ONLY
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling if world > 1 else "strong", "vs_baseline": None,
        "dtype": DTYPE, "data": "synthetic",
        "config": {"workload": "configs[1]: NVFP4 decode, 8 lanes (M=8), 27B-style dense layer (q,k,v,o,gate,up,down), hidden 5120",
                   "layers": args.layers, "tokens": tokens,
                   "policy": "AllowA4 (activations quantized to NVFP4 inside the product, W4A4 on tcgen05)" if policy == nvfp4.ALLOW_A4 else "A16",
                   "device_status": nvfp4.device_status(), "sharding": (f"column-wise over N, {world} rank(s); " +
                                ("every rank holds configs[1]-sized shards of a layer N times as wide (per-GPU work fixed)"
                                 if split == 1 and world > 1 else "configs[1] itself cut in N (total work fixed)")),
                   "calls_per_layer": len(calls), "cuda_graph": use_graph,
                   "l2": "inputs larger than L2: %.2f GB of distinct weights per rank per step" % (per_rank_bytes / 1e9),
                   "collective": collective, **({"ranks_missing_from_a_wait": int(got["missing"])} if mode >= 2 else {})},
        "e2e": {"value": e2e_value, "unit": UNIT,
                "h2d_bytes_per_step": sum(t.numel() * 2 for t in host_inputs.values()),
                "d2h_bytes_per_step": result_host.numel() * 2},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": per_gpu / peaks["hbm_gbs"],
                     "peak_source": f"{peaks['kind']} copy bandwidth", "frac_of_nominal_8000": per_gpu / 8000.0,
                     "kernel": "nvfp4_gemv_kernel<1>", "bytes_per_launch": per_rank_bytes / (len(calls) * args.layers),
                     "us_per_launch": ms_per_step * 1e3 / (len(calls) * args.layers),
                     "traffic": 196.08e6 / 4 if profiled else None,   # profiles/nvfp4_gemv_decode_m8.md: read + write of the four launches
                     "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, mean of one layer's four launches" if profiled else None},
    }
    if "allow_a4_ms" in extras:
        a4_ms = extras.pop("allow_a4_ms")
        a4_value = job_bytes / (a4_ms * 1e-3) / 1e9
        line["allow_a4"] = {"policy": "the reference engine's default AllowA4: activations quantized to NVFP4 inside each product "
                                      "(from 4 / 5 / 8 tokens by problem), W4A4 on tcgen05, weights from HBM to the tensor cores by TMA",
                            "value": a4_value, "unit": UNIT, "ms_per_step": a4_ms, "frac": a4_value / peaks["hbm_gbs"],
                            "kernel": "w4a4_decode_kernel", "us_per_launch": a4_ms * 1e3 / launches_per_step}
    if world == 1:
        line.update(extras)
    elif args.extras:
        pf = extras["prefill"]
        best = min(got["pf_replicated"], got["pf_token_sharded"])
        line["config2"] = {"metric": "nvfp4_prefill_gemm_tflops", "unit": "TFLOP/s", "value": pf["flops"] / 1e12 / (best * 1e-3),
                           "ms_per_step": best,
                           "replicated_quantizer": {"ms_per_step": got["pf_replicated"], "value": pf["flops"] / 1e12 / (got["pf_replicated"] * 1e-3)},
                           "token_sharded_quantizer_nccl_all_gather": {"ms_per_step": got["pf_token_sharded"],
                                                                       "value": pf["flops"] / 1e12 / (got["pf_token_sharded"] * 1e-3)},
                           "forms_agree_bit_for_bit": pf.get("forms_agree"), "device_status": int(got["pf_status"]),
                           "config": {"workload": f"configs[2] N-sharded: M={pf['tokens']}, up 5120->17408 and down 17408->5120 cut column-wise "
                                                  f"over {world} ranks, outputs stay sharded; value = whole-job FLOPs over the slowest rank's time"}}
        mo = dict(extras["moe"])
        mo["device_ms"], mo["e2e_ms"], mo["status"] = got["moe_device_ms"], got["moe_e2e_ms"], got["moe_status"]
        side_steps = max(3, min(args.steps, 10))
        line["config4"] = moe_line(mo, side_steps, 3, world, peaks)
    if world == 1 and not args.no_cpu_baseline:
        v, desc = cpu_sample()
        line["cpu_baseline"] = {"value": v, "unit": UNIT, **desc}
    emit(line)


def measure_timeline(stream, device, layers: int, tokens: int, policy_name: str) -> dict:
    """Where a decode launch's time goes, from the phase stamps of the trace build of the library
    (`python -m ignis_b200.build --trace`): the step is `layers` layers of configs[1] replayed as one
    CUDA graph; per call of a layer, medians over the steady-state layers of
      gap      predecessor's last CTA through its K reduction -> this grid's first CTA sees it complete
      rewrite  -> activations rewritten as fragments (median CTA; `rewrite_split_us`: per CTA, its first pass over
               the slice, the conversion and stores, the wait for the CTA's other warps)
      loop     -> K loop done (median CTA)
      straggle -> K loop done in the last CTA
      finish   -> last CTA through the cluster's meeting point (the epilogue's stores follow)
    all in microseconds. The stamps cost a little: the step runs about 1 % slower than the shipped one."""
    import ctypes as C

    import numpy as np
    import torch

    from ignis_b200 import _lib, nvfp4

    lib = _lib.load()
    if not hasattr(lib, "b200q_debug_gemv_trace"):
        raise SystemExit("the timeline needs the trace build: python -m ignis_b200.build --trace")
    weights, _, inputs, outputs = build_workload(layers, 0, 1, tokens, device)
    by_name = {name: (n, k, src) for name, n, k, src in LAYER}
    policy = nvfp4.ALLOW_A4 if policy_name == "a4" else nvfp4.A16_ONLY
    if policy != nvfp4.A16_ONLY:
        raise SystemExit("the phase stamps sit in the A16 decode kernel")

    def one_step() -> None:
        for layer in weights:
            for names in GROUPS:
                src = inputs[by_name[names[0]][2]]
                ws = [layer[nm] for nm in names]
                if len(names) == 1:
                    nvfp4.linear(src, ws[0], out=outputs[names[0]], policy=policy)
                else:
                    nvfp4.linear_group(src, ws, outs=[outputs[nm] for nm in names], policy=policy)

    step = graphed(stream, one_step, True)
    for _ in range(3):
        step()
    stream.synchronize()
    stamps = np.zeros((128, 512, 10), np.uint64)
    lib.b200q_debug_gemv_trace.restype = C.c_int32
    lib.b200q_debug_gemv_trace.argtypes = [C.c_void_p, C.c_uint64]
    assert lib.b200q_debug_gemv_trace(stamps.ctypes.data, stamps.nbytes) == 0      # drop the warm-up's stamps
    ms = time_region(stream, step, 1, 0)
    assert lib.b200q_debug_gemv_trace(stamps.ctypes.data, stamps.nbytes) == 0
    launches = []
    for slot in range(stamps.shape[0]):
        grid = int(stamps[slot, 0, 7] >> np.uint64(32))
        if grid:
            t = stamps[slot, :min(grid, 512), :].astype(np.int64)
            launches.append((int(t[:, 0].min()), grid, t))
    launches.sort(key=lambda e: e[0])
    if len(launches) != layers * len(GROUPS):
        raise SystemExit(f"expected {layers * len(GROUPS)} stamped launches, found {len(launches)}")
    rows = {i: [] for i in range(len(GROUPS))}
    prev_end = None
    for idx, (_, grid, t) in enumerate(launches):
        if prev_end is not None and idx >= 2 * len(GROUPS):     # the first two layers run behind a cold start
            ready, looped = np.median(t[:, 3]), np.median(t[:, 4])
            rows[idx % len(GROUPS)].append([(t[:, 2].min() - prev_end) / 1e3, (ready - t[:, 2].min()) / 1e3, (looped - ready) / 1e3,
                                            (t[:, 4].max() - looped) / 1e3, (t[:, 6].max() - t[:, 4].max()) / 1e3,
                                            (t[:, 6].max() - prev_end) / 1e3, float(np.mean(t[:, 0] < prev_end - 1000)), grid,
                                            np.median(t[:, 8] - t[:, 2]) / 1e3, np.median(t[:, 9] - t[:, 8]) / 1e3, np.median(t[:, 3] - t[:, 9]) / 1e3])
        prev_end = t[:, 6].max()
    calls = {}
    for i, names in enumerate(GROUPS):
        m = np.mean(np.array(rows[i]), axis=0)
        nbytes = sum(weight_bytes(by_name[nm][0], by_name[nm][1]) for nm in names)
        calls["|".join(names)] = {"ctas": int(m[7]), "weight_mb": nbytes / 1e6, "gap_us": m[0], "rewrite_us": m[1], "loop_us": m[2],
                                  "straggle_us": m[3], "finish_us": m[4], "total_us": m[5], "ctas_resident_early": m[6],
                                  "rewrite_split_us": {"maximum_pass": m[8], "convert_and_store": m[9], "cta_barrier": m[10]},
                                  "loop_gbs": nbytes / (m[2] * 1e-6) / 1e9, "call_gbs": nbytes / (m[5] * 1e-6) / 1e9}
    layer_us = sum(c["total_us"] for c in calls.values())
    return {"metric": "nvfp4_decode_layer_timeline_us", "value": layer_us, "unit": "us", "steps": 1, "warmup": 3, "ms_per_step": ms,
            "higher_is_better": False, "dtype": DTYPE,
            "config": {"workload": f"configs[1] decode chain, {layers} layers x {len(GROUPS)} calls, {tokens} tokens, one CUDA graph; "
                                   "phase stamps of the trace build", "l2": "weights larger than L2"},
            "calls": calls,
            "share": {k: sum(c[k] for c in calls.values()) / layer_us for k in ("gap_us", "rewrite_us", "loop_us", "straggle_us", "finish_us")}}


def run_side_workload(args) -> None:
    """`--workload X`: one of the other configs alone, one JSON line, same timing rules as the headline."""
    import torch
    import torch.distributed as dist

    from ignis_b200 import _lib, nvfp4, trellis

    if args.workload == "timeline":     # the library with the phase stamps compiled in stands in for the shipped one
        trace_lib = os.path.join(ROOT, "ignis_b200", "libignis_b200_trace.so")
        if not os.path.exists(trace_lib):
            raise SystemExit("the timeline needs the trace build: python -m ignis_b200.build --trace")
        _lib.LIB_PATH = trace_lib

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=device)
    nvfp4.prepare()
    trellis.prepare()
    peaks = measured_peaks()
    stream = torch.cuda.Stream()
    graph = bool(args.graph)
    base = {"n_gpus": world, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "data": "synthetic"}

    def barrier() -> None:
        if world > 1:
            dist.barrier()

    with torch.cuda.stream(stream):
        if args.workload == "moe":
            r = measure_moe(stream, device, args.steps, args.warmup, peaks, tokens=args.moe_tokens, rank=rank, world=world, graph=graph,
                            barrier=barrier, exchange=args.exchange)
            t = torch.tensor([r["device_ms"], r["e2e_ms"], float(r["status"])], dtype=torch.float64, device=device)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                dist.destroy_process_group()
            r["device_ms"], r["e2e_ms"], r["status"] = t.tolist()
            line = moe_line(r, args.steps, args.warmup, world, peaks)
        elif args.workload == "prefill":
            fp4 = measure_fp4_peak(stream, device) if args.peak else None
            form = "a16" if args.a16 else ("mlp" if args.mlp else "linear")
            line = {**base, **measure_prefill(stream, device, args.steps, args.warmup, peaks, fp4, tokens=args.tokens if args.tokens > 8 else 8192,
                                              form=form, graph=graph)}
            if fp4 is not None:
                line["fp4_peak"] = fp4
        elif args.workload == "peak":
            fp4 = measure_fp4_peak(stream, device, seconds=args.peak_seconds)
            line = {**base, "metric": "fp4_mma_peak_tflops", "value": fp4["burst_tflops"], "unit": "TFLOP/s", "steps": 0, "warmup": 0,
                    "ms_per_step": None, "dtype": "e2m1 x e2m1 (ue4m3 block scales) -> f32", "config": {"workload": fp4["how"]}, "fp4_peak": fp4}
        elif args.workload == "timeline":
            line = {**base, **measure_timeline(stream, device, min(args.layers, 24), args.tokens, args.policy)}
        elif args.workload == "config0":
            weights, _, _, _ = build_workload(args.layers, 0, 1, 1, device)
            line = {**base, **measure_config0(stream, device, weights, args.steps, args.warmup, peaks, graph=graph)}
        elif args.workload == "trellis" and args.tokens > 64:
            line = {**base, **measure_trellis_prefill(stream, device, args.steps, args.warmup, peaks, layers=min(args.layers, 8), tokens=args.tokens,
                                                      graph=graph)}
        elif args.workload == "head":
            line = {**base, **measure_head(stream, device, args.steps, args.warmup, peaks, args.tokens, graph=graph)}
        else:
            line = {**base, **measure_trellis(stream, device, args.steps, args.warmup, peaks, layers=args.layers, tokens=args.tokens,
                                              group=bool(args.group), graph=graph)}
    if rank == 0:
        emit(line)


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
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"],
                    help="decode workload under torchrun: strong = configs[1] cut in N (default), weak = per-GPU work fixed")
    ap.add_argument("--gather", type=int, default=3,
                    help="decode workload under torchrun, how rejoined outputs reach every rank: 3 peer stores + the barrier folded into "
                         "the consuming product (default), 2 peer stores + a barrier launch, 1 NCCL all-gather, 0 outputs stay sharded")
    ap.add_argument("--moe-tokens", type=int, default=4096, help="tokens of the --workload moe step (configs[4]: 4096; up to 8 takes the decode entry's item size)")
    ap.add_argument("--exchange", choices=["gathered", "compact"], default="gathered",
                    help="with --workload moe on N > 1 GPUs: the fixed-size all-gather / reduce-scatter exchange, or the counted all-to-all")
    ap.add_argument("--policy", choices=["a16", "a4"], default="a16",
                    help="decode workload: a16 (headline) or a4, the reference's AllowA4 policy (W4A4 from 4 / 5 / 8 tokens)")
    ap.add_argument("--a16", type=int, default=0, help="with --workload prefill: 1 runs the two products under the A16 policy")
    ap.add_argument("--mlp", type=int, default=0, help="with --workload prefill: 1 runs the fused MLP entry instead of two plain products")
    ap.add_argument("--peak", type=int, default=1, help="with --workload prefill: 0 skips the FP4 peak loop (the denominator falls back to 4 x BF16)")
    ap.add_argument("--peak-seconds", type=float, default=6.0, help="with --workload peak: seconds of back-to-back launches per issue form")
    ap.add_argument("--extras", type=int, default=1, help="0: the headline alone (no config0 / config2 / config3 / config4 objects)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="decode", choices=["decode", "config0", "prefill", "trellis", "moe", "head", "peak", "timeline"],
                    help="decode: configs[1] (the headline, with the other configs as objects); config0 / prefill / trellis / moe: "
                         "configs[0] / [2] / [3] / [4] alone; head: the output head; peak: the FP4 tensor-core loop; timeline: where a decode "
                         "launch's time goes (needs python -m ignis_b200.build --trace)")
    args = ap.parse_args()
    claim_stdout()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload != "decode":
        run_side_workload(args)
    else:
        run_cuda_arm(args)


if __name__ == "__main__":
    main()
