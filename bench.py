"""Benchmark of the quantized-linear forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload "c2": the large-codebook VQ linear — in 4096, out 14336, vector length 8, 65536 x 8
fp16 main codebook with uint16 indices, 256-entry residual codebook with uint8 indices, fp16
per-output-row scale; bf16 N(0,1) activations with 1, 2, 16, 128, 384 and 2048 rows.  One STEP
is one forward at each of the six row counts (2579 rows, "tokens") through ``NPVQLinear``.
Everything is synthetic and seeded (no dataset, no checkpoint).

Reported on ONE JSON line by rank 0:
  value      tokens/s over the whole job, inputs resident in HBM, timed with CUDA events
             around exactly K steps, max over ranks.
  e2e        the same steps driven from pinned HOST activations: host->device copy of every
             input and device->host copy of every output inside the timed region.
  bands      per row count: mean device time, GB/s on the packed weight bytes, TFLOP/s.
  roofline   the kernel that takes most of the step (the dense tcgen05 GEMM at 2048 rows):
             2*M*N*K flops / mean launch duration, against the measured dense bf16 peak.
  cpu_baseline  the CPU restatement of the reference's decode + matmul path, timed on this
             machine's host cores on a bounded sample of the same workload (rank 0, N=1 only).

Cold L2: the layer exists in 12 copies (264 MB of index data, L2 is 126 MB) and every forward
uses the next copy, so no forward finds its weights in L2.

N > 1 (torchrun, one process per GPU): the layer's output rows are sharded N ways, each rank
runs the same bands on its shard and the outputs are all-gathered with NCCL — total work is
fixed ("strong" scaling).

``--impl reference`` times the reference algorithm's CPU path (oracle port, all host threads)
on the same metric; each step is a bounded sample (rows 1 and 16).
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "quant-linear GEMV HBM GB/s & GEMM TFLOPS vs B200 peak; tokens/s at 1-8 GPUs"
N_OUT, K_IN = 14336, 4096
ROWS = (1, 2, 16, 128, 384, 2048)
N_COPIES = 12
REF_ROWS = (1, 16)


def load_peaks() -> tuple[dict, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        return json.loads(p.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# --------------------------------------------------------------------------- clocks ---
class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons every 200 ms while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index = index
        self.samples: list[list[str]] = []
        self._stop = threading.Event()
        self._ready = threading.Event()  # set once the first sample is in (or sampling failed)
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run_nvml(self) -> bool:
        """Read-only NVML polling (every 5 ms): clocks and clock-event reasons."""
        try:
            import pynvml as nv

            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            bits = {
                "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            }
            get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                nv.nvmlDeviceGetCurrentClocksThrottleReasons
        except Exception:
            return False
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        while True:
            try:
                sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                mask = get_reasons(h)
                self.samples.append([str(sm), str(mx), ""] +
                                    ["Active" if mask & bits[n] else "Not Active" for n in names])
            except Exception:
                pass
            self._ready.set()
            if self._stop.wait(0.002):
                break
        return True

    def _run(self) -> None:
        if self._run_nvml():
            return
        while not self._stop.is_set():
            self._ready.set()
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                     "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                if out.returncode == 0 and out.stdout.strip():
                    self.samples.append([c.strip() for c in out.stdout.strip().split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread.start()
        self._ready.wait(timeout=10)  # NVML start-up must not eat a short timed region
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- ours ---
def build_layers(device, rank: int, world: int):
    """N_COPIES copies (different seeds) of the layer, this rank's rows only."""
    from neuropress_b200.nn import NPVQLinear, VQProxy
    from neuropress_b200.sharding import ShardedLinear
    from synthetic import make_c2_layer

    layers = []
    packed_bytes = 0
    for c in range(N_COPIES):
        d = make_c2_layer(seed=c)
        packed_bytes = d.packed_bytes()
        full = NPVQLinear(VQProxy(d.centroids), d.packed, d.bits, d.out_features, d.in_features,
                          d.vector_len, backend="auto", residual_proxy=VQProxy(d.residual_centroids),
                          residual_indices=d.residual_indices, residual_bits=d.residual_bits,
                          row_scale=d.row_scale)
        if world > 1:
            layer = ShardedLinear.from_layer(full, rank, world)
            layer.local.proxy.to(device)
            layer.local.residual_proxy.to(device)
        else:
            layer = full
            layer.proxy.to(device)
            layer.residual_proxy.to(device)
        layers.append(layer.to(device))
        del full, d
    return layers, packed_bytes


class KernelTimer:
    """Launch observer: one CUDA event pair per C-ABI launch, keyed by (symbol, rows)."""

    def __init__(self) -> None:
        self.rows = 0
        self.pairs: dict[tuple[str, int], list] = {}
        self._open = None

    def __call__(self, symbol: str, begin: bool) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        if begin:
            self._open = ev
        else:
            self.pairs.setdefault((symbol, self.rows), []).append((self._open, ev))

    def mean_ms(self) -> dict[tuple[str, int], float]:
        return {k: sum(a.elapsed_time(b) for a, b in v) / len(v) for k, v in self.pairs.items()}


def run_ours(args) -> dict:
    import torch.distributed as dist

    from neuropress_b200 import kernels
    from synthetic import make_activations

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun for N > 1")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL prints its version banner on stdout at the first collective; stdout carries
        # exactly one JSON line, so stdout is pointed at stderr until the group is up.
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=device)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)

    layers, packed_bytes = build_layers(device, rank, world)
    gather_kind = "none"
    if world > 1:
        # Run every band once on the local shard first: module loading and one-time kernel
        # attributes then never fall inside a rank's bounded wait for its peers.
        for m in ROWS:
            layers[0].local(make_activations(m, K_IN, torch.bfloat16, seed=m).to(device))
        torch.cuda.synchronize()
        dist.barrier()
        gather_kind = "NCCL all-gather + re-layout copy"
        if not args.nccl_gather:
            try:
                from neuropress_b200.sharding import PushGather

                shared = PushGather(None, max(ROWS), N_OUT, torch.bfloat16, device)
                for layer in layers:
                    layer.push = shared
                gather_kind = "peer-store all-gather fused into the kernels (npb_gemm_allgather, npb_vq_gemv_allgather)"
            except Exception as exc:  # symmetric memory unavailable: keep NCCL
                print(f"[bench] push gather unavailable ({exc!r}); using NCCL", file=sys.stderr)
    xs_host = {m: make_activations(m, K_IN, torch.bfloat16, seed=m).pin_memory() for m in ROWS}
    xs = {m: xs_host[m].to(device) for m in ROWS}
    ys_host = {m: torch.empty((m, N_OUT), dtype=torch.bfloat16).pin_memory() for m in ROWS}
    tokens_per_step = sum(ROWS)
    counter = {"i": 0, "launches": 0}
    timer = KernelTimer()

    def count_hook(symbol, begin):
        if begin:
            counter["launches"] += 1
        timer(symbol, begin)

    # End-to-end steps move every input from pinned host memory and every output back to it.
    # The copies run on their own streams (one per direction) so that PCIe transfers overlap
    # the kernels of the neighbouring forwards; events order copy -> forward -> copy.
    h2d, d2h = torch.cuda.Stream(), torch.cuda.Stream()
    x_stage = {m: torch.empty_like(xs[m]) for m in ROWS}
    ev_in = {m: torch.cuda.Event() for m in ROWS}
    ev_used = {m: torch.cuda.Event() for m in ROWS}
    for m in ROWS:
        ev_used[m].record()

    def step(from_host: bool) -> None:
        cur = torch.cuda.current_stream()
        if from_host:
            with torch.cuda.stream(h2d):
                for m in ROWS:
                    h2d.wait_event(ev_used[m])  # last step's forward has consumed the buffer
                    x_stage[m].copy_(xs_host[m], non_blocking=True)
                    ev_in[m].record(h2d)
        for m in ROWS:
            layer = layers[counter["i"] % N_COPIES]
            counter["i"] += 1
            timer.rows = m
            if not from_host:
                layer(xs[m])
                continue
            cur.wait_event(ev_in[m])
            y = layer(x_stage[m])
            ev_used[m].record(cur)
            if world > 1:
                y = y.clone()  # the all-gather buffers are reused two calls later
            done = torch.cuda.Event()
            done.record(cur)
            d2h.wait_event(done)
            with torch.cuda.stream(d2h):
                ys_host[m].copy_(y, non_blocking=True)
            y.record_stream(d2h)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(from_host: bool, steps: int) -> float:
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            step(from_host)
        torch.cuda.current_stream().wait_stream(d2h)  # every output is on the host before t1
        t1.record()
        barrier()
        ms = torch.tensor([t0.elapsed_time(t1)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(args.warmup, 3)):
        step(False)
    step(True)
    barrier()

    # ---- CUDA graphs of the step.  A step rotates through half of the weight copies, so two
    # graphs (one per half) replayed alternately reproduce the eager sequence exactly; each
    # holds the six module forwards of one step (and, for N > 1, their six push all-gathers).
    graphs = None
    if not args.eager and N_COPIES == 2 * len(ROWS) and (world == 1 or gather_kind.startswith("peer-store")):
        graphs, keep = [], []
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for phase in range(2):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for j, m in enumerate(ROWS):
                        keep.append(layers[phase * len(ROWS) + j](xs[m]))
                graphs.append(g)
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(3):
            for g in graphs:
                g.replay()
        barrier()

    def timed_graph(steps: int) -> float:
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for s_ in range(steps):
            graphs[s_ & 1].replay()
        t1.record()
        barrier()
        ms = torch.tensor([t0.elapsed_time(t1)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # ---- timed regions: K steps with device-resident inputs (graph replay when available),
    # K eager steps with one CUDA-event pair per launch (kernel durations for the rooflines),
    # K end-to-end steps from / to pinned host memory.
    with ClockSampler(local_rank) as clocks:
        graph_ms = timed_graph(args.steps) if graphs else None
        counter["i"] = 0
        kernels.set_launch_hook(count_hook)
        eager_ms = timed(False, args.steps)
        launches = counter["launches"]
        kernels.set_launch_hook(None)
        e2e_ms = timed(True, args.steps)
    total_ms = graph_ms if graph_ms is not None else eager_ms
    kmean = timer.mean_ms()

    peaks, peak_src = load_peaks()
    n_local = N_OUT // world
    bands = {}
    for m in ROWS:
        ms = sum(v for (sym, r), v in kmean.items() if r == m)
        bands[str(m)] = {
            "ms": round(ms, 5),
            "kernels": {sym: round(v, 5) for (sym, r), v in kmean.items() if r == m},
            "packed_GBps": round(packed_bytes / world / (ms * 1e-3) / 1e9, 1),
            "TFLOPs": round(2.0 * m * n_local * K_IN / (ms * 1e-3) / 1e12, 2),
        }
    # Time per step by C-ABI entry point; the one with the largest share gets `roofline`.
    share: dict[str, float] = {}
    for (sym, r), v in kmean.items():
        share[sym] = share.get(sym, 0.0) + v
    dominant = max(share, key=share.get) if share else None
    gemm_ms = kmean.get(("npb_gemm", 2048))
    gemm_roofline = None
    if gemm_ms:
        achieved = 2.0 * 2048 * n_local * K_IN / (gemm_ms * 1e-3) / 1e12
        gemm_roofline = {"bound": "tensor", "kernel": "gemm_kernel (tcgen05, dense B) at 2048 rows",
                         "achieved": round(achieved, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": round(achieved / peaks["bf16_tflops"], 4), "traffic": 170.9e6,
                         "peak_source": f"{peak_src} burst cuBLAS bf16", "launch_ms": round(gemm_ms, 5),
                         "share_of_step": round(gemm_ms / sum(share.values()), 3)}
    dec = [v for (sym, r), v in kmean.items() if sym == "npb_vq_decode"]
    decode_roofline = None
    if dec:
        dec_ms = sum(dec) / len(dec)
        dec_bytes = packed_bytes / world + n_local * K_IN * 2  # packed in + dense bf16 weight out
        gbs = dec_bytes / (dec_ms * 1e-3) / 1e9
        decode_roofline = {"bound": "hbm", "kernel": "vq_decode_kernel (one-pass decode, bf16 out)",
                           "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                           "frac": round(gbs / peaks["hbm_gbs"], 4),
                           # dram__bytes_read + write of one launch (ncu); the rest of the output is
                           # still dirty in L2 when the kernel ends
                           "traffic": 83.3e6 / world, "algorithmic_bytes": dec_bytes,
                           "peak_source": f"{peak_src} copy bandwidth", "launch_ms": round(dec_ms, 5),
                           "launches_per_step": len(dec),
                           "share_of_step": round(share["npb_vq_decode"] / sum(share.values()), 3)}
    roofline = decode_roofline if dominant == "npb_vq_decode" else gemm_roofline
    # The 1-row forward alone from a CUDA graph: its event-pair time above includes the host's
    # enqueue latency, which a kernel this short does not hide.
    gemv_graph_ms = None
    if world == 1 and not args.eager:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                g1 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g1, stream=side):
                    for c in range(N_COPIES):
                        layers[c](xs[1])
                g1.replay()
                side.synchronize()
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record(side)
                g1.replay()
                t1.record(side)
                side.synchronize()
            gemv_graph_ms = t0.elapsed_time(t1) / N_COPIES
        except Exception as exc:  # measurement aid only
            print(f"[bench] 1-row graph timing skipped ({exc!r})", file=sys.stderr)
    gemv_ms = kmean.get(("npb_vq_gemv", 1))
    gemv = None
    if gemv_ms:
        gbs = packed_bytes / world / (gemv_ms * 1e-3) / 1e9
        gemv = {"bound": "hbm", "kernel": "npb_vq_gemv at 1 row (vq_gemv_mma_kernel)", "achieved": round(gbs, 1),
                "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(gbs / peaks["hbm_gbs"], 4),
                "launch_ms": round(gemv_ms, 5)}
        if gemv_graph_ms:
            gemv["graph_ms"] = round(gemv_graph_ms, 5)
            gemv["graph_achieved"] = round(packed_bytes / (gemv_graph_ms * 1e-3) / 1e9, 1)
            gemv["graph_frac"] = round(gemv["graph_achieved"] / peaks["hbm_gbs"], 4)

    line = {
        "metric": METRIC, "value": round(tokens_per_step * args.steps / (total_ms * 1e-3), 1),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(total_ms / args.steps, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "c2: VQ linear 4096->14336, VL8, 65536-entry fp16 codebook (uint16 idx) "
                               "+ 256-entry residual (uint8 idx) + fp16 row scale; bf16 rows "
                               + "/".join(map(str, ROWS)),
                   "tokens_per_step": tokens_per_step,
                   "l2": f"cold: {N_COPIES} weight copies ({N_COPIES * packed_bytes / 1e6:.0f} MB) rotated per forward",
                   "parallelism": "single GPU" if world == 1 else f"out-feature shards x{world} + {gather_kind}",
                   "launch": ("CUDA-graph replay of the module forwards (two graphs, one per half of the "
                              "weight copies)") if graphs else "eager module forwards"},
        "eager_ms_per_step": round(eager_ms / args.steps, 4),
        "e2e": {"value": round(tokens_per_step * args.steps / (e2e_ms * 1e-3), 1), "unit": "tokens/s",
                "h2d_bytes_per_step": tokens_per_step * K_IN * 2,
                "d2h_bytes_per_step": tokens_per_step * N_OUT * 2,
                "ms_per_step": round(e2e_ms / args.steps, 4)},
        "gpu_launches": launches,
        "clocks": clocks.summary(),
        "roofline": roofline, "gemm_roofline": gemm_roofline, "decode_roofline": decode_roofline,
        "gemv_roofline": gemv, "bands": bands,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(budget_s=20.0)
    if world > 1:
        dist.destroy_process_group()
    return line if rank == 0 else {}


# --------------------------------------------------------------------------- CPU ---
def _cpu_layer():
    from synthetic import make_activations, make_c2_layer

    d = make_c2_layer(seed=0)
    xs = {m: make_activations(m, K_IN, torch.bfloat16, seed=m) for m in REF_ROWS}
    return d, xs


def _cpu_step(d, xs) -> int:
    """One bounded sample: the reference's decode-every-call forward at 1 and 16 rows."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import oracle

    for m, x in xs.items():
        oracle.vq_forward(x, d.packed, d.centroids, d.bits, d.out_features, d.in_features, None,
                          unpack=oracle.unpack_indices_bitloop, **d.ext())
    return sum(xs.keys())


def cpu_baseline(budget_s: float) -> dict:
    d, xs = _cpu_layer()
    _cpu_step(d, xs)
    t0 = time.perf_counter()
    n = tok = 0
    while n < 1 or time.perf_counter() - t0 < budget_s:
        tok += _cpu_step(d, xs)
        n += 1
    dt = time.perf_counter() - t0
    return {"value": round(tok / dt, 2), "unit": "tokens/s", "cores": torch.get_num_threads(),
            "kind": "port",
            "sample": f"{n} passes of the c2 layer at rows {REF_ROWS} (decode on every call, "
                      f"bit-loop unpack, bf16 matmul), {dt:.1f} s"}


def run_reference(args) -> dict:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return {}
    d, xs = _cpu_layer()
    for _ in range(min(args.warmup, 1)):
        _cpu_step(d, xs)
    t0 = time.perf_counter()
    tok = 0
    steps = min(args.steps, 10)
    for _ in range(steps):
        tok += _cpu_step(d, xs)
    dt = time.perf_counter() - t0
    v = round(tok / dt, 2)
    return {
        "impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": round(dt / steps * 1e3, 2),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "c2 (same layer), bounded sample per step: rows 1 and 16",
                   "tokens_per_step": sum(REF_ROWS)},
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{steps} steps x rows {REF_ROWS}, decode on every call"},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def run_case(args) -> dict:
    """One band of the workload alone, a few launches: the command line profiled under ncu
    (small: four weight copies, one row count)."""
    from neuropress_b200 import kernels
    from synthetic import make_activations, make_q_layer

    global N_COPIES
    N_COPIES = 4
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    name, rows = args.case.split(":")
    rows = int(rows)
    x = make_activations(rows, K_IN, torch.bfloat16, seed=rows).to(device)
    if name == "vq":
        layers, nbytes = build_layers(device, 0, 1)
        run = lambda i: layers[i % N_COPIES](x)  # noqa: E731
    elif name in ("q40", "hqq"):
        from neuropress_b200.nn import NPLinear

        layers = []
        for c in range(N_COPIES):
            q = make_q_layer(N_OUT, K_IN, group_size=32 if name == "q40" else 64, asym=name == "hqq", seed=c)
            nbytes = q.packed_bytes()
            layers.append(NPLinear(q.codes, q.scale, N_OUT, K_IN, q.group_size, 4,
                                   "asym" if name == "hqq" else "sym", "auto", zero_point=q.zero_point).to(device))
        run = lambda i: layers[i % N_COPIES](x)  # noqa: E731
    else:
        raise SystemExit(f"unknown case {args.case}")
    timer = KernelTimer()
    timer.rows = rows
    for i in range(3):
        run(i)
    torch.cuda.synchronize()
    kernels.set_launch_hook(timer)
    for i in range(args.steps):
        run(i)
    torch.cuda.synchronize()
    kernels.set_launch_hook(None)
    out = {"case": args.case, "launches": args.steps, "packed_bytes": nbytes,
           "kernels_ms": {sym: round(v, 5) for (sym, _), v in timer.mean_ms().items()}}
    # The event pairs above include the host's enqueue latency when a kernel is shorter than a
    # Python call.  Replaying the same forwards from a CUDA graph removes the host from the
    # timed region: this is the device time per forward.
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(2):
                run(i)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(args.steps):
                    run(i)
            graph.replay()
            side.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record(side)
            graph.replay()
            t1.record(side)
            side.synchronize()
        ms = t0.elapsed_time(t1) / args.steps
        out["graph_ms_per_forward"] = round(ms, 5)
        out["graph_packed_GBps"] = round(nbytes / (ms * 1e-3) / 1e9, 1)
        out["graph_TFLOPs"] = round(2.0 * rows * N_OUT * K_IN / (ms * 1e-3) / 1e12, 2)
    except Exception as exc:  # graph capture is a measurement aid only
        out["graph_error"] = repr(exc)[:200]
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default=None,
                    help="run one band alone, e.g. vq:1, vq:2048, q40:1, hqq:256 (for profiling)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--eager", action="store_true",
                    help="time eager launches instead of CUDA-graph replay")
    ap.add_argument("--nccl-gather", action="store_true",
                    help="N > 1: all-gather with NCCL instead of the peer-store push kernel")
    args = ap.parse_args()
    if args.case:
        print(json.dumps(run_case(args)), flush=True)
        return
    line = run_reference(args) if args.impl == "reference" else run_ours(args)
    if line:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
