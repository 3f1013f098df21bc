"""Benchmark of the quantized-linear forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --case NAME            one kernel / band alone (the ncu command lines)

Headline workload "c5" (the same at every N): one decoder layer's linear set of the
Llama-3-70B shape -- q 8192x8192, k / v 1024x8192, o 8192x8192, gate / up 28672x8192, down
8192x28672 -- vector-quantized with vector length 8, one 65536-entry fp16 codebook and uint16
indices (uniform), driven with a 4096-row bf16 N(0,1) prefill and a 32-row decode batch.  One
PASS is those 14 ``NPVQLinear`` forwards (4128 rows, "tokens"); one STEP is PASSES_PER_STEP
passes, alternating between two independently drawn copies of the layer set.  Everything is
synthetic and seeded (no dataset, no checkpoint); the weights are drawn on the GPU.

N > 1 (torchrun, one process per GPU): every linear whose index stream is at least
SHARD_MIN_BYTES is sharded along its output features, each rank runs the same bands on its
shard, and the outputs are all-gathered (peer stores fused into the kernels, or NCCL with
--nccl-gather); the two small projections (k, v) stay replicated.  Total work is fixed
("strong" scaling).

Reported on ONE JSON line by rank 0:
  value        tokens/s over the whole job, inputs resident in HBM, CUDA events around exactly
               K steps, max over ranks.
  e2e          the same steps driven from pinned HOST activations: host->device copy of every
               input and device->host copy of every output inside the timed region.
  parity       max|err| / RMS(y_ref) of every linear at both row counts against the CPU oracle on
               sampled rows and columns, and whether every rank holds bit-identical outputs.
  roofline     the kernel with the largest share of a pass against its measured peak; more
               rooflines (GEMV bands, decode, group-affine kernels) under their own keys.
  cpu_baseline the CPU restatement of the reference's decode + matmul path on this machine's
               host cores, on a bounded sample of the same workload (rank 0, N=1 only).
  c2, c3, c4   (N=1 only) the single-layer band tables of the large-codebook layer and of the
               group-affine layers, and the Llama-3.2-1B-shape decoder stack end to end.

``--impl reference`` times the reference algorithm's CPU path (oracle port, all host threads) on
the same metric and config; each step is a bounded sample of one pass.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
for _p in (ROOT, ROOT / "tests"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

from synthetic import device_bytes, device_normal, pack_indices_device  # noqa: E402  (tests/synthetic.py)

METRIC = "quant-linear GEMV HBM GB/s & GEMM TFLOPS vs B200 peak; tokens/s at 1-8 GPUs"

# ---- headline workload ---------------------------------------------------------------------
C5_LINEARS = (("q", 8192, 8192), ("k", 1024, 8192), ("v", 1024, 8192), ("o", 8192, 8192),
              ("gate", 28672, 8192), ("up", 28672, 8192), ("down", 8192, 28672))
C5_ROWS = (4096, 32)
C5_INPUT = {"q": "h", "k": "h", "v": "h", "gate": "h", "up": "h", "o": "a", "down": "m"}
C5_INPUT_WIDTH = {"h": 8192, "a": 8192, "m": 28672}
PASSES_PER_STEP = 8
N_COPIES = 2
SHARD_MIN_BYTES = 8 << 20        # index-stream bytes from which a linear is sharded at N > 1
TOKENS_PER_PASS = sum(C5_ROWS)
PARITY_TOL = 1e-2

# ---- single-layer extras (N = 1) -------------------------------------------------------------
N_OUT, K_IN = 14336, 4096
C2_ROWS = (1, 2, 16, 128, 384, 2048)
C3_ROWS = (1, 8, 256, 4096)


def c5_config(world: int, gather_kind: str, launch: str) -> dict:
    return {
        "workload": "c5: Llama-3-70B-shape linear set (q/o 8192x8192, k/v 1024x8192, gate/up 28672x8192, "
                    "down 8192x28672), VQ VL8, 65536-entry fp16 codebook, uint16 indices; per pass a "
                    "4096-row bf16 prefill + a 32-row decode batch through all 7 linears",
        "tokens_per_pass": TOKENS_PER_PASS, "passes_per_step": PASSES_PER_STEP,
        "tokens_per_step": TOKENS_PER_PASS * PASSES_PER_STEP,
        "l2": f"cold: {N_COPIES} copies of the layer set alternate; one pass reads 214 MB of indices and "
              "writes / reads 1.7 GB of decoded weights (L2 is 126 MB)",
        "parallelism": "single GPU" if world == 1 else
                       f"out-feature shards x{world} for linears with >= {SHARD_MIN_BYTES >> 20} MiB of "
                       f"indices (k, v replicated) + {gather_kind}",
        "launch": launch,
    }


def load_peaks() -> tuple[dict, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        return json.loads(p.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# --------------------------------------------------------------------------- clocks ---
class ClockSampler:
    """Samples SM clocks / clock-event reasons while a timed region runs (read-only NVML, every
    few milliseconds; ``nvidia-smi`` every 200 ms when NVML cannot be loaded)."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index = index
        self.samples: list[list[str]] = []
        self._stop = threading.Event()
        self._ready = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run_nvml(self) -> bool:
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
        while True:
            try:
                sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                mask = get_reasons(h)
                self.samples.append([str(sm), str(mx), ""] +
                                    ["Active" if mask & bits[n] else "Not Active" for n in self.NAMES])
            except Exception:
                pass
            self._ready.set()
            if self._stop.wait(0.005):
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
        self._ready.wait(timeout=10)
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(self.NAMES, s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_min_mhz": sm[0] if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- helpers ---
class KernelTimer:
    """Launch observer: one CUDA event pair per C-ABI launch, keyed by (symbol, tag)."""

    def __init__(self) -> None:
        self.tag = None
        self.count = 0
        self.timing = True
        self.pairs: dict[tuple, list] = {}
        self._open = None

    def __call__(self, symbol: str, begin: bool) -> None:
        if begin:
            self.count += 1
        if not self.timing:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        if begin:
            self._open = ev
        else:
            self.pairs.setdefault((symbol, self.tag), []).append((self._open, ev))

    def mean_ms(self) -> dict[tuple, float]:
        return {k: sum(a.elapsed_time(b) for a, b in v) / len(v) for k, v in self.pairs.items()}


def graph_time_ms(calls, reps: int = 1) -> float:
    """Device time per call of ``calls`` (a list of no-argument callables) replayed from one
    CUDA graph: the host is out of the timed region, which matters for kernels shorter than a
    Python call.  The calls are run once eagerly first (module loading, attributes)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        keep = [c() for c in calls]
        side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            keep = [c() for c in calls]
        g.replay()
        side.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(side)
        for _ in range(reps):
            g.replay()
        t1.record(side)
        side.synchronize()
    torch.cuda.current_stream().wait_stream(side)
    del keep
    return t0.elapsed_time(t1) / (reps * len(calls))


# --------------------------------------------------------------------------- c5 ---
class C5:
    """The headline workload: N_COPIES copies of the 7-linear set, this rank's shards only."""

    def __init__(self, device, rank: int, world: int, nccl_gather: bool, decode_ahead: bool = False) -> None:
        from neuropress_b200.nn import NPVQLinear, VQProxy
        from neuropress_b200.sharding import ShardedLinear

        self.device, self.rank, self.world = device, rank, world
        self.copies: list[dict] = []
        self.sharded = {name: world > 1 and n * (k // 8) * 2 >= SHARD_MIN_BYTES for name, n, k in C5_LINEARS}
        self.index_bytes = sum(n * (k // 8) * 2 for _, n, k in C5_LINEARS)
        self.local_index_bytes = sum(n * (k // 8) * 2 // (world if self.sharded[name] else 1)
                                     for name, n, k in C5_LINEARS)
        for c in range(N_COPIES):
            proxy = VQProxy(device_normal((65536, 8), device, 1000 * c + 1, std=0.02, dtype=torch.float16))
            layers = {}
            for li, (name, n, k) in enumerate(C5_LINEARS):
                packed = device_bytes(n * (k // 8) * 2, device, 1000 * c + 10 + li)
                full = NPVQLinear(proxy, packed, 16, n, k, 8, backend="auto")
                if self.sharded[name]:
                    layers[name] = ShardedLinear.from_layer(full, rank, world).to(device)
                else:
                    layers[name] = full
                del full, packed
            self.copies.append(layers)
        torch.cuda.empty_cache()
        # the next linear's weight is decoded on a side stream under the current linear's GEMM
        from neuropress_b200.nn import DecodeAhead

        self.ahead = [DecodeAhead([layers[name] for name, _, _ in C5_LINEARS], torch.bfloat16)
                      for layers in self.copies] if decode_ahead else []
        self.x = {rows: {key: device_normal((rows, w), device, 7 + rows + 13 * i)
                         for i, (key, w) in enumerate(C5_INPUT_WIDTH.items())} for rows in C5_ROWS}
        self.gather_kind = "none"
        if world > 1:
            import torch.distributed as dist

            # Every band once on the local shards: module loading and one-time kernel attributes
            # then never fall inside a rank's bounded wait for its peers.
            for rows in C5_ROWS:
                for name, _, _ in C5_LINEARS:
                    layer = self.copies[0][name]
                    (layer.local if self.sharded[name] else layer)(self.x[rows][C5_INPUT[name]])
            torch.cuda.synchronize()
            dist.barrier()
            self.gather_kind = "NCCL all-gather + re-layout copy"
            if not nccl_gather:
                try:
                    from neuropress_b200.sharding import PushGather

                    shared: dict[int, PushGather] = {}
                    for name, n, _ in C5_LINEARS:
                        if not self.sharded[name]:
                            continue
                        if n not in shared:
                            shared[n] = PushGather(None, max(C5_ROWS), n, torch.bfloat16, device)
                        for layers in self.copies:
                            layers[name].push = shared[n]
                    self.gather_kind = ("peer-store all-gather fused into the kernels "
                                        "(npb_gemm_allgather, npb_vq_gemv_allgather)")
                except Exception as exc:  # symmetric memory unavailable: keep NCCL
                    print(f"[bench] push gather unavailable ({exc!r}); using NCCL", file=sys.stderr)

    # one pass over copy `c`; `sink(name, rows, y)` sees every output
    def run_pass(self, c: int, sink=None, timer: KernelTimer | None = None, xs=None) -> None:
        layers = self.copies[c % N_COPIES]
        xs = self.x if xs is None else xs
        for rows in C5_ROWS:
            for name, _, _ in C5_LINEARS:
                if timer is not None:
                    timer.tag = (name, rows)
                y = layers[name](xs[rows][C5_INPUT[name]])
                if sink is not None:
                    sink(name, rows, y)
            if self.ahead:
                self.ahead[c % N_COPIES].join()   # the side stream rejoins before the next part of the pass

    def set_decode_ahead(self, on: bool) -> None:
        for a in self.ahead:
            a.join()
            a.enabled = on

    def local_cols(self, name: str, n: int) -> tuple[int, int]:
        if not self.sharded[name]:
            return 0, n
        per = n // self.world
        return self.rank * per, (self.rank + 1) * per

    def parity(self) -> dict:
        """Every linear at both row counts against the CPU oracle on sampled rows and columns of
        this rank's own output columns, plus a checksum of the whole output that must be equal on
        all ranks.  Runs outside every timed region."""
        sys.path.insert(0, str(ROOT / "oracle"))
        import oracle

        out: dict = {"rows": {}, "ranks_equal": True, "tolerance": PARITY_TOL,
                     "bound": "max|err| <= tolerance * RMS(y_ref) + half an ulp of the bf16 output; rows = max|err|/RMS",
                     "sample": "8 activation rows x 48 output columns per linear and row count"}
        worst = worst_excess = 0.0
        sums = []
        gsel = torch.Generator().manual_seed(1234 + self.rank)
        for c in range(N_COPIES):
            layers = self.copies[c]
            for rows in C5_ROWS:
                for name, n, k in C5_LINEARS:
                    x = self.x[rows][C5_INPUT[name]]
                    y = layers[name](x)
                    torch.cuda.synchronize()
                    local = layers[name].local if self.sharded[name] else layers[name]
                    b, e = self.local_cols(name, n)
                    ri = torch.unique(torch.cat([torch.tensor([0, rows - 1]),
                                                 torch.randint(0, rows, (6,), generator=gsel)]))
                    ci = torch.unique(torch.cat([torch.tensor([0, e - b - 1]),
                                                 torch.randint(0, e - b, (46,), generator=gsel)]))
                    g = k // 8
                    stream = local.packed_indices.view(-1, g * 2)[ci.to(self.device)].reshape(-1).cpu()
                    w = oracle.vq_decode(stream, local.proxy.centroids.cpu(), 16, ci.numel(), k,
                                         torch.bfloat16)
                    ref = x[ri.to(self.device)].cpu().double() @ w.double().T
                    got = y[ri.to(self.device)][:, (ci + b).to(self.device)].cpu().double()
                    rms = max(float(ref.pow(2).mean().sqrt()), 1e-30)
                    err = (got - ref).abs()
                    rel = float(err.max()) / rms
                    # the output is stored in bf16: half a unit in its last place is allowed on top
                    half_ulp = 0.5 * torch.exp2(torch.floor(torch.log2(ref.abs().clamp_min(1e-30))) - 7)
                    excess = float(((err - half_ulp).clamp_min(0.0)).max()) / rms
                    key = f"{name}@{rows}"
                    out["rows"][key] = round(max(out["rows"].get(key, 0.0), rel), 5)
                    worst = max(worst, rel)
                    worst_excess = max(worst_excess, excess)
                    v = y.contiguous().view(torch.int16).to(torch.int64)
                    sums.append(int(v.sum().item()) ^ (int((v[::7] if v.dim() == 1 else v[::7, ::3]).sum().item()) << 1))
        out["max_err_over_rms"] = round(worst, 5)
        out["max_err_beyond_half_ulp_over_rms"] = round(worst_excess, 5)
        if self.world > 1:
            import torch.distributed as dist

            mine = torch.tensor(sums, dtype=torch.int64, device=self.device)
            allv = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(allv, mine)
            out["ranks_equal"] = all(bool(torch.equal(a, allv[0])) for a in allv)
            w = torch.tensor([worst, worst_excess], device=self.device)
            dist.all_reduce(w, op=dist.ReduceOp.MAX)
            out["max_err_over_rms"] = round(float(w[0].item()), 5)
            out["max_err_beyond_half_ulp_over_rms"] = round(float(w[1].item()), 5)
        # bound: |err| <= 1e-2 * RMS(y_ref) + half an ulp of the bf16 output
        out["ok"] = bool(out["max_err_beyond_half_ulp_over_rms"] <= PARITY_TOL and out["ranks_equal"])
        return out


def run_ours(args) -> dict:
    import torch.distributed as dist

    from neuropress_b200 import kernels

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

    wl = C5(device, rank, world, args.nccl_gather, args.decode_ahead)
    wl.set_decode_ahead(args.decode_ahead)
    steps, warmup = args.steps, max(args.warmup, 3)
    tokens_per_step = TOKENS_PER_PASS * PASSES_PER_STEP

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- warm-up: W steps (eager) ----
    p = 0
    for _ in range(warmup):
        for _ in range(PASSES_PER_STEP):
            wl.run_pass(p)
            p += 1
    barrier()

    # ---- CUDA graphs: one per copy of the layer set (14 module forwards and, for N > 1, their
    # all-gathers); a step replays them alternately.
    timer = KernelTimer()
    graphs = None
    launches_per_pass = None
    use_graphs = not args.eager and (world == 1 or wl.gather_kind.startswith("peer-store"))
    if use_graphs:
        graphs, keep = [], []
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        timer.timing = False
        kernels.set_launch_hook(timer)
        with torch.cuda.stream(side):
            for c in range(N_COPIES):
                g = torch.cuda.CUDAGraph()
                before = timer.count
                with torch.cuda.graph(g, stream=side):
                    wl.run_pass(c, sink=lambda name, rows, y: keep.append(y))
                launches_per_pass = timer.count - before
                graphs.append(g)
        kernels.set_launch_hook(None)
        timer.timing = True
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(2):
            for g in graphs:
                g.replay()
        barrier()

    def timed_device(n_steps: int) -> float:
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        q = 0
        for _ in range(n_steps):
            for _ in range(PASSES_PER_STEP):
                if graphs:
                    graphs[q % N_COPIES].replay()
                else:
                    wl.run_pass(q)
                q += 1
        t1.record()
        barrier()
        return max_over_ranks(t0.elapsed_time(t1))

    # ---- end to end: pinned host inputs -> device -> forwards -> pinned host outputs ----
    h2d, d2h = torch.cuda.Stream(), torch.cuda.Stream()
    # N > 1: a rank uploads only its 1/N of every activation matrix's rows (all PCIe links work in
    # parallel) and the ranks all-gather the slices over NVLink (NCCL), so the replicated inputs cross
    # PCIe once in total, not once per rank.
    def row_slice(rows: int) -> slice:
        per = rows // world
        return slice(rank * per, (rank + 1) * per)

    xs_host = {rows: {k: v[row_slice(rows)].cpu().pin_memory() for k, v in wl.x[rows].items()} for rows in C5_ROWS}
    stage = [{rows: {k: torch.empty_like(v) for k, v in wl.x[rows].items()} for rows in C5_ROWS}
             for _ in range(2)]
    part = [{rows: {k: torch.empty_like(v[row_slice(rows)]) for k, v in wl.x[rows].items()} for rows in C5_ROWS}
            for _ in range(2)] if world > 1 else None
    ys_host = {}
    d2h_bytes = 0
    for rows in C5_ROWS:
        for name, n, _ in C5_LINEARS:
            b, e = wl.local_cols(name, n)
            if not wl.sharded[name] and rank != 0:
                continue                       # replicated linears: rank 0 returns the result
            ys_host[(name, rows)] = torch.empty((rows, e - b), dtype=torch.bfloat16).pin_memory()
            d2h_bytes += rows * (e - b) * 2
    h2d_bytes = sum(v.numel() * 2 for rows in C5_ROWS for v in xs_host[rows].values())
    ev_free = [torch.cuda.Event() for _ in range(2)]
    for ev in ev_free:
        ev.record()

    def e2e_pass(q: int) -> None:
        cur = torch.cuda.current_stream()
        st = stage[q & 1]
        with torch.cuda.stream(h2d):
            h2d.wait_event(ev_free[q & 1])     # the pass that last used this staging set is done
            for rows in C5_ROWS:
                for k, v in st[rows].items():
                    if world == 1:
                        v.copy_(xs_host[rows][k], non_blocking=True)
                    else:
                        mine = part[q & 1][rows][k]
                        mine.copy_(xs_host[rows][k], non_blocking=True)
                        dist.all_gather_into_tensor(v, mine)
            ready = torch.cuda.Event()
            ready.record(h2d)
        cur.wait_event(ready)

        def to_host(name, rows, y):
            dst = ys_host.get((name, rows))
            if dst is None:
                return
            n = y.shape[-1]
            b, e = wl.local_cols(name, n)
            part = y if (b, e) == (0, n) and world == 1 else y[:, b:e].contiguous()
            done = torch.cuda.Event()
            done.record(cur)
            d2h.wait_event(done)
            with torch.cuda.stream(d2h):
                dst.copy_(part, non_blocking=True)
            part.record_stream(d2h)

        wl.run_pass(q, sink=to_host, xs=st)
        ev_free[q & 1].record(cur)

    def timed_e2e(n_steps: int) -> float:
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        q = 0
        for _ in range(n_steps):
            for _ in range(PASSES_PER_STEP):
                e2e_pass(q)
                q += 1
        torch.cuda.current_stream().wait_stream(d2h)   # every output is on the host before t1
        t1.record()
        barrier()
        return max_over_ranks(t0.elapsed_time(t1))

    e2e_pass(0)
    e2e_pass(1)
    barrier()

    # ---- timed regions ----
    with ClockSampler(local_rank) as clocks:
        total_ms = timed_device(steps)
    kernels.set_launch_hook(timer)
    timer.count = 0
    barrier()
    wl.set_decode_ahead(False)                           # per-launch device times: two eager passes,
    for q in range(2):                                   # one kernel at a time
        wl.run_pass(q, timer=timer)
    barrier()
    wl.set_decode_ahead(args.decode_ahead)
    eager_launches_per_pass = timer.count // 2
    kernels.set_launch_hook(None)
    with ClockSampler(local_rank) as clocks_e2e:
        e2e_ms = timed_e2e(steps)
    if launches_per_pass is None:
        launches_per_pass = eager_launches_per_pass
    kmean = timer.mean_ms()

    # ---- correctness of what was timed (outside the timed regions) ----
    parity = wl.parity()

    peaks, peak_src = load_peaks()
    line = {
        "metric": METRIC, "value": round(tokens_per_step * steps / (total_ms * 1e-3), 1),
        "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(total_ms / steps, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": c5_config(world, wl.gather_kind,
                            ("CUDA-graph replay of the 14 module forwards of a pass (one graph per copy of "
                             "the layer set)" if graphs else "eager module forwards")
                            + ("" if not args.decode_ahead else
                               "; in the 4096-row part the next linear's weight is decoded on a side stream "
                               "under the current linear's GEMM (nn.DecodeAhead)")),
        "kernel_timing": "pass_kernel_ms and the rooflines: two eager passes with one CUDA-event pair per "
                         "launch, kernels one at a time (decode-ahead off)",
        "timed_region_s": round(total_ms * 1e-3, 3),
        "ms_per_pass": round(total_ms / steps / PASSES_PER_STEP, 4),
        "e2e": {"value": round(tokens_per_step * steps / (e2e_ms * 1e-3), 1), "unit": "tokens/s",
                "h2d_bytes_per_step": h2d_bytes * PASSES_PER_STEP,
                "d2h_bytes_per_step": d2h_bytes * PASSES_PER_STEP,
                "ms_per_step": round(e2e_ms / steps, 4),
                "note": "per rank: uploads 1/N of the rows of every activation matrix (the ranks all-gather them "
                        "over NVLink with NCCL) and returns its own output columns" if world > 1
                        else "all inputs up, all outputs down"},
        "gpu_launches": launches_per_pass * PASSES_PER_STEP * steps,
        "clocks": clocks.summary(), "clocks_e2e": clocks_e2e.summary(),
        "parity": parity,
    }
    line.update(c5_rooflines(kmean, world, wl, peaks, peak_src, total_ms / steps / PASSES_PER_STEP))
    if world > 1:
        # what the all-gathers move: every rank receives the other ranks' columns of every sharded output
        recv = sum(rows * (n - n // world) * 2 for rows in C5_ROWS for name, n, _ in C5_LINEARS if wl.sharded[name])
        line["nvlink"] = {
            "received_bytes_per_pass_per_gpu": recv,
            "note": "algorithmic (P-1)/P * 2*M*N of the sharded linears; the fused epilogues and the push kernel "
                    "store every tile once per peer, so sent = received = algorithmic",
            "GBps_per_gpu_over_the_pass": round(recv / (total_ms / steps / PASSES_PER_STEP * 1e-3) / 1e9, 1),
        }
    if world == 1 and not args.no_extras:
        del graphs
        for a in wl.ahead:
            a.close()
        wl.ahead.clear()
        wl.copies.clear()
        torch.cuda.empty_cache()
        for key, fn in (("c2", lambda: run_c2(device, peaks, peak_src)),
                        ("c3", lambda: run_c3(device, peaks, peak_src)),
                        ("practical_roofs", lambda: run_probes(device, peaks)),
                        ("entropy_streams", lambda: run_entropy(device, peaks)),
                        ("c4", lambda: run_c4(device, peaks))):
            try:
                line[key] = fn()
            except Exception as exc:  # an extra never takes the headline down with it
                line[key] = {"error": repr(exc)[:300]}
            torch.cuda.empty_cache()
        for key in ("gemv_roofline", "gemv_small_codebook_roofline"):
            if isinstance(line.get("c2"), dict) and key in line["c2"]:
                line[key] = line["c2"][key]
        for key in ("q4_gemv_roofline", "q4_gemm_roofline"):
            if isinstance(line.get("c3"), dict) and key in line["c3"]:
                line[key] = line["c3"][key]
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(budget_s=25.0)
    if world > 1:
        dist.destroy_process_group()
    if not parity["ok"]:
        if rank == 0:
            print(json.dumps(line), flush=True)
        raise SystemExit(f"[bench] parity check failed: {parity}")
    return line if rank == 0 else {}


# DRAM bytes (read + write) of single launches on the unsharded gate projection at 4096 rows, from one
# `ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum` capture of `--case c5:gate:4096`.
NCU_GATE_GEMM_DRAM_BYTES = 1747335680 + 224843008
NCU_GATE_DECODE_DRAM_BYTES = 59789568 + 411090176


def c5_rooflines(kmean: dict, world: int, wl: C5, peaks: dict, peak_src: str, ms_per_pass: float) -> dict:
    """Per-kernel figures of one pass from the eager event pairs: the dense GEMM at 4096 rows
    (tensor roof), the one-pass decode (HBM roof) and the time share of each entry point."""
    def local_n(name, n):
        return n // world if wl.sharded[name] else n

    share: dict[str, float] = {}
    for (sym, _), v in kmean.items():
        share[sym] = share.get(sym, 0.0) + v
    total = sum(share.values()) or 1.0
    out: dict = {"pass_kernel_ms": {k: round(v, 4) for k, v in sorted(share.items())},
                 "pass_kernel_ms_total": round(total, 4)}
    gemm_syms = ("npb_gemm", "npb_gemm_allgather")
    # tensor roof: all 4096-row GEMM launches of a pass
    flops = ms = 0.0
    per_linear = {}
    for name, n, k in C5_LINEARS:
        for sym in gemm_syms:
            t = kmean.get((sym, (name, 4096)))
            if t:
                f = 2.0 * 4096 * local_n(name, n) * k
                flops += f
                ms += t
                per_linear[name] = round(f / (t * 1e-3) / 1e12, 1)
    if ms:
        ach = flops / (ms * 1e-3) / 1e12
        big = kmean.get(("npb_gemm", ("gate", 4096))) or kmean.get(("npb_gemm_allgather", ("gate", 4096)))
        out["gemm_roofline"] = {
            "bound": "tensor", "kernel": "gemm_kernel (tcgen05, dense B), the seven 4096-row launches of a pass",
            "achieved": round(ach, 1), "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
            "frac": round(ach / peaks["bf16_tflops_sustained"], 4),
            "frac_of_burst_peak": round(ach / peaks["bf16_tflops"], 4),
            "peak_source": f"{peak_src} sustained cuBLAS bf16 (the kernel runs inside a seconds-long loop)",
            "launch_ms_sum": round(ms, 4), "launch_ms_gate": None if not big else round(big, 4),
            "TFLOPs_per_linear": per_linear, "share_of_pass": round(ms / total, 3),
        }
        # dram__bytes_read.sum + dram__bytes_write.sum of the gate launch (4096 x 28672 x 8192), one ncu
        # capture (profiles/gemm_tcgen05_c5_gate_rows4096.md); a shard's launch is scaled by its columns
        gate_n = local_n("gate", 28672)
        out["gemm_roofline"].update({
            "traffic": int(NCU_GATE_GEMM_DRAM_BYTES * gate_n / 28672),
            "traffic_of": "the gate launch (launch_ms_gate), ncu capture of the unsharded launch"
                          + ("" if gate_n == 28672 else " scaled by this rank's columns"),
            "algorithmic_bytes_gate": 2 * (4096 * 8192 + gate_n * 8192 + 4096 * gate_n),
        })
    dec = [(name, n, k, rows, kmean.get(("npb_vq_decode", (name, rows)))) for name, n, k in C5_LINEARS
           for rows in C5_ROWS]
    dec = [d for d in dec if d[4]]
    if dec:
        nbytes = sum(local_n(name, n) * (k // 8) * 2 + local_n(name, n) * k * 2 for name, n, k, _, _ in dec)
        dms = sum(d[4] for d in dec)
        gbs = nbytes / (dms * 1e-3) / 1e9
        out["decode_roofline"] = {
            "bound": "hbm", "kernel": "vq_decode_copy_kernel (one-pass gather-copy decode, bf16 out), all launches of a pass",
            "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": round(gbs / peaks["hbm_gbs"], 4), "peak_source": f"{peak_src} copy bandwidth",
            "algorithmic_bytes": nbytes, "launch_ms_sum": round(dms, 4), "launches_per_pass": len(dec),
            "share_of_pass": round(dms / total, 3),
            # measured on the gate decode (59.8 MB read + 411.1 MB written of 58.7 + 1.0 + 469.8 MB
            # algorithmic: the tail of the output is still dirty in L2 when the kernel ends), applied
            # to the pass by the same ratio
            "traffic": int(nbytes * NCU_GATE_DECODE_DRAM_BYTES / (28672 * 1024 * 2 + 28672 * 8192 * 2)),
            "traffic_of": "all decode launches of a pass, from the ncu capture of the gate decode",
        }
    gem = out.get("gemm_roofline")
    dcr = out.get("decode_roofline")
    out["roofline"] = gem if gem and (not dcr or gem["launch_ms_sum"] >= dcr["launch_ms_sum"]) else dcr
    out["decode_batch_ms"] = round(sum(v for (sym, tag), v in kmean.items() if tag and tag[1] == 32), 4)
    out["prefill_ms"] = round(sum(v for (sym, tag), v in kmean.items() if tag and tag[1] == 4096), 4)
    out["hbm_floor_decode_batch_ms"] = round(wl.local_index_bytes / peaks["hbm_gbs"] / 1e6, 4)
    out["tensor_floor_prefill_ms"] = round(
        sum(2.0 * 4096 * local_n(name, n) * k for name, n, k in C5_LINEARS) / peaks["bf16_tflops_sustained"] / 1e9, 4)
    return out


# --------------------------------------------------------------------------- entropy extra ---
def run_entropy(device, peaks: dict) -> dict:
    """Entropy-coded index streams on the c2-shaped layer (14336 x 4096, 65536-entry codebook,
    Zipf(1.1)-distributed indices): coded size, the expansion kernel alone (CUDA events over
    back-to-back launches; algorithmic bytes = coded bytes in + 2 bytes per index out) and the
    1-row forward of the coded layer (expansion + GEMV) beside the plain layer's."""
    from neuropress_b200 import kernels
    from neuropress_b200.nn import NPVQLinear, VQProxy
    from neuropress_b200.transforms.vq_packing import (IndexPacking, NTieredIndexPacking, TieredIndexPacking,
                                                       ZeroEscapePacking, describe_entropy_buffer)

    n, k, nc = N_OUT, K_IN, 65536
    g = k // 8
    gen = torch.Generator(device=device).manual_seed(77)
    w = 1.0 / torch.arange(1, nc + 1, dtype=torch.float32, device=device) ** 1.1
    idx = torch.multinomial(w / w.sum(), n * g, replacement=True, generator=gen)
    proxy = VQProxy(device_normal((nc, 8), device, 78, std=0.02, dtype=torch.float16))
    x = device_normal((1, k), device, 79)

    def timed(fn, reps=30):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(reps):
            fn()
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / reps * 1e3

    plain = NPVQLinear(proxy, IndexPacking.pack(idx, 16), 16, n, k, 8, "cuda_wmma")
    out = {"workload": f"{n} x {k}, {nc}-entry codebook, Zipf(1.1) indices", "plain_bytes": n * g * 2,
           "plain_forward_1row_us": round(timed(lambda: plain(x)), 2), "schemes": {}}
    schemes = (("tiered_hot8", "tiered", lambda: TieredIndexPacking.pack(idx, 16, 8), dict(use_tiered=True, cold_bits=16)),
               ("ntier_4_8_12_16", "ntier", lambda: NTieredIndexPacking.pack(idx, [4, 8, 12, 16]), dict(tier_bits=[4, 8, 12, 16])),
               ("zero_escape", "zero_escape", lambda: ZeroEscapePacking.pack(idx, 16), dict(zero_escape=True)))
    for tag, scheme, pack, kw in schemes:
        buf = pack()
        layer = NPVQLinear(proxy, buf, 16, n, k, 8, "auto", **kw)
        lay = describe_entropy_buffer(buf, scheme)
        offs = [getattr(layer, nm) for nm in layer._entropy_names]
        table = torch.empty(n * g * 2, dtype=torch.uint8, device=device)
        us = timed(lambda: kernels.vq_entropy_expand(buf, lay, offs, n, g, out=table))
        assert torch.equal(table.view(torch.int16).to(torch.int64) & 0xFFFF, idx), tag
        out["schemes"][tag] = {
            "coded_bytes": buf.numel(), "bits_per_index": round(buf.numel() * 8 / (n * g), 3),
            "expand_us": round(us, 2),
            "expand_GBps": round((buf.numel() + n * g * 2) / (us * 1e-6) / 1e9, 1),
            "frac_of_hbm": round((buf.numel() + n * g * 2) / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], 4),
            "forward_1row_us": round(timed(lambda: layer(x)), 2),
        }
        del layer, buf, table
    return out


# --------------------------------------------------------------------------- c2 / c3 extras ---
def _vq_layers(device, copies: int, *, num_centroids: int, bits: int, residual: bool, scale: bool,
               cols_per_codebook: int = 0):
    """`copies` independently drawn [N_OUT, K_IN] VQ layers on the device (rotated for a cold L2)."""
    from neuropress_b200.nn import NPVQLinear, VQProxy

    G = K_IN // 8
    layers = []
    for c in range(copies):
        gen = torch.Generator(device=device)
        gen.manual_seed(500 + c)
        n_cb = K_IN // cols_per_codebook if cols_per_codebook else 0
        shape = (n_cb, num_centroids, 8) if n_cb else (num_centroids, 8)
        cent = device_normal(shape, device, 600 + c, std=0.02, dtype=torch.float16)
        idx = torch.randint(0, num_centroids, (N_OUT, G), device=device, generator=gen)
        packed = pack_indices_device(idx, bits)
        kw = {}
        if residual:
            kw.update(residual_proxy=VQProxy(device_normal((256, 8), device, 700 + c, std=0.005, dtype=torch.float16)),
                      residual_indices=device_bytes(N_OUT * G, device, 800 + c), residual_bits=8)
        if scale:
            kw["row_scale"] = torch.exp(device_normal((N_OUT,), device, 900 + c, std=0.1, dtype=torch.float32)).to(torch.float16)
        layers.append(NPVQLinear(VQProxy(cent), packed, bits, N_OUT, K_IN, 8, backend="auto",
                                 cols_per_codebook=cols_per_codebook, **kw).to(device))
    nbytes = layers[0].packed_indices.numel() + (N_OUT * G if residual else 0) + (2 * N_OUT if scale else 0)
    return layers, nbytes


def _band_table(layers, nbytes: int, rows_list, device, peaks, reps: int = 12) -> dict:
    """Per row count: device time per forward (CUDA-graph replay over rotating weight copies,
    cold L2), the C-ABI launches it is made of (eager event pairs), GB/s on packed bytes, TFLOP/s."""
    from neuropress_b200 import kernels

    out = {}
    n_copies = len(layers)
    for rows in rows_list:
        x = device_normal((rows, K_IN), device, 40 + rows)
        calls = [(lambda i=i: layers[i % n_copies](x)) for i in range(reps)]
        ms = graph_time_ms(calls, reps=2)
        timer = KernelTimer()
        timer.tag = rows
        kernels.set_launch_hook(timer)
        for c in calls:
            c()
        torch.cuda.synchronize()
        kernels.set_launch_hook(None)
        out[str(rows)] = {
            "ms": round(ms, 5),
            "kernels_eager_ms": {sym: round(v, 5) for (sym, _), v in timer.mean_ms().items()},
            "packed_GBps": round(nbytes / (ms * 1e-3) / 1e9, 1),
            "frac_of_hbm": round(nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
            "TFLOPs": round(2.0 * rows * N_OUT * K_IN / (ms * 1e-3) / 1e12, 2),
        }
    return out


def _gemv_roofline(kernel: str, ms: float, nbytes: int, peaks, peak_src: str, **more) -> dict:
    gbs = nbytes / (ms * 1e-3) / 1e9
    d = {"bound": "hbm", "kernel": kernel, "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
         "frac": round(gbs / peaks["hbm_gbs"], 4), "launch_ms": round(ms, 5), "algorithmic_bytes": nbytes,
         "peak_source": f"{peak_src} copy bandwidth", "timing": "CUDA-graph replay, cold L2 (rotating copies)"}
    d.update(more)
    return d


def run_c2(device, peaks, peak_src) -> dict:
    """The large-codebook single layer (in 4096, out 14336, 65536-entry codebook + 256-entry residual
    + row scale) at rows 1/2/16/128/384/2048, and the same shape with small codebooks at 1-2 rows."""
    layers, nbytes = _vq_layers(device, 12, num_centroids=65536, bits=16, residual=True, scale=True)
    out: dict = {"workload": "VQ linear 4096->14336, VL8, 65536-entry codebook (uint16) + 256-entry residual "
                             "(uint8) + fp16 row scale", "packed_bytes": nbytes,
                 "bands": _band_table(layers, nbytes, C2_ROWS, device, peaks)}
    b = out["bands"]
    out["gemv_roofline"] = _gemv_roofline(
        "npb_vq_gemv at 1 row (vq_gemv_mma_kernel), 65536-entry codebook: L2-gather bound", b["1"]["ms"], nbytes,
        peaks, peak_src, gathers=N_OUT * (K_IN // 8),
        gather_rate_G_per_s=round(N_OUT * (K_IN // 8) / (b["1"]["ms"] * 1e-3) / 1e9, 1))
    g2048 = b["2048"]["kernels_eager_ms"].get("npb_gemm")
    if g2048:
        ach = 2.0 * 2048 * N_OUT * K_IN / (g2048 * 1e-3) / 1e12
        out["gemm_roofline_2048"] = {"bound": "tensor", "kernel": "gemm_kernel (tcgen05, dense B) at 2048 rows",
                                     "achieved": round(ach, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                     "frac": round(ach / peaks["bf16_tflops"], 4), "launch_ms": round(g2048, 5),
                                     "peak_source": f"{peak_src} burst cuBLAS bf16 (a 0.17 ms launch timed alone)"}
    del layers
    torch.cuda.empty_cache()
    small = {}
    for bits in (16, 12):
        layers, nb = _vq_layers(device, 12, num_centroids=4096, bits=bits, residual=False, scale=False,
                                cols_per_codebook=2048)
        t = _band_table(layers, nb, (1, 2, 8), device, peaks)
        small[f"{bits}bit"] = {"packed_bytes": nb, "bands": t}
        if bits == 16:
            out["gemv_small_codebook_roofline"] = _gemv_roofline(
                "npb_vq_gemv at 1 row, one 4096-entry codebook per 2048 columns (64 KiB each), uint16 indices",
                t["1"]["ms"], nb, peaks, peak_src, lookups=N_OUT * (K_IN // 8))
        del layers
        torch.cuda.empty_cache()
    out["small_codebook"] = small
    return out


def _q_layers(device, copies: int, n_out: int, asym: bool):
    from neuropress_b200.nn import NPLinear

    gs = 64 if asym else 32
    layers = []
    for c in range(copies):
        codes = device_bytes(n_out * K_IN // 2, device, 300 + c).view(n_out, K_IN // 2)
        ng = n_out * K_IN // gs
        scale = torch.exp(device_normal((ng,), device, 310 + c, std=0.3, dtype=torch.float32) - 4.0).to(torch.float16)
        zp = None
        if asym:
            g = torch.Generator(device=device)
            g.manual_seed(320 + c)
            zp = (torch.rand(ng, device=device, generator=g) * 15.0).to(torch.float16)
        layers.append(NPLinear(codes, scale, n_out, K_IN, gs, 4, "asym" if asym else "sym", "auto",
                               zero_point=zp).to(device))
    nbytes = n_out * K_IN // 2 + (n_out * K_IN // gs) * 2 * (2 if asym else 1)
    return layers, nbytes


def run_c3(device, peaks, peak_src) -> dict:
    """Group-affine layers (in 4096; out 4096 and 14336): Q4_0 group 32 and HQQ-style group 64 with
    fp16 zero-points, rows 1/8/256/4096."""
    from neuropress_b200 import kernels

    out: dict = {}
    for n_out in (14336, 4096):
        for asym in (False, True):
            copies = 8 if n_out == 14336 else 28      # > 126 MB of codes in rotation
            layers, nbytes = _q_layers(device, copies, n_out, asym)
            table = {}
            for rows in C3_ROWS:
                x = device_normal((rows, K_IN), device, 60 + rows)
                calls = [(lambda i=i: layers[i % copies](x)) for i in range(copies)]
                ms = graph_time_ms(calls, reps=2)
                timer = KernelTimer()
                timer.tag = rows
                kernels.set_launch_hook(timer)
                for c in calls[:4]:
                    c()
                torch.cuda.synchronize()
                kernels.set_launch_hook(None)
                table[str(rows)] = {"ms": round(ms, 5),
                                    "kernels_eager_ms": {s: round(v, 5) for (s, _), v in timer.mean_ms().items()},
                                    "packed_GBps": round(nbytes / (ms * 1e-3) / 1e9, 1),
                                    "TFLOPs": round(2.0 * rows * n_out * K_IN / (ms * 1e-3) / 1e12, 2)}
            tag = f"{'hqq_g64' if asym else 'q4_0_g32'}_{n_out}x{K_IN}"
            out[tag] = {"packed_bytes": nbytes, "bands": table}
            if n_out == 14336 and not asym:
                out["q4_gemv_roofline"] = _gemv_roofline("npb_q_gemv at 1 row (q4_gemv_ring_kernel), Q4_0 g32 "
                                                         "14336x4096", table["1"]["ms"], nbytes, peaks, peak_src)
                g = table["4096"]["kernels_eager_ms"].get("npb_gemm")
                if g:
                    ach = 2.0 * 4096 * n_out * K_IN / (g * 1e-3) / 1e12
                    out["q4_gemm_roofline"] = {
                        "bound": "tensor", "kernel": "gemm_kernel (tcgen05, dense B) at 4096 rows after q4_decode16_kernel",
                        "achieved": round(ach, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                        "frac": round(ach / peaks["bf16_tflops"], 4), "launch_ms": round(g, 5),
                        "with_decode_TFLOPs": table["4096"]["TFLOPs"],
                        "peak_source": f"{peak_src} burst cuBLAS bf16 (a launch timed alone)"}
            del layers
            torch.cuda.empty_cache()
    return out


def run_probes(device, peaks) -> dict:
    """Hardware rates behind the GEMV bands, measured in this run by the probe library: what a
    plain read of the same bytes, random 16-byte L2 gathers, and random shared-memory reads
    reach.  They are the secondary roofs of kernels whose access pattern, not HBM, bounds them."""
    from neuropress_b200.build import BENCH_LIB_PATH

    lib = ctypes.CDLL(str(BENCH_LIB_PATH))
    for f in (lib.npbb_stream_read, lib.npbb_l2_gather, lib.npbb_smem_lookup):
        f.restype = ctypes.c_int
    lib.npbb_stream_read.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
    lib.npbb_l2_gather.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int64,
                                   ctypes.c_void_p, ctypes.c_void_p]
    lib.npbb_smem_lookup.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
                                     ctypes.c_void_p]
    out_buf = torch.zeros(16, dtype=torch.uint8, device=device)
    res: dict = {}

    def timed(fn, reps=10) -> float:
        st = torch.cuda.current_stream()
        for _ in range(2):
            fn(st.cuda_stream)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for i in range(reps):
            fn(st.cuda_stream, i)
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / reps

    # plain reads of 22 MB (the c2 layer's packed bytes), 33 MB (Q4 14336x4096) and 214 MB, cold L2
    pool = device_bytes(264 << 20, device, 1)
    for label, nbytes in (("22MB", 22048768 // 16 * 16), ("33MB", 33030144), ("214MB", 213909504)):
        copies = max(1, pool.numel() // nbytes)

        def fn(stream, i=0, nbytes=nbytes, copies=copies):
            rc = lib.npbb_stream_read(pool.data_ptr() + (i % copies) * nbytes, nbytes, out_buf.data_ptr(), stream)
            assert rc == 0, rc
        ms = timed(fn)
        res[f"stream_read_{label}"] = {"us": round(ms * 1e3, 2), "GBps": round(nbytes / ms / 1e6, 1),
                                        "frac_of_hbm": round(nbytes / ms / 1e6 / peaks["hbm_gbs"], 4)}
    # random 16-byte gathers: 7.34 M (the c2 layer) from a 65536-entry table
    n_idx = N_OUT * (K_IN // 8)
    idx = pool[: n_idx * 2 * 4]
    table = pool[64 << 20: (64 << 20) + (1 << 20)]

    def fg(stream, i=0):
        rc = lib.npbb_l2_gather(table.data_ptr(), 65536, idx.data_ptr() + (i % 4) * n_idx * 2, n_idx,
                                out_buf.data_ptr(), stream)
        assert rc == 0, rc
    ms = timed(fg)
    res["l2_gather_16B_65536_entries"] = {"us": round(ms * 1e3, 2), "G_per_s": round(n_idx / ms / 1e6, 1),
                                          "gathers": n_idx}
    for mode, label in ((0, "smem_gather_16B_4096_entries"), (1, "smem_lookup_4B_16384_entries")):
        def fs(stream, i=0, mode=mode):
            rc = lib.npbb_smem_lookup(mode, idx.data_ptr() + (i % 4) * n_idx * 2, n_idx, out_buf.data_ptr(), stream)
            assert rc == 0, rc
        ms = timed(fs)
        res[label] = {"us": round(ms * 1e3, 2), "G_per_s": round(n_idx / ms / 1e6, 1), "lookups": n_idx,
                      "equiv_GBps_on_uint16_indices": round(n_idx * 2 / ms / 1e6, 1)}
    return res


# --------------------------------------------------------------------------- c4 ---
def run_c4(device, peaks, layers_n: int = 16, bits: int = 16) -> dict:
    """Decoder stack of the Llama-3.2-1B shape with every q/k/v/o/gate/up/down linear lowered to
    ``NPVQLinear`` (4096-entry codebook per 2048 columns): single-token decoding on a KV cache at
    batch 1 / 8 / 64 and a 512-token prefill, each replayed from a CUDA graph."""
    from transformers import LlamaConfig, LlamaModel
    from transformers.cache_utils import StaticCache

    from neuropress_b200.nn import NPVQLinear, VQProxy, linearize_rms_norms

    cfg = LlamaConfig(hidden_size=2048, intermediate_size=8192, num_hidden_layers=layers_n,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=64, vocab_size=512,
                      max_position_embeddings=1024, attn_implementation="sdpa")
    torch.manual_seed(0)
    with torch.device("meta"):
        model = LlamaModel(cfg)
    model = model.to_empty(device=device).to(torch.bfloat16)
    for prm in model.parameters():
        torch.nn.init.normal_(prm, std=0.02) if prm.dim() > 1 else torch.nn.init.ones_(prm)
    # rotary tables are buffers computed in __init__: rebuild them on the device
    model.rotary_emb = type(model.rotary_emb)(config=cfg, device=device)
    seed = 0
    index_bytes = 0
    for mod in list(model.modules()):
        for child_name, child in list(mod.named_children()):
            if not isinstance(child, torch.nn.Linear):
                continue
            n, k = child.out_features, child.in_features
            seed += 1
            cent = device_normal((k // 2048, 4096, 8), device, 2000 + seed, std=0.02, dtype=torch.float16)
            gen = torch.Generator(device=device)
            gen.manual_seed(3000 + seed)
            idx = torch.randint(0, 4096, (n, k // 8), device=device, generator=gen)
            packed = pack_indices_device(idx, bits)
            index_bytes += packed.numel()
            setattr(mod, child_name, NPVQLinear(VQProxy(cent), packed, bits, n, k, 8, backend="auto",
                                                cols_per_codebook=2048).to(device))
    linearize_rms_norms(model)
    model.eval()
    out: dict = {"workload": f"{layers_n}-layer Llama-3.2-1B-shape stack, VQ VL8, 4096-entry codebook per 2048 "
                             "columns, uint16 indices; attention / norms / RoPE inside the timed region",
                 "index_bytes_per_token_step": index_bytes,
                 "hbm_ceiling_tok_s_batch1": round(peaks["hbm_gbs"] * 1e9 / index_bytes, 1)}
    ctx = 32

    def timed_graph(fn, reps=5) -> float:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            fn()
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                fn()
            g.replay()
            side.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record(side)
            for _ in range(reps):
                g.replay()
            t1.record(side)
            side.synchronize()
        torch.cuda.current_stream().wait_stream(side)
        return t0.elapsed_time(t1) / reps

    def measure(tag: str) -> None:
        with torch.no_grad():
            for batch in (1, 8, 64):
                cache = StaticCache(config=cfg, max_cache_len=ctx + 32)
                prompt = device_normal((batch, ctx, 2048), device, 11 + batch)
                model(inputs_embeds=prompt, past_key_values=cache, use_cache=True,
                      cache_position=torch.arange(ctx, device=device))
                tok = device_normal((batch, 1, 2048), device, 12 + batch)
                pos = torch.tensor([ctx], device=device)

                def step(tok=tok, cache=cache, pos=pos):
                    return model(inputs_embeds=tok, past_key_values=cache, use_cache=True, cache_position=pos)
                try:
                    ms = timed_graph(step)
                    how = "CUDA-graph replay"
                except Exception as exc:
                    torch.cuda.synchronize()
                    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    for _ in range(2):
                        step()
                    t0.record()
                    for _ in range(5):
                        step()
                    t1.record()
                    torch.cuda.synchronize()
                    ms = t0.elapsed_time(t1) / 5
                    how = f"eager ({type(exc).__name__} during capture)"
                out[f"decode_batch{batch}{tag}"] = {"ms_per_step": round(ms, 4),
                                                    "tokens_per_s": round(batch / (ms * 1e-3), 1), "launch": how}
            x = device_normal((1, 512, 2048), device, 99)

            def prefill():
                return model(inputs_embeds=x, use_cache=False)
            ms = timed_graph(prefill, reps=3)
            out[f"prefill512{tag}"] = {"ms": round(ms, 4), "tokens_per_s": round(512 / (ms * 1e-3), 1),
                                       "TFLOPs_linears": round(2.0 * 512 * (index_bytes // 2 * 8) / (ms * 1e-3) / 1e12, 1)}

    measure("_one_launch_per_module")
    # the 112 linears alone (same modules, one launch each, CUDA-graph replay): their share of a step; the
    # rest is attention / RoPE / norms / residual adds in torch
    lins = [m for m in model.modules() if isinstance(m, NPVQLinear)]
    with torch.no_grad():
        for batch in (1, 8, 64):
            xs = {k: device_normal((batch, k), device, 70 + k % 97) for k in {m.in_features for m in lins}}
            ms = graph_time_ms([(lambda m=m, x=xs[m.in_features]: m(x)) for m in lins], reps=3) * len(lins)
            key = f"decode_batch{batch}_one_launch_per_module"
            out[key]["linears_alone_ms"] = round(ms, 4)
            out[key]["linears_share_of_step"] = round(ms / out[key]["ms_per_step"], 3)
    # q / k / v and gate / up as one launch each, the norm in front of them folded in
    from neuropress_b200.nn import group_shared_input_linears

    out["groups_made"] = group_shared_input_linears(model)
    measure("")
    b1 = out.get("decode_batch1")
    if b1:
        out["frac_of_hbm_ceiling_batch1"] = round(b1["tokens_per_s"] / out["hbm_ceiling_tok_s_batch1"], 4)
        out["frac_of_hbm_ceiling_batch1_linears_alone"] = round(
            1e3 / out["decode_batch1_one_launch_per_module"]["linears_alone_ms"] / out["hbm_ceiling_tok_s_batch1"], 4)
    return out


# --------------------------------------------------------------------------- CPU ---
def _cpu_linear_seconds(name: str, n: int, k: int, rows_list, threads_note: list) -> float:
    """The reference's CPU forward of one c5 linear (decode on every call with the bit-loop
    unpack, then a bf16 ``F.linear``) at the given row counts; returns seconds."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import oracle

    g = torch.Generator().manual_seed(n * 31 + k + len(name))
    cent = (torch.randn(65536, 8, generator=g) * 0.02).to(torch.float16)
    packed = torch.randint(0, 256, (n * (k // 8) * 2,), dtype=torch.uint8, generator=g)
    xs = [torch.randn(rows, k, generator=g).to(torch.bfloat16) for rows in rows_list]
    t0 = time.perf_counter()
    for x in xs:
        oracle.vq_forward(x, packed, cent, 16, n, k, None, unpack=oracle.unpack_indices_bitloop)
    return time.perf_counter() - t0


def _cpu_sample(budget_s: float) -> tuple[float, float, list[str]]:
    """Run c5 linears, smallest first, until the budget is used; returns (seconds, fraction of a
    pass's weight elements covered, names).  CPU time is proportional to the weight elements
    (decode) and to rows x elements (matmul), so tokens/s of the pass = tokens / (seconds /
    fraction)."""
    order = sorted(C5_LINEARS, key=lambda t: t[1] * t[2])
    total_elems = sum(n * k for _, n, k in C5_LINEARS)
    spent, done_elems, names = 0.0, 0, []
    for name, n, k in order:
        est = spent / done_elems * n * k if done_elems else 0.0
        if names and spent + est > budget_s:
            break
        spent += _cpu_linear_seconds(name, n, k, C5_ROWS, [])
        done_elems += n * k
        names.append(name)
    return spent, done_elems / total_elems, names


def cpu_baseline(budget_s: float) -> dict:
    secs, frac, names = _cpu_sample(budget_s)
    v = TOKENS_PER_PASS / (secs / frac)
    return {"value": round(v, 3), "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"linears {'+'.join(names)} of one pass ({frac * 100:.1f} % of its weight elements) at rows "
                      f"{C5_ROWS}, decode on every call (bit-loop unpack) + bf16 matmul, {secs:.1f} s; scaled to a "
                      "whole pass by the weight fraction"}


def run_reference(args) -> dict:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return {}
    steps = max(1, min(args.steps, 2))
    per_step_budget = 90.0 / steps
    secs = frac_sum = 0.0
    names = []
    for _ in range(steps):
        s, f, names = _cpu_sample(per_step_budget)
        secs += s / f            # seconds a whole pass would take at the sampled rate
    v = round(TOKENS_PER_PASS * steps / secs, 3)
    return {
        "impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": 0, "ms_per_step": round(secs / steps * PASSES_PER_STEP * 1e3, 1),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": c5_config(1, "none", "CPU: oracle port of the reference's default backend, all host threads"),
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{steps} step(s); each step times linears {'+'.join(names)} of one pass at rows "
                                   f"{C5_ROWS} (decode on every call, bit-loop unpack, bf16 matmul) and scales to "
                                   "the whole pass by the weight fraction; a step of the GPU arm is "
                                   f"{PASSES_PER_STEP} such passes"},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


# --------------------------------------------------------------------------- cases (ncu) ---
def run_case(args) -> dict:
    """One band alone, a few launches, small footprint: the command lines profiled under ncu.
      vq:ROWS      the c2 layer (65536-entry codebook + residual + row scale)
      vqs16:ROWS / vqs12:ROWS   the same shape with 4096-entry codebooks per 2048 columns
      q40:ROWS / hqq:ROWS       group-affine 14336 x 4096
      c5:NAME:ROWS one linear of the headline layer set (NAME in q k v o gate up down)
      c5pass       the headline layer set, eager passes (the launch list)
      probes       the hardware-rate probes; c4 the decoder stack; entropy the entropy-coded streams"""
    from neuropress_b200 import kernels

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    peaks, peak_src = load_peaks()
    parts = args.case.split(":")
    name = parts[0]
    if name == "c5pass":   # the headline workload, eager: one warm-up pass, then --steps passes (launch list)
        wl = C5(device, 0, 1, False)
        timer = KernelTimer()
        wl.run_pass(0)
        torch.cuda.synchronize()
        kernels.set_launch_hook(timer)
        for q in range(args.steps):
            wl.run_pass(q + 1, timer=timer)
        torch.cuda.synchronize()
        kernels.set_launch_hook(None)
        per: dict[str, list] = {}
        for (sym, tag), v in timer.mean_ms().items():
            per.setdefault(sym, []).append(v)
        return {"case": "c5pass", "passes": args.steps, "launches_per_pass": timer.count // max(args.steps, 1),
                "ms_per_pass_by_entry_point": {k: round(sum(v), 4) for k, v in per.items()}}
    if name == "probes":
        return run_probes(device, peaks)
    if name == "c4":
        return run_c4(device, peaks)
    if name == "entropy":
        return run_entropy(device, peaks)
    if name == "c2":
        return run_c2(device, peaks, peak_src)
    if name == "c3":
        return run_c3(device, peaks, peak_src)
    copies = 4
    if name == "c5":
        from neuropress_b200.nn import NPVQLinear, VQProxy

        lin, rows = parts[1], int(parts[2])
        n, k = next((n, k) for nm, n, k in C5_LINEARS if nm == lin)
        if len(parts) > 3:
            n = int(parts[3])                       # a narrower slice of the same linear (small captures)
        copies = 2
        proxy = VQProxy(device_normal((65536, 8), device, 1, std=0.02, dtype=torch.float16))
        layers = [NPVQLinear(proxy, device_bytes(n * (k // 8) * 2, device, 10 + c), 16, n, k, 8,
                             backend="auto") for c in range(copies)]
        nbytes = n * (k // 8) * 2
        kk, nn = k, n
    else:
        rows = int(parts[1])
        kk, nn = K_IN, N_OUT
        if name == "vq":
            layers, nbytes = _vq_layers(device, copies, num_centroids=65536, bits=16, residual=True, scale=True)
        elif name in ("vqs16", "vqs12"):
            layers, nbytes = _vq_layers(device, copies, num_centroids=4096, bits=int(name[3:]), residual=False,
                                        scale=False, cols_per_codebook=2048)
        elif name in ("q40", "hqq"):
            layers, nbytes = _q_layers(device, copies, N_OUT, name == "hqq")
        else:
            raise SystemExit(f"unknown case {args.case}")
    x = device_normal((rows, kk), device, 40 + rows)
    run = lambda i: layers[i % copies](x)  # noqa: E731
    timer = KernelTimer()
    timer.tag = rows
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
    try:
        ms = graph_time_ms([(lambda i=i: run(i)) for i in range(args.steps)])
        out["graph_ms_per_forward"] = round(ms, 5)
        out["graph_packed_GBps"] = round(nbytes / (ms * 1e-3) / 1e9, 1)
        out["graph_TFLOPs"] = round(2.0 * rows * nn * kk / (ms * 1e-3) / 1e12, 2)
    except Exception as exc:  # graph capture is a measurement aid only
        out["graph_error"] = repr(exc)[:200]
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default=None, help="run one band / probe alone (see run_case)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="N = 1: skip the c2 / c3 / c4 / probe tables")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of CUDA-graph replay")
    ap.add_argument("--decode-ahead", action="store_true",
                    help="decode the next linear's weight on a side stream under the current linear's GEMM "
                         "(nn.DecodeAhead); measured neutral under the sustained power cap, so off by default")
    ap.add_argument("--nccl-gather", action="store_true",
                    help="N > 1: all-gather with NCCL instead of the peer-store epilogues")
    args = ap.parse_args()
    if args.case:
        print(json.dumps(run_case(args)), flush=True)
        return
    line = run_reference(args) if args.impl == "reference" else run_ours(args)
    if line:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
