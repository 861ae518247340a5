#!/usr/bin/env python
"""Benchmark of the GGUF block-quantized matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line.  A step is one pass over R distinct copies of the workload's weight (R chosen
so R * weight bytes >= 2 x L2, so every launch streams its weight from HBM): R calls of the
quantized matmul, each = activation quantizer + matvec kernel.

  value      whole-job algorithmic GB/s with inputs resident in HBM (CUDA-graph replay of a step,
             CUDA events on the launching stream, max over ranks)
  roofline   the matvec kernel alone: algorithmic bytes per launch / its average event-timed
             duration, against the measured HBM copy peak
  e2e        the same metric through the host-buffer entry (QLinear::forward on host tensors):
             pinned H2D of x and D2H of y inside the timed region, every call synchronized
  cpu_baseline / --impl reference
             xn's CPU path (AVX2-order restatement of the Rust kernels, all host threads)
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from xn_b200 import synth  # noqa: E402
from xn_b200.dtypes import GgmlDType as D  # noqa: E402

# name -> (dtype, n, k, m)
WORKLOADS = {
    "C1_q4_0_4096x4096_m1": (D.Q4_0, 4096, 4096, 1),
    "C2_q8_0_11008x4096_m1": (D.Q8_0, 11008, 4096, 1),
    "C2_q8_0_11008x4096_m16": (D.Q8_0, 11008, 4096, 16),
    "C3_q4k_14336x4096_m1": (D.Q4K, 14336, 4096, 1),
    "C3_q4k_14336x4096_m4": (D.Q4K, 14336, 4096, 4),
    "C3_q4k_14336x4096_m16": (D.Q4K, 14336, 4096, 16),
    "C4_q6k_128256x4096_m1": (D.Q6K, 128256, 4096, 1),
    "C4_q6k_128256x4096_m16": (D.Q6K, 128256, 4096, 16),   # the dp4a small-batch kernel (Q6_K has no integer tensor-core path)
    "C1_q4_0_4096x4096_m16": (D.Q4_0, 4096, 4096, 16),
    "C1_q4_0_4096x4096_m128": (D.Q4_0, 4096, 4096, 128),
    "C4_q6k_128256x4096_m32": (D.Q6K, 128256, 4096, 32),
    # prefill (m > 16): the tensor-core kernel; roofline is reported against the dense bf16/fp16 tensor peak
    "C2_q8_0_11008x4096_m128": (D.Q8_0, 11008, 4096, 128),
    "C2_q8_0_11008x4096_m512": (D.Q8_0, 11008, 4096, 512),
    "C3_q4k_14336x4096_m32": (D.Q4K, 14336, 4096, 32),   # the folded-scale variant of the integer tensor-core kernel (17..32 rows)
    "C3_q4k_14336x4096_m64": (D.Q4K, 14336, 4096, 64),
    "C3_q4k_14336x4096_m512": (D.Q4K, 14336, 4096, 512),
}


def captured_traffic(name: str):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of the workload's dominant kernel, as the committed
    ncu summary of that kernel recorded it (a small JSON file beside the summaries); None without a capture."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        return json.load(open(path)).get(name)
    except Exception:
        return None

DECODER_WORKLOADS = {"C5_llama7b_q4k_decode_b1": 1, "C5_llama7b_q4k_decode_b16": 16}  # batch
DEFAULT_WORKLOAD = "C3_q4k_14336x4096_m1"  # the matvec the metric's 75%-of-HBM target is quoted on
METRIC = "quant matvec HBM GB/s"
UNIT = "GB/s"


def algorithmic_bytes(dt: D, n: int, k: int, m: int) -> int:
    """GGUF weight bytes + f32 activations in + f32 outputs out, whatever the device layout."""
    return n * dt.row_bytes(k) + 4 * m * k + 4 * m * n


def measured_peaks() -> tuple[float, float, str]:
    """(HBM GB/s, dense bf16 TFLOP/s burst, "measured" | "fallback")."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, uuid: str | None = None):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            try:
                self._h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if uuid and not uuid.startswith("GPU-") else uuid)
            except Exception:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
            self._reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                getattr(pynvml, "nvmlDeviceGetCurrentClocksThrottleReasons")
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                 "hw_power_brake": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                r = self._reasons_fn(self._h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self._nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr:
            self._thr.join()

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def cpu_path(dt: D, n: int, k: int, m: int, weights: list, x: np.ndarray, calls: int, threads: int) -> float:
    """Seconds per call of xn's CPU path (quantize_lhs + AVX2 dots, all threads), rotating weights."""
    from oracle import oracle as O
    O.build()
    if not O.have_avx2():
        raise RuntimeError("host CPU lacks AVX2/FMA/F16C: the reference's x86 path cannot be restated here")
    O.matmul(int(dt), x, weights[0], n, threads=threads, order="avx2")  # warm the pool
    t0 = time.perf_counter()
    for i in range(calls):
        O.matmul(int(dt), x, weights[i % len(weights)], n, threads=threads, order="avx2")
    return (time.perf_counter() - t0) / calls


def run_reference(args, name, dt, n, k, m):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    O.build()
    threads = O.hw_threads()
    ncopies = max(2, min(8, int(np.ceil(512e6 / (n * dt.row_bytes(k))))))  # rotate > L3
    weights = [synth.make_weight(dt, n, k, seed=0, tensor_id=i) for i in range(ncopies)]
    x = synth.make_activation(m, k, seed=0)
    per_call0 = cpu_path(dt, n, k, m, weights, x, 4, threads)
    # bounded sample: the whole run (warm-up included) stays near one minute of CPU time
    calls_per_step = max(1, min(4 * ncopies, int(60.0 / ((args.steps + args.warmup) * max(per_call0, 1e-6)))))
    for _ in range(args.warmup):
        cpu_path(dt, n, k, m, weights, x, calls_per_step, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_path(dt, n, k, m, weights, x, calls_per_step, threads)
    dt_s = time.perf_counter() - t0
    per_call = dt_s / (args.steps * calls_per_step)
    gbs = algorithmic_bytes(dt, n, k, m) / per_call / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt_s / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "i8 block dots, f32 accumulate", "data": "synthetic",
        "config": {"workload": name, "ggml_dtype": dt.name, "n": n, "k": k, "m": m,
                   "cpu_calls_per_step": calls_per_step, "weight_copies": ncopies},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{args.steps} steps x {calls_per_step} matmul calls of the full workload, "
                                   f"{ncopies} rotating weight copies; AVX2-order C restatement of xn's Rust CPU path "
                                   "(the Rust original cannot be built offline)"},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    ref_gpu = reference_gpu_kernel(dt, n, k, m)
    if ref_gpu is not None:
        line["reference_gpu"] = ref_gpu
    print(json.dumps(line), flush=True)


def reference_gpu_kernel(dt, n, k, m):
    """Q8_0, m <= 16 only: the reference's own CUDA kernel (`matmul_q8_f32_m*`, compiled unmodified for sm_100a into
    oracle/_ref/reduce.cubin), launched with the reference's geometry on cold weights, timed with CUDA events. It
    multiplies unquantized activations, so it is a speed reference, not the parity target."""
    if dt != D.Q8_0 or m > 16:
        return None
    try:
        import torch
        from oracle import ref_cuda
        if not ref_cuda.available() or not torch.cuda.is_available():
            return None
        dev = torch.device("cuda", 0)
        l2 = int(getattr(torch.cuda.get_device_properties(dev), "L2_cache_size", 126 * 1024 * 1024))
        ncopies = int(min(16, max(2, np.ceil(2 * l2 / (n * dt.row_bytes(k))))))
        refs = [ref_cuda.RefQ8(synth.make_weight(dt, n, k, seed=0, tensor_id=i), n, k, dev) for i in range(ncopies)]
        x = torch.from_numpy(synth.make_activation(m, k, seed=0)).to(dev)
        y = torch.empty((m, n), dtype=torch.float32, device=dev)
        for r in refs:
            r.matmul_t(x, out=y)
        torch.cuda.synchronize(dev)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        rounds = 20
        ev0.record()
        for _ in range(rounds):
            for r in refs:
                r.matmul_t(x, out=y)
        ev1.record()
        torch.cuda.synchronize(dev)
        us = ev0.elapsed_time(ev1) * 1e3 / (rounds * ncopies)
        return {"kernel": f"matmul_q8_f32_m{1 << (m - 1).bit_length() if m > 1 else 1} (xn-core/cuda-kernels/reduce.cu, grid n/8 x 128 threads)",
                "launch_us": us, "value": algorithmic_bytes(dt, n, k, m) / (us * 1e-6) / 1e9, "unit": UNIT, "weight_copies": ncopies,
                "note": "plain launches back to back; activations are not quantized by this kernel"}
    except Exception as e:  # the CPU arm's line must not depend on this extra
        return {"unavailable": str(e)[:200]}



def _graph_us(torch, dev, fn, calls: int, reps: int) -> float:
    """Microseconds per call of `fn` (which makes `calls` library calls), replayed `reps` times from one CUDA graph and
    timed with CUDA events on the launching stream."""
    for _ in range(2):
        fn()
    torch.cuda.synchronize(dev)
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            fn()
    torch.cuda.current_stream(dev).wait_stream(side)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize(dev)
    return e0.elapsed_time(e1) * 1e3 / (reps * calls)


# the other BASELINE configurations, measured in the same run as the headline: (group, dtype, n, k, batch sizes)
EXTRA_MATMULS = [
    ("C1_q4_0_4096x4096", D.Q4_0, 4096, 4096, (1,)),
    ("C2_q8_0_11008x4096", D.Q8_0, 11008, 4096, (1, 16, 128, 512)),
    ("C3_q4k_14336x4096", D.Q4K, 14336, 4096, (4, 16, 32, 64, 512)),   # 32: the folded-scale variant of the integer kernel
    ("C4_q6k_128256x4096", D.Q6K, 128256, 4096, (1, 16, 32)),          # 16: the dp4a small-batch kernel
]


def extra_matmul_workloads(torch, L, Q, dev, l2: int, budget_s: float) -> list:
    """Cold (R distinct weights, R x bytes >= 2 x L2) and warm (one weight again and again) time per call of every other
    BASELINE matmul configuration, each with its roofline fraction against the measured peaks. Bounded in time: a
    configuration that would start after the budget is spent is listed as skipped."""
    peak, peak_tf, peak_kind = measured_peaks()
    out = []
    t_start = time.perf_counter()
    for group, dt, n, k, ms in EXTRA_MATMULS:
        if time.perf_counter() - t_start > budget_s:
            out += [{"workload": f"{group}_m{m}", "skipped": "time budget of the default run"} for m in ms]
            continue
        wb = n * dt.row_bytes(k)
        ncopies = int(min(32, max(2, np.ceil(2 * l2 / wb))))
        weights = []
        for i in range(ncopies):
            weights.append(Q.QCudaTensor.from_qtensor(Q.QTensor(synth.make_weight(dt, n, k, seed=0, tensor_id=i), (n, k), dt), dev))
        ref_gpu = {}
        for m in ms:
            x = torch.from_numpy(synth.make_activation(m, k, seed=0)).to(dev)
            ys = [torch.empty((m, n), dtype=torch.float32, device=dev) for _ in range(ncopies)]
            for w in weights:
                w.workspace(m)

            def cold():
                for i, w in enumerate(weights):
                    if m == 1:
                        weights[(i + 1) % ncopies].hint_next()
                    w.matmul_t(x, out=ys[i])

            def warm():
                for i in range(ncopies):
                    weights[0].matmul_t(x, out=ys[0])

            before = L.xnq_launch_count()
            cold()
            launches = (L.xnq_launch_count() - before) // ncopies
            reps = int(max(3, min(40, 4e5 / max(1.0, wb / 1e6 * ncopies))))   # a few hundred ms of device time at most
            cold_us = _graph_us(torch, dev, cold, ncopies, reps)
            warm_us = _graph_us(torch, dev, warm, ncopies, reps)
            bytes_ = algorithmic_bytes(dt, n, k, m)
            flops = 2.0 * m * n * k
            gbs, tf = bytes_ / cold_us / 1e3, flops / cold_us / 1e6
            tensor_bound = m > 16 and (flops / (peak_tf * 1e12)) > (bytes_ / (peak * 1e9))
            entry = {"workload": f"{group}_m{m}", "ggml_dtype": dt.name, "n": n, "k": k, "m": m, "weight_copies": ncopies,
                     "cold_us_per_call": cold_us, "warm_us_per_call": warm_us, "launches_per_call": int(launches),
                     "bound": "tensor" if tensor_bound else "hbm", "hbm_gbs": gbs, "tflops": tf,
                     "frac": (tf / peak_tf) if tensor_bound else (gbs / peak), "peak_kind": f"of {peak_kind}"}
            if dt == D.Q8_0 and m <= 16:
                try:
                    entry["reference_gpu"] = reference_gpu_kernel(dt, n, k, m)
                except Exception as e:
                    entry["reference_gpu"] = {"unavailable": str(e)[:160]}
            out.append(entry)
            del ys, x
        del weights
        torch.cuda.empty_cache()
    return out


class Ctx:
    """One process per GPU: device, rank, world, the loaded library."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        from xn_b200 import _lib, quantized as Q
        self.torch, self.dist, self.Q = torch, dist, Q
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus and self.world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        Q.init(self.dev)
        self.L = _lib.lib()
        for opt in args.option:
            oname, val = opt.split("=")
            _lib.check(self.L.xnq_set_option(oname.encode(), int(val)))

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def measure_matmul(ctx, args, name, dt, n, k, m, with_cpu=True):
    """The headline measurement of one matmul workload on ctx.world GPUs; returns the JSON line on rank 0, None elsewhere."""
    import ctypes

    from xn_b200 import _lib
    torch, dist, Q, L = ctx.torch, ctx.dist, ctx.Q, ctx.L
    world, rank, local, dev = ctx.world, ctx.rank, ctx.local, ctx.dev

    props = torch.cuda.get_device_properties(dev)
    l2 = int(getattr(props, "L2_cache_size", 126 * 1024 * 1024))
    w_bytes_full = n * dt.row_bytes(k)
    n_local = n // world
    if n % world:
        raise SystemExit(f"n={n} does not divide over {world} GPUs")
    w_bytes_local = n_local * dt.row_bytes(k)
    ncopies = int(max(2, np.ceil(2 * l2 / w_bytes_local)))
    ncopies = min(ncopies, 64)

    # weights: rank r holds rows [r*n/G, (r+1)*n/G) of every copy (column-sharded along N)
    weights = []
    for i in range(ncopies):
        rows = (rank * n_local, (rank + 1) * n_local)
        blocks = synth.make_weight(dt, n, k, seed=0, tensor_id=i, rows=rows)
        weights.append(Q.QCudaTensor.from_rows(dt, blocks, n, k, rows[0], n_local, dev))
    x_np = synth.make_activation(m, k, seed=0)
    x = torch.from_numpy(x_np).to(dev)
    y_local = [torch.empty((m, n_local), dtype=torch.float32, device=dev) for _ in range(ncopies)]
    fused = world > 1 and args.gather == "peer-stores"
    y_full = [torch.empty((world, m, n_local), dtype=torch.float32, device=dev) for _ in range(ncopies)] if world > 1 and not fused else None
    pg = None
    if fused:
        # every weight copy gathers into its own slot, so a replayed step never ends on the slot it starts with
        from xn_b200.parallel import PeerGather
        try:
            pg = PeerGather(dev, rank, world, slot_elems=m * n, nslots=ncopies)
            pg.set_deferred(True)   # every copy gathers into its own slot: one wait per step instead of one barrier per launch
        except RuntimeError as e:   # raised on every rank together: peer mappings unavailable on this box
            sys.stderr.write(f"[bench] rank {rank}: {e}; gathering with NCCL instead\n")
            fused, pg = False, None
            y_full = [torch.empty((world, m, n_local), dtype=torch.float32, device=dev) for _ in range(ncopies)]
    for w in weights:
        w.workspace(m)

    hint = m == 1 and not args.no_hint   # a caller that loops over known weights names the next one: the kernel asks it into L2 as it finishes

    def local_step():
        for i, w in enumerate(weights):
            if hint:
                L.xnq_hint_next_weight(weights[(i + 1) % ncopies]._h)
            w.matmul_t(x, out=y_local[i])

    def step():
        for i, w in enumerate(weights):
            if hint:
                L.xnq_hint_next_weight(weights[(i + 1) % ncopies]._h)
            if fused:
                pg.matmul_t(w, x, slot=i)       # the kernel stores its columns into every rank's slot i
            else:
                w.matmul_t(x, out=y_local[i])
                if world > 1:
                    dist.all_gather_into_tensor(y_full[i], y_local[i])
        if fused:
            pg.wait()                           # the peers' columns of the step's gathers

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    launches_before = L.xnq_launch_count()
    step()
    launches_per_step = L.xnq_launch_count() - launches_before
    for _ in range(max(args.warmup, 3) - 1):
        step()
    sync_all()

    # one step as a CUDA graph: the decode loop of the reference is graph-captured too
    graph = None
    if world == 1 or fused:   # NCCL calls stay outside graphs here: a capture that fails on one rank only would strand the others
        try:
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    step()
            torch.cuda.current_stream(dev).wait_stream(side)
            graph.replay()
            torch.cuda.synchronize(dev)
        except Exception as e:  # a failed capture must not take the benchmark down
            if world > 1:
                raise           # ranks must not diverge on how they launch
            sys.stderr.write(f"[bench] CUDA graph capture failed ({e}); timing plain launches\n")
            graph = None
    run_step = graph.replay if graph is not None else step

    sampler = ClockSampler(local, str(getattr(props, "uuid", "")) or None)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with sampler:
        sync_all()
        ev0.record()
        for _ in range(args.steps):
            run_step()
        ev1.record()
        sync_all()
        elapsed_ms = ev0.elapsed_time(ev1)
        # keep the load on while the sampler collects enough clock samples for a median
        t_end = time.perf_counter() + 0.6
        extra = 0
        while (extra < 4) if world > 1 else (len(sampler.samples) < 8 and time.perf_counter() < t_end):
            for _ in range(50):   # N > 1: the same count on every rank, since every gather needs all of them
                run_step()
            torch.cuda.synchronize(dev)
            extra += 1
    if world > 1:
        t = torch.tensor([elapsed_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    step_bytes = ncopies * algorithmic_bytes(dt, n, k, m)  # whole job, all ranks
    value = step_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- roofline: the matvec kernel alone, per-launch event pairs (separate pass, plain launches)
    peak, peak_tf, peak_kind = measured_peaks()
    prof_steps = max(1, min(args.steps, 64))
    chunk_calls = 0
    _lib.check(L.xnq_profile_begin(prof_steps * ncopies + 8))
    for _ in range(prof_steps):
        if chunk_calls == 0:
            torch.cuda._sleep(40_000_000)  # let the host run ahead so no event waits for its kernel's enqueue
        local_step()                       # this rank's kernel on its own rows; no rank waits for another here
        chunk_calls = (chunk_calls + ncopies) % 256
    tot = ctypes.c_double()
    cnt = ctypes.c_int()
    _lib.check(L.xnq_profile_end(ctypes.byref(tot), ctypes.byref(cnt)))
    kern_ms = tot.value / max(cnt.value, 1)
    isolated_us = kern_ms * 1e3
    single_kernel = (m == 1 and k <= 4096) and launches_per_step == ncopies
    if single_kernel and graph is not None:
        # the step is nothing but `ncopies` launches of this one kernel: its average duration over the timed
        # region is the region's device time divided by the launches (back-to-back, overlap included)
        kern_ms = ms_per_step / ncopies
    kern_bytes = algorithmic_bytes(dt, n_local, k, m)
    achieved = kern_bytes / (kern_ms * 1e-3) / 1e9 if kern_ms > 0 else None

    flops = 2.0 * m * n_local * k
    tflops = flops / (kern_ms * 1e-3) / 1e12 if kern_ms > 0 else None
    tensor_bound = m > 16 and (flops / (peak_tf * 1e12)) > (kern_bytes / (peak * 1e9))
    roofline = {"bound": "tensor" if tensor_bound else "hbm",
                "achieved": tflops if tensor_bound else achieved, "peak": peak_tf if tensor_bound else peak,
                "unit": "TFLOP/s" if tensor_bound else "GB/s",
                "frac": ((tflops / peak_tf) if tensor_bound else (achieved / peak)) if achieved else None,
                "traffic": captured_traffic(name) if world == 1 else None,
                "kernel": ("matvec_ring_kernel" if m == 1 else "imma_kernel (tcgen05 kind::i8)" if (m <= 64 and dt.name != "Q6K")
                           else "prefill_persistent_kernel (tcgen05 kind::f16)" if m > 16 else "matvec_q6k (dp4a)"),
                "launch_us": kern_ms * 1e3, "launches_timed": cnt.value, "peak_kind": f"of {peak_kind}",
                "bytes_per_launch": kern_bytes, "flops_per_launch": flops, "hbm_gbs": achieved, "tflops": tflops,
                "isolated_launch_us": isolated_us,
                "timing": ("timed region (CUDA events around the graph replays) / launches in it: the step is this one kernel; "
                           "isolated_launch_us is the same kernel between its own event pair with plain launches")
                if (single_kernel and graph is not None) else
                "CUDA event pair around each launch of the dominant kernel, separate pass with plain launches"}

    # ---- e2e: host buffers through the QLinear::forward-on-host entry, every call synchronized
    x_pin = torch.empty((m, k), dtype=torch.float32, pin_memory=True)
    x_pin.copy_(torch.from_numpy(x_np))
    x_host = x_pin.numpy()
    e2e_steps = max(1, min(args.steps, 50))
    y_pin = torch.empty((m, n_local), dtype=torch.float32, pin_memory=True)   # the result lands in page-locked host memory
    y_host = y_pin.numpy()
    if world == 1:
        for w in weights[:2]:
            w.forward_host(x_host, out=y_host)
    sync_all()
    if world == 1:
        # the timed calls go through the C entry itself (what a host binding calls), arguments prepared once
        fwd = L.xnq_linear_forward_host
        xp, yp = ctypes.c_void_p(x_host.ctypes.data), ctypes.c_void_p(y_host.ctypes.data)
        sp = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        handles = [w._h for w in weights]
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            for h in handles:
                if fwd(h, xp, m, None, yp, sp) != 0:
                    _lib.check(-1)
        torch.cuda.synchronize(dev)
        e2e_s = time.perf_counter() - t0
        d2h_per_step = ncopies * m * n_local * 4
        e2e_note = ("QLinear::forward on pinned host tensors (activations copied in, result stored to the pinned buffer by the kernel for "
                    "m <= 16, copied back otherwise); one synchronize per call")
    else:
        # the whole operator: activations from pinned host memory, sharded matmul, gather, the gathered [m, n] back to host
        x_dev = torch.empty_like(x)
        y_pin_full = torch.empty((m * n,), dtype=torch.float32, pin_memory=True)
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            for i, w in enumerate(weights):
                x_dev.copy_(x_pin, non_blocking=True)
                if fused:
                    yg = pg.matmul_t(w, x_dev, slot=i)
                    pg.wait()
                else:
                    w.matmul_t(x_dev, out=y_local[i])
                    dist.all_gather_into_tensor(y_full[i], y_local[i])
                    yg = y_full[i]
                y_pin_full.copy_(yg.reshape(-1), non_blocking=True)
                torch.cuda.synchronize(dev)
        e2e_s = time.perf_counter() - t0
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
        d2h_per_step = ncopies * m * n * 4
        e2e_note = "host activations in, N-sharded matmul, gather, the gathered [m, n] back to pinned host memory on every rank; one synchronize per call"
    e2e_value = e2e_steps * step_bytes / e2e_s / 1e9

    # ---- N > 1: one gathered [m, n] per workload against the unsharded product (outside the timed region) ----
    gather_check = None
    if world > 1:
        if fused:
            got = pg.matmul_t(weights[0], x, slot=0)
            pg.wait()
            got = got.clone()
            pg.matmul_t(weights[1 % ncopies], x, slot=1 % ncopies)   # a slot may not be named twice in a row
            pg.wait()
        else:
            dist.all_gather_into_tensor(y_full[0], weights[0].matmul_t(x, out=y_local[0]))
            got = y_full[0].permute(1, 0, 2).reshape(m, n).clone()
        torch.cuda.synchronize(dev)
        if rank == 0:
            whole = Q.QCudaTensor.from_qtensor(Q.QTensor(synth.make_weight(dt, n, k, seed=0, tensor_id=0), (n, k), dt), dev)
            want = whole.matmul_t(x)
            err = float(((got.view(m, n) - want).abs() / want.abs().clamp(min=1.0)).max().item())
            del whole
        else:
            err = 0.0
        t = torch.tensor([err], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        gather_check = {"gather_checked": True, "gather_max_err": float(t.item())}
        if float(t.item()) > 2e-3:
            raise SystemExit(f"rank {rank}: the gathered result differs from the unsharded one by {float(t.item()):.3e}; the numbers are void")

    late = pg.late_peers() if pg is not None else 0
    if pg is not None:
        dist.barrier()
        pg.close()
    if late:
        raise SystemExit(f"rank {rank}: gathers gave up waiting for peers {late:#x}; the numbers are void")
    del weights
    torch.cuda.empty_cache()
    if rank != 0:
        return None

    # ---- CPU baseline: bounded sample of the same workload on this box's host cores
    if not with_cpu:
        cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": "not timed for this entry"}
    else:
        try:
            from oracle import oracle as O
            threads = O.hw_threads()
            ncpu = max(2, min(4, int(np.ceil(300e6 / w_bytes_full))))
            cw = [synth.make_weight(dt, n, k, seed=0, tensor_id=i) for i in range(ncpu)]
            per0 = cpu_path(dt, n, k, m, cw, x_np, 2, threads)
            calls = int(max(4, min(400, 3.0 / max(per0, 1e-6))))
            per = cpu_path(dt, n, k, m, cw, x_np, calls, threads)
            cpu = {"value": algorithmic_bytes(dt, n, k, m) / per / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
                   "sample": f"{calls} matmul calls of the full workload ({per * 1e3:.3f} ms each), {ncpu} rotating weight copies; "
                             "AVX2-order C restatement of xn's Rust CPU path"}
        except Exception as e:
            cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": f"unavailable: {e}"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "i8 block dots (dp4a), f32 accumulate", "data": "synthetic",
        "config": {"workload": name, "ggml_dtype": dt.name, "n": n, "k": k, "m": m, "weight_copies_per_step": ncopies,
                   "cache": f"cold: {ncopies} distinct weights per step = {ncopies * w_bytes_local / 1e6:.0f} MB per GPU, "
                            f"L2 is {l2 / 1e6:.0f} MB",
                   "parallelism": f"N-sharded x{world}" + ((" + output gather by peer stores from the matmul kernel" if fused else " + NCCL all-gather") if world > 1 else ""),
                   "launch": "cuda graph replay" if graph is not None else "plain launches",
                   "options": args.option},
        "roofline": roofline,
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": ncopies * m * k * 4,
                "d2h_bytes_per_step": d2h_per_step, "steps": e2e_steps, "note": e2e_note},
        "gpu_launches": int(launches_per_step * args.steps),
        "clocks": sampler.summary(),
    }
    if gather_check:
        line.update(gather_check)
    return line


def summary_of(line: dict) -> dict:
    """The few figures of a full line that the headline line's "workloads" list carries."""
    out = {"workload": line["config"]["workload"], "metric": line["metric"], "value": line["value"], "unit": line["unit"],
           "n_gpus": line["n_gpus"], "ms_per_step": line["ms_per_step"], "frac": line["roofline"]["frac"], "bound": line["roofline"]["bound"],
           "clocks": line.get("clocks")}
    for key in ("gather_checked", "gather_max_err", "prefill"):
        if key in line:
            out[key] = line[key]
    if "launch_us" in line["roofline"]:
        out["cold_us_per_call"] = line["roofline"]["launch_us"]
    return out


def decoder_measure(args, name, batch, dev, rank, world, steps, L):
    """Config 5: the 32-layer Q4_K decoder (Q6_K LM head). Prefill 512 random tokens, then `steps` greedy decode steps
    replayed from one captured CUDA graph; a step is one token for each of `batch` sequences. Returns the JSON line
    (rank 0) or None. The process group, if any, is the caller's."""
    import torch
    import torch.distributed as dist

    from xn_b200.llama import LlamaConfig, QLlama

    local = dev.index
    cfg = LlamaConfig.llama_7b()
    prompt_len = 512
    steps = min(steps, 256)
    t0 = time.perf_counter()
    model = QLlama(cfg, dev, batch=batch, max_seq=prompt_len + steps + 8, rank=rank, world=world, max_prefill_rows=batch * prompt_len)
    torch.cuda.synchronize(dev)
    build_s = time.perf_counter() - t0
    g = torch.Generator(device="cpu"); g.manual_seed(0)
    prompt_host = torch.randint(0, cfg.vocab, (batch, prompt_len), generator=g).pin_memory()

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    model.prefill(prompt_host.to(dev))          # warm-up of the prefill path
    sync_all()
    ev[0].record()
    model.prefill(prompt_host.to(dev, non_blocking=True))
    ev[1].record()
    sync_all()
    prefill_ms = ev[0].elapsed_time(ev[1])
    model.capture_decode()
    for _ in range(max(args.warmup, 3)):
        model._graph.replay()
    model.prefill(prompt_host.to(dev))          # back to the end of the prompt
    sync_all()
    props = torch.cuda.get_device_properties(dev)
    sampler = ClockSampler(local, str(getattr(props, "uuid", "")) or None)
    with sampler:
        sync_all()
        t0 = time.perf_counter()
        ev[2].record()
        toks = model.decode(steps)
        ev[3].record()
        toks_host = toks.cpu()                  # the generated ids come back to the host
        e2e_s = time.perf_counter() - t0
        sync_all()
    launches = model.launches_per_step * steps   # replayed from the graph: counted once, at capture
    decode_ms = ev[2].elapsed_time(ev[3])
    if world > 1:
        t = torch.tensor([decode_ms, prefill_ms, e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        decode_ms, prefill_ms, e2e_s = (float(v) for v in t.tolist())
    late = model.pg.late_peers() if model.pg is not None else 0
    if world > 1:
        dist.barrier()
    model.close()
    del model
    torch.cuda.empty_cache()
    if late:
        raise SystemExit(f"rank {rank}: exchanges gave up waiting for peers {late:#x}; the numbers are void")
    if rank != 0:
        return None
    peak, peak_tf, peak_kind = measured_peaks()
    wbytes = cfg.weight_bytes_per_step()
    ms_per_step = decode_ms / steps
    return {
        "metric": "7B Q4_K decode tok/s", "value": batch * steps / (decode_ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "i8 block dots (dp4a, tcgen05 kind::i8), f32 accumulate; bf16 attention", "data": "synthetic",
        "config": {"workload": name, "layers": cfg.n_layers, "d_model": cfg.d_model, "heads": f"{cfg.n_heads}q/{cfg.n_kv_heads}kv x {cfg.head_dim}",
                   "ffn": cfg.ffn, "vocab": cfg.vocab, "linears": cfg.linear_dtype.name, "lm_head": cfg.head_dtype.name, "batch": batch,
                   "prompt": prompt_len, "decode_steps": steps,
                   "cache": f"{wbytes / 1e6:.0f} MB of weights per step, far above L2",
                   "parallelism": f"tensor parallel x{world}: head-sharded attention, N-sharded qkv / gate-up / LM head, K-sharded o / down whose kernels store their summands into every rank (2 exchanges per layer)" if world > 1 else "one GPU",
                   "launch": "one CUDA graph per decode step"},
        "roofline": {"bound": "hbm", "achieved": wbytes / (ms_per_step * 1e-3) / 1e9 / world, "peak": peak, "unit": "GB/s",
                     "frac": wbytes / (ms_per_step * 1e-3) / 1e9 / world / peak, "traffic": None, "peak_kind": f"of {peak_kind}",
                     "kernel": "whole decode step: weight bytes of all linears per GPU / step time", "bytes_per_step": wbytes},
        "cpu_baseline": None,
        "e2e": {"value": batch * steps / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": batch * 8,
                "note": "decode loop timed on the host including the copy of the generated ids back to host memory"},
        "prefill": {"tokens": batch * prompt_len, "ms": prefill_ms, "tok_s": batch * prompt_len / (prefill_ms * 1e-3)},
        "build_s": build_s, "gpu_launches": int(launches), "clocks": sampler.summary(),
        "generated_head": toks_host[0, :8].tolist(),
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS) + sorted(DECODER_WORKLOADS))
    ap.add_argument("--gather", default="peer-stores", choices=["peer-stores", "nccl"], help="N > 1: how output slices are gathered")
    ap.add_argument("--option", action="append", default=[], help="library switch NAME=INT (A/B measurements), e.g. matvec_tma=0")
    ap.add_argument("--no-extra", action="store_true", help="headline workload only: skip the list of the other BASELINE configurations")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg (profiling runs)")
    ap.add_argument("--no-hint", action="store_true", help="one-row workloads: do not name the next weight (xnq_hint_next_weight); a profiler that flushes the "
                    "caches between kernels would count the hinted prefetch as traffic of the launch")
    args = ap.parse_args()
    if args.impl == "reference":
        if args.workload in DECODER_WORKLOADS:
            print(json.dumps({"impl": "reference", "unavailable": "the decoder workloads have no CPU arm; the matmul workloads do"}), flush=True)
            return
        dt, n, k, m = WORKLOADS[args.workload]
        return run_reference(args, args.workload, dt, n, k, m)
    ctx = Ctx(args)
    try:
        if args.workload in DECODER_WORKLOADS:
            line = decoder_measure(args, args.workload, DECODER_WORKLOADS[args.workload], ctx.dev, ctx.rank, ctx.world, args.steps, ctx.L)
        else:
            dt, n, k, m = WORKLOADS[args.workload]
            line = measure_matmul(ctx, args, args.workload, dt, n, k, m, with_cpu=not args.no_cpu)
            if args.workload == DEFAULT_WORKLOAD and not args.no_extra and not args.option:
                # every other BASELINE configuration in the same run (bounded in time), so that one invocation records them all
                extras = []
                if ctx.world == 1:
                    l2 = int(getattr(ctx.torch.cuda.get_device_properties(ctx.dev), "L2_cache_size", 126 * 1024 * 1024))
                    extras += extra_matmul_workloads(ctx.torch, ctx.L, ctx.Q, ctx.dev, l2, budget_s=150.0)
                    for dname, batch in sorted(DECODER_WORKLOADS.items()):
                        dl = decoder_measure(args, dname, batch, ctx.dev, ctx.rank, ctx.world, 64, ctx.L)
                        extras.append(summary_of(dl))
                else:
                    # the configurations BASELINE shards: the Q6_K LM head and the 7B decoder
                    c4 = measure_matmul(ctx, args, "C4_q6k_128256x4096_m1", *WORKLOADS["C4_q6k_128256x4096_m1"], with_cpu=False)
                    dl = decoder_measure(args, "C5_llama7b_q4k_decode_b1", 1, ctx.dev, ctx.rank, ctx.world, 64, ctx.L)
                    if ctx.rank == 0:
                        extras += [summary_of(c4), summary_of(dl)]
                if line is not None:
                    line["workloads"] = extras
        if line is not None:
            print(json.dumps(line), flush=True)
    finally:
        ctx.close()


if __name__ == "__main__":
    main()
