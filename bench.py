"""Benchmark of the packed-weight GEMV (the headline metric: packed GEMV HBM GB/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (``config.workload``): BASELINE config 1 -- one 4096 x 4096 NINT3 (3, 24, 5) weight,
x = 1 x 4096 bf16, y = x W^T with float32 accumulation.  One weight is 7.2 MB and would sit in
the 126 MB L2, so a *step* is one GEMV over each of ``pool`` distinct seeded weights (pool x 7.2 MB
> 2.5 x L2): every launch streams its weight from HBM.  The step is captured once in a CUDA
graph and replayed.  ``value`` = algorithmic bytes of the step / device time, inputs resident
in HBM.  ``e2e`` = the same step through the host-buffer entry point (x copied in from pinned
memory and y copied back inside the timed region, every launch).

With N > 1 (torchrun, one rank per GPU) every rank runs the same step on its own replica of
the pool -- the GEMV microbenchmark does not shard, so this is "replicas only" weak scaling with
no collective on the data path; the time is the max over ranks.

``--impl reference`` times the reference CPU path (dequantize once, then float32
``x @ W.T`` per call, mfq/runtime/linear.py:17-46) restated in the oracle, on the host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

if "reference" in sys.argv:   # torchrun exports OMP_NUM_THREADS=1; the CPU arm may use every host core (set before numpy loads its BLAS)
    for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_v] = str(os.cpu_count() or 1)

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_ROWS, N_COLS = 4096, 4096
PROFILE = (3, 24, 5)
POOL = 48
WORKLOAD = "cfg1: NINT3 (bits=3, gs=24, sub_bits=5) 4096x4096 GEMV, x 1x4096 bf16, pool of 48 distinct weights per step"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def mark(self) -> float:
        """A point in time to pass to stop(since=...): only samples that arrived after it are used."""
        return time.perf_counter()

    def samples_since(self, since: float) -> int:
        return sum(1 for t, _ in list(self.lines) if t >= since)

    def stop(self, since: float = 0.0) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for _, line in [tl for tl in list(self.lines) if tl[0] >= since]:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def profile_traffic(name: str):
    """DRAM bytes per launch recorded with the ncu summary profiles/<name>.md, or None."""
    path = os.path.join(ROOT, "profiles", name + ".json")
    try:
        with open(path) as f:
            return json.load(f).get("dram_bytes_per_launch")
    except (OSError, ValueError):
        return None


def algorithmic_bytes(payload: int, m: int, n: int, k: int) -> int:
    """Packed payload of the weight record (file streams) + x (bf16) + y (bf16)."""
    return payload + m * k * 2 + m * n * 2


def _encode_standalone():
    """The blob writers, loaded by path: importing the package would load the CUDA library,
    which the reference arm must not touch."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("_mfqb_encode_standalone", os.path.join(ROOT, "tyloquant_b200", "encode.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def cpu_reference_arm(steps: int, warmup: int, budget_s: float = 20.0):
    """Reference CPU path (oracle port): dequantize once, then float32 x @ W.T per call."""
    from oracle import mfq_oracle as O
    encode = _encode_standalone()

    try:   # torchrun exports OMP_NUM_THREADS=1: the reference arm may use every host core
        import torch
        torch.set_num_threads(os.cpu_count() or 1)
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=os.cpu_count() or 1)
    except Exception:
        pass
    bits, gs, sb = PROFILE
    blob = encode.random_nint_blob(N_ROWS, N_COLS, bits, gs, sb, seed=1001)
    t0 = time.perf_counter()
    w = O.dequant_nint(O.unpack_nint(blob))
    t_cold = time.perf_counter() - t0
    x = encode.bf16_round(np.random.default_rng(1002).standard_normal((1, N_COLS), dtype=np.float32))
    payload = O.nint_payload_nbytes(N_ROWS, N_COLS, bits, gs, sb)
    nbytes = algorithmic_bytes(payload, 1, N_ROWS, N_COLS)
    for _ in range(max(warmup, 3)):
        O.linear(x, w)
    # one "step" of the reference arm = a bounded sample: `calls` cached products
    t0 = time.perf_counter()
    O.linear(x, w)
    one = max(time.perf_counter() - t0, 1e-6)
    calls = int(max(1, min(POOL, budget_s / max(steps, 1) / one)))
    t0 = time.perf_counter()
    for _ in range(steps):
        for _ in range(calls):
            O.linear(x, w)
    dt = time.perf_counter() - t0
    try:
        from threadpoolctl import threadpool_info
        cores = max([p.get("num_threads", 1) for p in threadpool_info()] or [1])
    except Exception:
        cores = os.cpu_count() or 1
    gbs = nbytes * calls * steps / dt / 1e9
    return {"value": gbs, "unit": "GB/s", "cores": int(cores), "kind": "port",
            "sample": f"{calls} cached float32 x@W.T calls per step on one dequantized 4096x4096 NINT3 weight "
                      f"(numpy/BLAS); cold unpack+dequantize of that weight took {t_cold * 1e3:.0f} ms "
                      f"({payload / t_cold / 1e9:.3f} GB/s)",
            "ms_per_call": dt / (calls * steps) * 1e3, "cold_dequant_ms": t_cold * 1e3}, dt / steps * 1e3


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-sweep", action="store_true", help="skip the per-profile sweep")
    ap.add_argument("--only", default=None, help="run one sweep case by name with a few plain launches "
                    "(small, for profilers) and print its line")
    ap.add_argument("--reps", type=int, default=3, help="launch rounds for --only")
    ap.add_argument("--gemv1-kernel", type=int, default=0, help="mfqb_tune gemv1_kernel: 0 by shape, 1 ring kernel, 2 streamed kernel")
    ap.add_argument("--match", default=None, help="with --only sweep: run the cases whose name contains this text")
    ap.add_argument("--tokens", type=int, nargs="*", default=None, help="token counts for --only moe")
    ap.add_argument("--batch", type=int, nargs="*", default=None, help="batch sizes for --only decoder")
    ap.add_argument("--tune", nargs="*", default=[], help="KEY=VALUE pairs passed to mfqb_tune before anything runs")
    ap.add_argument("--layers", type=int, default=32, help="blocks of the --only decoder model (fewer: a small case for profilers)")
    ap.add_argument("--no-parallel", action="store_true",
                    help="at --gpus > 1 skip the sharded paths (keys tp_rowparallel, ep_moe_cfg4) and time the replicas only")
    args = ap.parse_args()
    # The result line is the only thing that may reach standard output: libraries that print there
    # from native code (the collective library's version banner) go to standard error instead.
    result_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)

    def emit(obj) -> None:
        result_out.write(json.dumps(obj) + "\n")
        result_out.flush()
    steps, warmup = max(args.steps, 1), max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    base = {"metric": "packed GEMV HBM GB/s", "unit": "GB/s", "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u3 codes x s16 activations (bf16 quantised per group, two s8 planes), s32 accumulate, f32 scales",
            "data": "synthetic", "config": {"workload": WORKLOAD, "pool": POOL, "l2_policy": "inputs larger than L2 "
                                            f"({POOL} x 7.2 MB weights per step)", "parallelism": f"replicas x{args.gpus}"}}

    if args.tune and args.impl != "reference":
        from tyloquant_b200._capi import check as _tcheck, lib as _tlib
        for kv in args.tune:
            key, _, val = kv.partition("=")
            _tcheck(_tlib.mfqb_tune(key.encode(), int(val)))
    if args.only == "gemm":
        pk = measured_peaks()[0]
        emit(gemm_bench(local_rank, pk.get("bf16_tflops_sustained", pk["bf16_tflops"])))
        return
    if args.only == "decoder":
        emit({"decoder_cfg5": decoder_bench(local_rank, 0, 1, None, batches=tuple(args.batch or (1, 16)), layers=args.layers)})
        return
    if args.only == "moe":
        emit(moe_layer_bench(local_rank, measured_peaks()[0]["hbm_gbs"], token_counts=tuple(args.tokens or (1, 8, 32, 64, 128, 256, 1024))))
        return
    if args.impl != "reference" and args.gemv1_kernel:
        from tyloquant_b200._capi import check as _check, lib as _lib
        _check(_lib.mfqb_tune(b"gemv1_kernel", args.gemv1_kernel))
    if args.only == "sweep":   # every sweep case, graph-timed, nothing else
        emit({"sweep": sweep(local_rank, measured_peaks()[0]["hbm_gbs"], match=args.match)})
        return
    if args.only:
        emit(sweep(local_rank, measured_peaks()[0]["hbm_gbs"], only=args.only, reps=args.reps))
        return

    if args.impl == "reference":
        if rank != 0:
            return
        cb, ms = cpu_reference_arm(steps, warmup)
        line = dict(base)
        line.update({"impl": "reference", "value": cb["value"], "ms_per_step": ms, "n_gpus": args.gpus,
                     "cpu_baseline": cb, "gpu_launches": 0,
                     "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        emit(line)
        return

    import torch

    from tyloquant_b200 import QuantWeight, encode

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU execution path)")
    torch.cuda.set_device(local_rank)
    dev = local_rank
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{dev}"))

    bits, gs, sb = PROFILE
    weights = []
    for i in range(POOL):
        blob = encode.random_nint_blob(N_ROWS, N_COLS, bits, gs, sb, seed=1001 + i, device=f"cuda:{dev}")
        weights.append(QuantWeight.from_blob(f"NINT{bits}", blob, device=dev))
    payload = weights[0].payload_bytes
    step_bytes = POOL * algorithmic_bytes(payload, 1, N_ROWS, N_COLS)
    x = torch.from_numpy(encode.bf16_round(np.random.default_rng(1002).standard_normal((1, N_COLS), dtype=np.float32)))
    x = x.to(f"cuda:{dev}").to(torch.bfloat16)
    ys = [torch.empty((1, N_ROWS), dtype=torch.bfloat16, device=f"cuda:{dev}") for _ in range(POOL)]

    from tyloquant_b200._capi import BF16, check, lib

    stream = torch.cuda.Stream(device=dev)

    def run_step_direct():
        sp = torch.cuda.current_stream(dev).cuda_stream
        for w, y in zip(weights, ys):
            check(lib.mfqb_mul_mat(w._h, x.data_ptr(), 1, y.data_ptr(), BF16, sp))

    graph = None
    with torch.cuda.stream(stream):
        for _ in range(2):
            run_step_direct()
        stream.synchronize()
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                run_step_direct()
            graph = g
        except Exception as exc:  # capture refused: fall back to direct launches
            sys.stderr.write(f"graph capture failed, timing direct launches: {exc}\n")
            graph = None

    def run_step():
        if graph is not None:
            graph.replay()
        else:
            run_step_direct()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    with torch.cuda.stream(stream):
        sampler = ClockSampler(dev)
        sampler.start()   # before the warm-up: the sampling process is then up when the timed region starts
        for _ in range(warmup):
            run_step()
        barrier()
        region_start = sampler.mark()
        # one event per step boundary: the total (first to last) is the timed region, the gaps give the spread
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        marks[0].record(stream)
        for i in range(steps):
            run_step()
            marks[i + 1].record(stream)
        barrier()
        clock_note = None
        if sampler.samples_since(region_start) < 3:
            # a timed region shorter than a few sampling periods: keep the same load running (untimed) until there are samples
            clock_note = "timed region shorter than the sampling period: sampled under the same load right after it"
            t_load = time.perf_counter()
            while sampler.proc is not None and sampler.samples_since(region_start) < 3 and time.perf_counter() - t_load < 1.0:
                for _ in range(20):
                    run_step()
                torch.cuda.synchronize(dev)
        clocks = sampler.stop(since=region_start)
        if clock_note:
            clocks["note"] = clock_note
        ms = marks[0].elapsed_time(marks[-1])
        per_step = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
        step_p50, step_p95 = per_step[len(per_step) // 2], per_step[min(len(per_step) - 1, int(0.95 * len(per_step)))]
    if dist is not None:
        t = torch.tensor([ms], device=f"cuda:{dev}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / steps
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- the same 48 products, several weights per launch (what a decoder does for q|k|v, gate|up) ----
    import ctypes as C

    def grouped_ms(per_launch: int, reps: int = 200) -> float:
        calls = []
        for i in range(0, POOL, per_launch):
            ws = weights[i:i + per_launch]
            calls.append(((C.c_void_p * len(ws))(*[w._h for w in ws]), len(ws),
                          (C.c_void_p * len(ws))(*[y.data_ptr() for y in ys[i:i + per_launch]])))

        def go():
            sp = torch.cuda.current_stream(dev).cuda_stream
            for hs, cnt, ps in calls:
                check(lib.mfqb_mul_mat_multi(hs, cnt, x.data_ptr(), ps, BF16, sp))
        with torch.cuda.stream(stream):
            go()
            stream.synchronize()
            gg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gg, stream=stream):
                go()
            for _ in range(5):
                gg.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                gg.replay()
            e1.record(stream)
            stream.synchronize()
        return e0.elapsed_time(e1) / reps

    grouped = {}
    for per_launch in (2, 4, 8):
        gms = grouped_ms(per_launch)
        grouped[f"x{per_launch}"] = {"ms_per_step": gms, "GBps": step_bytes / (gms * 1e-3) / 1e9}

    # ---- end to end through the host-buffer entry point ---------------------------------
    xh = torch.from_numpy(encode.bf16_bits(x.float().cpu().numpy()).astype(np.int16)).pin_memory()
    yh = torch.empty((1, N_ROWS), dtype=torch.int16).pin_memory()
    e2e_steps = max(3, min(steps, 10))

    yhs = [torch.empty((1, N_ROWS), dtype=torch.int16).pin_memory() for _ in range(POOL)]
    h_arr = (C.c_void_p * POOL)(*[w._h for w in weights])
    x_arr = (C.c_void_p * POOL)(*[xh.data_ptr()] * POOL)
    y_arr = (C.c_void_p * POOL)(*[y.data_ptr() for y in yhs])

    def e2e_step():   # one call: the step's 48 products, x pulled from and y written to pinned host memory
        check(lib.mfqb_mul_mat_host_multi(h_arr, POOL, x_arr, 1, y_arr, BF16))

    def e2e_step_single():   # one call per product
        for w in weights:
            check(lib.mfqb_mul_mat_host(w._h, xh.data_ptr(), 1, yh.data_ptr(), BF16))

    def time_e2e(fn):
        for _ in range(2):
            fn()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            fn()
        torch.cuda.synchronize(dev)
        ms_ = (time.perf_counter() - t0) * 1e3 / e2e_steps
        if dist is not None:
            t_ = torch.tensor([ms_], device=f"cuda:{dev}")
            dist.all_reduce(t_, op=dist.ReduceOp.MAX)
            ms_ = float(t_.item())
        return ms_

    e2e_ms = time_e2e(e2e_step)
    e2e_single_ms = time_e2e(e2e_step_single)
    e2e_value = world * step_bytes / (e2e_ms * 1e-3) / 1e9

    tp = tp_rowparallel_bench(dev, rank, world, dist) if dist is not None and not args.no_parallel else None
    ep = ep_moe_bench(dev, rank, world, dist) if dist is not None and not args.no_parallel else None
    dc = decoder_bench(dev, rank, world, dist) if not args.no_sweep and not (dist is not None and args.no_parallel) else None

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peaks, peak_kind = measured_peaks()
    launch_us = ms_per_step * 1e3 / POOL
    achieved = algorithmic_bytes(payload, 1, N_ROWS, N_COLS) / (launch_us * 1e-6) / 1e9
    line = dict(base)
    line.update({
        "value": value, "ms_per_step": ms_per_step, "ms_per_step_p50": step_p50, "ms_per_step_p95": step_p95, "clocks": clocks,
        "gpu_launches": POOL * steps,
        "graph_replay": graph is not None,
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": POOL * N_COLS * 2,
                "d2h_bytes_per_step": POOL * N_ROWS * 2, "ms_per_step": e2e_ms,
                "api": "mfqb_mul_mat_host_multi: the step's 48 products in one call (pinned host x and y, weights resident)",
                "one_call_per_product": {"api": "mfqb_mul_mat_host", "ms_per_step": e2e_single_ms,
                                         "value": world * step_bytes / (e2e_single_ms * 1e-3) / 1e9}},
        "roofline": {"bound": "hbm", "kernel": "gemv1_bl_kernel<NintCodec<3,3>>", "achieved": achieved, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": f"{peak_kind} copy bandwidth",
                     "us_per_launch": launch_us, "algorithmic_bytes_per_launch": algorithmic_bytes(payload, 1, N_ROWS, N_COLS),
                     "device_bytes_per_launch": weights[0].device_bytes,
                     # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel and shape, from
                     # the ncu capture summarised under profiles/ (the JSON beside the summary)
                     "traffic": profile_traffic("gemv1_bl_nint3_4096x4096"),
                     # the same products with 2, 4 or 8 weights per launch (mfqb_mul_mat_multi)
                     "weights_per_launch": {k: dict(v, frac=v["GBps"] / peaks["hbm_gbs"]) for k, v in grouped.items()}},
    })
    if tp is not None:
        line["tp_rowparallel"] = tp
    if ep is not None:
        line["ep_moe_cfg4"] = ep
    if dc is not None:
        line["decoder_cfg5"] = dc
    if args.gpus == 1:
        cb, _ = cpu_reference_arm(3, 3, budget_s=12.0)
        line["cpu_baseline"] = cb
        if not args.no_sweep:
            line["sweep"] = sweep(dev, peaks["hbm_gbs"])
            line["moe_layer_cfg4"] = moe_layer_bench(dev, peaks["hbm_gbs"])
            line["gemm_cfg2"] = gemm_bench(dev, peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
    emit(line)
    if dist is not None:
        dist.destroy_process_group()


def sweep(dev: int, peak: float, only: str | None = None, reps: int = 10, match: str | None = None) -> dict:
    """GB/s of one GEMV launch per profile and shape (pool of distinct weights > L2, graph replay).

    With ``only`` a single case runs, without a graph and with a pool just above L2, so that a
    profiler sees a handful of plain launches."""
    import torch

    from tyloquant_b200 import QuantWeight, encode
    from tyloquant_b200._capi import BF16, check, lib

    out = {}
    d = f"cuda:{dev}"

    def nint_case(b, gs, sb, n, k):
        return (f"NINT{b}", lambda: encode.random_nint_blob(n, k, b, gs, sb, seed=77, device=d))

    def nvq_case(jsc, n, k):
        def make():
            rng = np.random.default_rng(3001)
            w = encode.bf16_round(rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
            banks = encode.synthetic_d4_banks(512, 2, seed=9) if jsc else encode.d4_256_codebook()[None]
            return encode.nvq_blob(encode.quantize_nvq3(w, banks, jsc=jsc, device=d))
        return ("NVQ3J-512" if jsc else "NVQ3", make)

    cases = [(f"NINT{b}_4096x4096_m1", nint_case(b, gs, sb, 4096, 4096), 4096, 4096, 1)
             for b, (_, gs, sb) in encode.CANONICAL_NINT.items()]
    # the FFN shape of the dense decoder (config 5), every canonical width: the target shape of the GEMV roofline
    cases += [(f"NINT{b}_14336x4096_m1", nint_case(b, gs, sb, 14336, 4096), 14336, 4096, 1)
              for b, (_, gs, sb) in encode.CANONICAL_NINT.items()]
    cases += [
              ("NINT3_4096x4096_m8", nint_case(3, 24, 5, 4096, 4096), 4096, 4096, 8),
              ("NINT4_4096x14336_m1", nint_case(4, 24, 6, 4096, 14336), 4096, 14336, 1),
              ("NVQ3_17408x5120_m1", nvq_case(False, 17408, 5120), 17408, 5120, 1),
              ("NVQ3_17408x5120_m4", nvq_case(False, 17408, 5120), 17408, 5120, 4),
              ("NVQ3_17408x5120_m8", nvq_case(False, 17408, 5120), 17408, 5120, 8),
              ("NVQ3J-512_17408x5120_m1", nvq_case(True, 17408, 5120), 17408, 5120, 1)]
    blob_cache = {}
    for name, (dtype, make_blob), n, k, m in cases:
        if (only and name != only) or (match and match not in name):
            continue
        key = name.rsplit("_m", 1)[0]
        if key not in blob_cache:
            blob_cache.clear()
            blob_cache[key] = make_blob()
        blob = blob_cache[key]
        probe = QuantWeight.from_blob(dtype, blob, device=dev)
        pool = int(max(4, min(64, (1.2 if only else 2.5) * 126e6 / probe.device_bytes + 1)))
        ws = [probe] + [QuantWeight.from_blob(dtype, blob, device=dev) for _ in range(pool - 1)]
        x = torch.randn((m, k), device=f"cuda:{dev}").to(torch.bfloat16)
        y = torch.empty((m, n), dtype=torch.bfloat16, device=f"cuda:{dev}")
        stream = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(stream):
            def step():
                sp = torch.cuda.current_stream(dev).cuda_stream
                for w in ws:
                    check(lib.mfqb_mul_mat(w._h, x.data_ptr(), m, y.data_ptr(), BF16, sp))
            step()
            stream.synchronize()
            if only:
                class _Direct:
                    replay = staticmethod(step)
                g = _Direct()
            else:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    step()
                for _ in range(3):
                    g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                g.replay()
            e1.record(stream)
            stream.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (reps * pool)
        nbytes = algorithmic_bytes(probe.payload_bytes, m, n, k)
        out[name] = {"us_per_launch": us, "GBps": nbytes / us / 1e3, "frac_of_peak": nbytes / us / 1e3 / peak,
                     "pool": pool, "device_over_payload": probe.device_bytes / probe.payload_bytes}
        for w in ws:
            w.free()
    return out


def gemm_bench(dev: int, peak_tflops: float, reps: int = 5) -> dict:
    """BASELINE config 2: M = 512 tokens, N = 14336, K = 4096, NINT4 (4,32,6), NINT8 (8,48,7) and its control (8,32,7):
    TFLOP/s of mfqb_mul_mat (x conversion pre-pass + tcgen05 tile kernel) against the dense bf16 peak."""
    import torch

    from tyloquant_b200 import QuantWeight, encode

    d = f"cuda:{dev}"
    m, n, k = 512, 14336, 4096
    out = {}
    for name, (b, gs, sb) in (("NINT4_gs32", (4, 32, 6)), ("NINT8_gs48", (8, 48, 7)), ("NINT8_gs32", (8, 32, 7)), ("NINT4_gs24", (4, 24, 6))):
        w = QuantWeight.from_blob(f"NINT{b}", encode.random_nint_blob(n, k, b, gs, sb, seed=2001, device=d), device=dev)
        x = torch.randn((m, k), device=d).to(torch.bfloat16)
        for _ in range(3):
            y = w.matmul(x)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            y = w.matmul(x)
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1) / reps
        tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        out[name] = {"ms": ms, "TFLOPs": tf, "frac_of_bf16_peak": tf / peak_tflops, "weight_payload_MB": w.payload_bytes / 1e6}
        w.free()
    return out


def tp_rowparallel_bench(dev: int, rank: int, world: int, dist, iters: int = 200) -> dict:
    """Row-parallel linears of a Llama-3-8B-shaped layer (o_proj 4096x4096 NINT4, down 4096x14336 NINT6)
    with the input axis sharded over the ranks on group boundaries: the product kernel that reduces
    over NVLink in its own epilogue against the same product followed by the stand-alone all-reduce.
    Every rank runs it; times are device times (CUDA events), max over ranks."""
    import torch

    from tyloquant_b200 import QuantWeight, comm, encode

    d = f"cuda:{dev}"
    c = comm.Communicator(rank, world, 1 << 14, dev).connect()
    out = {}
    for name, (n, k, bits, gs, sb) in {"o_proj_NINT4_4096x4096": (4096, 4096, 4, 24, 6), "down_NINT6_4096x14336": (4096, 14336, 6, 24, 7)}.items():
        ng = (k + gs - 1) // gs
        g0, g1 = comm.shard_range(ng, rank, world, 16)
        lo, hi = g0 * gs, min(g1 * gs, k)
        pool = []
        for i in range(6):   # distinct shards, together larger than one L2 share of a rank's traffic
            blob = encode.random_nint_blob(n, k, bits, gs, sb, seed=7000 + i, device=d)
            pool.append(QuantWeight.from_blob(f"NINT{bits}", blob, device=dev, axis=1, begin=lo, end=hi))
        x = torch.randn((1, hi - lo), device=d, generator=torch.Generator(d).manual_seed(9)).to(torch.bfloat16)
        part = torch.empty((1, n), dtype=torch.float32, device=d)
        y = torch.empty((1, n), dtype=torch.float32, device=d)
        from tyloquant_b200._capi import F32, check, lib
        sp = 0
        res = {}
        for mode in ("fused", "product_then_allreduce", "product_then_nccl"):
            def call(w):   # straight C-ABI calls on the capture stream `sp`
                if mode == "fused":
                    check(lib.mfqb_mul_mat_allreduce(w._h, x.data_ptr(), 1, c._h, y.data_ptr(), F32, sp))
                elif mode == "product_then_allreduce":
                    check(lib.mfqb_mul_mat(w._h, x.data_ptr(), 1, part.data_ptr(), F32, sp))
                    check(lib.mfqb_allreduce_f32(c._h, part.data_ptr(), y.data_ptr(), n, sp))
                else:   # what the reference does: float32 ncclAllReduce in place after the product
                    check(lib.mfqb_mul_mat(w._h, x.data_ptr(), 1, part.data_ptr(), F32, sp))
                    dist.all_reduce(part)
            # the sequence numbers of the collective live on the device, so the calls replay from a graph
            stream = torch.cuda.Stream(device=dev)
            with torch.cuda.stream(stream):
                sp = stream.cuda_stream
                for w in pool:
                    call(w)
                stream.synchronize()
                dist.barrier()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    for w in pool:
                        call(w)
                for _ in range(3):
                    g.replay()
                stream.synchronize()
                dist.barrier()
                reps = max(1, iters // len(pool))
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(reps):
                    g.replay()
                e1.record(stream)
                stream.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) * 1e3 / (reps * len(pool))], device=d)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res[mode + "_us"] = float(t.item())
        res["shard_payload_MB"] = pool[0].payload_bytes / 1e6
        res["status"] = c.status()
        out[name] = res
        for w in pool:
            w.free()
    dist.barrier()
    c.close()
    return out


def ep_moe_bench(dev: int, rank: int, world: int, dist, token_counts=(1, 32, 256), reps: int = 5) -> dict:
    """BASELINE config 4 expert-parallel: every rank holds a contiguous range of the 128 experts
    (reference slice planner), router and route plan are replicated, the partial [T, H] outputs are
    summed by the one-shot NVLink all-reduce.  A step = router + local expert FFN + all-reduce;
    16 different inputs per CUDA graph.  Device times, max over ranks."""
    import torch

    from tyloquant_b200 import comm, encode, moe
    from tyloquant_b200._capi import check, lib

    d = f"cuda:{dev}"
    h, e_count, f, k = 2048, 128, 768, 8
    bits = np.random.default_rng(4003).choice([2, 3, 4, 6], e_count)
    gen = torch.Generator(d).manual_seed(4001)   # same seed on every rank: same weights and inputs
    wgu = (torch.randn((e_count, 2 * f, h), device=d, generator=gen) * 0.02).to(torch.bfloat16).float()
    wdn = (torch.randn((e_count, h, f), device=d, generator=gen) * 0.02).to(torch.bfloat16).float()
    b, e = comm.shard_range(e_count, rank, world, 128)
    gu = moe.MoeWeight(encode.quantize_expertwise(wgu, bits, device=d), dev, b, e)
    dn = moe.MoeWeight(encode.quantize_expertwise(wdn, bits, device=d), dev, b, e)
    del wgu, wdn
    c = comm.Communicator(rank, world, max(token_counts) * h, dev).connect()
    out = {"experts_per_rank": e - b}
    nsets = 16
    for t in token_counts:
        xs = [torch.randn((t, h), device=d, generator=gen).to(torch.bfloat16) for _ in range(nsets)]
        zs = [torch.randn((t, e_count), device=d, generator=gen) for _ in range(nsets)]
        ysum = torch.empty((t, h), dtype=torch.float32, device=d)
        stream = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(stream):
            def step():
                for x, z in zip(xs, zs):
                    ids, wts = moe.moe_topk(z, k)
                    part = moe.moe_ffn(gu, dn, x, ids, wts, out_dtype=torch.float32)
                    check(lib.mfqb_allreduce_f32(c._h, part.data_ptr(), ysum.data_ptr(), t * h, stream.cuda_stream))
            step()
            stream.synchronize()
            dist.barrier()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                step()
            for _ in range(2):
                g.replay()
            stream.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                g.replay()
            e1.record(stream)
            stream.synchronize()
        tt = torch.tensor([e0.elapsed_time(e1) * 1e3 / (reps * nsets)], device=d)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        us = float(tt.item())
        out[f"T{t}"] = {"us_per_layer_step": us, "tokens_per_s": t / us * 1e6}
    out["status"] = c.status()
    dist.barrier()
    c.close()
    gu.free()
    dn.free()
    return out


def decoder_bench(dev: int, rank: int, world: int, dist, batches=(1, 16), steps: int = 24, layers: int = 32) -> dict:
    """BASELINE config 5: random-init 32-layer dense decoder (hidden 4096, 32 query / 8 KV heads of
    128, FFN 14336 SwiGLU, vocabulary 128256, RMSNorm, rotary embedding), attention projections NINT4
    (4, 24, 6), FFN and lm_head NINT6 (6, 24, 7), bf16 KV cache holding a 4096-token context, greedy
    decode at batch 1 and 16.  With world > 1 the model is tensor-parallel over the ranks (heads, FFN
    columns and vocabulary sharded; the two row-parallel products of a layer end in the NVLink
    reduction).  Two steps are captured in one CUDA graph and replayed; tokens/s is for the whole job.
    The cache is filled with seeded values instead of running a prefill (only its size matters here)."""
    import torch

    from tyloquant_b200 import comm as commod, decoder as D

    d = f"cuda:{dev}"
    ctx = 4096
    cfg = dict(hidden=4096, n_q_heads=32, n_kv_heads=8, ffn=14336, vocab=128256, layers=layers,
               max_ctx=ctx + 2 * steps + 8, max_batch=max(batches))
    c = commod.Communicator(rank, world, max(batches) * cfg["hidden"], dev).connect() if world > 1 else None
    dec, _ = D.random_decoder(**cfg, rank=rank, world=world, comm=c, device=dev, seed=5000)
    wbytes = sum(w.payload_bytes for w in dec._keep if hasattr(w, "payload_bytes"))
    kv_bytes_per_seq = 2 * cfg["layers"] * (cfg["n_kv_heads"] // world) * ctx * 128 * 2
    out = {"weight_payload_GB_per_rank": wbytes / 1e9, "kv_GB_per_sequence_per_rank": kv_bytes_per_seq / 1e9,
           "context": ctx, "tensor_parallel": world}
    peak = measured_peaks()[0]["hbm_gbs"]
    for b in batches:
        dec.fill_cache(ctx, seed=5001)
        ids = torch.randint(0, cfg["vocab"], (b,), device=d, generator=torch.Generator(d).manual_seed(5002), dtype=torch.int32)
        a, b2 = ids.clone(), torch.empty_like(ids)
        stream = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(stream):
            dec.step(a, b2)                      # warm-up outside the capture, then rewind the cache position
            stream.synchronize()
            dec.fill_cache(ctx, seed=5001)
            if dist is not None:
                dist.barrier()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                dec.step(a, b2)
                dec.step(b2, a)
            g.replay()                           # one untimed replay (positions ctx, ctx + 1)
            stream.synchronize()
            if dist is not None:
                dist.barrier()
            reps = max(1, steps // 2 - 1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                g.replay()
            e1.record(stream)
            stream.synchronize()
        ms = e0.elapsed_time(e1) / (2 * reps)
        if dist is not None:
            t = torch.tensor([ms], device=d)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        step_bytes = wbytes + b * kv_bytes_per_seq   # per rank: every weight once, every sequence's cache once
        out[f"batch{b}"] = {"ms_per_step": ms, "tokens_per_s": b / ms * 1e3, "GBps_per_rank": step_bytes / ms / 1e6,
                            "frac_of_hbm_peak": step_bytes / ms / 1e6 / peak,
                            "tokens_per_s_ceiling_at_peak": b / (step_bytes / (peak * 1e9)) }
    if c is not None:
        out["comm_status"] = c.status()
        dist.barrier()
    dec.free()
    if c is not None:
        c.close()
    return out


def moe_layer_bench(dev: int, peak: float, token_counts=(1, 32, 256), reps: int = 5) -> dict:
    """BASELINE config 4 on one GPU: hidden 2048, 128 experts, top-8, expert FFN width 768 (SwiGLU),
    per-expert NINT bits drawn from {2,3,4,6} with seed 4003.  A step = router + expert FFN for T
    tokens; 16 different (x, logits) inputs are cycled inside one CUDA graph so that successive steps
    touch different experts (all experts together are ~330 MB, more than L2)."""
    import torch

    from tyloquant_b200 import encode, moe

    d = f"cuda:{dev}"
    h, e_count, f, k = 2048, 128, 768, 8
    bits = np.random.default_rng(4003).choice([2, 3, 4, 6], e_count)
    gen = torch.Generator(d).manual_seed(4001)
    wgu = (torch.randn((e_count, 2 * f, h), device=d, generator=gen) * 0.02).to(torch.bfloat16).float()
    wdn = (torch.randn((e_count, h, f), device=d, generator=gen) * 0.02).to(torch.bfloat16).float()
    gu = moe.MoeWeight(encode.quantize_expertwise(wgu, bits, device=d), device=dev)
    dn = moe.MoeWeight(encode.quantize_expertwise(wdn, bits, device=d), device=dev)
    del wgu, wdn
    out = {"expert_payload_MB": (gu.info.payload_bytes + dn.info.payload_bytes) / 1e6}
    nsets = 16
    for t in token_counts:
        xs = [torch.randn((t, h), device=d, generator=gen).to(torch.bfloat16) for _ in range(nsets)]
        zs = [torch.randn((t, e_count), device=d, generator=gen) for _ in range(nsets)]
        touched = 0
        for z in zs:
            ids = torch.topk(z, k, dim=1).indices.unique().tolist()
            touched += sum(gu.expert_bytes(i) + dn.expert_bytes(i) for i in ids)
        stream = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(stream):
            def step():
                for x, z in zip(xs, zs):
                    ids, wts = moe.moe_topk(z, k)
                    moe.moe_ffn(gu, dn, x, ids, wts, out_dtype=torch.bfloat16)
            step()
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                step()
            for _ in range(2):
                g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                g.replay()
            e1.record(stream)
            stream.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (reps * nsets)
        out[f"T{t}"] = {"us_per_layer_step": us, "tokens_per_s": t / us * 1e6, "distinct_expert_MB_per_step": touched / nsets / 1e6,
                        "GBps": touched / nsets / us / 1e3, "frac_of_peak": touched / nsets / us / 1e3 / peak}
    gu.free()
    dn.free()
    return out


if __name__ == "__main__":
    main()
