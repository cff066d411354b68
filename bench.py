#!/usr/bin/env python
"""Benchmark of the W4A8 hot path on B200 (one JSON line on stdout, rank 0).

Workload (default, benchmark configuration 1): Llama-7B decode linears, fp16 in/out, M tokens
(default 8; 1 is reported beside it): per decoder layer four 4096->4096, two
4096->11008 and one 11008->4096 projection.  A step is one pass over a ring of
`--layers` distinct layers (>= 2x L2 of distinct weights, so nothing is re-read from
cache); weights are prepared once outside the timed region, as the reference's own
benchmark does.  `value` is algorithmic GB/s with activations resident in HBM (enqueue
entry points, one CUDA graph per step when capture works); `e2e` is the same pass through
the blocking reference ABI with pinned HOST activations and outputs, copies included.

N > 1 (torchrun): every linear is column-sharded over the ranks in contiguous 64-column
blocks (the reference's per-core split) and the shard outputs are reassembled by one
NCCL all-gather per step; total work is fixed, so scaling is "strong".

`--impl reference` times the reference's own CPU stages (oracle/_ref, or the C port when
that was not built) on the host cores for the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LLAMA7B_LAYER = [(4096, 4096)] * 4 + [(4096, 11008)] * 2 + [(11008, 4096)]   # (K, N)


def algorithmic_bytes(M, K, N, in_bytes=2, out_bytes=2):
    """Packed int4 weights + fp32 channel scales + activations in + outputs out."""
    return K * N // 2 + 4 * N + in_bytes * M * K + out_bytes * M * N


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(device)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def samples(self) -> int:
        """Rows written so far (nvidia-smi needs a second or two to produce its first one)."""
        try:
            self.file.flush()
            return sum(1 for r in Path(self.file.name).read_text().splitlines() if r.count(",") >= 8)
        except OSError:
            return 0

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "window": "extended warm-up + timed steps"}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [r.split(",") for r in Path(self.file.name).read_text().splitlines() if r.count(",") >= 8]
        os.unlink(self.file.name)
        clocks, reasons = [], set()
        for r in rows:
            try:
                clocks.append(float(r[1]))
                out["sm_max_mhz"] = float(r[2])
            except ValueError:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if r[col].strip().lower() == "active":
                    reasons.add(name)
        if clocks:
            busy = [c for c in clocks if c >= 0.5 * max(clocks)]
            out["sm_mhz"] = statistics.median(busy)
        out["reasons"] = sorted(reasons)
        return out


# ------------------------------------------------------------------ reference arm (CPU)
def run_reference(args, rank, world):
    if rank != 0:
        return
    if world > 1 and os.environ.get("OMP_NUM_THREADS") == "1":
        # torchrun pins every rank to one OpenMP thread; this arm is a single CPU process and may use the host
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    from oracle.harness import Oracle, Reference            # this arm IS the CPU checker being timed
    from rknpu2_matmul_open_b200.synthetic import make_activations, make_weights
    M = args.tokens
    use_ref = Reference.available()
    ref = Reference() if use_ref else None
    orc = Oracle()
    shapes = [(4096, 4096), (4096, 11008), (11008, 4096)]
    counts = [4, 2, 1]
    layers = []
    for i, (K, N) in enumerate(shapes):
        B, sw = make_weights(K, N, seed=i)
        A = make_activations(M, K, seed=i, dtype="f16")
        handle = ref.layer(B, sw, 480) if use_ref else None
        layers.append((K, N, B, sw, A, handle))
    cores = ref.host_threads() if use_ref else int(os.environ.get("OMP_NUM_THREADS", os.cpu_count() or 1))

    def one_pass():
        t0 = time.perf_counter()
        for (K, N, B, sw, A, handle), count in zip(layers, counts):
            for _ in range(count):
                if use_ref:
                    rc, _, _ = ref.layer_run(handle[0], handle[1], A, threads=4)
                else:
                    rc = orc.linear(A, B, sw)[0]
                assert rc == 0
        return time.perf_counter() - t0

    for _ in range(args.warmup):
        one_pass()
    t = sum(one_pass() for _ in range(args.steps))
    step_bytes = sum(algorithmic_bytes(M, K, N) * c for (K, N), c in zip(shapes, counts))
    step_ops = sum(2 * M * K * N * c for (K, N), c in zip(shapes, counts))
    gbs = step_bytes * args.steps / t / 1e9
    sample = (f"one decoder layer (4x 4096->4096, 2x 4096->11008, 1x 11008->4096) at M={M} per step; "
              + ("reference CPU stages (scan, MSD pack, INT16 reconstruct, dequant: 4 threads) around an "
                 "all-core int4 stand-in for the NPU step" if use_ref else "C port of the reference path"))
    line = {"impl": "reference", "metric": "w4a8_decode_weight_stream", "value": gbs, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": workload_config(args, world, layers=1),
            "tops": step_ops * args.steps / t / 1e12,
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "reference" if use_ref else "port",
                             "sample": sample},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(args, world, layers):
    return {"workload": f"llama7b_decode_linears_M{args.tokens}", "shapes_KxN": "4x4096x4096+2x4096x11008+1x11008x4096",
            "ring_layers": layers, "activation": "fp16 N(0,1), 0.5% channels x20", "weights": "int4 [-7,7] per-channel",
            "cache": "ring of distinct weights larger than 2x L2, no flush needed", "parallelism": f"column-shard x{world}"}


# ------------------------------------------------------------------ CUDA arm
def run_cuda(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    import rknpu2_matmul_open_b200 as rk
    from oracle.harness import Oracle, Reference            # checker of what is timed, and the cpu_baseline leg
    from rknpu2_matmul_open_b200.synthetic import make_activations, make_weights, sample_columns
    from rknpu2_matmul_open_b200.sharding import shard_columns

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # stdout carries the one JSON line only: NCCL's version banner (NCCL_DEBUG=VERSION) would precede it
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)
    ctx = rk.Context(f"cuda:{local_rank}")
    dom = ctx.domain(0)
    M = args.tokens
    hbm_peak, _, peak_kind = measured_peaks()

    # ---- the ring: `layers` distinct decoder layers, each linear column-sharded over ranks
    linears = []          # dicts: K, N(full), n0, n1, weights, workspace, dA, dC, hA, hC
    act = {}
    for K in (4096, 11008):
        A = make_activations(M, K, seed=K, dtype="f16")
        act[K] = (A, torch.from_numpy(A.view(np.int16)).to(dev))
    check = None
    generated = {}
    # every linear writes straight into one per-rank output buffer; with several ranks that buffer is
    # what the all-gather sends, so no packing copies sit between the GEMMs and the collective
    shard_cols = [shard_columns(N, world, rank) for _ in range(args.layers) for (_, N) in LLAMA7B_LAYER]
    out_cols = sum(n1 - n0 for n0, n1 in shard_cols)
    # Shards may differ by one 64-column block between ranks; NCCL's all-gather wants equal pieces, so every
    # rank's buffer has the size of the widest shard set (the tail of a narrower one stays zero).
    pad_cols = max(sum(b - a for a, b in (shard_columns(N, world, r) for _ in range(args.layers) for (_, N) in LLAMA7B_LAYER))
                   for r in range(world))
    out_buf = torch.zeros((M * pad_cols,), dtype=torch.float16, device=dev)   # binary16 bits (NCCL has no int16)
    out_off = 0
    for layer in range(args.layers):
        for j, (K, N) in enumerate(LLAMA7B_LAYER):
            seed = (layer * 16 + j) if args.distinct_values else j
            if (K, N, seed) not in generated:
                generated[(K, N, seed)] = make_weights(K, N, seed=seed)
            B, sw = generated[(K, N, seed)]
            n0, n1 = shard_columns(N, world, rank)
            Bs, ss = np.ascontiguousarray(B[:, n0:n1]), np.ascontiguousarray(sw[n0:n1])
            w = rk.Weights(dom, Bs, ss, k_tile=480)
            ws = rk.Workspace(dom, rk.default_config(M, n1 - n0, K, k_tile=480))
            dC = out_buf[out_off:out_off + M * (n1 - n0)].view(M, n1 - n0).view(torch.int16)
            out_off += M * (n1 - n0)
            hA = torch.from_numpy(act[K][0].view(np.int16)).pin_memory()
            hC = torch.zeros((M, n1 - n0), dtype=torch.int16).pin_memory()
            linears.append(dict(K=K, N=N, n0=n0, n1=n1, w=w, ws=ws, dA=act[K][1], dC=dC, hA=hA, hC=hC))
            if check is None:
                check = (act[K][0], Bs, ss, len(linears) - 1)
    step_bytes = sum(algorithmic_bytes(M, l["K"], l["N"]) for l in linears)          # whole job, all ranks
    step_ops = sum(2 * M * l["K"] * l["N"] for l in linears)
    gather_out = None
    if world > 1:
        gather_out = torch.zeros((world * M * pad_cols,), dtype=torch.float16, device=dev)

    stream = torch.cuda.Stream(device=dev)

    def enqueue_step(s):
        for l in linears:
            rc = l["ws"].enqueue_f16(l["w"], l["dA"], l["dC"], s.cuda_stream)
            if rc:
                raise RuntimeError(f"enqueue failed: {rc}")
        if world > 1:     # reassemble the column shards on every rank: the one exchange the path has
            with torch.cuda.stream(s):
                dist.all_gather_into_tensor(gather_out, out_buf)

    # ---- correctness of what is timed: first linear of the ring against the oracle
    oracle = Oracle()
    with torch.cuda.stream(stream):
        enqueue_step(stream)
    stream.synchronize()
    A0, B0, s0, idx = check
    ref_out = oracle.linear(A0, B0, s0)[1]
    got = linears[idx]["dC"].cpu().numpy().view(np.uint16)
    if not np.array_equal(got, ref_out):
        raise RuntimeError("CUDA output differs from the oracle; refusing to report a number")
    for l in linears:
        if l["ws"].finish() != 0:
            raise RuntimeError("device status not clean after the check step")
    count0 = sum(l["ws"].launch_count() for l in linears)
    with torch.cuda.stream(stream):
        enqueue_step(stream)
    stream.synchronize()
    launches_per_step = sum(l["ws"].launch_count() for l in linears) - count0   # this library's kernels per step

    # ---- device-resident timing (value)
    graph = None
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                enqueue_step(stream)
        except Exception as exc:   # capture is an optimisation; plain stream launches are the fallback
            print(f"[bench] graph capture unavailable ({type(exc).__name__}: {exc}); using stream launches", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()

    def do_step():
        if graph is not None:
            graph.replay()
        else:
            enqueue_step(stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # The clock sampler starts before the warm-up; the warm-up runs its W steps and then keeps
    # going (same launches) until the sampler has a few rows or three seconds have passed, so
    # that the clocks are recorded under the very load that is timed right after.
    sampler = ClockSampler(local_rank) if rank == 0 else None
    with torch.cuda.stream(stream):
        for _ in range(max(3, args.warmup)):
            do_step()
    barrier()
    t_warm = time.perf_counter()
    while True:
        with torch.cuda.stream(stream):
            for _ in range(50):
                do_step()
        stream.synchronize()
        enough = sampler is None or sampler.proc is None or sampler.samples() >= 4 or time.perf_counter() - t_warm > 3.0
        if world > 1:
            flag = torch.tensor([1 if enough else 0], device=dev)
            dist.broadcast(flag, src=0)
            enough = bool(flag.item())
        if enough:
            break
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(args.steps):
            do_step()
        e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler else None
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / args.steps

    # ---- end to end through the blocking reference ABI, pinned host tensors
    def e2e_step():
        for l in linears:
            rc = l["ws"].run_f16(l["w"], l["hA"], l["hC"])
            if rc:
                raise RuntimeError(f"run_f16 failed: {rc}")

    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    e2e_steps = max(1, min(args.steps, 10))
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    h2d = sum(M * l["K"] * 2 for l in linears)
    d2h = sum(M * (l["n1"] - l["n0"]) * 2 for l in linears)

    # ---- M = 1 beside it (single GPU only, same ring)
    also = {}
    if world == 1 and args.tokens != 1 and not args.quick:
        also["M1_GBps"] = _time_other_m(rk, dom, linears, 1, args, dev, stream)

    if world == 1 and not args.quick:
        also["independent_linears_4_streams_GBps"] = _time_streams(linears, step_bytes, args, dev, 4)
        also.update(_prefill_and_ffn(rk, dom, dev, stream, oracle, make_weights, make_activations, sample_columns))

    if world > 1 and not args.quick:
        try:
            also.update(_prefill_sharded(rk, dom, dev, stream, dist, world, rank, make_weights, make_activations, shard_columns))
        except Exception as exc:   # the extra figure must never cost the headline line
            also["prefill_sharded_error"] = f"{type(exc).__name__}: {exc}"
        try:
            also.update(_ffn_sharded(rk, dom, dev, stream, dist, world, rank, make_weights, make_activations))
        except Exception as exc:
            also["ffn_sharded_error"] = f"{type(exc).__name__}: {exc}"

    # ---- CPU baseline on a bounded sample (rank 0, one GPU only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_baseline(M, Reference if Reference.available() else None, oracle, make_weights, make_activations)

    if rank == 0:
        launches = launches_per_step * args.steps
        value = step_bytes / (ms_step * 1e-3) / 1e9
        gemm_bytes_per_launch = step_bytes / len(linears) / world   # what one rank's launch reads
        line = {"metric": "w4a8_decode_weight_stream", "value": value, "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                "config": workload_config(args, world, args.layers),
                "tops": step_ops / (ms_step * 1e-3) / 1e12,
                "launch_mode": "cuda_graph" if graph is not None else "stream",
                "clocks": clocks,
                "e2e": {"value": step_bytes / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                        "d2h_bytes_per_step": d2h, "ms_per_step": 1e3 * e2e_s},
                "gpu_launches": launches,
                "roofline": {"bound": "hbm", "achieved": value / world, "peak": hbm_peak, "unit": "GB/s",
                             "frac": value / world / hbm_peak,
                             # ncu (profiles/gemm_fused_kernel_decode_M8.md): 8,525,824 B read + 0 B written for the
                             # 4096 x 4096 linear whose algorithmic bytes are 8,536,064; traffic is one read per
                             # weight byte, so it scales with the bytes of the ring's average linear
                             "traffic": gemm_bytes_per_launch * (8525824.0 / 8536064.0), "peak_kind": peak_kind,
                             "kernel": "gemm_fused_kernel (scan + quantise + GEMM + dequantise in one launch)",
                             "frac_of_nominal": value / world / 8000.0, "nominal_peak": 8000.0,   # 8 TB/s data-sheet HBM3e
                             "bytes_per_launch": gemm_bytes_per_launch,
                             "us_per_launch": 1e3 * ms_step / len(linears)},
                "cpu_baseline": cpu, "also": also}
        print(json.dumps(line), flush=True)
    if world > 1:
        # The captured graph holds NCCL kernels; tearing the communicator down under it has hung at
        # exit.  Everything is finished: meet once more, then leave without running destructors.
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    for l in linears:
        l["ws"].free()
        l["w"].free()


def _time_other_m(rk, dom, linears, M, args, dev, stream):
    import torch
    from rknpu2_matmul_open_b200.synthetic import make_activations
    extra = []
    act = {K: torch.from_numpy(make_activations(M, K, seed=K, dtype="f16").view(np.int16)).to(dev) for K in (4096, 11008)}
    for l in linears:
        ws = rk.Workspace(dom, rk.default_config(M, l["n1"] - l["n0"], l["K"], k_tile=480))
        extra.append((ws, l["w"], act[l["K"]], torch.zeros((M, l["n1"] - l["n0"]), dtype=torch.int16, device=dev), l))

    def step():
        for ws, w, dA, dC, _ in extra:
            ws.enqueue_f16(w, dA, dC, stream.cuda_stream)

    graph = None
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step()
        except Exception:
            graph = None
            torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        for _ in range(3):
            graph.replay() if graph else step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay() if graph else step()
        e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    total = sum(algorithmic_bytes(M, l["K"], l["N"]) for l in linears)
    for ws, *_ in extra:
        ws.free()
    return total / (ms * 1e-3) / 1e9


def _time_streams(linears, step_bytes, args, dev, n_streams):
    """The same ring with its linears dealt round-robin onto `n_streams` CUDA streams (they are independent
    problems: own inputs, outputs and workspaces), captured as one graph with parallel branches.  The headline
    value keeps them on one stream, where each launch waits for the one in front."""
    import torch
    main = torch.cuda.Stream(device=dev)
    side = [torch.cuda.Stream(device=dev) for _ in range(n_streams)]

    def step():
        for s in side:
            s.wait_stream(main)
        for i, l in enumerate(linears):
            s = side[i % n_streams]
            with torch.cuda.stream(s):
                rc = l["ws"].enqueue_f16(l["w"], l["dA"], l["dC"], s.cuda_stream)
                if rc:
                    raise RuntimeError(f"enqueue failed: {rc}")
        for s in side:
            main.wait_stream(s)

    torch.cuda.synchronize()
    graph = None
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=main):
                step()
        except Exception as exc:
            print(f"[bench] multi-stream capture unavailable ({type(exc).__name__}: {exc})", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
    with torch.cuda.stream(main):
        for _ in range(3):
            graph.replay() if graph else step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(main):
        e0.record(main)
        for _ in range(args.steps):
            graph.replay() if graph else step()
        e1.record(main)
    torch.cuda.synchronize()
    return step_bytes / (e0.elapsed_time(e1) / args.steps * 1e-3) / 1e9


INT8_PEAK_TOPS = 4550.0   # dense int8 tcgen05 peak measured on this pool's B200 with lib/int8_peak (burst, 1965 MHz)


def _event_time(torch, stream, fn, reps):
    with torch.cuda.stream(stream):
        for _ in range(3):
            fn()
    stream.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(reps):
            fn()
        e1.record(stream)
    stream.synchronize()
    return e0.elapsed_time(e1) / reps


def _prefill_and_ffn(rk, dom, dev, stream, oracle, make_weights, make_activations, sample_columns):
    """Benchmark configuration 2 (prefill GEMM 2048 x 4096 x 14336, fp16) and config 3 (fused FFN 4096 -> 2 x 14336 -> 4096,
    M = 1 and 1024), device-resident, each checked against the oracle on sampled columns / rows."""
    import torch
    out = {}
    M, K, N = 2048, 4096, 14336
    B, sw = make_weights(K, N, seed=21)
    A = make_activations(M, K, seed=21, dtype="f16")
    w = rk.Weights(dom, B, sw)
    ws = rk.Workspace(dom, rk.default_config(M, N, K))
    dA = torch.from_numpy(A.view(np.int16)).to(dev)
    dC = torch.zeros((M, N), dtype=torch.int16, device=dev)
    ms = _event_time(torch, stream, lambda: ws.enqueue_f16(w, dA, dC, stream.cuda_stream), 10)
    cols = sample_columns(N)
    _, s, inv = oracle.scales(A)
    ref = oracle.dequant(oracle.gemm_i32_columns(oracle.quantize(A, inv), B, cols), s, sw[cols], True)
    exact = bool(np.array_equal(dC.cpu().numpy().view(np.uint16)[:, cols], ref))
    tops = 2.0 * M * K * N / (ms * 1e-3) / 1e12
    out["prefill_M2048_K4096_N14336"] = {"us": ms * 1e3, "tops": tops, "frac_of_measured_int8_peak": tops / INT8_PEAK_TOPS,
                                         "peak_tops": INT8_PEAK_TOPS, "frac_of_nominal_4500": tops / 4500.0, "sampled_exact": exact,
                                         "includes": "quantise kernel + tcgen05 GEMM"}
    ws.free()
    w.free()
    # the one complete-call figure the original project publishes: binary16, M = 128, K = 11008, N = 4096
    # (about 4.0 ms on its RK3588 target)
    M, K, N = 128, 11008, 4096
    B, sw = make_weights(K, N, seed=22)
    A = make_activations(M, K, seed=22, dtype="f16")
    w = rk.Weights(dom, B, sw)
    ws = rk.Workspace(dom, rk.default_config(M, N, K))
    dA = torch.from_numpy(A.view(np.int16)).to(dev)
    dC = torch.zeros((M, N), dtype=torch.int16, device=dev)
    ms = _event_time(torch, stream, lambda: ws.enqueue_f16(w, dA, dC, stream.cuda_stream), 10)
    cols = sample_columns(N)
    _, s, inv = oracle.scales(A)
    ref = oracle.dequant(oracle.gemm_i32_columns(oracle.quantize(A, inv), B, cols), s, sw[cols], True)
    out["published_shape_M128_K11008_N4096"] = {
        "us": ms * 1e3, "tops": 2.0 * M * K * N / (ms * 1e-3) / 1e12, "published_ms_on_rk3588": 4.0,
        "sampled_exact": bool(np.array_equal(dC.cpu().numpy().view(np.uint16)[:, cols], ref))}
    ws.free()
    w.free()
    K, F, N = 4096, 14336, 4096
    Bg, sg = make_weights(K, 2 * F, seed=31)
    Bd, sd = make_weights(F, N, seed=32)
    wg, wd = rk.Weights(dom, Bg, sg), rk.Weights(dom, Bd, sd)
    for M in (1, 128, 1024):
        A = make_activations(M, K, seed=31, dtype="f32")
        g = rk.Workspace(dom, rk.default_config(M, 2 * F, K))
        d = rk.Workspace(dom, rk.default_config(M, N, F))
        dA = torch.from_numpy(A).to(dev)
        dM = torch.zeros((M, F), dtype=torch.float32, device=dev)
        dC = torch.zeros((M, N), dtype=torch.float32, device=dev)
        ms = _event_time(torch, stream, lambda: rk.enqueue_ffn_f32(g, wg, d, wd, dA, dM, dC, stream.cuda_stream), 10)
        rows = min(M, 2)
        ref = oracle.ffn(A[:rows], Bg, sg, Bd, sd, mode=1)
        exact = bool(np.array_equal(dC.cpu().numpy()[:rows].view(np.uint32), ref["C"].view(np.uint32)))
        weight_bytes = K * 2 * F // 2 + F * N // 2
        out[f"ffn_M{M}"] = {"us": ms * 1e3, "weight_GBps": weight_bytes / (ms * 1e-3) / 1e9,
                            "tops": 2.0 * M * (K * 2 * F + F * N) / (ms * 1e-3) / 1e12, "rows_checked_exact": exact}
        g.free()
        d.free()
    wg.free()
    wd.free()
    return out


def _prefill_sharded(rk, dom, dev, stream, dist, world, rank, make_weights, make_activations, shard_columns):
    """Benchmark configuration 2 column-sharded over the ranks: every rank runs the 2048 x 4096 prefill GEMM on its run of
    64-column blocks of N = 14336; figures are whole-job TOPS from the slowest rank's device time, without and
    with the all-gather that reassembles the [M, N] output on every rank."""
    import torch
    M, K, N = 2048, 4096, 14336
    B, sw = make_weights(K, N, seed=21)
    A = make_activations(M, K, seed=21, dtype="f16")
    n0, n1 = shard_columns(N, world, rank)
    w = rk.Weights(dom, np.ascontiguousarray(B[:, n0:n1]), np.ascontiguousarray(sw[n0:n1]))
    ws = rk.Workspace(dom, rk.default_config(M, n1 - n0, K))
    dA = torch.from_numpy(A.view(np.int16)).to(dev)
    widest = max(b - a for a, b in (shard_columns(N, world, r) for r in range(world)))
    dC = torch.zeros((M * widest,), dtype=torch.float16, device=dev)          # equal pieces for the collective
    parts = torch.zeros((world * M * widest,), dtype=torch.float16, device=dev)

    def compute():
        rc = ws.enqueue_f16(w, dA, dC, stream.cuda_stream)
        if rc:
            raise RuntimeError(f"enqueue failed: {rc}")

    def with_gather():
        compute()
        dist.all_gather_into_tensor(parts, dC)

    out = {}
    for name, fn in (("compute", compute), ("compute_plus_all_gather", with_gather)):
        ms = _event_time(torch, stream, fn, 10)
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        out[name] = {"us": ms * 1e3, "tops": 2.0 * M * K * N / (ms * 1e-3) / 1e12}
    ws.free()
    w.free()
    return {"prefill_M2048_K4096_N14336_sharded": out}


def _ffn_sharded(rk, dom, dev, stream, dist, world, rank, make_weights, make_activations):
    """Benchmark configuration 4: the 70B-shaped FFN (hidden 8192, intermediate 28672) column-sharded over the ranks.
    Gate and up are sharded by the same feature slice so SwiGLU stays local.  The down projection contracts over
    all of F with the scale of the whole row: the ranks all-reduce (max) their slice maxima, quantise their slice
    with the combined scale and all-gather the int8 codes; the down projection is sharded by output columns and
    its outputs are all-gathered.  A maximum is a maximum however it is grouped, so results stay bit-exact."""
    import torch
    from rknpu2_matmul_open_b200.sharding import gather_columns, shard_columns, shard_ffn_weights, shard_weights
    K, F, N = 8192, 28672, 8192
    # weights with the benchmark's value distribution, generated once for a 2048-column block and repeated along N
    # (generating 700 M codes from fp32 normals would take most of a minute per rank; only time is measured here)
    blk_g, blk_sg = make_weights(K, 2048, seed=41)
    blk_d, blk_sd = make_weights(F, 2048, seed=42)
    Bg, sg = np.tile(blk_g, (1, 2 * F // 2048)), np.tile(blk_sg, 2 * F // 2048)
    Bd, sd = np.tile(blk_d, (1, N // 2048)), np.tile(blk_sd, N // 2048)
    Bg_s, sg_s, (f0, f1) = shard_ffn_weights(Bg, sg, world, rank)
    Bd_s, sd_s, (n0, n1) = shard_weights(Bd, sd, world, rank)
    del Bg, Bd
    wg, wd = rk.Weights(dom, Bg_s, sg_s), rk.Weights(dom, Bd_s, sd_s)
    out = {}
    for M in (32, 1024, 4096):
        A = make_activations(M, K, seed=41, dtype="f32")
        gu = rk.Workspace(dom, rk.default_config(M, 2 * (f1 - f0), K))
        dn = rk.Workspace(dom, rk.default_config(M, n1 - n0, F))
        dA = torch.from_numpy(A).to(dev)
        dMid = torch.zeros((M, f1 - f0), dtype=torch.float32, device=dev)
        dC = torch.zeros((M, n1 - n0), dtype=torch.float32, device=dev)

        # Equal feature slices that are multiples of 16: the ranks exchange int8 codes (a quarter of the fp32
        # middle's bytes) after agreeing on the row maxima; otherwise the fp32 middle is gathered.
        even = (F // 64) % world == 0 and (N // 64) % world == 0
        if even:
            maxima = torch.zeros(M, dtype=torch.int32, device=dev)
            codes = torch.empty((M, f1 - f0), dtype=torch.int8, device=dev)
            code_parts = torch.empty((world, M, f1 - f0), dtype=torch.int8, device=dev)
            out_parts = torch.empty((world, M, n1 - n0), dtype=torch.float32, device=dev)
            out_full = torch.empty((M, N), dtype=torch.float32, device=dev)
            mid_parts = torch.empty((world, M, f1 - f0), dtype=torch.float32, device=dev)
            mid_full = torch.empty((M, F), dtype=torch.float32, device=dev)

        def step(codes_exchange=even):
            if codes_exchange:
                rc = gu.enqueue_swiglu_collect_f32(wg, dA, dMid, maxima, stream.cuda_stream)
                dist.all_reduce(maxima, op=dist.ReduceOp.MAX)        # bit patterns of non-negative floats order like ints
                rc = rc or gu.enqueue_quantize_slice(dMid, maxima, codes, stream.cuda_stream)
                dist.all_gather_into_tensor(code_parts, codes)
                rc = rc or dn.enqueue_codes_f32(wd, code_parts, world, maxima, dC, stream.cuda_stream)
                if rc:
                    raise RuntimeError(f"enqueue failed: {rc}")
                dist.all_gather_into_tensor(out_parts, dC)
                out_full.view(M, world, n1 - n0).copy_(out_parts.permute(1, 0, 2))
                return out_full
            rc = gu.enqueue_swiglu_f32(wg, dA, dMid, stream.cuda_stream)
            if even:   # equal shards: one collective into [world, M, cols] and one strided copy into [M, world * cols]
                dist.all_gather_into_tensor(mid_parts, dMid)
                mid_full.view(M, world, f1 - f0).copy_(mid_parts.permute(1, 0, 2))
                middle = mid_full
            else:
                middle = gather_columns(dMid, F)                   # [M, F] on every rank, shards padded to the widest
            rc = rc or dn.enqueue_f32(wd, middle, dC, stream.cuda_stream)   # rescans the gathered rows: same maxima
            if rc:
                raise RuntimeError(f"enqueue failed: {rc}")
            if even:
                dist.all_gather_into_tensor(out_parts, dC)
                out_full.view(M, world, n1 - n0).copy_(out_parts.permute(1, 0, 2))
                return out_full
            return gather_columns(dC, N)

        # Both exchanges are timed where both apply: with few tokens the extra all-reduce of the code exchange
        # costs more than the bytes it saves; every rank takes the same (max-reduced) decision.
        timed = {}
        for name, flag in ([("int8 codes", True)] if even else []) + [("fp32 middle", False)]:
            t = torch.tensor([_event_time(torch, stream, lambda: step(flag), 5)], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            timed[name] = float(t.item())
        best = min(timed, key=timed.get)
        ms = timed[best]
        weight_bytes = K * 2 * F // 2 + F * N // 2
        out[f"M{M}"] = {"us": ms * 1e3, "weight_GBps_whole_job": weight_bytes / (ms * 1e-3) / 1e9,
                        "tops_whole_job": 2.0 * M * (K * 2 * F + F * N) / (ms * 1e-3) / 1e12,
                        "exchange": best, "us_by_exchange": {k: v * 1e3 for k, v in timed.items()}}
        gu.free()
        dn.free()
    wg.free()
    wd.free()
    return {"ffn_8192_28672_sharded": out}


def cpu_baseline(M, Reference, oracle, make_weights, make_activations):
    """One decoder layer's seven linears on the host, reference stages when built."""
    shapes, counts = [(4096, 4096), (4096, 11008), (11008, 4096)], [4, 2, 1]
    ref = Reference() if Reference else None
    prepared = []
    for i, (K, N) in enumerate(shapes):
        B, sw = make_weights(K, N, seed=i)
        A = make_activations(M, K, seed=i, dtype="f16")
        prepared.append((K, N, B, sw, A, ref.layer(B, sw, 480) if ref else None))
    best = None
    for _ in range(3):
        t0 = time.perf_counter()
        for (K, N, B, sw, A, handle), count in zip(prepared, counts):
            for _ in range(count):
                if ref:
                    ref.layer_run(handle[0], handle[1], A, threads=4)
                else:
                    oracle.linear(A, B, sw)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    total = sum(algorithmic_bytes(M, K, N) * c for (K, N), c in zip(shapes, counts))
    cores = ref.host_threads() if ref else int(os.environ.get("OMP_NUM_THREADS", os.cpu_count() or 1))
    return {"value": total / best / 1e9, "unit": "GB/s", "cores": cores, "kind": "reference" if ref else "port",
            "sample": f"one decoder layer (7 linears) at M={M}, best of 3 passes, {best * 1e3:.1f} ms per pass"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--tokens", type=int, default=8, help="decode batch M (benchmark configuration 1 uses 1 and 8)")
    ap.add_argument("--layers", type=int, default=4, help="distinct decoder layers in the ring (4 = 405 MB of int4)")
    ap.add_argument("--distinct-values", action="store_true", help="different weight values per ring layer (slower setup)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--quick", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    run_cuda(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
