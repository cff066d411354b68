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

N > 1 (torchrun, one rank per GPU): every rank opens a GROUP context; the library itself
shards each weight by output columns (contiguous 64-column blocks, the reference's
per-core split), runs this rank's columns and reassembles outputs with its own NCCL
communicator -- torch.distributed only carries the group id and the timing reductions.
The device-resident figure keeps column-parallel outputs sharded and gathers them once per
step; the end-to-end figure uses the blocking call, which gathers inside every call.
Total work is fixed, so scaling is "strong".

`--case decode|prefill|mid|ffn|moe|rmsnorm` runs a small fixed workload for a kernel profiler instead.

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
    sample = (f"a step of this arm is ONE decoder layer of the ring (4x 4096->4096, 2x 4096->11008, 1x 11008->4096) at M={M}; "
              + ("reference CPU stages (scan, MSD pack, INT16 reconstruct, dequant: 4 threads) around an "
                 "all-core int4 stand-in for the NPU step" if use_ref else "C port of the reference path"))
    line = {"impl": "reference", "metric": "w4a8_decode_weight_stream", "value": gbs, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": workload_config(args, world, args.layers),
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


def _max_over_ranks(torch, dist, dev, world, value):
    if world == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _all_ranks_agree(torch, dist, dev, world, ok):
    if world == 1:
        return bool(ok)
    t = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item())


def _graph_of(torch, stream, fn, enabled=True):
    if not enabled:
        return None
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            fn()
        return graph
    except Exception as exc:   # capture is an optimisation; plain stream launches are the fallback
        print(f"[bench] graph capture unavailable ({type(exc).__name__}: {exc}); using stream launches", file=sys.stderr)
        torch.cuda.synchronize()
        return None


def open_context(rk, torch, dist, rank, world, local_rank, dev):
    """One GPU: an ordinary context.  Several: every rank opens a group context -- the library shards the
    weights, runs this rank's columns and all-gathers over NVLink with its own NCCL communicator;
    torch.distributed only carries the 128-byte group id and the timing reductions."""
    if world == 1:
        return rk.Context(f"cuda:{local_rank}")
    ident = torch.zeros(128, dtype=torch.uint8, device=dev)
    if rank == 0:
        raw = (__import__("ctypes").c_ubyte * 128)()
        if rk.capi.load().rk_npu_b200_group_id(raw):
            raise RuntimeError("rk_npu_b200_group_id failed (NCCL not loadable)")
        ident.copy_(torch.tensor(list(raw), dtype=torch.uint8))
    dist.broadcast(ident, src=0)
    return rk.Context.open_group(f"cuda:{local_rank}", rank, world, bytes(ident.cpu().numpy().tobytes()))


def shard_of(N, world, rank):
    """Columns a rank holds (the library's rule): N % 128 == 0 -> the same slice of both halves of N, else one run."""
    from rknpu2_matmul_open_b200.sharding import shard_columns
    if world > 1 and N % 128 == 0:
        f0, f1 = shard_columns(N // 2, world, rank)
        return np.r_[f0:f1, N // 2 + f0:N // 2 + f1]
    n0, n1 = shard_columns(N, world, rank)
    return np.arange(n0, n1)


def measure_int8_peak():
    """Dense int8 tensor peak of this GPU, measured now: the issue loop of csrc/int8_peak.cu (bare tcgen05.mma
    kind::i8 on resident operands, every SM) run for a fraction of a second, with the SM clock sampled meanwhile."""
    exe = ROOT / "rknpu2_matmul_open_b200" / "lib" / "int8_peak"
    if not exe.exists():
        return None
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    try:
        run = subprocess.run([str(exe), "60000"], capture_output=True, text=True, timeout=120)
        out = run.stdout + run.stderr
    except (OSError, subprocess.TimeoutExpired) as exc:
        out = f"{type(exc).__name__}: {exc}"
    clocks = sampler.stop()
    best = 0.0
    for line in out.splitlines():
        if "N=256" in line and "TOPS (event)" in line:
            try:
                best = max(best, float(line.split("->")[1].split("TOPS")[0]))
            except (IndexError, ValueError):
                pass
    if not best:
        print(f"[bench] int8 peak tool gave no figure: {out[-400:]!r}", file=sys.stderr)
        return None
    return {"tops": best, "sm_mhz": clocks["sm_mhz"], "reasons": clocks["reasons"],
            "how": "lib/int8_peak 60000: 128x256x32 kind::i8 MMAs back to back on every SM, best of the runs"}


def run_cuda(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    import rknpu2_matmul_open_b200 as rk
    from oracle.harness import Oracle, Reference            # checker of what is timed, and the cpu_baseline leg
    from rknpu2_matmul_open_b200.synthetic import make_activations, make_weights, sample_columns

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # stdout carries the one JSON line only: NCCL's version banner (NCCL_DEBUG=VERSION) would precede it
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)
    ctx = open_context(rk, torch, dist, rank, world, local_rank, dev)
    dom = ctx.domain(0)
    M = args.tokens
    hbm_peak, _, peak_kind = measured_peaks()
    oracle = Oracle()
    stream = torch.cuda.Stream(device=dev)

    # ---- the ring: `layers` distinct decoder layers.  Every rank passes the FULL weights; a group context keeps
    # its columns.  The device-resident figure computes this rank's columns of all linears into one buffer and
    # reassembles them with ONE all-gather per step (column-parallel outputs stay sharded until somebody needs
    # all of them); the end-to-end figure goes through the blocking reference call, which gathers per linear.
    act = {K: make_activations(M, K, seed=K, dtype="f16") for K in (4096, 11008)}
    dact = {K: torch.from_numpy(a.view(np.int16)).to(dev) for K, a in act.items()}
    generated, linears = {}, []
    for layer in range(args.layers):
        for j, (K, N) in enumerate(LLAMA7B_LAYER):
            seed = (layer * 16 + j) if args.distinct_values else j
            if (K, N, seed) not in generated:
                generated[(K, N, seed)] = make_weights(K, N, seed=seed)
            B, sw = generated[(K, N, seed)]
            w = rk.Weights(dom, B, sw, k_tile=480)
            ws = rk.Workspace(dom, rk.default_config(M, N, K, k_tile=480))
            cols = ws.shard()[3]
            linears.append(dict(K=K, N=N, seed=seed, w=w, ws=ws, cols=cols, dA=dact[K],
                                hA=torch.from_numpy(act[K].view(np.int16)).pin_memory(),
                                hC=torch.zeros((M, N), dtype=torch.int16).pin_memory()))
    # slot of a rank in the step's output buffer: its linears' compact [M][columns] blocks one after the other,
    # padded to the widest rank so that every piece of the all-gather has one size
    def slot_elems(r):
        return sum(M * len(shard_of(l["N"], world, r)) for l in linears)
    slot = max(slot_elems(r) for r in range(world))
    out_buf = torch.zeros((world * slot,), dtype=torch.int16, device=dev)
    offset = rank * slot
    for l in linears:
        l["dC"] = out_buf[offset:offset + M * l["cols"]].view(M, l["cols"])
        offset += M * l["cols"]
    step_bytes = sum(algorithmic_bytes(M, l["K"], l["N"]) for l in linears)          # whole job, all ranks
    step_ops = sum(2 * M * l["K"] * l["N"] for l in linears)

    def enqueue_step(s):
        for l in linears:
            rc = l["ws"].enqueue_local_f16(l["w"], l["dA"], l["dC"], s.cuda_stream)
            if rc:
                raise RuntimeError(f"enqueue failed: {rc}")
        if world > 1:     # reassemble the column shards on every rank: the one exchange the path has
            rc = ctx.all_gather(out_buf, slot * 2, s.cuda_stream)
            if rc:
                raise RuntimeError(f"all-gather failed: {rc}")

    # ---- correctness of what is timed: the first linear, reassembled from ALL ranks' pieces, against the oracle
    with torch.cuda.stream(stream):
        enqueue_step(stream)
    stream.synchronize()
    first = linears[0]
    ref_out = oracle.linear(act[first["K"]], *generated[(first["K"], first["N"], first["seed"])])[1]
    gathered = out_buf.cpu().numpy().view(np.uint16)
    for r in range(world):
        cols = shard_of(first["N"], world, r)
        piece = gathered[r * slot:r * slot + M * len(cols)].reshape(M, len(cols))
        if not np.array_equal(piece, ref_out[:, cols]):
            raise RuntimeError(f"rank {rank}: the output gathered from rank {r} differs from the oracle; refusing to report a number")
    for l in linears:
        if l["ws"].finish() != 0:
            raise RuntimeError("device status not clean after the check step")
    count0 = sum(l["ws"].launch_count() for l in linears)
    with torch.cuda.stream(stream):
        enqueue_step(stream)
    stream.synchronize()
    launches_per_step = sum(l["ws"].launch_count() for l in linears) - count0   # this library's kernels per step

    # ---- device-resident timing (value)
    graph = _graph_of(torch, stream, lambda: enqueue_step(stream), not args.no_graph)

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
    ms = _max_over_ranks(torch, dist, dev, world, e0.elapsed_time(e1))
    clocks = sampler.stop() if sampler else None
    ms_step = ms / args.steps

    # ---- end to end through the blocking reference ABI, pinned host tensors (a group gathers inside every call)
    def e2e_step():
        for l in linears:
            rc = l["ws"].run_f16(l["w"], l["hA"], l["hC"])
            if rc:
                raise RuntimeError(f"run_f16 failed: {rc}")

    for _ in range(2):
        e2e_step()
    if not np.array_equal(first["hC"].numpy().view(np.uint16), ref_out):
        raise RuntimeError("blocking call: output differs from the oracle")
    barrier()
    t0 = time.perf_counter()
    e2e_steps = max(1, min(args.steps, 10))
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = _max_over_ranks(torch, dist, dev, world, (time.perf_counter() - t0) / e2e_steps)
    h2d = sum(M * l["K"] * 2 for l in linears)
    d2h = sum(M * l["N"] * 2 for l in linears)

    also = {}
    if world == 1 and not args.quick:
        if args.tokens != 1:
            also["M1_GBps"] = _time_other_m(rk, dom, linears, 1, args, dev, stream)
        also["independent_linears_4_streams_GBps"] = _time_streams(linears, step_bytes, args, dev, 4)
        try:
            also["layer_dependencies_only_GBps"] = _time_batched(rk, dom, M, linears, step_bytes, args, stream)
        except RuntimeError as exc:      # a forced kernel family without the batch form
            also["layer_dependencies_only_error"] = str(exc)
    if not args.quick:
        peak = measure_int8_peak() if rank == 0 else None
        for name, fn in (("prefill", _prefill), ("ffn_4096_14336", _ffn_llama8b), ("ffn_8192_28672", _ffn_70b), ("moe", _moe),
                         ("add_rmsnorm", _add_rmsnorm)):
            try:
                also.update(fn(rk, ctx, dom, dev, stream, oracle, dist, world, rank, peak))
            except Exception as exc:   # an extra figure must never cost the headline line
                also[f"{name}_error"] = f"{type(exc).__name__}: {exc}"
        if peak:
            also["int8_peak_measured_now"] = peak

    # ---- CPU baseline on a bounded sample (rank 0, one GPU only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_baseline(M, Reference if Reference.available() else None, oracle, make_weights, make_activations)

    if rank == 0:
        value = step_bytes / (ms_step * 1e-3) / 1e9
        bytes_per_launch = step_bytes / len(linears) / world   # what one rank's launch reads
        line = {"metric": "w4a8_decode_weight_stream", "value": value, "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                "config": workload_config(args, world, args.layers),
                "tops": step_ops / (ms_step * 1e-3) / 1e12,
                "launch_mode": "cuda_graph" if graph is not None else "stream",
                "clocks": clocks,
                "e2e": {"value": step_bytes / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                        "d2h_bytes_per_step": d2h, "ms_per_step": 1e3 * e2e_s},
                "gpu_launches": launches_per_step * args.steps,
                "roofline": {"bound": "hbm", "achieved": value / world, "peak": hbm_peak, "unit": "GB/s",
                             "frac": value / world / hbm_peak,
                             # one read per weight byte (ncu: DRAM bytes read equal the algorithmic bytes to 0.1 %), so the
                             # traffic of a launch is its algorithmic bytes
                             "traffic": bytes_per_launch, "peak_kind": peak_kind,
                             "kernel": {3: "gemm_fused_kernel (split-K clusters)", 5: "gemm_decode_kernel (whole-K CTAs)"}.get(
                                 linears[0]["ws"].schedule()[0], "quantize_kernel + gemm_mma_kernel") + ": scan + quantise + GEMM + dequantise",
                             "frac_of_nominal": value / world / 8000.0, "nominal_peak": 8000.0,   # 8 TB/s data-sheet HBM3e
                             "bytes_per_launch": bytes_per_launch,
                             "us_per_launch": 1e3 * ms_step / len(linears)},
                "cpu_baseline": cpu, "also": also}
        print(json.dumps(line), flush=True)
    torch.cuda.synchronize()
    if world > 1:
        # Everything is measured and printed.  Communicators that captured graphs still refer to have hung in their
        # teardown (NCCL's destroy waits for those references), so a group run ends here: the ranks meet on the
        # host-side store (no collective, bounded wait) and leave without tearing anything down.
        sys.stdout.flush()
        sys.stderr.flush()
        try:
            store = dist.distributed_c10d._get_default_store()
            store.add("bench_done", 1)
            limit = time.time() + 60
            while int(store.add("bench_done", 0)) < world and time.time() < limit:
                time.sleep(0.05)
        finally:
            os._exit(0)
    for l in linears:
        l["ws"].free()
        l["w"].free()
    dom.free()
    ctx.close()


def _time_other_m(rk, dom, linears, M, args, dev, stream):
    import torch
    from rknpu2_matmul_open_b200.synthetic import make_activations
    extra = []
    act = {K: torch.from_numpy(make_activations(M, K, seed=K, dtype="f16").view(np.int16)).to(dev) for K in (4096, 11008)}
    for l in linears:
        ws = rk.Workspace(dom, rk.default_config(M, l["N"], l["K"], k_tile=480))
        extra.append((ws, l["w"], act[l["K"]], torch.zeros((M, l["N"]), dtype=torch.int16, device=dev)))

    def step():
        for ws, w, dA, dC in extra:
            ws.enqueue_f16(w, dA, dC, stream.cuda_stream)

    with torch.cuda.stream(stream):
        step()
    stream.synchronize()
    graph = _graph_of(torch, stream, step, not args.no_graph)
    ms = _event_time(torch, stream, (graph.replay if graph else step), args.steps)
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
                rc = l["ws"].enqueue_local_f16(l["w"], l["dA"], l["dC"], s.cuda_stream)
                if rc:
                    raise RuntimeError(f"enqueue failed: {rc}")
        for s in side:
            main.wait_stream(s)

    torch.cuda.synchronize()
    with torch.cuda.stream(main):
        step()
    torch.cuda.synchronize()
    graph = _graph_of(torch, main, step, not args.no_graph)
    ms = _event_time(torch, main, (graph.replay if graph else step), args.steps)
    return step_bytes / (ms * 1e-3) / 1e9


def _time_batched(rk, dom, M, linears, step_bytes, args, stream):
    """The same ring with only the dependencies a decoder layer really has: q, k and v read the same activations and
    are independent of each other, so are gate and up.  Each such set goes out as ONE launch
    (rk_npu_b200_w4a8_enqueue_batch_f16); o and down stay launches of their own.  Four launches per layer instead of
    seven, each still waiting for the one in front."""
    import torch
    layers = [linears[i:i + len(LLAMA7B_LAYER)] for i in range(0, len(linears), len(LLAMA7B_LAYER))]
    # the batch form is the decode kernel's: workspaces of their own, scheduled on it whatever the default family is
    own = []
    for l in linears:
        ws = rk.Workspace(dom, rk.default_config(M, l["N"], l["K"]))
        if ws.set_schedule(5, 0) != 0:
            raise RuntimeError("the decode kernel does not run this shape")
        own.append(ws)
    batch_ws = {id(l): ws for l, ws in zip(linears, own)}

    def step():
        for layer in layers:
            for group in (layer[0:3], layer[3:4], layer[4:6], layer[6:7]):    # q|k|v, o, gate|up, down
                rc = rk.enqueue_batch_f16([batch_ws[id(l)] for l in group], [l["w"] for l in group], [l["dA"] for l in group],
                                          [l["dC"] for l in group], stream.cuda_stream)
                if rc:
                    raise RuntimeError(f"batched enqueue failed: {rc}")

    with torch.cuda.stream(stream):
        step()
    stream.synchronize()
    graph = _graph_of(torch, stream, step, not args.no_graph)
    ms = _event_time(torch, stream, (graph.replay if graph else step), args.steps)
    for ws in own:
        if ws.finish() != 0:
            raise RuntimeError("device status not clean after the batched run")
        ws.free()
    return step_bytes / (ms * 1e-3) / 1e9


def _tiled_weights(make_weights, K, N, seed, block=2048):
    """Weights with the benchmark's value distribution, generated for a 2048-column block and repeated along N
    (drawing hundreds of millions of fp32 normals would take most of a minute; only time and parity are measured)."""
    if N <= 2 * block or N % block:
        return make_weights(K, N, seed=seed)
    B, s = make_weights(K, block, seed=seed)
    return np.tile(B, (1, N // block)), np.tile(s, N // block)


def _prefill(rk, ctx, dom, dev, stream, oracle, dist, world, rank, peak):
    """Benchmark configuration 2: prefill GEMM 2048 x 4096 x 14336, fp16 in and out.  One GPU: quantise + GEMM.  A
    group: every rank's columns (compute) and the same with the all-gather and reassembly that leave the whole
    [M, N] tensor on every rank; the gathered tensor is compared with the oracle on sampled columns, all rows."""
    import torch
    from rknpu2_matmul_open_b200.synthetic import make_activations, make_weights, sample_columns
    M, K, N = 2048, 4096, 14336
    B, sw = make_weights(K, N, seed=21)
    A = make_activations(M, K, seed=21, dtype="f16")
    w = rk.Weights(dom, B, sw)
    ws = rk.Workspace(dom, rk.default_config(M, N, K))
    dA = torch.from_numpy(A.view(np.int16)).to(dev)
    dC = torch.zeros((M, N), dtype=torch.int16, device=dev)
    local = torch.zeros((M, ws.shard()[3]), dtype=torch.int16, device=dev)
    cols = sample_columns(N)
    _, s, inv = oracle.scales(A)
    ref = oracle.dequant(oracle.gemm_i32_columns(oracle.quantize(A, inv), B, cols), s, sw[cols], True)
    peak_tops = peak["tops"] if peak else None
    out = {}
    if world == 1:
        ms = _event_time(torch, stream, lambda: ws.enqueue_f16(w, dA, dC, stream.cuda_stream), 10)
        exact = bool(np.array_equal(dC.cpu().numpy().view(np.uint16)[:, cols], ref))
        tops = 2.0 * M * K * N / (ms * 1e-3) / 1e12
        out["prefill_M2048_K4096_N14336"] = {"us": ms * 1e3, "tops": tops, "sampled_exact": exact, "peak_tops_measured_now": peak_tops,
                                             "frac_of_measured_int8_peak": tops / peak_tops if peak_tops else None,
                                             "frac_of_nominal_4500": tops / 4500.0, "includes": "quantise kernel + tcgen05 GEMM"}
        # the one complete-call figure the original project publishes: binary16, M = 128, K = 11008, N = 4096
        # (about 4.0 ms on its RK3588 target)
        ws.free(); w.free()
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
        # next row of the path: the typed W8A8 operator (int8 weights) on the same prefill shape, through its blocking
        # call on device tensors (wall clock of the call, its stream drained inside)
        try:
            out["w8a8_f16_dynamic_M2048_K4096_N14336"] = _w8a8_prefill(rk, dom, dev, oracle, peak_tops)
        except Exception as exc:
            out["w8a8_error"] = f"{type(exc).__name__}: {exc}"
    else:
        timed = {}
        for name, fn in (("compute", lambda: ws.enqueue_local_f16(w, dA, local, stream.cuda_stream)),
                         ("compute_plus_all_gather", lambda: ws.enqueue_f16(w, dA, dC, stream.cuda_stream))):
            ms = _max_over_ranks(torch, dist, dev, world, _event_time(torch, stream, fn, 10))
            timed[name] = {"us": ms * 1e3, "tops_whole_job": 2.0 * M * K * N / (ms * 1e-3) / 1e12}
        exact = _all_ranks_agree(torch, dist, dev, world, np.array_equal(dC.cpu().numpy().view(np.uint16)[:, cols], ref))
        if not exact:
            raise RuntimeError("gathered prefill output differs from the oracle")
        timed["gathered_exact_on_every_rank"] = exact
        out["prefill_M2048_K4096_N14336_sharded"] = timed
    ws.free()
    w.free()
    return out


def _w8a8_prefill(rk, dom, dev, oracle, peak_tops):
    import torch
    from rknpu2_matmul_open_b200 import w8a8
    from rknpu2_matmul_open_b200.synthetic import make_activations, sample_columns
    M, K, N = 2048, 4096, 14336
    rng = np.random.default_rng(23)
    B = rng.integers(-127, 128, size=(K, 2048), dtype=np.int8)
    B = np.tile(B, (1, N // 2048))
    sw = np.tile(rng.uniform(1e-3, 2e-2, size=2048).astype(np.float32), N // 2048)
    A = make_activations(M, K, seed=23, dtype="f16")
    w = w8a8.MatmulWeights(dom, "f16i8f16", B, sw)
    ws = w8a8.MatmulWorkspace(dom, w8a8.default_strategy(w8a8.F16_DYNAMIC, M, N, K))
    dA = torch.from_numpy(A.view(np.int16)).to(dev)
    dC = torch.zeros((M, N), dtype=torch.int16, device=dev)
    for _ in range(3):
        if ws.run_dynamic(w, dA, dC) != 0:
            raise RuntimeError("W8A8 run failed")
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    reps = 10
    for _ in range(reps):
        ws.run_dynamic(w, dA, dC)
    sec = (time.perf_counter() - t0) / reps
    cols = sample_columns(N)
    ref = oracle.w8_linear(A, np.ascontiguousarray(B[:, cols]), sw[cols])
    exact = bool(np.array_equal(dC.cpu().numpy().view(np.uint16)[:, cols], ref["out"]))
    tops = 2.0 * M * K * N / sec / 1e12
    ws.free()
    w.free()
    return {"us": sec * 1e6, "tops": tops, "sampled_exact": exact, "frac_of_measured_int8_peak": tops / peak_tops if peak_tops else None,
            "includes": "w8_quantize_kernel + persistent tcgen05 GEMM with int8 weights + the call's host synchronisation"}


def _check_ffn(oracle, A, Bg, sg, Bd, sd, middle, C):
    """Sampled check of an FFN result: middle on 17 features x all rows; the output on 17 columns x all rows, from the
    given middle's own scales (the staged bar for large shapes); a NULL middle checks the first two rows end to end."""
    from rknpu2_matmul_open_b200.synthetic import sample_columns
    F, N = Bd.shape
    if middle is None:
        rows = min(A.shape[0], 2)
        ref = oracle.ffn(A[:rows], Bg, sg, Bd, sd, mode=1)
        return bool(np.array_equal(C[:rows].view(np.uint32), ref["C"].view(np.uint32)))
    feats = sample_columns(F)
    pair = np.concatenate([feats, feats + F]).astype(np.int32)
    _, s, inv = oracle.scales(A)
    ref_mid, _ = oracle.swiglu(oracle.gemm_i32_columns(oracle.quantize(A, inv), Bg, pair), s, sg[pair], mode=1)
    if not np.array_equal(middle[:, feats].view(np.uint32), ref_mid.view(np.uint32)):
        return False
    cols = sample_columns(N)
    _, s2, inv2 = oracle.scales(middle)
    ref_c = oracle.dequant(oracle.gemm_i32_columns(oracle.quantize(middle, inv2), Bd, cols), s2, sd[cols], False)
    return bool(np.array_equal(C[:, cols].view(np.uint32), ref_c.view(np.uint32)))


def _ffn_figures(rk, ctx, dom, dev, stream, oracle, dist, world, rank, name, K, F, N, batches, seeds):
    import torch
    from rknpu2_matmul_open_b200.synthetic import make_activations, make_weights
    Bg, sg = _tiled_weights(make_weights, K, 2 * F, seeds[0])
    Bd, sd = _tiled_weights(make_weights, F, N, seeds[1])
    wg, wd = rk.Weights(dom, Bg, sg), rk.Weights(dom, Bd, sd)
    weight_bytes = K * 2 * F // 2 + F * N // 2
    out = {}
    for M in batches:
        A = make_activations(M, K, seed=seeds[0], dtype="f32")
        g = rk.Workspace(dom, rk.default_config(M, 2 * F, K))
        d = rk.Workspace(dom, rk.default_config(M, N, F))
        dA = torch.from_numpy(A).to(dev)
        dM = torch.zeros((M, F), dtype=torch.float32, device=dev)
        dC = torch.zeros((M, N), dtype=torch.float32, device=dev)
        # a group may skip the fp32 middle and exchange int8 codes when the caller does not need the middle tensor
        forms = [("middle returned", dM)] + ([("int8 codes exchanged, middle not returned", None)] if world > 1 and (F // 64) % world == 0 else [])
        timed, exact = {}, True
        for label, mid in forms:
            ms = _event_time(torch, stream, lambda: rk.enqueue_ffn_f32(g, wg, d, wd, dA, mid, dC, stream.cuda_stream), 10 if M <= 1024 else 5)
            timed[label] = _max_over_ranks(torch, dist, dev, world, ms)
            ok = _check_ffn(oracle, A, Bg, sg, Bd, sd, dM.cpu().numpy() if mid is not None else None, dC.cpu().numpy())
            exact = exact and _all_ranks_agree(torch, dist, dev, world, ok)
        if not exact:
            raise RuntimeError(f"{name} M={M}: result differs from the oracle")
        best = min(timed, key=timed.get)
        ms = timed[best]
        key = f"{name}_M{M}" if world == 1 else f"M{M}"
        out[key] = {"us": ms * 1e3, "weight_GBps_whole_job": weight_bytes / (ms * 1e-3) / 1e9,
                    "tops_whole_job": 2.0 * M * (K * 2 * F + F * N) / (ms * 1e-3) / 1e12, "checked_exact": exact,
                    "form": best, "us_by_form": {k: v * 1e3 for k, v in timed.items()}}
        g.free()
        d.free()
    wg.free()
    wd.free()
    return out if world == 1 else {f"{name}_sharded": out}


def _ffn_llama8b(rk, ctx, dom, dev, stream, oracle, dist, world, rank, peak):
    """Benchmark configuration 3: fused FFN 4096 -> 2 x 14336 -> 4096 at 1, 128 and 1024 tokens (one GPU only)."""
    if world > 1:
        return {}
    return _ffn_figures(rk, ctx, dom, dev, stream, oracle, dist, world, rank, "ffn", 4096, 14336, 4096, (1, 128, 1024), (31, 32))


def _ffn_70b(rk, ctx, dom, dev, stream, oracle, dist, world, rank, peak):
    """Benchmark configuration 4: the 70B-shaped FFN (hidden 8192, intermediate 28672) at 32 and 4096 tokens, on one GPU
    (the baseline of the scaling figures) and column-sharded inside the library on a group."""
    return _ffn_figures(rk, ctx, dom, dev, stream, oracle, dist, world, rank, "ffn_8192_28672", 8192, 28672, 8192, (32, 4096), (41, 42))


def _moe(rk, ctx, dom, dev, stream, oracle, dist, world, rank, peak):
    """Routed experts (rk_npu_moe_w8): 128 int8 experts + a shared one, hidden 1536, intermediate 512, top-8 -- the
    largest geometry the original documents -- through the blocking host-array entry at 1, 8, 64 and 256 rows.
    Reported per batch: the complete call (host arrays in, host array out), the device time of the three launches
    (measured with events between them, which keeps them from overlapping), the expert weights one call streams and
    the rate that makes; four rows of every result are compared with the oracle bit for bit."""
    if world > 1:
        return {}
    from rknpu2_matmul_open_b200 import capi, moe
    H, I, R, shared, top = 1536, 512, 128, 1, 8
    rng = np.random.default_rng(31)
    E = R + shared
    ex = dict(gate_up=rng.integers(-127, 128, size=(E, H, 2 * I), dtype=np.int8),
              gate_up_scales=rng.uniform(2e-4, 6e-4, size=(E, 2 * I)).astype(np.float32),
              down=rng.integers(-127, 128, size=(E, I, H), dtype=np.int8),
              down_scales=rng.uniform(1e-3, 3e-3, size=(E, H)).astype(np.float32))
    w = moe.MoeWeights(dom, shared_expert=shared, **ex)
    ws = moe.MoeWorkspace(dom, moe.default_config(H, I, R, shared, top, 256))
    out_fig = {}
    for rows in (1, 8, 64, 256):
        codes = rng.integers(-127, 128, size=(rows, H), dtype=np.int8)
        scales = rng.uniform(0.01, 0.05, size=rows).astype(np.float32)
        ids = np.stack([rng.choice(R, size=top, replace=False) for _ in range(rows)]).astype(np.int32)
        routes = rng.uniform(0.05, 0.3, size=(rows, top)).astype(np.float32)
        out = np.zeros((rows, H), np.float32)
        t = capi.MoeTimings()
        stages = None
        for i in range(8):
            if ws.run_quantized(w, codes, scales, ids, routes, out, t) != 0:
                raise RuntimeError("rk_npu_moe_w8_run_quantized failed")
            if i >= 3 and (stages is None or t.gate_us + t.down_us < stages[0] + stages[1]):
                stages = (t.gate_us, t.down_us, t.combine_us)
        t0 = time.perf_counter()
        for _ in range(20):
            ws.run_quantized(w, codes, scales, ids, routes, out, None)
        call_us = (time.perf_counter() - t0) / 20 * 1e6
        check = sorted(set([0, rows // 3, rows // 2, rows - 1]))
        rc, ref = oracle.moe_run(ex, shared, top, codes[check], scales[check], ids[check], routes[check], mode=1)
        exact = rc == 0 and bool(np.array_equal(out[check].view(np.uint32), ref.view(np.uint32)))
        active = len(set(ids.reshape(-1).tolist())) + shared
        weight_bytes = active * 3 * H * I
        out_fig[f"rows_{rows}"] = {"call_us": call_us, "gate_up_us": stages[0], "down_us": stages[1], "combine_us": stages[2],
                                   "active_experts": active, "expert_weight_MB": weight_bytes / 1e6,
                                   "GBps_of_weights_per_call": weight_bytes / (call_us * 1e-6) / 1e9,
                                   "GBps_of_weights_in_the_two_projections": weight_bytes / ((stages[0] + stages[1]) * 1e-6) / 1e9,
                                   "rows_checked_exact": exact}
    ws.free(); w.free()
    # expert paging: one int4 expert of this geometry as a cache record, imported into a slot from ordinary host memory
    # and exchanged into a second bank (rk_npu_moe_quant_import_expert / _swap_slots)
    small = {k: (np.clip(v[:2], -7, 7) if v.dtype == np.int8 else v[:2]) for k, v in ex.items()}
    source = moe.MoeWeights(dom, form="quant", **small)
    hot, stage = moe.MoeWeights.slot_bank(dom, H, I, 2), moe.MoeWeights.slot_bank(dom, H, I, 2)
    record = np.zeros(source.record_bytes(), np.uint8)
    back = np.zeros_like(record)
    ok = source.export_expert(1, record) == 0
    for _ in range(3):
        ok = ok and stage.import_expert(0, record) == 0
    t0 = time.perf_counter()
    for _ in range(20):
        stage.import_expert(0, record)
    import_us = (time.perf_counter() - t0) / 20 * 1e6
    from rknpu2_matmul_open_b200 import rmsnorm
    locked = rmsnorm.Buffer(dom, record.nbytes)         # the same record kept in page-locked memory (rk_npu_mem_alloc)
    pinned = locked.array(np.uint8)
    pinned[:] = record
    for _ in range(3):
        ok = ok and stage.import_expert(0, pinned) == 0
    t0 = time.perf_counter()
    for _ in range(20):
        stage.import_expert(0, pinned)
    import_locked_us = (time.perf_counter() - t0) / 20 * 1e6
    locked.free()
    t0 = time.perf_counter()
    for _ in range(200):
        hot.swap_slot(0, stage, 0)
    swap_us = (time.perf_counter() - t0) / 200 * 1e6
    ok = ok and stage.export_expert(0, back) == 0 and bool(np.array_equal(back, record))
    out_fig["int4_expert_record"] = {"MB": record.nbytes / 1e6, "import_us": import_us, "import_GBps": record.nbytes / (import_us * 1e-6) / 1e9,
                                     "import_from_page_locked_us": import_locked_us,
                                     "import_from_page_locked_GBps": record.nbytes / (import_locked_us * 1e-6) / 1e9,
                                     "swap_slots_us": swap_us, "round_trip_exact": ok}
    for h in (stage, hot, source):
        h.free()
    return {"moe_w8_H1536_I512_E128_shared_top8": out_fig}


def _add_rmsnorm(rk, ctx, dom, dev, stream, oracle, dist, world, rank, peak):
    """Residual add + RMSNorm (rk_npu_add_rmsnorm_f16), the step before the quantised FFN.  Device tensors through the
    enqueue form: 4096 rows of 8192 and of 4096 in both layouts (each tensor set is 268 / 134 MB, larger than L2, and
    the launches rotate over two sets), HBM rate = 4 tensors x 2 M D bytes over the device time; 128 x 4096 and 1 x 4096
    as latency figures (launches queued back to back).  The original's blocking call on its own buffers (page-locked
    host memory the kernel addresses over PCIe) at its two validated shapes, wall clock.  Eight rows of every result
    are compared with the oracle bit for bit."""
    if world > 1:
        return {}
    import torch
    from rknpu2_matmul_open_b200 import rmsnorm
    hbm, _, hbm_source = measured_peaks()
    fig = {}
    rng = np.random.default_rng(41)

    def tensors(M, D):
        x = np.clip(rng.normal(0, 0.8, (M, D)), -3, 3).astype(np.float16).view(np.uint16)
        r = np.clip(rng.normal(0, 0.35, (M, D)), -1.5, 1.5).astype(np.float16).view(np.uint16)
        return x, r

    for M, D, reps in ((4096, 8192, 20), (4096, 4096, 20), (128, 4096, 100), (1, 4096, 100)):
        gamma = (0.75 + 0.5 * np.arange(D) / (D - 1)).astype(np.float16).view(np.uint16)
        plan = rmsnorm.AddRmsNormPlan(dom, rmsnorm.default_config(M, D), gamma)
        x, r = tensors(M, D)
        check = sorted(set(np.linspace(0, M - 1, 8).astype(int).tolist()))
        want_s, want_n = oracle.add_rmsnorm_f16(x[check], r[check], gamma)
        for row_major in (False, True):
            lay = (lambda a: a.reshape(-1)) if row_major else rmsnorm.to_block8
            sets = []
            for _ in range(2 if M > 1024 else 8):
                dx = torch.from_numpy(lay(x).astype(np.int16)).to(dev)
                dr = torch.from_numpy(lay(r).astype(np.int16)).to(dev)
                sets.append((dx, dr, torch.empty_like(dx), torch.empty_like(dx)))
            turn = [0]

            def one():
                dx, dr, ds, dn = sets[turn[0] % len(sets)]
                turn[0] += 1
                if plan.enqueue(M, row_major, dx.data_ptr(), dr.data_ptr(), ds.data_ptr(), dn.data_ptr(), stream.cuda_stream):
                    raise RuntimeError("rk_npu_b200_add_rmsnorm_f16_enqueue failed")

            us = _event_time(torch, stream, one, reps) * 1e3
            ds, dn = sets[0][2].cpu().numpy().view(np.uint16), sets[0][3].cpu().numpy().view(np.uint16)
            if not row_major:
                ds, dn = rmsnorm.from_block8(ds, M, D), rmsnorm.from_block8(dn, M, D)
            exact = bool(np.array_equal(ds.reshape(M, D)[check], want_s) and np.array_equal(dn.reshape(M, D)[check], want_n))
            gbps = 8.0 * M * D / (us * 1e-6) / 1e9
            fig[f"enqueue_{M}x{D}_{'rows' if row_major else 'block8'}"] = {
                "us": us, "GBps": gbps, f"frac_of_{hbm_source}_hbm": gbps / hbm, "rows_checked_exact": exact}
            del sets
        plan.free()
    for M, D in ((1, 4096), (128, 4096)):
        gamma = (0.75 + 0.5 * np.arange(D) / (D - 1)).astype(np.float16).view(np.uint16)
        cfg = rmsnorm.default_config(M, D)
        plan = rmsnorm.AddRmsNormPlan(dom, cfg, gamma)
        bufs = [rmsnorm.Buffer(dom, rmsnorm.query(cfg).tensor_bytes) for _ in range(4)]
        x, r = tensors(M, D)
        bufs[0].array()[:] = rmsnorm.to_block8(x)
        bufs[1].array()[:] = rmsnorm.to_block8(r)
        for _ in range(3):
            if plan.run(*bufs):
                raise RuntimeError("rk_npu_add_rmsnorm_f16_run failed")
        t0 = time.perf_counter()
        for _ in range(50):
            plan.run(*bufs)
        call_us = (time.perf_counter() - t0) / 50 * 1e6
        want_s, want_n = oracle.add_rmsnorm_f16(x, r, gamma)
        exact = bool(np.array_equal(rmsnorm.from_block8(bufs[2].array(), M, D), want_s) and
                     np.array_equal(rmsnorm.from_block8(bufs[3].array(), M, D), want_n))
        fig[f"blocking_{M}x{D}_host_buffers"] = {"call_us": call_us, "exact": exact}
        for b in bufs:
            b.free()
        plan.free()
    return {"add_rmsnorm_f16": fig}


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


# ------------------------------------------------------------------ small fixed workloads for profilers
def _case_weights(rng, K, N):
    B = rng.integers(-7, 8, size=(K, N), dtype=np.int8)
    scale = rng.uniform(0.001, 0.01, size=N).astype(np.float32)
    return B, scale


def _case_activations(rng, M, K, dtype):
    x = rng.standard_normal((M, K)).astype(np.float32)
    x[:, rng.random(K) < 0.005] *= 20.0
    return x.astype(dtype)


def run_case(args):
    """`--case decode|prefill|mid|ffn [--repeat R] [--tokens M] [--stamps]`: a handful of launches of one hot-path
    configuration on seeded synthetic data, so that a kernel profiler can capture one to three launches of the
    kernel of interest in a minute or two (no JSON line, no timing claims):
      decode   the seven Llama-7B decode linears (4 x 4096->4096, 2 x 4096->11008, 11008->4096), M = 8, binary16
      prefill  one 2048 x 4096 x 14336 linear, binary16
      mid      one 128 x 11008 x 8192 linear, binary16 (few tiles, long K)
      ffn      gate/up 4096 -> 2 x 14336, SwiGLU, down 14336 -> 4096 at M = 1024, fp32
      moe      routed experts: 128 + 1 int8 experts, hidden 1536, intermediate 512, top-8, 64 rows (--case-tokens)
      rmsnorm  residual add + RMSNorm, 4096 rows (--case-tokens) of 4096 on device tensors, block-8 layout
    --stamps enables the kernels' phase stamps after the launches, runs the set again (the decode set as one CUDA
    graph, the steady state of a dependent chain) and prints them."""
    import torch

    import rknpu2_matmul_open_b200 as rk

    rng = np.random.default_rng(0)
    ctx = rk.Context()
    dom = ctx.domain(0)
    dev = torch.device("cuda", ctx.device)
    stream = torch.cuda.Stream(device=dev)
    calls = []
    if args.case == "moe":
        # routed experts, the geometry of the bench's `moe` figures; blocking calls with host arrays
        from rknpu2_matmul_open_b200 import moe
        rows = args.case_tokens or 64
        H, I, R, shared, top = 1536, 512, 128, 1, 8
        E = R + shared
        ex = dict(gate_up=rng.integers(-127, 128, size=(E, H, 2 * I), dtype=np.int8),
                  gate_up_scales=rng.uniform(2e-4, 6e-4, size=(E, 2 * I)).astype(np.float32),
                  down=rng.integers(-127, 128, size=(E, I, H), dtype=np.int8),
                  down_scales=rng.uniform(1e-3, 3e-3, size=(E, H)).astype(np.float32))
        w = moe.MoeWeights(dom, shared_expert=shared, **ex)
        ws = moe.MoeWorkspace(dom, moe.default_config(H, I, R, shared, top, max(rows, 1)))
        codes = rng.integers(-127, 128, size=(rows, H), dtype=np.int8)
        scales = rng.uniform(0.01, 0.05, size=rows).astype(np.float32)
        ids = np.stack([rng.choice(R, size=top, replace=False) for _ in range(rows)]).astype(np.int32)
        routes = rng.uniform(0.05, 0.3, size=(rows, top)).astype(np.float32)
        out = np.zeros((rows, H), np.float32)
        t0 = time.perf_counter()
        for _ in range(args.repeat):
            rc = ws.run_quantized(w, codes, scales, ids, routes, out, None)
            if rc:
                raise RuntimeError(f"rk_npu_moe_w8_run_quantized failed: {rc}")
        active = len(set(ids.reshape(-1).tolist())) + shared
        print(f"moe: rows={rows}, {active} active experts ({active * 3 * H * I / 1e6:.1f} MB of int8 weights per call), "
              f"{(time.perf_counter() - t0) / args.repeat * 1e6:.1f} us per call over {args.repeat} calls")
        return
    if args.case == "rmsnorm":
        # residual add + RMSNorm on device tensors: --case-tokens rows (default 4096) of 4096, block-8 layout
        from rknpu2_matmul_open_b200 import rmsnorm
        M, D = args.case_tokens or 4096, 4096
        gamma = (0.75 + 0.5 * np.arange(D) / (D - 1)).astype(np.float16).view(np.uint16)
        plan = rmsnorm.AddRmsNormPlan(dom, rmsnorm.default_config(M, D), gamma)
        dx = (torch.randn(M * D, device=dev) * 0.8).half()
        dr = (torch.randn(M * D, device=dev) * 0.35).half()
        ds, dn = torch.empty_like(dx), torch.empty_like(dx)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            for rep in range(args.repeat):
                if rep == args.repeat - 1:
                    e0.record(stream)
                rc = plan.enqueue(M, False, dx.data_ptr(), dr.data_ptr(), ds.data_ptr(), dn.data_ptr(), stream.cuda_stream)
                if rc:
                    raise RuntimeError(f"rk_npu_b200_add_rmsnorm_f16_enqueue failed: {rc}")
            e1.record(stream)
        stream.synchronize()
        print(f"rmsnorm: {M} x {D}, last launch {e0.elapsed_time(e1) * 1e3:.1f} us ({8 * M * D / 1e6:.0f} MB of tensors)")
        return
    if args.case in ("decode", "prefill", "mid"):
        M = args.case_tokens or {"decode": 8, "prefill": 2048, "mid": 128}[args.case]
        shapes = {"decode": LLAMA7B_LAYER, "prefill": [(4096, 14336)], "mid": [(11008, 8192)]}[args.case]
        for K, N in shapes:
            B, sw = _case_weights(rng, K, N)
            w = rk.Weights(dom, B, sw)
            ws = rk.Workspace(dom, rk.default_config(M, N, K))
            dA = torch.from_numpy(_case_activations(rng, M, K, np.float16).view(np.int16)).to(dev)
            dC = torch.zeros((M, N), dtype=torch.int16, device=dev)
            calls.append((lambda ws=ws, w=w, dA=dA, dC=dC: ws.enqueue_f16(w, dA, dC, stream.cuda_stream), ws))
    else:
        M = args.case_tokens or 1024
        K, F, N = 4096, 14336, 4096
        Bg, sg = _case_weights(rng, K, 2 * F)
        Bd, sd = _case_weights(rng, F, N)
        wg, wd = rk.Weights(dom, Bg, sg), rk.Weights(dom, Bd, sd)
        g = rk.Workspace(dom, rk.default_config(M, 2 * F, K))
        d = rk.Workspace(dom, rk.default_config(M, N, F))
        dA = torch.from_numpy(_case_activations(rng, M, K, np.float32)).to(dev)
        dM = torch.zeros((M, F), dtype=torch.float32, device=dev)
        dC = torch.zeros((M, N), dtype=torch.float32, device=dev)
        calls.append((lambda: rk.enqueue_ffn_f32(g, wg, d, wd, dA, dM, dC, stream.cuda_stream), d))
        calls.append((lambda: 0, g))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for rep in range(args.repeat):
        with torch.cuda.stream(stream):
            if rep == args.repeat - 1:
                e0.record(stream)
            for fn, _ in calls:
                rc = fn()
                if rc:
                    raise RuntimeError(f"enqueue failed: {rc}")
            if rep == args.repeat - 1:
                e1.record(stream)
        stream.synchronize()
    for _, ws in calls:
        if ws.finish() != 0:
            raise RuntimeError("device status not clean")
    print(f"{args.case}: M={M}, last set {e0.elapsed_time(e1) * 1e3:.1f} us for {len(calls)} call(s)")
    if args.stamps:
        _print_stamps(rk, args.case, calls, stream, torch)


def _print_stamps(rk, case, calls, stream, torch):
    lib = rk.capi.load()
    for _, ws in calls:
        lib.rk_npu_b200_w4a8_trace_enable(ws.handle, 1)
    graph = None
    if case == "decode":     # steady state of a dependent chain: replay the set as one CUDA graph
        with torch.cuda.stream(stream):
            for fn, _ in calls:
                fn()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for fn, _ in calls:
                fn()
    for _ in range(3):
        with torch.cuda.stream(stream):
            if graph is not None:
                graph.replay()
            else:
                for fn, _ in calls:
                    fn()
        stream.synchronize()
    torch.cuda.synchronize()
    if graph is not None:
        ms = _event_time(torch, stream, graph.replay, 20)
        print(f"graph replay: {ms * 1e3:.1f} us per set of {len(calls)} linears")
    if case == "decode":
        prev_end = None
        family = calls[0][1].schedule()[0]
        phases = ("before the dependency wait, dependency met, share quantised and sent, all codes landed, last contraction done,"
                  " last output stored" if family == 5 else
                  "weights requested, dependency met, scales known, slice quantised, contraction done, partial sums exchanged")
        print(f"kernel family {family}; per linear, ns relative to the previous linear's last CTA end: first/last CTA start,"
              f" first/last CTA end; then median cycles since CTA start at: {phases}")
        for i, (_, ws) in enumerate(calls):
            buf = np.zeros((4112, 8), np.uint64)
            lib.rk_npu_b200_w4a8_trace_read(ws.handle, buf.ctypes.data, 4112)
            stages = buf[4096:4098].reshape(-1).astype(np.int64)
            scan = buf[4104].astype(np.int64)[:4]
            v = buf[:4096]
            v = v[v[:, 0] > 0].astype(np.int64)
            if not len(v):
                continue
            s0, s1, e0, e1 = v[:, 0].min(), v[:, 0].max(), v[:, 7].min(), v[:, 7].max()
            ref = prev_end if prev_end is not None else s0
            cyc = [int(x) for x in np.median(v[:, 1:7], axis=0)]
            print(f"linear {i}: K={ws.cfg.K} N={ws.cfg.N} ctas={len(v)} start[{s0 - ref},{s1 - ref}] end[{e0 - ref},{e1 - ref}] cycles {cyc}")
            if family == 5:
                print(f"   CTA 0, cycles since its start: loads issued, own maxima in, row maxima known, share quantised: {[int(x) for x in scan]};"
                      f" first weight stages (wait begins, wait ends): {[int(x) for x in stages]}")
            prev_end = e1
    elif case == "prefill":
        raw = np.zeros(256, np.uint64)
        lib.rk_npu_b200_w4a8_trace_read(calls[0][1].handle, raw.ctypes.data, 32)
        print(f"clusters in the grid: {int(raw[200])}; per tile of cluster 0 (cycles since kernel start): MMA issuer begins,"
              " first MMA issued, last commit, epilogue sees the accumulator, tensor memory handed back, tile stored,"
              " cycles the issuer waited for operands | unpack warp: waited for weights, for a free buffer, for activations")
        for j in range(7):
            print(f"tile {j}: {[int(x) for x in raw[j * 8:j * 8 + 7]]} | {int(raw[128 + 2 * j])} {int(raw[129 + 2 * j])} {int(raw[160 + j])}")


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
    ap.add_argument("--case", choices=["decode", "prefill", "mid", "ffn", "moe", "rmsnorm"], help="run a small profiler workload instead of the benchmark")
    ap.add_argument("--repeat", type=int, default=4, help="--case: launch sets")
    ap.add_argument("--case-tokens", type=int, default=0, help="--case: override the batch")
    ap.add_argument("--stamps", action="store_true", help="--case: print the kernels' phase stamps")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.case:
        run_case(args)
        return
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    run_cuda(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
