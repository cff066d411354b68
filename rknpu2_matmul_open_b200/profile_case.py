"""Small fixed workloads for profilers: `python -m rknpu2_matmul_open_b200.profile_case <case>`.

Each case runs a handful of launches of one hot-path configuration on seeded synthetic data
and exits, so that a kernel profiler can capture one to three launches of the kernel of
interest in a minute or two.  Cases:

  decode   the seven Llama-7B decode linears (4 x 4096->4096, 2 x 4096->11008, 11008->4096)
           at M = 8, binary16 in and out, one decoder layer, stream launches
  prefill  one 2048 x 4096 x 14336 linear, binary16 in and out
  mid      one 128 x 11008 x 8192 linear, binary16 (64 tiles, long K: the streaming tcgen05 kernel)
  ffn      gate/up 4096 -> 2 x 14336, SwiGLU, down 14336 -> 4096 at M = 1024, fp32

Options: --repeat R (launch sets, default 4), --tokens M (override the batch), --stamps (after
the launches, enable the kernels' phase stamps, run one more set and print them: per linear of
the decode case the dependent phases of the fused kernel, for the prefill case the per-tile
timeline of the persistent GEMM's MMA issuer and epilogue).
"""
from __future__ import annotations

import argparse

import numpy as np


def _weights(rng, K, N):
    B = rng.integers(-7, 8, size=(K, N), dtype=np.int8)
    scale = rng.uniform(0.001, 0.01, size=N).astype(np.float32)
    return B, scale


def _activations(rng, M, K, dtype):
    x = rng.standard_normal((M, K)).astype(np.float32)
    x[:, rng.random(K) < 0.005] *= 20.0
    return x.astype(dtype)


def main() -> None:
    import torch

    import rknpu2_matmul_open_b200 as rk

    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["decode", "prefill", "mid", "ffn"])
    ap.add_argument("--repeat", type=int, default=4)
    ap.add_argument("--tokens", type=int, default=0)
    ap.add_argument("--stamps", action="store_true")
    args = ap.parse_args()
    rng = np.random.default_rng(0)
    ctx = rk.Context()
    dom = ctx.domain(0)
    dev = torch.device("cuda", ctx.device)
    stream = torch.cuda.Stream(device=dev)
    calls = []
    if args.case in ("decode", "prefill", "mid"):
        M = args.tokens or {"decode": 8, "prefill": 2048, "mid": 128}[args.case]
        shapes = {"decode": [(4096, 4096)] * 4 + [(4096, 11008)] * 2 + [(11008, 4096)], "prefill": [(4096, 14336)],
                  "mid": [(11008, 8192)]}[args.case]
        for K, N in shapes:
            B, sw = _weights(rng, K, N)
            w = rk.Weights(dom, B, sw)
            ws = rk.Workspace(dom, rk.default_config(M, N, K))
            dA = torch.from_numpy(_activations(rng, M, K, np.float16).view(np.int16)).to(dev)
            dC = torch.zeros((M, N), dtype=torch.int16, device=dev)
            calls.append((lambda ws=ws, w=w, dA=dA, dC=dC: ws.enqueue_f16(w, dA, dC, stream.cuda_stream), ws))
    else:
        M = args.tokens or 1024
        K, F, N = 4096, 14336, 4096
        Bg, sg = _weights(rng, K, 2 * F)
        Bd, sd = _weights(rng, F, N)
        wg, wd = rk.Weights(dom, Bg, sg), rk.Weights(dom, Bd, sd)
        g = rk.Workspace(dom, rk.default_config(M, 2 * F, K))
        d = rk.Workspace(dom, rk.default_config(M, N, F))
        dA = torch.from_numpy(_activations(rng, M, K, np.float32)).to(dev)
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
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            t0.record(stream)
            for _ in range(20):
                graph.replay()
            t1.record(stream)
        stream.synchronize()
        print(f"graph replay: {t0.elapsed_time(t1) * 1e3 / 20:.1f} us per set of {len(calls)} linears")
    if case == "decode":
        prev_end = None
        print("per linear, ns relative to the previous linear's last CTA end: first/last CTA start, first/last CTA end;"
              " then median cycles since CTA start at (decode kernel): before the dependency wait, dependency met, share"
              " quantised and sent, all codes landed, last contraction done, last output stored")
        for i, (_, ws) in enumerate(calls):
            buf = np.zeros((4112, 8), np.uint64)
            lib.rk_npu_b200_w4a8_trace_read(ws.handle, buf.ctypes.data, 4112)
            extra = buf[4096:4098].reshape(-1).astype(np.int64)
            fine = buf[4104].astype(np.int64)[:4]
            buf = buf[:4096]
            v = buf[buf[:, 0] > 0].astype(np.int64)
            if not len(v):
                continue
            s0, s1, e0, e1 = v[:, 0].min(), v[:, 0].max(), v[:, 7].min(), v[:, 7].max()
            ref = prev_end if prev_end is not None else s0
            cyc = np.median(v[:, 1:7], axis=0).astype(int)
            print(f"linear {i}: K={ws.cfg.K} N={ws.cfg.N} ctas={len(v)} start[{s0 - ref},{s1 - ref}] end[{e0 - ref},{e1 - ref}]"
                  f" cycles {list(cyc)}")
            prev_end = e1
            print(f"   CTA 0, first stages (cycles since its start: wait begins, wait ends): {[int(x) for x in extra]}")
            print(f"   CTA 0, scan (cycles since its start): loads issued, own maxima in, row maxima known, share quantised: {[int(x) for x in fine]}")
    elif case == "prefill":
        raw = np.zeros(256, np.uint64)
        lib.rk_npu_b200_w4a8_trace_read(calls[0][1].handle, raw.ctypes.data, 32)
        print(f"clusters in the grid: {int(raw[200])}; per tile of cluster 0 (cycles since kernel start): MMA issuer begins,"
              " first MMA issued, last commit, epilogue sees the accumulator, tensor memory handed back, tile stored,"
              " cycles the issuer waited for operands | unpack warp: waited for weights, for a free buffer, for activations")
        for j in range(7):
            print(f"tile {j}: {[int(x) for x in raw[j * 8:j * 8 + 7]]} | {int(raw[128 + 2 * j])} {int(raw[129 + 2 * j])} {int(raw[160 + j])}")


if __name__ == "__main__":
    main()
