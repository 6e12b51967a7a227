#!/usr/bin/env python
"""Benchmark of the GGUF quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl kq|reference]

Workload (N=1): decode GEMV at 27B-class shapes - a stack of LAYERS distinct MLP blocks, each with
gate and up projections in Q4_K (K=5120, N=17408) and a down projection in Q6_K (K=17408, N=5120),
seeded synthetic blocks, bf16 N(0,1) activations.  One STEP is one pass over the whole stack for every
M in {1, 2, 8, 16}; the stack (2.8 GB at 16 layers) is far larger than the 126 MB L2, so every weight byte
comes from HBM.  The op called per matrix follows the reference's own regime dispatch
(quantization/linear.py:40-63): ggml_mul_mat_vec_a8 for small M, ggml_mul_mat_a8 above.

value     whole-job algorithmic GB/s, activations and weights resident in HBM, calls made through the
          C ABI and replayed as one CUDA graph per step (the reference serves under CUDA graphs too)
e2e       same metric through the plugin-facing op API (kaillm_b200.linear.fused_mul_mat_gguf ->
          torch.ops._C_gguf.*) with HOST activations/outputs: pinned host -> device copy of every call's
          input and device -> host read of every call's output inside the timed region
roofline  the dominant kernel alone (the Q4_K GEMV over all Q4_K matrices and all M, activations already
          quantized), algorithmic bytes / CUDA-event time against the measured HBM copy bandwidth
With N > 1 the weights are row-sharded over the ranks and every call ends with an all-gather of the
output slices over NCCL (total work fixed: strong scaling).

--impl reference times the reference's CPU path (gguf-reader style dequantize + torch matmul) on the host
cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

Q4_K, Q6_K = 12, 14
K_HID, N_FF = 5120, 17408
MS = (1, 2, 8, 16)


# DRAM bytes per Q4_K 17408x5120 GEMV launch measured by ncu (dram__bytes_read.sum + dram__bytes_write.sum):
# 50.16 MB for the row-streaming kernel (1-2 tokens), 50.24 MB for the shared-stage kernel (8-16 tokens)
DRAM_TRAFFIC_Q4K = 50.2e6


def algorithmic_bytes(qt: int, n: int, k: int, m: int, esize: int = 2) -> int:
    blk, nb = {12: (256, 144), 14: (256, 210)}[qt]
    return n * (k // blk) * nb + m * k * esize + m * n * esize


def use_mmq(m: int, n: int) -> bool:
    """The reference's choice for K-quant types (quantization/linear.py:43-54)."""
    return m > (2 if n > 5120 else 6)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        self.t.join(timeout=2)
        sm, smax, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                smax.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower() == "active":
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------- reference arm
def reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import torch

    from kaillm_b200 import synth
    from oracle import gguf_oracle as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    m = 16
    rows_q4, rows_q6 = 17408 // 8, 5120 // 8          # a 1/8 row slice of each matrix keeps a step to seconds
    wq4 = synth.wire_numpy(Q4_K, rows_q4, K_HID, seed=1)
    wq6 = synth.wire_numpy(Q6_K, rows_q6, N_FF, seed=2)
    x1 = torch.from_numpy(synth.activations_numpy(m, K_HID, seed=3, dtype="bf16"))
    x2 = torch.from_numpy(synth.activations_numpy(m, N_FF, seed=4, dtype="bf16"))
    bytes_step = 2 * algorithmic_bytes(Q4_K, rows_q4, K_HID, m) + algorithmic_bytes(Q6_K, rows_q6, N_FF, m)

    def step():
        for w, qt, x in ((wq4, Q4_K, x1), (wq4, Q4_K, x1), (wq6, Q6_K, x2)):
            W = torch.from_numpy(O.dequantize_f32(w, qt, iq3s_top=60))
            torch.matmul(x, W.T)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = bytes_step / dt / 1e9
    sample = (f"1/8 row slice of one MLP block at M={m}: Q4_K gate+up {rows_q4}x{K_HID}, Q6_K down {rows_q6}x{N_FF}; "
              "numpy dequantize (gguf-reader arithmetic) + torch.matmul fp32")
    print(json.dumps({
        "impl": "reference", "metric": "quantized GEMV HBM GB/s", "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "27B-class decode GEMV, Q4_K gate/up + Q6_K down", "M": [m], "sample": "1/8 rows"},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------------------------- our arm
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="kq", choices=["kq", "reference"])
    ap.add_argument("--layers", type=int, default=16, help="distinct MLP blocks in the stack")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--small", action="store_true", help="2-layer stack, for profiler captures")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "kq" and not args.small:
        args.warmup = 3
    if args.impl == "reference":
        reference_arm(args)
        return
    if args.small:
        args.layers = 2

    import torch

    from kaillm_b200 import capi, linear, synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the GGUF kernels have no CPU fallback)")
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    # ---- the stack: per layer gate, up (Q4_K) and down (Q6_K); rows sharded over ranks
    def make(qt, n, k, seed):
        w = synth.wire_torch(qt, n, k, seed, dev)
        if world > 1:
            per = n // world
            w = w[rank * per:(rank + 1) * per].contiguous()
        return w

    mats = []  # (W, qt, n_full, k)
    for layer in range(args.layers):
        mats.append((make(Q4_K, N_FF, K_HID, 10 * layer + 1), Q4_K, N_FF, K_HID))
        mats.append((make(Q4_K, N_FF, K_HID, 10 * layer + 2), Q4_K, N_FF, K_HID))
        mats.append((make(Q6_K, K_HID, N_FF, 10 * layer + 3), Q6_K, K_HID, N_FF))
    g = torch.Generator(device=dev)
    g.manual_seed(1234)
    xs = {(m, k): torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16) for m in MS for k in (K_HID, N_FF)}
    ys = {(m, n): torch.empty((m, n // world), dtype=torch.bfloat16, device=dev) for m in MS for n in (K_HID, N_FF)}
    yg = {(m, n): torch.empty((world, m, n // world), dtype=torch.bfloat16, device=dev) for m in MS for n in (K_HID, N_FF)}
    ws = max(capi.workspace_bytes(qt, 16, n // world, k) for _, qt, n, k in mats)
    scratch = torch.empty(ws, dtype=torch.uint8, device=dev)
    bytes_step = sum(algorithmic_bytes(qt, n, k, m) for m in MS for _, qt, n, k in mats)
    calls_step = len(MS) * len(mats)

    # N > 1: every output slice is all-gathered.  The gather is the library's own peer-store kernel over NVLink
    # (kq_p2p_allgather on torch symmetric memory; NCCL all_gather_into_tensor if symmetric memory cannot be set up).
    # The three GEMVs of an MLP block write their [M, N/world] slices side by side into one buffer and ONE gather per
    # block carries all three to every rank.  The gathers run on a second stream and overlap the next block's GEMVs
    # (the blocks of this workload are independent); every block has its own slice and gather buffers, and a step
    # ends only when all gathers have completed (the side stream is joined into the main one).
    comm = torch.cuda.Stream(device=dev) if world > 1 else None
    p2p = None
    gather_how = None
    if world > 1:
        from kaillm_b200 import sharded
        blk_elems = {m: sum(m * (n // world) for _, _, n, _ in mats[:3]) for m in MS}
        nblocks = len(mats) // 3
        yblk = [torch.empty((1, blk_elems[m]), dtype=torch.bfloat16, device=dev) for m in MS for _ in range(nblocks)]
        ysl = []                                   # per call: a [M, N/world] view into its block's buffer
        for bi, m in enumerate(m for m in MS for _ in range(nblocks)):
            off = 0
            for _, _, n, _ in mats[:3]:
                ysl.append(yblk[bi][0, off:off + m * (n // world)].view(m, n // world))
                off += m * (n // world)
        try:
            p2p = sharded.P2PGather(max_bytes=blk_elems[max(MS)] * 2, nbuf=len(ysl), device=dev)
            gather_how = "kq_p2p_allgather (peer stores over NVLink)"
        except Exception as e:  # noqa: BLE001 - keep the NCCL path
            print(f"[bench] symmetric memory unavailable ({e!r}); using NCCL all_gather_into_tensor", file=sys.stderr)
            ygl = [torch.empty((world, 1, b.numel()), dtype=torch.bfloat16, device=dev) for b in yblk]
            gather_how = "NCCL all_gather_into_tensor"

    def step():
        cur = torch.cuda.current_stream()
        if world > 1:
            comm.wait_stream(cur)
        i = 0
        for m in MS:
            for W, qt, n, k in mats:
                out = ysl[i] if world > 1 else ys[(m, n)]
                capi.mul_mat(W, xs[(m, k)], qt, mmq=use_mmq(m, n), out=out, scratch=scratch, n=n // world)
                i += 1
                if world > 1 and i % 3 == 0:         # the block's three slices are written: one gather for all of them
                    bi = i // 3 - 1
                    ev = torch.cuda.Event()
                    ev.record(cur)
                    with torch.cuda.stream(comm):
                        comm.wait_event(ev)
                        if p2p is not None:
                            p2p.gather_raw(yblk[bi], bi)
                        else:
                            dist.all_gather_into_tensor(ygl[bi], yblk[bi])
        if world > 1:
            cur.wait_stream(comm)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.Stream(device=dev)
    graph = None
    with torch.cuda.stream(stream):
        l0 = capi.get_option("launch_count")
        step()
        launches_step = capi.get_option("launch_count") - l0
        torch.cuda.synchronize()
        if not args.no_graph:
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    step()
            except Exception as e:  # noqa: BLE001 - report and fall back to eager launches
                print(f"[bench] CUDA graph capture failed ({e!r}); running eagerly", file=sys.stderr)
                graph = None
        run = graph.replay if graph is not None else step
        for _ in range(args.warmup):
            run()
        barrier()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            run()
        e1.record(stream)
        barrier()
        ms_total = e0.elapsed_time(e1)
        clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms_total], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    value = bytes_step / (ms_step * 1e-3) / 1e9

    # ---- roofline of the dominant kernel: Q4_K GEMV alone, activations already quantized
    q4 = [(W, n, k) for W, qt, n, k in mats if qt == Q4_K]
    roof = None
    with torch.cuda.stream(stream):
        def q4_region():
            for m in MS:
                capi.prepare_q8(xs[(m, K_HID)], Q4_K, N_FF // world, scratch)
                for W, n, k in q4:
                    capi.mul_mat_prepared(W, Q4_K, m, k, ys[(m, n)], scratch, mmq=use_mmq(m, n))
        q4_region()
        torch.cuda.synchronize()
        g4 = None
        if not args.no_graph:
            try:
                g4 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g4, stream=stream):
                    q4_region()
            except Exception:  # noqa: BLE001
                g4 = None
        run4 = g4.replay if g4 is not None else q4_region
        for _ in range(3):
            run4()
        torch.cuda.synchronize()
        reps = 10
        e0.record(stream)
        for _ in range(reps):
            run4()
        e1.record(stream)
        torch.cuda.synchronize()
        n_launch = len(MS) * len(q4)
        us = e0.elapsed_time(e1) * 1e3 / (reps * n_launch)
        alg = sum(algorithmic_bytes(Q4_K, N_FF // world, K_HID, m) for m in MS) / len(MS)
        peak, how = measured_peaks()
        ach = alg / (us * 1e-6) / 1e9
        roof = {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": DRAM_TRAFFIC_Q4K / world,
                "kernel": "Q4_K decode GEMV (gate/up 17408x5120), mean over M=1,2,8,16", "us_per_launch": us,
                "algorithmic_bytes_per_launch": alg, "peak_source": f"of {how} (MEASURED_PEAKS.json hbm_gbs)",
                "note": "region = 4 q8_1 quantize launches + %d GEMV launches, divided by the GEMV launches; traffic = "
                        "dram__bytes_read+write per launch from the ncu captures summarised under profiles/ "
                        "(50.16 MB row-streaming kernel, 50.24 MB shared-stage kernel; full matrix, scaled by 1/ranks)" % n_launch}

    # ---- prefill GEMM (tcgen05): Q4_K N=17408 K=5120 at M=2048, TFLOP/s against the measured bf16 tensor peak
    prefill = None
    if world == 1:
        with torch.cuda.stream(stream):
            mp = 2048
            Wp = mats[0][0]
            xp = torch.randn((mp, K_HID), device=dev, generator=g).to(torch.bfloat16)
            yp = torch.empty((mp, N_FF), dtype=torch.bfloat16, device=dev)
            sp = torch.empty(capi.workspace_bytes(Q4_K, mp, N_FF, K_HID), dtype=torch.uint8, device=dev)
            l0 = capi.get_option("launch_count")
            capi.mul_mat(Wp, xp, Q4_K, mmq=True, out=yp, scratch=sp)
            gl = capi.get_option("launch_count") - l0
            for _ in range(3):
                capi.mul_mat(Wp, xp, Q4_K, mmq=True, out=yp, scratch=sp)
            torch.cuda.synchronize()
            reps = 10
            e0.record(stream)
            for _ in range(reps):
                capi.mul_mat(Wp, xp, Q4_K, mmq=True, out=yp, scratch=sp)
            e1.record(stream)
            torch.cuda.synchronize()
            msg = e0.elapsed_time(e1) / reps
            tf = 2.0 * mp * N_FF * K_HID / (msg * 1e-3) / 1e12
            pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
            peak_tf = float(pk.get("bf16_tflops", 1590.0))
            prefill = {"workload": "Q4_K N=17408 K=5120, bf16 activations M=2048 (quantize + tcgen05 GEMM)", "ms": msg,
                       "tflops": tf, "peak_tflops": peak_tf, "frac": tf / peak_tf,
                       "peak_source": "of measured (bf16_tflops burst)" if pk else "of fallback", "launches_per_call": gl}
            del yp, sp
            # LM head of the same configuration: Q6_K N=248320 K=5120 (1.04 GB of wire bytes)
            n_lm = 248320
            Wl = synth.wire_torch(Q6_K, n_lm, K_HID, 777, dev)
            yl = torch.empty((mp, n_lm), dtype=torch.bfloat16, device=dev)
            sl = torch.empty(capi.workspace_bytes(Q6_K, mp, n_lm, K_HID), dtype=torch.uint8, device=dev)
            for _ in range(2):
                capi.mul_mat(Wl, xp, Q6_K, mmq=True, out=yl, scratch=sl)
            torch.cuda.synchronize()
            e0.record(stream)
            for _ in range(3):
                capi.mul_mat(Wl, xp, Q6_K, mmq=True, out=yl, scratch=sl)
            e1.record(stream)
            torch.cuda.synchronize()
            msl = e0.elapsed_time(e1) / 3
            tfl = 2.0 * mp * n_lm * K_HID / (msl * 1e-3) / 1e12
            prefill["lm_head_q6k"] = {"workload": "Q6_K N=248320 K=5120, M=2048", "ms": msl, "tflops": tfl, "frac": tfl / peak_tf}
            del xp, Wl, yl, sl

    # ---- end to end through the op API with host buffers
    e2e = None
    with torch.cuda.stream(stream):
        hx = {key: v.cpu().pin_memory() for key, v in xs.items()}
        h2d = sum(hx[(m, k)].numel() * 2 for m in MS for _, _, _, k in mats)
        d2h = sum(m * (n // world) * 2 for m in MS for _, _, n, _ in mats)
        # one device input buffer and one pinned host result buffer per call: no reuse hazards inside a step
        calls = [(m, W, qt, n, k) for m in MS for W, qt, n, k in mats]
        dxs = [torch.empty_like(xs[(m, k)]) for m, _, _, _, k in calls]
        hys = [torch.empty((m, n // world), dtype=torch.bfloat16).pin_memory() for m, _, _, n, _ in calls]
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

        GROUP = 12   # calls per synchronisation point between the streams (4 MLP blocks)

        def e2e_enqueue(keep):
            """H2D copies on one side stream, the op on the main stream, D2H reads on another side stream.  The streams
            meet once per GROUP calls, not per call, so that consecutive kernels of the main stream stay adjacent
            (programmatic dependent launch needs a kernel as the direct predecessor)."""
            s_in.wait_stream(stream)
            s_out.wait_stream(stream)
            evs = []
            with torch.cuda.stream(s_in):            # every input copy of the step, an event after each group
                for i, (m, W, qt, n, k) in enumerate(calls):
                    dxs[i].copy_(hx[(m, k)], non_blocking=True)
                    if (i + 1) % GROUP == 0 or i + 1 == len(calls):
                        ev = torch.cuda.Event()
                        ev.record(s_in)
                        evs.append(ev)
            for g0 in range(0, len(calls), GROUP):
                stream.wait_event(evs[g0 // GROUP])
                ys_g = []
                for i in range(g0, min(g0 + GROUP, len(calls))):
                    m, W, qt, n, k = calls[i]
                    y = linear.fused_mul_mat_gguf(dxs[i], W, qt)
                    if world > 1:
                        if p2p is not None:
                            p2p.gather_raw(y, i)
                        else:
                            dist.all_gather_into_tensor(yg[(m, n)], y)
                    ys_g.append((i, y))
                    keep.append(y)   # outputs stay alive until the copies that read them are done
                ev2 = torch.cuda.Event()
                ev2.record(stream)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev2)
                    for i, y in ys_g:
                        hys[i].copy_(y, non_blocking=True)
            stream.wait_stream(s_in)
            stream.wait_stream(s_out)

        keep: list = []
        e2e_enqueue(keep)
        torch.cuda.synchronize()
        eg = None
        if not args.no_graph:
            try:
                keep_g: list = []
                eg = torch.cuda.CUDAGraph()
                with torch.cuda.graph(eg, stream=stream):
                    e2e_enqueue(keep_g)
            except Exception as e:  # noqa: BLE001
                print(f"[bench] e2e graph capture failed ({e!r}); running eagerly", file=sys.stderr)
                eg = None

        def e2e_step():
            if eg is not None:
                eg.replay()
            else:
                keep.clear()
                e2e_enqueue(keep)
            torch.cuda.current_stream().synchronize()   # the step's results are in host memory here

        for _ in range(3):
            e2e_step()
        barrier()
        esteps = max(2, min(args.steps, 10))
        e0.record(stream)
        for _ in range(esteps):
            e2e_step()
        e1.record(stream)
        barrier()
        # every host result of the last step against a separate eager call of the same op on the device-resident input
        bad = 0
        for i, (m, W, qt, n, k) in enumerate(calls):
            ref = linear.fused_mul_mat_gguf(xs[(m, k)], W, qt)
            bad += int(not torch.equal(ref.cpu(), hys[i]))
        if bad:
            raise SystemExit(f"[bench] e2e results differ from the eager op on {bad} of {len(calls)} calls")
        t2 = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        ms_e2e = float(t2.item()) / esteps
        e2e = {"value": bytes_step / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e, "results_checked": len(calls),
               "api": "kaillm_b200.linear.fused_mul_mat_gguf -> torch.ops._C_gguf.ggml_mul_mat_{vec_,}a8; per call: "
                      "H2D of x from pinned memory, the op, D2H of y into pinned memory (copies on side streams that meet the "
                      "compute stream every 12 calls); "
                      + ("whole step replayed as one CUDA graph" if eg is not None else "eager")}

    # ---- CPU baseline (oracle port of the reference's CPU path) on rank 0, bounded sample
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import numpy as np

        from oracle import gguf_oracle as O
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        m = 16
        r4, r6 = N_FF, K_HID
        w4 = synth.wire_numpy(Q4_K, r4, K_HID, seed=1)
        w6 = synth.wire_numpy(Q6_K, r6, N_FF, seed=2)
        x1 = torch.from_numpy(synth.activations_numpy(m, K_HID, seed=3, dtype="bf16"))
        x2 = torch.from_numpy(synth.activations_numpy(m, N_FF, seed=4, dtype="bf16"))
        t0 = time.perf_counter()
        for w, qt, x in ((w4, Q4_K, x1), (w4, Q4_K, x1), (w6, Q6_K, x2)):
            Wd = torch.from_numpy(O.dequantize_f32(w, qt, iq3s_top=60))
            torch.matmul(x, Wd.T)
        dt = time.perf_counter() - t0
        b = 2 * algorithmic_bytes(Q4_K, r4, K_HID, m) + algorithmic_bytes(Q6_K, r6, N_FF, m)
        cpu = {"value": b / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port", "seconds": dt,
               "sample": f"one whole MLP block at M={m} (Q4_K gate+up {r4}x{K_HID}, Q6_K down {r6}x{N_FF}): "
                         "numpy dequantize with gguf-reader arithmetic + torch.matmul fp32"}

    if p2p is not None:
        p2p.check()
    if rank == 0:
        out = {
            "metric": "quantized GEMV HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": "27B-class decode GEMV: Q4_K gate/up (K=5120,N=17408) + Q6_K down (K=17408,N=5120)",
                       "layers": args.layers, "M": list(MS), "activations": "bf16 N(0,1)",
                       "calls_per_step": calls_step, "bytes_per_step": bytes_step,
                       "l2": "stack of %.2f GB per rank >> 126 MB L2, no flush needed" % (sum(w.numel() for w, *_ in mats) / 1e9),
                       "launch": "cuda graph replay" if graph is not None else "eager",
                       "parallelism": (f"row-sharded x{world} + all-gather of every output by {gather_how} (one gather per MLP block carries "
                                       "its three output slices; the gathers run on a second stream and overlap the next block; joined "
                                       "at the end of each step)")
                       if world > 1 else "single GPU"},
            "frac_of_measured_hbm": value / measured_peaks()[0], "frac_of_nominal_8tbs": value / 8000.0,
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches_step * args.steps,
            "roofline": roof, "cpu_baseline": cpu, "prefill_gemm": prefill,
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        # leave without tearing the communicator down: destroy_process_group() after graph-captured collectives
        # hung at exit on this stack; every rank is past its last collective here
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
