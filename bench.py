#!/usr/bin/env python
"""Benchmark of the GGUF quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl kq|reference]

N = 1   decode GEMV at 27B-class shapes: a stack of 16 distinct MLP blocks, each with gate and up projections in Q4_K
        (K=5120, N=17408) and a down projection in Q6_K (K=17408, N=5120), seeded synthetic blocks, bf16 N(0,1)
        activations.  One STEP is one pass over the whole stack for every M in {1, 2, 8, 16} (192 calls); the stack
        (2.8 GB) is far larger than the 126 MB L2, so every weight byte comes from HBM.  The op per call follows the
        reference's regime dispatch (quantization/linear.py:40-63).
          value     algorithmic GB/s, everything resident in HBM, calls through the C ABI, one CUDA graph per step
          e2e       the same through the plugin-facing op API with HOST activations and outputs (pinned memory; the
                    copies of every call are inside the timed region)
          roofline  the dominant kernel alone (Q4_K GEMV, activations already quantized) against the measured HBM
                    copy bandwidth
        Further blocks of the same JSON line: `decode_table` (per shape and M), `config3` (the decoder-stack workload
        of the multi-GPU runs on one GPU), `lowbit` (IQ3_S / Q2_K at M in {1, 16, 80} through the op API), `dequantize`
        (LM head), `prefill_gemm` (M in {256, 1024, 2048} and the LM head), `reference_cuda` (the reference's own CUDA
        kernels, built unmodified into oracle/_ref, on the same inputs in the same run), `moe` (the mixture-of-experts
        ops, with the reference's beside them) and `cpu_baseline`.
N > 1   the mixed-quant decoder stack: 64 layers, per layer merged q/k/v (Q8_0, N=8192), o (Q8_0, N=5120), merged
        gate/up (Q4_K, N=34816) and down (Q6_K, K=17408), batch 16, every projection sharded on its output rows over the
        ranks and all-gathered; each projection consumes the gathered output of the one before it (RMSNorm / SwiGLU /
        plain q8_1 producers), so nothing overlaps artificially.  Total work is fixed (strong scaling).  Before the line
        is printed every rank's gathered outputs are compared with single-GPU results on the full matrices, and the
        ranks' final outputs with each other.  `same_workload_one_gpu`: the same stack, unsharded, timed on rank 0 in
        the same run - the N = 1 line above measures another configuration, so this is what the N-GPU value compares with.

--impl reference times the reference's CPU path (gguf-reader dequantize + torch matmul) on the host cores, on a
bounded sample of the same configuration.
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

Q8_0, Q2_K, Q4_K, Q6_K, IQ3_S = 8, 10, 12, 14, 21
K_HID, N_FF = 5120, 17408
MS = (1, 2, 8, 16)
BLOCKS = {Q8_0: (32, 34), Q2_K: (256, 84), Q4_K: (256, 144), Q6_K: (256, 210), IQ3_S: (256, 110)}
NAMES = {Q8_0: "Q8_0", Q2_K: "Q2_K", Q4_K: "Q4_K", Q6_K: "Q6_K", IQ3_S: "IQ3_S"}
# config 3: (name, type, N, K) per layer; merged projections are one tensor
C3_LAYERS, C3_M = 64, 16
C3_GROUPS = (("qkv", Q8_0, 6144 + 1024 + 1024, K_HID), ("o", Q8_0, K_HID, K_HID), ("gate_up", Q4_K, 2 * N_FF, K_HID),
             ("down", Q6_K, K_HID, N_FF))

# DRAM bytes per Q4_K 17408x5120 GEMV launch measured by ncu (dram__bytes_read.sum + dram__bytes_write.sum):
# 50.16 MB for the row-streaming kernel (1-2 tokens), 50.24 MB for the shared-stage kernel (8-16 tokens)
DRAM_TRAFFIC_Q4K = 50.2e6


def algorithmic_bytes(qt: int, n: int, k: int, m: int, esize: int = 2) -> int:
    blk, nb = BLOCKS[qt]
    return n * (k // blk) * nb + m * k * esize + m * n * esize


def use_mmq(m: int, n: int) -> bool:
    """The reference's choice for K-quant and legacy types (quantization/linear.py:43-54)."""
    return m > (2 if n > 5120 else 6)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm": float(d["hbm_gbs"]), "tf": float(d["bf16_tflops"]), "how": "of measured (MEASURED_PEAKS.json)"}
    return {"hbm": 6650.0, "tf": 1590.0, "how": "of fallback"}


def workload_config(world: int) -> dict:
    """What is measured, as a function of the rank count only (the reference arm prints the same dict)."""
    if world == 1:
        return {"workload": "27B-class decode GEMV: 16 MLP blocks of Q4_K gate/up (K=5120,N=17408) + Q6_K down (K=17408,N=5120)",
                "layers": 16, "M": list(MS), "activations": "bf16 N(0,1)", "calls_per_step": 16 * 3 * len(MS),
                "l2": "2.8 GB of weights >> 126 MB L2, no flush needed"}
    return {"workload": "mixed-quant decoder stack: 64 layers of merged q/k/v Q8_0 (N=8192) + o Q8_0 (N=5120) + merged gate/up "
                        "Q4_K (N=34816) + down Q6_K (K=17408,N=5120), hidden 5120",
            "layers": C3_LAYERS, "M": [C3_M], "activations": "bf16 N(0,1)", "calls_per_step": 4 * C3_LAYERS,
            "parallelism": "weights row-sharded over the ranks, all-gather of every output",
            "l2": "15.7 GB of weights >> 126 MB L2, no flush needed"}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 100 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.rows, self.proc = gpu_index, [], None

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
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower() == "active":
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------- the reference's CPU path
def _reference_reader():
    """The reference's own gguf-reader (staged by oracle/stage_ref.py under baseline/_ref), or None."""
    stage = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.exists(os.path.join(stage, "gguf", "quants.py")):
        return None
    if stage not in sys.path:
        sys.path.insert(0, stage)
    try:
        import gguf
        from gguf import quants
        from gguf.constants import GGMLQuantizationType
        if not os.path.realpath(gguf.__file__).startswith(os.path.realpath(stage)):
            return None
        return lambda w, qt: quants.dequantize(w, GGMLQuantizationType(qt))
    except Exception:  # noqa: BLE001 - fall back to the port
        return None


def cpu_path_sample(world: int, frac: int):
    """A bounded sample of the configuration: the first 1/frac of the rows of each distinct matrix, every M of the
    configuration.  Returns (step function, algorithmic bytes per step, kind, description)."""
    import torch

    from kaillm_b200 import synth

    deq = _reference_reader()
    kind = "reference" if deq is not None else "port"
    if deq is None:
        from oracle import gguf_oracle as O
        deq = lambda w, qt: O.dequantize_f32(w, qt, iq3s_top=60)   # noqa: E731
    if world == 1:
        mats = [(Q4_K, N_FF, K_HID), (Q4_K, N_FF, K_HID), (Q6_K, K_HID, N_FF)]
        ms = MS
    else:
        mats = [(qt, n, k) for _, qt, n, k in C3_GROUPS]
        ms = (C3_M,)
    wires = [(qt, max(8, n // frac), k, synth.wire_numpy(qt, max(8, n // frac), k, seed=i + 1)) for i, (qt, n, k) in enumerate(mats)]
    xs = {(m, k): torch.from_numpy(synth.activations_numpy(m, k, seed=3, dtype="bf16")) for m in ms for k in (K_HID, N_FF)}
    nbytes = sum(algorithmic_bytes(qt, n, k, m) for m in ms for qt, n, k, _ in wires)

    def step():
        for m in ms:
            for qt, n, k, w in wires:
                W = torch.from_numpy(deq(w, qt).astype("float32", copy=False))   # the reference dequantizes on every call
                torch.matmul(xs[(m, k)], W.T)

    desc = (f"first 1/{frac} of the rows of each matrix of one block/layer ({', '.join(f'{NAMES[qt]} {n}x{k}' for qt, n, k, _ in wires)}), "
            f"M in {list(ms)}: " + ("the reference's gguf.quants.dequantize (gguf-reader/gguf/quants.py:68)" if kind == "reference"
                                   else "numpy port of the gguf-reader arithmetic") + " + torch.matmul fp32, per call")
    return step, nbytes, kind, desc


def reference_arm(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch

    world = args.gpus
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    step, nbytes, kind, desc = cpu_path_sample(world, frac=32)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = nbytes / dt / 1e9
    print(json.dumps({
        "impl": "reference", "metric": "quantized GEMV HBM GB/s", "value": val, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(world),
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": kind, "sample": desc},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


# ---------------------------------------------------------------------------------------------- timing helpers
class Timer:
    def __init__(self, torch, stream, no_graph):
        self.torch, self.stream, self.no_graph = torch, stream, no_graph

    def graph(self, fn):
        """fn captured as a CUDA graph on self.stream (eager fallback); returns (callable, captured?)."""
        torch = self.torch
        fn()
        torch.cuda.synchronize()
        if self.no_graph:
            return fn, False
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=self.stream):
                fn()
            return g.replay, True
        except Exception as e:  # noqa: BLE001
            print(f"[bench] CUDA graph capture failed ({e!r}); running eagerly", file=sys.stderr)
            return fn, False

    def time(self, run, reps, warm=3):
        """milliseconds per call of run(), CUDA events on self.stream."""
        torch = self.torch
        for _ in range(warm):
            run()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(self.stream)
        for _ in range(reps):
            run()
        e1.record(self.stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps


def make_stack(torch, synth, dev, rank, world, layers):
    """Config-3 weights: every tensor generated whole from its seed, this rank's rows kept."""
    out = []
    for li in range(layers):
        d = {}
        for gi, (name, qt, n, k) in enumerate(C3_GROUPS):
            w = synth.wire_torch(qt, n, k, 1000 + 10 * li + gi, dev)
            per = n // world
            d[name] = (w[rank * per:(rank + 1) * per].contiguous() if world > 1 else w, qt, n, k)
            del w
        out.append(d)
    return out


def c3_bytes(layers):
    return layers * sum(algorithmic_bytes(qt, n, k, C3_M) for _, qt, n, k in C3_GROUPS)


# ---------------------------------------------------------------------------------------------- N > 1: config 3
def run_multi(args, torch, dist, dev, rank, world, local):
    from kaillm_b200 import capi, sharded, synth

    pk = peaks()
    layers = args.layers if args.layers else C3_LAYERS
    weights = make_stack(torch, synth, dev, rank, world, layers)
    p2p, gather_how = None, "NCCL all_gather_into_tensor + transposing copy"
    if not args.nccl:
        try:
            maxb = C3_M * max(n for _, _, n, _ in C3_GROUPS) // world * 2
            p2p = sharded.P2PGather(max_bytes=maxb, nbuf=4, device=dev)
            gather_how = "kq_mul_mat_prepared_gather: 16-byte peer stores over NVLink from the GEMV's own epilogue into every rank's row-major buffer"
            if args.no_fused_gather:
                capi.set_option("no_fused_gather", 1)
                gather_how = "kq_mul_mat_prepared_gather, two kernels (GEMV, then peer-store gather kernel)"
        except Exception as e:  # noqa: BLE001 - keep the NCCL path
            print(f"[bench] symmetric memory unavailable ({e!r}); using NCCL", file=sys.stderr)
    stack = sharded.DecoderStack(weights, C3_M, K_HID, dev, p2p=p2p, wait_in_consumer=not args.flag_gather)
    if stack.wait_in_consumer:
        gather_how = ("kq_mul_mat_prepared_gather, wait_in_consumer: the GEMV's epilogue stores its slice into every rank's row-major "
                      "buffer over NVLink; no hand-shake - the next producer polls the values against the arrival sentinel")
    g = torch.Generator(device=dev)
    g.manual_seed(1234)
    x0 = torch.randn((C3_M, K_HID), device=dev, generator=g).to(torch.bfloat16)
    hx0 = x0.cpu().pin_memory()
    hout = torch.empty((C3_M, K_HID), dtype=torch.bfloat16).pin_memory()
    xin = torch.empty_like(x0)
    stream = torch.cuda.Stream(device=dev)
    tm = Timer(torch, stream, args.no_graph)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    # ---- verification: every rank's gathered outputs against single-GPU results on the full matrices, which are
    # regenerated from their seeds for a subset of the layers (the chain itself runs through all of them)
    check_layers = sorted({0, 1, layers // 2, layers - 2, layers - 1} & set(range(layers)))
    big = torch.empty(max(capi.workspace_bytes(qt, C3_M, n, k) for _, qt, n, k in C3_GROUPS), dtype=torch.uint8, device=dev)
    checked = {"calls": 0, "bad": 0}

    def on_output(li, name, full, prep):
        if li not in check_layers:
            return
        gi = [nm for nm, *_ in C3_GROUPS].index(name)
        _, qt, n, k = C3_GROUPS[gi]
        wfull = synth.wire_torch(qt, n, k, 1000 + 10 * li + gi, dev)
        prep(big)
        ref = torch.empty((C3_M, n), dtype=torch.bfloat16, device=dev)
        capi.mul_mat_prepared(wfull, qt, C3_M, k, ref, big)
        checked["calls"] += 1
        # The same rows on a differently sized shard meet the CTA's warps in another order, so a sum may differ in
        # its last fp32 bit and a bf16 output may round the other way: equal up to such flips, never more.
        rel = float((ref.float() - full.float()).norm() / ref.float().norm().clamp_min(1e-30))
        same = float((ref == full).float().mean())
        checked["worst_rel"] = max(checked.get("worst_rel", 0.0), rel)
        checked["least_equal"] = min(checked.get("least_equal", 1.0), same)
        if rel > 1e-4 or same < 0.99:
            checked["bad"] += 1
            checked.setdefault("detail", []).append(f"layer {li} {name}: rel-L2 {rel:.3e}, equal {same:.4f}")

    with torch.cuda.stream(stream):
        barrier()                                   # every rank has set up its buffers before the first peer store
        h_ref = stack.forward(x0, on_output=on_output).clone()
        torch.cuda.synchronize()
        stack.check()
        # every rank must hold the same gathered bits: compare a checksum of the final hidden state across ranks
        cs = h_ref.view(torch.int16).to(torch.int64).sum().reshape(1)
        lo, hi = cs.clone(), cs.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        if int(lo.item()) != int(hi.item()):
            raise SystemExit(f"[bench] rank {rank}: the ranks hold different gathered outputs")
        if checked["bad"]:
            raise SystemExit(f"[bench] rank {rank}: gathered outputs differ from single-GPU results on {checked['bad']} of "
                             f"{checked['calls']} calls: {'; '.join(checked.get('detail', [])[:8])}")

        # ---- value: activations resident
        l0 = capi.get_option("launch_count")
        run, captured = tm.graph(lambda: stack.forward(x0))
        launches_step = (capi.get_option("launch_count") - l0) // (2 if captured else 1)
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
        clocks = sampler.stop() if rank == 0 else None
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step = float(t.item()) / args.steps
        h_last = stack.forward(x0)
        if not torch.equal(h_last, h_ref):
            raise SystemExit(f"[bench] rank {rank}: the stack's output after the timed steps differs from the verified pass")

        # ---- e2e: the step's input comes from pinned host memory, its output goes back to pinned host memory
        def e2e_body():
            xin.copy_(hx0, non_blocking=True)
            h = stack.forward(xin)
            hout.copy_(h, non_blocking=True)
        erun, _ = tm.graph(e2e_body)

        def e2e_step():
            erun()
            torch.cuda.current_stream().synchronize()
        for _ in range(3):
            e2e_step()
        barrier()
        esteps = max(2, min(args.steps, 20))
        e0.record(stream)
        for _ in range(esteps):
            e2e_step()
        e1.record(stream)
        barrier()
        if not torch.equal(hout, h_ref.cpu()):
            raise SystemExit(f"[bench] rank {rank}: the end-to-end result differs from the verified pass")
        t2 = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        ms_e2e = float(t2.item()) / esteps
    stack.check()
    nbytes = c3_bytes(layers)
    value = nbytes / (ms_step * 1e-3) / 1e9
    # ---- the same workload on ONE GPU, measured in this run (rank 0, whole tensors, the other ranks wait): the N = 1
    # line of this program measures another configuration, so this is the figure the N-GPU value divides by
    one = None
    if rank == 0 and not args.no_one_gpu:
        try:
            solo = sharded.DecoderStack(make_stack(torch, synth, dev, 0, 1, layers), C3_M, K_HID, dev, unsharded=True)
            with torch.cuda.stream(stream):
                solo.forward(x0)
                r1, cap1 = tm.graph(lambda: solo.forward(x0))
                ms1 = tm.time(r1, max(3, min(args.steps, 10)))
            one = {"ms_per_step": ms1, "value": nbytes / (ms1 * 1e-3) / 1e9, "unit": "GB/s", "speedup_of_this_run": ms1 / ms_step,
                   "launch": "cuda graph replay" if cap1 else "eager",
                   "how": "rank 0 alone, unsharded weights from the same seeds, after the timed region of the sharded run"}
            del solo, r1
        except Exception as e:  # noqa: BLE001 - the comparison figure is optional
            one = {"unavailable": repr(e)[:200]}
    barrier()
    if rank == 0:
        cfg = workload_config(world)
        cfg.update({"layers": layers, "bytes_per_step": nbytes, "gather": gather_how,
                    "launch": "cuda graph replay" if captured else "eager", "launches_per_step": launches_step,
                    "gemv_and_gather_in_one_kernel": dict(stack.fused),
                    "per_layer": "4 x (activation producer + GEMV with gather): RMSNorm->q8_1, q8_1, RMSNorm->q8_1, SwiGLU->q8_1"})
        print(json.dumps({
            "metric": "quantized GEMV HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8", "data": "synthetic", "config": cfg,
            "frac_of_measured_hbm": value / (world * pk["hbm"]), "frac_of_nominal_8tbs": value / (world * 8000.0),
            "per_gpu_gbs": value / world, "us_per_projection": ms_step * 1e3 / (4 * layers),
            "same_workload_one_gpu": one,
            "clocks": clocks, "gpu_launches": launches_step * args.steps,
            "verified": {"gathered_outputs_vs_single_gpu_full_matrices": "equal up to last-bit rounding flips",
                         "worst_rel_l2": checked.get("worst_rel"), "least_fraction_bit_equal": checked.get("least_equal"),
                         "calls_checked_per_rank": checked["calls"], "layers_checked": check_layers,
                         "all_ranks_hold_identical_bits": True, "final_output_checked_after_timed_steps": True},
            "e2e": {"value": nbytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": x0.numel() * 2,
                    "d2h_bytes_per_step": x0.numel() * 2, "ms_per_step": ms_e2e,
                    "api": "kaillm_b200.sharded.DecoderStack.forward over the C ABI: H2D of the step's [16, 5120] input from pinned "
                           "memory, 64 layers, D2H of the final hidden state into pinned memory; result compared with the verified pass"},
            "roofline": {"bound": "hbm", "achieved": value / world, "peak": pk["hbm"], "unit": "GB/s", "frac": value / world / pk["hbm"],
                         "traffic": None, "kernel": "whole decoder-stack step per GPU (producers + GEMVs + gathers)",
                         "peak_source": pk["how"]},
            "cpu_baseline": None,
        }), flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)   # leave without tearing the communicator down (destroy_process_group after captured collectives hung at exit)


# ---------------------------------------------------------------------------------------------- N = 1
def run_single(args, torch, dev, local):
    from kaillm_b200 import capi, linear, sharded, synth

    pk = peaks()
    layers = args.layers if args.layers else 16
    stream = torch.cuda.Stream(device=dev)
    tm = Timer(torch, stream, args.no_graph)
    mats = []
    for layer in range(layers):
        mats.append((synth.wire_torch(Q4_K, N_FF, K_HID, 10 * layer + 1, dev), Q4_K, N_FF, K_HID))
        mats.append((synth.wire_torch(Q4_K, N_FF, K_HID, 10 * layer + 2, dev), Q4_K, N_FF, K_HID))
        mats.append((synth.wire_torch(Q6_K, K_HID, N_FF, 10 * layer + 3, dev), Q6_K, K_HID, N_FF))
    g = torch.Generator(device=dev)
    g.manual_seed(1234)
    xs = {(m, k): torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16) for m in MS for k in (K_HID, N_FF)}
    ys = {(m, n): torch.empty((m, n), dtype=torch.bfloat16, device=dev) for m in MS for n in (K_HID, N_FF)}
    scratch = torch.empty(max(capi.workspace_bytes(qt, 16, n, k) for _, qt, n, k in mats), dtype=torch.uint8, device=dev)
    bytes_step = sum(algorithmic_bytes(qt, n, k, m) for m in MS for _, qt, n, k in mats)

    def step():
        for m in MS:
            for W, qt, n, k in mats:
                capi.mul_mat(W, xs[(m, k)], qt, mmq=use_mmq(m, n), out=ys[(m, n)], scratch=scratch)

    with torch.cuda.stream(stream):
        l0 = capi.get_option("launch_count")
        run, captured = tm.graph(step)
        launches_step = (capi.get_option("launch_count") - l0) // (2 if captured else 1)
        for _ in range(args.warmup):
            run()
        torch.cuda.synchronize()
        sampler = ClockSampler(local)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            run()
        e1.record(stream)
        torch.cuda.synchronize()
        ms_step = e0.elapsed_time(e1) / args.steps
        clocks = sampler.stop()
    value = bytes_step / (ms_step * 1e-3) / 1e9
    extra = {}

    with torch.cuda.stream(stream):
        # ---- per shape and M: the whole call (quantizer included), graph replay over all matrices of the shape
        table = []
        for qt, n, k in ((Q4_K, N_FF, K_HID), (Q6_K, K_HID, N_FF)):
            ws_ = [W for W, t, *_ in mats if t == qt]
            for m in MS:
                def region(m=m, ws_=ws_, qt=qt, n=n, k=k):
                    for W in ws_:
                        capi.mul_mat(W, xs[(m, k)], qt, mmq=use_mmq(m, n), out=ys[(m, n)], scratch=scratch)
                l0 = capi.get_option("launch_count")
                region()
                lpc = (capi.get_option("launch_count") - l0) / len(ws_)
                r, _ = tm.graph(region)
                us = tm.time(r, 10) * 1e3 / len(ws_)
                gbs = algorithmic_bytes(qt, n, k, m) / us / 1e3
                table.append({"type": NAMES[qt], "n": n, "k": k, "m": m, "us_per_call": round(us, 2), "gbs": round(gbs, 1),
                              "frac_of_measured_hbm": round(gbs / pk["hbm"], 3), "launches_per_call": lpc})
        extra["decode_table"] = table

        # ---- roofline of the dominant kernel: Q4_K GEMV alone, activations already quantized
        q4 = [W for W, qt, *_ in mats if qt == Q4_K]

        def q4_region():
            for m in MS:
                capi.prepare_q8(xs[(m, K_HID)], Q4_K, N_FF, scratch)
                for W in q4:
                    capi.mul_mat_prepared(W, Q4_K, m, K_HID, ys[(m, N_FF)], scratch, mmq=use_mmq(m, N_FF))
        r4, _ = tm.graph(q4_region)
        n_launch = len(MS) * len(q4)
        us = tm.time(r4, 10) * 1e3 / n_launch
        alg = sum(algorithmic_bytes(Q4_K, N_FF, K_HID, m) for m in MS) / len(MS)
        ach = alg / us / 1e3
        roof = {"bound": "hbm", "achieved": ach, "peak": pk["hbm"], "unit": "GB/s", "frac": ach / pk["hbm"], "traffic": DRAM_TRAFFIC_Q4K,
                "kernel": "Q4_K decode GEMV (gate/up 17408x5120), mean over M=1,2,8,16", "us_per_launch": us,
                "algorithmic_bytes_per_launch": alg, "peak_source": pk["how"],
                "note": "region = 4 q8_1 quantize launches + %d GEMV launches, divided by the GEMV launches; traffic = "
                        "dram__bytes_read+write per launch from the ncu captures summarised under profiles/" % n_launch}

        # ---- end to end through the op API with host buffers
        hx = {key: v.cpu().pin_memory() for key, v in xs.items()}
        calls = [(m, W, qt, n, k) for m in MS for W, qt, n, k in mats]
        h2d = sum(hx[(m, k)].numel() * 2 for m, _, _, _, k in calls)
        d2h = sum(m * n * 2 for m, _, _, n, _ in calls)
        dxs = [torch.empty_like(xs[(m, k)]) for m, _, _, _, k in calls]
        hys = [torch.empty((m, n), dtype=torch.bfloat16).pin_memory() for m, _, _, n, _ in calls]
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        GROUP = 12   # calls per meeting point of the streams (4 MLP blocks)

        def e2e_enqueue(keep):
            """H2D copies on one side stream, the op on the main stream, D2H reads on another; the streams meet once per
            GROUP calls so that consecutive kernels stay adjacent (programmatic dependent launch needs that)."""
            s_in.wait_stream(stream)
            s_out.wait_stream(stream)
            evs = []
            with torch.cuda.stream(s_in):
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
                    ys_g.append((i, y))
                    keep.append(y)
                ev2 = torch.cuda.Event()
                ev2.record(stream)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev2)
                    for i, y in ys_g:
                        hys[i].copy_(y, non_blocking=True)
            stream.wait_stream(s_in)
            stream.wait_stream(s_out)

        keep: list = []
        erun, ecap = tm.graph(lambda: e2e_enqueue(keep))

        def e2e_step():
            if not ecap:
                keep.clear()
            erun()
            torch.cuda.current_stream().synchronize()   # the step's results are in host memory here
        esteps = max(2, min(args.steps, 10))
        ms_e2e = tm.time(e2e_step, esteps)
        bad = sum(int(not torch.equal(linear.fused_mul_mat_gguf(xs[(m, k)], W, qt).cpu(), hys[i])) for i, (m, W, qt, n, k) in enumerate(calls))
        if bad:
            raise SystemExit(f"[bench] e2e results differ from the eager op on {bad} of {len(calls)} calls")
        e2e = {"value": bytes_step / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": ms_e2e, "results_checked": len(calls),
               "api": "kaillm_b200.linear.fused_mul_mat_gguf -> torch.ops._C_gguf.ggml_mul_mat_{vec_,}a8; per call: H2D of x from "
                      "pinned memory, the op, D2H of y into pinned memory (copies on side streams that meet the compute stream every "
                      "12 calls); " + ("whole step replayed as one CUDA graph" if ecap else "eager")}
        del dxs, keep

        if not args.quick:
            # ---- the multi-GPU workload on this one GPU (config 3)
            c3_layers = C3_LAYERS
            stack = sharded.DecoderStack(make_stack(torch, synth, dev, 0, 1, c3_layers), C3_M, K_HID, dev)
            x0 = xs[(16, K_HID)]
            l0 = capi.get_option("launch_count")
            h1 = stack.forward(x0).clone()
            l3 = capi.get_option("launch_count") - l0
            r3, cap3 = tm.graph(lambda: stack.forward(x0))
            ms3 = tm.time(r3, max(3, min(args.steps, 20)))
            assert torch.equal(stack.forward(x0), h1) and bool(torch.isfinite(h1).all())
            v3 = c3_bytes(c3_layers) / (ms3 * 1e-3) / 1e9
            extra["config3"] = {"workload": workload_config(2)["workload"], "layers": c3_layers, "M": C3_M, "ms_per_step": ms3,
                                "value": v3, "unit": "GB/s", "frac_of_measured_hbm": v3 / pk["hbm"], "launches_per_step": l3,
                                "us_per_projection": ms3 * 1e3 / (4 * c3_layers), "launch": "cuda graph replay" if cap3 else "eager",
                                "bytes_per_step": c3_bytes(c3_layers)}
            del stack, r3
            torch.cuda.empty_cache()

            # ---- config 5: IQ3_S / Q2_K at M in {1, 16, 80} through the op API (the reference's dispatch decides the branch)
            low = []
            for qt in (IQ3_S, Q2_K):
                for n, k in ((8192, 2048), (N_FF, K_HID)):
                    nm = max(4, min(32, int(3e8 // (n * (k // 256) * BLOCKS[qt][1]))))
                    ws_ = [synth.wire_torch(qt, n, k, 300 + i, dev) for i in range(nm)]
                    for m in (1, 16, 80):
                        x = torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16)
                        outs = []
                        def region(ws_=ws_, x=x, qt=qt, outs=outs):
                            outs.clear()
                            for W in ws_:
                                outs.append(linear.fused_mul_mat_gguf(x, W, qt))
                        r, _ = tm.graph(region)
                        us = tm.time(r, 5) * 1e3 / nm
                        gbs = algorithmic_bytes(qt, n, k, m) / us / 1e3
                        safe = (8 if n > 5120 else 16) if qt == IQ3_S else (2 if n > 5120 else 6)
                        branch = "ggml_mul_mat_vec_a8" if m <= safe else ("ggml_mul_mat_a8" if qt != IQ3_S else "ggml_dequantize + torch matmul")
                        low.append({"type": NAMES[qt], "n": n, "k": k, "m": m, "branch": branch, "us_per_call": round(us, 2),
                                    "gbs": round(gbs, 1), "frac_of_measured_hbm": round(gbs / pk["hbm"], 3)})
                    del ws_
            extra["lowbit"] = low
            torch.cuda.empty_cache()

            # ---- ggml_dequantize of the LM head (write-bound)
            n_lm = 248320
            Wl = synth.wire_torch(Q6_K, n_lm, K_HID, 777, dev)
            msd = tm.time(lambda: capi.dequantize(Wl, Q6_K, n_lm * K_HID, torch.bfloat16), 3, warm=2)
            dq_bytes = Wl.numel() + n_lm * K_HID * 2
            extra["dequantize"] = {"workload": "Q6_K LM head 248320x5120 -> bf16", "ms": msd, "gbs": dq_bytes / (msd * 1e-3) / 1e9,
                                   "frac_of_measured_hbm": dq_bytes / (msd * 1e-3) / 1e9 / pk["hbm"],
                                   "bytes": dq_bytes, "bound": "hbm (2.54 GB written, 1.04 GB read)"}
            torch.cuda.empty_cache()

            # ---- prefill GEMM (tcgen05): TFLOP/s against the measured bf16 tensor peak
            pf = []
            Wp = mats[0][0]
            for mp in (256, 1024, 2048):
                xp = torch.randn((mp, K_HID), device=dev, generator=g).to(torch.bfloat16)
                yp = torch.empty((mp, N_FF), dtype=torch.bfloat16, device=dev)
                sp = torch.empty(capi.workspace_bytes(Q4_K, mp, N_FF, K_HID), dtype=torch.uint8, device=dev)
                msg = tm.time(lambda: capi.mul_mat(Wp, xp, Q4_K, mmq=True, out=yp, scratch=sp), 10)
                tf = 2.0 * mp * N_FF * K_HID / (msg * 1e-3) / 1e12
                pf.append({"type": "Q4_K", "n": N_FF, "k": K_HID, "m": mp, "ms": msg, "tflops": tf, "frac": tf / pk["tf"]})
            xp = torch.randn((2048, K_HID), device=dev, generator=g).to(torch.bfloat16)
            yl = torch.empty((2048, n_lm), dtype=torch.bfloat16, device=dev)
            sl = torch.empty(capi.workspace_bytes(Q6_K, 2048, n_lm, K_HID), dtype=torch.uint8, device=dev)
            msl = tm.time(lambda: capi.mul_mat(Wl, xp, Q6_K, mmq=True, out=yl, scratch=sl), 3, warm=2)
            tfl = 2.0 * 2048 * n_lm * K_HID / (msl * 1e-3) / 1e12
            pf.append({"type": "Q6_K", "n": n_lm, "k": K_HID, "m": 2048, "ms": msl, "tflops": tfl, "frac": tfl / pk["tf"]})
            extra["prefill_gemm"] = {"cases": pf, "peak_tflops": pk["tf"], "peak_source": pk["how"] + " bf16 burst",
                                     "note": "quantizer launch included (2 launches per call); fp16 operands, fp32 accumulation in TMEM"}
            del Wl, yl, sl
            torch.cuda.empty_cache()

            # ---- the reference's own CUDA kernels on the same GPU, same inputs, same run
            extra["reference_cuda"] = reference_cuda_leg(torch, tm, mats, xs, table, pf, dev, g, synth)

            # ---- mixture-of-experts ops (32 experts of Q4_K 2816x2048, top-4), with the reference's kernels beside them
            extra["moe"] = moe_leg(torch, tm, dev, synth)

    cpu = None
    if not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        stepf, nb, kind, desc = cpu_path_sample(1, frac=2)
        stepf()                                     # one untimed pass (imports, allocator, thread pool)
        passes, t0 = 0, time.perf_counter()
        while passes < 8 and (passes == 0 or time.perf_counter() - t0 < 10.0):   # about ten seconds of CPU work
            stepf()
            passes += 1
        dt = (time.perf_counter() - t0) / passes
        cpu = {"value": nb / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": kind, "seconds": dt * passes, "passes": passes,
               "sample": desc}

    cfg = workload_config(1)
    cfg.update({"layers": layers, "bytes_per_step": bytes_step, "launch": "cuda graph replay" if captured else "eager",
                "parallelism": "single GPU"})
    out = {"metric": "quantized GEMV HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
           "dtype": "int8", "data": "synthetic", "config": cfg, "frac_of_measured_hbm": value / pk["hbm"],
           "frac_of_nominal_8tbs": value / 8000.0, "clocks": clocks, "e2e": e2e, "gpu_launches": launches_step * args.steps,
           "roofline": roof, "cpu_baseline": cpu}
    out.update(extra)
    print(json.dumps(out), flush=True)


def moe_leg(torch, tm, dev, synth):
    """ggml_moe_a8_vec (8 tokens) and ggml_moe_a8 (256 tokens, expert-sorted blocks) through torch.ops._C_gguf, and the
    same calls on the reference's own build where it exists.  Synthetic routing: top_k distinct experts per token."""
    from kaillm_b200 import linear
    E, n, k, qt, top_k = 32, 2816, 2048, Q4_K, 4
    try:
        W = torch.stack([synth.wire_torch(qt, n, k, 500 + i, dev) for i in range(E)])
        ref = None
        path = os.path.join(ROOT, "oracle", "_ref", "_C_gguf_ref.so")
        if os.path.exists(path):
            torch.ops.load_library(path)
            ref = torch.ops._C_gguf_ref
        g = torch.Generator(device=dev)
        rows = []
        for tokens, which in ((8, "ggml_moe_a8_vec"), (256, "ggml_moe_a8")):
            g.manual_seed(tokens)
            x = torch.randn((tokens, k), device=dev, generator=g).to(torch.bfloat16)
            ids = torch.stack([torch.randperm(E, device=dev, generator=g)[:top_k] for _ in range(tokens)]).to(torch.int32)
            def call(ops_):
                if which == "ggml_moe_a8_vec":
                    return lambda: ops_.ggml_moe_a8_vec(x, W, ids, top_k, qt, n, tokens)
                bs = int(ops_.ggml_moe_get_block_size(qt))
                s_, e_, t_ = linear.moe_align_block_size(ids, bs, E)
                used = int(t_.item())                  # only the blocks that hold slots (set-up, outside the timed region)
                s_, e_ = s_[:used].contiguous(), e_[:used // bs].contiguous()
                return lambda: ops_.ggml_moe_a8(x, W, s_, e_, t_, qt, n, top_k, tokens)
            mine = call(torch.ops._C_gguf)
            r, _ = tm.graph(mine)
            us = tm.time(r, 10) * 1e3
            row = {"op": which, "tokens": tokens, "pairs": tokens * top_k, "experts_hit": int(torch.unique(ids).numel()), "us_per_call": round(us, 1)}
            if ref is not None:
                theirs = call(ref)
                a, b = mine().float(), theirs().float()
                row["rel_l2_to_reference"] = float((a - b).norm() / b.norm().clamp_min(1e-30))
                rr, _ = tm.graph(theirs)
                rus = tm.time(rr, 3, warm=1) * 1e3
                row.update({"reference_us": round(rus, 1), "speedup": round(rus / us, 2)})
            rows.append(row)
        return {"workload": f"{E} experts x Q4_K {n}x{k}, top-{top_k}, bf16 activations", "cases": rows}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{e!r}"[:300]}


def reference_cuda_leg(torch, tm, mats, xs, table, pf, dev, g, synth):
    """Times torch.ops._C_gguf_ref.* (the reference's csrc built unmodified by oracle/build_ref.py) on this run's inputs."""
    path = os.path.join(ROOT, "oracle", "_ref", "_C_gguf_ref.so")
    if not os.path.exists(path):
        return {"unavailable": "oracle/_ref/_C_gguf_ref.so is not built (python oracle/build_ref.py needs the reference tree)"}
    try:
        torch.ops.load_library(path)
        ref = torch.ops._C_gguf_ref
        rows = []
        mine = {(r["type"], r["m"]): r["us_per_call"] for r in table}
        for qt, n, k in ((Q4_K, N_FF, K_HID), (Q6_K, K_HID, N_FF)):
            ws_ = [W for W, t, *_ in mats if t == qt][:4]
            for m in MS:
                op = ref.ggml_mul_mat_a8 if use_mmq(m, n) else ref.ggml_mul_mat_vec_a8
                outs = []
                def region(ws_=ws_, m=m, k=k, qt=qt, n=n, op=op, outs=outs):
                    outs.clear()
                    for W in ws_:
                        outs.append(op(W, xs[(m, k)], qt, n))
                r, _ = tm.graph(region)
                us = tm.time(r, 3, warm=1) * 1e3 / len(ws_)
                rows.append({"type": NAMES[qt], "n": n, "k": k, "m": m, "op": "ggml_mul_mat_a8" if use_mmq(m, n) else "ggml_mul_mat_vec_a8",
                             "reference_us": round(us, 1), "this_us": mine[(NAMES[qt], m)], "speedup": round(us / mine[(NAMES[qt], m)], 2)})
        W = mats[0][0]
        xp = torch.randn((2048, K_HID), device=dev, generator=g).to(torch.bfloat16)
        msr = tm.time(lambda: ref.ggml_mul_mat_a8(W, xp, Q4_K, N_FF), 2, warm=1)
        ours = [c for c in pf if c["type"] == "Q4_K" and c["m"] == 2048][0]["ms"]
        return {"decode": rows, "prefill_q4k_m2048": {"reference_ms": msr, "this_ms": ours, "speedup": msr / ours,
                                                        "reference_tflops": 2.0 * 2048 * N_FF * K_HID / (msr * 1e-3) / 1e12},
                "what": "vllm_gguf_plugin/csrc/gguf/gguf_kernel.cu + torch_bindings.cpp compiled unmodified for sm_100a (oracle/build_ref.py), "
                        "called through their own torch ops in CUDA-graph replay over 4 distinct matrices (cold L2)"}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{e!r}"[:300]}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="kq", choices=["kq", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="layers of the stack (default: 16 MLP blocks at N=1, 64 decoder layers at N>1)")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--flag-gather", action="store_true", help="N>1: end every gather with the flag hand-shake instead of sentinel polling")
    ap.add_argument("--no-fused-gather", action="store_true", help="N>1: GEMV and peer-store gather as two kernels")
    ap.add_argument("--nccl", action="store_true", help="N>1: gather with NCCL instead of the library's peer-store kernel")
    ap.add_argument("--quick", action="store_true", help="N=1: only the main workload, roofline and e2e (no further legs)")
    ap.add_argument("--no-one-gpu", action="store_true", help="N>1: skip the one-GPU run of the same workload on rank 0")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    if args.warmup < 3:
        args.warmup = 3

    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the GGUF kernels have no CPU fallback)")
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        run_multi(args, torch, dist, dev, rank, world, local)
    else:
        run_single(args, torch, dev, local)


if __name__ == "__main__":
    main()
