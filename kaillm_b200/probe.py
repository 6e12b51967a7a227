"""Run one configuration of the decode / prefill path a few times - the unit a profiler captures.

    python -m kaillm_b200.probe --type 12 --n 17408 --k 5120 --m 16 [--opt gemv_impl=6 ...] [--mats 4] [--mmq] [--full]

`--dequantize` runs kq_dequantize of each matrix instead; `--moe E` runs kq_moe_a8 (expert-sorted blocks) over E experts of
n x k with `--m` tokens and `--topk` experts per token, `--mats` times.  `--mats` distinct weight matrices are generated from seeds (so the weights of a launch are never in L2 from the launch
before), the activations are prepared once (`--full`: with every call, through kq_mul_mat_vec_a8 / kq_mul_mat_a8) and
each matrix is multiplied once; the status word of the scratch is checked at the end.  Under `ncu` pick the kernel with
`-k regex:...` and skip the first launch (`-s 1`).  Options are those of kq_set_option (gemv_impl, kres, umma, pdl ...).
"""
from __future__ import annotations

import argparse
import sys

import torch

from . import capi, synth


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--type", type=int, default=12, help="GGML type id")
    ap.add_argument("--n", type=int, default=17408)
    ap.add_argument("--k", type=int, default=5120)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--mats", type=int, default=4)
    ap.add_argument("--mmq", action="store_true", help="MMQ arithmetic (kq_mul_mat_a8)")
    ap.add_argument("--full", action="store_true", help="quantize the activations with every call")
    ap.add_argument("--dequantize", action="store_true", help="run kq_dequantize of the matrices (to bf16) instead of the product")
    ap.add_argument("--moe", type=int, default=0, metavar="E", help="run kq_moe_a8 over E experts of n x k instead")
    ap.add_argument("--topk", type=int, default=4)
    ap.add_argument("--opt", action="append", default=[], metavar="NAME=VALUE")
    args = ap.parse_args(argv)
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    for o in args.opt:
        name, val = o.split("=")
        capi.set_option(name, int(val))
    qt, n, k, m = args.type, args.n, args.k, args.m
    if args.moe:
        from . import linear
        e = args.moe
        W = torch.stack([synth.wire_torch(qt, n, k, 100 + i, dev) for i in range(e)])
        g = torch.Generator(device=dev)
        g.manual_seed(m)
        x = torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16)
        ids = torch.stack([torch.randperm(e, device=dev, generator=g)[:args.topk] for _ in range(m)]).to(torch.int32)
        s_, e_, t_ = linear.moe_align_block_size(ids, capi.lib.kq_moe_block_size(qt), e)
        ys = [capi.moe_a8(W, x, s_, e_, t_, args.topk, qt) for _ in range(args.mats)]
        torch.cuda.synchronize()
        ok = all(bool(torch.isfinite(y.float()).all()) for y in ys)
        print(f"type {qt}: {e} experts of {n} x {k}, {m} tokens, top-{args.topk}: {args.mats} calls, finite {ok}")
        return 0 if ok else 1
    ws = [synth.wire_torch(qt, n, k, 100 + i, dev) for i in range(args.mats)]
    if args.dequantize:
        outs = [capi.dequantize(w, qt, n * k, torch.bfloat16) for w in ws]
        torch.cuda.synchronize()
        ok = all(bool(torch.isfinite(o.float()).all()) for o in outs)
        print(f"type {qt} n {n} k {k}: {args.mats} matrices dequantized to bf16, finite {ok}")
        return 0 if ok else 1
    x = torch.randn((m, k), device=dev).to(torch.bfloat16)
    y = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    scratch = torch.empty(capi.workspace_bytes(qt, m, n, k), dtype=torch.uint8, device=dev)
    torch.cuda.synchronize()
    if not args.full:
        capi.prepare_q8(x, qt, n, scratch)
    for w in ws:
        if args.full:
            capi.mul_mat(w, x, qt, mmq=args.mmq, out=y, scratch=scratch)
        else:
            capi.mul_mat_prepared(w, qt, m, k, y, scratch, mmq=args.mmq)
    torch.cuda.synchronize()
    status = capi.read_status(qt, m, n, k, scratch)
    print(f"type {qt} n {n} k {k} m {m}: {args.mats} matrices, status {status}, launches {capi.get_option('launch_count')}")
    return 0 if status == 0 and bool(torch.isfinite(y.float()).all()) else 1


if __name__ == "__main__":
    sys.exit(main())
