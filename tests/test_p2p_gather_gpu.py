"""kq_p2p_allgather and kq_mul_mat_prepared_gather on two GPUs: the pushed slices equal an NCCL all-gather, eagerly
and in a replayed CUDA graph; the GEMV with the gather in its epilogue equals GEMV + NCCL gather bit for bit; a decoder
stack gives the same bits with NCCL gathers, with the flag hand-shake and with sentinel-polled gathers.

Runs as two child processes (one per GPU, rendezvous on 127.0.0.1); skipped on a box with fewer than two GPUs."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank: int, world: int, port: int, q) -> None:
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        sys.path.insert(0, ROOT)
        import torch.distributed as dist

        from kaillm_b200 import sharded
        dev = torch.device(f"cuda:{rank}")
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", device_id=dev)
        pg = sharded.P2PGather(max_bytes=16 * 2176 * 2, nbuf=2, device=dev)
        g = torch.Generator(device=dev)
        g.manual_seed(100 + rank)
        ok = True
        for m, per, dt in [(1, 2176, torch.bfloat16), (16, 2176, torch.bfloat16), (5, 640, torch.float32), (3, 7, torch.float16)]:
            y = torch.randn((m, per), device=dev, generator=g).to(dt)
            want = sharded.gather_columns(y)
            for rep in range(3):                      # the same buffer three times: epochs advance in step
                got = pg.gather(y, rep & 1)
                ok &= bool(torch.equal(got, want))
        # replay inside a CUDA graph
        y = torch.randn((8, 2176), device=dev, generator=g).to(torch.bfloat16)
        want = sharded.gather_columns(y)
        st = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(st):
            pg.gather(y, 0)
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=st):
                out = pg.gather(y, 0)
            for _ in range(4):
                gr.replay()
            torch.cuda.synchronize()
            ok &= bool(torch.equal(out, want))
        pg.check()
        dist.barrier()
        q.put((rank, "ok" if ok else "mismatch"))
    except Exception as e:  # noqa: BLE001 - reported to the parent
        q.put((rank, f"error: {e!r}"))
    finally:
        os._exit(0)


@pytest.mark.gpu
def test_p2p_allgather_matches_nccl():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()          # synchronous put: the children leave through os._exit right after it
    procs = [ctx.Process(target=_worker, args=(r, 2, 29533, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=150)
    res = {}
    while not q.empty():
        r, msg = q.get()
        res[r] = msg
    for p in procs:
        if p.is_alive():
            p.kill()
    assert res == {0: "ok", 1: "ok"}, res


def _fused_worker(rank: int, world: int, port: int, q) -> None:
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                          NCCL_NVLS_ENABLE="0")
        sys.path.insert(0, ROOT)
        import torch.distributed as dist

        from kaillm_b200 import capi, sharded, synth
        dev = torch.device(f"cuda:{rank}")
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", device_id=dev)
        pg = sharded.P2PGather(max_bytes=20 * 8704 * 4, nbuf=4, device=dev)
        bad = []
        # (type, N, K, tokens, dtype, expect one kernel)
        cases = [(12, 17408, 5120, 16, torch.bfloat16, True), (12, 17408, 5120, 5, torch.float16, True),
                 (14, 5120, 17408, 16, torch.bfloat16, True), (14, 5120, 17408, 1, torch.float32, True),    # split-K finish
                 (8, 8192, 5120, 16, torch.bfloat16, True), (2, 4096, 4096, 9, torch.bfloat16, True),
                 (21, 2048, 2048, 3, torch.bfloat16, True), (10, 2048, 2048, 16, torch.float16, True),
                 (12, 4096, 2048, 20, torch.bfloat16, False),      # more than one pass of 16 tokens: two kernels
                 (13, 2048, 1024, 4, torch.bfloat16, False),       # a format only the general kernel covers
                 (8, 2 * 1031, 512, 2, torch.float32, False)]      # slices whose rows are not 16-byte aligned
        for ci, (qt, n, k, m, dt, want_fused) in enumerate(cases):
            per = n // world
            wfull = torch.from_numpy(synth.wire_numpy(qt, n, k, seed=50 + ci))
            w = sharded.shard_rows(wfull, rank, world).contiguous().to(dev)
            x = torch.from_numpy(synth.activations_numpy(m, k, seed=70 + ci)).to(dev).to(dt)
            scratch = torch.empty(capi.workspace_bytes(qt, m, per, k), dtype=torch.uint8, device=dev)
            yl = torch.empty((m, per), dtype=dt, device=dev)
            capi.prepare_q8(x, qt, per, scratch)
            if want_fused:
                capi.set_option("gemv_impl", 6)      # the kernel the one-kernel path runs, on the same shard
            capi.mul_mat_prepared(w, qt, m, k, yl, scratch)
            capi.set_option("gemv_impl", 0)
            want = sharded.gather_columns(yl)
            for rep in range(3):
                got, fused = pg.project(w, qt, m, k, scratch, dt, ci & 3)
                torch.cuda.synchronize()
                if fused != want_fused or not torch.equal(got, want):
                    bad.append((ci, rep, fused, float((got.float() - want.float()).abs().max())))
            if want_fused:                           # the option turns the epilogue off: same result from two kernels
                capi.set_option("no_fused_gather", 1)
                got, fused = pg.project(w, qt, m, k, scratch, dt, ci & 3)
                capi.set_option("no_fused_gather", 0)
                torch.cuda.synchronize()
                if fused or float((got.float() - want.float()).abs().max()) > 1e-2 * float(want.float().abs().max()):
                    bad.append((ci, "two-kernel", fused))
            dist.barrier()
        # a replayed graph of prepare + fused projection
        qt, n, k, m, dt = 12, 17408, 5120, 16, torch.bfloat16
        per = n // world
        w = sharded.shard_rows(torch.from_numpy(synth.wire_numpy(qt, n, k, seed=9)), rank, world).contiguous().to(dev)
        x = torch.from_numpy(synth.activations_numpy(m, k, seed=10)).to(dev).to(dt)
        scratch = torch.empty(capi.workspace_bytes(qt, m, per, k), dtype=torch.uint8, device=dev)
        yl = torch.empty((m, per), dtype=dt, device=dev)
        capi.prepare_q8(x, qt, per, scratch)
        capi.set_option("gemv_impl", 6)
        capi.mul_mat_prepared(w, qt, m, k, yl, scratch)
        capi.set_option("gemv_impl", 0)
        want = sharded.gather_columns(yl)
        st = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(st):
            capi.prepare_q8(x, qt, per, scratch)
            pg.project(w, qt, m, k, scratch, dt, 0)
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=st):
                capi.prepare_q8(x, qt, per, scratch)
                out, fused = pg.project(w, qt, m, k, scratch, dt, 0)
            for _ in range(5):
                gr.replay()
            torch.cuda.synchronize()
            if not fused or not torch.equal(out, want):
                bad.append(("graph", fused))
        pg.check()
        if capi.read_status(qt, m, per, k, scratch):
            bad.append(("status", capi.read_status(qt, m, per, k, scratch)))
        dist.barrier()
        # ---- a small decoder stack three ways: NCCL gathers, flag hand-shake in the GEMV, sentinel-polled gathers
        hidden, ffn, mm, layers = 2048, 4096, 16, 3
        groups = [("qkv", 8, 3072, hidden), ("o", 8, hidden, hidden), ("gate_up", 12, 2 * ffn, hidden), ("down", 14, hidden, ffn)]
        weights = []
        for li in range(layers):
            d = {}
            for gi, (name, qt_, n_, k_) in enumerate(groups):
                wf = torch.from_numpy(synth.wire_numpy(qt_, n_, k_, seed=300 + 10 * li + gi))
                d[name] = (sharded.shard_rows(wf, rank, world).contiguous().to(dev), qt_, n_, k_)
            weights.append(d)
        h0 = (torch.from_numpy(synth.activations_numpy(mm, hidden, seed=77)).to(dev) * 0.5).to(torch.bfloat16)
        pg2 = sharded.P2PGather(max_bytes=mm * 2 * ffn // world * 2, nbuf=4, device=dev)
        pg3 = sharded.P2PGather(max_bytes=mm * 2 * ffn // world * 2, nbuf=4, device=dev)
        ref = sharded.DecoderStack(weights, mm, hidden, dev).forward(h0).clone()
        flag = sharded.DecoderStack(weights, mm, hidden, dev, p2p=pg2, wait_in_consumer=False)
        poll = sharded.DecoderStack(weights, mm, hidden, dev, p2p=pg3, wait_in_consumer=True)
        for name, stk in (("flag", flag), ("poll", poll)):
            for rep in range(3):                 # buffers are reused from the second pass on
                out = stk.forward(h0).clone()
                torch.cuda.synchronize()
                if not torch.equal(out, ref):
                    bad.append((name, rep, float((out.float() - ref.float()).abs().max())))
            stk.check()
            if not all(stk.fused.values()):
                bad.append((name, "not fused", dict(stk.fused)))
            seen = []
            stk.forward(h0, on_output=lambda li, nm, y, prep: seen.append(bool(torch.isfinite(y.float()).all())))
            if len(seen) != 4 * layers or not all(seen):
                bad.append((name, "hook", seen))
        # sentinel-polled stack with the gather as a second kernel (the fall-back of shapes the GEMV epilogue cannot carry)
        capi.set_option("no_fused_gather", 1)
        for rep in range(2):
            out = poll.forward(h0).clone()
            torch.cuda.synchronize()
            if not torch.equal(out, ref) or any(poll.fused.values()):
                bad.append(("poll, two kernels", rep, dict(poll.fused)))
        capi.set_option("no_fused_gather", 0)
        dist.barrier()
        with torch.cuda.stream(st):
            poll.forward(h0)
            torch.cuda.synchronize()
            gr2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr2, stream=st):
                out = poll.forward(h0)
            for _ in range(4):
                gr2.replay()
            torch.cuda.synchronize()
            if not torch.equal(out, ref):
                bad.append(("poll graph", float((out.float() - ref.float()).abs().max())))
        poll.check()
        if capi.arrival_status():
            bad.append(("arrival flag", capi.arrival_status()))
        dist.barrier()
        # ---- a peer that does not take part: the bounded wait of the flag hand-shake runs out (about two seconds), the
        # kernel returns, the status word names the silent rank, and the context stays usable.  Rank 1 simply makes no
        # call (it is alive and idle: nothing faults, nothing is killed).
        pg4 = sharded.P2PGather(max_bytes=16 * 1024 * 2, nbuf=1, device=dev)
        qt_, n_, k_, m_ = 12, 2048, 1024, 4
        w_ = sharded.shard_rows(torch.from_numpy(synth.wire_numpy(qt_, n_, k_, seed=5)), rank, world).contiguous().to(dev)
        x_ = torch.from_numpy(synth.activations_numpy(m_, k_, seed=6)).to(dev).to(torch.bfloat16)
        sc_ = torch.empty(capi.workspace_bytes(qt_, m_, n_ // world, k_), dtype=torch.uint8, device=dev)
        if rank == 0:
            capi.prepare_q8(x_, qt_, n_ // world, sc_)
            pg4.project(w_, qt_, m_, k_, sc_, torch.bfloat16, 0)
            torch.cuda.synchronize()
            try:
                pg4.check()
                bad.append(("silent peer not reported",))
            except RuntimeError as e:
                if "rank 1" not in str(e):
                    bad.append(("wrong report", str(e)))
            y_ = torch.empty((m_, n_ // world), dtype=torch.bfloat16, device=dev)
            capi.mul_mat_prepared(w_, qt_, m_, k_, y_, sc_)          # the GPU still works
            torch.cuda.synchronize()
            if not bool(torch.isfinite(y_.float()).all()):
                bad.append(("context unusable after the time-out",))
        dist.barrier()
        q.put((rank, "ok" if not bad else f"mismatch: {bad[:6]}"))
    except Exception as e:  # noqa: BLE001 - reported to the parent
        import traceback
        q.put((rank, f"error: {e!r} {traceback.format_exc()[-600:]}"))
    finally:
        os._exit(0)


@pytest.mark.gpu
def test_gemv_with_gather_in_its_epilogue_matches_gemv_plus_nccl():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    procs = [ctx.Process(target=_fused_worker, args=(r, 2, 29537, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=400)
    res = {}
    while not q.empty():
        r, msg = q.get()
        res[r] = msg
    for p in procs:
        if p.is_alive():
            p.kill()
    assert res == {0: "ok", 1: "ok"}, res
