"""kq_p2p_allgather on two GPUs: the pushed slices equal an NCCL all-gather, eagerly and in a replayed CUDA graph.

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
