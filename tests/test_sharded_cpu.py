"""world_size-2 gloo test of the row-shard + all-gather glue (CPU; the matmul is the oracle's)."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    try:
        _worker_body(rank, world, port, q)
    except Exception as e:  # report instead of leaving the parent to time out
        q.put((rank, False, repr(e)))
        raise


def _worker_body(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from kaillm_b200 import sharded, synth
    from oracle import gguf_oracle as O

    qt, n, k, m = 12, 64, 512, 3
    w = torch.from_numpy(synth.wire_numpy(qt, n, k, seed=1))
    x = torch.from_numpy(synth.activations_numpy(m, k, seed=2))

    def matmul(xx, ww, t):
        return torch.from_numpy(O.mul_mat(ww.numpy(), t, xx.numpy(), "mmvq"))

    layer = sharded.ShardedGGUFLinear.from_full(w, qt, matmul)
    assert layer.qweight.shape[0] == n // world
    y = layer.apply(x)
    full = matmul(x, w, qt)
    ok = bool(torch.equal(y, full))      # row sharding does not change per-row arithmetic
    try:
        sharded.shard_rows(w[:63], rank, world)
        ok = False
    except ValueError:
        pass
    q.put((rank, ok, tuple(y.shape)))
    dist.barrier()
    dist.destroy_process_group()


def test_row_shard_all_gather_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=90) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in res) == [0, 1]
    assert all(r[1] for r in res) and all(r[2] == (3, 64) for r in res)
