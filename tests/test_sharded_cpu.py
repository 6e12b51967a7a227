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


class _OracleCapi:
    """Stands in for the C-ABI bindings on a box without a GPU: the producers keep the activations as fp32, the GEMV is
    the oracle's.  Only the orchestration of DecoderStack (sharding, gathers, chaining) is under test here."""

    def __init__(self, real):
        self.workspace_bytes = real.workspace_bytes
        self.act = None

    def prepare_q8_rmsnorm(self, h, gamma, eps, qt, n, scratch, **kw):
        x = h.float()
        self.act = (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)).to(h.dtype).float() * gamma.float()

    def prepare_q8(self, a, qt, n, scratch, **kw):
        self.act = a.float()

    def prepare_q8_swiglu(self, gu, qt, n, scratch, **kw):
        f = gu.shape[1] // 2
        self.act = torch.nn.functional.silu(gu[:, :f].float()) * gu[:, f:].float()

    def mul_mat_prepared(self, W, qt, m, k, out, scratch):
        from oracle import gguf_oracle as O
        out.copy_(torch.from_numpy(O.mul_mat(W.numpy(), qt, self.act.contiguous().numpy(), "mmvq")))

    def read_status(self, *a):
        return 0


def _stack_worker(rank, world, port, q):
    try:
        sys.path.insert(0, ROOT)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        singles = [dist.new_group([r]) for r in range(world)]
        from kaillm_b200 import capi, sharded, synth

        hidden, ffn, m, layers = 256, 512, 3, 2
        groups = [("qkv", 8, 512, hidden), ("o", 8, hidden, hidden), ("gate_up", 12, 2 * ffn, hidden), ("down", 14, hidden, ffn)]
        full, mine = [], []
        for li in range(layers):
            f, s = {}, {}
            for gi, (name, qt, n, k) in enumerate(groups):
                w = torch.from_numpy(synth.wire_numpy(qt, n, k, seed=100 + 10 * li + gi))
                f[name] = (w, qt, n, k)
                s[name] = (sharded.shard_rows(w, rank, world).contiguous(), qt, n, k)
            full.append(f)
            mine.append(s)
        h0 = torch.from_numpy(synth.activations_numpy(m, hidden, seed=5)).to(torch.bfloat16)
        cpu = torch.device("cpu")
        one = sharded.DecoderStack(full, m, hidden, cpu, group=singles[rank])
        one._capi = _OracleCapi(capi)
        two = sharded.DecoderStack(mine, m, hidden, cpu)
        two._capi = _OracleCapi(capi)
        seen = []
        want = one.forward(h0).clone()
        got = two.forward(h0, on_output=lambda li, name, y, prep: seen.append((li, name, tuple(y.shape))))
        ok = one.world == 1 and two.world == world and bool(torch.equal(got, want)) and bool(torch.isfinite(got.float()).all())
        ok = ok and seen == [(li, name, (m, n)) for li in range(layers) for name, _, n, _ in groups]
        two.check()
        q.put((rank, ok, tuple(got.shape)))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:
        q.put((rank, False, repr(e)))
        raise


def test_decoder_stack_two_ranks_equals_one_rank():
    """Row-sharded chain of producers, projections and gathers over two gloo ranks = the same chain on the whole
    matrices (per-row arithmetic does not depend on the shard), with the GEMV done by the oracle."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_stack_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(r[1] is True for r in res) and all(r[2] == (3, 256) for r in res), res
