"""Row-sharded multi-GPU execution of a GGUF linear layer.

Output rows are independent, so a weight `uint8 [N, rowbytes]` is split on dim 0 into `world` contiguous
slices of N/world rows - exactly the column-parallel slicing the reference's loader performs
(`load_column_parallel_weight`, vllm_gguf_plugin/quantization/params.py:230-247).  Activations are
replicated; every rank computes `[M, N/world]` and the slices are all-gathered along N.  The reference
has no collective of its own (the gather lives in vLLM's ColumnParallelLinear); here it is one
`all_gather_into_tensor` on the rank-major buffer `[world, M, N/world]` followed by a strided view.

One process per GPU (`torch.distributed`, backend "nccl" on GPUs; "gloo" works for the CPU tests with a
stand-in compute function).
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def shard_rows(qweight: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rows [rank*N/world, (rank+1)*N/world) of a wire tensor (N must divide evenly)."""
    n = qweight.shape[0]
    if n % world:
        raise ValueError(f"N={n} is not divisible by the number of ranks {world}")
    per = n // world
    return qweight.narrow(0, rank * per, per)


def gather_columns(y_local: torch.Tensor, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather `[M, N/world]` slices into `[M, N]` (rank r owns columns r*N/world ...)."""
    world = dist.get_world_size(group)
    m, per = y_local.shape
    if world == 1:
        return y_local
    buf = out if out is not None else torch.empty((world, m, per), dtype=y_local.dtype, device=y_local.device)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(buf, y_local.contiguous(), group=group)
    else:  # gloo has no flat all-gather; a list of views into the same buffer is equivalent
        dist.all_gather([buf[r] for r in range(world)], y_local.contiguous(), group=group)
    return buf.permute(1, 0, 2).reshape(m, world * per)


class P2PGather:
    """All-gather of output slices by peer stores (kq_p2p_allgather) over buffers in torch symmetric memory.

    One instance owns `nbuf` gather buffers of `max_bytes * world` bytes each plus the flag arrays, all carved from
    one symmetric allocation; buffer b uses flag slot b.  `gather(y_local, b)` launches one kernel on the current
    stream and returns the local buffer viewed as [M, N] columns (rank r owns columns r*N/world ...).  Use a different
    buffer index for calls that may be in flight at the same time, and alternate two indices on one stream when the
    gathered data is read by later kernels.  Raises if symmetric memory cannot be set up (the caller then keeps
    the NCCL path)."""

    FLAG_BYTES_PER_SLOT = 8 * 4

    def __init__(self, max_bytes: int, nbuf: int, device: torch.device, group=None):
        import os
        # only plain peer loads/stores are used here: ask torch not to bind the allocation to an NVLink multicast object
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        from . import capi
        self._capi = capi
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("P2PGather supports at most 8 ranks")
        self.max_bytes = (max_bytes + 255) // 256 * 256
        self.nbuf = nbuf
        self.buf_bytes = self.max_bytes * self.world
        flag_bytes = (nbuf * self.FLAG_BYTES_PER_SLOT + 255) // 256 * 256
        total = flag_bytes + nbuf * self.buf_bytes
        self.mem = symm.empty((total,), dtype=torch.uint8, device=device)
        self.mem.zero_()
        self.mem[flag_bytes:].fill_(0xFF)       # data buffers start as "nothing has arrived" (the arrival sentinel)
        torch.cuda.synchronize(device)
        self.hdl = symm.rendezvous(self.mem, group.group_name)
        self.hdl.barrier()                      # every rank's flags are zero before anyone publishes
        bases = [int(p) for p in self.hdl.buffer_ptrs]
        self.flag_ptrs = bases
        self.data_ptrs = [b + flag_bytes for b in bases]
        self.flag_bytes = flag_bytes
        self.epoch = torch.zeros(nbuf, dtype=torch.int32, device=device)
        self.done = torch.zeros(nbuf, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    def gather(self, y_local: torch.Tensor, b: int) -> torch.Tensor:
        """Columns of all ranks as one [M, N] tensor (a copy out of the gather buffer)."""
        m, per = y_local.shape
        return self.gather_raw(y_local, b).permute(1, 0, 2).reshape(m, self.world * per)

    def gather_raw(self, y_local: torch.Tensor, b: int) -> torch.Tensor:
        """One kernel launch; returns the local gather buffer itself, viewed as [world, M, N/world]."""
        m, per = y_local.shape
        y_local = y_local.contiguous()
        nbytes = y_local.numel() * y_local.element_size()
        if nbytes > self.max_bytes or not 0 <= b < self.nbuf:
            raise ValueError(f"slice of {nbytes} bytes / buffer {b} outside what this P2PGather was sized for")
        dst = [p + b * self.buf_bytes for p in self.data_ptrs]
        self._capi.p2p_allgather(y_local, dst, self.flag_ptrs, self.epoch, self.done, b, self.rank, self.status)
        off = self.flag_bytes + b * self.buf_bytes
        return self.mem[off:off + self.world * nbytes].view(y_local.dtype).view(self.world, m, per)

    def gather_cols(self, y_local: torch.Tensor, b: int) -> torch.Tensor:
        """One kernel launch; returns the local buffer viewed as the row-major [M, N] output (rank r wrote columns
        r*N/world ..), ready to be read by the next layer without a transposing copy."""
        m, per = y_local.shape
        y_local = y_local.contiguous()
        nbytes = y_local.numel() * y_local.element_size()
        if nbytes > self.max_bytes or not 0 <= b < self.nbuf:
            raise ValueError(f"slice of {nbytes} bytes / buffer {b} outside what this P2PGather was sized for")
        dst = [p + b * self.buf_bytes for p in self.data_ptrs]
        row_stride = self.world * per * y_local.element_size()
        self._capi.p2p_allgather_2d(y_local, dst, row_stride, self.flag_ptrs, self.epoch, self.done, b, self.rank, self.status)
        off = self.flag_bytes + b * self.buf_bytes
        return self.mem[off:off + self.world * nbytes].view(y_local.dtype).view(m, self.world * per)

    def buffer(self, b: int, m: int, n: int, dtype: torch.dtype) -> torch.Tensor:
        """Gather buffer `b` viewed as a row-major [m, n] tensor."""
        nbytes = m * n * torch.empty((), dtype=dtype).element_size()
        off = self.flag_bytes + b * self.buf_bytes
        return self.mem[off:off + nbytes].view(dtype).view(m, n)

    def project(self, W: torch.Tensor, qtype: int, m: int, k: int, scratch: torch.Tensor, dtype: torch.dtype, b: int,
                mmq: bool = False, wait_in_consumer: bool = False, reset: torch.Tensor | None = None) -> tuple[torch.Tensor, bool]:
        """This rank's weight slice times the activations prepared in `scratch`, gathered into buffer `b` by the
        GEMV's own epilogue where the library can do that (kq_mul_mat_prepared_gather; otherwise GEMV + gather kernel).
        Returns (local buffer viewed as the row-major [M, N] output, whether it was one kernel).
        wait_in_consumer: no hand-shake; the buffer's next reader polls the elements against the arrival sentinel
        (prepare_q8*(wait_arrival=True) or capi.wait_arrival), and `reset` - the gather buffer the producer of this call's
        activations has consumed - is refilled with the sentinel for its next use."""
        per = W.shape[0]
        esz = torch.empty((), dtype=dtype).element_size()
        nbytes = m * per * esz
        if nbytes > self.max_bytes or not 0 <= b < self.nbuf:
            raise ValueError(f"slice of {nbytes} bytes / buffer {b} outside what this P2PGather was sized for")
        dst = [p + b * self.buf_bytes for p in self.data_ptrs]
        fused = self._capi.mul_mat_prepared_gather(W, qtype, m, k, scratch, dst, self.world * per, dtype, self.flag_ptrs,
                                                   self.epoch, self.done, b, self.rank, self.status, mmq, wait_in_consumer,
                                                   reset.data_ptr() if reset is not None else 0,
                                                   (reset.numel() * reset.element_size() + 15) // 16 * 16 if reset is not None else 0)
        off = self.flag_bytes + b * self.buf_bytes
        return self.mem[off:off + self.world * nbytes].view(dtype).view(m, self.world * per), fused

    def check(self) -> None:
        """Synchronises; raises if any gather's bounded wait for a peer ran out."""
        st = int(self.status.item())
        if st:
            who = "the gathered values (sentinel poll)" if st >= 40 else f"rank {st - 16 if st >= 16 else st - 1}"
            raise RuntimeError(f"peer gather: wait for {who} timed out (status {st})")


class ShardedGGUFLinear:
    """One rank's slice of a row-sharded layer plus the gather."""

    def __init__(self, qweight_local: torch.Tensor, qweight_type: int,
                 matmul: Callable[[torch.Tensor, torch.Tensor, int], torch.Tensor], group=None):
        self.qweight = qweight_local
        self.qweight_type = qweight_type
        self.matmul = matmul
        self.group = group

    @classmethod
    def from_full(cls, qweight: torch.Tensor, qweight_type: int, matmul, group=None):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        return cls(shard_rows(qweight, rank, world).contiguous(), qweight_type, matmul, group)

    def local(self, x: torch.Tensor) -> torch.Tensor:
        return self.matmul(x, self.qweight, self.qweight_type)

    def apply(self, x: torch.Tensor) -> torch.Tensor:
        return gather_columns(self.local(x), self.group)


class DecoderStack:
    """The linear layers of a decoder stack, row-sharded, chained through the fused activation producers.

    Per layer, in the order a transformer runs them (attention itself is not part of this path and is left out):

        h  -> RMSNorm -> q8_1 -> merged q/k/v projection  [M, 8192]   -> all-gather
           -> q8_1 of the first `hidden` columns -> o projection [M, hidden] -> all-gather
           -> RMSNorm -> q8_1 -> merged gate/up projection [M, 2*ffn] -> all-gather
           -> silu(gate) * up -> q8_1 -> down projection [M, hidden]  -> all-gather -> h of the next layer

    Merged projections are ONE weight tensor and ONE call, as the reference runs same-type merged layers
    (quantization/linear.py:377-381); every projection is sharded on its output rows (quantization/params.py:230-247), so
    each call ends in an all-gather of `[M, N/world]` slices into a row-major `[M, N]` buffer that the next producer
    reads in place.  Each projection group costs one producer launch (activation + quantization) and one GEMV launch
    whose epilogue stores the slice into every rank's buffer (kq_mul_mat_prepared_gather); shapes that kernel does not
    cover cost a separate gather launch.

    weights: per layer a dict {"qkv", "o", "gate_up", "down"} -> (local shard uint8 [N/world, rowbytes], type, N, K).
    """

    GROUPS = ("qkv", "o", "gate_up", "down")

    def __init__(self, weights: list[dict], m: int, hidden: int, device: torch.device, p2p: "P2PGather | None" = None,
                 group=None, eps: float = 1e-6, dtype: torch.dtype = torch.bfloat16, wait_in_consumer: bool = True,
                 unsharded: bool = False):
        """`unsharded`: the weights are whole tensors and this process runs the stack alone, whatever process group
        exists (a single-GPU baseline inside a multi-rank job)."""
        from . import capi
        self._capi = capi
        self.w = weights
        self.m, self.hidden, self.eps, self.dtype = m, hidden, eps, dtype
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized() and not unsharded) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.group = group
        self.p2p = p2p
        self.dev = device
        # gathers without a hand-shake: the next producer polls the gathered values against the arrival sentinel
        self.wait_in_consumer = bool(wait_in_consumer) and p2p is not None
        self.gamma = torch.ones(hidden, dtype=dtype, device=device)
        ws = 0
        self.nfull = {}
        for name in self.GROUPS:
            _, qt, n, k = weights[0][name]
            self.nfull[name] = n
            ws = max(ws, capi.workspace_bytes(qt, m, n // self.world, k))
        self.scratch = torch.empty(ws, dtype=torch.uint8, device=device)
        self.ylocal = {name: torch.empty((m, self.nfull[name] // self.world), dtype=dtype, device=device) for name in self.GROUPS}
        # world == 1: the GEMV writes the full output itself; otherwise the gather buffers (slot = index in GROUPS)
        self.yfull = {name: torch.empty((m, self.nfull[name]), dtype=dtype, device=device) for name in self.GROUPS} if self.world == 1 else {}
        self.nccl_buf = {}
        self.fused = {}     # per group: did the last call run GEMV + gather as one kernel
        self.ws_shape = {name: (weights[0][name][1], m, self.nfull[name] // self.world, weights[0][name][3]) for name in self.GROUPS}
        if self.world > 1 and p2p is None:
            self.nccl_buf = {name: torch.empty((self.world, m, self.nfull[name] // self.world), dtype=dtype, device=device)
                             for name in self.GROUPS}

    def _project(self, name: str, W: torch.Tensor, qt: int, n: int, k: int, check=None) -> torch.Tensor:
        """GEMV on the activations held in self.scratch, then the gather; returns the row-major [M, N] output."""
        capi = self._capi
        if self.world == 1:
            out = self.yfull[name]
            capi.mul_mat_prepared(W, qt, self.m, k, out, self.scratch)
            return out
        if self.p2p is not None:
            slot = self.GROUPS.index(name)
            reset = None
            if self.wait_in_consumer:      # the buffer this call's activations came from has been consumed: refill it
                prev = self.GROUPS[slot - 1]
                reset = self.p2p.buffer((slot - 1) % len(self.GROUPS), self.m, self.nfull[prev], self.dtype)
            out, self.fused[name] = self.p2p.project(W, qt, self.m, k, self.scratch, self.dtype, slot,
                                                     wait_in_consumer=self.wait_in_consumer, reset=reset)
            return out
        yl = self.ylocal[name]
        capi.mul_mat_prepared(W, qt, self.m, k, yl, self.scratch)
        buf = self.nccl_buf[name]
        dist.all_gather_into_tensor(buf.view(self.world * self.m, -1), yl, group=self.group)
        return buf.permute(1, 0, 2).reshape(self.m, n)     # a transposing copy: the baseline the peer-store gather removes

    def check(self) -> None:
        """Synchronises; raises if a bounded wait inside any kernel of the stack ran out."""
        for name, (qt, m, n, k) in self.ws_shape.items():
            st = self._capi.read_status(qt, m, n, k, self.scratch)
            if st:
                raise RuntimeError(f"decoder stack: kernel status {st} (a bounded wait inside the last GEMV ran out)")
            break   # the status word sits at offset 0 for every shape
        if self.p2p is not None:
            self.p2p.check()
            if self.wait_in_consumer:
                with torch.cuda.device(self.dev):
                    st = self._capi.arrival_status()
                if st:
                    raise RuntimeError(f"decoder stack: an arrival poll ran out (status {st}): a rank stopped storing its outputs")

    def forward(self, h: torch.Tensor, on_output=None) -> torch.Tensor:
        """One pass over all layers.  on_output(layer, name, full_output, prepare): hook for verification - `prepare(s)`
        re-runs this group's producer into another scratch `s`."""
        capi = self._capi
        m, hid = self.m, self.hidden
        wa = self.wait_in_consumer

        def seen(name, buf):      # the hook reads the buffer with ordinary kernels: everything must have arrived
            if on_output:
                if wa:
                    capi.wait_arrival(buf, self.p2p.status)
                return True
            return False

        def keep(t):              # the hook's `prepare` re-reads a producer's input after the buffer has been refilled
            return t.clone() if (on_output and wa) else t

        for li, layer in enumerate(self.w):
            W, qt, n, k = layer["qkv"]
            prep = lambda s, n_=n, qt_=qt, h_=keep(h): capi.prepare_q8_rmsnorm(h_, self.gamma, self.eps, qt_, n_, s)   # noqa: E731
            capi.prepare_q8_rmsnorm(h, self.gamma, self.eps, qt, n // self.world, self.scratch, wait_arrival=wa and li > 0)
            qkv = self._project("qkv", W, qt, n, k)
            if seen("qkv", qkv): on_output(li, "qkv", qkv, prep)
            W, qt, n, k = layer["o"]
            a = qkv[:, :hid]                                   # stands in for the attention output: [M, hidden], row stride 8192
            prep = lambda s, n_=n, qt_=qt, a_=keep(a): capi.prepare_q8(a_, qt_, n_, s)   # noqa: E731
            capi.prepare_q8(a, qt, n // self.world, self.scratch, wait_arrival=wa)
            o = self._project("o", W, qt, n, k)
            if seen("o", o): on_output(li, "o", o, prep)
            W, qt, n, k = layer["gate_up"]
            prep = lambda s, n_=n, qt_=qt, o_=keep(o): capi.prepare_q8_rmsnorm(o_, self.gamma, self.eps, qt_, n_, s)   # noqa: E731
            capi.prepare_q8_rmsnorm(o, self.gamma, self.eps, qt, n // self.world, self.scratch, wait_arrival=wa)
            gu = self._project("gate_up", W, qt, n, k)
            if seen("gate_up", gu): on_output(li, "gate_up", gu, prep)
            W, qt, n, k = layer["down"]
            prep = lambda s, n_=n, qt_=qt, gu_=keep(gu): capi.prepare_q8_swiglu(gu_, qt_, n_, s)   # noqa: E731
            capi.prepare_q8_swiglu(gu, qt, n // self.world, self.scratch, wait_arrival=wa)
            h = self._project("down", W, qt, n, k)
            if seen("down", h): on_output(li, "down", h, prep)
        if wa:
            capi.wait_arrival(h, self.p2p.status)      # the caller reads h with kernels that do not poll
        return h
