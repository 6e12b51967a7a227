"""ctypes binding of libkq's C ABI (include/kq_gguf.h).

The wrappers take torch tensors only to obtain device pointers, strides and the current stream; every
call goes through the `extern "C"` entry points, so tests and benchmarks that use this module exercise
exactly what a cgo/JNI/ctypes host of the reference would bind.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libkq.so")

KQ_OK, KQ_EINVAL, KQ_EUNSUPPORTED, KQ_ESCRATCH, KQ_ECUDA, KQ_ELIMIT = 0, 1, 2, 3, 4, 5
KQ_F32, KQ_F16, KQ_BF16 = 0, 1, 2
_DT = {torch.float32: KQ_F32, torch.float16: KQ_F16, torch.bfloat16: KQ_BF16}

EXPORTS = (
    "kq_last_error", "kq_abi_version", "kq_block_geometry", "kq_workspace_bytes", "kq_quantize_q8_1",
    "kq_mul_mat_vec_a8", "kq_mul_mat_a8", "kq_dequantize", "kq_debug_group_dots", "kq_set_option",
    "kq_get_option", "kq_prepare_q8", "kq_mul_mat_prepared", "kq_read_status", "kq_mul_mat_vec_a8_static",
    "kq_p2p_allgather", "kq_read_status_static", "kq_debug_copy_window", "kq_prepare_q8_rmsnorm", "kq_prepare_q8_swiglu",
    "kq_p2p_allgather_2d", "kq_mul_mat_prepared_gather", "kq_moe_a8_vec", "kq_moe_a8", "kq_moe_block_size", "kq_dequantize_rows", "kq_wait_arrival", "kq_arrival_status",
)


class KqError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"libkq error {code}: {msg}")
        self.code = code


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m kaillm_b200._build` "
            "(there is no CPU fallback for the GGUF kernels)")
    lib = ctypes.CDLL(LIB_PATH)
    vp, i32, i64, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t
    lib.kq_last_error.restype = ctypes.c_char_p
    lib.kq_last_error.argtypes = []
    lib.kq_abi_version.restype = i32
    lib.kq_block_geometry.argtypes = [i32, ctypes.POINTER(i32), ctypes.POINTER(i32)]
    lib.kq_workspace_bytes.restype = sz
    lib.kq_workspace_bytes.argtypes = [i32, i64, i64, i64]
    lib.kq_quantize_q8_1.argtypes = [vp, i32, i64, i64, i64, vp, vp]
    mm = [vp, i32, i64, i64, vp, i32, i64, i64, vp, i32, i64, vp, sz, vp]
    lib.kq_mul_mat_vec_a8.argtypes = mm
    lib.kq_mul_mat_a8.argtypes = mm
    lib.kq_prepare_q8.argtypes = [i32, i64, i64, vp, i32, i64, i64, vp, sz, i32, vp]
    lib.kq_prepare_q8_rmsnorm.argtypes = [i32, i64, i64, vp, i32, i64, i64, vp, ctypes.c_float, vp, vp, sz, i32, vp]
    lib.kq_prepare_q8_swiglu.argtypes = [i32, i64, i64, vp, i32, i64, i64, vp, sz, i32, vp]
    lib.kq_wait_arrival.argtypes = [vp, sz, i32, vp, vp]
    lib.kq_arrival_status.argtypes = [ctypes.POINTER(i32), i32]
    lib.kq_mul_mat_prepared.argtypes = [vp, i32, i64, i64, i64, vp, i32, i64, i32, vp, sz, vp]
    lib.kq_mul_mat_vec_a8_static.argtypes = [vp, i32, i64, i64, vp, i32, i64, i64, vp, i32, i64, vp]
    lib.kq_dequantize.argtypes = [vp, i32, i64, vp, i32, vp]
    lib.kq_read_status.argtypes = [i32, i64, i64, i64, vp, sz, ctypes.POINTER(i32)]
    lib.kq_debug_group_dots.argtypes = [vp, i32, i64, i64, vp, i32, i64, i64, vp, vp, vp, sz, vp]
    lib.kq_p2p_allgather.argtypes = [vp, sz, ctypes.POINTER(vp), ctypes.POINTER(vp), vp, vp, i32, i32, i32, vp, vp]
    lib.kq_read_status_static.argtypes = [ctypes.POINTER(i32)]
    u64p = ctypes.POINTER(ctypes.c_uint64)
    lib.kq_debug_copy_window.argtypes = [ctypes.c_uint64, i64, i64, i64, i64, i64, i64, ctypes.POINTER(i64), u64p, u64p]
    lib.kq_p2p_allgather_2d.argtypes = [vp, i64, sz, ctypes.POINTER(vp), sz, ctypes.POINTER(vp), vp, vp, i32, i32, i32, vp, vp]
    lib.kq_mul_mat_prepared_gather.argtypes = [vp, i32, i64, i64, i64, i32, i32, vp, sz, ctypes.POINTER(vp), i64,
                                               ctypes.POINTER(vp), vp, vp, i32, i32, i32, vp, i32, vp, sz, ctypes.POINTER(i32), vp]
    lib.kq_moe_a8_vec.argtypes = [vp, i32, i64, i64, i64, vp, i32, i64, i64, vp, i32, vp, i32, i64, vp, sz, vp]
    lib.kq_moe_a8.argtypes = [vp, i32, i64, i64, i64, vp, i32, i64, i64, vp, i64, vp, vp, i32, vp, i32, i64, vp, sz, vp]
    lib.kq_moe_block_size.argtypes = [i32]
    lib.kq_dequantize_rows.argtypes = [vp, i32, i64, i64, vp, i64, vp, i32, i32, vp]
    lib.kq_set_option.argtypes = [ctypes.c_char_p, i32]
    lib.kq_get_option.argtypes = [ctypes.c_char_p, ctypes.POINTER(i32)]
    return lib


lib = _load()


def _check(rc: int) -> None:
    if rc != KQ_OK:
        raise KqError(rc, lib.kq_last_error().decode())


def _stream(dev) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def block_geometry(qtype: int) -> tuple[int, int]:
    a, b = ctypes.c_int(), ctypes.c_int()
    _check(lib.kq_block_geometry(qtype, ctypes.byref(a), ctypes.byref(b)))
    return a.value, b.value


def workspace_bytes(qtype: int, m: int, n: int, k: int) -> int:
    return int(lib.kq_workspace_bytes(qtype, m, n, k))


def set_option(name: str, value: int) -> None:
    _check(lib.kq_set_option(name.encode(), value))


def get_option(name: str) -> int:
    v = ctypes.c_int()
    _check(lib.kq_get_option(name.encode(), ctypes.byref(v)))
    return v.value


def quantize_q8_1(x: torch.Tensor) -> torch.Tensor:
    """x [m,k] -> uint8 [m, kpad/32, 36] in the reference's block_q8_1 layout."""
    m, k = x.shape
    kpad = (k + 511) // 512 * 512
    out = torch.empty((m, kpad // 32, 36), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _check(lib.kq_quantize_q8_1(x.data_ptr(), _DT[x.dtype], m, k, x.stride(0), out.data_ptr(), _stream(x.device)))
    return out


def _k_of(W: torch.Tensor, qtype: int) -> int:
    blk, nb = block_geometry(qtype)
    return W.shape[1] // nb * blk


def mul_mat(W: torch.Tensor, x: torch.Tensor, qtype: int, *, mmq: bool = False, out_dtype=None,
            out: torch.Tensor | None = None, scratch: torch.Tensor | None = None, n: int | None = None) -> torch.Tensor:
    """y[m,n] through kq_mul_mat_vec_a8 (mmq=False) or kq_mul_mat_a8 (mmq=True)."""
    m, k = x.shape
    n = W.shape[0] if n is None else n
    odt = out_dtype or x.dtype
    if out is None:
        out = torch.empty((m, n), dtype=odt, device=x.device)
    ws = workspace_bytes(qtype, m, n, k)
    if scratch is None:
        scratch = torch.empty(ws, dtype=torch.uint8, device=x.device)
    fn = lib.kq_mul_mat_a8 if mmq else lib.kq_mul_mat_vec_a8
    with torch.cuda.device(x.device):
        _check(fn(W.data_ptr(), qtype, n, k, x.data_ptr(), _DT[x.dtype], m, x.stride(0), out.data_ptr(),
                  _DT[out.dtype], out.stride(0), scratch.data_ptr(), scratch.numel(), _stream(x.device)))
    return out


def prepare_q8(x: torch.Tensor, qtype: int, n: int, scratch: torch.Tensor, wait_arrival: bool = False) -> None:
    """Quantize x [m,k] into `scratch` (kq_prepare_q8).  wait_arrival: x is a gather buffer still being filled by the
    peers; every element is polled against the arrival sentinel (KQ_PREP_WAIT_ARRIVAL)."""
    m, k = x.shape
    with torch.cuda.device(x.device):
        _check(lib.kq_prepare_q8(qtype, n, k, x.data_ptr(), _DT[x.dtype], m, x.stride(0), scratch.data_ptr(),
                                 scratch.numel(), int(wait_arrival), _stream(x.device)))


def prepare_q8_rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float, qtype: int, n: int, scratch: torch.Tensor,
                       y_norm: torch.Tensor | None = None, wait_arrival: bool = False) -> None:
    """RMSNorm(x) * gamma quantized into `scratch` in one launch (kq_prepare_q8_rmsnorm)."""
    m, k = x.shape
    with torch.cuda.device(x.device):
        _check(lib.kq_prepare_q8_rmsnorm(qtype, n, k, x.data_ptr(), _DT[x.dtype], m, x.stride(0), gamma.data_ptr(), eps,
                                         y_norm.data_ptr() if y_norm is not None else None, scratch.data_ptr(),
                                         scratch.numel(), int(wait_arrival), _stream(x.device)))


def prepare_q8_swiglu(gate_up: torch.Tensor, qtype: int, n: int, scratch: torch.Tensor, wait_arrival: bool = False) -> None:
    """silu(gate) * up of a merged [m, 2k] gate/up output quantized into `scratch` in one launch (kq_prepare_q8_swiglu)."""
    m, k2 = gate_up.shape
    with torch.cuda.device(gate_up.device):
        _check(lib.kq_prepare_q8_swiglu(qtype, n, k2 // 2, gate_up.data_ptr(), _DT[gate_up.dtype], m, gate_up.stride(0),
                                        scratch.data_ptr(), scratch.numel(), int(wait_arrival), _stream(gate_up.device)))


def mul_mat_prepared(W: torch.Tensor, qtype: int, m: int, k: int, out: torch.Tensor, scratch: torch.Tensor,
                     *, mmq: bool = False) -> torch.Tensor:
    """y = activations held in `scratch` times W (kq_mul_mat_prepared)."""
    n = W.shape[0]
    with torch.cuda.device(W.device):
        _check(lib.kq_mul_mat_prepared(W.data_ptr(), qtype, n, k, m, out.data_ptr(), _DT[out.dtype], out.stride(0),
                                       int(mmq), scratch.data_ptr(), scratch.numel(), _stream(W.device)))
    return out


def read_status(qtype: int, m: int, n: int, k: int, scratch: torch.Tensor) -> int:
    """Device-side status word of a scratch buffer (synchronises)."""
    v = ctypes.c_int()
    with torch.cuda.device(scratch.device):
        _check(lib.kq_read_status(qtype, m, n, k, scratch.data_ptr(), scratch.numel(), ctypes.byref(v)))
    return v.value


def read_status_static() -> int:
    """Status word of the library-owned scratch array of the current device (synchronises)."""
    v = ctypes.c_int()
    _check(lib.kq_read_status_static(ctypes.byref(v)))
    return v.value


def copy_window(base: int, n: int, rowbytes: int, row_a: int, row_b: int, seg_off: int = 0, seg_len: int = 0):
    """(streamed_rows, bulk_start, bulk_bytes) of the streaming kernels for these rows (host arithmetic only)."""
    ns, a, b = ctypes.c_int64(), ctypes.c_uint64(), ctypes.c_uint64()
    _check(lib.kq_debug_copy_window(base, n, rowbytes, row_a, row_b, seg_off, seg_len, ctypes.byref(ns), ctypes.byref(a),
                                    ctypes.byref(b)))
    return ns.value, a.value, b.value


def mul_mat_vec_static(W: torch.Tensor, x: torch.Tensor, qtype: int, out: torch.Tensor) -> torch.Tensor:
    """kq_mul_mat_vec_a8_static: the scratch-free entry point (library-owned device array; m<=16, n,k<=32768).

    `out` must be preallocated by the caller, so the call itself allocates nothing on the device."""
    m, k = x.shape
    n = W.shape[0]
    with torch.cuda.device(x.device):
        _check(lib.kq_mul_mat_vec_a8_static(W.data_ptr(), qtype, n, k, x.data_ptr(), _DT[x.dtype], m, x.stride(0),
                                            out.data_ptr(), _DT[out.dtype], out.stride(0), _stream(x.device)))
    return out


def p2p_allgather(src: torch.Tensor, peer_dst: list[int], peer_flags: list[int], epoch: torch.Tensor,
                  done: torch.Tensor, slot: int, rank: int, status: torch.Tensor) -> None:
    """kq_p2p_allgather: push `src` (contiguous) into slot `rank` of every rank's gather buffer and wait for the peers.

    peer_dst / peer_flags are device addresses (ints) valid in this process, one per rank."""
    world = len(peer_dst)
    dst = (ctypes.c_void_p * world)(*peer_dst)
    flg = (ctypes.c_void_p * world)(*peer_flags)
    with torch.cuda.device(src.device):
        _check(lib.kq_p2p_allgather(src.data_ptr(), src.numel() * src.element_size(), dst, flg, epoch.data_ptr(),
                                    done.data_ptr(), slot, rank, world, status.data_ptr(), _stream(src.device)))


def p2p_allgather_2d(src: torch.Tensor, peer_dst: list[int], dst_row_stride: int, peer_flags: list[int], epoch: torch.Tensor,
                     done: torch.Tensor, slot: int, rank: int, status: torch.Tensor) -> None:
    """kq_p2p_allgather_2d: `src` [M, N/world] (contiguous) becomes columns rank*N/world.. of every rank's row-major
    [M, N] buffer (rows `dst_row_stride` bytes apart)."""
    world = len(peer_dst)
    dst = (ctypes.c_void_p * world)(*peer_dst)
    flg = (ctypes.c_void_p * world)(*peer_flags)
    rows, per = src.shape
    with torch.cuda.device(src.device):
        _check(lib.kq_p2p_allgather_2d(src.data_ptr(), rows, per * src.element_size(), dst, dst_row_stride, flg,
                                       epoch.data_ptr(), done.data_ptr(), slot, rank, world, status.data_ptr(),
                                       _stream(src.device)))


def mul_mat_prepared_gather(W: torch.Tensor, qtype: int, m: int, k: int, scratch: torch.Tensor, peer_y: list[int],
                            stride_y: int, dtype, peer_flags: list[int], epoch: torch.Tensor, done: torch.Tensor,
                            slot: int, rank: int, status: torch.Tensor, mmq: bool = False, wait_in_consumer: bool = False,
                            reset_ptr: int = 0, reset_bytes: int = 0) -> bool:
    """kq_mul_mat_prepared_gather: this rank's weight slice `W` [N/world, row bytes] times the activations prepared in
    `scratch`, written as columns rank*N/world.. of every rank's row-major buffer (`peer_y`: device addresses, rows
    `stride_y` elements apart).  Returns True when GEMV and gather ran as one kernel."""
    world = len(peer_y)
    ys = (ctypes.c_void_p * world)(*peer_y)
    flg = (ctypes.c_void_p * world)(*peer_flags)
    fused = ctypes.c_int(0)
    with torch.cuda.device(W.device):
        _check(lib.kq_mul_mat_prepared_gather(W.data_ptr(), qtype, W.shape[0], k, m, _DT[dtype], int(mmq), scratch.data_ptr(),
                                              scratch.numel(), ys, stride_y, flg, epoch.data_ptr(), done.data_ptr(), slot,
                                              rank, world, status.data_ptr(), int(wait_in_consumer), reset_ptr or None, reset_bytes,
                                              ctypes.byref(fused), _stream(W.device)))
    return bool(fused.value)


def moe_a8_vec(W: torch.Tensor, x: torch.Tensor, topk_ids: torch.Tensor, qtype: int, out_dtype=None) -> torch.Tensor:
    """kq_moe_a8_vec: W [E, n, row bytes], x [tokens, k], topk_ids int32 [tokens, top_k] -> [tokens * top_k, n]."""
    experts, n = W.shape[0], W.shape[1]
    tokens, k = x.shape
    top_k = topk_ids.shape[1]
    y = torch.zeros((tokens * top_k, n), dtype=out_dtype or x.dtype, device=x.device)
    scratch = torch.empty(max(1, workspace_bytes(qtype, tokens, n, k)), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _check(lib.kq_moe_a8_vec(W.data_ptr(), qtype, experts, n, k, x.data_ptr(), _DT[x.dtype], tokens, x.stride(0),
                                 topk_ids.data_ptr(), top_k, y.data_ptr(), _DT[y.dtype], y.stride(0), scratch.data_ptr(),
                                 scratch.numel(), _stream(x.device)))
    return y


def moe_a8(W: torch.Tensor, x: torch.Tensor, sorted_token_ids: torch.Tensor, expert_ids: torch.Tensor,
           num_tokens_post_padded: torch.Tensor, top_k: int, qtype: int, out_dtype=None) -> torch.Tensor:
    """kq_moe_a8: expert-sorted blocks of kq_moe_block_size slots -> [tokens * top_k, n] (rows nobody writes stay zero)."""
    experts, n = W.shape[0], W.shape[1]
    tokens, k = x.shape
    y = torch.zeros((tokens * top_k, n), dtype=out_dtype or x.dtype, device=x.device)
    scratch = torch.empty(max(1, workspace_bytes(qtype, tokens, n, k)), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _check(lib.kq_moe_a8(W.data_ptr(), qtype, experts, n, k, x.data_ptr(), _DT[x.dtype], tokens, x.stride(0),
                             sorted_token_ids.data_ptr(), sorted_token_ids.numel(), expert_ids.data_ptr(),
                             num_tokens_post_padded.data_ptr(), top_k, y.data_ptr(), _DT[y.dtype], y.stride(0),
                             scratch.data_ptr(), scratch.numel(), _stream(x.device)))
    return y


def wait_arrival(buf: torch.Tensor, status: torch.Tensor) -> None:
    """kq_wait_arrival: on the current stream, until no element of the (contiguous) gather buffer holds the sentinel."""
    with torch.cuda.device(buf.device):
        _check(lib.kq_wait_arrival(buf.data_ptr(), buf.numel() * buf.element_size(), _DT[buf.dtype], status.data_ptr(),
                                   _stream(buf.device)))


def arrival_status(clear: bool = False) -> int:
    """kq_arrival_status on the current device (synchronises): non-zero when an arrival poll has run out."""
    v = ctypes.c_int()
    _check(lib.kq_arrival_status(ctypes.byref(v), int(clear)))
    return v.value


def dequantize(W: torch.Tensor, qtype: int, count: int, dtype=torch.float16) -> torch.Tensor:
    out = torch.empty(count, dtype=dtype, device=W.device)
    with torch.cuda.device(W.device):
        _check(lib.kq_dequantize(W.data_ptr(), qtype, count, out.data_ptr(), _DT[dtype], _stream(W.device)))
    return out


def dequantize_rows(W: torch.Tensor, qtype: int, k: int, row_ids: torch.Tensor, dtype=torch.float16,
                    f32_math: bool = False) -> torch.Tensor:
    """kq_dequantize_rows: rows `row_ids` (int64, any shape) of the [n, row bytes] wire tensor W -> [*row_ids.shape, k]."""
    ids = row_ids.reshape(-1).to(torch.int64).contiguous()
    out = torch.empty((ids.numel(), k), dtype=dtype, device=W.device)
    with torch.cuda.device(W.device):
        _check(lib.kq_dequantize_rows(W.data_ptr(), qtype, W.shape[0], k, ids.data_ptr(), ids.numel(), out.data_ptr(),
                                      _DT[dtype], int(f32_math), _stream(W.device)))
    return out.view(*row_ids.shape, k)


def debug_group_dots(W: torch.Tensor, x: torch.Tensor, qtype: int):
    m, k = x.shape
    n = W.shape[0]
    g = 16 if qtype in (10, 11, 14) else 32
    dots = torch.empty((m, n, k // g), dtype=torch.int32, device=x.device)
    sums = torch.empty((m, k // g), dtype=torch.int32, device=x.device)
    ws = workspace_bytes(qtype, m, n, k)
    scratch = torch.empty(ws, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _check(lib.kq_debug_group_dots(W.data_ptr(), qtype, n, k, x.data_ptr(), _DT[x.dtype], m, x.stride(0),
                                       dots.data_ptr(), sums.data_ptr(), scratch.data_ptr(), scratch.numel(),
                                       _stream(x.device)))
    return dots, sums
