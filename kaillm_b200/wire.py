"""Load path: GGUF file -> device wire tensors the kernels stream.

What the reference does between its GGUF reader and the linear method's parameters:

* gguf-reader maps the file and hands out every tensor as uint8 rows in wire format (gguf-reader/gguf/gguf_reader.py:116-360);
* the weight loader keeps a rank's dim-0 slice of column-parallel layers (quantization/params.py:230-247) and stacks the
  shards of merged layers (quantization/linear.py:290-339);
* `align_native_wire` gives the rows a 128-byte aligned base and an owned, zeroed tail (quantization/native_wire.py:7-61).

Here: a small reader of the GGUF container (`GGUFFile`; format versions 2 and 3, little endian), `load_wire` (only the
rank's rows leave the file, through pinned memory), `align_wire` (aligned base + zeroed tail of the allocation, so a
bulk-copy window rounded up to 16 bytes stays inside memory this tensor owns) and `merge_wire` for same-type merged
layers.  A writer for the same container (`write_gguf`) exists for tests and synthetic checkpoints.  Pure Python, numpy
and torch; no kernel is involved.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass

import numpy as np
import torch

from .synth import BLOCK

GGUF_MAGIC = 0x46554747            # "GGUF"
DEFAULT_ALIGNMENT = 32
WIRE_ALIGN = 128                   # base alignment of a device wire tensor
TAIL_BYTES = 16                    # owned zero bytes after the last row (one bulk-copy unit)

# element sizes of the unquantized ggml types (type id -> (elements per block, bytes per block))
PLAIN = {0: (1, 4), 1: (1, 2), 30: (1, 2), 24: (1, 1), 25: (1, 2), 26: (1, 4), 27: (1, 8), 28: (1, 8)}

_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_T_STRING, _T_ARRAY = 8, 9


def type_geometry(qtype: int) -> tuple[int, int]:
    """(weights per block, bytes per block) of a ggml type id."""
    if qtype in BLOCK:
        return BLOCK[qtype]
    if qtype in PLAIN:
        return PLAIN[qtype]
    raise NotImplementedError(f"ggml type {qtype} is not known to this loader")


@dataclass
class TensorInfo:
    name: str
    shape: tuple[int, ...]          # torch order: (rows, ..., k); the file stores the dimensions innermost first
    qtype: int
    offset: int                     # from the start of the file
    nbytes: int

    @property
    def k(self) -> int:
        return self.shape[-1]

    @property
    def rows(self) -> int:
        return int(np.prod(self.shape[:-1])) if len(self.shape) > 1 else 1

    @property
    def row_bytes(self) -> int:
        blk, size = type_geometry(self.qtype)
        return self.k // blk * size


class GGUFFile:
    """Metadata and tensor directory of a GGUF file; tensor bytes are mapped, not read, until asked for."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._pos = 0
        magic, self.version = self._unpack("<II")
        if magic != GGUF_MAGIC:
            raise ValueError(f"{path}: not a GGUF file (magic {magic:#x})")
        if self.version not in (2, 3):
            raise ValueError(f"{path}: GGUF version {self.version} is not supported (2 and 3 are)")
        n_tensors, n_kv = self._unpack("<QQ")
        self.metadata: dict[str, object] = {}
        for _ in range(n_kv):
            key = self._string()
            (vtype,) = self._unpack("<I")
            self.metadata[key] = self._value(vtype)
        self.alignment = int(self.metadata.get("general.alignment", DEFAULT_ALIGNMENT))
        infos = []
        for _ in range(n_tensors):
            name = self._string()
            (nd,) = self._unpack("<I")
            dims = self._unpack("<" + "Q" * nd)
            qtype, off = self._unpack("<IQ")
            infos.append((name, tuple(int(d) for d in reversed(dims)), int(qtype), int(off)))
        self.data_offset = (self._pos + self.alignment - 1) // self.alignment * self.alignment
        self.tensors: dict[str, TensorInfo] = {}
        for name, shape, qtype, off in infos:
            blk, size = type_geometry(qtype)
            if shape[-1] % blk:
                raise ValueError(f"{name}: innermost dimension {shape[-1]} is not a multiple of the block size {blk}")
            nbytes = int(np.prod(shape)) // blk * size
            if self.data_offset + off + nbytes > len(self._mm):
                raise ValueError(f"{name}: tensor data runs past the end of the file")
            self.tensors[name] = TensorInfo(name, shape, qtype, self.data_offset + off, nbytes)

    # ---- parsing helpers
    def _unpack(self, fmt: str):
        size = struct.calcsize(fmt)
        out = struct.unpack_from(fmt, self._mm, self._pos)
        self._pos += size
        return out

    def _string(self) -> str:
        (n,) = self._unpack("<Q")
        s = self._mm[self._pos:self._pos + n].decode("utf-8", errors="replace")
        self._pos += n
        return s

    def _value(self, vtype: int):
        if vtype in _SCALARS:
            return self._unpack(_SCALARS[vtype])[0]
        if vtype == _T_STRING:
            return self._string()
        if vtype == _T_ARRAY:
            etype, n = self._unpack("<IQ")
            return [self._value(etype) for _ in range(n)]
        raise ValueError(f"unknown GGUF metadata value type {vtype}")

    # ---- tensor access
    def rows(self, name: str, row_a: int = 0, row_b: int | None = None) -> np.ndarray:
        """Rows [row_a, row_b) of a tensor as a uint8 view [rows, row bytes] of the mapping (no copy)."""
        t = self.tensors[name]
        row_b = t.rows if row_b is None else row_b
        if not 0 <= row_a <= row_b <= t.rows:
            raise ValueError(f"{name}: rows [{row_a}, {row_b}) outside [0, {t.rows})")
        rb = t.row_bytes
        buf = np.frombuffer(self._mm, dtype=np.uint8, count=(row_b - row_a) * rb, offset=t.offset + row_a * rb)
        return buf.reshape(row_b - row_a, rb)

    def close(self) -> None:
        try:
            self._mm.close()
        except BufferError:      # views handed out by rows() are still alive: the mapping goes when they do
            pass
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def shard_range(rows: int, rank: int, world: int) -> tuple[int, int]:
    """The rank's dim-0 slice of a column-parallel layer (quantization/params.py:230-247)."""
    if rows % world:
        raise ValueError(f"{rows} rows do not divide over {world} ranks")
    per = rows // world
    return rank * per, (rank + 1) * per


def align_wire(data: torch.Tensor, qtype: int, k: int) -> tuple[torch.Tensor, dict]:
    """A uint8 row matrix whose base is 128-byte aligned and whose storage continues, zeroed, for at least TAIL_BYTES
    bytes after the last row; `data` itself when it already is (then no copy).  Returns (tensor, report) with the
    reference's report keys (quantization/native_wire.py:19-26, 50-60)."""
    if data.ndim != 2 or data.dtype != torch.uint8:
        raise ValueError("wire alignment wants a uint8 row matrix")
    blk, size = type_geometry(qtype)
    n, row_bytes = (int(v) for v in data.shape)
    if row_bytes != k // blk * size:
        raise ValueError("wire width differs from K / type")
    logical = n * row_bytes
    info = {"copy_performed": False, "extra_resident_quant_bytes": 0, "logical_wire_bytes": logical,
            "original_GPU_input_pointer_reused": True, "logical_values_preserved": True, "additional_dense_weight_bytes": 0}
    store = data.untyped_storage()
    after = store.nbytes() - (data.storage_offset() + logical) if data.is_contiguous() else -1
    if data.is_contiguous() and data.data_ptr() % WIRE_ALIGN == 0 and logical % 16 == 0 and after >= 0:
        return data, info
    need = logical + TAIL_BYTES + (-logical) % 16
    storage = torch.zeros(need + WIRE_ALIGN - 1, dtype=torch.uint8, device=data.device)
    off = (-storage.data_ptr()) % WIRE_ALIGN
    out = storage[off:off + logical].view(n, row_bytes)
    out.copy_(data)
    info.update(copy_performed=True, original_GPU_input_pointer_reused=False, extra_resident_quant_bytes=storage.numel() - logical,
                allocation_quant_bytes=storage.numel(), alignment_reserve_quant_bytes=WIRE_ALIGN - 1,
                tail_owned_and_zero_initialized=True)
    return out, info


def load_wire(gguf: GGUFFile, name: str, device, rank: int = 0, world: int = 1) -> tuple[torch.Tensor, int, tuple[int, int]]:
    """The rank's rows of tensor `name` as an aligned device wire tensor: (uint8 [rows, row bytes], ggml type, (rows, k)).
    Only those rows are read from the file; they go through pinned memory when the target is a CUDA device."""
    t = gguf.tensors[name]
    a, b = shard_range(t.rows, rank, world)
    host = torch.from_numpy(np.array(gguf.rows(name, a, b)))      # the one copy out of the file mapping
    device = torch.device(device)
    if device.type == "cuda":
        host = host.pin_memory()
    wire, _ = align_wire(host.to(device, non_blocking=True), t.qtype, t.k)
    if device.type == "cuda":
        torch.cuda.current_stream(device).synchronize()      # the pinned staging buffer is dropped on return
    return wire, t.qtype, (b - a, t.k)


def merge_wire(shards: list[tuple[torch.Tensor, int]]) -> tuple[torch.Tensor, int] | None:
    """The shards of a merged layer (q/k/v, gate/up) as ONE wire tensor when their types agree - the layout the
    reference runs as a single call (quantization/linear.py:377-381); None for mixed types (they run per shard)."""
    types = {t for _, t in shards}
    if len(types) != 1:
        return None
    qtype = next(iter(types))
    cat = torch.cat([w for w, _ in shards], dim=0)
    blk, size = type_geometry(qtype)
    merged, _ = align_wire(cat, qtype, cat.shape[1] // size * blk)
    return merged, qtype


# ---------------------------------------------------------------------------------------------- writer (tests, synthetic checkpoints)
def _w_string(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _w_value(v) -> bytes:
    if isinstance(v, bool):
        return struct.pack("<I?", 7, v)
    if isinstance(v, int):
        return struct.pack("<Iq", 11, v) if v < 0 else struct.pack("<II", 4, v) if v < 2 ** 32 else struct.pack("<IQ", 10, v)
    if isinstance(v, float):
        return struct.pack("<If", 6, v)
    if isinstance(v, str):
        return struct.pack("<I", _T_STRING) + _w_string(v)
    if isinstance(v, (list, tuple)):
        if not v:
            return struct.pack("<IIQ", _T_ARRAY, 4, 0)
        first = _w_value(v[0])
        etype = struct.unpack_from("<I", first)[0]
        body = b"".join(_w_value(e)[4:] for e in v)
        return struct.pack("<IIQ", _T_ARRAY, etype, len(v)) + body
    raise TypeError(f"cannot store {type(v).__name__} as GGUF metadata")


def write_gguf(path: str, tensors: dict[str, tuple[np.ndarray, int, tuple[int, ...]]], metadata: dict | None = None,
               alignment: int = DEFAULT_ALIGNMENT) -> None:
    """tensors: name -> (uint8 bytes in wire format, ggml type, shape in torch order)."""
    metadata = dict(metadata or {})
    metadata.setdefault("general.alignment", alignment)
    head = struct.pack("<IIQQ", GGUF_MAGIC, 3, len(tensors), len(metadata))
    for k, v in metadata.items():
        head += _w_string(k) + _w_value(v)
    off = 0
    blobs = []
    for name, (data, qtype, shape) in tensors.items():
        raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        blk, size = type_geometry(qtype)
        if raw.size != int(np.prod(shape)) // blk * size:
            raise ValueError(f"{name}: {raw.size} bytes do not match shape {shape} of type {qtype}")
        head += _w_string(name) + struct.pack("<I", len(shape)) + struct.pack("<" + "Q" * len(shape), *reversed(shape))
        head += struct.pack("<IQ", qtype, off)
        blobs.append((off, raw))
        off = (off + raw.size + alignment - 1) // alignment * alignment
    start = (len(head) + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * (start - len(head)))
        for o, raw in blobs:
            f.seek(start + o)
            f.write(raw.tobytes())
        f.truncate(start + off)
