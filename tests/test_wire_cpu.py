"""Load path on CPU: the GGUF container reader/writer against the reference's gguf-reader package (when it is at hand),
rank slices, aligned wire tensors with an owned zero tail, merged layers."""
import os
import sys

import numpy as np
import pytest
import torch

from kaillm_b200 import synth, wire

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference_gguf():
    """The reference's gguf-reader package: from the reference tree, else from the staged copy; None when neither is there."""
    from oracle.build_ref import reference_root
    for base in (os.path.join(reference_root(), "runtime-source", "gguf-reader"), os.path.join(ROOT, "baseline", "_ref")):
        if os.path.exists(os.path.join(base, "gguf", "gguf_reader.py")):
            if base not in sys.path:
                sys.path.insert(0, base)
            for m in [m for m in sys.modules if m == "gguf" or m.startswith("gguf.")]:
                if not os.path.realpath(getattr(sys.modules[m], "__file__", "") or "").startswith(os.path.realpath(base)):
                    del sys.modules[m]
            import gguf
            if os.path.realpath(gguf.__file__).startswith(os.path.realpath(base)):
                return gguf
    return None


def _tensors():
    out = {}
    for i, (qt, n, k) in enumerate([(12, 48, 512), (14, 33, 256), (8, 10, 64), (2, 7, 96), (21, 16, 256), (13, 4, 1024)]):
        out[f"blk.{i}.w"] = (synth.wire_numpy(qt, n, k, seed=i), qt, (n, k))
    out["norm.weight"] = (np.arange(40, dtype=np.float32).view(np.uint8), 0, (40,))
    out["experts.w"] = (np.stack([synth.wire_numpy(12, 8, 256, seed=30 + e) for e in range(3)]), 12, (3, 8, 256))
    return out


def test_write_then_read_round_trip(tmp_path):
    path = str(tmp_path / "a.gguf")
    ts = _tensors()
    meta = {"general.architecture": "test", "test.count": 7, "test.neg": -3, "test.scale": 0.5, "test.flag": True,
            "test.list": [1, 2, 3], "test.names": ["a", "bc"], "test.big": 2 ** 40}
    wire.write_gguf(path, ts, meta)
    with wire.GGUFFile(path) as g:
        assert g.version == 3 and g.alignment == 32
        for k, v in meta.items():
            assert g.metadata[k] == v, k
        assert list(g.tensors) == list(ts)
        for name, (data, qt, shape) in ts.items():
            t = g.tensors[name]
            assert (t.qtype, t.shape) == (qt, shape) and t.offset % 32 == 0
            got = g.rows(name)
            assert got.shape == (t.rows, t.row_bytes)
            np.testing.assert_array_equal(got.reshape(-1), np.ascontiguousarray(data).view(np.uint8).reshape(-1))
        np.testing.assert_array_equal(g.rows("blk.0.w", 5, 9), ts["blk.0.w"][0][5:9])
        with pytest.raises(ValueError):
            g.rows("blk.0.w", 40, 60)


def test_container_against_the_reference_reader_and_writer(tmp_path):
    gguf = _reference_gguf()
    if gguf is None:
        pytest.skip("the reference's gguf-reader package is not available")
    ts = _tensors()
    mine = str(tmp_path / "mine.gguf")
    wire.write_gguf(mine, ts, {"general.architecture": "test", "test.count": 7})
    r = gguf.GGUFReader(mine)
    assert [t.name for t in r.tensors] == list(ts)
    for t in r.tensors:
        data, qt, shape = ts[t.name]
        assert int(t.tensor_type) == qt and tuple(int(d) for d in reversed(t.shape)) == shape
        np.testing.assert_array_equal(np.asarray(t.data).view(np.uint8).reshape(-1), np.ascontiguousarray(data).view(np.uint8).reshape(-1))
    assert int(r.fields["test.count"].parts[-1][0]) == 7
    # the other direction: a file the reference's writer made, read here
    theirs = str(tmp_path / "theirs.gguf")
    w = gguf.GGUFWriter(theirs, "test")
    w.add_uint32("test.count", 9)
    w.add_string("test.name", "kq")
    for name, (data, qt, shape) in ts.items():
        if qt == 0:
            w.add_tensor(name, np.ascontiguousarray(data).view(np.float32).reshape(shape))
        else:
            rows = np.ascontiguousarray(data).reshape(*shape[:-1], -1)
            w.add_tensor(name, rows, raw_dtype=gguf.GGMLQuantizationType(qt))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    with wire.GGUFFile(theirs) as g:
        assert g.metadata["test.count"] == 9 and g.metadata["test.name"] == "kq" and g.metadata["general.architecture"] == "test"
        for name, (data, qt, shape) in ts.items():
            t = g.tensors[name]
            assert (t.qtype, t.shape) == (qt, shape)
            np.testing.assert_array_equal(g.rows(name).reshape(-1), np.ascontiguousarray(data).view(np.uint8).reshape(-1))


def test_rank_slices_alignment_and_merge(tmp_path):
    path = str(tmp_path / "b.gguf")
    ts = _tensors()
    wire.write_gguf(path, ts)
    with wire.GGUFFile(path) as g:
        full, qt, (n, k) = wire.load_wire(g, "blk.0.w", "cpu")
        assert (qt, n, k) == (12, 48, 512) and full.data_ptr() % 128 == 0
        parts = [wire.load_wire(g, "blk.0.w", "cpu", r, 4)[0] for r in range(4)]
        assert all(p.shape == (12, full.shape[1]) and p.data_ptr() % 128 == 0 for p in parts)
        assert torch.equal(torch.cat(parts), full) and torch.equal(full, torch.from_numpy(ts["blk.0.w"][0]))
        with pytest.raises(ValueError):
            wire.load_wire(g, "blk.1.w", "cpu", 0, 2)            # 33 rows do not divide over 2 ranks
    # an odd-sized tensor (33 rows of 210 bytes): copied once into storage that continues, zeroed, past the last row
    odd = torch.from_numpy(ts["blk.1.w"][0])
    al, info = wire.align_wire(odd[1:], 14, 256)
    assert info["copy_performed"] and info["tail_owned_and_zero_initialized"] and al.data_ptr() % 128 == 0
    assert torch.equal(al, odd[1:])
    st = al.untyped_storage()
    end = al.storage_offset() + al.numel()
    tail = torch.empty(0, dtype=torch.uint8).set_(st)[end:]
    assert tail.numel() >= 16 and not tail.any()
    again, info2 = wire.align_wire(al, 14, 256)
    assert not info2["copy_performed"] or al.numel() % 16 != 0
    with pytest.raises(ValueError):
        wire.align_wire(odd, 12, 256)
    a, b = torch.from_numpy(ts["blk.0.w"][0][:8]), torch.from_numpy(ts["blk.0.w"][0][8:24])
    m = wire.merge_wire([(a, 12), (b, 12)])
    assert m is not None and m[1] == 12 and m[0].data_ptr() % 128 == 0 and torch.equal(m[0], torch.from_numpy(ts["blk.0.w"][0][:24]))
    assert wire.merge_wire([(a, 12), (odd, 14)]) is None
