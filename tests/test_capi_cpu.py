"""CPU-side checks of the C-ABI library: it loads, exports what include/kq_gguf.h declares, and rejects
bad arguments with the documented codes before touching a GPU."""
import ctypes
import os
import re

import pytest

from kaillm_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    txt = open(os.path.join(ROOT, "include", "kq_gguf.h")).read()
    txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
    return sorted(set(re.findall(r"\b(kq_[a-z0-9_]+)\s*\(", txt)))


def test_every_declared_symbol_is_exported():
    names = _declared()
    assert len(names) >= 11
    for n in names:
        assert hasattr(capi.lib, n), n
    assert set(capi.EXPORTS) <= set(names)


def test_header_cites_reference_for_each_compute_entry():
    txt = open(os.path.join(ROOT, "include", "kq_gguf.h")).read()
    for fn in ("kq_quantize_q8_1", "kq_mul_mat_vec_a8", "kq_mul_mat_a8", "kq_dequantize"):
        head = txt[: txt.index(f"int {fn}(")]
        comment = head[head.rindex("/*"):]
        assert "gguf_kernel.cu" in comment, fn


def test_geometry_and_workspace():
    assert capi.lib.kq_abi_version() == 1
    assert capi.block_geometry(2) == (32, 18) and capi.block_geometry(8) == (32, 34)
    assert capi.block_geometry(10) == (256, 84) and capi.block_geometry(12) == (256, 144)
    assert capi.block_geometry(14) == (256, 210) and capi.block_geometry(21) == (256, 110)
    with pytest.raises(capi.KqError) as e:
        capi.block_geometry(16)
    assert e.value.code == capi.KQ_EUNSUPPORTED and "16" in str(e.value)
    assert capi.block_geometry(3) == (32, 20) and capi.block_geometry(6) == (32, 22) and capi.block_geometry(7) == (32, 24)
    assert capi.block_geometry(11) == (256, 110) and capi.block_geometry(13) == (256, 176)
    assert capi.block_geometry(20) == (32, 18) and capi.block_geometry(23) == (256, 136)
    assert capi.workspace_bytes(12, 16, 17408, 5120) >= 16 * 5120 + 16 * 160 * 4
    assert capi.workspace_bytes(16, 1, 1, 256) == 0
    assert capi.workspace_bytes(12, 1, 64, 300) >= 512 + 64     # k padded to 512
    # everything but the last region is independent of n and of the type; Q4_0 above 16 tokens adds its per-call table of
    # -8 * d: fp16 [n][k / 32 rounded up to 128]
    n, k = 4096, 5120
    base = capi.workspace_bytes(8, 32, n, k)
    assert capi.workspace_bytes(12, 32, n, k) == base == capi.workspace_bytes(14, 32, n, k)
    assert capi.workspace_bytes(2, 16, n, k) == capi.workspace_bytes(8, 16, n, k)
    extra = capi.workspace_bytes(2, 32, n, k) - base
    assert n * 256 * 2 <= extra < n * 256 * 2 + 256
    assert capi.workspace_bytes(8, 32, 2 * n, k) > base          # the split-K area grows with n


def _mm(fn, W=0x1000, qt=12, n=8, k=256, x=0x2000, xdt=0, m=1, sx=256, y=0x3000, ydt=0, sy=8, scratch=0x4000, sb=1 << 30):
    return fn(W, qt, n, k, x, xdt, m, sx, y, ydt, sy, scratch, sb, None)


@pytest.mark.parametrize("fn", ["kq_mul_mat_vec_a8", "kq_mul_mat_a8"])
def test_mul_mat_argument_validation(fn):
    f = getattr(capi.lib, fn)
    assert _mm(f, qt=16) == capi.KQ_EUNSUPPORTED
    assert "not supported" in capi.lib.kq_last_error().decode()
    assert _mm(f, k=200, sx=200) == capi.KQ_EINVAL
    assert "multiple of the block" in capi.lib.kq_last_error().decode()
    assert _mm(f, W=0) == capi.KQ_EINVAL
    assert _mm(f, x=0) == capi.KQ_EINVAL
    assert _mm(f, y=0) == capi.KQ_EINVAL
    assert _mm(f, m=0) == capi.KQ_EINVAL
    assert _mm(f, n=0) == capi.KQ_EINVAL
    assert _mm(f, xdt=7) == capi.KQ_EUNSUPPORTED
    assert _mm(f, ydt=7) == capi.KQ_EUNSUPPORTED
    assert _mm(f, sx=100) == capi.KQ_EINVAL
    assert _mm(f, sy=4) == capi.KQ_EINVAL
    assert _mm(f, W=0x1002) == capi.KQ_EINVAL          # Q4_K blocks need 4-byte alignment
    assert _mm(f, scratch=0) == capi.KQ_ESCRATCH
    assert _mm(f, scratch=0x4010) == capi.KQ_ESCRATCH   # not 256-aligned
    assert _mm(f, sb=16) == capi.KQ_ESCRATCH
    assert "scratch too small" in capi.lib.kq_last_error().decode()


def test_imatrix_formats_have_no_mmq():
    for qt in (21, 20, 23):
        assert _mm(capi.lib.kq_mul_mat_a8, qt=qt, k=256, sx=256) == capi.KQ_EUNSUPPORTED
        assert "no MMQ kernel" in capi.lib.kq_last_error().decode()


def test_dequantize_and_quantize_validation():
    d = capi.lib.kq_dequantize
    assert d(0x1000, 12, 100, 0x2000, 1, None) == capi.KQ_EINVAL
    assert d(0x1000, 5, 256, 0x2000, 1, None) == capi.KQ_EUNSUPPORTED
    assert d(0x1000, 12, 256, 0x2000, 9, None) == capi.KQ_EUNSUPPORTED
    assert d(0, 12, 256, 0x2000, 1, None) == capi.KQ_EINVAL
    assert d(0x1000, 12, 0, 0x2000, 1, None) == capi.KQ_OK       # nothing to do
    q = capi.lib.kq_quantize_q8_1
    assert q(0, 0, 1, 32, 32, 0x1000, None) == capi.KQ_EINVAL
    assert q(0x1000, 0, 1, 32, 16, 0x2000, None) == capi.KQ_EINVAL
    assert q(0x1000, 5, 1, 32, 32, 0x2000, None) == capi.KQ_EUNSUPPORTED


def test_options_roundtrip():
    old = capi.get_option("gemv_impl")
    capi.set_option("gemv_impl", 1)
    assert capi.get_option("gemv_impl") == 1
    capi.set_option("gemv_impl", old)
    with pytest.raises(capi.KqError):
        capi.set_option("nope", 1)
    # the defaults of the dispatch options
    for name, want in (("gemm_min_m", 81), ("gemm_small_m", 1), ("gemm_wide", 1), ("row_stage_kb", 24), ("tile_two_stage", 1),
                       ("moe_smem", 1), ("umma", 0), ("no_fused_gather", 0)):
        assert capi.get_option(name) == want, name


def test_error_message_is_thread_local_text():
    capi.lib.kq_block_geometry(99, None, None)
    assert isinstance(capi.lib.kq_last_error(), bytes) and b"99" in capi.lib.kq_last_error()


def test_torch_extension_registers_reference_schemas():
    import torch

    from kaillm_b200 import ops  # noqa: F401

    want = {
        "ggml_dequantize": "_C_gguf::ggml_dequantize(Tensor W, int type, SymInt m, SymInt n, ScalarType? dtype) -> Tensor",
        "ggml_mul_mat_vec_a8": "_C_gguf::ggml_mul_mat_vec_a8(Tensor W, Tensor X, int type, SymInt row) -> Tensor",
        "ggml_mul_mat_a8": "_C_gguf::ggml_mul_mat_a8(Tensor W, Tensor X, int type, SymInt row) -> Tensor",
        "ggml_moe_get_block_size": "_C_gguf::ggml_moe_get_block_size(int type) -> int",
    }
    for name, schema in want.items():
        assert str(getattr(torch.ops._C_gguf, name).default._schema) == schema
    assert hasattr(torch.ops._C_gguf, "ggml_moe_a8") and hasattr(torch.ops._C_gguf, "ggml_moe_a8_vec")


@pytest.mark.parametrize("rowbytes", [18 * 3, 34 * 5, 210 * 20, 110 * 8, 144 * 20, 84 * 7, 210, 22, 136 * 3])
@pytest.mark.parametrize("n", [1, 2, 7, 8, 9, 33])
def test_streaming_kernels_never_read_outside_the_tensor(rowbytes, n):
    """Host arithmetic of the dispatch and of the bulk-copy windows (the kernels call the same functions): the
    streaming kernels get only rows whose total size is a multiple of 16 bytes, at most 7 rows are left to the general
    kernel, and no 16-byte rounded window of whole rows or of row segments leaves [base, base + n * rowbytes)."""
    base = 0x7F0000001000
    end = base + n * rowbytes
    ns, _, _ = capi.copy_window(base, n, rowbytes, 0, 1)
    assert 0 <= n - ns <= 7 and (ns * rowbytes) % 16 == 0
    assert ns == n or ((ns + 1) * rowbytes) % 16 != 0 or ns + 1 > n
    cases = []
    for rows in (1, 2, 8, 16):
        for a in range(0, ns, rows):
            cases.append((a, min(a + rows, ns), 0, 0))
    seg = max(2, (rowbytes // 4) // 2 * 2)
    for r in range(ns):
        for off in range(0, rowbytes, seg):
            cases.append((r, r + 1, off, min(seg, rowbytes - off)))
    for a, b, off, ln in cases:
        _, start, bulk = capi.copy_window(base, n, rowbytes, a, b, off, ln)
        ga = base + a * rowbytes + off
        ge = ga + ln if ln else base + b * rowbytes
        assert start % 16 == 0 and bulk % 16 == 0 and bulk > 0
        assert base <= start <= ga and start + bulk >= ge and start + bulk <= end
    # rows beyond the streamed part have no window
    if ns < n:
        assert capi.copy_window(base, n, rowbytes, ns, n)[1:] == (0, 0)


def test_copy_window_rejects_bad_arguments():
    with pytest.raises(capi.KqError):
        capi.copy_window(4096 + 2, 4, 144, 0, 1)
    with pytest.raises(capi.KqError):
        capi.copy_window(4096, 4, 144, 0, 1, 100, 80)
