"""GPU tests against the reference's own `_C_gguf` extension (built unmodified by oracle/build_ref.py and
loaded as torch.ops._C_gguf_ref): same seeded inputs, same op, both implementations on the same GPU.
Skipped when that library has not been built."""
import numpy as np
import pytest
import torch

from kaillm_b200 import capi, ops  # noqa: F401  (ops registers torch.ops._C_gguf)
from oracle import gguf_oracle as O
from tests.gpu_util import TDT, act, dev, rel_l2, to_np, wire

pytestmark = pytest.mark.gpu
QT = O.QTYPES
GATE = 1e-3
TIGHT = 2e-5


@pytest.mark.parametrize("qt", QT)
@pytest.mark.parametrize("n,k,m", [(64, 512, 1), (136, 2048, 2), (512, 5120, 6), (64, 1024, 16)])
def test_mul_mat_vec_matches_reference_kernels(ref_ops, qt, n, k, m):
    w, wt = wire(qt, n, k, seed=qt)
    x, xt = act(m, k, seed=m, dt="f32")
    ref = to_np(ref_ops.ggml_mul_mat_vec_a8(wt, xt, qt, n))
    mine = to_np(torch.ops._C_gguf.ggml_mul_mat_vec_a8(wt, xt, qt, n))
    assert rel_l2(mine, ref) < TIGHT < GATE
    assert rel_l2(ref, O.mul_mat(w, qt, x, "mmvq")) < TIGHT      # the oracle is pinned by the reference itself


@pytest.mark.parametrize("qt", [2, 8, 10, 12, 14])
@pytest.mark.parametrize("n,k,m", [(64, 512, 3), (160, 2048, 16), (96, 1024, 80), (512, 5120, 8)])
def test_mul_mat_a8_matches_reference_kernels(ref_ops, qt, n, k, m):
    w, wt = wire(qt, n, k, seed=qt + 1)
    x, xt = act(m, k, seed=m + 1, dt="f32")
    ref = to_np(ref_ops.ggml_mul_mat_a8(wt, xt, qt, n))
    mine = to_np(torch.ops._C_gguf.ggml_mul_mat_a8(wt, xt, qt, n))
    assert rel_l2(mine, ref) < TIGHT < GATE
    assert rel_l2(ref, O.mul_mat(w, qt, x, "mmq")) < TIGHT


@pytest.mark.parametrize("qt", [2, 8, 10, 12, 14])
@pytest.mark.parametrize("n,k,m", [(256, 1024, 200), (300, 2048, 130), (7808, 512, 48), (15488, 256, 17)])
def test_prefill_gemm_matches_reference_kernels(ref_ops, qt, n, k, m):
    """More than 80 tokens - and from 17 tokens on matrices with enough 128-row tiles - this library switches to the
    tcgen05 GEMM with fp16 operands; the reference stays on its integer MMQ kernels.  The gate is the path's 1e-3."""
    w, wt = wire(qt, n, k, seed=qt + 5)
    x, xt = act(m, k, seed=m + 5, dt="f32")          # fp32 in, fp32 out: no output rounding in the comparison
    ref = to_np(ref_ops.ggml_mul_mat_a8(wt, xt, qt, n))
    mine = to_np(torch.ops._C_gguf.ggml_mul_mat_a8(wt, xt, qt, n))
    assert mine.shape == ref.shape == (m, n)
    assert rel_l2(mine, ref) < GATE


@pytest.mark.parametrize("qt", QT)
@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_low_precision_io_matches_reference(ref_ops, qt, dt):
    n, k, m = 128, 1024, 2
    _, wt = wire(qt, n, k, seed=3)
    _, xt = act(m, k, seed=3, dt=dt)
    ref = ref_ops.ggml_mul_mat_vec_a8(wt, xt, qt, n)
    mine = torch.ops._C_gguf.ggml_mul_mat_vec_a8(wt, xt, qt, n)
    assert mine.dtype == ref.dtype == TDT[dt]
    assert rel_l2(to_np(mine), to_np(ref)) < GATE
    assert (mine == ref).float().mean() > 0.98


@pytest.mark.parametrize("qt", QT)
@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
def test_dequantize_bit_identical_to_reference(ref_ops, qt, dt):
    n, k = 64, 1024
    w, wt = wire(qt, n, k, seed=qt + 40)
    ref = ref_ops.ggml_dequantize(wt, qt, n, k, TDT[dt])
    mine = torch.ops._C_gguf.ggml_dequantize(wt, qt, n, k, TDT[dt])
    assert torch.equal(mine, ref)
    np.testing.assert_array_equal(to_np(ref), O.dequantize(w, qt, dt, half_fma=capi.get_option("half_fma")))


def _q8_probe_weights(k):
    """Q8_0 weights whose rows read out single activation codes: row i = unit code at column i, d = 1."""
    w = np.zeros((k, k // 32, 34), np.uint8)
    w[:, :, 0:2] = np.array([1.0], np.float16).view(np.uint8)
    for i in range(k):
        w[i, i // 32, 2 + i % 32] = 1
    return w.reshape(k, -1)


def test_q8_1_codes_and_scales_match_reference_through_a_probe(ref_ops):
    """The reference never exposes its q8_1 scratch.  With one-hot Q8_0 rows (d=1) the op returns
    d8*q per activation exactly (fp16 x int8 fits fp32), which pins both the codes and the block scale;
    a Q4_0 row of zero nibbles returns -8*d*s8 and pins the fp16 block sum."""
    k, m = 512, 4
    x, xt = act(m, k, seed=123, dt="f32")
    wq = torch.from_numpy(_q8_probe_weights(k)).to(dev())
    ref = to_np(ref_ops.ggml_mul_mat_vec_a8(wq, xt, 8, k))
    mine = to_np(torch.ops._C_gguf.ggml_mul_mat_vec_a8(wq, xt, 8, k))
    a = O.quantize_q8_1(x)
    want = a["q"][:, :k].astype(np.float32) * np.repeat(a["d"][:, : k // 32].astype(np.float32), 32, 1)
    np.testing.assert_array_equal(ref, want)
    np.testing.assert_array_equal(mine, want)
    # block sums: Q4_0, one row per 32-block with d=1 in that block only and all nibbles 0
    nb = k // 32
    w4 = np.zeros((nb, nb, 18), np.uint8)
    for b in range(nb):
        w4[b, b, 0:2] = np.array([1.0], np.float16).view(np.uint8)
    w4t = torch.from_numpy(w4.reshape(nb, -1)).to(dev())
    ref4 = to_np(ref_ops.ggml_mul_mat_vec_a8(w4t, xt, 2, nb))
    mine4 = to_np(torch.ops._C_gguf.ggml_mul_mat_vec_a8(w4t, xt, 2, nb))
    want4 = -8.0 * a["s"][:, :nb].astype(np.float32)
    np.testing.assert_array_equal(ref4, want4)
    np.testing.assert_array_equal(mine4, want4)
