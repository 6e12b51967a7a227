"""The formats beyond the benchmark's six that real mixed-precision GGUF checkpoints contain and that the reference's
Python gate sends to the `_C_gguf` ops (vllm_gguf_plugin/ops.py:54-90): Q4_1, Q5_0, Q5_1, Q3_K, Q5_K, IQ4_NL, IQ4_XS.
They run on the general kernels (row-streaming and dp4a GEMV at every token count, dequantize); checked against the
CPU oracle and against the reference's own CUDA build."""
import numpy as np
import pytest
import torch

from kaillm_b200 import capi, ops  # noqa: F401  (ops registers torch.ops._C_gguf)
from oracle import gguf_oracle as O
from tests.gpu_util import TDT, act, dev, rel_l2, to_np, wire

pytestmark = pytest.mark.gpu
MORE = O.MORE_QTYPES
MORE_MMQ = tuple(t for t in MORE if t not in O.NO_MMQ)
GATE = 1e-3
TIGHT = 2e-5


@pytest.mark.parametrize("qt", MORE)
@pytest.mark.parametrize("n,k,m", [(1, 256, 1), (33, 512, 2), (64, 1024, 5), (200, 2048, 16), (70, 5120, 3), (24, 256, 81)])
@pytest.mark.parametrize("impl", [0, 1, 3])
def test_mul_mat_vec_matches_oracle(qt, n, k, m, impl):
    w, wt = wire(qt, n, k, seed=qt + n)
    x, xt = act(m, k, seed=m, dt="bf16")
    scratch = torch.empty(capi.workspace_bytes(qt, m, n, k), dtype=torch.uint8, device=dev())
    capi.set_option("gemv_impl", impl)
    try:
        y = capi.mul_mat(wt, xt, qt, out_dtype=torch.float32, scratch=scratch)
        assert capi.read_status(qt, m, n, k, scratch) == 0
    finally:
        capi.set_option("gemv_impl", 0)
    assert rel_l2(to_np(y), O.mul_mat(w, qt, x, "mmvq")) < TIGHT


@pytest.mark.parametrize("qt", MORE_MMQ)
@pytest.mark.parametrize("n,k,m", [(33, 512, 3), (64, 1024, 16), (40, 2048, 80), (48, 512, 130)])
@pytest.mark.parametrize("impl", [0, 1])
def test_mul_mat_a8_matches_oracle(qt, n, k, m, impl):
    w, wt = wire(qt, n, k, seed=qt + n + 1)
    x, xt = act(m, k, seed=m, dt="f16")
    capi.set_option("gemv_impl", impl)
    try:
        y = capi.mul_mat(wt, xt, qt, mmq=True, out_dtype=torch.float32)
    finally:
        capi.set_option("gemv_impl", 0)
    assert rel_l2(to_np(y), O.mul_mat(w, qt, x, "mmq")) < TIGHT


@pytest.mark.parametrize("qt", [20, 23])
def test_imatrix_formats_have_no_mmq(qt):
    _, wt = wire(qt, 8, 256, seed=1)
    _, xt = act(2, 256, seed=1, dt="f32")
    with pytest.raises(capi.KqError) as e:
        capi.mul_mat(wt, xt, qt, mmq=True)
    assert e.value.code == capi.KQ_EUNSUPPORTED


@pytest.mark.parametrize("qt", MORE)
def test_integer_group_dots_bit_exact(qt):
    n, k, m = 12, 512, 3
    w, wt = wire(qt, n, k, seed=2)
    x, xt = act(m, k, seed=2, dt="f32")
    dots, sums = capi.debug_group_dots(wt, xt, qt)
    _, _, I, S = O.mul_mat(w, qt, x, "mmvq", return_parts=True)
    np.testing.assert_array_equal(dots.cpu().numpy(), I)
    np.testing.assert_array_equal(sums.cpu().numpy(), S)


@pytest.mark.parametrize("qt", MORE)
@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
def test_dequantize_bit_exact(qt, dt):
    n, k = 24, 1024
    w, wt = wire(qt, n, k, seed=qt * 3)
    got = to_np(capi.dequantize(wt, qt, n * k, TDT[dt])).reshape(n, k)
    np.testing.assert_array_equal(got, O.dequantize(w, qt, dt, half_fma=capi.get_option("half_fma")))


# ------------------------------------------------------------------ against the reference's own CUDA build
@pytest.mark.parametrize("qt", MORE)
@pytest.mark.parametrize("n,k,m", [(64, 512, 1), (136, 2048, 2), (96, 5120, 6), (64, 1024, 16)])
def test_mul_mat_vec_matches_reference_kernels(ref_ops, qt, n, k, m):
    w, wt = wire(qt, n, k, seed=qt)
    x, xt = act(m, k, seed=m, dt="f32")
    ref = to_np(ref_ops.ggml_mul_mat_vec_a8(wt, xt, qt, n))
    mine = to_np(torch.ops._C_gguf.ggml_mul_mat_vec_a8(wt, xt, qt, n))
    assert rel_l2(mine, ref) < TIGHT < GATE
    assert rel_l2(ref, O.mul_mat(w, qt, x, "mmvq")) < TIGHT      # the oracle is pinned by the reference itself


@pytest.mark.parametrize("qt", MORE_MMQ)
@pytest.mark.parametrize("n,k,m", [(64, 512, 3), (160, 2048, 16), (96, 1024, 80)])
def test_mul_mat_a8_matches_reference_kernels(ref_ops, qt, n, k, m):
    w, wt = wire(qt, n, k, seed=qt + 1)
    x, xt = act(m, k, seed=m + 1, dt="f32")
    ref = to_np(ref_ops.ggml_mul_mat_a8(wt, xt, qt, n))
    mine = to_np(torch.ops._C_gguf.ggml_mul_mat_a8(wt, xt, qt, n))
    assert rel_l2(mine, ref) < TIGHT < GATE
    assert rel_l2(ref, O.mul_mat(w, qt, x, "mmq")) < TIGHT


@pytest.mark.parametrize("qt", MORE)
@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
def test_dequantize_bit_identical_to_reference(ref_ops, qt, dt):
    n, k = 40, 1024
    _, wt = wire(qt, n, k, seed=qt + 9)
    ref = ref_ops.ggml_dequantize(wt, qt, n, k, TDT[dt])
    mine = torch.ops._C_gguf.ggml_dequantize(wt, qt, n, k, TDT[dt])
    assert torch.equal(mine, ref)


@pytest.mark.parametrize("qt", O.ALL_QTYPES)
@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
def test_embedding_rows_match_oracle(qt, dt):
    """kq_dequantize_rows / linear.apply_gguf_embedding: the selected rows, read in place, equal the dequantized gather
    (vllm_gguf_plugin/quantization/vocal_embeds.py:29-58); Q4_K / Q5_K / Q6_K with fp32 products (gguf-reader's
    arithmetic), the others with ggml_dequantize's."""
    from kaillm_b200 import linear
    vocab, hidden = 300, 1024
    w, wt = wire(qt, vocab, hidden, seed=9 + qt)
    ids = torch.tensor([[5, 299, 0], [17, 5, 123]], dtype=torch.long, device=dev())
    out = linear.apply_gguf_embedding(ids, wt, qt, hidden, TDT[dt])
    assert out.shape == (2, 3, hidden) and out.dtype == TDT[dt]
    rows = w[ids.flatten().cpu().numpy()]
    if qt in (12, 13, 14):
        want = O.round_to_dtype(O.dequantize_f32(rows, qt), dt)
    else:
        want = O.dequantize(rows, qt, dt, half_fma=capi.get_option("half_fma"))
    np.testing.assert_array_equal(to_np(out).reshape(-1, hidden), want)
    bad = torch.tensor([0, vocab, -1, 7], dtype=torch.long, device=dev())
    got = capi.dequantize_rows(wt, qt, hidden, bad, TDT[dt], f32_math=qt in (12, 13, 14))
    assert not got[1].any() and not got[2].any() and torch.equal(got[3], capi.dequantize_rows(wt, qt, hidden, bad[3:], TDT[dt], f32_math=qt in (12, 13, 14))[0])
