"""GPU parity tests proper: the CUDA path, called through the C ABI, against the CPU oracle.

Bars: q8_1 activation bytes and integer group dots bit-exact; `ggml_dequantize` bit-exact; fp32 outputs
within rel-L2 1e-3 of the q8_1-semantics oracle (asserted two orders tighter, at 2e-5, so that a wrong
arithmetic flavour - MMVQ vs MMQ differ by ~1e-3 on Q4_K - cannot hide inside the gate).
"""
import numpy as np
import pytest
import torch

from kaillm_b200 import capi
from oracle import gguf_oracle as O
from tests.gpu_util import TDT, act, dev, rel_l2, to_np, wire

pytestmark = pytest.mark.gpu

QT = O.QTYPES
GATE = 1e-3      # the contract
TIGHT = 2e-5     # what fp32 accumulation of exact integer dots should give


# ------------------------------------------------------------------ q8_1
@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("m,k", [(1, 2048), (16, 5120), (3, 700), (2, 17408), (80, 512), (1, 32)])
def test_q8_1_bit_exact(dt, m, k):
    x, xt = act(m, k, seed=m * 7 + k, dt=dt)
    got = capi.quantize_q8_1(xt).cpu().numpy()
    want = O.q8_1_wire(O.quantize_q8_1(x))
    np.testing.assert_array_equal(got, want)


def test_q8_1_special_values():
    x = np.zeros((4, 512), np.float32)
    x[0, 32:64] = np.linspace(-127, 127, 32)
    x[0, 33], x[0, 34] = 2.5, -2.5                  # ties round away from zero
    x[1, :] = 1e-7                                  # tiny: d underflows towards fp16 subnormals
    x[2, :64] = 3000.0                              # fp16 block sum overflows to inf (reference behaviour)
    x[3, ::2] = 65504.0
    x[3, 1::2] = -1e-3
    xt = torch.from_numpy(x).to(dev())
    got = capi.quantize_q8_1(xt).cpu().numpy()
    np.testing.assert_array_equal(got, O.q8_1_wire(O.quantize_q8_1(x)))


def test_q8_1_strided_rows():
    x, _ = act(5, 1024, seed=3, dt="bf16")
    big = torch.zeros((5, 1500), dtype=torch.bfloat16, device=dev())
    big[:, :1024] = torch.from_numpy(x).to(torch.bfloat16)
    got = capi.quantize_q8_1(big[:, :1024]).cpu().numpy()
    np.testing.assert_array_equal(got, O.q8_1_wire(O.quantize_q8_1(x)))


# ------------------------------------------------------------------ integer dots
@pytest.mark.parametrize("qt", QT)
@pytest.mark.parametrize("n,k,m", [(33, 1024, 3), (8, 256, 1), (64, 2048, 16)])
def test_group_dots_bit_exact(qt, n, k, m):
    w, wt = wire(qt, n, k, seed=qt)
    x, xt = act(m, k, seed=11, dt="bf16")
    dots, sums = capi.debug_group_dots(wt, xt, qt)
    _, _, I, S = O.mul_mat(w, qt, x, "mmvq", return_parts=True)
    np.testing.assert_array_equal(dots.cpu().numpy().astype(np.int64), I)
    np.testing.assert_array_equal(sums.cpu().numpy().astype(np.int64), S)


# ------------------------------------------------------------------ mul_mat, fp32 outputs
SHAPES = [(64, 512, 1), (33, 1024, 5), (130, 2048, 16), (17, 256, 2), (256, 5120, 8)]


@pytest.mark.parametrize("qt", QT)
@pytest.mark.parametrize("n,k,m", SHAPES)
@pytest.mark.parametrize("impl", [1, 0, 3])
def test_mul_mat_vec_fp32(qt, n, k, m, impl):
    w, wt = wire(qt, n, k, seed=qt + n)
    x, xt = act(m, k, seed=k + m, dt="bf16")
    capi.set_option("gemv_impl", impl)
    try:
        y = capi.mul_mat(wt, xt, qt, mmq=False, out_dtype=torch.float32)
    finally:
        capi.set_option("gemv_impl", 0)
    want = O.mul_mat(w, qt, x, "mmvq")
    r = rel_l2(to_np(y), want)
    assert r < TIGHT < GATE, r


@pytest.mark.parametrize("qt", [2, 8, 10, 12, 14])
@pytest.mark.parametrize("n,k,m", SHAPES)
@pytest.mark.parametrize("impl", [1, 0])
def test_mul_mat_a8_fp32(qt, n, k, m, impl):
    w, wt = wire(qt, n, k, seed=qt + n)
    x, xt = act(m, k, seed=k + m, dt="f16")
    capi.set_option("gemv_impl", impl)
    try:
        y = capi.mul_mat(wt, xt, qt, mmq=True, out_dtype=torch.float32)
    finally:
        capi.set_option("gemv_impl", 0)
    want = O.mul_mat(w, qt, x, "mmq")
    r = rel_l2(to_np(y), want)
    assert r < TIGHT < GATE, r


@pytest.mark.parametrize("qt", QT)
@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_mul_mat_low_precision_output(qt, dt):
    n, k, m = 96, 1024, 4
    w, wt = wire(qt, n, k, seed=5)
    x, xt = act(m, k, seed=6, dt=dt)
    y = capi.mul_mat(wt, xt, qt)                           # output dtype = activation dtype, as the reference
    assert y.dtype == TDT[dt]
    want = O.round_to_dtype(O.mul_mat(w, qt, x, "mmvq"), dt)
    got = to_np(y)
    assert rel_l2(got, want) < GATE
    assert (got == want).mean() > 0.98                     # only rounding-boundary cases may differ


# ------------------------------------------------------------------ the streaming kernels specifically
@pytest.mark.parametrize("qt", QT)
@pytest.mark.parametrize("n,k,m", [(16, 512, 1), (17, 1024, 2), (100, 2048, 3), (2368, 2048, 5), (1200, 5120, 9),
                                   (333, 4352, 17), (64, 17408, 4), (48, 768, 33), (5, 256, 80)])
def test_streaming_dp4a_gemv_matches_oracle(qt, n, k, m):
    w, wt = wire(qt, n, k, seed=n + k + qt)
    x, xt = act(m, k, seed=m, dt="bf16")
    ws = capi.workspace_bytes(qt, m, n, k)
    scratch = torch.empty(ws, dtype=torch.uint8, device=dev())
    capi.set_option("gemv_impl", 3)
    try:
        y = capi.mul_mat(wt, xt, qt, out_dtype=torch.float32, scratch=scratch)
        assert capi.read_status(qt, m, n, k, scratch) == 0
        yb = capi.mul_mat(wt, xt, qt, out_dtype=torch.float32, scratch=scratch)
    finally:
        capi.set_option("gemv_impl", 0)
    assert rel_l2(to_np(y), O.mul_mat(w, qt, x, "mmvq")) < TIGHT
    assert torch.equal(y, yb)


@pytest.mark.parametrize("qt", [12, 14, 8, 2, 21, 10])
@pytest.mark.parametrize("n,k,m", [(8, 256, 5), (17, 512, 8), (100, 1024, 9), (2368, 2048, 12), (4736, 5120, 16),
                                   (333, 4352, 16), (70, 17408, 5), (1190, 17408, 16), (48, 768, 33), (3000, 14336, 13)])
@pytest.mark.parametrize("mmq", [False, True])
@pytest.mark.parametrize("segments", [0, 1])
def test_shared_stage_mma_gemv_matches_oracle_and_dp4a(qt, n, k, m, mmq, segments):
    """gemv_impl=6: sixteen warps share each stage of 8 rows, tokens on the mma's M side, K split when the
    activation slice would not fit; with tile_segments=1 the rows are fetched as separate segments."""
    if segments and m not in (8, 16):
        pytest.skip("segment mode is covered at two token counts")
    if qt == 21 and mmq:
        pytest.skip("IQ3_S has no MMQ flavour")
    _, wt = wire(qt, n, k, seed=n + k)
    x, xt = act(m, k, seed=m, dt="bf16")
    w = wt.cpu().numpy()
    scratch = torch.empty(capi.workspace_bytes(qt, m, n, k), dtype=torch.uint8, device=dev())
    capi.set_option("gemv_impl", 6)
    capi.set_option("tile_segments", segments)
    try:
        y = capi.mul_mat(wt, xt, qt, mmq=mmq, out_dtype=torch.float32, scratch=scratch)
        assert capi.read_status(qt, m, n, k, scratch) == 0
        yb = capi.mul_mat(wt, xt, qt, mmq=mmq, out_dtype=torch.float32, scratch=scratch)   # counters self-reset
        capi.set_option("gemv_impl", 1)
        y1 = capi.mul_mat(wt, xt, qt, mmq=mmq, out_dtype=torch.float32)
    finally:
        capi.set_option("gemv_impl", 0)
        capi.set_option("tile_segments", 0)
    rows = np.r_[0:min(n, 150), max(0, n - 150):n]
    want = O.mul_mat(w[rows], qt, x, "mmq" if mmq else "mmvq")
    assert rel_l2(to_np(y)[:, rows], want) < TIGHT
    assert torch.equal(y, yb)
    assert rel_l2(to_np(y), to_np(y1)) < TIGHT          # every row, against the general kernel


@pytest.mark.parametrize("qt", [12])
@pytest.mark.parametrize("n,k,m", [(8, 256, 5), (17, 512, 8), (100, 1024, 9), (2368, 2048, 12), (4736, 5120, 16), (4736, 5120, 7),
                                   (333, 4352, 16), (70, 17408, 5), (1190, 17408, 8), (48, 768, 33), (3000, 14336, 3),
                                   (1000, 4096, 16), (1000, 8192, 16), (520, 8192, 6), (600, 11008, 11),
                                   (400, 2816, 8), (1001, 5632, 16)])
@pytest.mark.parametrize("mmq", [False, True])
def test_register_resident_gemv_matches_oracle_and_dp4a(qt, n, k, m, mmq):
    """gemv_impl=7: every consumer warp keeps the activations of its own K units in registers; split-K where a warp's
    share would not fit.  Shapes the kernel does not cover are reported as such, never computed wrongly."""
    _, wt = wire(qt, n, k, seed=n + k)
    x, xt = act(m, k, seed=m, dt="bf16")
    w = wt.cpu().numpy()
    scratch = torch.empty(capi.workspace_bytes(qt, m, n, k), dtype=torch.uint8, device=dev())
    capi.set_option("gemv_impl", 7)
    try:
        try:
            y = capi.mul_mat(wt, xt, qt, mmq=mmq, out_dtype=torch.float32, scratch=scratch)
        except capi.KqError as e:
            assert e.code == capi.KQ_EUNSUPPORTED
            pytest.skip("shape not covered by the register-resident kernel")
        assert capi.read_status(qt, m, n, k, scratch) == 0
        yb = capi.mul_mat(wt, xt, qt, mmq=mmq, out_dtype=torch.float32, scratch=scratch)   # counters self-reset
        capi.set_option("gemv_impl", 1)
        y1 = capi.mul_mat(wt, xt, qt, mmq=mmq, out_dtype=torch.float32)
    finally:
        capi.set_option("gemv_impl", 0)
    rows = np.r_[0:min(n, 150), max(0, n - 150):n]
    want = O.mul_mat(w[rows], qt, x, "mmq" if mmq else "mmvq")
    assert rel_l2(to_np(y)[:, rows], want) < TIGHT
    assert torch.equal(y, yb)
    assert rel_l2(to_np(y), to_np(y1)) < TIGHT          # every row, against the general kernel


@pytest.mark.parametrize("n,k,m", [(128, 256, 1), (256, 512, 5), (200, 1024, 16), (1000, 5120, 3), (17408, 5120, 16), (17408, 5120, 7),
                                   (5120, 17408, 16), (640, 5120, 9), (130, 2048, 21), (4352, 5120, 16), (3000, 4096, 40)])
@pytest.mark.parametrize("mmq", [False, True])
@pytest.mark.parametrize("box", [1, 0])
def test_tensor_memory_gemv_matches_oracle_and_dp4a(n, k, m, mmq, box):
    """gemv_impl=8 (Q4_K): integer dots by tcgen05.mma.kind::i8 with the accumulators in tensor memory, weights staged by
    tiled TMA copies (box=1) or cp.async (box=0); row tiles shared between CTAs meet through partial sums whose order
    does not depend on timing, so two runs are bit-identical."""
    qt = 12
    _, wt = wire(qt, n, k, seed=n + k)
    x, xt = act(m, k, seed=m, dt="bf16")
    w = wt.cpu().numpy()
    scratch = torch.empty(capi.workspace_bytes(qt, m, n, k), dtype=torch.uint8, device=dev())
    capi.set_option("gemv_impl", 8)
    capi.set_option("umma_box", box)
    try:
        l0 = capi.get_option("launch_count")
        y = capi.mul_mat(wt, xt, qt, mmq=mmq, out_dtype=torch.float32, scratch=scratch)
        assert capi.get_option("launch_count") - l0 == 1 + (m + 15) // 16      # quantizer + one launch per 16 tokens
        assert capi.read_status(qt, m, n, k, scratch) == 0
        yb = capi.mul_mat(wt, xt, qt, mmq=mmq, out_dtype=torch.float32, scratch=scratch)   # counters self-reset
        yh = capi.mul_mat(wt, xt, qt, mmq=mmq, out_dtype=torch.bfloat16, scratch=scratch)
        capi.set_option("gemv_impl", 1)
        y1 = capi.mul_mat(wt, xt, qt, mmq=mmq, out_dtype=torch.float32)
    finally:
        capi.set_option("gemv_impl", 0)
        capi.set_option("umma_box", 1)
    rows = np.r_[0:min(n, 150), max(0, n - 150):n]
    want = O.mul_mat(w[rows], qt, x, "mmq" if mmq else "mmvq")
    assert rel_l2(to_np(y)[:, rows], want) < TIGHT
    assert torch.equal(y, yb)
    assert torch.equal(yh, y.to(torch.bfloat16))
    assert rel_l2(to_np(y), to_np(y1)) < TIGHT          # every row, against the general kernel


def test_tensor_memory_gemv_reports_what_it_does_not_cover():
    _, wt = wire(14, 256, 512, seed=3)
    _, xt = act(4, 512, seed=4, dt="bf16")
    capi.set_option("gemv_impl", 8)
    try:
        with pytest.raises(capi.KqError) as e:
            capi.mul_mat(wt, xt, 14, out_dtype=torch.float32)
        assert e.value.code == capi.KQ_EUNSUPPORTED
    finally:
        capi.set_option("gemv_impl", 0)


@pytest.mark.parametrize("qt", QT)
@pytest.mark.parametrize("n,k,m", [(64, 512, 1), (333, 2048, 2), (1200, 5120, 1), (100, 17408, 2), (17, 256, 1)])
@pytest.mark.parametrize("dt", ["bf16", "f16", "f32"])
def test_in_kernel_quantization_equals_quantizer_launch(qt, n, k, m, dt):
    """1-2 tokens: the row-streaming kernel can quantize the activations itself (fuse_q8); the result must be
    bit-identical to the two-launch path (quantizer kernel + GEMV) and match the oracle."""
    w, wt = wire(qt, n, k, seed=n + k + qt)
    x, xt = act(m, k, seed=m + 7, dt=dt)
    scratch = torch.empty(capi.workspace_bytes(qt, m, n, k), dtype=torch.uint8, device=dev())
    capi.set_option("fuse_q8", 2)          # also on matrices too small for the default heuristic
    capi.set_option("gemv_impl", 3)        # the row-streaming kernel for every format (auto mode sends some to the mma kernel)
    try:
        l0 = capi.get_option("launch_count")
        y1 = capi.mul_mat(wt, xt, qt, out_dtype=torch.float32, scratch=scratch)
        fused_launches = capi.get_option("launch_count") - l0
        assert capi.read_status(qt, m, n, k, scratch) == 0
        capi.set_option("fuse_q8", 0)
        l0 = capi.get_option("launch_count")
        y0 = capi.mul_mat(wt, xt, qt, out_dtype=torch.float32, scratch=scratch)
        plain_launches = capi.get_option("launch_count") - l0
    finally:
        capi.set_option("fuse_q8", 1)
        capi.set_option("gemv_impl", 0)
    assert torch.equal(y1, y0)
    if wt.numel() % 16 == 0:
        assert plain_launches == fused_launches + 1
    else:   # a tensor that ends inside a 16-byte unit leaves its last rows to the general kernel, which needs the quantizer
        assert plain_launches == fused_launches
    assert rel_l2(to_np(y1), O.mul_mat(w, qt, x, "mmvq")) < TIGHT


def test_streaming_gemv_declines_unaligned_weights():
    qt, n, k = 14, 32, 512
    _, wt = wire(qt, n, k, seed=1)
    _, xt = act(2, k, seed=1, dt="bf16")
    buf = torch.zeros(wt.numel() + 64, dtype=torch.uint8, device=dev())
    buf[2:2 + wt.numel()] = wt.flatten()
    wv = buf[2:2 + wt.numel()].view(n, -1)            # 2-byte aligned only
    ref = capi.mul_mat(wt, xt, qt, out_dtype=torch.float32)
    got = capi.mul_mat(wv, xt, qt, out_dtype=torch.float32)     # auto: falls back to the general kernel
    assert rel_l2(to_np(got), to_np(ref)) < TIGHT
    capi.set_option("gemv_impl", 6)
    try:
        with pytest.raises(capi.KqError) as e:
            capi.mul_mat(wv, xt, qt, out_dtype=torch.float32)
        assert e.value.code == capi.KQ_EUNSUPPORTED
    finally:
        capi.set_option("gemv_impl", 0)


# ------------------------------------------------------------------ the benchmark configurations at full size
def test_config1_q4_0_single_linear():
    """Q4_0 N=8192 K=2048, fp32 activation [1,2048], seed 0."""
    w, wt = wire(2, 8192, 2048, seed=0)
    x, xt = act(1, 2048, seed=0, dt="f32")
    y = capi.mul_mat(wt, xt, 2, out_dtype=torch.float32)
    assert rel_l2(to_np(y), O.mul_mat(w, 2, x, "mmvq")) < TIGHT


@pytest.mark.parametrize("qt,n,k", [(12, 17408, 5120), (14, 5120, 17408)])
@pytest.mark.parametrize("m", [1, 2, 8, 16])
def test_config2_27b_shapes(qt, n, k, m):
    """Full-size launch; the oracle checks the first and last 96 rows (rows are independent)."""
    _, wt = wire(qt, n, k, seed=qt)
    x, xt = act(m, k, seed=m, dt="bf16")
    w = wt.cpu().numpy()
    rows = np.r_[0:96, n - 96:n]
    scratch = torch.empty(capi.workspace_bytes(qt, m, n, k), dtype=torch.uint8, device=dev())
    for mmq in (False, True):
        yt = capi.mul_mat(wt, xt, qt, mmq=mmq, out_dtype=torch.float32, scratch=scratch)
        assert capi.read_status(qt, m, n, k, scratch) == 0
        y = to_np(yt)
        want = O.mul_mat(w[rows], qt, x, "mmq" if mmq else "mmvq")
        assert rel_l2(y[:, rows], want) < TIGHT
        assert np.isfinite(y).all()
        # every row, against the general kernel (rows are independent, so this covers the middle of the matrix)
        capi.set_option("gemv_impl", 1)
        try:
            y1 = to_np(capi.mul_mat(wt, xt, qt, mmq=mmq, out_dtype=torch.float32))
        finally:
            capi.set_option("gemv_impl", 0)
        assert rel_l2(y, y1) < TIGHT


@pytest.mark.parametrize("qt", [21, 10])
@pytest.mark.parametrize("n,k", [(8192, 2048), (17408, 5120)])
@pytest.mark.parametrize("m", [1, 16, 80])
def test_config5_lowbit_and_verify_shapes(qt, n, k, m):
    _, wt = wire(qt, n, k, seed=qt + 1)
    x, xt = act(m, k, seed=m + 2, dt="bf16")
    w = wt.cpu().numpy()
    rows = np.r_[0:64, n - 64:n]
    want = O.mul_mat(w[rows], qt, x, "mmvq")
    # the integer path everywhere: fp32 rounding only
    capi.set_option("gemm_small_m", 0)
    try:
        y = to_np(capi.mul_mat(wt, xt, qt, out_dtype=torch.float32))
    finally:
        capi.set_option("gemm_small_m", 1)
    assert rel_l2(y[:, rows], want) < TIGHT
    # the default dispatch: Q2_K at 80 tokens goes to the tensor-core GEMM (fp16 operands), inside the gate
    y = to_np(capi.mul_mat(wt, xt, qt, out_dtype=torch.float32))
    assert rel_l2(y[:, rows], want) < (GATE if m > 16 else TIGHT)


# ------------------------------------------------------------------ edge cases
@pytest.mark.parametrize("qt", QT)
def test_edge_shapes(qt):
    blk = O.BLOCK[qt][0]
    for n, k, m in [(1, blk, 1), (3, blk, 7), (5, 3 * blk, 80), (1, 2 * blk, 17)]:
        w, wt = wire(qt, n, k, seed=n + k)
        x, xt = act(m, k, seed=9, dt="f32")
        y = capi.mul_mat(wt, xt, qt, out_dtype=torch.float32)
        assert rel_l2(to_np(y), O.mul_mat(w, qt, x, "mmvq")) < TIGHT


@pytest.mark.parametrize("qt", [12, 14])
def test_strided_output_and_canaries(qt):
    n, k, m = 40, 1024, 6
    w, wt = wire(qt, n, k, seed=1)
    x, xt = act(m, k, seed=2, dt="bf16")
    ybuf = torch.full((m, n + 24), 777.0, dtype=torch.float32, device=dev())
    ws = capi.workspace_bytes(qt, m, n, k)
    sbuf = torch.full((ws + 512,), 0xAB, dtype=torch.uint8, device=dev())
    wpad = torch.full((wt.numel() + 512,), 0xCD, dtype=torch.uint8, device=dev())
    wpad[256:256 + wt.numel()] = wt.flatten()
    wv = wpad[256:256 + wt.numel()].view(n, -1)
    capi.mul_mat(wv, xt, qt, out=ybuf[:, :n], scratch=sbuf[:ws])
    got = to_np(ybuf)
    assert rel_l2(got[:, :n], O.mul_mat(w, qt, x, "mmvq")) < TIGHT
    assert (got[:, n:] == 777.0).all()                       # output padding untouched
    assert (sbuf[ws:] == 0xAB).all()                         # nothing written past the scratch
    assert (wpad[:256] == 0xCD).all() and (wpad[256 + wt.numel():] == 0xCD).all()   # weights never mutated around
    assert torch.equal(wv, wt)


@pytest.mark.parametrize("qt", QT)
def test_repeated_launches_are_deterministic(qt):
    w, wt = wire(qt, 512, 2048, seed=4)
    _, xt = act(16, 2048, seed=4, dt="bf16")
    a = capi.mul_mat(wt, xt, qt, out_dtype=torch.float32)
    b = capi.mul_mat(wt, xt, qt, out_dtype=torch.float32)
    c = capi.mul_mat(wt, xt, qt, out_dtype=torch.float32)
    assert torch.equal(a, b) and torch.equal(a, c)


def test_unsupported_type_raises_on_gpu_too():
    _, wt = wire(12, 8, 256, seed=0)
    _, xt = act(1, 256, seed=0, dt="f32")
    with pytest.raises(capi.KqError) as e:
        capi.mul_mat(wt, xt, 16)
    assert e.value.code == capi.KQ_EUNSUPPORTED


# ------------------------------------------------------------------ dequantize
@pytest.mark.parametrize("qt", QT)
@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
def test_dequantize_bit_exact(qt, dt):
    n, k = 48, 1024
    w, wt = wire(qt, n, k, seed=qt * 3)
    got = to_np(capi.dequantize(wt, qt, n * k, TDT[dt])).reshape(n, k)
    want = O.dequantize(w, qt, dt, half_fma=capi.get_option("half_fma"))
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("qt", [10, 12])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_dequantize_rounding_modes_match_oracle(qt, mode):
    if qt == 12 and mode == 2:
        mode = 1
    n, k = 16, 512
    w, wt = wire(qt, n, k, seed=77)
    old = capi.get_option("half_fma")
    capi.set_option("half_fma", mode)
    try:
        got = to_np(capi.dequantize(wt, qt, n * k, torch.float16)).reshape(n, k)
    finally:
        capi.set_option("half_fma", old)
    np.testing.assert_array_equal(got, O.dequantize(w, qt, "f16", half_fma=mode))
