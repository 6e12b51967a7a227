"""GPU tests of the tcgen05 prefill GEMM (M > 80 tokens) through the C ABI.

The GEMM multiplies fp16-dequantized weights (bit-identical to ggml_dequantize) with fp16(d8*q8) activations and
accumulates in fp32, so two checks apply: (1) against the dense product of exactly those fp16 operands it must agree
to fp32 accumulation error - this pins tile layout, swizzle, descriptors and the K pipeline; (2) against the
q8_1-semantics oracle (what the reference's MMQ kernels compute) it must stay inside the 1e-3 gate."""
import numpy as np
import pytest
import torch

from kaillm_b200 import capi
from oracle import gguf_oracle as O
from tests.gpu_util import act, dev, rel_l2, to_np, wire

pytestmark = pytest.mark.gpu
GATE = 1e-3


def fp16_operand_product(w, qt, x, mmq):
    """float64 product of the operands the GEMM feeds its tensor cores (incl. the raw-sum correction steps)."""
    a = O.quantize_q8_1(x)
    k = x.shape[1]
    d = np.repeat(a["d"][:, : k // 32].astype(np.float32), 32, axis=1)
    xh = (d * a["q"][:, :k].astype(np.float32)).astype(np.float16).astype(np.float64)
    s8 = a["s"][:, : k // 32].astype(np.float64)
    if qt == O.Q4_0:
        u = O.unpack(w, qt)
        wh = O.hmul(O.f2h(u["q"]), np.repeat(u["d"], 32, axis=1)).astype(np.float64)      # d*q without the -8
        c = O.hmul(np.float16(-8.0), u["d"]).astype(np.float64)
        return xh @ wh.T + s8 @ c.T
    if qt == O.Q4_K and mmq:
        u = O.unpack(w, qt)
        d1 = O.hmul(np.repeat(u["d"], 8, axis=1), O.f2h(u["sc"]))                           # [n, k/32]
        wh = O.hmul(np.repeat(d1, 32, axis=1), O.f2h(u["q"])).astype(np.float64)
        c = -O.hmul(np.repeat(u["dmin"], 8, axis=1), O.f2h(u["mn"])).astype(np.float64)
        return xh @ wh.T + s8 @ c.T
    wh = O.dequantize(w, qt, "f16", half_fma=capi.get_option("half_fma")).astype(np.float64)
    return xh @ wh.T


@pytest.fixture(params=[0, 2], ids=["tile256x128", "tile128x256"])
def tile_shape(request):
    """Both tile shapes of the GEMM kernel (option gemm_wide), whatever the token count."""
    old = capi.get_option("gemm_wide")
    capi.set_option("gemm_wide", request.param)
    yield request.param
    capi.set_option("gemm_wide", old)


@pytest.mark.parametrize("qt", O.QTYPES)
@pytest.mark.parametrize("n,k,m", [(128, 256, 128), (256, 1024, 96), (200, 512, 81), (384, 2048, 300), (130, 768, 129),
                                   (300, 1280, 520)])
def test_gemm_matches_fp16_operand_product_and_oracle(qt, n, k, m, tile_shape):
    w, wt = wire(qt, n, k, seed=qt + n)
    x, xt = act(m, k, seed=k + m, dt="bf16")
    ws = capi.workspace_bytes(qt, m, n, k)
    scratch = torch.empty(ws, dtype=torch.uint8, device=dev())
    mmq = qt != 21
    y = to_np(capi.mul_mat(wt, xt, qt, mmq=mmq, out_dtype=torch.float32, scratch=scratch))
    assert capi.read_status(qt, m, n, k, scratch) == 0
    assert rel_l2(y, fp16_operand_product(w, qt, x, mmq)) < 5e-6
    assert rel_l2(y, O.mul_mat(w, qt, x, "mmq" if mmq else "mmvq")) < GATE


@pytest.mark.parametrize("qt", [2, 8])
@pytest.mark.parametrize("n,k,m", [(136, 640, 260), (128, 128, 90), (260, 384, 257)])
def test_gemm_odd_number_of_k_steps(qt, n, k, m, tile_shape):
    """32-weight formats allow K = an odd multiple of 128: in the 128 x 256 tile the two unpacking groups take
    alternate steps, so one of them has one step fewer (Q4_0 adds its correction step on top)."""
    w, wt = wire(qt, n, k, seed=qt + k)
    x, xt = act(m, k, seed=k + m, dt="bf16")
    scratch = torch.empty(capi.workspace_bytes(qt, m, n, k), dtype=torch.uint8, device=dev())
    y = to_np(capi.mul_mat(wt, xt, qt, mmq=True, out_dtype=torch.float32, scratch=scratch))
    assert capi.read_status(qt, m, n, k, scratch) == 0
    assert rel_l2(y, fp16_operand_product(w, qt, x, True)) < 5e-6
    assert rel_l2(y, O.mul_mat(w, qt, x, "mmq")) < GATE


def test_gemm_q4k_vec_flavour_folds_the_min_term():
    qt, n, k, m = 12, 256, 1024, 96
    w, wt = wire(qt, n, k, seed=2)
    x, xt = act(m, k, seed=2, dt="bf16")
    y = to_np(capi.mul_mat(wt, xt, qt, mmq=False, out_dtype=torch.float32))
    assert rel_l2(y, fp16_operand_product(w, qt, x, False)) < 5e-6
    assert rel_l2(y, O.mul_mat(w, qt, x, "mmvq")) < GATE


@pytest.mark.parametrize("m", [256, 1024, 2048])
def test_config4_q4k_prefill(m):
    """Prefill benchmark shape: Q4_K N=17408 K=5120, bf16 activations; oracle on the first and last 64 rows."""
    qt, n, k = 12, 17408, 5120
    _, wt = wire(qt, n, k, seed=4)
    x, xt = act(m, k, seed=m, dt="bf16")
    w = wt.cpu().numpy()
    y = capi.mul_mat(wt, xt, qt, mmq=True)
    assert y.dtype == torch.bfloat16 and bool(torch.isfinite(y).all())
    rows = np.r_[0:64, n - 64:n]
    got = to_np(y)[:, rows]
    want = O.mul_mat(w[rows], qt, x, "mmq")
    assert rel_l2(got, O.round_to_dtype(want, "bf16")) < 3e-3      # includes the bf16 rounding of the outputs
    y32 = to_np(capi.mul_mat(wt, xt, qt, mmq=True, out_dtype=torch.float32))[:, rows]
    assert rel_l2(y32, want) < GATE


def _takes_gemm(qt, n, m):
    """The library's rule for 17..80 tokens (kq_api.cu: gemm_wanted), restated."""
    tiles = (n + 127) // 128
    if tiles >= 120:
        return m >= (33 if qt == 2 else 17)
    if tiles >= 60:
        return m >= (49 if qt == 14 else 33)
    if tiles >= 30:
        return qt != 14 and m >= 49
    return False


@pytest.mark.parametrize("qt,n,k", [(12, 16384, 1024), (14, 15488, 512), (12, 7808, 1024), (8, 4096, 512), (2, 7808, 512)])
@pytest.mark.parametrize("m", [17, 33, 80])
def test_calls_of_17_to_80_tokens_take_the_gemm_where_it_is_faster(qt, n, k, m):
    """Two or more 16-token GEMV passes against one GEMM launch: with enough 128-row tiles the GEMM takes the call
    (option gemm_small_m).  Both paths must pass the gate; the fused producers must feed the GEMM as well."""
    _, wt = wire(qt, n, k, seed=qt + m)
    x, xt = act(m, k, seed=m, dt="bf16")
    w = wt.cpu().numpy()
    rows = np.r_[0:64, n - 64:n]
    want = O.mul_mat(w[rows], qt, x, "mmvq")
    y = capi.mul_mat(wt, xt, qt, out_dtype=torch.float32)
    capi.set_option("gemm_small_m", 0)
    try:
        y_int = capi.mul_mat(wt, xt, qt, out_dtype=torch.float32)
    finally:
        capi.set_option("gemm_small_m", 1)
    assert rel_l2(to_np(y_int)[:, rows], want) < 2e-5                # integer dots: fp32 rounding only
    assert rel_l2(to_np(y)[:, rows], want) < GATE
    assert torch.equal(y, y_int) != _takes_gemm(qt, n, m)                      # fp16 operands differ from integer dots in the last bits
    # the same call in two halves, activations from the SwiGLU producer
    g = torch.Generator(device=dev()); g.manual_seed(m)
    gu = torch.randn((m, 2 * k), device=dev(), generator=g).to(torch.bfloat16)
    a = (torch.nn.functional.silu(gu[:, :k]) * gu[:, k:]).contiguous()
    scratch = torch.full((capi.workspace_bytes(qt, m, n, k),), 0xFF, dtype=torch.uint8, device=dev())
    capi.prepare_q8_swiglu(gu, qt, n, scratch)
    y2 = torch.empty((m, n), dtype=torch.float32, device=dev())
    capi.mul_mat_prepared(wt, qt, m, k, y2, scratch)
    assert capi.read_status(qt, m, n, k, scratch) == 0
    assert rel_l2(to_np(y2)[:, rows], O.mul_mat(w[rows], qt, a.float().cpu().numpy(), "mmvq")) < GATE


def test_one_preparation_serves_types_with_different_gemm_thresholds():
    """A preparation made for a Q6_K tensor (GEMM from 49 tokens at this size) is then used by a Q4_K and a Q4_0 tensor
    that take the GEMM at 40 tokens: the preparation writes the GEMM's operands whatever type it was told."""
    n, k, m = 8192, 512, 40
    x, xt = act(m, k, seed=11, dt="bf16")
    ws = max(capi.workspace_bytes(qt, m, n, k) for qt in (14, 12, 2))
    scratch = torch.full((ws,), 0xFF, dtype=torch.uint8, device=dev())
    capi.prepare_q8(xt, 14, n, scratch)
    rows = np.r_[0:64, n - 64:n]
    for qt in (12, 2, 14):
        w, wt = wire(qt, n, k, seed=qt)
        y = torch.empty((m, n), dtype=torch.float32, device=dev())
        capi.mul_mat_prepared(wt, qt, m, k, y, scratch)
        assert capi.read_status(qt, m, n, k, scratch) == 0
        assert rel_l2(to_np(y)[:, rows], O.mul_mat(w[rows], qt, x, "mmvq")) < GATE


def test_gemm_and_gemv_paths_agree():
    qt, n, k, m = 14, 512, 2048, 96
    _, wt = wire(qt, n, k, seed=9)
    _, xt = act(m, k, seed=9, dt="f16")
    y_gemm = capi.mul_mat(wt, xt, qt, mmq=True, out_dtype=torch.float32)
    old = capi.get_option("gemm_min_m")
    capi.set_option("gemm_min_m", 1 << 30)
    try:
        y_gemv = capi.mul_mat(wt, xt, qt, mmq=True, out_dtype=torch.float32)
    finally:
        capi.set_option("gemm_min_m", old)
    assert rel_l2(to_np(y_gemm), to_np(y_gemv)) < GATE


@pytest.mark.parametrize("dt", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("qt,n,k,m", [(12, 256, 1024, 200), (14, 384, 2048, 96), (2, 128, 512, 130)])
def test_gemm_only_quantizer_equals_full_quantizer(qt, n, k, m, dt):
    """kq_mul_mat_a8 at large M quantizes with the lane-per-block kernel that writes only the GEMM's operands;
    kq_prepare_q8 + kq_mul_mat_prepared goes through the warp-per-block kernel that writes everything.  Same bits."""
    _, wt = wire(qt, n, k, seed=n + qt)
    _, xt = act(m, k, seed=m + 1, dt=dt)
    scratch = torch.empty(capi.workspace_bytes(qt, m, n, k), dtype=torch.uint8, device=dev())
    y1 = capi.mul_mat(wt, xt, qt, mmq=True, out_dtype=torch.float32, scratch=scratch)
    y0 = torch.empty_like(y1)
    capi.prepare_q8(xt, qt, n, scratch)
    capi.mul_mat_prepared(wt, qt, m, k, y0, scratch, mmq=True)
    assert torch.equal(y1, y0)


@pytest.mark.parametrize("qt,k,n_max,n_small", [(14, 17408, 1024, 296), (12, 17408, 1024, 136), (14, 17408, 4096, 40)])
@pytest.mark.parametrize("m", [8, 16])
def test_one_preparation_serves_weight_tensors_of_different_n(qt, k, n_max, n_small, m):
    """q/k/v-style sharing: kq_prepare_q8 sized for the widest tensor, then split-K launches on a narrower and on the
    widest one, in both orders, on a scratch that held 0xFF everywhere before the preparation."""
    _, w_big = wire(qt, n_max, k, seed=1)
    _, w_small = wire(qt, n_small, k, seed=2)
    x, xt = act(m, k, seed=3, dt="bf16")
    ws = capi.workspace_bytes(qt, m, n_max, k)
    for order in ((w_small, w_big), (w_big, w_small), (w_small, w_small)):
        scratch = torch.full((ws,), 0xFF, dtype=torch.uint8, device=dev())
        capi.prepare_q8(xt, qt, n_max, scratch)
        for wt in order:
            n = wt.shape[0]
            y = torch.full((m, n), float("nan"), dtype=torch.float32, device=dev())
            capi.mul_mat_prepared(wt, qt, m, k, y, scratch)
            assert capi.read_status(qt, m, n_max, k, scratch) == 0
            want = O.mul_mat(wt.cpu().numpy(), qt, x, "mmvq")
            assert rel_l2(to_np(y), want) < 2e-5
