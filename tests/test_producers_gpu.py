"""Fused activation producers (kq_prepare_q8_rmsnorm, kq_prepare_q8_swiglu): one launch that computes the activation
and quantizes it must give what the separate elementwise kernel + kq_prepare_q8 give."""
import numpy as np
import pytest
import torch

from kaillm_b200 import capi
from tests.gpu_util import TDT, act, dev, rel_l2, to_np, wire

pytestmark = pytest.mark.gpu


def _gemv_from_scratch(wt, qt, m, k, scratch):
    y = torch.empty((m, wt.shape[0]), dtype=torch.float32, device=dev())
    capi.mul_mat_prepared(wt, qt, m, k, y, scratch)
    return y


@pytest.mark.parametrize("dt", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("qt,n,k,m", [(8, 256, 5120, 16), (12, 128, 1024, 3), (14, 64, 2048, 1), (8, 96, 512, 80)])
def test_rmsnorm_producer_equals_norm_then_quantize(qt, n, k, m, dt):
    _, wt = wire(qt, n, k, seed=3)
    g = torch.Generator(device=dev()); g.manual_seed(5)
    x = (torch.randn((m, k), device=dev(), generator=g) * 3.0).to(TDT[dt])
    gamma = (1.0 + 0.1 * torch.randn((k,), device=dev(), generator=g)).to(TDT[dt])
    eps = 1e-6
    # the two roundings of vLLM's rms_norm kernel: (x * inv_rms) to the storage type, then * gamma in the storage type
    inv = torch.rsqrt(x.float().pow(2).mean(dim=1, keepdim=True) + eps)
    xn = (x.float() * inv).to(TDT[dt]) * gamma
    ws = capi.workspace_bytes(qt, m, n, k)
    s_ref = torch.empty(ws, dtype=torch.uint8, device=dev())
    s_fused = torch.full((ws,), 0xFF, dtype=torch.uint8, device=dev())
    capi.prepare_q8(xn, qt, n, s_ref)
    y_norm = torch.empty_like(x)
    capi.prepare_q8_rmsnorm(x, gamma, eps, qt, n, s_fused, y_norm=y_norm)
    assert capi.read_status(qt, m, n, k, s_fused) == 0
    # the normalised tensor: identical up to the last-bit effect of the row sum's order on a few values
    if dt != "f32":   # (in fp32 the last bit of rsqrt reaches every value; the relative check below covers it)
        same = (y_norm == xn).float().mean().item()
        assert same > 0.995, same
    assert rel_l2(to_np(y_norm), to_np(xn)) < 2e-3
    y_ref, y_fused = _gemv_from_scratch(wt, qt, m, k, s_ref), _gemv_from_scratch(wt, qt, m, k, s_fused)
    assert rel_l2(to_np(y_fused), to_np(y_ref)) < 1e-3
    # with the library's own normalised output as input, the separate path reproduces the fused one bit for bit
    capi.prepare_q8(y_norm, qt, n, s_ref)
    assert torch.equal(_gemv_from_scratch(wt, qt, m, k, s_ref), y_fused)


@pytest.mark.parametrize("dt", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("qt,n,k,m", [(14, 128, 17408, 16), (14, 64, 2048, 2), (12, 96, 1024, 7), (8, 64, 512, 33)])
def test_swiglu_producer_equals_act_and_mul_then_quantize(qt, n, k, m, dt):
    _, wt = wire(qt, n, k, seed=4)
    g = torch.Generator(device=dev()); g.manual_seed(6)
    gu = (torch.randn((m, 2 * k), device=dev(), generator=g) * 2.0).to(TDT[dt])
    act = torch.nn.functional.silu(gu[:, :k]) * gu[:, k:]            # SiluAndMul: silu rounded to the dtype, then the product
    ws = capi.workspace_bytes(qt, m, n, k)
    s_ref = torch.empty(ws, dtype=torch.uint8, device=dev())
    s_fused = torch.full((ws,), 0xFF, dtype=torch.uint8, device=dev())
    capi.prepare_q8(act.contiguous(), qt, n, s_ref)
    capi.prepare_q8_swiglu(gu, qt, n, s_fused)
    assert capi.read_status(qt, m, n, k, s_fused) == 0
    y_ref, y_fused = _gemv_from_scratch(wt, qt, m, k, s_ref), _gemv_from_scratch(wt, qt, m, k, s_fused)
    assert rel_l2(to_np(y_fused), to_np(y_ref)) < 1e-3
    assert np.isfinite(to_np(y_fused)).all()


def test_producers_validate_arguments():
    _, wt = wire(12, 8, 256, seed=1)
    x = torch.zeros((2, 256), dtype=torch.bfloat16, device=dev())
    s = torch.empty(capi.workspace_bytes(12, 2, 8, 256), dtype=torch.uint8, device=dev())
    with pytest.raises(capi.KqError) as e:
        capi.prepare_q8_swiglu(x, 12, 8, s[:1024])          # scratch too small (and k = 128 is not a block multiple)
    assert e.value.code in (capi.KQ_ESCRATCH, capi.KQ_EINVAL)
    with pytest.raises(capi.KqError) as e:
        capi.prepare_q8_rmsnorm(torch.zeros((90, 256), dtype=torch.bfloat16, device=dev()), x[0], 1e-6, 12, 8,
                                torch.empty(capi.workspace_bytes(12, 90, 8, 256), dtype=torch.uint8, device=dev()))
    assert e.value.code == capi.KQ_ELIMIT


def test_arrival_poll_gives_up_and_reports():
    """KQ_PREP_WAIT_ARRIVAL on a buffer nobody fills: the bounded poll (about two seconds) runs out, the kernel returns,
    the status word and the per-GPU flag say so, later polls give up at once, and after clearing the flag a buffer whose
    values have arrived is read normally.  Nothing faults: the wait is a loop on ordinary loads with a clock limit."""
    import time
    m, k, qt = 2, 256, 12
    empty = torch.full((m, k), -1, dtype=torch.int16, device=dev()).view(torch.bfloat16)      # every element = the sentinel
    scratch = torch.zeros(capi.workspace_bytes(qt, m, 64, k), dtype=torch.uint8, device=dev())
    assert capi.arrival_status(clear=True) in (0, 40, 41)
    t0 = time.time()
    capi.prepare_q8(empty, qt, 64, scratch, wait_arrival=True)
    torch.cuda.synchronize()
    first = time.time() - t0
    assert capi.read_status(qt, m, 64, k, scratch) == 40 and capi.arrival_status() == 40
    t0 = time.time()
    capi.prepare_q8(empty, qt, 64, scratch, wait_arrival=True)      # gives up at once now
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    capi.wait_arrival(empty, status)
    torch.cuda.synchronize()
    assert time.time() - t0 < 0.5 * first + 0.2 and int(status.item()) == 41
    assert capi.arrival_status(clear=True) != 0 and capi.arrival_status() == 0
    # values that have arrived: identical to the plain preparation
    x, xt = act(m, k, seed=3, dt="bf16")
    s2 = torch.zeros_like(scratch)
    capi.prepare_q8(xt, qt, 64, scratch, wait_arrival=True)
    capi.prepare_q8(xt, qt, 64, s2)
    capi.wait_arrival(xt, status.zero_())
    torch.cuda.synchronize()
    assert capi.read_status(qt, m, 64, k, scratch) == 0 and int(status.item()) == 0 and capi.arrival_status() == 0
    _, wt = wire(qt, 64, k, seed=5)
    y1 = torch.empty((m, 64), dtype=torch.float32, device=dev())
    y2 = torch.empty_like(y1)
    capi.mul_mat_prepared(wt, qt, m, k, y1, scratch)
    capi.mul_mat_prepared(wt, qt, m, k, y2, s2)
    assert torch.equal(y1, y2)
