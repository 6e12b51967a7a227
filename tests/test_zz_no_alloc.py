"""The scratch-free entry point kq_mul_mat_vec_a8_static (collected last on purpose: a failure here cannot hide the
other tests from a run that stops at the first failure).

Hosts that may not allocate device memory at call time - an engine whose arena already owns the whole GPU, a plug-in
bound by a no-cudaMalloc rule on its hot path - call this variant: its quantized-activation scratch is a device array
inside the library.  It must give exactly what kq_mul_mat_vec_a8 gives with caller scratch, call after call, because
the array keeps the previous call's contents."""
import numpy as np
import pytest
import torch

from kaillm_b200 import capi
from oracle import gguf_oracle as O
from tests.gpu_util import act, dev, rel_l2, to_np, wire

TIGHT = 2e-5


@pytest.mark.gpu
def test_static_scratch_entry_matches_regular_entry_twice_in_a_row():
    # call 1: Q4_K, 13 tokens (tensor-core kernel with split-K counters); call 2: Q6_K, 3 tokens, other sizes
    for qt, n, k, m in ((12, 2368, 5120, 13), (14, 1000, 2048, 3)):
        w, wt = wire(qt, n, k, seed=qt + m)
        x, xt = act(m, k, seed=m, dt="bf16")
        ref = capi.mul_mat(wt, xt, qt, out_dtype=torch.float32)            # caller-provided scratch
        out = torch.empty((m, n), dtype=torch.float32, device=dev())
        capi.mul_mat_vec_static(wt, xt, qt, out)                            # first call: kernels get loaded
        torch.cuda.synchronize()
        assert torch.equal(out, ref)                                        # same kernels, same bits
        out.zero_()
        free_before = torch.cuda.mem_get_info()[0]
        capi.mul_mat_vec_static(wt, xt, qt, out)                            # second call in a row, same array
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before                 # no device memory was allocated
        assert rel_l2(to_np(out), to_np(ref)) < TIGHT
        assert torch.equal(out, ref)
        assert rel_l2(to_np(out), O.mul_mat(w, qt, x, "mmvq")) < TIGHT


@pytest.mark.gpu
def test_static_scratch_entry_rejects_sizes_beyond_its_limits():
    _, wt = wire(12, 16, 256, seed=1)
    _, xt = act(17, 256, seed=1, dt="bf16")
    out = torch.empty((17, 16), dtype=torch.bfloat16, device=dev())
    with pytest.raises(capi.KqError) as e:
        capi.mul_mat_vec_static(wt, xt, 12, out)
    assert e.value.code == capi.KQ_ELIMIT and "m <= 16" in str(e.value)


def test_static_scratch_entry_limit_check_needs_no_gpu():
    rc = capi.lib.kq_mul_mat_vec_a8_static(0x1000, 12, 40000, 256, 0x2000, 0, 1, 256, 0x3000, 0, 40000, None)
    assert rc == capi.KQ_ELIMIT
    assert b"n <= 32768" in capi.lib.kq_last_error()
