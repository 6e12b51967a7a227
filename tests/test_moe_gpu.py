"""Mixture-of-experts ops: `ggml_moe_a8_vec` / `ggml_moe_a8` / `ggml_moe_get_block_size` through the C ABI and through
`torch.ops._C_gguf`, against the CPU oracle (every (token, expert) pair is an ordinary quantized mat-vec,
vllm_gguf_plugin/csrc/gguf/moe_vec.cuh:4-52 and moe.cuh:9-128) and, where it was built, against the reference's own CUDA
kernels."""
import os

import numpy as np
import pytest
import torch

from kaillm_b200 import capi, ops as kq_ops, synth  # noqa: F401 - ops registers torch.ops._C_gguf
from oracle import gguf_oracle as O
from tests.gpu_util import TDT, act, dev, rel_l2, to_np

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TIGHT = 2e-5


def experts_wire(qt, e, n, k, seed):
    w = np.stack([synth.wire_numpy(qt, n, k, seed=seed + i) for i in range(e)])
    return w, torch.from_numpy(w).to(dev())


def routing(tokens, top_k, e, seed):
    rng = np.random.default_rng(seed)
    ids = np.stack([rng.choice(e, size=top_k, replace=False) for _ in range(tokens)]).astype(np.int32)
    return ids


def align(topk_ids, block, e):
    """What vLLM's moe_align_block_size produces: slots sorted by expert, every expert's run padded to a multiple of
    `block` with the value tokens * top_k, one expert id per block, the padded total."""
    flat = topk_ids.reshape(-1)
    pad = flat.size
    sorted_ids, expert_ids = [], []
    for ex in range(e):
        z = np.nonzero(flat == ex)[0]
        if z.size == 0:
            continue
        nb = (z.size + block - 1) // block
        sorted_ids += list(z) + [pad] * (nb * block - z.size)
        expert_ids += [ex] * nb
    return (np.asarray(sorted_ids, np.int32), np.asarray(expert_ids, np.int32), np.asarray([len(sorted_ids)], np.int32))


def expected(w, qt, x, topk_ids, flavour):
    tokens, top_k = topk_ids.shape
    out = np.zeros((tokens * top_k, w.shape[1]), np.float32)
    for z in range(tokens * top_k):
        t, ex = z // top_k, int(topk_ids.reshape(-1)[z])
        out[z] = O.mul_mat(w[ex], qt, x[t:t + 1], flavour)[0]
    return out


@pytest.fixture(scope="module")
def ref_cuda():
    path = os.path.join(ROOT, "oracle", "_ref", "_C_gguf_ref.so")
    if not os.path.exists(path):
        return None
    if not hasattr(torch.ops, "_C_gguf_ref") or not hasattr(torch.ops._C_gguf_ref, "ggml_moe_a8_vec"):
        torch.ops.load_library(path)
    return torch.ops._C_gguf_ref


@pytest.mark.parametrize("qt", O.ALL_QTYPES)
@pytest.mark.parametrize("e,n,k,tokens,top_k", [(4, 96, 512, 5, 2), (8, 33, 1024, 1, 4), (3, 130, 256, 9, 1)])
def test_moe_vec_matches_oracle(qt, e, n, k, tokens, top_k):
    w, wt = experts_wire(qt, e, n, k, seed=qt * 10)
    x, xt = act(tokens, k, seed=3 + tokens, dt="bf16")
    ids = routing(tokens, top_k, e, seed=qt)
    y = capi.moe_a8_vec(wt, xt, torch.from_numpy(ids).to(dev()), qt, out_dtype=torch.float32)
    assert rel_l2(to_np(y), expected(w, qt, x, ids, "mmvq")) < TIGHT


@pytest.mark.parametrize("qt", [q for q in O.ALL_QTYPES if q not in O.NO_MMQ])
@pytest.mark.parametrize("e,n,k,tokens,top_k", [(4, 64, 512, 70, 2), (6, 40, 256, 13, 3), (2, 130, 1024, 3, 1)])
def test_moe_block_matches_oracle(qt, e, n, k, tokens, top_k):
    w, wt = experts_wire(qt, e, n, k, seed=qt * 10 + 1)
    x, xt = act(tokens, k, seed=5 + tokens, dt="f16")
    ids = routing(tokens, top_k, e, seed=qt + 1)
    bs = capi.lib.kq_moe_block_size(qt)
    assert bs == 8
    s, ex, tot = (torch.from_numpy(a).to(dev()) for a in align(ids, bs, e))
    y = capi.moe_a8(wt, xt, s, ex, tot, top_k, qt, out_dtype=torch.float32)
    assert rel_l2(to_np(y), expected(w, qt, x, ids, "mmq")) < TIGHT


def test_moe_skips_bad_experts_and_padding():
    qt, e, n, k, tokens, top_k = 12, 3, 48, 256, 6, 2
    w, wt = experts_wire(qt, e, n, k, seed=77)
    x, xt = act(tokens, k, seed=8, dt="bf16")
    ids = routing(tokens, top_k, e, seed=9)
    bad = ids.copy()
    bad[1, 0], bad[4, 1] = 99, -1
    y = to_np(capi.moe_a8_vec(wt, xt, torch.from_numpy(bad).to(dev()), qt, out_dtype=torch.float32))
    want = expected(w, qt, x, np.where((bad < 0) | (bad >= e), ids, bad), "mmvq")
    want[1 * top_k + 0] = 0
    want[4 * top_k + 1] = 0
    assert rel_l2(y, want) < TIGHT and not y[2].any() and not y[9].any()
    s, ex, tot = align(ids, 8, e)
    ex = ex.copy()
    ex[0] = 300                                        # a block of an unknown expert is skipped
    y = to_np(capi.moe_a8(wt, xt, *(torch.from_numpy(a).to(dev()) for a in (s, ex, tot)), top_k, qt, out_dtype=torch.float32))
    want = expected(w, qt, x, ids, "mmq")
    skipped = [int(z) for z in s[:8] if z < tokens * top_k]
    want[skipped] = 0
    assert rel_l2(y, want) < TIGHT and not y[skipped].any()
    with pytest.raises(capi.KqError):
        capi.moe_a8(wt, xt, *(torch.from_numpy(a).to(dev()) for a in (s, ex, tot)), top_k, 21)     # IQ3_S: no MMQ flavour


@pytest.mark.parametrize("qt", [12, 14, 8, 2, 10, 13])
@pytest.mark.parametrize("dt", ["bf16", "f16"])
def test_moe_torch_ops_match_oracle_and_reference_cuda(qt, dt, ref_cuda):
    """The registered ops, as the reference's fused MoE layer calls them (quantization/fused_moe.py:34-133): two chained
    projections per path, routing weights applied outside."""
    e, n, k, tokens, top_k = 4, 128, 512, 67, 2
    w, wt = experts_wire(qt, e, n, k, seed=qt)
    x, xt = act(tokens, k, seed=21, dt=dt)
    ids = routing(tokens, top_k, e, seed=qt + 5)
    idt = torch.from_numpy(ids).to(dev())
    g = torch.ops._C_gguf
    bs = g.ggml_moe_get_block_size(qt)
    assert bs == 8 and g.ggml_moe_get_block_size(16) == 0
    yv = g.ggml_moe_a8_vec(xt, wt, idt, top_k, qt, n, tokens)
    assert yv.dtype == TDT[dt] and tuple(yv.shape) == (tokens * top_k, n)
    want_v = expected(w, qt, x, ids, "mmvq")
    assert rel_l2(to_np(yv), want_v) < 5e-3          # 16-bit outputs
    s, ex, tot = (torch.from_numpy(a).to(dev()) for a in align(ids, bs, e))
    yb = g.ggml_moe_a8(xt, wt, s, ex, tot, qt, n, top_k, tokens)
    want_b = expected(w, qt, x, ids, "mmq")
    assert rel_l2(to_np(yb), want_b) < 5e-3
    if ref_cuda is not None:
        rv = ref_cuda.ggml_moe_a8_vec(xt, wt, idt, top_k, qt, n, tokens)
        assert rel_l2(to_np(yv), to_np(rv)) < 5e-3 and float((yv == rv).float().mean()) > 0.98
        rbs = ref_cuda.ggml_moe_get_block_size(qt)
        rs, rex, rtot = (torch.from_numpy(a).to(dev()) for a in align(ids, rbs, e))
        rb = ref_cuda.ggml_moe_a8(xt, wt, rs, rex, rtot, qt, n, top_k, tokens)
        assert rel_l2(to_np(yb), to_np(rb)) < 5e-3 and float((yb == rb).float().mean()) > 0.98


@pytest.mark.parametrize("tokens", [5, 80])
def test_fused_moe_layer_and_align(tokens):
    """The host mirror of the reference's fused MoE layer: both branches (per-pair op for few tokens, expert-sorted blocks
    above 64 tokens) against a per-pair loop over the oracle; `moe_align_block_size` against the plain-Python layout."""
    from kaillm_b200 import linear
    qt1, qt2, e, hidden, inter, top_k = 12, 14, 4, 256, 256, 2
    w1, w1t = experts_wire(qt1, e, 2 * inter, hidden, seed=1)
    w2, w2t = experts_wire(qt2, e, hidden, inter, seed=2)
    x, xt = act(tokens, hidden, seed=3, dt="f32")
    ids = routing(tokens, top_k, e, seed=4)
    idt = torch.from_numpy(ids).to(dev())
    tw = torch.rand((tokens, top_k), device=dev())
    s, ex, tot = linear.moe_align_block_size(idt, 8, e)
    ws, wex, wtot = align(ids, 8, e)
    n = int(tot.item())
    assert n == int(wtot[0]) and np.array_equal(s[:n].cpu().numpy(), ws) and np.array_equal(ex[:n // 8].cpu().numpy(), wex)
    assert bool((s[n:] == tokens * top_k).all()) and bool((ex[n // 8:] == -1).all())   # unused blocks: no expert
    y = linear.fused_moe_gguf(xt, w1t, w2t, tw, idt, qt1, qt2)
    flavour = "mmq" if tokens > 64 else "mmvq"
    h1 = expected(w1, qt1, x, ids, flavour)
    a = h1[:, :inter] / (1 + np.exp(-h1[:, :inter])) * h1[:, inter:]
    h2 = np.stack([O.mul_mat(w2[int(ids.reshape(-1)[z])], qt2, a[z:z + 1].astype(np.float32), flavour)[0]
                   for z in range(tokens * top_k)])
    want = (h2.reshape(tokens, top_k, hidden) * tw.cpu().numpy()[:, :, None]).sum(1)
    assert rel_l2(to_np(y), want) < 2e-4            # the activation between the projections is fp32 on both sides
