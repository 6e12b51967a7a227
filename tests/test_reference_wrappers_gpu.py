"""The reference's own Python layer, unmodified, on top of this repository's `_C_gguf` module.

`oracle/stage_ref.py` copies the reference's `vllm_gguf_plugin` package (Python files only) and its gguf-reader
package into the git-ignored directory baseline/_ref/.  Here that package is imported as it stands, with this
repository's extension made importable as `vllm_gguf_plugin._C_gguf` (the module the reference imports at
vllm_gguf_plugin/ops.py:42-48), and driven through its public entry points:

  * `vllm_gguf_plugin.ops.ggml_dequantize / ggml_mul_mat_vec_a8 / ggml_mul_mat_a8`      (ops.py:181-208)
  * `torch.ops.vllm._fused_mul_mat_gguf`, every (type, M, N) regime                      (quantization/linear.py:40-63)
  * `GGUFLinearMethod.apply`: plain, merged same-type, merged mixed-type, bias           (quantization/linear.py:341-407)
  * `torch.ops.vllm._apply_gguf_embedding`                                               (quantization/vocal_embeds.py:29-58)

Results are checked against the CPU oracle, against the reference's own CUDA build (`_C_gguf_ref`) where it is
present, and this repository's mirror of the dispatch (`kaillm_b200.linear`) is checked against the original
decision for decision.  Everything is skipped when the staging directory is absent.
"""
import os
import sys
import types

import numpy as np
import pytest
import torch

from kaillm_b200 import capi, linear as kq_linear, synth
from oracle import gguf_oracle as O
from tests.gpu_util import TDT, act, dev, rel_l2, to_np, wire

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STAGE = os.path.join(ROOT, "baseline", "_ref")
ALL_TYPES = [2, 8, 10, 12, 14, 21, 3, 6, 7, 11, 13, 20, 23]


@pytest.fixture(scope="module")
def plugin():
    if not os.path.exists(os.path.join(STAGE, "vllm_gguf_plugin", "ops.py")):
        pytest.skip("baseline/_ref is not staged (python oracle/stage_ref.py needs the reference tree)")
    pytest.importorskip("vllm")
    if STAGE not in sys.path:
        sys.path.insert(0, STAGE)
    os.environ["VLLM_GGUF_USE_CUDA"] = "1"
    import vllm_gguf_plugin

    assert os.path.realpath(vllm_gguf_plugin.__file__).startswith(os.path.realpath(STAGE))
    pkg_dir = os.path.join(ROOT, "kaillm_b200")        # holds _C_gguf.so: found by `from . import _C_gguf`
    if pkg_dir not in vllm_gguf_plugin.__path__:
        vllm_gguf_plugin.__path__.append(pkg_dir)
    from vllm_gguf_plugin import ops as ref_py_ops
    from vllm_gguf_plugin.quantization import linear as ref_linear
    from vllm_gguf_plugin.quantization import vocal_embeds as ref_embed

    assert ref_py_ops._CUDA_AVAILABLE and ref_py_ops._CUDA_ENABLED, "the reference wrapper did not pick up _C_gguf"
    so = os.path.realpath(sys.modules["vllm_gguf_plugin._C_gguf"].__file__)
    assert so == os.path.realpath(os.path.join(pkg_dir, "_C_gguf.so")), so
    return types.SimpleNamespace(ops=ref_py_ops, linear=ref_linear, embed=ref_embed)


@pytest.fixture(scope="module")
def ref_cuda():
    """torch.ops._C_gguf_ref (the reference's own CUDA build) or None when it was not built."""
    path = os.path.join(ROOT, "oracle", "_ref", "_C_gguf_ref.so")
    if not os.path.exists(path):
        return None
    if not hasattr(torch.ops, "_C_gguf_ref") or not hasattr(torch.ops._C_gguf_ref, "ggml_dequantize"):
        torch.ops.load_library(path)
    return torch.ops._C_gguf_ref


def _flavour(qt, m, n):
    """Which branch quantization/linear.py:40-63 takes."""
    imatrix = qt in (20, 21, 23)
    safe = (8 if n > 5120 else 16) if imatrix else (2 if n > 5120 else 6)
    if m <= safe:
        return "mmvq"
    return "dense" if imatrix else "mmq"


def _expect(w, qt, x, xdt, flavour):
    if flavour == "dense":
        deq = O.dequantize(w, qt, xdt, half_fma=capi.get_option("half_fma"))
        return x.astype(np.float64) @ deq.astype(np.float64).T
    return O.mul_mat(w, qt, x, flavour)


# ------------------------------------------------------------------ ops.py wrappers
@pytest.mark.parametrize("qt", ALL_TYPES)
def test_reference_ops_wrappers(plugin, qt):
    n, k, m = 192, 1024, 3
    w, wt = wire(qt, n, k, seed=qt)
    x, xt = act(m, k, seed=3, dt="bf16")
    y = plugin.ops.ggml_mul_mat_vec_a8(wt, xt, qt, n)
    assert y.shape == (m, n) and y.dtype == torch.bfloat16
    assert rel_l2(to_np(y), O.round_to_dtype(O.mul_mat(w, qt, x, "mmvq"), "bf16")) < 3e-3
    if qt not in (20, 21, 23):
        y = plugin.ops.ggml_mul_mat_a8(wt, xt, qt, n)
        assert rel_l2(to_np(y), O.round_to_dtype(O.mul_mat(w, qt, x, "mmq"), "bf16")) < 3e-3
    d = plugin.ops.ggml_dequantize(wt, qt, n, k, torch.float16)
    assert d.shape == (n, k)
    np.testing.assert_array_equal(to_np(d), O.dequantize(w, qt, "f16", half_fma=capi.get_option("half_fma")))


# ------------------------------------------------------------------ _fused_mul_mat_gguf, every regime
@pytest.mark.parametrize("qt", ALL_TYPES)
@pytest.mark.parametrize("n", [5120, 5128])
@pytest.mark.parametrize("m", [1, 2, 3, 6, 7, 8, 9, 16, 17, 80, 130])
def test_fused_mul_mat_gguf_regimes(plugin, ref_cuda, qt, n, m):
    k = 512
    w, wt = wire(qt, n, k, seed=qt + n)
    x, xt = act(m, k, seed=m, dt="f16")
    flavour = _flavour(qt, m, n)
    y = torch.ops.vllm._fused_mul_mat_gguf(xt, wt, qt)
    assert y.shape == (m, n) and y.dtype == torch.float16
    got = to_np(y)
    want = _expect(w, qt, x, "f16", flavour)
    # fp16 outputs: 2^-11 relative rounding per element on top of the arithmetic
    assert rel_l2(got, want) < (1.2e-3 if flavour == "dense" or m > 80 else 6e-4), (flavour, rel_l2(got, want))
    # this repository's mirror takes the same branch and gives the same bits
    assert torch.equal(kq_linear.fused_mul_mat_gguf(xt, wt, qt), y)
    # the reference's own CUDA kernels on the same inputs
    if ref_cuda is not None:
        if flavour == "mmvq":
            yr = ref_cuda.ggml_mul_mat_vec_a8(wt, xt, qt, n)
        elif flavour == "mmq":
            yr = ref_cuda.ggml_mul_mat_a8(wt, xt, qt, n)
        else:
            yr = xt @ ref_cuda.ggml_dequantize(wt, qt, n, k, xt.dtype).T
        assert rel_l2(got, to_np(yr)) < 1.2e-3


def test_fused_mul_mat_gguf_empty_batch(plugin):
    _, wt = wire(12, 64, 512, seed=1)
    xt = torch.empty((0, 512), dtype=torch.bfloat16, device=dev())
    y = torch.ops.vllm._fused_mul_mat_gguf(xt, wt, 12)
    assert y.shape == (0, 64)
    assert kq_linear.fused_mul_mat_gguf(xt, wt, 12).shape == (0, 64)


@pytest.mark.parametrize("qt,n,k", [(21, 17408, 5120), (21, 8192, 2048)])
@pytest.mark.parametrize("m", [16, 80])
def test_iq3s_verify_shapes_through_the_op_api(plugin, qt, n, k, m):
    """IQ3_S above the vector threshold is dequantize + dense matmul in the reference's dispatch
    (quantization/linear.py:55-59); the dense weight must be bit-exact and the product within the gate."""
    _, wt = wire(qt, n, k, seed=5)
    x, xt = act(m, k, seed=m, dt="bf16")
    w = wt.cpu().numpy()
    rows = np.r_[0:48, n - 48:n]
    y = torch.ops.vllm._fused_mul_mat_gguf(xt, wt, qt)
    deq = O.dequantize(w[rows], qt, "bf16", half_fma=capi.get_option("half_fma"))
    want = x.astype(np.float64) @ deq.astype(np.float64).T
    assert rel_l2(to_np(y)[:, rows], want) < 4e-3          # bf16 outputs of a K=5120 dense product
    d = plugin.ops.ggml_dequantize(wt, qt, n, k, torch.bfloat16)
    np.testing.assert_array_equal(to_np(d)[rows], deq)


# ------------------------------------------------------------------ GGUFLinearMethod.apply
class _Layer:
    pass


def _make_layer(shards, merged_ids=None):
    """shards: list of (wire tensor, type).  A stand-in for what create_weights + process_weights_after_loading leave
    on a vLLM linear layer: `qweight` (rows of all shards, padded to the widest row) with shard_id / shard_offset_map,
    `qweight_type` with weight_type / shard_weight_type."""
    layer = _Layer()
    width = max(w.shape[1] for w, _ in shards)
    rows = sum(w.shape[0] for w, _ in shards)
    data = torch.zeros((rows, width), dtype=torch.uint8, device=dev())
    offs, r = {}, 0
    ids = merged_ids if merged_ids is not None else []
    for i, (w, t) in enumerate(shards):
        data[r:r + w.shape[0], :w.shape[1]] = w
        if ids:
            offs[ids[i]] = (r, r + w.shape[0], w.shape[1])
        r += w.shape[0]
    qweight = torch.nn.Parameter(data, requires_grad=False)
    qweight.shard_id = list(ids)
    qweight.shard_offset_map = offs
    qtype = torch.nn.Parameter(torch.zeros(max(1, len(shards)), dtype=torch.uint8), requires_grad=False)
    qtype.weight_type = shards[0][1]
    qtype.shard_weight_type = {ids[i]: t for i, (_, t) in enumerate(shards)} if ids else {}
    layer.qweight, layer.qweight_type = qweight, qtype
    return layer


@pytest.mark.parametrize("m", [1, 4, 16, 90])
@pytest.mark.parametrize("case", ["plain", "qkv_same", "gate_up_same", "qkv_mixed", "gate_up_mixed"])
@pytest.mark.parametrize("with_bias", [False, True])
def test_linear_method_apply(plugin, case, m, with_bias):
    k = 1024
    spec = {
        "plain": ([(12, 320)], None),
        "qkv_same": ([(8, 256), (8, 64), (8, 64)], ["q", "k", "v"]),
        "gate_up_same": ([(12, 384), (12, 384)], [0, 1]),
        "qkv_mixed": ([(12, 256), (14, 64), (8, 64)], ["q", "k", "v"]),
        "gate_up_mixed": ([(12, 384), (10, 384)], [0, 1]),
    }[case]
    types_n, ids = spec
    shards_np, shards_t = [], []
    for i, (qt, n) in enumerate(types_n):
        w, wt = wire(qt, n, k, seed=100 + i)
        shards_np.append((w, qt))
        shards_t.append((wt, qt))
    x, xt = act(m, k, seed=m, dt="bf16")
    ntot = sum(n for _, n in types_n)
    bias_np = np.linspace(-1.0, 1.0, ntot, dtype=np.float32)
    bias = torch.from_numpy(bias_np).to(torch.bfloat16).to(dev()) if with_bias else None
    layer = _make_layer(shards_t, ids)
    method = plugin.linear.GGUFLinearMethod(quant_config=None)
    y = method.apply(layer, xt, bias)
    assert y.shape == (m, ntot) and y.dtype == torch.bfloat16
    # expected: per shard, the flavour the dispatch picks for the tensor it is called with
    same = len({t for _, t in shards_np}) == 1
    parts = []
    if same:
        wcat = np.concatenate([w for w, _ in shards_np], axis=0)
        parts.append(O.mul_mat(wcat, shards_np[0][1], x, _flavour(shards_np[0][1], m, ntot)))
    else:
        for w, qt in shards_np:
            parts.append(O.mul_mat(w, qt, x, _flavour(qt, m, w.shape[0])))
    want = O.round_to_dtype(np.concatenate(parts, axis=1), "bf16")
    if with_bias:
        want = O.round_to_dtype(want + O.round_to_dtype(bias_np, "bf16")[None, :], "bf16")
    assert rel_l2(to_np(y), want) < 4e-3
    # this repository's mirror of apply gives the same bits
    mine = kq_linear.GGUFLinear(shards_t).apply(xt, bias)
    assert torch.equal(mine, y)


# ------------------------------------------------------------------ embedding caller
@pytest.mark.parametrize("qt", [8, 2, 10, 21])
def test_reference_embedding_over_the_dequantize_op(plugin, qt):
    """`_apply_gguf_embedding` gathers rows of the wire tensor and calls ggml_dequantize on them (K-quants other than
    Q2_K/Q3_K take the reference's Triton decoder and never reach this library)."""
    vocab, hidden = 300, 1024
    w, wt = wire(qt, vocab, hidden, seed=9)
    ids = torch.tensor([[5, 299, 0], [17, 5, 123]], dtype=torch.long, device=dev())
    out = torch.ops.vllm._apply_gguf_embedding(ids, wt, qt, hidden, torch.float16)
    assert out.shape == (2, 3, hidden) and out.dtype == torch.float16
    want = O.dequantize(w[ids.flatten().cpu().numpy()], qt, "f16", half_fma=capi.get_option("half_fma"))
    np.testing.assert_array_equal(to_np(out).reshape(-1, hidden), want)


# ------------------------------------------------------------------ mixture-of-experts wrappers
@pytest.mark.parametrize("qt", [12, 14, 8, 21])
def test_reference_moe_wrappers_reach_this_library(plugin, qt):
    """`ops.ggml_moe_a8_vec / ggml_moe_a8 / ggml_moe_get_block_size` (vllm_gguf_plugin/ops.py:211-284) take their CUDA
    branch on this repository's `_C_gguf` and return the oracle's per-pair results."""
    e, n, k, tokens, top_k = 4, 64, 512, 9, 2
    w = np.stack([synth.wire_numpy(qt, n, k, seed=qt + i) for i in range(e)])
    wt = torch.from_numpy(w).to(dev())
    x, xt = act(tokens, k, seed=31, dt="bf16")
    rng = np.random.default_rng(qt)
    ids = np.stack([rng.choice(e, size=top_k, replace=False) for _ in range(tokens)]).astype(np.int32)
    idt = torch.from_numpy(ids).to(dev())
    y = plugin.ops.ggml_moe_a8_vec(xt, wt, idt, top_k, qt, n, tokens)
    want = np.stack([O.mul_mat(w[int(ids.reshape(-1)[z])], qt, x[z // top_k:z // top_k + 1], "mmvq")[0] for z in range(tokens * top_k)])
    assert y.dtype == torch.bfloat16 and rel_l2(to_np(y), want) < 5e-3
    if qt in (12, 14, 8):
        bs = plugin.ops.ggml_moe_get_block_size(qt)
        assert bs == capi.lib.kq_moe_block_size(qt) == 8
        s, ex, tot = kq_linear.moe_align_block_size(idt, bs, e)
        yb = plugin.ops.ggml_moe_a8(xt, wt, s, ex, tot, qt, n, top_k, tokens)
        wantb = np.stack([O.mul_mat(w[int(ids.reshape(-1)[z])], qt, x[z // top_k:z // top_k + 1], "mmq")[0] for z in range(tokens * top_k)])
        assert rel_l2(to_np(yb), wantb) < 5e-3
