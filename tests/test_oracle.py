"""CPU tests of the oracle: against the reference gguf-reader fixtures and its own invariants."""
import os

import numpy as np
import pytest

from kaillm_b200 import synth
from oracle import gguf_oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
QT = O.QTYPES
ALL = O.ALL_QTYPES


@pytest.mark.parametrize("qt", ALL)
def test_dequantize_matches_reference_reader_fixture(qt):
    g = np.load(os.path.join(GOLD, "reader_dequant.npz"))
    w, ref = g[f"wire_{qt}"], g[f"deq_{qt}"]
    np.testing.assert_array_equal(synth.wire_numpy(qt, 6, ref.shape[1], seed=100 + qt), w)  # generator is stable
    mine = O.dequantize_f32(w, qt, iq3s_top=60)
    np.testing.assert_array_equal(mine, ref)


def test_iq3s_cuda_grid_differs_only_on_top_level():
    g62, g60 = O.iq3s_grid(62), O.iq3s_grid(60)
    assert g62.shape == (512, 4)
    diff = g62 != g60
    assert diff.any() and set(np.unique(g62[diff])) == {62} and set(np.unique(g60[diff])) == {60}
    assert int(diff.any(axis=1).sum()) == 146  # entries holding the top level
    assert set(np.unique(g62)) == {4, 12, 20, 28, 36, 44, 52, 62}


def test_q8_1_basic_properties():
    x = synth.activations_numpy(3, 700, seed=3)
    a = O.quantize_q8_1(x)
    assert a["kpad"] == 1024 and a["q"].shape == (3, 1024)
    assert not a["q"][:, 700:].any()                       # zero padding
    assert not a["d"][:, 22:].any() and not a["s"][:, 22:].any()
    assert np.abs(a["q"]).max() == 127
    # every block reaches +-127 at its amax position
    qb = a["q"][:, :672].reshape(3, 21, 32)
    assert (np.abs(qb).max(-1) == 127).all()
    # dequantized activations are within half a step (plus the fp16 rounding of d itself: 127 * d * 2^-11)
    d = np.repeat(a["d"][:, :22].astype(np.float32), 32, 1)
    err = np.abs(x - (a["q"][:, :704] * d)[:, :700])
    assert (err <= (0.5 + 127 * 2.0 ** -11) * d[:, :700] * 1.001 + 1e-7).all()


def test_q8_1_zero_block_and_ties():
    x = np.zeros((1, 64), np.float32)
    x[0, 32:] = np.linspace(-127, 127, 32, dtype=np.float32)   # d == 1 exactly
    x[0, 33] = 2.5                                             # tie -> away from zero
    x[0, 34] = -2.5
    a = O.quantize_q8_1(x)
    assert not a["q"][0, :32].any() and a["d"][0, 0] == 0 and a["s"][0, 0] == 0
    assert a["d"][0, 1] == np.float16(1.0)
    assert a["q"][0, 33] == 3 and a["q"][0, 34] == -3


def test_q8_1_sum_is_butterfly_order_and_fp16():
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((1, 32)) * 1000).astype(np.float32)
    a = O.quantize_q8_1(x)
    t = x[0].copy()
    for m in (16, 8, 4, 2, 1):
        t = (t + t[np.arange(32) ^ m]).astype(np.float32)
    assert a["s"][0, 0] == np.float16(t[0])
    big = np.full((1, 32), 3000.0, np.float32)                 # 32*3000 > 65504 -> fp16 sum overflows, as in the reference
    assert np.isinf(O.quantize_q8_1(big)["s"][0, 0])


def test_q8_1_wire_layout():
    x = synth.activations_numpy(2, 512, seed=9)
    a = O.quantize_q8_1(x)
    w = O.q8_1_wire(a)
    assert w.shape == (2, 16, 36)
    assert np.array_equal(w[1, 3, 4:].view(np.int8), a["q"][1, 96:128])
    assert w[1, 3, 0:2].view(np.float16)[0] == a["d"][1, 3]
    assert w[1, 3, 2:4].view(np.float16)[0] == a["s"][1, 3]


@pytest.mark.parametrize("qt", O.MORE_QTYPES)
def test_more_formats_equal_dense_product_of_dequantized_operands(qt):
    """The same identity for the other formats.  Where the reference uses the fp16 raw block sum (Q5_0's MMVQ
    flavour, Q5_K's MMQ flavour) or rounds scale products to fp16 (Q4_1, Q5_1) the agreement is to that effect."""
    k = 1024
    w = synth.wire_numpy(qt, 24, k, seed=qt)
    x = synth.activations_numpy(5, k, seed=qt, dtype="bf16")
    a = O.quantize_q8_1(x)
    xq = a["q"][:, :k].astype(np.float64) * np.repeat(a["d"][:, : k // 32].astype(np.float64), 32, 1)
    dense = xq @ O.dequantize_f32(w, qt).astype(np.float64).T
    rel = lambda y: np.linalg.norm(y - dense) / np.linalg.norm(dense)   # noqa: E731
    y = O.mul_mat(w, qt, x, "mmvq")
    if qt in (O.Q4_1, O.Q5_1):
        assert rel(y) < 3e-2               # m * (raw fp16 sum) instead of m * d8 * (sum of codes), fp16 products
    elif qt == O.Q5_0:
        assert rel(y) < 3e-2               # -16 through the raw fp16 sum
    else:
        assert rel(y) < 1e-6
    if qt in O.NO_MMQ:
        with pytest.raises(ValueError):
            O.mul_mat(w, qt, x, "mmq")
    else:
        y2 = O.mul_mat(w, qt, x, "mmq")
        if qt == O.Q5_0:
            assert rel(y2) < 1e-6          # the MMQ tile loader subtracts 16 from the codes: exact
        elif qt == O.Q5_K:
            assert 1e-7 < rel(y2) < 5e-3   # raw-sum min term
        elif qt == O.Q3_K:
            assert rel(y2) < 1e-6
        else:
            np.testing.assert_array_equal(y2, y)


@pytest.mark.parametrize("qt", QT)
def test_mul_mat_equals_dense_product_of_dequantized_operands(qt):
    """The integer-dot formulation is algebraically the dense product of the dequantized weight with the
    dequantized q8_1 activations (except Q4_0 and MMQ-Q4_K, which use the raw fp16 block sum)."""
    k = 1024
    w = synth.wire_numpy(qt, 24, k, seed=qt)
    x = synth.activations_numpy(5, k, seed=qt, dtype="bf16")
    y = O.mul_mat(w, qt, x, "mmvq")
    a = O.quantize_q8_1(x)
    xq = a["q"][:, :k].astype(np.float64) * np.repeat(a["d"][:, : k // 32].astype(np.float64), 32, 1)
    dense = xq @ O.dequantize_f32(w, qt).astype(np.float64).T
    rel = np.linalg.norm(y - dense) / np.linalg.norm(dense)
    if qt == O.Q4_0:
        assert rel < 3e-2          # raw-sum min term: differs by the activation quantization error
    else:
        assert rel < 1e-6
    if qt != O.IQ3_S:
        y2 = O.mul_mat(w, qt, x, "mmq")
        rel2 = np.linalg.norm(y - y2) / np.linalg.norm(y)
        assert rel2 < (5e-3 if qt == O.Q4_K else 1e-6)
    else:
        with pytest.raises(ValueError):
            O.mul_mat(w, qt, x, "mmq")


@pytest.mark.parametrize("qt", ALL)
def test_group_dots_shapes_and_linearity(qt):
    k = 512
    w = synth.wire_numpy(qt, 8, k, seed=1)
    x = synth.activations_numpy(2, k, seed=2)
    y, act, I, S = O.mul_mat(w, qt, x, "mmvq", return_parts=True)
    g = O.GROUP[qt]
    assert I.shape == (2, 8, k // g) and S.shape == (2, k // g)
    np.testing.assert_array_equal(S, act["q"][:, :k].astype(np.int64).reshape(2, k // g, g).sum(-1))
    # doubling the activations leaves the codes unchanged and doubles d (power of two) -> y doubles exactly
    y2 = O.mul_mat(w, qt, 2 * x, "mmvq")
    if qt in (O.Q4_1, O.Q5_1):   # their fp16 scale products can be subnormal, where rounding is not scale-invariant
        assert np.linalg.norm(y2 - 2 * y) / np.linalg.norm(y) < 1e-3
    else:
        np.testing.assert_allclose(y2, 2 * y, rtol=1e-6)


@pytest.mark.parametrize("qt", ALL)
@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
def test_dequantize_half_path_close_to_f32_and_representable(qt, dt):
    w = synth.wire_numpy(qt, 16, 512, seed=qt + 7)
    d = O.dequantize(w, qt, dt)
    f = O.dequantize_f32(w, qt)
    rel = np.linalg.norm(d - f) / np.linalg.norm(f)
    assert rel < (6e-3 if dt == "bf16" else 1e-3)
    np.testing.assert_array_equal(O.round_to_dtype(d, dt), d)


def test_dequantize_fma_mode_changes_only_kquants_with_min():
    for qt in ALL:
        w = synth.wire_numpy(qt, 16, 512, seed=3)
        a, b = O.dequantize(w, qt, "f16", half_fma=0), O.dequantize(w, qt, "f16", half_fma=1)
        if qt in (O.Q2_K, O.Q4_K, O.Q5_K, O.Q4_1, O.Q5_1):
            assert (a != b).any()
        else:
            np.testing.assert_array_equal(a, b)


def test_row_bytes_and_errors():
    assert O.row_bytes(O.Q4_K, 5120) == 2880 and O.row_bytes(O.Q6_K, 17408) == 14280
    assert O.row_bytes(O.Q8_0, 5120) == 5440 and O.row_bytes(O.IQ3_S, 5120) == 2200
    with pytest.raises(ValueError):
        O.row_bytes(O.Q4_K, 5000)
    with pytest.raises(ValueError):
        O.unpack(np.zeros((1, 18), np.uint8), 16)
