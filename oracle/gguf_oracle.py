"""CPU restatement of the GGUF block-quantized linear path (TEST INFRASTRUCTURE ONLY).

This module is the checker for the CUDA kernels, never the product: only the
test-suite, the smoke check and the CPU-baseline leg of the benchmark may import
it.  It restates, in numpy, the arithmetic of the reference's `_C_gguf` ops for
Q4_0, Q8_0, Q2_K, Q4_K, Q6_K and IQ3_S weights:

* `quantize_q8_1`      - activation quantizer
                         (vllm_gguf_plugin/csrc/gguf/gguf_kernel.cu:32-85)
* `unpack`             - wire bytes -> integer codes + scales
                         (vllm_gguf_plugin/csrc/gguf/ggml-common.h:20-150)
* `subblock_dots`      - exact integer dot products per scale group
* `mul_mat`            - fp combine of the integer dots, in the two flavours the
                         reference has: "mmvq" (vecdotq.cuh:46-66, 165-177,
                         204-230, 328-351, 447-465, 1649-1672) and "mmq"
                         (vecdotq.cuh:232-263, 353-379, 467-491)
* `dequantize`         - `ggml_dequantize` with its fp16 intermediate roundings
                         (vllm_gguf_plugin/csrc/gguf/dequantize.cuh:3-16, 69-78,
                         101-121, 156-196, 232-256, 334-353)
* `dequantize_f32`     - plain fp32 dequantization, the arithmetic of
                         gguf-reader/gguf/quants.py (used for the CPU baseline
                         and for cross-checking `unpack` against gguf-reader)

Parity status: the reference ships no test, golden vector or fixture for this
path, so the restatement is pinned two other ways: `dequantize_f32` is compared
with the reference's own gguf-reader (imported where the reference tree is
present; committed fixtures elsewhere), and every function here is compared on
the GPU box with the reference's own `_C_gguf` extension built unmodified from
its sources (oracle/build_ref.py).

IQ3_S note: the reference's CUDA table (ggml-common.h:685) has top level 62
where gguf-reader's has 60 (=4*15) and its scale is d*(0.5+s)*0.5 on 4x-scaled
grid bytes; the CUDA semantics are the parity target (`iq3s_top=62`).
"""
from __future__ import annotations

import numpy as np

Q4_0, Q8_0, Q2_K, Q4_K, Q6_K, IQ3_S = 2, 8, 10, 12, 14, 21
Q4_1, Q5_0, Q5_1, Q3_K, Q5_K, IQ4_NL, IQ4_XS = 3, 6, 7, 11, 13, 20, 23
QTYPES = (Q4_0, Q8_0, Q2_K, Q4_K, Q6_K, IQ3_S)                       # the benchmark's six formats
MORE_QTYPES = (Q4_1, Q5_0, Q5_1, Q3_K, Q5_K, IQ4_NL, IQ4_XS)         # the other formats of real mixed checkpoints
ALL_QTYPES = QTYPES + MORE_QTYPES
NAMES = {Q4_0: "Q4_0", Q8_0: "Q8_0", Q2_K: "Q2_K", Q4_K: "Q4_K", Q6_K: "Q6_K", IQ3_S: "IQ3_S", Q4_1: "Q4_1",
         Q5_0: "Q5_0", Q5_1: "Q5_1", Q3_K: "Q3_K", Q5_K: "Q5_K", IQ4_NL: "IQ4_NL", IQ4_XS: "IQ4_XS"}
# (weights per block, bytes per block) - gguf-reader/gguf/constants.py:5958
BLOCK = {Q4_0: (32, 18), Q8_0: (32, 34), Q2_K: (256, 84), Q4_K: (256, 144), Q6_K: (256, 210), IQ3_S: (256, 110),
         Q4_1: (32, 20), Q5_0: (32, 22), Q5_1: (32, 24), Q3_K: (256, 110), Q5_K: (256, 176), IQ4_NL: (32, 18),
         IQ4_XS: (256, 136)}
# weights per integer-dot group (one weight-side scale per group)
GROUP = {Q4_0: 32, Q8_0: 32, Q2_K: 16, Q4_K: 32, Q6_K: 16, IQ3_S: 32, Q4_1: 32, Q5_0: 32, Q5_1: 32, Q3_K: 16, Q5_K: 32,
         IQ4_NL: 32, IQ4_XS: 32}
# types without an MMQ kernel in the reference (quantization/utils.py: MMQ_QUANT_TYPES has no i-matrix formats)
NO_MMQ = (IQ3_S, IQ4_NL, IQ4_XS)
# the 16 code values of IQ4_NL / IQ4_XS (ggml-common.h:1060)
KVALUES_IQ4NL = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.int16)


def row_bytes(qtype: int, k: int) -> int:
    blk, nb = BLOCK[qtype]
    if k % blk:
        raise ValueError(f"K={k} is not a multiple of the {NAMES[qtype]} block ({blk})")
    return k // blk * nb


# ----------------------------------------------------------------------------
# IQ3_S codebook: 512 entries x 4 levels (3 bits each), stored as 12-bit codes.
# ----------------------------------------------------------------------------
def _load_iq3s_codes() -> np.ndarray:
    import os
    here = os.path.dirname(os.path.abspath(__file__))
    path = os.path.join(here, "..", "kaillm_b200", "csrc", "kq_iq3s_codes.inc")
    txt = open(path).read()
    vals = [int(t, 16) for t in txt.replace("\n", " ").split(",") if t.strip().startswith("0x")]
    assert len(vals) == 512
    return np.array(vals, dtype=np.uint16)


_IQ3S_CODES = None


def iq3s_grid(top: int = 62) -> np.ndarray:
    """[512,4] uint8 grid bytes: level l<7 -> 8l+4, level 7 -> `top` (62 CUDA, 60 gguf-reader)."""
    global _IQ3S_CODES
    if _IQ3S_CODES is None:
        _IQ3S_CODES = _load_iq3s_codes()
    lv = np.stack([(_IQ3S_CODES >> (3 * j)) & 7 for j in range(4)], axis=1).astype(np.int32)
    g = 8 * lv + 4
    g[lv == 7] = top
    return g.astype(np.uint8)


# ----------------------------------------------------------------------------
# rounding helpers
# ----------------------------------------------------------------------------
def f2h(x) -> np.ndarray:
    """Round to fp16 (nearest-even) from an exactly held value (float64 in)."""
    with np.errstate(over="ignore"):
        return np.asarray(x, dtype=np.float64).astype(np.float16)


def h2d(x) -> np.ndarray:
    return np.asarray(x).astype(np.float64)


def hmul(a, b):
    """fp16 * fp16 -> fp16, one rounding (the product is exact in float64)."""
    return f2h(h2d(a) * h2d(b))


def hsub(a, b):
    return f2h(h2d(a) - h2d(b))


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_to_dtype(y: np.ndarray, dtype: str) -> np.ndarray:
    """Round fp32 values to `dtype` ("f32" | "f16" | "bf16") and return them as fp32."""
    y = np.asarray(y, dtype=np.float32)
    if dtype == "f32":
        return y
    if dtype == "f16":
        with np.errstate(over="ignore"):
            return y.astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        return bf16_bits_to_f32(f32_to_bf16_bits(y))
    raise ValueError(dtype)


# ----------------------------------------------------------------------------
# q8_1 activation quantizer  (gguf_kernel.cu:32-85)
# ----------------------------------------------------------------------------
def quantize_q8_1(x: np.ndarray) -> dict:
    """x: [M,K] float32 (already converted from its storage dtype).

    Returns q int8 [M,Kpad], d fp16 [M,Kpad/32], s fp16 [M,Kpad/32] with
    Kpad = ceil(K/512)*512; positions >= K are zero.  d = amax/127 (fp32
    division), q = roundf(x/d) (half away from zero), s = fp16 of the fp32 sum
    taken in the xor-butterfly order 16,8,4,2,1.
    """
    x = np.asarray(x, dtype=np.float32)
    m, k = x.shape
    kpad = (k + 511) // 512 * 512
    xp = np.zeros((m, kpad), dtype=np.float32)
    xp[:, :k] = x
    xb = xp.reshape(m, kpad // 32, 32)
    amax = np.abs(xb).max(axis=-1)
    t = xb.copy()
    lane = np.arange(32)
    for mask in (16, 8, 4, 2, 1):
        t = (t + t[..., lane ^ mask]).astype(np.float32)
    ssum = t[..., 0]
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        v = (xb / d[..., None]).astype(np.float32)
    v64 = v.astype(np.float64)
    r = np.trunc(v64 + np.copysign(0.5, v64))
    r = np.where(amax[..., None] == 0, 0.0, r)
    q = r.astype(np.int32).astype(np.int8).reshape(m, kpad)
    with np.errstate(over="ignore"):
        return {"q": q, "d": d.astype(np.float16), "s": ssum.astype(np.float16), "kpad": kpad}


def q8_1_wire(act: dict) -> np.ndarray:
    """The reference scratch layout: [M, Kpad/32, 36] bytes = {half d, half s, int8 q[32]}."""
    q, d, s = act["q"], act["d"], act["s"]
    m, kpad = q.shape
    out = np.empty((m, kpad // 32, 36), dtype=np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(m, -1, 2)
    out[..., 2:4] = s.view(np.uint8).reshape(m, -1, 2)
    out[..., 4:] = q.view(np.uint8).reshape(m, -1, 32)
    return out


# ----------------------------------------------------------------------------
# wire format -> integer codes and scales  (ggml-common.h:20-150)
# ----------------------------------------------------------------------------
def _blocks(wire: np.ndarray, qtype: int):
    wire = np.ascontiguousarray(wire, dtype=np.uint8)
    n, rb = wire.shape
    if qtype not in BLOCK:
        raise ValueError(f"unsupported GGML type {qtype}")
    blk, nb = BLOCK[qtype]
    if rb % nb:
        raise ValueError("row bytes not a multiple of the block size")
    return wire.reshape(n, rb // nb, nb), n, rb // nb


def _h(b: np.ndarray) -> np.ndarray:
    """two bytes (last axis) -> fp16"""
    return np.ascontiguousarray(b).view(np.float16)[..., 0]


def q4k_scale_min(sc12: np.ndarray):
    """12 packed bytes -> (sc[8], m[8]) 6-bit each (dequantize.cuh:156-163)."""
    q = sc12.astype(np.int32)
    sc = np.empty(q.shape[:-1] + (8,), np.int32)
    mn = np.empty_like(sc)
    for j in range(8):
        if j < 4:
            sc[..., j] = q[..., j] & 63
            mn[..., j] = q[..., j + 4] & 63
        else:
            sc[..., j] = (q[..., j + 4] & 15) | ((q[..., j - 4] >> 6) << 4)
            mn[..., j] = (q[..., j + 4] >> 4) | ((q[..., j] >> 6) << 4)
    return sc, mn


def unpack(wire: np.ndarray, qtype: int, iq3s_top: int = 62) -> dict:
    """Decode wire bytes [N,rowbytes] to integer codes and scales.

    Returns a dict with
      q    int16 [N,K]      integer code in the dot domain (Q4_0: 0..15, Q8_0: int8,
                            Q2_K: 0..3, Q4_K: 0..15, Q6_K: -32..31, IQ3_S: +-grid byte)
      d    fp16  [N,K/blk]  block scale; dmin likewise for Q2_K/Q4_K
      sc   int32 [N,K/G]    integer group scale (Q2_K 0..15, Q4_K 0..63, Q6_K int8, IQ3_S 0..15)
      mn   int32 [N,K/G]    integer group min (Q2_K, Q4_K)
    """
    b, n, nblk = _blocks(wire, qtype)
    out = {"qtype": qtype}
    if qtype == Q4_0:
        out["d"] = _h(b[..., 0:2])
        qs = b[..., 2:18].astype(np.int16)
        out["q"] = np.concatenate([qs & 15, qs >> 4], axis=-1).reshape(n, -1)
    elif qtype == Q8_0:
        out["d"] = _h(b[..., 0:2])
        out["q"] = b[..., 2:34].view(np.int8).astype(np.int16).reshape(n, -1)
    elif qtype == Q2_K:
        scales = b[..., 0:16].astype(np.int32)
        qs = b[..., 16:80].astype(np.int16).reshape(n, nblk, 2, 32)
        out["d"] = _h(b[..., 80:82])
        out["dmin"] = _h(b[..., 82:84])
        q = np.stack([(qs >> (2 * j)) & 3 for j in range(4)], axis=3)  # [n,nblk,2,4,32]
        out["q"] = q.reshape(n, -1)
        out["sc"] = (scales & 15).reshape(n, -1)
        out["mn"] = (scales >> 4).reshape(n, -1)
    elif qtype == Q4_K:
        out["d"] = _h(b[..., 0:2])
        out["dmin"] = _h(b[..., 2:4])
        sc, mn = q4k_scale_min(b[..., 4:16])
        qs = b[..., 16:144].astype(np.int16).reshape(n, nblk, 4, 32)
        q = np.stack([qs & 15, qs >> 4], axis=3)  # [n,nblk,4,2,32]
        out["q"] = q.reshape(n, -1)
        out["sc"] = sc.reshape(n, -1)
        out["mn"] = mn.reshape(n, -1)
    elif qtype == Q6_K:
        ql = b[..., 0:128].astype(np.int16).reshape(n, nblk, 2, 2, 32)  # [ip][half][il]
        qh = b[..., 128:192].astype(np.int16).reshape(n, nblk, 2, 32)
        out["sc"] = b[..., 192:208].view(np.int8).astype(np.int32).reshape(n, -1)
        out["d"] = _h(b[..., 208:210])
        quarters = []
        for q4 in range(4):
            lo = ql[:, :, :, q4 & 1, :]
            nib = (lo & 15) if q4 < 2 else (lo >> 4)
            hi = (qh >> (2 * q4)) & 3
            quarters.append((nib | (hi << 4)) - 32)
        q = np.stack(quarters, axis=3)  # [n,nblk,2(ip),4(q4),32]
        out["q"] = q.reshape(n, -1)
    elif qtype == IQ3_S:
        out["d"] = _h(b[..., 0:2])
        qs = b[..., 2:66].astype(np.int32)                     # [n,nblk,64]
        qh = b[..., 66:74].astype(np.int32)                    # [n,nblk,8]
        signs = b[..., 74:106].astype(np.int32)                # [n,nblk,32]
        scales = b[..., 106:110].astype(np.int32)              # [n,nblk,4]
        bit9 = (qh[..., :, None] >> np.arange(8)) & 1          # [n,nblk,8,8]
        idx = qs | (bit9.reshape(n, nblk, 64) << 8)            # [n,nblk,64]
        g = iq3s_grid(iq3s_top)[idx].astype(np.int16)          # [n,nblk,64,4] -> weights 4*i..4*i+3
        g = g.reshape(n, nblk, 32, 8)                          # per signs byte: 8 weights
        sg = (signs[..., :, None] >> np.arange(8)) & 1         # [n,nblk,32,8]
        out["q"] = np.where(sg == 1, -g, g).astype(np.int16).reshape(n, -1)
        s = np.stack([scales & 15, scales >> 4], axis=-1)      # [n,nblk,4,2] -> ib = 2*i + e
        out["sc"] = s.reshape(n, -1)
    elif qtype == Q4_1:                                          # ggml-common.h: block_q4_1 {half2 dm; qs[16]}
        out["d"] = _h(b[..., 0:2])
        out["m"] = _h(b[..., 2:4])
        qs = b[..., 4:20].astype(np.int16)
        out["q"] = np.concatenate([qs & 15, qs >> 4], axis=-1).reshape(n, -1)
    elif qtype in (Q5_0, Q5_1):                                  # block_q5_0 {half d; qh[4]; qs[16]}, q5_1 {half2 dm; ...}
        o = 2 if qtype == Q5_0 else 4
        out["d"] = _h(b[..., 0:2])
        if qtype == Q5_1:
            out["m"] = _h(b[..., 2:4])
        qh = np.ascontiguousarray(b[..., o:o + 4]).view(np.uint32)[..., 0].astype(np.int64)     # [n,nblk]
        qs = b[..., o + 4:o + 20].astype(np.int16)
        bits = ((qh[..., None] >> np.arange(32)) & 1).astype(np.int16)                          # [n,nblk,32]
        lo = (qs & 15) | (bits[..., 0:16] << 4)
        hi = (qs >> 4) | (bits[..., 16:32] << 4)
        out["q"] = np.concatenate([lo, hi], axis=-1).reshape(n, -1)                             # 0..31, unsigned
    elif qtype == Q3_K:                                          # block_q3_K {hmask[32]; qs[64]; scales[12]; half d}
        hm = b[..., 0:32].astype(np.int16)
        qs = b[..., 32:96].astype(np.int16).reshape(n, nblk, 2, 32)
        scb = b[..., 96:108].astype(np.int32)
        out["d"] = _h(b[..., 108:110])
        q = np.empty((n, nblk, 2, 4, 32), np.int16)
        for nn in range(2):
            for j in range(4):
                low = (qs[:, :, nn, :] >> (2 * j)) & 3
                has = (hm >> (4 * nn + j)) & 1
                q[:, :, nn, j, :] = low - np.where(has == 1, 0, 4)      # dequantize.cuh:150 -> -4..3
        out["q"] = q.reshape(n, -1)
        sc = np.empty((n, nblk, 16), np.int32)
        for i in range(16):                                      # dequantize.cuh:139-142, minus 32
            if i < 4:
                us = (scb[..., i] & 15) | (((scb[..., i + 8] >> 0) & 3) << 4)
            elif i < 8:
                us = (scb[..., i] & 15) | (((scb[..., i + 4] >> 2) & 3) << 4)
            elif i < 12:
                us = (scb[..., i - 8] >> 4) | (((scb[..., i] >> 4) & 3) << 4)
            else:
                us = (scb[..., i - 8] >> 4) | (((scb[..., i - 4] >> 6) & 3) << 4)
            sc[..., i] = us - 32
        out["sc"] = sc.reshape(n, -1)
    elif qtype == Q5_K:                                          # block_q5_K {half2 dm; scales[12]; qh[32]; qs[128]}
        out["d"] = _h(b[..., 0:2])
        out["dmin"] = _h(b[..., 2:4])
        sc, mn = q4k_scale_min(b[..., 4:16])
        qh = b[..., 16:48].astype(np.int16)                                  # [n,nblk,32]
        qs = b[..., 48:176].astype(np.int16).reshape(n, nblk, 4, 32)
        parts = []
        for il in range(4):
            lo = (qs[:, :, il, :] & 15) | (((qh >> (2 * il)) & 1) << 4)
            hi = (qs[:, :, il, :] >> 4) | (((qh >> (2 * il + 1)) & 1) << 4)
            parts += [lo, hi]
        out["q"] = np.stack(parts, axis=2).reshape(n, -1)                    # 0..31
        out["sc"] = sc.reshape(n, -1)
        out["mn"] = mn.reshape(n, -1)
    elif qtype == IQ4_NL:                                        # block_iq4_nl {half d; qs[16]}
        out["d"] = _h(b[..., 0:2])
        qs = b[..., 2:18].astype(np.int16)
        out["q"] = KVALUES_IQ4NL[np.concatenate([qs & 15, qs >> 4], axis=-1)].reshape(n, -1)
    elif qtype == IQ4_XS:                                        # block_iq4_xs {half d; u16 scales_h; scales_l[4]; qs[128]}
        out["d"] = _h(b[..., 0:2])
        sh = np.ascontiguousarray(b[..., 2:4]).view(np.uint16)[..., 0].astype(np.int32)         # [n,nblk]
        sl = b[..., 4:8].astype(np.int32)
        qs = b[..., 8:136].astype(np.int16).reshape(n, nblk, 8, 16)
        out["q"] = KVALUES_IQ4NL[np.concatenate([qs & 15, qs >> 4], axis=-1)].reshape(n, -1)
        ls = np.empty((n, nblk, 8), np.int32)
        for ib in range(8):
            ls[..., ib] = ((sl[..., ib // 2] >> (4 * (ib % 2))) & 15) | (((sh >> (2 * ib)) & 3) << 4)
        out["sc"] = (ls - 32).reshape(n, -1)
    else:
        raise ValueError(f"unsupported GGML type {qtype}")
    return out


# ----------------------------------------------------------------------------
# exact integer sub-block dots
# ----------------------------------------------------------------------------
def subblock_dots(w: dict, act: dict, k: int):
    """I[m,n,g] = sum_{i in group g} q_w[n,i] * q_a[m,i]  and  S[m,g] = sum q_a[m,i] (int64)."""
    g = GROUP[w["qtype"]]
    qw = w["q"].astype(np.int64)
    qa = act["q"][:, :k].astype(np.int64)
    n = qw.shape[0]
    m = qa.shape[0]
    qw3 = qw.reshape(n, k // g, g)
    qa3 = qa.reshape(m, k // g, g)
    I = np.einsum("ngi,mgi->mng", qw3, qa3, optimize=True)
    S = qa3.sum(axis=-1)
    return I, S


# ----------------------------------------------------------------------------
# the matmul ops
# ----------------------------------------------------------------------------
def mul_mat(wire: np.ndarray, qtype: int, x: np.ndarray, semantics: str = "mmvq",
            iq3s_top: int = 62, return_parts: bool = False):
    """y[M,N] (float32) = the reference op on q8_1-quantized activations.

    `x` is float32 [M,K].  `semantics`: "mmvq" restates ggml_mul_mat_vec_a8,
    "mmq" restates ggml_mul_mat_a8 (they differ in how Q4_K's min term and
    Q2_K's per-block combine are formed).  Scale products are evaluated in
    float64 from the exact fp16/int factors; the GPU accumulates in fp32, so
    agreement is to fp32 rounding, far inside the 1e-3 gate.
    """
    if semantics not in ("mmvq", "mmq"):
        raise ValueError(semantics)
    if semantics == "mmq" and qtype in NO_MMQ:
        raise ValueError("the reference has no MMQ kernel for the i-matrix formats")
    x = np.asarray(x, dtype=np.float32)
    m, k = x.shape
    act = quantize_q8_1(x)
    w = unpack(wire, qtype, iq3s_top)
    I, S = subblock_dots(w, act, k)              # [m,n,G], [m,G]
    I = I.astype(np.float64)
    S = S.astype(np.float64)
    blk = BLOCK[qtype][0]
    grp = GROUP[qtype]
    nb8 = k // 32
    d8 = h2d(act["d"][:, :nb8])                   # [m,K/32]
    s8 = h2d(act["s"][:, :nb8])
    d = h2d(w["d"])                               # [n,K/blk]
    gpb = blk // grp                              # groups per weight block
    d8g = np.repeat(d8, 32 // grp, axis=1) if grp < 32 else d8   # [m,G]
    if qtype == Q4_0:
        y = np.einsum("nb,mnb->mn", d, d8[:, None, :] * I - 8.0 * s8[:, None, :])
    elif qtype == Q8_0:
        y = np.einsum("nb,mb,mnb->mn", d, d8, I, optimize=True)
    elif qtype == IQ4_NL:                                         # vecdotq.cuh: vec_dot_iq4_nl_q8_1
        y = np.einsum("nb,mb,mnb->mn", d, d8, I, optimize=True)
    elif qtype in (Q4_1, Q5_1):
        # vecdotq.cuh:71-92 / 131-160: the products d*d8 and m*s8 are formed in fp16 (__hmul2), then used in fp32
        mw = w["m"]
        dd = h2d(hmul(w["d"][None, :, :], act["d"][:, None, :nb8]))      # [m,n,b]
        ms = h2d(hmul(mw[None, :, :], act["s"][:, None, :nb8]))
        y = (dd * I + ms).sum(-1)
    elif qtype == Q5_0:
        if semantics == "mmq":                                    # load_tiles_q5_0 subtracts 16 from the codes: exact
            y = np.einsum("nb,mnb->mn", d, d8[:, None, :] * (I - 16.0 * S[:, None, :]))
        else:                                                     # vecdotq.cuh:94-126: -16 through the fp16 raw sum
            y = np.einsum("nb,mnb->mn", d, d8[:, None, :] * I - 16.0 * s8[:, None, :])
    elif qtype in (Q6_K, Q3_K, IQ4_XS):
        sc = w["sc"].astype(np.float64)
        t = (I * sc[None] * d8g[:, None, :]).reshape(m, -1, k // blk, gpb).sum(-1)
        y = (t * d[None]).sum(-1)
    elif qtype == IQ3_S:
        sc = (0.5 + w["sc"].astype(np.float64)) * 0.5
        t = (I * sc[None] * d8g[:, None, :]).reshape(m, -1, k // blk, gpb).sum(-1)
        y = (t * d[None]).sum(-1)
    elif qtype in (Q2_K, Q4_K, Q5_K):
        sc = w["sc"].astype(np.float64)
        mn = w["mn"].astype(np.float64)
        dmin = h2d(w["dmin"])
        td = (I * sc[None] * d8g[:, None, :]).reshape(m, -1, k // blk, gpb).sum(-1)
        if qtype in (Q4_K, Q5_K) and semantics == "mmq":
            tm = (mn[None] * s8[:, None, :]).reshape(m, -1, k // blk, gpb).sum(-1)
        else:
            tm = (mn[None] * (S * d8g)[:, None, :]).reshape(m, -1, k // blk, gpb).sum(-1)
        y = (td * d[None]).sum(-1) - (tm * dmin[None]).sum(-1)
    else:
        raise ValueError(qtype)
    y = y.astype(np.float32)
    if return_parts:
        return y, act, I.astype(np.int64), S.astype(np.int64)
    return y


# ----------------------------------------------------------------------------
# dequantization
# ----------------------------------------------------------------------------
def dequantize_f32(wire: np.ndarray, qtype: int, iq3s_top: int = 62) -> np.ndarray:
    """fp32 dequantization [N,K]: the arithmetic of gguf-reader/gguf/quants.py.

    With iq3s_top=60 the IQ3_S result equals gguf-reader's d*(1+2s)*{1,3,..,15};
    with 62 it is the CUDA kernels' d*(0.5+s)*0.5*grid (dequantize.cuh:347).
    """
    w = unpack(wire, qtype, iq3s_top)
    blk = BLOCK[qtype][0]
    grp = GROUP[qtype]
    n, k = w["q"].shape
    q = w["q"].astype(np.float32)
    d = np.repeat(w["d"].astype(np.float32), blk, axis=1)
    if qtype == Q4_0:
        return d * (q - np.float32(8))
    if qtype == Q5_0:
        return d * (q - np.float32(16))
    if qtype in (Q4_1, Q5_1):
        return d * q + np.repeat(w["m"].astype(np.float32), blk, axis=1)
    if qtype in (Q8_0, IQ4_NL):
        return d * q
    if qtype in (Q6_K, Q3_K, IQ4_XS):
        sc = np.repeat(w["sc"].astype(np.float32), grp, axis=1)
        return (d * sc) * q
    if qtype == IQ3_S:
        s = np.repeat(w["sc"].astype(np.float32), grp, axis=1)
        if iq3s_top == 60:
            return (d * (1 + 2 * s)) * (q / np.float32(4))
        return (d * (np.float32(0.5) + s) * np.float32(0.5)) * q
    sc = np.repeat(w["sc"].astype(np.float32), grp, axis=1)
    mn = np.repeat(w["mn"].astype(np.float32), grp, axis=1)
    dmin = np.repeat(w["dmin"].astype(np.float32), blk, axis=1)
    return (d * sc) * q - dmin * mn


def hfma_sub(a, b, c):
    """fp16 a*b-c with a single rounding (a contracted multiply-subtract)."""
    return f2h(h2d(a) * h2d(b) - h2d(c))


def dequantize(wire: np.ndarray, qtype: int, dtype: str = "f16", half_fma: int = 1) -> np.ndarray:
    """`ggml_dequantize` with the reference's intermediate fp16 roundings.

    Returns fp32 values that are exactly representable in `dtype`
    ("f16" | "bf16" | "f32"), shape [N,K].

    half_fma: the reference writes `__hsub(__hmul(a, b), c)` for Q2_K and Q4_K; PTX lets the compiler
    contract that pair into one fused multiply-add, so what the built reference computes depends on the
    toolchain.  0 = two roundings, 1 = first product fused (a*b-c in one rounding), 2 = (Q2_K only) the
    second product fused instead.  The value the reference build for sm_100a shows is the default.
    """
    w = unpack(wire, qtype, 62)
    blk = BLOCK[qtype][0]
    grp = GROUP[qtype]
    q = w["q"].astype(np.int32)
    d = np.repeat(w["d"], blk, axis=1)                      # fp16
    if qtype == Q4_0:
        v = hmul(hsub(f2h(q), np.float16(8)), d)            # dequantize.cuh:10-15
    elif qtype == Q5_0:
        v = hmul(hsub(f2h(q), np.float16(16)), d)           # dequantize.cuh:35-50
    elif qtype in (Q4_1, Q5_1):                             # dequantize.cuh:18-33, 52-67: hmul2 then hadd2
        mm = np.repeat(w["m"], blk, axis=1)
        v = f2h(h2d(f2h(q)) * h2d(d) + h2d(mm)) if half_fma else f2h(h2d(hmul(f2h(q), d)) + h2d(mm))
    elif qtype == Q3_K:                                     # dequantize.cuh:143-151
        sc = np.repeat(w["sc"], grp, axis=1)
        v = hmul(hmul(d, f2h(sc)), f2h(q))
    elif qtype == Q5_K:                                     # dequantize.cuh:198-230
        sc = np.repeat(w["sc"], grp, axis=1)
        mn = np.repeat(w["mn"], grp, axis=1)
        dmin = np.repeat(w["dmin"], blk, axis=1)
        d1 = hmul(d, f2h(sc))
        m1 = hmul(dmin, f2h(mn))
        v = hfma_sub(d1, f2h(q), m1) if half_fma else hsub(hmul(d1, f2h(q)), m1)
    elif qtype in (IQ4_NL, IQ4_XS):                         # dequantize.cuh:401-437: fp32, then conversion to dst
        df = d.astype(np.float32)
        if qtype == IQ4_XS:
            df = (df * np.repeat(w["sc"], grp, axis=1).astype(np.float32)).astype(np.float32)
        return round_to_dtype((df * q.astype(np.float32)).astype(np.float32), dtype)
    elif qtype == Q8_0:
        v = hmul(f2h(q), d)                                 # dequantize.cuh:74-77
    elif qtype == Q2_K:
        sc = np.repeat(w["sc"], grp, axis=1)
        mn = np.repeat(w["mn"], grp, axis=1)
        dmin = np.repeat(w["dmin"], blk, axis=1)
        if half_fma == 1:                                    # dequantize.cuh:117-120
            v = hfma_sub(d, f2h(sc * q), hmul(dmin, f2h(mn)))
        elif half_fma == 2:
            v = f2h(h2d(hmul(d, f2h(sc * q))) - h2d(dmin) * h2d(f2h(mn)))
        else:
            v = hsub(hmul(d, f2h(sc * q)), hmul(dmin, f2h(mn)))
    elif qtype == Q4_K:
        sc = np.repeat(w["sc"], grp, axis=1)
        mn = np.repeat(w["mn"], grp, axis=1)
        dmin = np.repeat(w["dmin"], blk, axis=1)
        d1 = hmul(d, f2h(sc))
        m1 = hmul(dmin, f2h(mn))
        v = hfma_sub(d1, f2h(q), m1) if half_fma else hsub(hmul(d1, f2h(q)), m1)  # dequantize.cuh:187-194
    elif qtype == Q6_K:
        sc = np.repeat(w["sc"], grp, axis=1)
        v = hmul(d, f2h(sc * q))                            # dequantize.cuh:252-255
    elif qtype == IQ3_S:
        s = np.repeat(w["sc"], grp, axis=1).astype(np.float32)
        df = (d.astype(np.float32) * (np.float32(0.5) + s)).astype(np.float32)
        df = (df * np.float32(0.5)).astype(np.float32)
        mag = (df * np.abs(q).astype(np.float32)).astype(np.float32)
        v32 = np.where(q < 0, -mag, mag).astype(np.float32)  # dequantize.cuh:347-352
        return round_to_dtype(v32, dtype)
    else:
        raise ValueError(qtype)
    # K/legacy kernels produce fp16, then convert_from_half<dst_t> (ggml-common.h:1080-1096)
    return round_to_dtype(v.astype(np.float32), dtype)


# ----------------------------------------------------------------------------
# the reference's CPU path (timed baseline; unquantized activations)
# ----------------------------------------------------------------------------
def cpu_dense_path(wire: np.ndarray, qtype: int, x: np.ndarray) -> np.ndarray:
    """gguf-reader dequantize + matmul (linear.py:55-59 with the CPU reader):
    W = dequantize_f32(wire) with gguf-reader's IQ3_S grid, y = x @ W.T."""
    W = dequantize_f32(wire, qtype, iq3s_top=60)
    return np.asarray(x, np.float32) @ W.T
