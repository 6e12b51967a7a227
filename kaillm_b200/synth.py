"""Seeded synthetic GGUF wire tensors and activations.

Real GGUF checkpoints are not needed to exercise the quantized linear path: a
weight tensor is `uint8 [N, K/blk * block_bytes]` whose blocks hold fp16
scales and packed integer codes.  The generators below fill blocks with the
distributions the benchmark configurations prescribe:

* fp16 block scales `d` (and `dmin`) = |N(0,1)| * 0.02
* every other byte uniform, which makes 4/2/6-bit codes, 6-bit and 4-bit
  sub-scales, IQ3_S codebook indices and sign bits uniform
* Q6_K int8 sub-scales uniform in [-32, 31]

`wire_numpy` is the reproducible CPU generator (tests, fixtures);
`wire_torch` draws the same distributions directly on a CUDA device for the
multi-gigabyte benchmark stacks.
"""
from __future__ import annotations

import numpy as np

Q4_0, Q8_0, Q2_K, Q4_K, Q6_K, IQ3_S = 2, 8, 10, 12, 14, 21
Q4_1, Q5_0, Q5_1, Q3_K, Q5_K, IQ4_NL, IQ4_XS = 3, 6, 7, 11, 13, 20, 23
BLOCK = {Q4_0: (32, 18), Q8_0: (32, 34), Q2_K: (256, 84), Q4_K: (256, 144), Q6_K: (256, 210), IQ3_S: (256, 110),
         Q4_1: (32, 20), Q5_0: (32, 22), Q5_1: (32, 24), Q3_K: (256, 110), Q5_K: (256, 176), IQ4_NL: (32, 18),
         IQ4_XS: (256, 136)}
NAMES = {Q4_0: "Q4_0", Q8_0: "Q8_0", Q2_K: "Q2_K", Q4_K: "Q4_K", Q6_K: "Q6_K", IQ3_S: "IQ3_S", Q4_1: "Q4_1",
         Q5_0: "Q5_0", Q5_1: "Q5_1", Q3_K: "Q3_K", Q5_K: "Q5_K", IQ4_NL: "IQ4_NL", IQ4_XS: "IQ4_XS"}
# byte offsets of the fp16 scale fields inside one block
SCALE_FIELDS = {Q4_0: (0,), Q8_0: (0,), Q2_K: (80, 82), Q4_K: (0, 2), Q6_K: (208,), IQ3_S: (0,), Q4_1: (0, 2), Q5_0: (0,),
                Q5_1: (0, 2), Q3_K: (108,), Q5_K: (0, 2), IQ4_NL: (0,), IQ4_XS: (0,)}


def row_bytes(qtype: int, k: int) -> int:
    blk, nb = BLOCK[qtype]
    if k % blk:
        raise ValueError(f"K={k} is not a multiple of the {NAMES[qtype]} block size {blk}")
    return k // blk * nb


def weight_bytes(qtype: int, n: int, k: int) -> int:
    return n * row_bytes(qtype, k)


def wire_numpy(qtype: int, n: int, k: int, seed: int = 0) -> np.ndarray:
    rng = np.random.default_rng(seed)
    blk, nb = BLOCK[qtype]
    nblk = k // blk
    row_bytes(qtype, k)
    w = rng.integers(0, 256, size=(n, nblk, nb), dtype=np.uint8)
    for off in SCALE_FIELDS[qtype]:
        d = (np.abs(rng.standard_normal((n, nblk))) * 0.02).astype(np.float16)
        w[:, :, off:off + 2] = d.view(np.uint8).reshape(n, nblk, 2)
    if qtype == Q6_K:
        sc = rng.integers(-32, 32, size=(n, nblk, 16), dtype=np.int8)
        w[:, :, 192:208] = sc.view(np.uint8)
    return w.reshape(n, nblk * nb)


def activations_numpy(m: int, k: int, seed: int = 0, dtype: str = "f32") -> np.ndarray:
    """fp32 array holding N(0,1) values already rounded to `dtype` (f32|f16|bf16)."""
    rng = np.random.default_rng(seed + 1_000_003)
    x = rng.standard_normal((m, k)).astype(np.float32)
    if dtype == "f16":
        x = x.astype(np.float16).astype(np.float32)
    elif dtype == "bf16":
        u = x.view(np.uint32)
        u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
        x = u.astype(np.uint32).view(np.float32)
    elif dtype != "f32":
        raise ValueError(dtype)
    return x


def wire_torch(qtype: int, n: int, k: int, seed: int, device):
    """Same distributions as `wire_numpy`, generated on `device` (different stream of numbers)."""
    import torch

    blk, nb = BLOCK[qtype]
    nblk = k // blk
    row_bytes(qtype, k)
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    w = torch.randint(0, 256, (n, nblk, nb), dtype=torch.uint8, device=device, generator=g)
    for off in SCALE_FIELDS[qtype]:
        d = (torch.randn((n, nblk), device=device, generator=g).abs() * 0.02).to(torch.float16)
        w[:, :, off:off + 2] = d.view(torch.uint8).reshape(n, nblk, 2)
    if qtype == Q6_K:
        sc = torch.randint(-32, 32, (n, nblk, 16), dtype=torch.int8, device=device, generator=g)
        w[:, :, 192:208] = sc.view(torch.uint8)
    return w.reshape(n, nblk * nb)
