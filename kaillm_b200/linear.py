"""Regime dispatch and `apply` of the GGUF linear method.

`fused_mul_mat_gguf` follows `_fused_mul_mat_gguf` (vllm_gguf_plugin/quantization/linear.py:40-63)
decision for decision, so the same op is called for the same (M, N, type) as in the reference and the
numerical flavour (MMVQ vs MMQ arithmetic) is the reference's.  `GGUFLinear.apply` follows
`GGUFLinearMethod.apply` (linear.py:341-407) for plain and merged (q/k/v, gate/up) layers.
"""
from __future__ import annotations

import torch

from . import ops
from .synth import BLOCK

# the reference's type sets (quantization/utils.py:45-75), restricted to the formats this library serves
IMATRIX_QUANT_TYPES = frozenset({20, 21, 23})    # IQ4_NL, IQ3_S, IQ4_XS
MMVQ_QUANT_TYPES = frozenset({2, 3, 6, 7, 8, 10, 11, 12, 13, 14, 20, 21, 23})
MMQ_QUANT_TYPES = frozenset({2, 3, 6, 7, 8, 10, 11, 12, 13, 14})
DEQUANT_TYPES = MMVQ_QUANT_TYPES


def fused_mul_mat_gguf(x: torch.Tensor, qweight: torch.Tensor, qweight_type: int) -> torch.Tensor:
    if qweight_type in IMATRIX_QUANT_TYPES:
        mmvq_safe = 8 if qweight.shape[0] > 5120 else 16
    else:
        mmvq_safe = 2 if qweight.shape[0] > 5120 else 6
    if x.shape[0] == 0:
        return torch.empty(x.shape[0], qweight.shape[0], dtype=x.dtype, device=x.device)
    if x.shape[0] <= mmvq_safe and qweight_type in MMVQ_QUANT_TYPES:
        return ops.ggml_mul_mat_vec_a8(qweight, x, qweight_type, qweight.shape[0])
    if qweight_type in MMQ_QUANT_TYPES:
        return ops.ggml_mul_mat_a8(qweight, x, qweight_type, qweight.shape[0])
    if qweight_type in DEQUANT_TYPES:
        block_size, type_size = BLOCK[qweight_type]
        shape = (qweight.shape[0], qweight.shape[1] // type_size * block_size)
        weight = ops.ggml_dequantize(qweight, qweight_type, *shape, x.dtype)
        return x @ weight.T
    raise NotImplementedError(f"Unsupported GGUF quantization type: {qweight_type}")


class GGUFLinear:
    """A (possibly merged) GGUF linear layer: wire bytes + type per shard.

    shards: list of (qweight uint8 [N_i, rowbytes_i], qweight_type).  Shards of one type are stored
    as one concatenated tensor and run as a single call, as the reference does when all shard types
    agree (linear.py:377-381); mixed types run per shard and are concatenated (linear.py:382-397).
    """

    def __init__(self, shards):
        self.shards = list(shards)
        types = {t for _, t in self.shards}
        if len(types) == 1 and len(self.shards) > 1:
            self.merged = (torch.cat([w for w, _ in self.shards], dim=0).contiguous(), self.shards[0][1])
        else:
            self.merged = None

    def apply(self, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        if self.merged is not None:
            out = fused_mul_mat_gguf(x, *self.merged)
        elif len(self.shards) == 1:
            out = fused_mul_mat_gguf(x, *self.shards[0])
        else:
            out = torch.cat([fused_mul_mat_gguf(x, w, t) for w, t in self.shards], dim=1)
        if bias is not None:
            out.add_(bias)
        return out
