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


UNQUANTIZED_TYPES = frozenset({0, 1, 30})        # F32, F16, BF16: plain tensors, torch.embedding serves them
F32_MATH_EMBEDDING_TYPES = frozenset({12, 13, 14})


def apply_gguf_embedding(x: torch.Tensor, qweight: torch.Tensor, qweight_type: int, hidden_size: int,
                         dtype: torch.dtype | None = None) -> torch.Tensor:
    """`_apply_gguf_embedding` (vllm_gguf_plugin/quantization/vocal_embeds.py:29-58): rows `x` of the quantized vocabulary
    table, dequantized.  The reference gathers the wire rows with index_select and dequantizes the copy; here one kernel
    reads the selected rows in place (kq_dequantize_rows).  Q4_K / Q5_K / Q6_K are reconstructed with fp32 products, as
    the reference does for exactly these three formats (vocal_embeds.py:43-50); the others with ggml_dequantize's fp16
    arithmetic."""
    from . import capi
    if qweight_type in UNQUANTIZED_TYPES:
        return torch.embedding(qweight, x)
    if qweight_type in DEQUANT_TYPES:
        block_size, type_size = BLOCK[qweight_type]
        assert hidden_size == qweight.shape[1] // type_size * block_size
        return capi.dequantize_rows(qweight, qweight_type, hidden_size, x, dtype or torch.float16,
                                    f32_math=qweight_type in F32_MATH_EMBEDDING_TYPES)
    raise NotImplementedError(f"Unsupported GGUF quantization type: {qweight_type}")


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int):
    """What vLLM's moe_align_block_size returns (fused_moe.py, called at quantization/fused_moe.py:62-64): the flattened
    (token, k) slots sorted by expert, every expert's run padded to a multiple of `block_size` with the value
    topk_ids.numel(), one expert id per block, the padded total.  Torch ops only (no host synchronisation)."""
    flat = topk_ids.reshape(-1).to(torch.int64)
    total = flat.numel()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)[:num_experts]
    padded = (counts + block_size - 1) // block_size * block_size
    starts = torch.cumsum(padded, 0) - padded                       # where each expert's run starts after padding
    raw_starts = torch.cumsum(counts, 0) - counts
    max_slots = total + num_experts * (block_size - 1)
    max_slots = (max_slots + block_size - 1) // block_size * block_size
    sorted_ids = torch.full((max_slots,), total, dtype=torch.int32, device=topk_ids.device)
    e_of = flat[order]
    pos = starts[e_of] + (torch.arange(total, device=topk_ids.device) - raw_starts[e_of])
    sorted_ids[pos] = order.to(torch.int32)
    nblocks = max_slots // block_size
    block_start = torch.arange(nblocks, device=topk_ids.device) * block_size
    ends = torch.cumsum(padded, 0)
    expert_ids = torch.searchsorted(ends, block_start, right=True).to(torch.int32)
    # blocks past the padded total belong to nobody: -1, which every kernel skips.  (An id equal to num_experts would be
    # taken for a real expert by a kernel that only checks 0..255, as the reference's does, and read past the weights.)
    expert_ids = torch.where(expert_ids >= num_experts, torch.full_like(expert_ids, -1), expert_ids)
    return sorted_ids, expert_ids, ends[-1:].to(torch.int32)


def fused_moe_gguf(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                   qweight_type: int, qweight_type2: int) -> torch.Tensor:
    """`_fused_moe_gguf` with the SiLU-and-multiply activation (quantization/fused_moe.py:34-133): gate/up projection of
    every (token, expert) pair, activation, down projection, routing weights, sum over the experts of a token.  More than
    64 tokens of MMQ formats take the expert-sorted block op, otherwise the per-pair op - the reference's two branches."""
    num_tokens = x.shape[0]
    e, n = w1.shape[0], w1.shape[1]
    top_k = topk_ids.shape[1]

    def act(t):
        d = t.shape[-1] // 2
        return torch.nn.functional.silu(t[..., :d]) * t[..., d:]

    if qweight_type in MMQ_QUANT_TYPES and qweight_type2 in MMQ_QUANT_TYPES and num_tokens > 64:
        block = ops.ggml_moe_get_block_size(qweight_type)
        s, ex, tot = moe_align_block_size(topk_ids, block, e)
        out = ops.ggml_moe_a8(x, w1, s, ex, tot, qweight_type, n, top_k, num_tokens)
        out = ops.ggml_moe_a8(act(out), w2, s, ex, tot, qweight_type2, w2.shape[1], 1, num_tokens * top_k)
    elif qweight_type in MMVQ_QUANT_TYPES and qweight_type2 in MMVQ_QUANT_TYPES:
        ids = topk_ids.to(torch.int32)
        out = ops.ggml_moe_a8_vec(x, w1, ids, top_k, qweight_type, n, num_tokens)
        out = ops.ggml_moe_a8_vec(act(out), w2, ids, 1, qweight_type2, w2.shape[1], num_tokens * top_k)
    else:
        raise NotImplementedError(f"Unsupported GGUF quantization types: {qweight_type}, {qweight_type2}")
    out = out.reshape(num_tokens, top_k, w2.shape[1]) * topk_weights.view(num_tokens, top_k, 1).to(out.dtype)
    return out.sum(dim=1)
