"""Public op wrappers with the reference's names, arguments and error behaviour.

Mirrors the public section of vllm_gguf_plugin/ops.py:181-208: `ggml_dequantize`,
`ggml_mul_mat_vec_a8` and `ggml_mul_mat_a8` forward to `torch.ops._C_gguf.*`.  Unlike the reference
there is no Triton fallback behind them: if the `_C_gguf` extension cannot be loaded the import fails.

Importing this module loads `kaillm_b200/_C_gguf.so`, which registers the six op schemas of the
reference's extension (vllm_gguf_plugin/csrc/torch_bindings.cpp:22-41) under the same namespace, so
code that calls `torch.ops._C_gguf.ggml_*` directly works unchanged.
"""
from __future__ import annotations

import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
EXT_PATH = os.path.join(_HERE, "_C_gguf.so")

# GGML type ids served by the CUDA kernels (gguf-reader/gguf/constants.py:5763-5799)
SUPPORTED_QUANT_TYPES = frozenset({2, 3, 6, 7, 8, 10, 11, 12, 13, 14, 20, 21, 23})
GEMM_QUANT_TYPES = frozenset({2, 3, 6, 7, 8, 10, 11, 12, 13, 14})


def _load_extension() -> None:
    if hasattr(torch.ops, "_C_gguf") and hasattr(torch.ops._C_gguf, "ggml_mul_mat_vec_a8"):
        return
    if not os.path.exists(EXT_PATH):
        raise ImportError(
            f"{EXT_PATH} is missing: build it with `python -m kaillm_b200._build` "
            "(the GGUF ops have no Triton or CPU fallback)")
    torch.ops.load_library(EXT_PATH)


_load_extension()


def ggml_dequantize(W: torch.Tensor, quant_type: int, m: int, n: int, dtype: torch.dtype | None) -> torch.Tensor:
    return torch.ops._C_gguf.ggml_dequantize(W, quant_type, m, n, dtype)


def ggml_mul_mat_vec_a8(W: torch.Tensor, X: torch.Tensor, quant_type: int, row: int) -> torch.Tensor:
    return torch.ops._C_gguf.ggml_mul_mat_vec_a8(W, X, quant_type, row)


def ggml_mul_mat_a8(W: torch.Tensor, X: torch.Tensor, quant_type: int, row: int) -> torch.Tensor:
    return torch.ops._C_gguf.ggml_mul_mat_a8(W, X, quant_type, row)


def ggml_moe_a8(X: torch.Tensor, W: torch.Tensor, sorted_token_ids: torch.Tensor, expert_ids: torch.Tensor,
                num_tokens_post_padded: torch.Tensor, quant_type: int, row: int, top_k: int, tokens: int) -> torch.Tensor:
    """vllm_gguf_plugin/ops.py:211-246."""
    return torch.ops._C_gguf.ggml_moe_a8(X, W, sorted_token_ids, expert_ids, num_tokens_post_padded, quant_type, row, top_k,
                                         tokens)


def ggml_moe_a8_vec(X: torch.Tensor, W: torch.Tensor, topk_ids: torch.Tensor, top_k: int, quant_type: int, row: int,
                    tokens: int) -> torch.Tensor:
    """vllm_gguf_plugin/ops.py:249-278."""
    return torch.ops._C_gguf.ggml_moe_a8_vec(X, W, topk_ids, top_k, quant_type, row, tokens)


def ggml_moe_get_block_size(quant_type: int) -> int:
    """vllm_gguf_plugin/ops.py:281-284."""
    return torch.ops._C_gguf.ggml_moe_get_block_size(quant_type)
