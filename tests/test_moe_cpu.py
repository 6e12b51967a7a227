"""Host logic of the mixture-of-experts mirror on CPU: the expert-sorted block layout (what vLLM's
moe_align_block_size returns, vllm_gguf_plugin/quantization/fused_moe.py:60-64) against a plain-Python construction."""
import numpy as np
import pytest
import torch

from kaillm_b200 import linear


def plain_align(topk_ids, block, e):
    flat = topk_ids.reshape(-1)
    pad = flat.size
    sorted_ids, expert_ids = [], []
    for ex in range(e):
        z = np.nonzero(flat == ex)[0]
        nb = (z.size + block - 1) // block
        sorted_ids += list(z) + [pad] * (nb * block - z.size)
        expert_ids += [ex] * nb
    return np.asarray(sorted_ids, np.int64), np.asarray(expert_ids, np.int64), len(sorted_ids)


@pytest.mark.parametrize("tokens,top_k,e,block", [(1, 1, 4, 8), (5, 2, 4, 8), (70, 2, 8, 8), (33, 4, 16, 4), (9, 3, 3, 16)])
def test_moe_align_block_size_layout(tokens, top_k, e, block):
    rng = np.random.default_rng(tokens + e)
    ids = np.stack([rng.choice(e, size=top_k, replace=False) for _ in range(tokens)]).astype(np.int32)
    s, ex, tot = linear.moe_align_block_size(torch.from_numpy(ids), block, e)
    ws, wex, wtot = plain_align(ids, block, e)
    n = int(tot.item())
    assert n == wtot and n % block == 0 and s.dtype == torch.int32 and ex.dtype == torch.int32
    np.testing.assert_array_equal(s[:n].numpy(), ws)
    np.testing.assert_array_equal(ex[:n // block].numpy(), wex)
    assert bool((s[n:] == tokens * top_k).all())             # slots past the total are padding
    assert bool((ex[n // block:] == -1).all())               # and their blocks belong to no expert
    assert s.numel() % block == 0 and ex.numel() == s.numel() // block
    # every (token, k) slot appears exactly once
    real = s[s < tokens * top_k].numpy()
    assert sorted(real.tolist()) == list(range(tokens * top_k))


def test_moe_align_keeps_empty_experts_out():
    ids = torch.tensor([[0, 3], [3, 0]], dtype=torch.int32)       # experts 1 and 2 get nothing
    s, ex, tot = linear.moe_align_block_size(ids, 8, 4)
    assert int(tot.item()) == 16 and ex[:2].tolist() == [0, 3]
