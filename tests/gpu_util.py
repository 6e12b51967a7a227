"""Helpers shared by the GPU tests."""
import numpy as np
import torch

from kaillm_b200 import synth
from oracle import gguf_oracle as O

TDT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def dev():
    return torch.device("cuda:0")


def act(m, k, seed, dt):
    """(numpy fp32 values already representable in dt, torch tensor of dtype dt on the GPU)"""
    x = synth.activations_numpy(m, k, seed=seed, dtype=dt)
    return x, torch.from_numpy(x).to(TDT[dt]).to(dev())


def wire(qt, n, k, seed):
    w = synth.wire_numpy(qt, n, k, seed=seed)
    return w, torch.from_numpy(w).to(dev())


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def to_np(t):
    return t.detach().float().cpu().numpy()
