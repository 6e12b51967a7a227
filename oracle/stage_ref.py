"""Stage the reference's Python callers of the GGUF ops under baseline/_ref/ (TEST INFRASTRUCTURE).

The drop-in claim of this repository is that the reference's own, unmodified Python layer - `vllm_gguf_plugin.ops`
(ops.py:181-208), `torch.ops.vllm._fused_mul_mat_gguf` and `GGUFLinearMethod.apply` (quantization/linear.py:40-63,
341-407), `GGUFEmbeddingMethod` (quantization/vocal_embeds.py) - runs on top of this repository's `_C_gguf` module.
To test that where the reference tree itself is absent (the GPU box), its Python package and the gguf-reader package
are copied, byte for byte, into the git-ignored directory baseline/_ref/:

    baseline/_ref/vllm_gguf_plugin/...   every .py and .json file of runtime-source/vllm_gguf_plugin (no csrc binaries)
    baseline/_ref/gguf/...               runtime-source/gguf-reader/gguf

Nothing staged is ever committed, imported by the product, or modified.  Only tests and the benchmark's reference
legs read it.

usage: python oracle/stage_ref.py [--force]
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
STAGE = os.path.join(ROOT, "baseline", "_ref")


def _ref_root() -> str:
    sys.path.insert(0, ROOT)
    from oracle.build_ref import reference_root

    return reference_root()


def available() -> bool:
    return os.path.exists(os.path.join(_ref_root(), "runtime-source", "vllm_gguf_plugin", "ops.py"))


def staged() -> bool:
    return os.path.exists(os.path.join(STAGE, "vllm_gguf_plugin", "ops.py")) and os.path.exists(
        os.path.join(STAGE, "gguf", "quants.py"))


def stage(force: bool = False) -> str | None:
    if not available():
        return STAGE if staged() else None
    if staged() and not force:
        return STAGE
    src = os.path.join(_ref_root(), "runtime-source")

    def keep(_dir, names):
        return [n for n in names if n in ("csrc", "__pycache__") or n.endswith((".so", ".o", ".cu", ".cuh", ".cubin"))]

    for name, sub in (("vllm_gguf_plugin", "vllm_gguf_plugin"), ("gguf", os.path.join("gguf-reader", "gguf"))):
        dst = os.path.join(STAGE, name)
        if os.path.isdir(dst):
            shutil.rmtree(dst)
        shutil.copytree(os.path.join(src, sub), dst, ignore=keep)
    return STAGE


if __name__ == "__main__":
    print(stage(force="--force" in sys.argv))
