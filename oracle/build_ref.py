"""Build the reference's own `_C_gguf` extension, unmodified, into oracle/_ref/ (TEST INFRASTRUCTURE).

The reference's CUDA implementation of the GGUF ops compiles from two of its own source files
(vllm_gguf_plugin/csrc/gguf/gguf_kernel.cu and csrc/torch_bindings.cpp, which include the vendored
headers next to them).  They are compiled where they lie in the reference tree; nothing is copied.
The only build-time change is the preprocessor definition `-D_C_gguf=_C_gguf_ref`, which makes the
library register its ops as `torch.ops._C_gguf_ref.*` so it can be loaded next to this repository's
`_C_gguf` and compared in one process.  Compiled for sm_100a without fast-math (IEEE division in the
q8_1 quantizer), like the PyTorch/vLLM extension defaults.

The output (`oracle/_ref/_C_gguf_ref.so`) is git-ignored but travels to the GPU box, where the
reference tree itself is absent.  Only tests, the smoke check and the benchmark's reference legs load it.

usage: python oracle/build_ref.py [--force]
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))


def reference_root() -> str:
    """The kaiLLM source tree: $KQ_REFERENCE_ROOT, else a `reference` directory beside this repository."""
    env = os.environ.get("KQ_REFERENCE_ROOT")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


REF_CSRC = os.environ.get("KQ_REFERENCE_CSRC") or os.path.join(reference_root(), "runtime-source", "vllm_gguf_plugin", "csrc")
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "_C_gguf_ref.so")
NVCC = os.environ.get("KQ_NVCC", "/usr/local/cuda/bin/nvcc")


def available() -> bool:
    return os.path.exists(os.path.join(REF_CSRC, "gguf", "gguf_kernel.cu"))


def build(force: bool = False) -> str | None:
    if not available():
        return OUT if os.path.exists(OUT) else None
    if os.path.exists(OUT) and not force:
        return OUT
    import torch
    from torch.utils import cpp_extension

    os.makedirs(OUT_DIR, exist_ok=True)
    inc = []
    for p in cpp_extension.include_paths("cuda"):
        inc += ["-I", p]
    inc += ["-I", sysconfig.get_paths()["include"]]
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    defs = ["-DUSE_CUDA", "-D_C_gguf=_C_gguf_ref", f"-D_GLIBCXX_USE_CXX11_ABI={abi}"]
    o_cu = os.path.join(OUT_DIR, "gguf_kernel.o")
    o_cpp = os.path.join(OUT_DIR, "torch_bindings.o")
    cmds = [
        [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", *defs, *inc,
         "-c", os.path.join(REF_CSRC, "gguf", "gguf_kernel.cu"), "-o", o_cu],
        ["g++", "-O2", "-std=c++17", "-fPIC", *defs, *inc, "-c", os.path.join(REF_CSRC, "torch_bindings.cpp"), "-o", o_cpp],
    ]
    procs = [subprocess.Popen(c) for c in cmds]
    for p, c in zip(procs, cmds):
        if p.wait() != 0:
            raise RuntimeError("reference build failed: " + " ".join(c))
    subprocess.run(["g++", "-shared", "-o", OUT, o_cu, o_cpp, "-L", libdir, "-ltorch", "-ltorch_cpu", "-ltorch_cuda",
                    "-lc10", "-lc10_cuda", "-L", "/usr/local/cuda/lib64", "-lcudart", f"-Wl,-rpath,{libdir}"], check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
