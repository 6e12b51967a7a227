"""In-tree build of the native pieces.

  kaillm_b200/libkq.so      hand-written sm_100a CUDA kernels behind the C ABI (include/kq_gguf.h)
  kaillm_b200/_C_gguf.so    PyTorch extension registering torch.ops._C_gguf.* on top of libkq

Both are built with explicit nvcc / g++ command lines (no JIT cache), so the files sit next to the
package and travel with it.  `python -m kaillm_b200._build` rebuilds what is out of date.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
ROOT = os.path.dirname(HERE)
NVCC = os.environ.get("KQ_NVCC", "/usr/local/cuda/bin/nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]

CU_SOURCES = ["kq_api.cu", "kq_quantize.cu", "kq_gemv_dp4a.cu", "kq_gemv_mma.cu", "kq_gemv_tile.cu", "kq_gemv_kres.cu", "kq_gemv_umma.cu", "kq_moe.cu", "kq_gemm_tc.cu", "kq_p2p.cu", "kq_dequant.cu"]
CU_DEPS = ["kq_common.cuh", "kq_tile_common.cuh", "kq_tma.cuh", "kq_iq3s_codes.inc", os.path.join(ROOT, "include", "kq_gguf.h")]


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _run(cmd: list[str]) -> None:
    print("[kq build]", " ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)


def build_libkq(force: bool = False, verbose_ptxas: bool = False) -> str:
    out = os.path.join(HERE, "libkq.so")
    srcs = [os.path.join(CSRC, s) for s in CU_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    deps = srcs + [d if os.path.isabs(d) else os.path.join(CSRC, d) for d in CU_DEPS]
    if not force and not _newer(out, deps):
        return out
    objs = []
    procs = []
    for s in srcs:
        o = os.path.join(CSRC, os.path.basename(s)[:-3] + ".o")
        if force or _newer(o, [s] + deps[len(srcs):]):
            cmd = [NVCC, *ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-c", s, "-o", o]
            if verbose_ptxas:
                cmd += ["-Xptxas", "-v"]
            print("[kq build]", " ".join(cmd), flush=True)
            procs.append((subprocess.Popen(cmd), s))
        objs.append(o)
    for p, s in procs:
        if p.wait() != 0:
            raise RuntimeError(f"nvcc failed on {s}")
    _run([NVCC, *ARCH_FLAGS, "-shared", "-cudart", "shared", "-o", out, *objs,
          "-Xlinker", "-rpath,/usr/local/cuda/lib64"])
    return out


def build_torch_ext(force: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension

    out = os.path.join(HERE, "_C_gguf.so")
    src = os.path.join(CSRC, "torch_bindings.cpp")
    if not force and not _newer(out, [src, os.path.join(ROOT, "include", "kq_gguf.h")]):
        return out
    inc = []
    for p in cpp_extension.include_paths("cuda"):
        inc += ["-I", p]
    inc += ["-I", sysconfig.get_paths()["include"]]
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
           "-DTORCH_EXTENSION_NAME=_C_gguf", *inc, src, "-o", out,
           "-L", HERE, "-lkq", "-L", libdir, "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
           "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{libdir}"]
    _run(cmd)
    return out


def build_all(force: bool = False) -> None:
    build_libkq(force)
    build_torch_ext(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
