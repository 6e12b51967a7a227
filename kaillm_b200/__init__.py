"""kaillm_b200 - B200-native GGUF quantized linear kernels (drop-in for kaiLLM's `_C_gguf` ops).

Layout:
  capi.py     ctypes binding of the C ABI (include/kq_gguf.h) taking torch tensors
  ops.py      the public op wrappers with the reference's names and argument meaning
              (vllm_gguf_plugin/ops.py:181-208)
  linear.py   regime dispatch and the linear method's apply (quantization/linear.py:40-63, 341-407)
  sharded.py  row-sharded multi-GPU execution with an all-gather of the output slices
  synth.py    seeded synthetic wire tensors

There is no CPU or eager fallback: importing `capi` fails if libkq.so has not been built
(`python -m kaillm_b200._build`), and the ops raise if the `_C_gguf` extension is missing.
"""

__all__ = ["capi", "ops", "linear", "sharded", "synth"]
