"""Generate tests/golden/reader_dequant.npz from the reference's own gguf-reader.

Run in a container that has the reference tree (it cannot travel to the GPU box):
    python tests/golden/make_golden_reader.py [<path of the kaiLLM tree>]
(default: $KQ_REFERENCE_ROOT, else a `reference` directory beside this repository)
For each supported GGML type a small seeded wire tensor (kaillm_b200.synth.wire_numpy) is dequantized
with `gguf.quants.dequantize` (gguf-reader/gguf/quants.py:68) imported from the reference tree; inputs
and outputs are stored so the oracle can be checked against the reference's arithmetic anywhere.
"""
import importlib.util
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
ref = sys.argv[1] if len(sys.argv) > 1 else (os.environ.get("KQ_REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference"))
sys.path.insert(0, os.path.join(ref, "runtime-source", "gguf-reader"))
import gguf  # noqa: E402
from gguf import quants  # noqa: E402
from gguf.constants import GGMLQuantizationType  # noqa: E402

assert gguf.__file__.startswith(ref), gguf.__file__
spec = importlib.util.spec_from_file_location("kq_synth", os.path.join(ROOT, "kaillm_b200", "synth.py"))
synth = importlib.util.module_from_spec(spec)
spec.loader.exec_module(synth)

out = {}
for qt in sorted(synth.BLOCK):
    blk, _ = synth.BLOCK[qt]
    w = synth.wire_numpy(qt, 6, 2 * max(blk, 256), seed=100 + qt)
    out[f"wire_{qt}"] = w
    out[f"deq_{qt}"] = quants.dequantize(w, GGMLQuantizationType(qt)).astype(np.float32)
np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "reader_dequant.npz"), **out)
print("wrote reader_dequant.npz", {k: v.shape for k, v in out.items()})
