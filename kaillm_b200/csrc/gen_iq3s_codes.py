"""Regenerate kq_iq3s_codes.inc: the IQ3_S codebook as 512 twelve-bit codes.

The codebook is part of the GGUF IQ3_S format (512 entries of four magnitudes,
eight possible levels each).  This script reads the 512 packed words of the
`iq3xs_grid` table from a ggml-common.h given on the command line
(vllm_gguf_plugin/csrc/gguf/ggml-common.h:685 in the reference tree) and stores
level indices only: code = l0 | l1<<3 | l2<<6 | l3<<9 with byte_j = 8*l_j+4,
except that level 7 is the format variant's top byte (62 in that table).

usage: python gen_iq3s_codes.py <path/to/ggml-common.h>
"""
import os
import re
import sys


def main(path: str) -> None:
    src = open(path).read()
    m = re.search(r"iq3xs_grid\[512\]\s*=\s*\{(.*?)\};", src, re.S)
    words = [int(t, 16) for t in re.findall(r"0x[0-9a-fA-F]+", m.group(1))]
    assert len(words) == 512
    codes = []
    for w in words:
        code = 0
        for j in range(4):
            b = (w >> (8 * j)) & 0xFF
            lvl = 7 if b == 62 else (b - 4) // 8
            assert 0 <= lvl <= 7 and (b == 62 or b == 8 * lvl + 4), hex(w)
            code |= lvl << (3 * j)
        codes.append(code)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kq_iq3s_codes.inc")
    with open(out, "w") as f:
        for i in range(0, 512, 16):
            f.write(", ".join(f"0x{c:03x}" for c in codes[i:i + 16]) + ",\n")
    print("wrote", out)


if __name__ == "__main__":
    main(sys.argv[1])
