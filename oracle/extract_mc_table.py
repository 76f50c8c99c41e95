"""Test infrastructure: reads the 256 x 16 marching-cubes case table out of the reference source where it lies
(src/marching_cubes.cu, a third-party table under its own licence) into oracle/_ref/mc_tri_table.npy, which is git-ignored
and travels to the GPU box with the other built files.  Nothing of the table is committed.  Used by the marching-cubes
parity tests to drive the oracle and the CUDA kernel with the table the reference would pass."""
import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
# the checkout of 19reborn/NeuS2 to read: NEUS2_REFERENCE, else a folder named "reference" beside this repository;
# without either nothing is extracted
REF = os.environ.get("NEUS2_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
OUT = os.path.join(HERE, "_ref", "mc_tri_table.npy")


def extract():
    if not REF:
        return None
    path = os.path.join(REF, "src", "marching_cubes.cu")
    if not os.path.exists(path):
        return None
    src = open(path).read()
    m = re.search(r"triangle_table\s*\[256\]\s*\[16\]\s*=\s*\{(.*?)\};", src, re.S)
    if not m:
        return None
    nums = [int(x) for x in re.findall(r"-?\d+", m.group(1))]
    if len(nums) != 256 * 16:
        return None
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    t = np.array(nums, np.int8).reshape(256, 16)
    np.save(OUT, t)
    return OUT


def load():
    """The extracted table, or None when neither the reference nor a previous extraction is available."""
    if not os.path.exists(OUT):
        extract()
    return np.load(OUT) if os.path.exists(OUT) else None


if __name__ == "__main__":
    print(extract() or "reference source not found", file=sys.stderr)
