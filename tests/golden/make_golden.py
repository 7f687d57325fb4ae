"""Generate tests/golden/reference_cases.npz from the reference's own CPU code.

Run in a container that has the reference checkout (it is only needed to build
oracle/_ref/libxcorr_ref.so, see oracle/Makefile):

    make -C oracle && python tests/golden/make_golden.py

Each case stores the seeded float32 inputs and the outputs of the unmodified reference
routines cpu_cross_corr_* (repo/cross-corr/src/validate.hpp:214-298) instantiated for float
(`f32`) and for double (`f64`).  n_to_mn is in the reference's FILE order (result t*n + r
pairs with left r).  The reference ships no golden vectors, so these are the fixtures the
CPU restatement (oracle/xcorr_oracle.c) and the CUDA library are pinned to.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
import pyoracle  # noqa: E402

# (name, mode, rows, cols, n_left, n_right, seed)
CASES = [
    ("o2o_1x1", "one_to_one", 1, 1, 1, 1, 11),
    ("o2o_3x5", "one_to_one", 3, 5, 1, 1, 12),
    ("o2o_16x16", "one_to_one", 16, 16, 1, 1, 1001),   # BASELINE config 1 shape and seed rule
    ("o2o_17x9", "one_to_one", 17, 9, 1, 1, 13),
    ("o2o_33x32", "one_to_one", 33, 32, 1, 1, 14),
    ("o2m_8x8x5", "one_to_many", 8, 8, 1, 5, 21),
    ("o2m_12x20x3", "one_to_many", 12, 20, 1, 3, 22),
    ("n2mn_6x7_3x6", "n_to_mn", 6, 7, 3, 6, 31),
    ("n2mn_16x16_2x8", "n_to_mn", 16, 16, 2, 8, 32),
    ("n2m_5x4_3x4", "n_to_m", 5, 4, 3, 4, 41),
    ("n2m_16x24_2x3", "n_to_m", 16, 24, 2, 3, 42),
]


def inputs(rows, cols, n_left, n_right, seed):
    """uniform[0,1) float32; left from `seed`, right from `seed + 1000`."""
    left = np.random.default_rng(seed).random((n_left, rows, cols), dtype=np.float32)
    right = np.random.default_rng(seed + 1000).random((n_right, rows, cols), dtype=np.float32)
    return left, right


def main():
    ref = pyoracle.Reference()
    blob = {}
    names = []
    for name, mode, rows, cols, nl, nr, seed in CASES:
        left, right = inputs(rows, cols, nl, nr, seed)
        blob[f"{name}/left"] = left
        blob[f"{name}/right"] = right
        blob[f"{name}/f32"] = ref.run(mode, left, right, acc64=False)
        blob[f"{name}/f64"] = ref.run(mode, left, right, acc64=True)
        names.append(f"{name}|{mode}|{rows}|{cols}|{nl}|{nr}|{seed}")
    blob["cases"] = np.array(names)
    path = os.path.join(HERE, "reference_cases.npz")
    np.savez_compressed(path, **blob)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
