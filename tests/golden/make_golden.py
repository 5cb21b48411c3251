"""Regenerates tests/golden/oracle_cases.npz from the CPU oracle.

    python tests/golden/make_golden.py

The file pins the oracle's own outputs on small seeded inputs (weights
0.02*N(0,1), activations N(0,1), numpy default_rng seeds as below), so that a
change to the oracle shows up as a diff, and so that the CUDA path is compared
with committed bytes as well as with the oracle as built on the day.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle  # noqa: E402

CASES = {"q4_k": (48, 768, 3), "q6_k": (40, 512, 2), "q8_0": (56, 160, 5)}


def main():
    out = {}
    for i, (fmt, (rows, cols, n)) in enumerate(CASES.items()):
        rng = np.random.default_rng(100 + i)
        w = (0.02 * rng.standard_normal((rows, cols))).astype(np.float32)
        x = rng.standard_normal((n, cols)).astype(np.float32)
        blocks = oracle.quantize(fmt, w)
        out[f"{fmt}_w"] = w
        out[f"{fmt}_x"] = x
        out[f"{fmt}_blocks"] = blocks
        out[f"{fmt}_dequant"] = oracle.dequantize(fmt, blocks, rows, cols)
        out[f"{fmt}_matmul"] = oracle.matmul(fmt, blocks, rows, cols, x)
        up = oracle.quantize(fmt, w[::-1].copy())          # the `up` matrix: the same rows, reversed
        out[f"{fmt}_up_blocks"] = up
        out[f"{fmt}_swiglu"] = oracle.swiglu(fmt, blocks, up, rows, cols, x)
    np.savez_compressed(os.path.join(HERE, "oracle_cases.npz"), **out)
    print("wrote", os.path.join(HERE, "oracle_cases.npz"))


if __name__ == "__main__":
    main()
