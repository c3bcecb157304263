"""Regenerates ``q4_0_gguf_seed5.npz``: Q4_0 bytes of a seeded matrix as produced by the ``gguf``
Python package (the ggml project's own NumPy quantizer), an implementation independent of both
the oracle and the CUDA quantizer.  The reference project contains no Q4_0 quantizer; its block
layout (src/cuda/mm_q4_0_q8_1.cu:35-38) is ggml's.

    python tests/golden/make_q4_0_gguf_golden.py
"""
import os

import numpy as np


def make_input() -> np.ndarray:
    rng = np.random.default_rng(np.random.PCG64(5))
    w = (rng.standard_normal((48, 512), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    w[3, 32:64] = 0.0  # an all-zero block
    w[5, 0] = -w[5, 7]  # a tie in magnitude with opposite signs: the first one must win
    w[5, 1:7] *= 0.1
    w[5, 8:32] *= 0.1
    return w


def main() -> None:
    import gguf
    from gguf import quants

    w = make_input()
    q = quants.quantize(w, gguf.GGMLQuantizationType.Q4_0)
    here = os.path.dirname(os.path.abspath(__file__))
    np.savez_compressed(os.path.join(here, "q4_0_gguf_seed5.npz"), q4_0=np.ascontiguousarray(q).reshape(48, -1))
    print("wrote q4_0_gguf_seed5.npz", q.shape)


if __name__ == "__main__":
    main()
