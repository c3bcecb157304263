"""Regenerates ``ref_gpu_sm100.npz``: outputs of the reference's own CUDA operators on a B200.

Run on a machine with a GPU, after ``make -C oracle ref`` has compiled the reference's
``src/cuda/q8_1.cu`` and ``src/cuda/mm_q4_0_q8_1.cu`` (unmodified, sm_100a) into
``oracle/_ref/libjjj_ref.so``::

    python tests/golden/make_ref_gpu_golden.py [output.npz]

For a few seeded cases it stores what the reference's ``q8_1()`` host entry (src/cuda/q8_1.cu:148)
writes and what ``mat_mul_q4_0_q8_1_device`` (src/cuda/mm_q4_0_q8_1.cu:394) computes.  Inputs are
not stored; ``case_inputs`` below regenerates them, and the CPU tests import it.  The Q4_0 bytes
fed to the multiply come from the oracle's quantizer (itself pinned by the gguf fixture), the
activations fed to it are the reference quantizer's own output re-ordered to the order its multiply
reads (block m * (K/128) + k/128, src/cuda/mm_q4_0_q8_1.cu:230).
"""
import ctypes
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
CASES = {"a": (1024, 64, 1, 101), "b": (1024, 96, 5, 102), "c": (4096, 128, 8, 103), "d": (2048, 40, 13, 104)}


def case_inputs(tag):
    K, N, M, seed = CASES[tag]
    rng = np.random.default_rng(np.random.PCG64(seed))
    w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    x = rng.standard_normal((M, K), dtype=np.float32)
    return K, N, M, w, x


def reorder_ksuper_col_to_col_ksuper(raw, K, M):
    return np.ascontiguousarray(raw.reshape(K // 128, M, 144).transpose(1, 0, 2)).reshape(-1)


def main():
    sys.path.insert(0, ROOT)
    import torch

    from oracle import jq_oracle as O
    from tests.test_gpu_vs_reference_kernels import REF_LIB, ref_mul_mat_device, ref_q8_1, _StdVectorInt

    lib = ctypes.CDLL(REF_LIB)
    lib.q8_1.restype = None
    lib.q8_1.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(_StdVectorInt)]
    lib.mat_mul_q4_0_q8_1_device.restype = None
    lib.mat_mul_q4_0_q8_1_device.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 3 + [ctypes.c_void_p]
    dev = torch.device("cuda:0")
    out = {}
    for tag in CASES:
        K, N, M, w, x = case_inputs(tag)
        xq_ref = ref_q8_1(lib, x)  # order (k/128)*M + m, s = sum(x)
        wq = O.quantize_q4_0(w)
        xq_mm = reorder_ksuper_col_to_col_ksuper(xq_ref, K, M)
        y = ref_mul_mat_device(lib, torch, torch.from_numpy(wq).to(dev), torch.from_numpy(xq_mm).to(dev), K, N, M)
        out[tag + "_xq"] = xq_ref
        out[tag + "_y"] = y.cpu().numpy()
        y_orc = O.mul_mat_ref(wq, xq_mm, K, N, M, O.ORDER_COL_KSUPER)
        print(tag, "oracle vs reference kernel: max abs diff", float(np.abs(y_orc - out[tag + "_y"]).max()),
              "bit-equal" if np.array_equal(y_orc, out[tag + "_y"]) else "not bit-equal")
    path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_gpu_sm100.npz")
    np.savez_compressed(path, **out)
    print("wrote", path)


if __name__ == "__main__":
    main()
