"""Regenerates ``rms_norm_fused_add_seed24.npz`` from the reference's own torch restatement.

Run where the reference checkout is mounted::

    python tests/golden/make_rms_norm_fused_add_golden.py /path/to/JJJetson_Ops

It imports ``torch_rms_norm_fused_add_ref`` from the reference's ``tests/test_rms_norm_fused_add.py``
(:14-28) with the compiled ``rms_norm_fused_add_me`` module and the ``utils`` helper stubbed out, feeds
it the exact inputs of the reference test (:31-41: ``np.random.seed(24)``, hidden 128, 13 tokens,
epsilon 1e-6, Fortran order) and stores what it returns.  The inputs are not stored: the legacy
``np.random.seed`` stream is stable across NumPy versions, and the tests regenerate them.
"""
import importlib.util
import os
import sys
import types

import numpy as np


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: %s /path/to/JJJetson_Ops" % sys.argv[0])
    ref_root = sys.argv[1]
    sys.modules["rms_norm_fused_add_me"] = types.ModuleType("rms_norm_fused_add_me")  # the GPU entry point lives there
    sys.modules.setdefault("utils", types.ModuleType("utils"))
    spec = importlib.util.spec_from_file_location(
        "ref_test_rms", os.path.join(ref_root, "tests", "test_rms_norm_fused_add.py")
    )
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    np.random.seed(mod.SEED)
    shape = (mod.HIDDEN_SIZE, mod.NUM_TOKENS, 1, mod.BATCH)
    input_np = np.asfortranarray(np.random.randn(*shape).astype(np.float32))
    residual_np = np.asfortranarray(np.random.randn(*shape).astype(np.float32))
    weight_np = np.random.randn(mod.HIDDEN_SIZE).astype(np.float32)
    ref_input, ref_residual = mod.torch_rms_norm_fused_add_ref(input_np, residual_np, weight_np, mod.EPS)
    here = os.path.dirname(os.path.abspath(__file__))
    path = os.path.join(here, "rms_norm_fused_add_seed24.npz")
    # stored token-major ([token][hidden]), the memory order of the reference's column-major [hidden, token]
    np.savez_compressed(
        path, seed=np.int64(mod.SEED), hidden=np.int64(mod.HIDDEN_SIZE), tokens=np.int64(mod.NUM_TOKENS),
        eps=np.float64(mod.EPS),
        normed=np.ascontiguousarray(ref_input.reshape(mod.HIDDEN_SIZE, mod.NUM_TOKENS).T),
        residual=np.ascontiguousarray(ref_residual.reshape(mod.HIDDEN_SIZE, mod.NUM_TOKENS).T))
    print("wrote", path)


if __name__ == "__main__":
    main()
