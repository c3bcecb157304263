"""B200 (sm_100a) drop-in for the Q4_0 x Q8_1 quantized-linear path of JJJetson_Ops.

The product is ``libjq_b200.so`` (C ABI, ``include/jq_b200.h``) plus the two pybind11 modules the
reference ships for this path (``q8_1_me`` and ``mm_q4_0_q8_1_me``, under ``python/``, where the
reference-named loader module ``weight_loader_me`` sits too).  This
package is the thin host-side layer above them: ``capi`` binds the C ABI with ctypes and takes
torch CUDA tensors as plain device memory, ``synth`` builds the seeded synthetic workloads,
``sharded`` runs one linear N-sharded over several GPUs.

There is no CPU fallback: importing ``capi`` without the built library raises.
"""
from __future__ import annotations

import os
import sys

__all__ = ["package_dir", "python_module_dir", "import_reference_modules"]


def package_dir() -> str:
    return os.path.dirname(os.path.abspath(__file__))


def python_module_dir() -> str:
    """Directory holding ``q8_1_me`` and ``mm_q4_0_q8_1_me`` (the reference's ``python/``)."""
    return os.path.join(package_dir(), "python")


def import_reference_modules():
    """Import the two reference-named extension modules and return them."""
    d = python_module_dir()
    if d not in sys.path:
        sys.path.insert(0, d)
    import mm_q4_0_q8_1_me  # noqa: WPS433
    import q8_1_me  # noqa: WPS433

    return q8_1_me, mm_q4_0_q8_1_me
