"""Q4_0 tensors in the reference's weight formats: readers, writers and offline quantizer.

Thin ctypes layer over ``include/jq_weights_io.h``.  A fixture is the directory format of the
reference's loader (src/model/weight_loader.h:37-40; tests/fixture_utils.py:74-103): ``config.txt``,
``manifest.txt`` and one raw file per tensor; files ending in ``.q4_0`` hold 18-byte Q4_0 blocks.
The single-file format is safetensors (weight_loader.h:42-47): F32 tensors as the reference reads
them, a Q4_0 tensor ``w`` as ``w.q4_0`` with dtype ``U8`` and shape ``[rows, K / 32, 18]``.

Command line::

    python -m jjjetson_ops_b200.weights_io SRC_FIXTURE_DIR DST_FIXTURE_DIR      # quantize (needs a CUDA device:
                                                                                # runs the library's quantizer kernel)
    python -m jjjetson_ops_b200.weights_io SRC_FIXTURE_DIR DST.safetensors      # repack as one file (CPU only)
"""
from __future__ import annotations

import ctypes
import os
import sys
from typing import Dict, Mapping, NamedTuple, Tuple

import numpy as np

from . import capi

DTYPE_F32, DTYPE_Q4_0 = 0, 1


class _HostTensor(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("data", ctypes.c_void_p), ("dims", ctypes.POINTER(ctypes.c_int64)),
                ("ndim", ctypes.c_int), ("dtype", ctypes.c_int), ("nbytes", ctypes.c_size_t)]


class _WeightSet(ctypes.Structure):
    _fields_ = [("tensors", ctypes.POINTER(_HostTensor)), ("num_tensors", ctypes.c_int), ("config_text", ctypes.c_char_p)]


class Tensor(NamedTuple):
    dtype: int            # DTYPE_F32 or DTYPE_Q4_0
    dims: Tuple[int, ...]  # as in the manifest; [rows, K] for Q4_0
    data: np.ndarray      # float32 of shape dims, or uint8 [rows, K / 32 * 18]


_lib = capi.lib()
_lib.jq_weights_load_fixture.restype = ctypes.c_int
_lib.jq_weights_load_fixture.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.POINTER(_WeightSet))]
_lib.jq_weight_set_destroy.restype = None
_lib.jq_weight_set_destroy.argtypes = [ctypes.POINTER(_WeightSet)]
_lib.jq_weight_set_find.restype = ctypes.POINTER(_HostTensor)
_lib.jq_weight_set_find.argtypes = [ctypes.POINTER(_WeightSet), ctypes.c_char_p]
_lib.jq_weight_set_config_value.restype = ctypes.c_int
_lib.jq_weight_set_config_value.argtypes = [ctypes.POINTER(_WeightSet), ctypes.c_char_p, ctypes.POINTER(ctypes.c_double)]
_lib.jq_weights_quantize_fixture.restype = ctypes.c_int
_lib.jq_weights_quantize_fixture.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_int)]
_lib.jq_weights_load_safetensors.restype = ctypes.c_int
_lib.jq_weights_load_safetensors.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.POINTER(_WeightSet))]
_lib.jq_weights_save_safetensors.restype = ctypes.c_int
_lib.jq_weights_save_safetensors.argtypes = [ctypes.POINTER(_WeightSet), ctypes.c_char_p]


def _unpack(ps) -> Tuple[Dict[str, float], Dict[str, Tensor]]:
    """Copies a loaded set into numpy arrays; the caller still owns (and destroys) the set."""
    ws = ps.contents
    tensors: Dict[str, Tensor] = {}
    for i in range(ws.num_tensors):
        t = ws.tensors[i]
        dims = tuple(int(t.dims[d]) for d in range(t.ndim))
        raw = np.ctypeslib.as_array(ctypes.cast(t.data, ctypes.POINTER(ctypes.c_uint8)), shape=(t.nbytes,)).copy()
        if t.dtype == DTYPE_Q4_0:
            data = raw.reshape(dims[0], dims[1] // 32 * capi.Q4_BYTES)
        else:
            data = raw.view(np.float32).reshape(dims)
        found = _lib.jq_weight_set_find(ps, t.name)
        assert bool(found) and found.contents.nbytes == t.nbytes
        tensors[t.name.decode()] = Tensor(int(t.dtype), dims, data)
    config: Dict[str, float] = {}
    for line in (ws.config_text or b"").decode().splitlines():
        key = line.split("=", 1)[0].strip()
        v = ctypes.c_double()
        if key and _lib.jq_weight_set_config_value(ps, key.encode(), ctypes.byref(v)):
            config[key] = v.value
    return config, tensors


def load_fixture(path: str) -> Tuple[Dict[str, float], Dict[str, Tensor]]:
    """-> (config as numbers, tensors by name).  Raises ``capi.JqError`` on a malformed fixture."""
    ps = ctypes.POINTER(_WeightSet)()
    capi.check(_lib.jq_weights_load_fixture(os.fsencode(path), ctypes.byref(ps)))
    try:
        return _unpack(ps)
    finally:
        _lib.jq_weight_set_destroy(ps)


def load_safetensors(path: str) -> Tuple[Dict[str, float], Dict[str, Tensor]]:
    """One ``.safetensors`` file -> (config of the ``config.txt`` beside it, or ``{}``; tensors by name)."""
    ps = ctypes.POINTER(_WeightSet)()
    capi.check(_lib.jq_weights_load_safetensors(os.fsencode(path), ctypes.byref(ps)))
    try:
        return _unpack(ps)
    finally:
        _lib.jq_weight_set_destroy(ps)


def fixture_to_safetensors(src_dir: str, dst_path: str) -> int:
    """Repacks a fixture directory (F32 and Q4_0 tensors alike) as one safetensors file; returns the number
    of tensors written.  ``config.txt`` is not part of the file: copy it beside ``dst_path``."""
    ps = ctypes.POINTER(_WeightSet)()
    capi.check(_lib.jq_weights_load_fixture(os.fsencode(src_dir), ctypes.byref(ps)))
    try:
        capi.check(_lib.jq_weights_save_safetensors(ps, os.fsencode(dst_path)))
        return int(ps.contents.num_tensors)
    finally:
        _lib.jq_weight_set_destroy(ps)


def write_safetensors(path: str, tensors: Mapping[str, "np.ndarray | Tensor"]) -> None:
    """Writes a safetensors file from arrays, in the layout of the reference's test helper
    (tests/fixture_utils.py:30-53): entries and data in name order, no ``__metadata__``."""
    import json
    import struct

    header, blobs, offset = {}, [], 0
    for name in sorted(tensors):
        t = tensors[name]
        if isinstance(t, Tensor) and t.dtype == DTYPE_Q4_0:
            rows, K = t.dims
            blob = np.ascontiguousarray(t.data, dtype=np.uint8).tobytes()
            key, entry = name + ".q4_0", {"dtype": "U8", "shape": [int(rows), int(K) // 32, capi.Q4_BYTES]}
        else:
            arr = np.ascontiguousarray(t.data if isinstance(t, Tensor) else t, dtype=np.float32)
            blob = arr.tobytes()
            key, entry = name, {"dtype": "F32", "shape": [int(d) for d in arr.shape]}
        entry["data_offsets"] = [offset, offset + len(blob)]
        header[key] = entry
        blobs.append(blob)
        offset += len(blob)
    head = json.dumps(header, separators=(",", ":")).encode("utf-8")
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for blob in blobs:
            f.write(blob)


def write_fixture(path: str, config: Mapping[str, float], tensors: Mapping[str, np.ndarray | Tensor]) -> None:
    """Writes a fixture directory.  float32 arrays become ``.f32`` files; ``Tensor`` values with
    ``DTYPE_Q4_0`` become ``.q4_0`` files with dims ``[rows, K]``."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.txt"), "w", encoding="utf-8") as f:
        for k, v in config.items():
            f.write("%s=%s\n" % (k, v))
    lines = []
    for name in sorted(tensors):
        t = tensors[name]
        if isinstance(t, Tensor) and t.dtype == DTYPE_Q4_0:
            fname = name.replace(".", "_") + ".q4_0"
            np.ascontiguousarray(t.data, dtype=np.uint8).tofile(os.path.join(path, fname))
            dims = t.dims
        else:
            arr = np.ascontiguousarray(t.data if isinstance(t, Tensor) else t, dtype=np.float32)
            fname = name.replace(".", "_") + ".f32"
            arr.tofile(os.path.join(path, fname))
            dims = arr.shape
        lines.append("%s %d %s %s" % (name, len(dims), " ".join(str(int(d)) for d in dims), fname))
    with open(os.path.join(path, "manifest.txt"), "w", encoding="utf-8") as f:
        f.write("\n".join(lines) + "\n")


def quantize_fixture(src: str, dst: str) -> int:
    """Offline quantizer: every linear weight of the fixture at ``src`` in Q4_0 form at ``dst``; returns
    how many tensors were converted.  Runs the library's CUDA quantizer."""
    n = ctypes.c_int(0)
    capi.check(_lib.jq_weights_quantize_fixture(os.fsencode(src), os.fsencode(dst), ctypes.byref(n)))
    return n.value


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 2:
        print(__doc__, file=sys.stderr)
        return 2
    if argv[1].endswith(".safetensors"):
        n = fixture_to_safetensors(argv[0], argv[1])
        print("wrote %d tensor(s) to %s" % (n, argv[1]))
        return 0
    n = quantize_fixture(argv[0], argv[1])
    print("quantized %d tensor(s) into %s" % (n, argv[1]))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
