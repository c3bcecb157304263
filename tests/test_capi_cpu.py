"""CPU-only checks of the C-ABI library: it loads, exports every declared symbol, and its
argument validation and pure-host functions behave.  No kernel is launched here."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = "".join(open(os.path.join(ROOT, "include", h)).read() for h in ("jq_b200.h", "jq_weights_io.h", "jq_model.h"))
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(jq_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = _declared_symbols()
    for must in ("jq_quantize_q8_1_device", "jq_mul_mat_q4_0_q8_1_device", "jq_linear_q4_0_device",
                 "jq_q8_1_host", "jq_parse_q8_1_output", "jq_mat_mul_q4_0_q8_1_host"):
        assert must in names


def test_library_exports_every_declared_symbol(native_lib):
    lib = ctypes.CDLL(native_lib.LIB_PATH)
    missing = [n for n in _declared_symbols() if not hasattr(lib, n)]
    assert not missing, missing
    # the reference's own four entry points stay linkable (q8_1.cu:148,197; mm_q4_0_q8_1.cu:318,394)
    for n in ("q8_1", "parse_q8_1_output", "mat_mul_q4_0_q8_1", "mat_mul_q4_0_q8_1_device"):
        assert hasattr(lib, n)


def test_sizes_and_strings(native_lib):
    c = native_lib
    assert c.q8_1_bytes(2048, 13) == 208 * 144  # tests/test_q8_1.py:75-79 of the reference
    assert c.q8_1_bytes(4096, 1) == 4608 and c.q8_1_bytes(160, 2) == 2 * 2 * 144
    assert c.q4_0_bytes(4096, 4096) == 9437184 and c.q4_0_bytes(28672, 8192) == 132120576
    assert c.q8_1_bytes(0, 5) == 0 and c.q4_0_bytes(-1, 32) == 0
    assert c.status_string(c.OK) == "ok" and "shape" in c.status_string(c.ERR_SHAPE)
    assert c.lib().jq_version() >= 100


def test_validation_needs_no_gpu(native_lib):
    c, L = native_lib, native_lib.lib()
    assert L.jq_quantize_q8_1_device(None, None, None, 33, 1, 0, 0) == c.ERR_SHAPE
    assert "33" in c.last_error()
    assert L.jq_quantize_q8_1_device(None, None, None, 64, 1, 7, 0) == c.ERR_INVALID_ARG
    assert L.jq_quantize_q8_1_device(None, None, None, 64, 1, 0, 9) == c.ERR_INVALID_ARG
    assert L.jq_quantize_q8_1_device(None, None, None, 64, 0, 0, 0) == c.OK  # empty input
    assert L.jq_quantize_q8_1_device(None, None, None, 64, 1, 0, 0) == c.ERR_INVALID_ARG  # null pointers
    assert L.jq_quantize_q8_1_device(None, 8, 16, 64, 1, 0, 0) == c.ERR_ALIGN
    # the multiply keeps the reference's two shape checks (mm_q4_0_q8_1.cu:331-340)
    assert L.jq_mul_mat_q4_0_q8_1_device(None, 2, 16, 4, 48, 8, 1, 1) == c.ERR_SHAPE
    assert "multiple of 32" in c.last_error()
    assert L.jq_mul_mat_q4_0_q8_1_device(None, 2, 16, 4, 96, 8, 1, 1) == c.ERR_SHAPE
    assert "block_q8_1_mmq" in c.last_error()
    assert L.jq_mul_mat_q4_0_q8_1_device(None, 2, 16, 4, 128, 0, 1, 1) == c.OK  # no rows
    assert L.jq_mul_mat_q4_0_q8_1_device(None, 3, 16, 4, 128, 8, 1, 1) == c.ERR_ALIGN
    assert L.jq_mul_mat_q4_0_q8_1_device(None, 2, 24, 4, 128, 8, 1, 1) == c.ERR_ALIGN
    assert L.jq_mul_mat_q4_0_q8_1_device(None, 2, 16, 4, 128, 8, -1, 1) == c.ERR_INVALID_ARG
    assert L.jq_linear_q4_0_device(None, 2, 16, 16, 4, 100, 8, 1, 1) == c.ERR_SHAPE
    dims = (ctypes.c_int * 4)(100, 1, 1, 1)
    assert L.jq_mat_mul_q4_0_q8_1_host(None, None, None, None, dims, 4, 8, 128) == c.ERR_SHAPE
    assert "must equal ncols_k" in c.last_error()  # mm_q4_0_q8_1.cu:326-330


def test_parse_is_pure_host_and_matches_oracle(native_lib, oracle):
    rng = np.random.default_rng(9)
    x = rng.standard_normal((3, 384), dtype=np.float32)
    raw = oracle.quantize_q8_1(x, oracle.ORDER_KSUPER_COL)
    nb = 9
    qs = np.empty((nb, 128), np.int8)
    d = np.empty((nb, 4), np.float32)
    s = np.empty((nb, 4), np.float32)
    rc = native_lib.lib().jq_parse_q8_1_output(raw.ctypes.data, qs.ctypes.data, d.ctypes.data, s.ctypes.data, nb)
    assert rc == 0
    qo, do, so = oracle.parse_q8_1(raw, nb)
    assert np.array_equal(qs, qo) and np.array_equal(d, do) and np.array_equal(s, so)


def test_reference_named_modules_import_and_validate(native_lib):
    import jjjetson_ops_b200 as pkg

    q8, mm = pkg.import_reference_modules()
    assert hasattr(q8, "quantize") and hasattr(q8, "parse") and hasattr(mm, "mmq")
    with pytest.raises(ValueError):
        q8.quantize(np.zeros(64, np.float64), np.zeros(144, np.uint8), [64, 1, 1, 1])  # wrong dtype
    with pytest.raises(ValueError):
        q8.quantize(np.zeros(256, np.float32), np.zeros(100, np.uint8), [256, 1, 1, 1])  # output too small
    with pytest.raises(ValueError):
        mm.mmq(weight_q4_0=np.zeros(10, np.uint8), input=np.zeros(128, np.float32),
               quant_workspace=np.zeros(144, np.uint8), output=np.zeros(8, np.float32),
               input_dims=[128, 1, 1, 1], nrows_out=8, ncols_k=128)  # weight buffer too small
    qs, d, s = q8.parse(np.zeros(288, np.uint8), 2)
    assert qs.shape == (2, 128) and d.shape == (2, 4) and s.dtype == np.float32


def test_options_round_trip():
    """Process-wide switches are plain host state: set, read back, reject unknown ones."""
    from jjjetson_ops_b200 import capi

    for opt in (capi.OPT_STATIC_WEIGHTS, capi.OPT_PREFILL_EXACT):
        assert capi.get_option(opt) == 0  # both default to off
        capi.set_option(opt, 1)
        try:
            assert capi.get_option(opt) == 1
        finally:
            capi.set_option(opt, 0)
        assert capi.get_option(opt) == 0
    with pytest.raises(capi.JqError):
        capi.set_option(99, 1)


def test_public_headers_are_plain_c():
    """The boundary is a C ABI: every public header compiles as C99 on its own, warnings included."""
    import subprocess

    inc = os.path.join(ROOT, "include")
    for h in sorted(os.listdir(inc)):
        if not h.endswith(".h"):
            continue
        r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", "-I", inc, "-x", "c", "-"],
                           input='#include "%s"\n' % h, capture_output=True, text=True)
        assert r.returncode == 0, (h, r.stderr)
