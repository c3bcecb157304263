"""GPU parity against the reference's own CUDA operators, rebuilt unmodified for sm_100a.

``oracle/_ref/libjjj_ref.so`` is compiled by ``make -C oracle ref`` from the reference's
src/cuda/q8_1.cu and src/cuda/mm_q4_0_q8_1.cu where they lie; it is a checker only.  The same
run also pins the CPU oracle to the reference: its quantized blocks must be bit-identical to what
the reference kernel writes, and its multiply must reproduce the reference kernel's fp32 outputs.
"""
import ctypes
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libjjj_ref.so")


class _StdVectorInt(ctypes.Structure):
    """libstdc++ layout of std::vector<int>: begin, end, end of storage."""

    _fields_ = [("begin", ctypes.c_void_p), ("end", ctypes.c_void_p), ("cap", ctypes.c_void_p)]


@pytest.fixture(scope="module")
def ref(cuda_device):
    if not os.path.exists(REF_LIB):
        pytest.skip("reference kernels not built (make -C oracle ref)")
    lib = ctypes.CDLL(REF_LIB)
    lib.q8_1.restype = None
    lib.q8_1.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(_StdVectorInt)]
    lib.mat_mul_q4_0_q8_1_device.restype = None
    lib.mat_mul_q4_0_q8_1_device.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                             ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return lib


def ref_q8_1(lib, x_mk: np.ndarray) -> np.ndarray:
    """Calls the reference's q8_1() (src/cuda/q8_1.cu:148) on [M][K] rows."""
    M, K = x_mk.shape
    dims = (ctypes.c_int * 4)(K, M, 1, 1)
    base = ctypes.addressof(dims)
    vec = _StdVectorInt(base, base + 16, base + 16)
    out = np.zeros(M * ((K + 127) // 128) * 144, dtype=np.uint8)
    x = np.ascontiguousarray(x_mk, dtype=np.float32)
    lib.q8_1(x.ctypes.data, out.ctypes.data, ctypes.byref(vec))
    return out


def ref_mul_mat_device(lib, torch, d_w, d_xq, K, N, M):
    y = torch.empty((M, N), dtype=torch.float32, device=d_w.device)
    lib.mat_mul_q4_0_q8_1_device(d_w.data_ptr(), d_xq.data_ptr(), y.data_ptr(), K, N, M,
                                 torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return y


@pytest.mark.parametrize("M,K", [(13, 2048), (1, 4096), (4, 1024)])
def test_quantizer_bit_identical_to_reference_kernel(ref, native_lib, oracle, cuda_device, M, K):
    import torch

    rng = np.random.default_rng(M * 1000 + K)
    x = rng.standard_normal((M, K), dtype=np.float32)  # no all-zero group: there the reference stores +inf
    want = ref_q8_1(ref, x)
    got = native_lib.quantize_q8_1(torch.from_numpy(x).to(cuda_device), native_lib.ORDER_KSUPER_COL,
                                   native_lib.S_SUM_X).cpu().numpy()
    assert np.array_equal(got, want)
    assert np.array_equal(oracle.quantize_q8_1(x, oracle.ORDER_KSUPER_COL, oracle.S_SUM_X), want)  # pins the oracle


@pytest.mark.parametrize("K,N,M", [(4096, 4096, 1), (4096, 11008, 8), (1024, 100, 5), (8192, 512, 1), (2048, 256, 64)])
def test_multiply_matches_reference_kernel(ref, native_lib, oracle, cuda_device, K, N, M):
    import torch

    c = native_lib
    rng = np.random.default_rng(K + N + M)
    w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    x = rng.standard_normal((M, K), dtype=np.float32)
    wq = oracle.quantize_q4_0(w)
    # the reference kernel reads block m*(K/128) + k/128 (mm_q4_0_q8_1.cu:230): feed it that order
    xq = oracle.quantize_q8_1(x, oracle.ORDER_COL_KSUPER, oracle.S_SUM_X)
    d_w, d_xq = torch.from_numpy(wq).to(cuda_device), torch.from_numpy(xq).to(cuda_device)
    y_ref = ref_mul_mat_device(ref, torch, d_w, d_xq, K, N, M).cpu().numpy()
    y_orc = oracle.mul_mat_ref(wq, xq, K, N, M, oracle.ORDER_COL_KSUPER)
    # the oracle restates the kernel's arithmetic and accumulation order: same bits expected
    assert oracle.err_max_rel(y_orc, y_ref) <= 1e-7, "oracle drifted from the reference kernel"
    y = c.mul_mat_q4_0_q8_1(d_w, d_xq, K, N, M, c.ORDER_COL_KSUPER).cpu().numpy()
    if M >= 64:
        # the automatic choice for 64 columns and more rounds the scaled operands to fp16: 1e-3; the exact-integer
        # kernels behind JQ_OPT_PREFILL_EXACT meet the same bar as the decode kernels
        assert oracle.err_max_rel(y, y_ref) <= 1e-3
        c.set_option(c.OPT_PREFILL_EXACT, 1)
        try:
            y_exact = c.mul_mat_q4_0_q8_1(d_w, d_xq, K, N, M, c.ORDER_COL_KSUPER).cpu().numpy()
        finally:
            c.set_option(c.OPT_PREFILL_EXACT, 0)
        assert oracle.err_max_rel(y_exact, y_ref) <= 1e-5
    else:
        assert oracle.err_max_rel(y, y_ref) <= 1e-5
    # drop-in symbol with the reference's own name and signature
    lib = c.lib()
    lib.mat_mul_q4_0_q8_1_device.restype = None
    lib.mat_mul_q4_0_q8_1_device.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                             ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    y2 = torch.empty((M, N), dtype=torch.float32, device=cuda_device)
    lib.mat_mul_q4_0_q8_1_device(d_w.data_ptr(), d_xq.data_ptr(), y2.data_ptr(), K, N, M,
                                 torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert np.array_equal(y2.cpu().numpy(), y)
