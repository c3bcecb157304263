"""The range-checked debug build (``libjq_b200_check.so``, compiled with ``-DJQ_BOUNDS_CHECK``) on a GPU.

It stands in for a memory checker on boxes where none may run: its kernels check every global access against
the extent the entry point's shape arguments give the buffer, and every dynamic shared-memory offset against
the launch's size; an access outside is skipped and the fault word reads 3.  The test runs in a subprocess
(the library is chosen when ``jjjetson_ops_b200.capi`` is imported):

* every small and ragged shape of the parity suite through every kernel family, both block orders, the fused
  linear, the quantizer and both forms of the fused all-gather on one rank: right answers and fault word 0,
  i.e. no kernel indexes outside what its shapes describe;
* the same calls with every extent declared 64 bytes shorter than it is: the checks must fire (fault word 3),
  the kernels must return by themselves, and with the extents restored the next calls must be right again.
  Nothing faults or hangs here: the accesses that are skipped are in range in fact.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import importlib.util, os, sys
import numpy as np, torch
ROOT = sys.argv[1]
sys.path.insert(0, ROOT)
from jjjetson_ops_b200 import capi as c
from jjjetson_ops_b200.sharded import PeerBands, TaggedBands, segments_of
from oracle import jq_oracle as O
O.build()
assert c.lib().jq_bounds_checked() == 1, "not the range-checked build"
spec = importlib.util.spec_from_file_location("parity", os.path.join(ROOT, "tests", "test_gpu_parity.py"))
parity = importlib.util.module_from_spec(spec); spec.loader.exec_module(parity)
dev = torch.device("cuda:0")
up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
KERNELS = (c.KERNEL_GENERIC, c.KERNEL_GEMV_DP4A, c.KERNEL_GEMV_MMA, c.KERNEL_GEMM_MMA, c.KERNEL_GEMM_TC, c.KERNEL_GEMM_F16, c.KERNEL_AUTO)

def fault(clear=True):
    v = c.ctypes.c_int(0)
    c.lib().jq_device_fault(1 if clear else 0, c.ctypes.byref(v))
    return v.value

def run_shape(K, N, M, order, check_values):
    rng = np.random.default_rng(K + N + M)
    w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    x = rng.standard_normal((M, K), dtype=np.float32)
    wq = O.quantize_q4_0(w)
    d_w, d_x = up(wq), up(x)
    xq = c.quantize_q8_1(d_x, order, c.S_D_SUM_Q)                      # the device quantizer
    xq_ref = O.quantize_q8_1(x, order, c.S_D_SUM_Q)
    if check_values:
        assert np.array_equal(xq.cpu().numpy(), xq_ref), ("quantizer", K, M, order)
        ref = O.mul_mat_ref(wq, xq_ref, K, N, M, order)
    ran = 0
    for kernel in KERNELS:
        try:
            y = c.mul_mat_q4_0_q8_1(d_w, up(xq_ref), K, N, M, order, kernel).cpu().numpy()
        except c.JqError as e:
            assert e.status == c.ERR_UNSUPPORTED, e
            continue
        ran += 1
        if check_values:
            tol = 1e-3 if kernel == c.KERNEL_GEMM_F16 or (kernel == c.KERNEL_AUTO and M >= 64) else 1e-5
            assert O.err_max_rel(y, ref) <= tol, (K, N, M, order, kernel, O.err_max_rel(y, ref))
    assert ran >= 2
    y = c.linear_q4_0(d_w, d_x, N, c.S_D_SUM_Q).cpu().numpy()        # quantize + multiply through the dispatcher
    if check_values:
        ref1 = O.mul_mat_ref(wq, O.quantize_q8_1(x, c.ORDER_COL_KSUPER, c.S_D_SUM_Q), K, N, M, c.ORDER_COL_KSUPER)
        assert O.err_max_rel(y, ref1) <= (1e-3 if M >= 64 else 1e-5), ("linear", K, N, M)
    sums = c.block_sums(d_w, up(xq_ref), K, N, M, order).cpu().numpy()
    if check_values:
        assert np.array_equal(sums, O.block_sums(wq, xq_ref, K, N, M, order))

def run_gathers(check_values):
    rng = np.random.default_rng(9)
    K, N = 1024, 320
    w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    wq = O.quantize_q4_0(w); d_w = up(wq)
    K2, N2 = 256, 64
    wq2 = O.quantize_q4_0((rng.standard_normal((N2, K2), dtype=np.float32) * np.float32(0.02)).astype(np.float32)); d_w2 = up(wq2)
    for M in (1, 2, 5):
        x = rng.standard_normal((M, K), dtype=np.float32)
        ref = O.mul_mat_ref(wq, O.quantize_q8_1(x, c.ORDER_COL_KSUPER, c.S_D_SUM_Q), K, N, M, c.ORDER_COL_KSUPER)
        ws = torch.zeros(c.q8_1_bytes(K, M), dtype=torch.uint8, device=dev)
        pb = PeerBands(M, N, dev)
        pb.linear(d_w, up(x), ws, 0, N); pb.wait()
        y = pb.latest().cpu().numpy()
        if check_values: assert O.err_max_rel(y, ref) <= 1e-5
        pb.close()
        if M <= 2:
            tb = TaggedBands(M, N, dev)
            tb2 = TaggedBands(M, N2, dev, share_with=tb)
            tb.linear(d_w, K, 0, N, x=up(x))
            y1 = tb.read().cpu().numpy()
            tb2.linear(d_w2, K2, 0, N2, source=tb, seg_len=8, seg_stride=10)   # fed by the words of the first
            y2 = tb2.read().cpu().numpy()
            if check_values:
                assert O.err_max_rel(y1, ref) <= 1e-5
                x2 = segments_of(torch.from_numpy(y1), K2, 8, 10).numpy()
                ref2 = O.mul_mat_ref(wq2, O.quantize_q8_1(x2, c.ORDER_COL_KSUPER, c.S_D_SUM_Q), K2, N2, M, c.ORDER_COL_KSUPER)
                assert O.err_max_rel(y2, ref2) <= 1e-5
            tb2.close(); tb.close()

# ---- 1. every small and ragged shape: right answers, no range check fires ------------------------------
for (K, N, M) in parity.SMALL:
    for order in (0, 1):
        run_shape(K, N, M, order, True)
run_gathers(True)
assert fault() == 0, "a range check fired on a legal call"

# ---- 2. extents declared 64 bytes short: the checks fire, the kernels return, the device stays usable ---
c.set_option(c.OPT_WAIT_POLL_LIMIT, 20000)   # a skipped copy leaves its consumer waiting: keep that wait short
c.lib().jq_debug_set_extent_shrink(64)
fired = 0
for (K, N, M) in ((256, 33, 5), (1024, 257, 1), (2048, 130, 4), (512, 200, 33), (768, 256, 128)):
    run_shape(K, N, M, 1, False)
    f = fault()
    assert f == 3, (K, N, M, f)
    fired += 1
run_gathers(False)
assert fault() == 3
c.lib().jq_debug_set_extent_shrink(0)
c.set_option(c.OPT_WAIT_POLL_LIMIT, 0)
for (K, N, M) in ((256, 33, 5), (1024, 257, 1), (768, 256, 128)):
    run_shape(K, N, M, 1, True)
assert fault() == 0
print("BOUNDS-CHECK-OK", fired)
'''


def test_range_checked_build_small_shapes(cuda_device):
    lib = os.path.join(ROOT, "jjjetson_ops_b200", "libjq_b200_check.so")
    if not os.path.exists(lib):
        from jjjetson_ops_b200 import _build

        _build.build_check()
    env = dict(os.environ, JQ_B200_LIBRARY="libjq_b200_check.so")
    proc = subprocess.run([sys.executable, "-c", WORKER, ROOT], capture_output=True, text=True, env=env, timeout=900)
    assert proc.returncode == 0 and "BOUNDS-CHECK-OK" in proc.stdout, (proc.stdout[-2000:], proc.stderr[-4000:])
