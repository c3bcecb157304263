"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.

Bars: bit-exact for the int8 activations, the fp16 (d, s) pairs, the Q4_0 bytes and the int32
block sums; max|y - ref| / max|ref| <= 1e-5 against the oracle's reference-formula multiply on
the same quantized inputs (only fp32 summation order differs) and <= 1e-3 against
dequantise-then-matmul in float64 (with s = d * sum(q)).  The one exception is what the automatic
choice runs for prefill batches of 64 columns and more, the fp16-operand GEMM: it rounds the scaled
operands to fp16 and is held to <= 1e-3 against both; the same cases run once more with
JQ_OPT_PREFILL_EXACT, at the 1e-5 bar.
"""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TOL_FORMULA = 1e-5  # same formula, different fp32 summation order
TOL_DEQUANT = 1e-3  # the accuracy target against dequantise-then-matmul
TOL_FP16_OPERANDS = 1e-3  # the fp16-operand prefill GEMM against the reference formula


def _formula_tol(c, kernel, K, M):
    """The bar against the reference formula for what `kernel` runs on this shape."""
    takes_fp16 = kernel == c.KERNEL_GEMM_F16 or (kernel == c.KERNEL_AUTO and M >= 64 and K % 256 == 0 and
                                                 c.get_option(c.OPT_PREFILL_EXACT) == 0)
    return TOL_FP16_OPERANDS if takes_fp16 else TOL_FORMULA


class _exact_prefill:
    """`with _exact_prefill(c):` - the automatic choice is an exact-integer kernel inside the block."""

    def __init__(self, c):
        self.c = c

    def __enter__(self):
        self.c.set_option(self.c.OPT_PREFILL_EXACT, 1)

    def __exit__(self, *exc):
        self.c.set_option(self.c.OPT_PREFILL_EXACT, 0)


@pytest.fixture(scope="module")
def env(native_lib, oracle, cuda_device):
    import torch

    class Env:
        c = native_lib
        O = oracle
        dev = cuda_device
        t = torch

        def up(self, a):
            return torch.from_numpy(np.ascontiguousarray(a)).to(cuda_device)

    e = Env()
    yield e
    assert native_lib.device_fault(clear=True) == 0  # no kernel gave up on a bounded wait


def _case(rng, K, N, M, sigma=0.02):
    w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(sigma)).astype(np.float32)
    x = rng.standard_normal((M, K), dtype=np.float32)
    return w, x


# ------------------------------------------------------------------------------- quantizers
@pytest.mark.parametrize("order", [0, 1])
@pytest.mark.parametrize("s_mode", [0, 1])
@pytest.mark.parametrize("shape", [(1, 128), (1, 4096), (13, 2048), (5, 640), (2, 160), (3, 32), (64, 11008)])
def test_quantize_q8_1_bit_exact(env, order, s_mode, shape):
    M, K = shape
    rng = np.random.default_rng(100 + M + K)
    x = rng.standard_normal((M, K), dtype=np.float32)
    if K >= 96:
        x[M // 2, 64:96] = 0.0  # all-zero group: d = 0 (not the reference's +inf)
    x[0, 0] = 300.0
    raw = env.c.quantize_q8_1(env.up(x), order, s_mode).cpu().numpy()
    assert np.array_equal(raw, env.O.quantize_q8_1(x, order, s_mode))


def test_quantize_q8_1_reference_golden(env):
    """The reference's own test case (tests/test_q8_1.py:65-123) on the device entry."""
    g = np.load(os.path.join(GOLDEN, "q8_1_ref_seed24.npz"))
    np.random.seed(24)
    x = np.ascontiguousarray(np.random.randn(2048, 13, 1, 1).astype(np.float32)[:, :, 0, 0].T)
    raw = env.c.quantize_q8_1(env.up(x), env.c.ORDER_KSUPER_COL, env.c.S_SUM_X).cpu().numpy()
    qs, d, s = env.O.parse_q8_1(raw, 208)
    assert np.array_equal(qs, g["a_qs"])
    assert np.allclose(d, g["a_scale"], atol=1e-5) and np.allclose(s, g["a_sum"], atol=1e-2)


def test_quantize_q4_0_bit_exact(env):
    from tests.golden.make_q4_0_gguf_golden import make_input

    w = make_input()
    got = env.c.quantize_q4_0(env.up(w)).cpu().numpy()
    assert np.array_equal(got, np.load(os.path.join(GOLDEN, "q4_0_gguf_seed5.npz"))["q4_0"])
    rng = np.random.default_rng(12)
    w2 = (rng.standard_normal((333, 1024), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    w2[7, 96:128] = 0.0
    assert np.array_equal(env.c.quantize_q4_0(env.up(w2)).cpu().numpy(), env.O.quantize_q4_0(w2))


# ------------------------------------------------------------------------------- block sums
@pytest.mark.parametrize("order", [0, 1])
def test_block_sums_bit_exact(env, order):
    rng = np.random.default_rng(13)
    K, N, M = 512, 100, 5
    w, x = _case(rng, K, N, M)
    wq = env.O.quantize_q4_0(w)
    xq = env.O.quantize_q8_1(x, order, 1)
    got = env.c.block_sums(env.up(wq), env.up(xq), K, N, M, order).cpu().numpy()
    assert np.array_equal(got, env.O.block_sums(wq, xq, K, N, M, order))


# ------------------------------------------------------------------------------- the multiply
def _check_mul_mat(env, wq, x, K, N, M, kernel, order, s_mode, rows=None):
    """Runs the kernel on (wq, quantized x) and compares against the oracle."""
    xq = env.O.quantize_q8_1(x, order, s_mode)
    y = env.c.mul_mat_q4_0_q8_1(env.up(wq), env.up(xq), K, N, M, order, kernel).cpu().numpy()
    assert y.shape == (M, N) and np.isfinite(y).all()
    if rows is None:
        ref = env.O.mul_mat_ref(wq, xq, K, N, M, order)
        deq = env.O.mul_mat_deq_f64(wq, xq, K, N, M, order)
        ysel = y
    else:  # full-size case: the oracle checks a sample of weight rows
        wsel = np.ascontiguousarray(wq.reshape(N, -1)[rows])
        ref = env.O.mul_mat_ref(wsel, xq, K, len(rows), M, order)
        deq = env.O.mul_mat_deq_f64(wsel, xq, K, len(rows), M, order)
        ysel = y[:, rows]
    e_ref = env.O.err_max_rel(ysel, ref)
    assert e_ref <= _formula_tol(env.c, kernel, K, M), (e_ref, kernel)
    if s_mode == env.c.S_D_SUM_Q:
        e_deq = env.O.err_max_rel(ysel, deq)
        assert e_deq <= TOL_DEQUANT, (e_deq, kernel)
    return y


SMALL = [(128, 32, 1), (256, 32, 2), (256, 33, 5), (512, 100, 8), (768, 7, 3), (1024, 257, 1), (256, 1, 1),
         (2048, 130, 4), (4096, 300, 2), (8192, 70, 1), (11008, 50, 1), (16384, 40, 1), (1280, 64, 8),
         (512, 200, 33), (1024, 129, 130), (256, 64, 300), (768, 256, 128), (4096, 384, 17),
         (1024, 96, 9), (2048, 64, 32), (768, 40, 24), (6144, 33, 12), (512, 72, 48), (512, 72, 49)]


@pytest.mark.parametrize("K,N,M", SMALL)
@pytest.mark.parametrize("order", [0, 1])
def test_mul_mat_small_shapes_all_kernels(env, K, N, M, order):
    c = env.c
    rng = np.random.default_rng(K + N + M)
    w, x = _case(rng, K, N, M)
    wq = env.O.quantize_q4_0(w)
    ran = []
    for kernel in (c.KERNEL_GENERIC, c.KERNEL_GEMV_DP4A, c.KERNEL_GEMV_MMA, c.KERNEL_GEMM_MMA, c.KERNEL_GEMM_TC, c.KERNEL_AUTO):
        try:
            _check_mul_mat(env, wq, x, K, N, M, kernel, order, c.S_D_SUM_Q)
            ran.append(kernel)
        except c.JqError as e:
            assert e.status == c.ERR_UNSUPPORTED, e  # a family may refuse a shape, never fail on it
    assert c.KERNEL_GENERIC in ran and c.KERNEL_AUTO in ran
    if K % 256 == 0 and M <= 2 and K <= 16384 and not (M == 2 and K > 8192):
        assert c.KERNEL_GEMV_DP4A in ran
    if K % 256 == 0 and K <= 6144 and M <= 8:
        assert c.KERNEL_GEMV_MMA in ran
    if K % 256 == 0:
        assert c.KERNEL_GEMM_MMA in ran and c.KERNEL_GEMM_TC in ran


def test_mul_mat_reference_s_mode(env):
    """With the reference's s = sum(x) the kernels still follow the reference formula exactly;
    only the distance to dequantise-then-matmul grows (about 1e-2)."""
    c = env.c
    rng = np.random.default_rng(77)
    K, N, M = 1024, 96, 3
    w, x = _case(rng, K, N, M)
    wq = env.O.quantize_q4_0(w)
    for kernel in (c.KERNEL_GENERIC, c.KERNEL_GEMV_MMA, c.KERNEL_AUTO):
        _check_mul_mat(env, wq, x, K, N, M, kernel, c.ORDER_COL_KSUPER, c.S_SUM_X)


def test_mul_mat_empty_and_degenerate(env):
    c, t = env.c, env.t
    w = t.zeros(18 * 4 * 8, dtype=t.uint8, device=env.dev)
    xq = t.zeros(144, dtype=t.uint8, device=env.dev)
    assert c.mul_mat_q4_0_q8_1(w, xq, 128, 0, 1).shape == (1, 0)
    assert c.mul_mat_q4_0_q8_1(w, xq, 128, 8, 0).shape == (0, 8)
    y = c.mul_mat_q4_0_q8_1(w, xq, 128, 8, 1)  # all-zero blocks: d = 0 everywhere -> exact zeros
    assert not y.cpu().numpy().any()
    with pytest.raises(c.JqError) as ei:
        c.mul_mat_q4_0_q8_1(w, xq, 96, 8, 1)
    assert ei.value.status == c.ERR_SHAPE


def _config_case(env, cfg, linear, M, rows=None):
    from jjjetson_ops_b200 import synth

    w, x, lin = synth.make_linear_case(cfg, linear, M)
    wq = env.c.quantize_q4_0(env.up(w)).cpu().numpy()  # the device quantizer is itself checked above
    check = slice(None) if rows is None and w.shape[0] <= 4096 else rows
    if check is not None:  # the synthetic weights really are what the oracle's quantizer makes of them
        assert np.array_equal(wq[check], env.O.quantize_q4_0(np.ascontiguousarray(w[check])))
    return wq, x, lin


def test_config1_decode_gemv(env):
    c = env.c
    wq, x, lin = _config_case(env, 1, 0, 1)
    for kernel in (c.KERNEL_AUTO, c.KERNEL_GEMV_DP4A, c.KERNEL_GEMV_MMA, c.KERNEL_GENERIC):
        _check_mul_mat(env, wq, x, lin.K, lin.N, 1, kernel, c.ORDER_COL_KSUPER, c.S_D_SUM_Q)


@pytest.mark.parametrize("M", [1, 2, 4, 8])
def test_config2_decode_batch(env, M):
    c = env.c
    wq, x, lin = _config_case(env, 2, 0, M)
    kernels = [c.KERNEL_AUTO, c.KERNEL_GEMV_MMA] + ([c.KERNEL_GEMV_DP4A] if M <= 2 else [])
    for kernel in kernels:
        _check_mul_mat(env, wq, x, lin.K, lin.N, M, kernel, c.ORDER_COL_KSUPER, c.S_D_SUM_Q)


def test_config3_prefill(env):
    c = env.c
    wq, x, lin = _config_case(env, 3, 0, 512)
    _check_mul_mat(env, wq, x, lin.K, lin.N, 512, c.KERNEL_AUTO, c.ORDER_COL_KSUPER, c.S_D_SUM_Q)
    _check_mul_mat(env, wq, x, lin.K, lin.N, 512, c.KERNEL_AUTO, c.ORDER_KSUPER_COL, c.S_D_SUM_Q)
    with _exact_prefill(c):
        _check_mul_mat(env, wq, x, lin.K, lin.N, 512, c.KERNEL_AUTO, c.ORDER_COL_KSUPER, c.S_D_SUM_Q)
    for kernel in (c.KERNEL_GEMM_TC, c.KERNEL_GEMM_MMA):
        _check_mul_mat(env, wq, x, lin.K, lin.N, 512, kernel, c.ORDER_COL_KSUPER, c.S_D_SUM_Q)


def test_config4_large_shapes(env):
    c = env.c
    rows = np.sort(np.random.default_rng(44).choice(28672, size=96, replace=False))
    wq, x, lin = _config_case(env, 4, 0, None, rows=rows)
    _check_mul_mat(env, wq, x[:1], lin.K, lin.N, 1, c.KERNEL_AUTO, c.ORDER_COL_KSUPER, c.S_D_SUM_Q, rows=rows)
    _check_mul_mat(env, wq, x, lin.K, lin.N, 2048, c.KERNEL_AUTO, c.ORDER_COL_KSUPER, c.S_D_SUM_Q, rows=rows)
    with _exact_prefill(c):
        _check_mul_mat(env, wq, x, lin.K, lin.N, 2048, c.KERNEL_AUTO, c.ORDER_COL_KSUPER, c.S_D_SUM_Q, rows=rows)


@pytest.mark.parametrize("M", [1, 128])
def test_config5_layer_chain(env, M):
    c = env.c
    for linear in range(5):
        rows = np.sort(np.random.default_rng(50 + linear).choice(4096, size=128, replace=False))
        wq, x, lin = _config_case(env, 5, linear, M, rows=rows)
        _check_mul_mat(env, wq, x, lin.K, lin.N, M, c.KERNEL_AUTO, c.ORDER_COL_KSUPER, c.S_D_SUM_Q, rows=rows)
        if M >= 64:
            with _exact_prefill(c):
                _check_mul_mat(env, wq, x, lin.K, lin.N, M, c.KERNEL_AUTO, c.ORDER_COL_KSUPER, c.S_D_SUM_Q, rows=rows)


# ------------------------------------------------------------------------------- fused linear
@pytest.mark.parametrize("K,N,M", [(4096, 4096, 1), (4096, 11008, 2), (4096, 11008, 8), (8192, 2048, 1),
                                   (11008, 4096, 1), (2048, 100, 5), (4096, 512, 64), (1280, 96, 3)])
@pytest.mark.parametrize("s_mode", [0, 1])
def test_linear_fused_equals_two_steps(env, K, N, M, s_mode):
    c = env.c
    rng = np.random.default_rng(K * 3 + N + M)
    w, x = _case(rng, K, N, M)
    wq = env.O.quantize_q4_0(w)
    d_w, d_x = env.up(wq), env.up(x)
    ws = env.t.zeros(c.q8_1_bytes(K, M), dtype=env.t.uint8, device=env.dev)
    y = c.linear_q4_0(d_w, d_x, N, s_mode, ws=ws).cpu().numpy()
    xq = env.O.quantize_q8_1(x, c.ORDER_COL_KSUPER, s_mode)
    assert np.array_equal(ws.cpu().numpy(), xq)  # the workspace holds the quantized activations
    y2 = c.mul_mat_q4_0_q8_1(d_w, env.up(xq), K, N, M, c.ORDER_COL_KSUPER).cpu().numpy()
    assert np.array_equal(y, y2)  # same kernels, same arithmetic: identical bits
    assert env.O.err_max_rel(y, env.O.mul_mat_ref(wq, xq, K, N, M)) <= _formula_tol(c, c.KERNEL_AUTO, K, M)


@pytest.mark.parametrize("static_weights", [0, 1])
@pytest.mark.parametrize("M", [1, 4])
def test_dependent_chain_back_to_back(env, static_weights, M):
    """Three linears queued without any synchronisation, each consuming the previous output.  With
    JQ_OPT_STATIC_WEIGHTS the kernels overlap their weight stream with the predecessor's tail; the
    activations must still be ordered, so the chain has to equal the step-by-step oracle chain."""
    c = env.c
    rng = np.random.default_rng(300 + M)
    dims = [(4096, 4096), (4096, 2048), (2048, 512)]  # (K, N)
    ws_host = [env.O.quantize_q4_0((rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.03)).astype(np.float32))
               for k, n in dims]
    x0 = rng.standard_normal((M, dims[0][0]), dtype=np.float32)
    d_ws = [env.up(w) for w in ws_host]
    d_x = env.up(x0)
    scratch = [env.t.zeros(c.q8_1_bytes(k, M), dtype=env.t.uint8, device=env.dev) for k, _ in dims]
    c.set_option(c.OPT_STATIC_WEIGHTS, static_weights)
    try:
        assert c.get_option(c.OPT_STATIC_WEIGHTS) == static_weights
        for _ in range(3):  # repeat so that kernels of different rounds overlap too
            h = d_x
            for (k, n), d_w, ws in zip(dims, d_ws, scratch):
                h = c.linear_q4_0(d_w, h, n, c.S_D_SUM_Q, ws=ws)
        got = h.cpu().numpy()
    finally:
        c.set_option(c.OPT_STATIC_WEIGHTS, 0)
    ref = x0
    for (k, n), w in zip(dims, ws_host):
        xq = env.O.quantize_q8_1(ref, c.ORDER_COL_KSUPER, c.S_D_SUM_Q)
        ref = env.O.mul_mat_ref(w, xq, k, n, M)
    # fp32 summation order differs per layer and requantization can flip a rounding: loose bound
    assert env.O.err_max_rel(got, ref) <= 2e-2
    # the last layer, fed the GPU's own input to it, must match tightly
    h2 = d_x
    for (k, n), d_w, ws in zip(dims[:2], d_ws[:2], scratch[:2]):
        h2 = c.linear_q4_0(d_w, h2, n, c.S_D_SUM_Q, ws=ws)
    x_last = h2.cpu().numpy()
    xq = env.O.quantize_q8_1(x_last, c.ORDER_COL_KSUPER, c.S_D_SUM_Q)
    assert env.O.err_max_rel(got, env.O.mul_mat_ref(ws_host[2], xq, dims[2][0], dims[2][1], M)) <= TOL_FORMULA


def test_multiply_is_linear_in_the_integer_activations(env):
    """Size-independent property at full cfg2 size: block sums of q1 + q2 equal the sum of block
    sums, checked through the real kernels with unit scales (d = 1, s = 0 -> y = d4 * sumi summed)."""
    c = env.c
    from jjjetson_ops_b200 import synth

    w, _, lin = synth.make_linear_case(2, 0, 1)
    d_w = c.quantize_q4_0(env.up(w))
    K, N = lin.K, lin.N
    rng = np.random.default_rng(91)
    qa = rng.integers(-60, 60, size=K, dtype=np.int8)
    qb = rng.integers(-60, 60, size=K, dtype=np.int8)

    def blocks(q):
        b = np.zeros((K // 128, 144), dtype=np.uint8)
        b[:, :16] = np.tile(np.array([1.0, 0.0], dtype=np.float16).view(np.uint8), 4)
        b[:, 16:] = q.reshape(K // 128, 128).view(np.uint8)
        return b.reshape(-1)

    ys = [c.mul_mat_q4_0_q8_1(d_w, env.up(blocks(q)), K, N, 1).cpu().numpy().astype(np.float64)
          for q in (qa, qb, (qa + qb).astype(np.int8))]
    scale = np.abs(ys[2]).max()
    assert np.abs(ys[0] + ys[1] - ys[2]).max() <= 1e-5 * scale


# ------------------------------------------------------------------------------- host entry points
def test_reference_module_flow_q8_1(env):
    """The reference's tests/test_q8_1.py:65-123, against this library's q8_1_me module."""
    import jjjetson_ops_b200 as pkg

    q8_1_me, _ = pkg.import_reference_modules()
    np.random.seed(24)
    input_np = np.asfortranarray(np.random.randn(2048, 13, 1, 1).astype(np.float32))
    n_blocks = 13 * ((2048 + 127) // 128)
    q_output = np.zeros(n_blocks * 144, dtype=np.uint8)
    q8_1_me.quantize(input_np, q_output, [2048, 13, 1, 1])
    qs, scale, ssum = q8_1_me.parse(q_output, n_blocks)
    g = np.load(os.path.join(GOLDEN, "q8_1_ref_seed24.npz"))
    assert qs.shape == g["a_qs"].shape and np.all(qs == g["a_qs"])
    assert np.allclose(scale, g["a_scale"], atol=1e-5) and np.allclose(ssum, g["a_sum"], atol=1e-2)


@pytest.mark.parametrize("M", [1, 5])
def test_reference_module_flow_mmq(env, M):
    import jjjetson_ops_b200 as pkg

    _, mm = pkg.import_reference_modules()
    rng = np.random.default_rng(5 + M)
    K, N = 1024, 200
    w, x = _case(rng, K, N, M)
    wq = env.O.quantize_q4_0(w)
    ws = np.zeros(env.c.q8_1_bytes(K, M), dtype=np.uint8)
    y = np.zeros((M, N), dtype=np.float32)
    mm.mmq(wq.reshape(-1), x, ws, y, [K, M, 1, 1], N, K)
    xq = env.O.quantize_q8_1(x, env.c.ORDER_KSUPER_COL, env.c.S_SUM_X)  # what q8_1() writes
    assert np.array_equal(ws, xq)
    assert env.O.err_max_rel(y, env.O.mul_mat_ref(wq, xq, K, N, M, env.c.ORDER_KSUPER_COL)) <= TOL_FORMULA
    y2 = np.zeros_like(y)
    mm.mmq(wq.reshape(-1), x, ws, y2, [K, M, 1, 1], N, K, s_mode=1)
    xq1 = env.O.quantize_q8_1(x, env.c.ORDER_KSUPER_COL, env.c.S_D_SUM_Q)
    assert env.O.err_max_rel(y2, env.O.mul_mat_deq_f64(wq, xq1, K, N, M, env.c.ORDER_KSUPER_COL)) <= TOL_DEQUANT


def test_resident_weights_host_linear(env):
    c = env.c
    rng = np.random.default_rng(31)
    K, N = 4096, 1000
    w, x = _case(rng, K, N, 8)
    wq = env.O.quantize_q4_0(w)
    rw = c.ResidentWeights(wq, N, K)
    try:
        for M in (1, 8, 3):
            xin = np.ascontiguousarray(x[:M])
            y = np.zeros((M, N), dtype=np.float32)
            ws = np.zeros(c.q8_1_bytes(K, M), dtype=np.uint8)
            rw.linear(xin.ctypes.data, y.ctypes.data, M, c.S_D_SUM_Q, ws.ctypes.data)
            xq = env.O.quantize_q8_1(xin, c.ORDER_COL_KSUPER, c.S_D_SUM_Q)
            assert np.array_equal(ws, xq)
            assert env.O.err_max_rel(y, env.O.mul_mat_ref(wq, xq, K, N, M)) <= TOL_FORMULA
    finally:
        rw.close()


def test_resident_weights_host_linear_pinned_buffers(env):
    """Pinned (mapped) host buffers take the path without copy-engine transfers: the quantizer reads
    x over the bus, a copy kernel writes y back.  Same results as with pageable buffers."""
    c, t = env.c, env.t
    rng = np.random.default_rng(32)
    K, N = 4096, 11008
    w, x = _case(rng, K, N, 8)
    wq = env.O.quantize_q4_0(w)
    rw = c.ResidentWeights(wq, N, K)
    try:
        for M in (1, 8, 2):
            x_pin = t.from_numpy(np.ascontiguousarray(x[:M])).pin_memory()
            y_pin = t.zeros((M, N), dtype=t.float32).pin_memory()
            for _ in range(2):  # second call reuses the cached buffer attributes
                y_pin.zero_()
                rw.linear(x_pin.data_ptr(), y_pin.data_ptr(), M, c.S_D_SUM_Q)
                xq = env.O.quantize_q8_1(x[:M], c.ORDER_COL_KSUPER, c.S_D_SUM_Q)
                assert env.O.err_max_rel(y_pin.numpy(), env.O.mul_mat_ref(wq, xq, K, N, M)) <= TOL_FORMULA
            # pageable output with pinned input, and the other way round
            y_page = np.zeros((M, N), dtype=np.float32)
            rw.linear(x_pin.data_ptr(), y_page.ctypes.data, M, c.S_D_SUM_Q)
            assert np.array_equal(y_page, y_pin.numpy())
            x_page = np.ascontiguousarray(x[:M])
            y_pin.zero_()
            rw.linear(x_page.ctypes.data, y_pin.data_ptr(), M, c.S_D_SUM_Q)
            assert env.O.err_max_rel(y_pin.numpy(), y_page) <= TOL_FORMULA
    finally:
        rw.close()


def test_device_hw_info(env):
    info = env.c.query_device_hw_info(0)
    assert info["sm_count"] > 0 and info["cc_major"] >= 10, info
    assert info["peak_dram_gbs"] > 1000 and info["peak_int8_dense_tops"] > 1000


def test_show_device_info_prints_the_reference_line_format(native_lib, cuda_device, capsys):
    from jjjetson_ops_b200 import show_device_info

    assert show_device_info.main(["0"]) == 0
    out = capsys.readouterr().out.strip().splitlines()
    assert all(line.startswith("[DeviceHwInfo] ") for line in out)
    keys = {line.split("] ", 1)[1].split(":", 1)[0] for line in out}
    for k in ("device_id", "name", "compute_capability", "sm_count", "peak_dram_theoretical", "peak_tc_int8_dense_tops_nominal"):
        assert k in keys
    assert show_device_info.main(["4096"]) == 1  # no such device: message on stderr, status 1, no exit()


def test_trace_stamps_of_a_decode_launch_are_ordered(native_lib, cuda_device):
    """jq_trace_enable: the next launch of a streaming GEMV writes eight increasing time stamps per CTA."""
    import torch

    c = native_lib
    K, N = 1024, 2048
    rng = np.random.default_rng(3)
    w = torch.from_numpy(rng.integers(0, 256, size=c.q4_0_bytes(N, K), dtype=np.uint8)).to(cuda_device)
    blocks = w.view(N, K // 32, 18)
    blocks[:, :, 0] = 0
    blocks[:, :, 1] = 0x20
    x = torch.from_numpy(rng.standard_normal((1, K)).astype(np.float32)).to(cuda_device)
    ref = c.linear_q4_0(w, x, N)
    buf = torch.zeros(2 * 512 * 8, dtype=torch.int64, device=cuda_device)
    c.check(c.lib().jq_trace_enable(buf.data_ptr(), 2))
    y = c.linear_q4_0(w, x, N)
    torch.cuda.synchronize()
    c.check(c.lib().jq_trace_enable(None, 0))
    assert torch.equal(y, ref)  # tracing does not change the result
    t = buf.cpu().numpy()[: 512 * 8].reshape(512, 8)
    live = t[t[:, 0] > 0]
    assert len(live) >= 1 and len(live) <= 296
    # start <= predecessor finished <= activations staged <= first stage seen <= last stage seen <= done
    for a, b in ((0, 3), (3, 4), (4, 5), (5, 6), (6, 7)):
        assert (live[:, a] <= live[:, b]).all(), (a, b)
    assert (buf.cpu().numpy()[512 * 8:] == 0).all()  # only one launch happened
    y2 = c.linear_q4_0(w, x, N)  # tracing is off again
    assert torch.equal(y2, ref)
