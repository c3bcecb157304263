"""GPU parity of the fp16-operand tcgen05 GEMM (JQ_KERNEL_GEMM_F16), called through the C ABI.

This kernel rounds every scaled operand ((q4 - 8) * d4 and q8 * d8) to fp16 before the tensor core
multiplies them with fp32 accumulation, so its bar is not the integer kernels' 1e-5: it is
max|y - ref| / max|ref| <= 1e-3 against the oracle's reference-formula multiply on the same
quantized inputs (about 3e-4 is expected) and <= 1e-3 against dequantise-then-matmul in float64
when the quantizer stored s = d * sum(q).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL_F16_FORMULA = 1e-3  # operands rounded to fp16 (2^-11 relative each), fp32 accumulation
TOL_DEQUANT = 1e-3      # the accuracy target against dequantise-then-matmul


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


def _check(env, wq, x, K, N, M, order, s_mode, rows=None):
    c = env.c
    xq = env.O.quantize_q8_1(x, order, s_mode)
    y = c.mul_mat_q4_0_q8_1(env.up(wq), env.up(xq), K, N, M, order, c.KERNEL_GEMM_F16).cpu().numpy()
    assert y.shape == (M, N) and np.isfinite(y).all()
    if rows is not None:
        wq = np.ascontiguousarray(wq.reshape(N, -1)[rows])
        y = y[:, rows]
        N = len(rows)
    e_ref = env.O.err_max_rel(y, env.O.mul_mat_ref(wq, xq, K, N, M, order))
    assert e_ref <= TOL_F16_FORMULA, e_ref
    if s_mode == c.S_D_SUM_Q:
        e_deq = env.O.err_max_rel(y, env.O.mul_mat_deq_f64(wq, xq, K, N, M, order))
        assert e_deq <= TOL_DEQUANT, e_deq
    return e_ref


@pytest.mark.parametrize("K,N,M", [(2560, 40, 20), (256, 64, 9), (512, 200, 33), (1024, 129, 130), (768, 256, 128),
                                   (4096, 384, 17), (1280, 1, 1), (11008, 50, 40), (1792, 300, 257)])
@pytest.mark.parametrize("order", [0, 1])
@pytest.mark.parametrize("s_mode", [0, 1])
def test_gemm_f16_small_and_ragged_shapes(env, K, N, M, order, s_mode):
    rng = np.random.default_rng(K + 3 * N + 7 * M)
    w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    x = rng.standard_normal((M, K), dtype=np.float32)
    if K >= 256:
        x[:, 5] *= 20.0          # an outlier channel
        x[M // 2, 128:160] = 0.0  # an all-zero group: d = 0
    _check(env, env.O.quantize_q4_0(w), x, K, N, M, order, s_mode)


def test_gemm_f16_refuses_odd_super_block_counts(env):
    """The tensor copies need a weight-row pitch that is a multiple of 16 bytes: K % 256 == 0."""
    c = env.c
    w = env.t.zeros(c.q4_0_bytes(8, 384), dtype=env.t.uint8, device=env.dev)
    xq = env.t.zeros(c.q8_1_bytes(384, 16), dtype=env.t.uint8, device=env.dev)
    with pytest.raises(c.JqError) as ei:
        c.mul_mat_q4_0_q8_1(w, xq, 384, 8, 16, c.ORDER_COL_KSUPER, c.KERNEL_GEMM_F16)
    assert ei.value.status == c.ERR_UNSUPPORTED


def test_gemm_f16_prefill_config(env):
    """K = N = 4096, M = 512: the prefill configuration, oracle on a sample of the weight rows."""
    from jjjetson_ops_b200 import synth

    c = env.c
    w, x, lin = synth.make_linear_case(3, 0, 512)
    wq = c.quantize_q4_0(env.up(w)).cpu().numpy()
    rows = np.sort(np.random.default_rng(33).choice(lin.N, size=256, replace=False))
    for order in (c.ORDER_COL_KSUPER, c.ORDER_KSUPER_COL):
        _check(env, wq, x, lin.K, lin.N, 512, order, c.S_D_SUM_Q, rows=rows)


def test_gemm_f16_matches_integer_kernel_closely(env):
    """Same inputs through the integer GEMM and the fp16-operand GEMM: they differ only by the
    operand rounding."""
    c = env.c
    rng = np.random.default_rng(91)
    K, N, M = 2048, 512, 256
    w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    x = rng.standard_normal((M, K), dtype=np.float32)
    d_w = env.up(env.O.quantize_q4_0(w))
    d_xq = env.up(env.O.quantize_q8_1(x, c.ORDER_COL_KSUPER, c.S_D_SUM_Q))
    y_int = c.mul_mat_q4_0_q8_1(d_w, d_xq, K, N, M, c.ORDER_COL_KSUPER, c.KERNEL_GEMM_MMA).cpu().numpy()
    y_f16 = c.mul_mat_q4_0_q8_1(d_w, d_xq, K, N, M, c.ORDER_COL_KSUPER, c.KERNEL_GEMM_F16).cpu().numpy()
    assert env.O.err_max_rel(y_f16, y_int) <= TOL_F16_FORMULA


@pytest.mark.parametrize("K,N,M", [(4096, 4096, 128), (11008, 4096, 128), (8192, 300, 70), (2048, 1000, 64)])
def test_gemm_f16_split_k_is_ordered(env, K, N, M):
    """Few output tiles and a long K: the kernel splits K over several CTAs per tile, which add their parts to y in a
    fixed order.  Right against the oracle (a sample of rows at the large sizes), and bit-equal from run to run."""
    c = env.c
    rng = np.random.default_rng(K + N + M)
    w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    x = rng.standard_normal((M, K), dtype=np.float32)
    wq = env.O.quantize_q4_0(w)
    rows = None if N <= 1000 else np.sort(rng.choice(N, size=96, replace=False))
    _check(env, wq, x, K, N, M, c.ORDER_COL_KSUPER, c.S_D_SUM_Q, rows)
    xq = env.up(env.O.quantize_q8_1(x, c.ORDER_COL_KSUPER, c.S_D_SUM_Q))
    d_w = env.up(wq)
    runs = [c.mul_mat_q4_0_q8_1(d_w, xq, K, N, M, c.ORDER_COL_KSUPER, c.KERNEL_GEMM_F16).cpu().numpy() for _ in range(4)]
    for y in runs[1:]:
        assert np.array_equal(y, runs[0])
    exact = c.mul_mat_q4_0_q8_1(d_w, xq, K, N, M, c.ORDER_COL_KSUPER, c.KERNEL_GEMM_MMA).cpu().numpy()
    assert env.O.err_max_rel(runs[0], exact) <= TOL_F16_FORMULA
