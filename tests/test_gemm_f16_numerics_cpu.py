"""The precision claim of the fp16-operand GEMM (JQ_KERNEL_GEMM_F16), checked on the CPU.

A NumPy model of the kernel's arithmetic: both scaled operands, (q4 - 8) * d4 and q8 * d8, are
rounded once to fp16, the rank-one term uses fp16(s8 - d8 * sum(q8)) and the exact -8 * d4, and
everything is accumulated in fp32 (the tensor core's summation order differs, which moves the
result by fp32 rounding only).  On the value distributions of the five benchmark configurations
the model must stay within 1e-3 of the largest output, both against the reference formula on the
same quantized inputs and, with s = d * sum(q), against dequantise-then-matmul in float64.
"""
import numpy as np
import pytest

from jjjetson_ops_b200 import synth

TOL = 1e-3


def fp16_operand_model(O, wq, xq, K, N, M):
    d4, q4 = O.np_unpack_q4_0(wq, K)
    d8, s8, q8 = O.np_unpack_q8_1(xq, K, M)
    nb = K // 32
    d4 = np.asarray(d4, np.float32).reshape(N, nb)
    q4 = np.asarray(q4, np.float32).reshape(N, nb, 32)
    d8 = np.asarray(d8, np.float32).reshape(M, nb)
    s8 = np.asarray(s8, np.float32).reshape(M, nb)
    q8 = np.asarray(q8, np.float32).reshape(M, nb, 32)
    b = ((q4 - 8.0) * d4[:, :, None]).astype(np.float16).astype(np.float32).reshape(N, K)
    a = (q8 * d8[:, :, None]).astype(np.float16).astype(np.float32).reshape(M, K)
    za = (s8 - d8 * q8.sum(-1)).astype(np.float16).astype(np.float32)
    zb = (-8.0 * d4).astype(np.float16).astype(np.float32)
    assert np.array_equal(zb, -8.0 * d4)  # a power-of-two multiple of an fp16 value
    return a @ b.T + za @ zb.T


CASES = [  # (configuration, linear, M)
    (1, 0, 1), (2, 0, 8), (3, 0, 64), (4, 0, 16), (5, 0, 16), (5, 4, 16),
]


def _case(cfg, linear, M, rows=192):
    if cfg == 4:  # 28672 x 8192 weights would be drawn in full: same K, sigma and seed, only `rows` rows
        spec = synth.CONFIGS[4].linears[0]
        rng = np.random.default_rng(np.random.PCG64(synth.CONFIGS[4].seed))
        w = rng.standard_normal((rows, spec.K), dtype=np.float32) * np.float32(spec.sigma_w)
        return w, rng.standard_normal((M, spec.K), dtype=np.float32), spec
    return synth.make_linear_case(cfg, linear, M, rows=rows)


@pytest.mark.parametrize("cfg,linear,M", CASES)
@pytest.mark.parametrize("s_mode", [0, 1])
def test_fp16_operand_arithmetic_meets_the_tolerance(oracle, cfg, linear, M, s_mode):
    O = oracle
    w, x, lin = _case(cfg, linear, M)
    K, N = lin.K, w.shape[0]
    wq = O.quantize_q4_0(w)
    xq = O.quantize_q8_1(x, O.ORDER_COL_KSUPER, s_mode)
    y = fp16_operand_model(O, wq, xq, K, N, M)
    e_formula = O.err_max_rel(y, O.mul_mat_ref(wq, xq, K, N, M))
    assert e_formula <= TOL, e_formula
    if s_mode == O.S_D_SUM_Q:
        e_deq = O.err_max_rel(y, O.mul_mat_deq_f64(wq, xq, K, N, M))
        assert e_deq <= TOL, e_deq


def test_fp16_operand_arithmetic_needs_the_rank_one_term(oracle):
    """With the reference's s = sum(x), leaving the rank-one term out would miss the formula by
    about 1e-2: the term is what keeps the kernel on the reference's arithmetic in that mode."""
    O = oracle
    w, x, lin = synth.make_linear_case(3, 0, 32, rows=128)
    K, N, M = lin.K, w.shape[0], 32
    wq = O.quantize_q4_0(w)
    xq = O.quantize_q8_1(x, O.ORDER_COL_KSUPER, O.S_SUM_X)
    ref = O.mul_mat_ref(wq, xq, K, N, M)
    full = fp16_operand_model(O, wq, xq, K, N, M)
    without = O.mul_mat_deq_f64(wq, xq, K, N, M)  # sum((q4 - 8) d4 q8 d8), no correction
    assert O.err_max_rel(full, ref) <= TOL
    assert O.err_max_rel(without, ref) > 3e-3
