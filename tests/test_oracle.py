"""CPU tests of the oracle itself: golden vectors first, then C against the NumPy mirror."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _ref_test_input(seed: int, ne1: int) -> np.ndarray:
    """Input of the reference's tests/test_q8_1.py:71-73 as [M][K] rows."""
    np.random.seed(seed)
    x = np.random.randn(2048, ne1, 1, 1).astype(np.float32)
    return np.ascontiguousarray(x[:, :, 0, 0].T)


@pytest.mark.parametrize("tag", ["a", "b"])
def test_q8_1_matches_reference_numpy_golden(oracle, tag):
    """The reference's own q8_1_ref outputs (tests/test_q8_1.py:5-62) with its tolerances (:119-121)."""
    g = np.load(os.path.join(GOLDEN, "q8_1_ref_seed24.npz"))
    seed, ne1 = int(g[f"{tag}_seed"]), int(g[f"{tag}_ne1"])
    x = _ref_test_input(seed, ne1)
    for impl in (oracle.quantize_q8_1, oracle.np_quantize_q8_1):
        raw = impl(x, oracle.ORDER_KSUPER_COL, oracle.S_SUM_X)
        qs, d, s = oracle.parse_q8_1(raw, ne1 * 16)
        assert np.array_equal(qs, g[f"{tag}_qs"])  # exact, block order group*ne1 + j (:33)
        assert np.allclose(d, g[f"{tag}_scale"], atol=1e-5)
        assert np.allclose(s, g[f"{tag}_sum"], atol=1e-2)


@pytest.mark.parametrize("tag", ["a", "b", "c", "d"])
def test_oracle_matches_reference_kernels_run_on_b200(oracle, tag):
    """Outputs of the reference's own CUDA operators, rebuilt unmodified for sm_100a and run on a
    B200 (tests/golden/make_ref_gpu_golden.py): the quantized blocks and the fp32 products of
    mat_mul_q4_0_q8_1_device must come out of the oracle bit for bit."""
    from tests.golden.make_ref_gpu_golden import case_inputs, reorder_ksuper_col_to_col_ksuper

    g = np.load(os.path.join(GOLDEN, "ref_gpu_sm100.npz"))
    K, N, M, w, x = case_inputs(tag)
    xq = oracle.quantize_q8_1(x, oracle.ORDER_KSUPER_COL, oracle.S_SUM_X)
    assert np.array_equal(xq, g[tag + "_xq"])
    assert np.array_equal(oracle.np_quantize_q8_1(x, oracle.ORDER_KSUPER_COL, oracle.S_SUM_X), g[tag + "_xq"])
    wq = oracle.quantize_q4_0(w)
    xq_mm = reorder_ksuper_col_to_col_ksuper(xq, K, M)
    assert np.array_equal(xq_mm, oracle.quantize_q8_1(x, oracle.ORDER_COL_KSUPER, oracle.S_SUM_X))
    y = oracle.mul_mat_ref(wq, xq_mm, K, N, M, oracle.ORDER_COL_KSUPER)
    assert np.array_equal(y, g[tag + "_y"])


def test_q4_0_matches_gguf_golden(oracle):
    from tests.golden.make_q4_0_gguf_golden import make_input

    g = np.load(os.path.join(GOLDEN, "q4_0_gguf_seed5.npz"))["q4_0"]
    w = make_input()
    assert np.array_equal(oracle.quantize_q4_0(w), g)
    assert np.array_equal(oracle.np_quantize_q4_0(w), g)


def test_fp16_conversions_match_numpy(oracle):
    L = oracle.lib()
    rng = np.random.default_rng(11)
    xs = np.concatenate(
        [rng.standard_normal(3000).astype(np.float32) * np.float32(s) for s in (1e-8, 1e-5, 1e-3, 1.0, 300.0, 7e4)]
        + [np.array([0, -0.0, 65504, 65519.99, 65520, 2.0**-25, 2.0**-24, 2.0**-14, 6.1e-5, 1e9], dtype=np.float32)]
    )
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    got = np.array([L.jqo_f32_to_f16(float(v)) for v in xs], dtype=np.uint16)
    assert np.array_equal(got, want)
    hs = np.arange(0, 65536, dtype=np.uint16)
    hs = hs[~np.isnan(hs.view(np.float16))]
    back = np.array([L.jqo_f16_to_f32(int(h)) for h in hs], dtype=np.float32)
    assert np.array_equal(back.view(np.uint32), hs.view(np.float16).astype(np.float32).view(np.uint32))


@pytest.mark.parametrize("order", [0, 1])
@pytest.mark.parametrize("s_mode", [0, 1])
def test_c_and_numpy_quantizers_agree(oracle, order, s_mode):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 640), dtype=np.float32)
    x[2, 64:96] = 0.0  # all-zero group -> d = 0, s = 0, qs = 0
    x[0, 5] = 1000.0
    a = oracle.quantize_q8_1(x, order, s_mode)
    b = oracle.np_quantize_q8_1(x, order, s_mode)
    assert np.array_equal(a, b)
    d, s, q = oracle.np_unpack_q8_1(a, 640, 5, order)
    assert d[2, 2] == 0 and s[2, 2] == 0 and not q[2, 2].any()
    assert np.abs(q).max() == 127


def test_q8_1_orders_are_permutations(oracle):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((3, 256), dtype=np.float32)
    a = oracle.quantize_q8_1(x, oracle.ORDER_KSUPER_COL).reshape(2, 3, 144)
    b = oracle.quantize_q8_1(x, oracle.ORDER_COL_KSUPER).reshape(3, 2, 144)
    assert np.array_equal(a.transpose(1, 0, 2), b)
    one = rng.standard_normal((1, 512), dtype=np.float32)
    assert np.array_equal(oracle.quantize_q8_1(one, 0), oracle.quantize_q8_1(one, 1))  # M = 1: same


def test_q8_1_partial_superblock_is_zero_filled(oracle):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((2, 160), dtype=np.float32)  # 128 + 32
    raw = oracle.quantize_q8_1(x, oracle.ORDER_COL_KSUPER).reshape(2, 2, 144)
    full = oracle.quantize_q8_1(np.ascontiguousarray(x[:, :128]), oracle.ORDER_COL_KSUPER).reshape(2, 1, 144)
    assert np.array_equal(raw[:, 0], full[:, 0])
    assert not raw[:, 1, 4:16].any() and not raw[:, 1, 16 + 32:].any()


def test_block_sums_and_formulas(oracle):
    rng = np.random.default_rng(6)
    K, N, M = 512, 96, 5
    w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    x = rng.standard_normal((M, K), dtype=np.float32)
    wq = oracle.quantize_q4_0(w)
    for order in (0, 1):
        xq = oracle.quantize_q8_1(x, order, oracle.S_D_SUM_Q)
        s_c = oracle.block_sums(wq, xq, K, N, M, order)
        assert np.array_equal(s_c, oracle.np_block_sums(wq, xq, K, N, M, order))
        deq = oracle.mul_mat_deq_f64(wq, xq, K, N, M, order)
        assert oracle.err_max_rel(deq, oracle.np_mul_mat_deq(wq, xq, K, N, M, order)) < 1e-6
        # reference formula with s = d * sum(q): within 1e-3 of dequantise-then-matmul
        assert oracle.err_max_rel(oracle.mul_mat_ref(wq, xq, K, N, M, order), deq) < 1e-3
    # with the reference's s = sum(x) the formula is an order of magnitude further away
    xq0 = oracle.quantize_q8_1(x, 1, oracle.S_SUM_X)
    e0 = oracle.err_max_rel(oracle.mul_mat_ref(wq, xq0, K, N, M, 1), oracle.mul_mat_deq_f64(wq, xq0, K, N, M, 1))
    assert 1e-3 < e0 < 5e-2
    # dequantised weights are close to the originals (half a step, a full step where +max clamps to q = 15)
    assert np.abs(oracle.dequantize_q4_0(wq, K) - w).max() <= np.abs(w).max() / 8 * 1.01 + 1e-6


def test_cpu_baseline_path_matches_yardstick(oracle):
    rng = np.random.default_rng(7)
    K, N, M = 1024, 64, 3
    w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    x = rng.standard_normal((M, K), dtype=np.float32)
    wq = oracle.quantize_q4_0(w)
    xq = oracle.quantize_q8_1(x, oracle.ORDER_COL_KSUPER, oracle.S_D_SUM_Q)
    y = oracle.linear_cpu_baseline(wq, x, K, N, M)
    assert oracle.err_max_rel(y, oracle.mul_mat_deq_f64(wq, xq, K, N, M)) < 1e-5
    assert oracle.num_threads() >= 1


def test_linearity_of_block_sums(oracle):
    """sumi(w, x1) + sumi(w, x2) = sumi(w, x1 + x2) on the integer level (size-independent property)."""
    rng = np.random.default_rng(8)
    K, N = 256, 16
    wq = oracle.quantize_q4_0((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    q1 = rng.integers(-60, 60, size=(1, K), dtype=np.int8)
    q2 = rng.integers(-60, 60, size=(1, K), dtype=np.int8)

    def blocks(q):
        b = np.zeros((1, K // 128, 144), dtype=np.uint8)
        b[..., 16:] = q.reshape(1, K // 128, 128).view(np.uint8)
        return b.reshape(-1)

    s1 = oracle.block_sums(wq, blocks(q1), K, N, 1)
    s2 = oracle.block_sums(wq, blocks(q2), K, N, 1)
    s12 = oracle.block_sums(wq, blocks((q1 + q2).astype(np.int8)), K, N, 1)
    assert np.array_equal(s1 + s2, s12)
