"""GPU parity of the producers of the quantized linear's input (RMSNorm with / without the residual add,
SwiGLU, each with the Q8_1 quantizer folded in) and of the reference-named entry points around them.

Three checkers: the reference's own golden case (tests/test_rms_norm_fused_add.py, tolerance 1e-5), the
reference's own kernels rebuilt unmodified for sm_100a (``oracle/_ref``: bit-exact, fp32 and blocks),
and the CPU oracle (which cannot restate rsqrtf / the device expf exactly: last-bit tolerance).
"""
import ctypes
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libjjj_ref.so")
GOLDEN = os.path.join(ROOT, "tests", "golden", "rms_norm_fused_add_seed24.npz")


@pytest.fixture(scope="module")
def ref(cuda_device):
    if not os.path.exists(REF_LIB):
        pytest.skip("reference kernels not built (make -C oracle ref)")
    lib = ctypes.CDLL(REF_LIB)
    vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    if not hasattr(lib, "rms_norm_fused_add_forward_device"):
        pytest.skip("reference checker library predates the producer kernels (make -C oracle ref)")
    lib.rms_norm_fused_add_forward_device.restype = ci
    lib.rms_norm_fused_add_forward_device.argtypes = [vp, vp, vp, vp, ci, ci, cf]
    lib.rms_norm_forward_device.restype = ci
    lib.rms_norm_forward_device.argtypes = [vp, vp, vp, vp, ci, ci, cf]
    lib.swiglu_silu_mul_launch_device.restype = None
    lib.swiglu_silu_mul_launch_device.argtypes = [vp, vp, vp, vp, ci]
    return lib


def _golden_inputs():
    g = np.load(GOLDEN)
    H, T = int(g["hidden"]), int(g["tokens"])
    np.random.seed(int(g["seed"]))
    x = np.asfortranarray(np.random.randn(H, T, 1, 1).astype(np.float32))
    r = np.asfortranarray(np.random.randn(H, T, 1, 1).astype(np.float32))
    w = np.random.randn(H).astype(np.float32)
    return (np.ascontiguousarray(x.reshape(H, T).T), np.ascontiguousarray(r.reshape(H, T).T), w, float(g["eps"]),
            g["normed"], g["residual"])


def test_rms_norm_fused_add_reference_golden_case(native_lib, cuda_device):
    """The reference test's own case and tolerance, through the reference-named entry point (in place)."""
    import torch

    c = native_lib
    x, r, w, eps, want_normed, want_res = _golden_inputs()
    T, H = x.shape
    dx, dr, dw = (torch.from_numpy(a).to(cuda_device) for a in (x, r, w))
    stream = torch.cuda.Stream(device=cuda_device)  # the reference refuses the null stream
    stream.wait_stream(torch.cuda.current_stream(cuda_device))
    rc = c.lib().rms_norm_fused_add_forward_device(stream.cuda_stream, dx.data_ptr(), dr.data_ptr(), dw.data_ptr(), H, T, eps)
    assert rc == 0
    stream.synchronize()
    np.testing.assert_allclose(dx.cpu().numpy(), want_normed, atol=1e-5, rtol=1e-5)
    np.testing.assert_allclose(dr.cpu().numpy(), want_res, atol=1e-5, rtol=1e-5)
    assert c.lib().rms_norm_fused_add_forward_device(None, dx.data_ptr(), dr.data_ptr(), dw.data_ptr(), H, T, eps) == -1


SHAPES_RMS = [(1, 4096), (13, 128), (5, 11008), (64, 4096), (3, 256), (2, 8192)]


@pytest.mark.parametrize("T,H", SHAPES_RMS)
@pytest.mark.parametrize("fused_add", [True, False])
def test_rms_norm_q8_1_equals_reference_kernel_then_quantizer(ref, native_lib, cuda_device, T, H, fused_add):
    import torch

    c = native_lib
    rng = np.random.default_rng(1000 + T + H)
    x = (rng.standard_normal((T, H)) * 1.7).astype(np.float32)
    r = rng.standard_normal((T, H)).astype(np.float32)
    w = (1.0 + 0.2 * rng.standard_normal(H)).astype(np.float32)
    eps = 1e-6
    st = torch.cuda.current_stream(cuda_device)
    side = torch.cuda.Stream(device=cuda_device)
    # reference kernel (in place on its copies)
    rx, rr, dw = torch.from_numpy(x).to(cuda_device), torch.from_numpy(r).to(cuda_device), torch.from_numpy(w).to(cuda_device)
    torch.cuda.synchronize()
    if fused_add:
        assert ref.rms_norm_fused_add_forward_device(side.cuda_stream, rx.data_ptr(), rr.data_ptr(), dw.data_ptr(), H, T, eps) == 0
        ref_normed = rx
    else:
        ref_normed = torch.empty_like(rx)
        assert ref.rms_norm_forward_device(side.cuda_stream, rx.data_ptr(), dw.data_ptr(), ref_normed.data_ptr(), H, T, eps) == 0
    side.synchronize()
    for order in (c.ORDER_COL_KSUPER, c.ORDER_KSUPER_COL):
        for s_mode in (c.S_SUM_X, c.S_D_SUM_Q):
            mx, mr = torch.from_numpy(x).to(cuda_device), torch.from_numpy(r).to(cuda_device)
            normed = torch.empty_like(mx)
            xq = c.rms_norm_q8_1(mx, dw, eps, residual=mr if fused_add else None, normed=normed, order=order, s_mode=s_mode)
            st.synchronize()
            assert torch.equal(normed, ref_normed), "fp32 output differs from the reference kernel"
            if fused_add:
                assert torch.equal(mr, rr), "residual differs from the reference kernel"
            assert torch.equal(mx, torch.from_numpy(x).to(cuda_device)), "input must stay untouched when it is not the output"
            want = c.quantize_q8_1(ref_normed, order, s_mode)
            assert torch.equal(xq[: want.numel()], want), "blocks differ from quantize_q8_1(reference output)"
    # Q8_1 only (no fp32 output), and in place
    mx, mr = torch.from_numpy(x).to(cuda_device), torch.from_numpy(r).to(cuda_device)
    xq = c.rms_norm_q8_1(mx, dw, eps, residual=mr if fused_add else None)
    assert torch.equal(xq[: c.q8_1_bytes(H, T)], c.quantize_q8_1(ref_normed, c.ORDER_COL_KSUPER, c.S_D_SUM_Q)[: c.q8_1_bytes(H, T)])
    mx2, mr2 = torch.from_numpy(x).to(cuda_device), torch.from_numpy(r).to(cuda_device)
    c.rms_norm_q8_1(mx2, dw, eps, residual=mr2 if fused_add else None, normed=mx2, want_q8=False)
    assert torch.equal(mx2, ref_normed)


@pytest.mark.parametrize("T,H", [(1, 4096), (13, 128), (4, 1024)])
def test_rms_norm_q8_1_against_cpu_oracle(native_lib, oracle, cuda_device, T, H):
    import torch

    c, O = native_lib, oracle
    rng = np.random.default_rng(77 + H)
    x = rng.standard_normal((T, H)).astype(np.float32)
    r = rng.standard_normal((T, H)).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    want_normed, want_res = O.rms_norm(x, w, 1e-5, r)
    dx, dr, dw = (torch.from_numpy(a).to(cuda_device) for a in (x, r, w))
    normed = torch.empty_like(dx)
    xq = c.rms_norm_q8_1(dx, dw, 1e-5, residual=dr, normed=normed, s_mode=c.S_D_SUM_Q)
    torch.cuda.synchronize()
    assert np.array_equal(dr.cpu().numpy(), want_res)  # one exact addition
    # rsqrtf on the device against 1/sqrtf on the host: a few ulp
    np.testing.assert_allclose(normed.cpu().numpy(), want_normed, rtol=1e-6, atol=1e-7)
    got_d, _, got_q = O.np_unpack_q8_1(xq.cpu().numpy()[: c.q8_1_bytes(H, T)], H, T)
    want_d, _, want_q = O.np_unpack_q8_1(O.quantize_q8_1(want_normed, O.ORDER_COL_KSUPER, O.S_D_SUM_Q), H, T)
    dq = np.abs(got_q.astype(np.int32) - want_q.astype(np.int32))
    assert dq.max() <= 1 and (dq != 0).mean() < 2e-3
    np.testing.assert_allclose(got_d, want_d, rtol=1e-3)


SHAPES_SWIGLU = [(1, 11008), (7, 256), (128, 11008), (3, 128), (2, 14336)]


@pytest.mark.parametrize("T,I", SHAPES_SWIGLU)
def test_swiglu_q8_1_equals_reference_kernel_then_quantizer(ref, native_lib, cuda_device, T, I):
    import torch

    c = native_lib
    rng = np.random.default_rng(5 + T + I)
    g = (rng.standard_normal((T, I)) * 2.5).astype(np.float32)
    u = rng.standard_normal((T, I)).astype(np.float32)
    g[0, :8] = [0.0, -0.0, 88.0, -88.0, 104.0, -104.0, 1e-30, -1e-30]  # saturating and tiny arguments of expf
    dg, du = torch.from_numpy(g).to(cuda_device), torch.from_numpy(u).to(cuda_device)
    ref_mid = torch.empty_like(dg)
    side = torch.cuda.Stream(device=cuda_device)
    torch.cuda.synchronize()
    ref.swiglu_silu_mul_launch_device(side.cuda_stream, dg.data_ptr(), du.data_ptr(), ref_mid.data_ptr(), T * I)
    side.synchronize()
    for order in (c.ORDER_COL_KSUPER, c.ORDER_KSUPER_COL):
        for s_mode in (c.S_SUM_X, c.S_D_SUM_Q):
            mid = torch.empty_like(dg)
            xq = c.swiglu_q8_1(dg, du, mid=mid, order=order, s_mode=s_mode)
            torch.cuda.synchronize()
            assert torch.equal(mid.view(torch.int32), ref_mid.view(torch.int32)), "fp32 output differs from the reference kernel"
            want = c.quantize_q8_1(ref_mid, order, s_mode)
            assert torch.equal(xq[: want.numel()], want)
    xq = c.swiglu_q8_1(dg, du)  # blocks only
    assert torch.equal(xq[: c.q8_1_bytes(I, T)], c.quantize_q8_1(ref_mid, c.ORDER_COL_KSUPER, c.S_D_SUM_Q)[: c.q8_1_bytes(I, T)])


def test_swiglu_against_cpu_oracle_and_reference_named_entry(native_lib, oracle, cuda_device):
    import torch

    c, O = native_lib, oracle
    rng = np.random.default_rng(9)
    for n in (1, 100, 4096, 11008 * 3 + 5):  # the reference takes a flat element count, any size
        g = (rng.standard_normal(n) * 3).astype(np.float32)
        u = rng.standard_normal(n).astype(np.float32)
        dg, du = torch.from_numpy(g).to(cuda_device), torch.from_numpy(u).to(cuda_device)
        mid = torch.full((n,), 7.0, dtype=torch.float32, device=cuda_device)
        c.lib().swiglu_silu_mul_launch_device(torch.cuda.current_stream().cuda_stream, dg.data_ptr(), du.data_ptr(), mid.data_ptr(), n)
        torch.cuda.synchronize()
        np.testing.assert_allclose(mid.cpu().numpy(), O.swiglu(g, u), rtol=2e-6, atol=1e-30)
    # Q8_1 output needs whole 128-value blocks
    dg = torch.zeros((2, 100), dtype=torch.float32, device=cuda_device)
    with pytest.raises(c.JqError) as e:
        c.swiglu_q8_1(dg, dg)
    assert e.value.status == c.ERR_UNSUPPORTED


def test_rms_norm_argument_errors(native_lib, cuda_device):
    import torch

    c = native_lib
    x = torch.zeros((2, 100), dtype=torch.float32, device=cuda_device)
    w = torch.ones(100, dtype=torch.float32, device=cuda_device)
    with pytest.raises(c.JqError) as e:
        c.rms_norm_q8_1(x, w, 1e-6)  # blocks need hidden % 128 == 0
    assert e.value.status == c.ERR_UNSUPPORTED
    out = torch.empty_like(x)
    x.normal_()
    c.rms_norm_q8_1(x, w, 1e-6, normed=out, want_q8=False)  # fp32 only: any hidden size
    torch.cuda.synchronize()
    want = x * torch.rsqrt((x * x).mean(dim=1, keepdim=True) + 1e-6)
    assert torch.allclose(out, want, rtol=1e-5, atol=1e-6)
    rc = c.lib().jq_rms_norm_q8_1_device(None, x.data_ptr(), None, w.data_ptr(), None, None, 100, 2, 1e-6, 0, 0)
    assert rc == c.ERR_INVALID_ARG  # nothing to write


def test_linear_q4_0_forward_device_is_the_linear_path(native_lib, oracle, cuda_device):
    """The reference-named wrapper for the layer's call sites: same result as jq_linear_q4_0_device, within
    1e-3 of dequantise-then-matmul."""
    import torch

    c, O = native_lib, oracle
    rng = np.random.default_rng(3)
    for (T, K, N) in ((1, 4096, 4096), (13, 256, 384), (40, 1024, 96)):
        w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
        x = rng.standard_normal((T, K)).astype(np.float32)
        wq = O.quantize_q4_0(w)
        dwq = torch.from_numpy(wq).to(cuda_device)
        dx = torch.from_numpy(x).to(cuda_device)
        ws = torch.empty(c.q8_1_bytes(K, T) + 16, dtype=torch.uint8, device=cuda_device)
        y = torch.empty((T, N), dtype=torch.float32, device=cuda_device)
        rc = c.lib().linear_q4_0_forward_device(torch.cuda.current_stream().cuda_stream, dx.data_ptr(), dwq.data_ptr(),
                                                ws.data_ptr(), y.data_ptr(), K, N, T)
        assert rc == 0
        want = c.linear_q4_0(dwq, dx, N, c.S_D_SUM_Q)
        torch.cuda.synchronize()
        assert torch.equal(y, want)
        xq = O.quantize_q8_1(x, O.ORDER_COL_KSUPER, O.S_D_SUM_Q)
        assert O.err_max_rel(y.cpu().numpy(), O.mul_mat_deq_f64(wq, xq, K, N, T)) <= 1e-3
    assert c.lib().linear_q4_0_forward_device(None, dx.data_ptr(), dwq.data_ptr(), ws.data_ptr(), y.data_ptr(), 100, N, T) == -1


def test_layer_dataflow_with_folded_quantizers(native_lib, oracle, cuda_device):
    """The reference layer's FFN half (transformer_runner.cpp:311-328) two ways: fp32 hand-offs with a quantize
    inside every linear, and Q8_1 hand-offs from the producers.  Same bytes, so the same outputs bit for bit."""
    import torch

    c, O = native_lib, oracle
    rng = np.random.default_rng(11)
    H, I = 1024, 2816
    for T in (1, 5, 24):
        wq = {k: torch.from_numpy(O.quantize_q4_0((rng.standard_normal(s) * 0.02).astype(np.float32))).to(cuda_device)
              for k, s in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I)))}
        h = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).to(cuda_device)
        res = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).to(cuda_device)
        wn = torch.from_numpy((1 + 0.1 * rng.standard_normal(H)).astype(np.float32)).to(cuda_device)
        # (a) fp32 hand-offs
        h_a, res_a = h.clone(), res.clone()
        c.rms_norm_q8_1(h_a, wn, 1e-6, residual=res_a, normed=h_a, want_q8=False)
        gate = c.linear_q4_0(wq["gate"], h_a, I)
        up = c.linear_q4_0(wq["up"], h_a, I)
        mid = torch.empty_like(gate)
        c.swiglu_q8_1(gate, up, mid=mid, want_q8=False)
        out_a = c.linear_q4_0(wq["down"], mid, H)
        # (b) Q8_1 hand-offs: one quantization serves gate and up, none is a launch of its own
        h_b, res_b = h.clone(), res.clone()
        hq = c.rms_norm_q8_1(h_b, wn, 1e-6, residual=res_b)
        gate_b = c.mul_mat_q4_0_q8_1(wq["gate"], hq, H, I, T, c.ORDER_COL_KSUPER)
        up_b = c.mul_mat_q4_0_q8_1(wq["up"], hq, H, I, T, c.ORDER_COL_KSUPER)
        midq = c.swiglu_q8_1(gate_b, up_b)
        out_b = c.mul_mat_q4_0_q8_1(wq["down"], midq, I, H, T, c.ORDER_COL_KSUPER)
        torch.cuda.synchronize()
        assert torch.equal(res_a, res_b)
        assert torch.equal(gate, gate_b) and torch.equal(up, up_b)
        assert torch.equal(out_a, out_b)
        assert torch.isfinite(out_b).all()


def test_lm_head_q4_0_after_final_norm(native_lib, oracle, cuda_device):
    """Final RMSNorm (no residual) -> logits over a Q4_0 table, fp32 hand-off and Q8_1 hand-off: same logits,
    within 1e-3 of dequantise-then-matmul."""
    import torch

    c, O = native_lib, oracle
    rng = np.random.default_rng(21)
    H, V = 512, 1000  # a vocabulary that is not a multiple of 32
    table = (rng.standard_normal((V, H)) * 0.05).astype(np.float32)
    tq = O.quantize_q4_0(table)
    dt = torch.from_numpy(tq).to(cuda_device)
    wn = torch.from_numpy((1 + 0.1 * rng.standard_normal(H)).astype(np.float32)).to(cuda_device)
    st = torch.cuda.current_stream().cuda_stream
    for T in (1, 3, 17):
        h = torch.from_numpy(rng.standard_normal((T, H)).astype(np.float32)).to(cuda_device)
        normed = torch.empty_like(h)
        hq = c.rms_norm_q8_1(h, wn, 1e-6, normed=normed)
        ws = torch.empty(c.q8_1_bytes(H, T) + 16, dtype=torch.uint8, device=cuda_device)
        la = torch.empty((T, V), dtype=torch.float32, device=cuda_device)
        lb = torch.empty((T, V), dtype=torch.float32, device=cuda_device)
        assert c.lib().lm_head_q4_0_forward_device(st, dt.data_ptr(), normed.data_ptr(), None, ws.data_ptr(), la.data_ptr(), H, V, T) == 0
        assert c.lib().lm_head_q4_0_forward_device(st, dt.data_ptr(), None, hq.data_ptr(), None, lb.data_ptr(), H, V, T) == 0
        torch.cuda.synchronize()
        assert torch.equal(la, lb)
        xq = O.quantize_q8_1(normed.cpu().numpy(), O.ORDER_COL_KSUPER, O.S_D_SUM_Q)
        assert np.array_equal(xq, hq.cpu().numpy()[: xq.size])
        assert O.err_max_rel(lb.cpu().numpy(), O.mul_mat_deq_f64(tq, xq, H, V, T)) <= 1e-3


def test_swiglu_in_place_on_the_gate_buffer(native_lib, oracle, cuda_device):
    """mid may be the gate buffer itself: each thread reads its values before it writes them."""
    import torch

    c = native_lib
    rng = np.random.default_rng(31)
    g = torch.from_numpy((rng.standard_normal((6, 512)) * 2).astype(np.float32)).to(cuda_device)
    u = torch.from_numpy(rng.standard_normal((6, 512)).astype(np.float32)).to(cuda_device)
    want = torch.empty_like(g)
    want_q = c.swiglu_q8_1(g, u, mid=want)
    got_q = c.swiglu_q8_1(g, u, mid=g)
    torch.cuda.synchronize()
    assert torch.equal(g, want) and torch.equal(got_q, want_q)


@pytest.mark.parametrize("M", [1, 2, 3, 8, 20])
def test_multi_linear_equals_separate_linears(native_lib, oracle, cuda_device, M):
    """q / k / v (and gate / up) in one launch over the concatenated rows: same bits as separate calls, from fp32
    input and from Q8_1 blocks; row counts that make a stage straddle two matrices."""
    import torch

    c, O = native_lib, oracle
    rng = np.random.default_rng(100 + M)
    for K, Ns in ((1024, (512, 136, 136)), (4096, (1000, 1000)), (768, (40, 7, 300, 33)), (2048, (96,))):
        wq = [torch.from_numpy(O.quantize_q4_0((rng.standard_normal((n, K)) * 0.03).astype(np.float32))).to(cuda_device) for n in Ns]
        x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(cuda_device)
        want = [c.linear_q4_0(w, x, n) for w, n in zip(wq, Ns)]
        got = c.linear_q4_0_multi(wq, Ns, x=x)
        xq = c.quantize_q8_1(x, c.ORDER_COL_KSUPER, c.S_D_SUM_Q)
        got_q = c.linear_q4_0_multi(wq, Ns, xq=xq, K=K, M=M)
        torch.cuda.synchronize()
        for a, b, d, n in zip(want, got, got_q, Ns):
            assert a.shape == (M, n)
            assert torch.equal(a, b), (K, Ns, M, "fp32 input")
            assert torch.equal(a, d), (K, Ns, M, "Q8_1 input")
    with pytest.raises(c.JqError):
        c.linear_q4_0_multi(wq, Ns, x=x, xq=xq, K=K, M=M)  # both kinds of input
    with pytest.raises(c.JqError):
        c.linear_q4_0_multi(wq * 5, list(Ns) * 5, x=x)  # more than four matrices
