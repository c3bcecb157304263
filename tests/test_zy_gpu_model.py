"""The quantized model container on the GPU: upload, then the layer's fused views through the multiply
(the host-side planning is covered by test_model_q4_0_cpu.py)."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

CONFIG = {"hidden_size": 256, "intermediate_size": 512, "num_layers": 2, "num_q_heads": 4, "num_kv_heads": 2, "head_dim": 64,
          "vocab_size": 96, "max_seq_len": 32, "freq_base": 10000.0, "rms_norm_epsilon": 1e-6, "tie_word_embeddings": 1}
H, I, Q, KV, V = 256, 512, 256, 128, 96
LINEARS = {"w_q": (Q, H), "w_k": (KV, H), "w_v": (KV, H), "w_o": (H, Q), "w_gate": (I, H), "w_up": (I, H), "w_down": (H, I)}


def test_upload_and_fused_views(native_lib, oracle, cuda_device, tmp_path):
    import torch
    from jjjetson_ops_b200 import model, weights_io as W

    c, O = native_lib, oracle
    rng = np.random.default_rng(11)
    mk = lambda *s: (rng.standard_normal(s) * 0.05).astype(np.float32)
    tensors, wq = {}, {}
    for layer in range(2):
        for name, (rows, K) in LINEARS.items():
            key = "layer%d.%s" % (layer, name)
            wq[key] = O.quantize_q4_0(mk(rows, K))
            tensors[key] = W.Tensor(W.DTYPE_Q4_0, (rows, K), wq[key])
        tensors["layer%d.w_input_layernorm" % layer] = mk(H)
        tensors["layer%d.w_post_attention_layernorm" % layer] = mk(H)
    tensors["embed"], tensors["final_norm"] = mk(V, H), mk(H)
    W.write_fixture(str(tmp_path), CONFIG, tensors)

    m = model.ModelQ4_0(str(tmp_path))
    try:
        assert m.config["num_layers"] == 2 and m.total_bytes > 0
        lib = c.lib()
        M = 3
        x = rng.standard_normal((M, H), dtype=np.float32)
        d_x = torch.from_numpy(x).to(cuda_device)
        d_ws = torch.zeros(c.q8_1_bytes(H, M), dtype=torch.uint8, device=cuda_device)
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        xq = O.quantize_q8_1(x, O.ORDER_COL_KSUPER, O.S_D_SUM_Q)
        for layer in range(2):
            lw = m.layer(layer)
            p = "layer%d." % layer
            assert lw["d_w_qkv"] == lw["d_w_q"] and lw["d_w_k"] - lw["d_w_q"] == wq[p + "w_q"].size
            assert lw["d_w_gate_up"] == lw["d_w_gate"] and lw["d_w_up"] - lw["d_w_gate"] == wq[p + "w_gate"].size
            # q | k | v as one matrix in one launch, against the oracle on the concatenated rows
            for view, names in (("d_w_qkv", ("w_q", "w_k", "w_v")), ("d_w_gate_up", ("w_gate", "w_up"))):
                cat = np.concatenate([wq[p + n].reshape(-1) for n in names])
                N = sum(LINEARS[n][0] for n in names)
                d_y = torch.zeros((M, N), dtype=torch.float32, device=cuda_device)
                c.check(lib.jq_linear_q4_0_device(stream, ctypes.c_void_p(lw[view]), ctypes.c_void_p(d_x.data_ptr()),
                                                  ctypes.c_void_p(d_ws.data_ptr()), ctypes.c_void_p(d_y.data_ptr()), H, N, M, c.S_D_SUM_Q))
                torch.cuda.synchronize()
                ref = O.mul_mat_ref(cat, xq, H, N, M)
                assert O.err_max_rel(d_y.cpu().numpy(), ref) <= 1e-5
            # and one projection on its own pointer
            d_y = torch.zeros((M, KV), dtype=torch.float32, device=cuda_device)
            c.check(lib.jq_linear_q4_0_device(stream, ctypes.c_void_p(lw["d_w_v"]), ctypes.c_void_p(d_x.data_ptr()),
                                              ctypes.c_void_p(d_ws.data_ptr()), ctypes.c_void_p(d_y.data_ptr()), H, KV, M, c.S_D_SUM_Q))
            torch.cuda.synchronize()
            assert O.err_max_rel(d_y.cpu().numpy(), O.mul_mat_ref(wq[p + "w_v"], xq, H, KV, M)) <= 1e-5
        addr, dtype = m.table("lm_head")
        assert dtype == W.DTYPE_F32 and addr == m.table("embed")[0] and m.table("final_norm")[0] != 0
    finally:
        m.close()
    assert c.device_fault(clear=True) == 0


def test_prefill_option_routes_the_automatic_choice(native_lib, oracle, cuda_device):
    """The automatic dispatch gives the fp16-operand kernel's result for a prefill batch and an exact-integer
    kernel's with JQ_OPT_PREFILL_EXACT (and for a small batch either way); the switch is put back whatever happens."""
    import torch

    c, O = native_lib, oracle
    rng = np.random.default_rng(5)
    K, N = 512, 256
    w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    wq = O.quantize_q4_0(w)
    d_w = torch.from_numpy(wq).to(cuda_device)
    for M in (128, 16):
        x = rng.standard_normal((M, K), dtype=np.float32)
        xq = O.quantize_q8_1(x, O.ORDER_COL_KSUPER, O.S_D_SUM_Q)
        d_xq = torch.from_numpy(xq).to(cuda_device)
        auto = c.mul_mat_q4_0_q8_1(d_w, d_xq, K, N, M, c.ORDER_COL_KSUPER, c.KERNEL_AUTO).cpu().numpy()
        named = c.mul_mat_q4_0_q8_1(d_w, d_xq, K, N, M, c.ORDER_COL_KSUPER, c.KERNEL_GEMM_F16).cpu().numpy()
        c.set_option(c.OPT_PREFILL_EXACT, 1)
        try:
            exact = c.mul_mat_q4_0_q8_1(d_w, d_xq, K, N, M, c.ORDER_COL_KSUPER, c.KERNEL_AUTO).cpu().numpy()
        finally:
            c.set_option(c.OPT_PREFILL_EXACT, 0)
        ref = O.mul_mat_ref(wq, xq, K, N, M)
        assert O.err_max_rel(exact, ref) <= 1e-5
        if M >= 64:
            assert np.array_equal(auto, named) and O.err_max_rel(auto, ref) <= 1e-3
        else:
            assert np.array_equal(auto, exact)
    assert c.get_option(c.OPT_PREFILL_EXACT) == 0 and c.device_fault(clear=True) == 0
