"""The Q4_0 extension of the reference's weight-fixture format: reader (CPU) and offline quantizer (GPU)."""
import os

import numpy as np
import pytest

CONFIG = {"hidden_size": 128, "intermediate_size": 256, "num_layers": 1, "num_q_heads": 4, "num_kv_heads": 2, "head_dim": 32,
          "vocab_size": 64, "max_seq_len": 32, "freq_base": 10000.0, "rms_norm_epsilon": 1e-6, "tie_word_embeddings": 1}


def _tensors(rng):
    """Shapes as the reference's tests write them (tests/test_transformer_model_load_weights.py:41-52)."""
    H, I, Q, KV, V = 128, 256, 128, 64, 64
    mk = lambda *s: (rng.standard_normal(s) * 0.05).astype(np.float32)
    return {"embed": mk(V, H), "layer0.w_q": mk(H, Q), "layer0.w_k": mk(H, KV), "layer0.w_v": mk(H, KV), "layer0.w_o": mk(Q, H),
            "layer0.w_gate": mk(H, I), "layer0.w_up": mk(H, I), "layer0.w_down": mk(I, H),
            "layer0.w_input_layernorm": mk(H), "layer0.w_post_attention_layernorm": mk(H), "final_norm": mk(H)}


def test_fixture_roundtrip_f32_and_q4_0(native_lib, oracle, tmp_path):
    from jjjetson_ops_b200 import weights_io as W

    rng = np.random.default_rng(0)
    tensors = dict(_tensors(rng))
    wq = oracle.quantize_q4_0(tensors["layer0.w_down"].reshape(128, 256))  # the engine's view: [out=128][in=256]
    tensors["layer0.w_down"] = W.Tensor(W.DTYPE_Q4_0, (128, 256), wq)
    W.write_fixture(str(tmp_path / "fx"), CONFIG, tensors)
    config, got = W.load_fixture(str(tmp_path / "fx"))
    assert config["hidden_size"] == 128 and config["rms_norm_epsilon"] == 1e-6 and config["tie_word_embeddings"] == 1
    assert set(got) == set(tensors)
    for name, t in got.items():
        if name == "layer0.w_down":
            assert t.dtype == W.DTYPE_Q4_0 and t.dims == (128, 256)
            assert np.array_equal(t.data.reshape(-1), wq.reshape(-1))
        else:
            assert t.dtype == W.DTYPE_F32 and t.dims == tensors[name].shape
            assert np.array_equal(t.data, tensors[name])


def test_fixture_errors_are_reported(native_lib, tmp_path):
    from jjjetson_ops_b200 import weights_io as W

    c = native_lib
    with pytest.raises(c.JqError):
        W.load_fixture(str(tmp_path / "missing"))
    d = tmp_path / "bad"
    W.write_fixture(str(d), CONFIG, {"a": np.zeros((4, 8), np.float32)})
    with open(d / "a.f32", "ab") as f:
        f.write(b"\0\0\0\0")  # one float too many
    with pytest.raises(c.JqError) as e:
        W.load_fixture(str(d))
    assert e.value.status == c.ERR_SHAPE and "expected" in str(e.value)
    (d / "manifest.txt").write_text("w 2 4 48 w.q4_0\n")  # K not a multiple of 32
    (d / "w.q4_0").write_bytes(b"\0" * 18)
    with pytest.raises(c.JqError):
        W.load_fixture(str(d))
    (d / "sub").mkdir()
    (d / "manifest.txt").write_text("w 2 4 8 sub\n")  # a directory where a tensor file should be
    with pytest.raises(c.JqError):
        W.load_fixture(str(d))
    (d / "manifest.txt").write_text("w 3 3037000500 3037000500 3037000500 a.f32\n")  # dims whose product overflows
    with pytest.raises(c.JqError):
        W.load_fixture(str(d))
    (d / "manifest.txt").write_text("w 2 4 8 ../escape.f32\n")
    with pytest.raises(c.JqError):
        W.load_fixture(str(d))
    (d / "manifest.txt").write_text("# comment\n\nw 1 0 w.f32\n")  # zero dimension, as the reference refuses
    with pytest.raises(c.JqError):
        W.load_fixture(str(d))


@pytest.mark.gpu
def test_offline_quantizer_and_linear_on_loaded_weights(native_lib, oracle, cuda_device, tmp_path):
    import torch

    from jjjetson_ops_b200 import weights_io as W

    c, O = native_lib, oracle
    rng = np.random.default_rng(1)
    tensors = _tensors(rng)
    W.write_fixture(str(tmp_path / "src"), CONFIG, tensors)
    n = W.quantize_fixture(str(tmp_path / "src"), str(tmp_path / "dst"))
    assert n == 8  # seven linears + the tied embedding table
    config, got = W.load_fixture(str(tmp_path / "dst"))
    assert config == {k: float(v) for k, v in CONFIG.items()}
    in_features = {"w_q": 128, "w_k": 128, "w_v": 128, "w_o": 128, "w_gate": 128, "w_up": 128, "w_down": 256}
    for name, t in got.items():
        suffix = name.split(".")[-1]
        if suffix in in_features or name == "embed":
            K = in_features.get(suffix, 128)
            want = O.quantize_q4_0(tensors[name].reshape(-1, K))
            assert t.dtype == W.DTYPE_Q4_0 and t.dims == (tensors[name].size // K, K)
            assert np.array_equal(t.data.reshape(-1), want.reshape(-1)), name
        else:
            assert t.dtype == W.DTYPE_F32 and np.array_equal(t.data, tensors[name])
    # the loaded blocks drive the linear as they are
    t = got["layer0.w_down"]
    x = rng.standard_normal((3, 256)).astype(np.float32)
    y = c.linear_q4_0(torch.from_numpy(t.data).to(cuda_device), torch.from_numpy(x).to(cuda_device), t.dims[0])
    xq = O.quantize_q8_1(x, O.ORDER_COL_KSUPER, O.S_D_SUM_Q)
    assert O.err_max_rel(y.cpu().numpy(), O.mul_mat_deq_f64(t.data, xq, 256, 128, 3)) <= 1e-3
    # quantizing an already quantized fixture converts nothing and keeps the bytes
    assert W.quantize_fixture(str(tmp_path / "dst"), str(tmp_path / "dst2")) == 0
    _, again = W.load_fixture(str(tmp_path / "dst2"))
    assert all(np.array_equal(again[k].data, got[k].data) for k in got)
