"""The quantized model container (include/jq_model.h): config parsing and the device layout, both host-only."""
import numpy as np
import pytest

CONFIG = {"hidden_size": 128, "intermediate_size": 256, "num_layers": 2, "num_q_heads": 4, "num_kv_heads": 2, "head_dim": 32,
          "vocab_size": 64, "max_seq_len": 32, "freq_base": 10000.0, "rms_norm_epsilon": 1e-6, "tie_word_embeddings": 1}
H, I, Q, KV, V = 128, 256, 128, 64, 64
LINEARS = {"w_q": (Q, H), "w_k": (KV, H), "w_v": (KV, H), "w_o": (H, Q), "w_gate": (I, H), "w_up": (I, H), "w_down": (H, I)}


def _quantized_tensors(oracle, W, config, quantize=True, tied_embed_q4=False):
    """A model's tensors as the offline quantizer leaves them: linears Q4_0 [out, in], the rest fp32."""
    rng = np.random.default_rng(7)
    mk = lambda *s: (rng.standard_normal(s) * 0.05).astype(np.float32)
    t = {}
    for layer in range(config["num_layers"]):
        for name, (rows, K) in LINEARS.items():
            w = mk(rows, K)
            t["layer%d.%s" % (layer, name)] = W.Tensor(W.DTYPE_Q4_0, (rows, K), oracle.quantize_q4_0(w)) if quantize else w
        t["layer%d.w_input_layernorm" % layer] = mk(H)
        t["layer%d.w_post_attention_layernorm" % layer] = mk(H)
    e = mk(V, H)
    t["embed"] = W.Tensor(W.DTYPE_Q4_0, (V, H), oracle.quantize_q4_0(e)) if tied_embed_q4 else e
    t["final_norm"] = mk(H)
    if not config["tie_word_embeddings"]:
        t["lm_head"] = mk(H, V)
    return t


def test_config_parse_and_validation(native_lib):
    from jjjetson_ops_b200 import model

    c = native_lib
    text = "".join("%s=%s\n" % kv for kv in CONFIG.items())
    cfg = model.parse_config(text)
    assert cfg["hidden_size"] == 128 and cfg["num_layers"] == 2 and cfg["tie_word_embeddings"] == 1
    assert cfg["freq_base"] == 10000.0 and abs(cfg["rms_norm_epsilon"] - 1e-6) < 1e-12
    for key in CONFIG:  # every key is required, as in the reference's loader
        with pytest.raises(c.JqError) as e:
            model.parse_config("".join("%s=%s\n" % kv for kv in CONFIG.items() if kv[0] != key))
        assert key in str(e.value)
    for bad in ({"num_kv_heads": 8}, {"head_dim": 31}, {"hidden_size": 0}, {"rms_norm_epsilon": 0.0}, {"tie_word_embeddings": 2},
                {"num_layers": 1.5}):
        with pytest.raises(c.JqError):
            model.parse_config("".join("%s=%s\n" % kv for kv in dict(CONFIG, **bad).items()))


@pytest.mark.parametrize("container", ["fixture", "safetensors"])
def test_layout_of_a_quantized_model(native_lib, oracle, tmp_path, container):
    from jjjetson_ops_b200 import model, weights_io as W

    tensors = _quantized_tensors(oracle, W, CONFIG, tied_embed_q4=True)
    W.write_fixture(str(tmp_path), CONFIG, tensors)
    path = str(tmp_path)
    if container == "safetensors":
        path = str(tmp_path / "model.safetensors")
        W.write_safetensors(path, tensors)
    cfg, slots, total = model.plan(path)
    assert cfg["num_layers"] == 2 and len(slots) == 2 * 9 + 2
    assert [s.name for s in slots[:9]] == model.layer_names(0) and [s.name for s in slots[9:18]] == model.layer_names(1)
    assert [s.name for s in slots[18:]] == ["embed", "final_norm"]
    by = {s.name: s for s in slots}
    for layer in range(2):
        p = "layer%d." % layer
        for name, (rows, K) in LINEARS.items():
            s = by[p + name]
            assert (s.dtype, s.rows, s.K, s.nbytes) == (W.DTYPE_Q4_0, rows, K, rows * K // 32 * 18)
        # q | k | v and gate | up are single matrices: each follows its predecessor directly
        assert by[p + "w_k"].offset == by[p + "w_q"].offset + by[p + "w_q"].nbytes
        assert by[p + "w_v"].offset == by[p + "w_k"].offset + by[p + "w_k"].nbytes
        assert by[p + "w_up"].offset == by[p + "w_gate"].offset + by[p + "w_gate"].nbytes
        for name in ("w_q", "w_o", "w_gate", "w_down", "w_input_layernorm"):
            assert by[p + name].offset % 256 == 0
        for name in ("w_k", "w_v", "w_up"):  # still 16-byte aligned for use on their own (hidden % 256 == 0 would give it for any size)
            assert by[p + name].offset % 16 == 0
        assert by[p + "w_input_layernorm"].dtype == W.DTYPE_F32 and by[p + "w_input_layernorm"].nbytes == H * 4
    assert by["embed"].dtype == W.DTYPE_Q4_0 and (by["embed"].rows, by["embed"].K) == (V, H)
    # slots do not overlap, are in address order and fit the allocation
    ends = 0
    for s in slots:
        assert s.offset >= ends
        ends = s.offset + s.nbytes
    assert ends <= total and total % 256 == 0


def test_untied_model_keeps_an_fp32_lm_head(native_lib, oracle, tmp_path):
    from jjjetson_ops_b200 import model, weights_io as W

    cfg = dict(CONFIG, tie_word_embeddings=0, num_layers=1)
    W.write_fixture(str(tmp_path), cfg, _quantized_tensors(oracle, W, cfg))
    _, slots, _ = model.plan(str(tmp_path))
    assert [s.name for s in slots[-3:]] == ["embed", "final_norm", "lm_head"]
    assert slots[-1].dtype == W.DTYPE_F32 and slots[-1].nbytes == V * H * 4 and slots[-3].dtype == W.DTYPE_F32


def test_layout_errors(native_lib, oracle, tmp_path):
    from jjjetson_ops_b200 import model, weights_io as W

    c = native_lib
    cfg = dict(CONFIG, num_layers=1)
    good = _quantized_tensors(oracle, W, cfg)

    def plan_of(tensors, config=cfg, sub="x"):
        d = tmp_path / sub
        W.write_fixture(str(d), config, tensors)
        return model.plan(str(d))

    plan_of(good, sub="ok")
    with pytest.raises(c.JqError) as e:  # a linear that was never quantized
        plan_of(dict(good, **{"layer0.w_o": np.zeros((H, Q), np.float32)}), sub="a")
    assert e.value.status == c.ERR_UNSUPPORTED and "layer0.w_o" in str(e.value) and "quantize" in str(e.value)
    with pytest.raises(c.JqError) as e:  # stored [in, out] instead of [out, in]
        plan_of(dict(good, **{"layer0.w_down": W.Tensor(W.DTYPE_Q4_0, (I, H), oracle.quantize_q4_0(np.zeros((I, H), np.float32)))}), sub="b")
    assert e.value.status == c.ERR_SHAPE and "layer0.w_down" in str(e.value)
    with pytest.raises(c.JqError) as e:
        plan_of({k: v for k, v in good.items() if k != "layer0.w_up"}, sub="c")
    assert "missing tensor layer0.w_up" in str(e.value)
    with pytest.raises(c.JqError):  # a norm of the wrong length
        plan_of(dict(good, **{"final_norm": np.zeros(H + 1, np.float32)}), sub="d")
    with pytest.raises(c.JqError):  # a quantized norm
        plan_of(dict(good, **{"layer0.w_input_layernorm": W.Tensor(W.DTYPE_Q4_0, (1, H), oracle.quantize_q4_0(np.zeros((1, H), np.float32)))}), sub="e")
    with pytest.raises(c.JqError):  # a quantized embed in an untied model
        untied = dict(cfg, tie_word_embeddings=0)
        t = _quantized_tensors(oracle, W, untied, tied_embed_q4=True)
        plan_of(t, config=untied, sub="f")
    with pytest.raises(c.JqError):  # two layers promised, one present
        plan_of(good, config=dict(cfg, num_layers=2), sub="g")
    with pytest.raises(c.JqError):  # no config.txt values at all
        plan_of(good, config={}, sub="h")


def test_create_fails_loudly_without_a_device(native_lib, oracle, tmp_path):
    """The upload is the CUDA path or nothing: on a machine without a GPU it reports the CUDA error."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from jjjetson_ops_b200 import model, weights_io as W

    cfg = dict(CONFIG, num_layers=1)
    W.write_fixture(str(tmp_path), cfg, _quantized_tensors(oracle, W, cfg))
    with pytest.raises(native_lib.JqError) as e:
        model.ModelQ4_0(str(tmp_path))
    assert e.value.status == native_lib.ERR_CUDA


def test_command_line_prints_the_layout(native_lib, oracle, tmp_path, capsys):
    from jjjetson_ops_b200 import model, weights_io as W

    cfg = dict(CONFIG, num_layers=1)
    W.write_fixture(str(tmp_path / "ok"), cfg, _quantized_tensors(oracle, W, cfg))
    assert model.main([str(tmp_path / "ok")]) == 0
    out = capsys.readouterr().out
    assert "layer0.w_down" in out and "Q4_0" in out and "total" in out
    W.write_fixture(str(tmp_path / "fp32"), cfg, _quantized_tensors(oracle, W, cfg, quantize=False))
    assert model.main([str(tmp_path / "fp32")]) == 1
    assert "quantize" in capsys.readouterr().err
    assert model.main([]) == 2
