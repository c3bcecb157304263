"""The reference's loader module ``weight_loader_me`` over this library: the reference's own cases
(tests/test_weight_loader.py:43-189 of the reference) restated, plus Q4_0 tensors."""
import os

import numpy as np
import pytest

HIDDEN_SIZE, INTERMEDIATE_SIZE, NUM_Q_HEADS, NUM_KV_HEADS, HEAD_DIM = 128, 256, 4, 2, 32
Q_DIM, KV_DIM, VOCAB_SIZE, MAX_SEQ_LEN, SEED = NUM_Q_HEADS * HEAD_DIM, NUM_KV_HEADS * HEAD_DIM, 32000, 256, 24


def _tiny_config() -> dict:
    return {"hidden_size": HIDDEN_SIZE, "intermediate_size": INTERMEDIATE_SIZE, "num_layers": 1, "num_q_heads": NUM_Q_HEADS,
            "num_kv_heads": NUM_KV_HEADS, "head_dim": HEAD_DIM, "vocab_size": VOCAB_SIZE, "max_seq_len": MAX_SEQ_LEN,
            "freq_base": 10000.0, "rms_norm_epsilon": 1e-6, "tie_word_embeddings": 0}


def _one_layer_tensors() -> dict:
    rng = np.random.RandomState(SEED)
    r = lambda *s: rng.randn(*s).astype(np.float32)
    return {"layer0.w_q": r(HIDDEN_SIZE, Q_DIM), "layer0.w_k": r(HIDDEN_SIZE, KV_DIM), "layer0.w_v": r(HIDDEN_SIZE, KV_DIM),
            "layer0.w_o": r(Q_DIM, HIDDEN_SIZE), "layer0.w_gate": r(HIDDEN_SIZE, INTERMEDIATE_SIZE),
            "layer0.w_up": r(HIDDEN_SIZE, INTERMEDIATE_SIZE), "layer0.w_down": r(INTERMEDIATE_SIZE, HIDDEN_SIZE),
            "layer0.w_input_layernorm": r(HIDDEN_SIZE), "layer0.w_post_attention_layernorm": r(HIDDEN_SIZE),
            "embed": r(512, HIDDEN_SIZE), "lm_head": r(HIDDEN_SIZE, 512), "final_norm": r(HIDDEN_SIZE)}


@pytest.fixture(scope="module")
def wl(native_lib):
    import sys

    import jjjetson_ops_b200 as pkg

    d = pkg.python_module_dir()
    if d not in sys.path:
        sys.path.insert(0, d)
    import weight_loader_me

    return weight_loader_me


def _check_config(got: dict):
    for key, value in _tiny_config().items():
        if isinstance(value, float):
            assert np.isclose(got[key], value, rtol=0.0, atol=1e-9), key
        else:
            assert got[key] == value and isinstance(got[key], int), key


def test_validate_config(wl):
    assert wl.validate_config(**_tiny_config()) is True
    assert wl.validate_config(128, 256, 1, 4, 2, 32, 1000, 64) is True  # the three defaults
    for bad in ({"head_dim": 31}, {"num_kv_heads": 8}, {"vocab_size": 0}, {"tie_word_embeddings": 3}):
        with pytest.raises(ValueError):
            wl.validate_config(**dict(_tiny_config(), **bad))


def test_load_fixture_roundtrip(wl, tmp_path):
    from jjjetson_ops_b200 import weights_io as W

    tensors = _one_layer_tensors()
    W.write_fixture(str(tmp_path), _tiny_config(), tensors)
    loaded = wl.load_fixture(str(tmp_path))
    assert loaded["num_tensors"] == len(tensors)
    _check_config(loaded["config"])
    for name, expected in tensors.items():
        assert np.array_equal(np.asarray(loaded["tensors"][name], dtype=np.float32), expected), name
    with pytest.raises(RuntimeError):
        wl.load_fixture(str(tmp_path / "missing"))


def test_safetensors_cases(wl, tmp_path):
    from jjjetson_ops_b200 import weights_io as W

    small = {"embed": np.array([[1.0, 2.0], [3.0, 4.0]], dtype=np.float32), "layer0.w_q": np.array([0.5, -0.25, 1.25, 0.0], dtype=np.float32),
             "final_norm": np.array([0.1, 0.2, 0.3], dtype=np.float32)}
    p = str(tmp_path / "a" / "w.safetensors")
    os.makedirs(os.path.dirname(p))
    W.write_safetensors(p, small)
    loaded = wl.load_safetensors(p)
    assert loaded["num_tensors"] == 3 and all(np.array_equal(loaded["tensors"][k], v) for k, v in small.items())
    assert loaded["config"]["hidden_size"] == 0 and loaded["config"]["freq_base"] == 0.0  # no config.txt: all zero
    # fixture directory -> one file beside its config.txt -> both loaders agree, config included
    tensors = _one_layer_tensors()
    fx = tmp_path / "fx"
    W.write_fixture(str(fx), _tiny_config(), tensors)
    st = str(fx / "weights.safetensors")
    W.fixture_to_safetensors(str(fx), st)
    from_fx, from_st = wl.load_fixture(str(fx)), wl.load_safetensors(st)
    assert from_fx["num_tensors"] == from_st["num_tensors"] == len(tensors)
    _check_config(from_st["config"])
    for name, expected in tensors.items():
        assert np.array_equal(from_fx["tensors"][name], expected) and np.array_equal(from_st["tensors"][name], expected)
    with pytest.raises(RuntimeError):
        wl.load_safetensors(str(tmp_path / "none.safetensors"))


def test_q4_0_tensors_come_back_as_raw_blocks(wl, oracle, tmp_path):
    from jjjetson_ops_b200 import weights_io as W

    tensors = dict(_one_layer_tensors())
    wq = oracle.quantize_q4_0(np.ascontiguousarray(tensors["layer0.w_down"].reshape(HIDDEN_SIZE, INTERMEDIATE_SIZE)))
    tensors["layer0.w_down"] = W.Tensor(W.DTYPE_Q4_0, (HIDDEN_SIZE, INTERMEDIATE_SIZE), wq)
    W.write_fixture(str(tmp_path), _tiny_config(), tensors)
    loaded = wl.load_fixture(str(tmp_path))
    got = loaded["tensors"]["layer0.w_down"]
    assert got.dtype == np.uint8 and got.shape == (HIDDEN_SIZE, INTERMEDIATE_SIZE // 32 * 18) and np.array_equal(got.reshape(-1), wq.reshape(-1))
    assert loaded["dtypes"]["layer0.w_down"] == "Q4_0" and loaded["dims"]["layer0.w_down"] == [HIDDEN_SIZE, INTERMEDIATE_SIZE]
    assert loaded["dtypes"]["embed"] == "F32"
