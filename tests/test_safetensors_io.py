"""The safetensors side of the weight formats (CPU): the reference's loader cases restated
(tests/test_weight_loader.py:90-189 of the reference) plus the Q4_0 tensor type."""
import json
import struct

import numpy as np
import pytest

CONFIG = {"hidden_size": 128, "intermediate_size": 256, "num_layers": 1, "num_q_heads": 4, "num_kv_heads": 2, "head_dim": 32,
          "vocab_size": 64, "max_seq_len": 32, "freq_base": 10000.0, "rms_norm_epsilon": 1e-6, "tie_word_embeddings": 0}


def _raw_file(path, header: dict, data: bytes, pad=b""):
    head = json.dumps(header, separators=(",", ":")).encode("utf-8") + pad
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        f.write(data)


def test_read_format_small_tensors(native_lib, tmp_path):
    """Three F32 tensors of one, one and two dims, as the reference's read-format case."""
    from jjjetson_ops_b200 import weights_io as W

    tensors = {"embed": np.array([[1.0, 2.0], [3.0, 4.0]], dtype=np.float32),
               "layer0.w_q": np.array([0.5, -0.25, 1.25, 0.0], dtype=np.float32),
               "final_norm": np.array([0.1, 0.2, 0.3], dtype=np.float32)}
    p = str(tmp_path / "w.safetensors")
    W.write_safetensors(p, tensors)
    config, got = W.load_safetensors(p)
    assert config == {}  # no config.txt beside the file
    assert set(got) == set(tensors)
    for name, exp in tensors.items():
        assert got[name].dtype == W.DTYPE_F32 and got[name].dims == exp.shape and np.array_equal(got[name].data, exp)


def test_optional_config_beside_the_file(native_lib, tmp_path):
    from jjjetson_ops_b200 import weights_io as W

    W.write_fixture(str(tmp_path), CONFIG, {})
    p = str(tmp_path / "weights.safetensors")
    W.write_safetensors(p, {"embed": np.array([[1.0, 2.0]], dtype=np.float32)})
    config, got = W.load_safetensors(p)
    assert len(got) == 1 and config["hidden_size"] == 128 and config["num_layers"] == 1 and config["rms_norm_epsilon"] == 1e-6


def test_fixture_to_safetensors_roundtrip_with_q4_0(native_lib, oracle, tmp_path):
    """fixture directory -> one file (written by the library) -> loader: tensor by tensor what the fixture
    loader returns, F32 and Q4_0 alike; and the file is plain safetensors for any other reader."""
    from jjjetson_ops_b200 import weights_io as W

    rng = np.random.default_rng(24)
    mk = lambda *s: rng.standard_normal(s).astype(np.float32)
    tensors = {"layer0.w_q": mk(128, 128), "layer0.w_down": mk(256, 128), "layer0.w_input_layernorm": mk(128), "embed": mk(64, 128)}
    wq = oracle.quantize_q4_0(tensors["layer0.w_down"].reshape(128, 256))  # the engine's view: [out=128][in=256]
    tensors["layer0.w_down"] = W.Tensor(W.DTYPE_Q4_0, (128, 256), wq)
    fx = tmp_path / "fx"
    W.write_fixture(str(fx), CONFIG, tensors)
    st = str(fx / "weights.safetensors")
    assert W.fixture_to_safetensors(str(fx), st) == len(tensors)
    cfg_fx, from_fx = W.load_fixture(str(fx))
    cfg_st, from_st = W.load_safetensors(st)
    assert cfg_fx == cfg_st and set(from_fx) == set(from_st) == set(tensors)
    for name in tensors:
        a, b = from_fx[name], from_st[name]
        assert a.dtype == b.dtype and a.dims == b.dims and np.array_equal(a.data, b.data)
    assert from_st["layer0.w_down"].dtype == W.DTYPE_Q4_0 and np.array_equal(from_st["layer0.w_down"].data.reshape(-1), wq.reshape(-1))
    # the file as another reader sees it
    blob = open(st, "rb").read()
    (n,) = struct.unpack("<Q", blob[:8])
    assert n % 8 == 0
    header = json.loads(blob[8:8 + n])
    assert list(header) == sorted(header) and "__metadata__" not in header
    e = header["layer0.w_down.q4_0"]
    assert e["dtype"] == "U8" and e["shape"] == [128, 8, 18] and e["data_offsets"][1] - e["data_offsets"][0] == 128 * 8 * 18
    assert header["embed"] == {"dtype": "F32", "shape": [64, 128], "data_offsets": header["embed"]["data_offsets"]}
    ends = sorted(v["data_offsets"] for v in header.values())
    assert ends[0][0] == 0 and all(a[1] == b[0] for a, b in zip(ends, ends[1:])) and ends[-1][1] == len(blob) - 8 - n
    # and the Python writer's file loads the same way
    st2 = str(tmp_path / "py.safetensors")
    W.write_safetensors(st2, tensors)
    _, from_py = W.load_safetensors(st2)
    for name in tensors:
        assert from_py[name].dims == from_st[name].dims and np.array_equal(from_py[name].data, from_st[name].data)


def test_header_details(native_lib, tmp_path):
    """__metadata__ and unknown keys are skipped, escapes in names are decoded, whitespace is allowed."""
    from jjjetson_ops_b200 import weights_io as W

    a = np.arange(6, dtype=np.float32).reshape(2, 3)
    head = ('{ "__metadata__" : {"format":"pt","nested":{"x":[1,2,{"y":null}]}},\n'
            ' "a\\u0041\\"q" : {"dtype":"F32", "extra": [true, 1.5e3, "s"], "shape":[2,3], "data_offsets":[0,24]} }   ')
    p = str(tmp_path / "m.safetensors")
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head.encode())
        f.write(a.tobytes())
    _, got = W.load_safetensors(p)
    assert list(got) == ['aA"q'] and np.array_equal(got['aA"q'].data, a)


def test_errors_are_reported(native_lib, tmp_path):
    from jjjetson_ops_b200 import weights_io as W

    c = native_lib
    p = str(tmp_path / "bad.safetensors")
    with pytest.raises(c.JqError):
        W.load_safetensors(str(tmp_path / "missing.safetensors"))
    open(p, "wb").write(b"\x01\x02")
    with pytest.raises(c.JqError):
        W.load_safetensors(p)
    open(p, "wb").write(struct.pack("<Q", 1000) + b"{}")  # header length beyond the file
    with pytest.raises(c.JqError):
        W.load_safetensors(p)
    _raw_file(p, {}, b"")  # no tensors: an error, as in the reference
    with pytest.raises(c.JqError):
        W.load_safetensors(p)
    _raw_file(p, {"__metadata__": {"a": "b"}}, b"")
    with pytest.raises(c.JqError):
        W.load_safetensors(p)
    _raw_file(p, {"h": {"dtype": "F16", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 4)  # a dtype the loader does not know
    with pytest.raises(c.JqError) as e:
        W.load_safetensors(p)
    assert e.value.status == c.ERR_UNSUPPORTED and "F16" in str(e.value)
    _raw_file(p, {"u": {"dtype": "U8", "shape": [2, 1, 18], "data_offsets": [0, 36]}}, b"\0" * 36)  # U8 without the .q4_0 name
    with pytest.raises(c.JqError):
        W.load_safetensors(p)
    _raw_file(p, {"w.q4_0": {"dtype": "U8", "shape": [2, 1, 17], "data_offsets": [0, 34]}}, b"\0" * 34)  # not 18-byte blocks
    with pytest.raises(c.JqError):
        W.load_safetensors(p)
    _raw_file(p, {"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}, b"\0" * 16)  # offsets do not match the shape
    with pytest.raises(c.JqError) as e:
        W.load_safetensors(p)
    assert e.value.status == c.ERR_SHAPE
    _raw_file(p, {"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8)  # data past the end of the file
    with pytest.raises(c.JqError):
        W.load_safetensors(p)
    _raw_file(p, {"a": {"dtype": "F32", "shape": [], "data_offsets": [0, 4]}}, b"\0" * 4)  # no dims, as the reference refuses
    with pytest.raises(c.JqError):
        W.load_safetensors(p)
    open(p, "wb").write(struct.pack("<Q", 9) + b'{"a":{"d')  # truncated JSON
    with pytest.raises(c.JqError):
        W.load_safetensors(p)
    _raw_file(p, {"w.q4_0": {"dtype": "U8", "shape": [2, 1, 18], "data_offsets": [0, 36]}}, b"\x11" * 36)  # and a good one
    _, got = W.load_safetensors(p)
    assert got["w"].dtype == W.DTYPE_Q4_0 and got["w"].dims == (2, 32) and got["w"].data.shape == (2, 18)


def test_random_tensor_sets_round_trip(native_lib, tmp_path):
    """Seeded random sets of tensors (names with dots, 1 to 4 dims, F32 and Q4_0 mixed) survive
    writer -> loader through both writers, byte for byte."""
    import ctypes

    from jjjetson_ops_b200 import weights_io as W

    rng = np.random.default_rng(2024)
    for case in range(12):
        tensors = {}
        for i in range(int(rng.integers(1, 9))):
            name = "t%d.%s" % (i, "".join(rng.choice(list("abw_q0"), size=int(rng.integers(1, 8)))))
            if rng.random() < 0.4:
                rows, K = int(rng.integers(1, 20)), 32 * int(rng.integers(1, 9))
                raw = rng.integers(0, 256, size=(rows, K // 32 * 18), dtype=np.uint8)
                tensors[name] = W.Tensor(W.DTYPE_Q4_0, (rows, K), raw)
            else:
                shape = tuple(int(d) for d in rng.integers(1, 7, size=int(rng.integers(1, 5))))
                tensors[name] = rng.standard_normal(shape).astype(np.float32)
        py_file = str(tmp_path / ("py%d.safetensors" % case))
        W.write_safetensors(py_file, tensors)
        _, got = W.load_safetensors(py_file)
        # the library's own writer, fed with what it just loaded
        ps = ctypes.POINTER(W._WeightSet)()
        native_lib.check(W._lib.jq_weights_load_safetensors(py_file.encode(), ctypes.byref(ps)))
        c_file = str(tmp_path / ("c%d.safetensors" % case))
        try:
            native_lib.check(W._lib.jq_weights_save_safetensors(ps, c_file.encode()))
        finally:
            W._lib.jq_weight_set_destroy(ps)
        _, again = W.load_safetensors(c_file)
        assert set(got) == set(again) == set(tensors)
        for name, t in tensors.items():
            exp = t.data if isinstance(t, W.Tensor) else t
            for loaded in (got[name], again[name]):
                assert loaded.dims == (t.dims if isinstance(t, W.Tensor) else t.shape)
                assert loaded.dtype == (W.DTYPE_Q4_0 if isinstance(t, W.Tensor) else W.DTYPE_F32)
                assert np.array_equal(loaded.data.reshape(-1), np.asarray(exp).reshape(-1))
