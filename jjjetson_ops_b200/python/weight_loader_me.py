"""``weight_loader_me``: the reference's loader module, same names and results, over this library's readers.

The reference builds this module with pybind11 (src/bindings/weight_loader_binding.cpp:54-110):
``validate_config(**ModelConfig fields) -> True`` (``ValueError`` when the values are inconsistent),
``load_fixture(path)`` and ``load_safetensors(path)`` -> ``{"config": {...}, "tensors": {name: array},
"num_tensors": n}`` (``RuntimeError`` when the loader fails).  Here the same three functions sit on
``jq_weights_load_fixture`` / ``jq_weights_load_safetensors`` / ``jq_model_config_parse`` of the C ABI, so
that they also read the Q4_0 tensor type: such a tensor comes back as a ``uint8`` array
``[rows, K / 32 * 18]`` of raw 18-byte blocks, and the extra key ``"dtypes"`` says which
(``"F32"`` or ``"Q4_0"``) with ``"dims"`` giving ``[rows, K]``.

Differences to know: a fixture's ``config.txt`` must hold all eleven keys, as in the reference; a
safetensors file without a ``config.txt`` beside it yields the reference's all-zero config.
"""
from __future__ import annotations

import os
import sys

_pkg_parent = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if _pkg_parent not in sys.path:
    sys.path.insert(0, _pkg_parent)

from jjjetson_ops_b200 import capi as _capi  # noqa: E402
from jjjetson_ops_b200 import model as _model  # noqa: E402
from jjjetson_ops_b200 import weights_io as _wio  # noqa: E402

_KEYS = ("hidden_size", "intermediate_size", "num_layers", "num_q_heads", "num_kv_heads", "head_dim", "vocab_size",
         "max_seq_len", "freq_base", "rms_norm_epsilon", "tie_word_embeddings")
_INT_KEYS = frozenset(k for k in _KEYS if k not in ("freq_base", "rms_norm_epsilon"))


def validate_config(hidden_size, intermediate_size, num_layers, num_q_heads, num_kv_heads, head_dim, vocab_size, max_seq_len,
                    freq_base=10000.0, rms_norm_epsilon=1e-5, tie_word_embeddings=0) -> bool:
    """model_config_validate: True, or ``ValueError("invalid ModelConfig")``."""
    values = dict(zip(_KEYS, (hidden_size, intermediate_size, num_layers, num_q_heads, num_kv_heads, head_dim, vocab_size,
                              max_seq_len, freq_base, rms_norm_epsilon, tie_word_embeddings)))
    text = "".join("%s=%r\n" % (k, int(v) if k in _INT_KEYS else float(v)) for k, v in values.items())
    try:
        _model.parse_config(text)
    except _capi.JqError as e:
        raise ValueError("invalid ModelConfig") from e
    return True


def _config_of(path_of_config_txt: str, required: bool) -> dict:
    try:
        with open(path_of_config_txt, "r", encoding="utf-8") as f:
            text = f.read()
    except OSError:
        if required:
            raise RuntimeError("weight_loader_load_fixture failed") from None
        return {k: (0 if k in _INT_KEYS else 0.0) for k in _KEYS}
    cfg = _model.parse_config(text)
    return {k: (int(cfg[k]) if k in _INT_KEYS else float(cfg[k])) for k in _KEYS}


def _result(config: dict, tensors: dict) -> dict:
    return {
        "config": config,
        "tensors": {name: t.data for name, t in tensors.items()},
        "num_tensors": len(tensors),
        "dtypes": {name: ("Q4_0" if t.dtype == _wio.DTYPE_Q4_0 else "F32") for name, t in tensors.items()},
        "dims": {name: list(t.dims) for name, t in tensors.items()},
    }


def load_fixture(path: str) -> dict:
    try:
        config = _config_of(os.path.join(path, "config.txt"), required=True)
        _, tensors = _wio.load_fixture(path)
    except _capi.JqError as e:
        raise RuntimeError("weight_loader_load_fixture failed: %s" % e) from e
    return _result(config, tensors)


def load_safetensors(path: str) -> dict:
    try:
        config = _config_of(os.path.join(os.path.dirname(os.path.abspath(path)), "config.txt"), required=False)
        _, tensors = _wio.load_safetensors(path)
    except _capi.JqError as e:
        raise RuntimeError("weight_loader_load_safetensors failed: %s" % e) from e
    return _result(config, tensors)
