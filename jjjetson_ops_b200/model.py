"""The model's weights on the device with Q4_0 linears: ctypes layer over ``include/jq_model.h``.

The quantized counterpart of the reference's weight container (``TransformerModel`` /
``TransformerLayerWeights``, src/model/transformer_model.h:13-52): one device allocation per model, per
layer the seven linears as Q4_0 blocks (q, k, v adjacent and gate, up adjacent, so each group is also one
matrix for a single launch) and the two norm vectors in fp32.  Planning the layout needs no GPU.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, NamedTuple, Optional

from . import capi
from .weights_io import _WeightSet  # the loaders' result type
from . import weights_io as _wio

_lib = capi.lib()


class _Config(ctypes.Structure):
    _fields_ = [(k, ctypes.c_int) for k in ("hidden_size", "intermediate_size", "num_layers", "num_q_heads", "num_kv_heads",
                                            "head_dim", "vocab_size", "max_seq_len")] + \
               [("freq_base", ctypes.c_float), ("rms_norm_epsilon", ctypes.c_float), ("tie_word_embeddings", ctypes.c_int)]


class _Slot(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char * 96), ("dtype", ctypes.c_int), ("rows", ctypes.c_int64), ("K", ctypes.c_int64),
                ("offset", ctypes.c_size_t), ("nbytes", ctypes.c_size_t)]


class _Plan(ctypes.Structure):
    _fields_ = [("config", _Config), ("slots", ctypes.POINTER(_Slot)), ("num_slots", ctypes.c_int), ("total_bytes", ctypes.c_size_t)]


class _LayerWeights(ctypes.Structure):
    _fields_ = [(k, ctypes.c_void_p) for k in ("d_w_q", "d_w_k", "d_w_v", "d_w_o", "d_w_gate", "d_w_up", "d_w_down",
                                               "d_w_input_layernorm", "d_w_post_attention_layernorm", "d_w_qkv", "d_w_gate_up")]


_PP = ctypes.POINTER
_lib.jq_model_config_parse.restype = ctypes.c_int
_lib.jq_model_config_parse.argtypes = [ctypes.c_char_p, _PP(_Config)]
_lib.jq_model_q4_0_plan.restype = ctypes.c_int
_lib.jq_model_q4_0_plan.argtypes = [_PP(_WeightSet), _PP(_PP(_Plan))]
_lib.jq_model_plan_destroy.restype = None
_lib.jq_model_plan_destroy.argtypes = [_PP(_Plan)]
_lib.jq_model_q4_0_create.restype = ctypes.c_int
_lib.jq_model_q4_0_create.argtypes = [_PP(_WeightSet), _PP(ctypes.c_void_p)]
_lib.jq_model_q4_0_destroy.restype = None
_lib.jq_model_q4_0_destroy.argtypes = [ctypes.c_void_p]
_lib.jq_model_q4_0_config.restype = _PP(_Config)
_lib.jq_model_q4_0_config.argtypes = [ctypes.c_void_p]
_lib.jq_model_q4_0_layout.restype = _PP(_Plan)
_lib.jq_model_q4_0_layout.argtypes = [ctypes.c_void_p]
_lib.jq_model_q4_0_layer.restype = _PP(_LayerWeights)
_lib.jq_model_q4_0_layer.argtypes = [ctypes.c_void_p, ctypes.c_int]
_lib.jq_model_q4_0_embed.restype = ctypes.c_void_p
_lib.jq_model_q4_0_embed.argtypes = [ctypes.c_void_p, _PP(ctypes.c_int)]
_lib.jq_model_q4_0_final_norm.restype = ctypes.c_void_p
_lib.jq_model_q4_0_final_norm.argtypes = [ctypes.c_void_p]
_lib.jq_model_q4_0_lm_head.restype = ctypes.c_void_p
_lib.jq_model_q4_0_lm_head.argtypes = [ctypes.c_void_p, _PP(ctypes.c_int)]


class Slot(NamedTuple):
    name: str
    dtype: int
    rows: int
    K: int
    offset: int
    nbytes: int


def _config_dict(c: _Config) -> Dict[str, float]:
    return {k: getattr(c, k) for k, _ in _Config._fields_}


def parse_config(text: str) -> Dict[str, float]:
    """The eleven keys of a ``config.txt``, validated as the reference validates a ``ModelConfig``."""
    c = _Config()
    capi.check(_lib.jq_model_config_parse(text.encode(), ctypes.byref(c)))
    return _config_dict(c)


def _load(path: str):
    ps = _PP(_WeightSet)()
    load = _wio._lib.jq_weights_load_safetensors if os.path.isfile(path) else _wio._lib.jq_weights_load_fixture
    capi.check(load(os.fsencode(path), ctypes.byref(ps)))
    return ps


def _plan_tuple(plan: _Plan):
    slots = [Slot(plan.slots[i].name.decode(), plan.slots[i].dtype, plan.slots[i].rows, plan.slots[i].K, plan.slots[i].offset,
                  plan.slots[i].nbytes) for i in range(plan.num_slots)]
    return _config_dict(plan.config), slots, int(plan.total_bytes)


def plan(path: str):
    """Validates the weights at ``path`` (fixture directory or ``.safetensors`` file) and lays the model out:
    -> (config, slots in device order, total bytes).  Host only."""
    ps = _load(path)
    try:
        pp = _PP(_Plan)()
        capi.check(_lib.jq_model_q4_0_plan(ps, ctypes.byref(pp)))
        try:
            return _plan_tuple(pp.contents)
        finally:
            _lib.jq_model_plan_destroy(pp)
    finally:
        _wio._lib.jq_weight_set_destroy(ps)


class ModelQ4_0:
    """Weights resident on the current CUDA device.  ``layer(i)`` gives device addresses by slot name."""

    def __init__(self, path: str):
        self._h: Optional[ctypes.c_void_p] = None
        ps = _load(path)
        try:
            h = ctypes.c_void_p()
            capi.check(_lib.jq_model_q4_0_create(ps, ctypes.byref(h)))
            self._h = h
        finally:
            _wio._lib.jq_weight_set_destroy(ps)
        self.config, self.slots, self.total_bytes = _plan_tuple(_lib.jq_model_q4_0_layout(self._h).contents)

    def layer(self, i: int) -> Dict[str, int]:
        p = _lib.jq_model_q4_0_layer(self._h, i)
        if not p:
            raise IndexError(i)
        return {k: int(getattr(p.contents, k) or 0) for k, _ in _LayerWeights._fields_}

    def table(self, which: str):
        """-> (device address, dtype) of ``embed`` or ``lm_head``; (address, F32) of ``final_norm``."""
        d = ctypes.c_int(0)
        if which == "embed":
            return int(_lib.jq_model_q4_0_embed(self._h, ctypes.byref(d)) or 0), d.value
        if which == "lm_head":
            return int(_lib.jq_model_q4_0_lm_head(self._h, ctypes.byref(d)) or 0), d.value
        if which == "final_norm":
            return int(_lib.jq_model_q4_0_final_norm(self._h) or 0), _wio.DTYPE_F32
        raise KeyError(which)

    def close(self) -> None:
        if self._h is not None:
            _lib.jq_model_q4_0_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()


def layer_names(i: int) -> List[str]:
    return ["layer%d.%s" % (i, s) for s in ("w_q", "w_k", "w_v", "w_o", "w_gate", "w_up", "w_down", "w_input_layernorm",
                                            "w_post_attention_layernorm")]


def main(argv=None) -> int:
    """``python -m jjjetson_ops_b200.model PATH``: validate a quantized checkpoint (fixture directory or
    safetensors file) and print its device layout.  Needs no GPU."""
    import sys

    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 1:
        print(main.__doc__, file=sys.stderr)
        return 2
    try:
        config, slots, total = plan(argv[0])
    except capi.JqError as e:
        print("not a loadable quantized model: %s" % e, file=sys.stderr)
        return 1
    print(" ".join("%s=%g" % kv for kv in config.items()))
    print("%-44s %-5s %10s %8s %14s %12s" % ("tensor", "type", "rows", "K", "offset", "bytes"))
    for s in slots:
        print("%-44s %-5s %10d %8d %14d %12d" % (s.name, "Q4_0" if s.dtype == _wio.DTYPE_Q4_0 else "F32", s.rows, s.K, s.offset, s.nbytes))
    print("total %d bytes in one allocation" % total)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
