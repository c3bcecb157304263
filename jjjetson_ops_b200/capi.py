"""ctypes binding of ``libjq_b200.so`` with torch tensors as device memory.

Every function here is a direct call through the C ABI declared in ``include/jq_b200.h``; torch
only provides allocations and the current stream.  The library is loaded at import time and a
missing build is an error, never a fallback.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
# JQ_B200_LIBRARY names another build of the same library beside this file (the range-checked debug build,
# libjq_b200_check.so, for the test that runs the kernels with their range checks on)
LIB_PATH = os.path.join(_PKG, os.path.basename(os.environ.get("JQ_B200_LIBRARY", "") or "libjq_b200.so"))

OK = 0
ERR_INVALID_ARG, ERR_SHAPE, ERR_ALIGN, ERR_CUDA, ERR_UNSUPPORTED, ERR_TIMEOUT, ERR_TOO_LARGE = range(1, 8)
ORDER_KSUPER_COL, ORDER_COL_KSUPER = 0, 1
S_SUM_X, S_D_SUM_Q = 0, 1
KERNEL_AUTO, KERNEL_GENERIC, KERNEL_GEMV_DP4A, KERNEL_GEMV_MMA, KERNEL_GEMM_MMA, KERNEL_GEMM_TC, KERNEL_GEMM_F16 = range(7)
KERNEL_NAMES = {
    KERNEL_AUTO: "auto",
    KERNEL_GENERIC: "generic",
    KERNEL_GEMV_DP4A: "gemv_dp4a",
    KERNEL_GEMV_MMA: "gemv_mma",
    KERNEL_GEMM_MMA: "gemm_mma",
    KERNEL_GEMM_TC: "gemm_tc",
    KERNEL_GEMM_F16: "gemm_f16",
}

Q4_BYTES = 18
Q8_BYTES = 144


class JqError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__("jq status %d (%s): %s" % (status, status_string(status), message))
        self.status = status


if not os.path.exists(LIB_PATH):
    raise ImportError(
        "%s is missing: build it with `python -m jjjetson_ops_b200._build` "
        "(there is no CPU or PyTorch fallback for this path)" % LIB_PATH
    )
_lib = ctypes.CDLL(LIB_PATH)

_vp, _i64, _ci, _sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
_SIGS = {
    "jq_status_string": (ctypes.c_char_p, [_ci]),
    "jq_last_error": (ctypes.c_char_p, []),
    "jq_version": (_ci, []),
    "jq_set_option": (_ci, [_ci, _ci]),
    "jq_trace_enable": (_ci, [_vp, _i64]),
    "jq_get_option": (_ci, [_ci, ctypes.POINTER(_ci)]),
    "jq_q8_1_bytes": (_sz, [_i64, _i64]),
    "jq_q4_0_bytes": (_sz, [_i64, _i64]),
    "jq_quantize_q8_1_device": (_ci, [_vp, _vp, _vp, _i64, _i64, _ci, _ci]),
    "jq_mul_mat_q4_0_q8_1_device": (_ci, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _ci]),
    "jq_mul_mat_q4_0_q8_1_device_ex": (_ci, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _ci, _ci]),
    "jq_linear_q4_0_device": (_ci, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _ci]),
    "jq_rms_norm_q8_1_device": (_ci, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, ctypes.c_float, _ci, _ci]),
    "jq_swiglu_q8_1_device": (_ci, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _ci, _ci]),
    "rms_norm_fused_add_forward_device": (_ci, [_vp, _vp, _vp, _vp, _ci, _ci, ctypes.c_float]),
    "rms_norm_forward_device": (_ci, [_vp, _vp, _vp, _vp, _ci, _ci, ctypes.c_float]),
    "swiglu_silu_mul_launch_device": (None, [_vp, _vp, _vp, _vp, _ci]),
    "linear_q4_0_forward_device": (_ci, [_vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci]),
    "lm_head_q4_0_forward_device": (_ci, [_vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci]),
    "jq_linear_q4_0_multi_device": (_ci, [_vp, _ci, ctypes.POINTER(_vp), ctypes.POINTER(_i64), ctypes.POINTER(_vp), _vp, _vp, _vp,
                                          _i64, _i64, _ci]),
    "jq_peer_alloc": (_ci, [_sz, ctypes.POINTER(_vp), ctypes.c_char_p]),
    "jq_peer_open": (_ci, [ctypes.c_char_p, ctypes.POINTER(_vp)]),
    "jq_peer_close": (_ci, [_vp]),
    "jq_peer_free": (_ci, [_vp]),
    "jq_linear_q4_0_allgather_device": (_ci, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _ci, ctypes.POINTER(_vp),
                                              ctypes.POINTER(_vp), _ci, _ci, _i64, _i64, _sz, _ci, _vp, _vp]),
    "jq_allgather_wait_device": (_ci, [_vp, _vp, _ci, _vp]),
    "jq_linear_q4_0_allgather_tagged_device": (_ci, [_vp, _vp, _vp, _vp, _sz, _i64, _i64, _i64, _ci, _i64, _i64, _i64, _ci,
                                                     ctypes.POINTER(_vp), _ci, _ci, _i64, _i64, _sz, _vp]),
    "jq_allgather_tagged_read_device": (_ci, [_vp, _vp, _sz, _i64, _i64, _vp, _vp]),
    "jq_linear_q4_0_device_noalloc": (_ci, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _ci]),
    "jq_block_sums_q4_0_q8_1_device": (_ci, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _ci]),
    "jq_quantize_q4_0_device": (_ci, [_vp, _vp, _vp, _i64, _i64]),
    "jq_device_fault": (_ci, [_ci, ctypes.POINTER(_ci)]),
    "jq_bounds_checked": (_ci, []),
    "jq_debug_set_extent_shrink": (_ci, [ctypes.c_ulonglong]),
    "jq_q8_1_host": (_ci, [_vp, _vp, ctypes.POINTER(_ci), _ci]),
    "jq_parse_q8_1_output": (_ci, [_vp, _vp, _vp, _vp, _i64]),
    "jq_mat_mul_q4_0_q8_1_host": (_ci, [_vp, _vp, _vp, _vp, ctypes.POINTER(_ci), _ci, _ci, _ci]),
    "jq_mat_mul_q4_0_q8_1_host_ex": (_ci, [_vp, _vp, _vp, _vp, ctypes.POINTER(_ci), _ci, _ci, _ci, _ci]),
    "jq_weights_create": (_ci, [_vp, _i64, _i64, ctypes.POINTER(_vp)]),
    "jq_weights_destroy": (_ci, [_vp]),
    "jq_weights_device_ptr": (_vp, [_vp]),
    "jq_linear_q4_0_host": (_ci, [_vp, _vp, _vp, _vp, _i64, _ci]),
    "jq_query_device_hw_info": (_ci, [_ci, _vp]),
}
for _name, (_res, _args) in _SIGS.items():
    _fn = getattr(_lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def lib() -> ctypes.CDLL:
    return _lib


def status_string(status: int) -> str:
    return _lib.jq_status_string(status).decode()


def last_error() -> str:
    return _lib.jq_last_error().decode()


def check(status: int) -> None:
    if status != OK:
        raise JqError(status, last_error())


OPT_STATIC_WEIGHTS = 0
OPT_PREFILL_EXACT = 1
OPT_WAIT_POLL_LIMIT = 2


def set_option(option: int, value: int) -> None:
    check(_lib.jq_set_option(option, value))


def get_option(option: int) -> int:
    v = ctypes.c_int(0)
    check(_lib.jq_get_option(option, ctypes.byref(v)))
    return int(v.value)


def q8_1_bytes(K: int, M: int) -> int:
    return int(_lib.jq_q8_1_bytes(K, M))


def q4_0_bytes(N: int, K: int) -> int:
    return int(_lib.jq_q4_0_bytes(N, K))


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _dev(t: torch.Tensor, dtype: torch.dtype, name: str) -> int:
    if not t.is_cuda or t.dtype != dtype or not t.is_contiguous():
        raise ValueError("%s must be a contiguous CUDA tensor of dtype %s" % (name, dtype))
    return t.data_ptr()


def quantize_q8_1(x: torch.Tensor, order: int = ORDER_COL_KSUPER, s_mode: int = S_SUM_X,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 ``[M, K]`` -> raw ``block_q8_1_mmq`` bytes on the same device."""
    M, K = x.shape
    if out is None:
        out = torch.empty(q8_1_bytes(K, M), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        check(_lib.jq_quantize_q8_1_device(_stream(x), _dev(x, torch.float32, "x"), _dev(out, torch.uint8, "out"),
                                           K, M, order, s_mode))
    return out


def mul_mat_q4_0_q8_1(w: torch.Tensor, xq: torch.Tensor, K: int, N: int, M: int,
                      order: int = ORDER_COL_KSUPER, kernel: int = KERNEL_AUTO,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Q4_0 weights x Q8_1 activations -> fp32 ``[M, N]``."""
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=w.device)
    with torch.cuda.device(w.device):
        check(_lib.jq_mul_mat_q4_0_q8_1_device_ex(_stream(w), _dev(w, torch.uint8, "w"), _dev(xq, torch.uint8, "xq"),
                                                  _dev(out, torch.float32, "out"), K, N, M, order, kernel))
    return out


def linear_q4_0(w: torch.Tensor, x: torch.Tensor, N: int, s_mode: int = S_D_SUM_Q,
                ws: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 activations ``[M, K]`` -> quantize -> multiply -> fp32 ``[M, N]`` in one call."""
    M, K = x.shape
    if ws is None:
        ws = torch.empty(max(q8_1_bytes(K, M), 16), dtype=torch.uint8, device=x.device)
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(_lib.jq_linear_q4_0_device(_stream(x), _dev(w, torch.uint8, "w"), _dev(x, torch.float32, "x"),
                                         _dev(ws, torch.uint8, "ws"), _dev(out, torch.float32, "out"), K, N, M, s_mode))
    return out


def linear_q4_0_multi(ws_list, N_list, x: Optional[torch.Tensor] = None, xq: Optional[torch.Tensor] = None,
                      K: Optional[int] = None, M: Optional[int] = None, s_mode: int = S_D_SUM_Q,
                      ws: Optional[torch.Tensor] = None, outs=None):
    """Several linears that share their input in one call (separate q/k/v or gate/up weights).  Give ``x``
    (fp32 ``[M, K]``) or ``xq`` (Q8_1 blocks, with ``K`` and ``M``).  Returns the list of outputs."""
    dev = ws_list[0].device
    if x is not None:
        M, K = x.shape
        if ws is None:
            ws = torch.empty(max(q8_1_bytes(K, M), 16), dtype=torch.uint8, device=dev)
    n = len(ws_list)
    if outs is None:
        outs = [torch.empty((M, int(Ni)), dtype=torch.float32, device=dev) for Ni in N_list]
    wp = (_vp * n)(*[_dev(w, torch.uint8, "w") for w in ws_list])
    yp = (_vp * n)(*[_dev(y, torch.float32, "out") for y in outs])
    np_ = (_i64 * n)(*[int(v) for v in N_list])
    with torch.cuda.device(dev):
        check(_lib.jq_linear_q4_0_multi_device(
            _stream(ws_list[0]), n, wp, np_, yp, None if x is None else _dev(x, torch.float32, "x"),
            None if xq is None else _dev(xq, torch.uint8, "xq"), None if ws is None else _dev(ws, torch.uint8, "ws"), K, M, s_mode))
    return outs


def rms_norm_q8_1(x: torch.Tensor, weight: torch.Tensor, epsilon: float, residual: Optional[torch.Tensor] = None,
                  normed: Optional[torch.Tensor] = None, want_q8: bool = True, order: int = ORDER_COL_KSUPER,
                  s_mode: int = S_D_SUM_Q, xq: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """RMSNorm of ``x`` ``[T, H]`` (with ``residual`` given: z = x + residual, residual <- z first) with the
    Q8_1 quantizer folded in.  ``normed`` (may be ``x`` itself) receives the fp32 result; the returned uint8
    tensor holds the Q8_1 blocks of it (``None`` when ``want_q8`` is false)."""
    T, H = x.shape
    if want_q8 and xq is None:
        xq = torch.empty(max(q8_1_bytes(H, T), 16), dtype=torch.uint8, device=x.device)
    if not want_q8:
        xq = None
    with torch.cuda.device(x.device):
        check(_lib.jq_rms_norm_q8_1_device(
            _stream(x), _dev(x, torch.float32, "x"), None if residual is None else _dev(residual, torch.float32, "residual"),
            _dev(weight, torch.float32, "weight"), None if normed is None else _dev(normed, torch.float32, "normed"),
            None if xq is None else xq.data_ptr(), H, T, float(epsilon), order, s_mode))
    return xq


def swiglu_q8_1(gate: torch.Tensor, up: torch.Tensor, mid: Optional[torch.Tensor] = None, want_q8: bool = True,
                order: int = ORDER_COL_KSUPER, s_mode: int = S_D_SUM_Q,
                xq: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """silu(gate) * up over ``[T, I]`` with the Q8_1 quantizer folded in; ``mid`` receives the fp32 result."""
    T, I = gate.shape
    if want_q8 and xq is None:
        xq = torch.empty(max(q8_1_bytes(I, T), 16), dtype=torch.uint8, device=gate.device)
    if not want_q8:
        xq = None
    with torch.cuda.device(gate.device):
        check(_lib.jq_swiglu_q8_1_device(
            _stream(gate), _dev(gate, torch.float32, "gate"), _dev(up, torch.float32, "up"),
            None if mid is None else _dev(mid, torch.float32, "mid"), None if xq is None else xq.data_ptr(), I, T, order, s_mode))
    return xq


NOALLOC_WS_BYTES = 4 << 20


def linear_q4_0_noalloc(w: torch.Tensor, x: torch.Tensor, N: int, s_mode: int = S_D_SUM_Q,
                        out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``linear_q4_0`` through the entry point that owns its scratch (no workspace argument, no
    allocation inside the library; ``out`` is allocated here by torch only if not given)."""
    M, K = x.shape
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(_lib.jq_linear_q4_0_device_noalloc(_stream(x), _dev(w, torch.uint8, "w"), _dev(x, torch.float32, "x"),
                                                 _dev(out, torch.float32, "out"), K, N, M, s_mode))
    return out


def peer_alloc(nbytes: int):
    """Zeroed device memory that other processes of the node can map -> (device pointer, 64-byte handle)."""
    ptr = _vp()
    handle = ctypes.create_string_buffer(64)
    check(_lib.jq_peer_alloc(nbytes, ctypes.byref(ptr), handle))
    return int(ptr.value), handle.raw


def peer_open(handle: bytes) -> int:
    ptr = _vp()
    check(_lib.jq_peer_open(handle, ctypes.byref(ptr)))
    return int(ptr.value)


def peer_close(ptr: int) -> None:
    check(_lib.jq_peer_close(ptr))


def peer_free(ptr: int) -> None:
    check(_lib.jq_peer_free(ptr))


class _RawDeviceMemory:
    """Lets torch view memory this library allocated (``__cuda_array_interface__``)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3}


def tensor_from_ptr(ptr: int, shape, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    typestr = {torch.float32: "<f4", torch.uint8: "|u1", torch.int32: "<i4"}[dtype]
    return torch.as_tensor(_RawDeviceMemory(ptr, shape, typestr), device=device)


def linear_q4_0_allgather(w: torch.Tensor, x: torch.Tensor, ws: torch.Tensor, N_local: int, s_mode: int,
                          y_peers, flag_peers, world: int, rank: int, n_offset: int, N_total: int,
                          y_stride_bytes: int, wait_previous: bool, epoch: torch.Tensor, counter: torch.Tensor) -> None:
    """This rank's quantize + multiply with its output band stored into every rank's buffer."""
    M, K = x.shape
    yp = (_vp * world)(*y_peers)
    fp = (_vp * world)(*flag_peers)
    with torch.cuda.device(x.device):
        check(_lib.jq_linear_q4_0_allgather_device(
            _stream(x), _dev(w, torch.uint8, "w"), _dev(x, torch.float32, "x"), _dev(ws, torch.uint8, "ws"), K, N_local, M,
            s_mode, yp, fp, world, rank, n_offset, N_total, y_stride_bytes, 1 if wait_previous else 0,
            _dev(epoch, torch.int32, "epoch"), _dev(counter, torch.int32, "counter")))


def allgather_wait(device: torch.device, flags_ptr: int, world: int, epoch: torch.Tensor) -> None:
    with torch.cuda.device(device):
        check(_lib.jq_allgather_wait_device(torch.cuda.current_stream(device).cuda_stream, flags_ptr, world,
                                            _dev(epoch, torch.int32, "epoch")))


def linear_q4_0_allgather_tagged(w: torch.Tensor, x: Optional[torch.Tensor], x_words_ptr: int, x_stride_bytes: int,
                                 x_row_words: int, x_seg_len: int, x_seg_stride: int, x_back: int, K: int, N_local: int, M: int,
                                 s_mode: int, word_peers, world: int, rank: int, n_offset: int, N_total: int,
                                 y_stride_bytes: int, ticket: torch.Tensor) -> None:
    """Decode form of the fused all-gather: this rank's band goes to every rank as tagged 8-byte words.  The
    activations are either the plain tensor ``x`` or the words at ``x_words_ptr`` (the previous all-gather)."""
    wp = (_vp * world)(*word_peers)
    with torch.cuda.device(w.device):
        check(_lib.jq_linear_q4_0_allgather_tagged_device(
            _stream(w), _dev(w, torch.uint8, "w"), None if x is None else _dev(x, torch.float32, "x"),
            x_words_ptr if x is None else None, x_stride_bytes, x_row_words, x_seg_len, x_seg_stride, x_back, K, N_local, M, s_mode, wp,
            world, rank, n_offset, N_total, y_stride_bytes, _dev(ticket, torch.int64, "ticket")))


def allgather_tagged_read(device: torch.device, words_ptr: int, stride_bytes: int, M: int, N_total: int,
                          ticket: torch.Tensor, out: torch.Tensor) -> None:
    with torch.cuda.device(device):
        check(_lib.jq_allgather_tagged_read_device(torch.cuda.current_stream(device).cuda_stream, words_ptr, stride_bytes, M,
                                                   N_total, _dev(ticket, torch.int64, "ticket"), _dev(out, torch.float32, "out")))


def block_sums(w: torch.Tensor, xq: torch.Tensor, K: int, N: int, M: int,
               order: int = ORDER_COL_KSUPER) -> torch.Tensor:
    """Exact int32 block dot products ``[M, N, K/32]``."""
    out = torch.empty((M, N, K // 32), dtype=torch.int32, device=w.device)
    with torch.cuda.device(w.device):
        check(_lib.jq_block_sums_q4_0_q8_1_device(_stream(w), _dev(w, torch.uint8, "w"), _dev(xq, torch.uint8, "xq"),
                                                  _dev(out, torch.int32, "out"), K, N, M, order))
    return out


def quantize_q4_0(w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 ``[N, K]`` -> Q4_0 bytes ``[N, K/32*18]``."""
    N, K = w.shape
    if out is None:
        out = torch.empty((N, K // 32 * Q4_BYTES), dtype=torch.uint8, device=w.device)
    with torch.cuda.device(w.device):
        check(_lib.jq_quantize_q4_0_device(_stream(w), _dev(w, torch.float32, "w"), _dev(out, torch.uint8, "out"), N, K))
    return out


def device_fault(clear: bool = True) -> int:
    """The device's fault word (0: no bounded wait has given up).  A non-zero word comes with status
    JQ_ERR_TIMEOUT, which is reported through the return value here, not raised."""
    v = ctypes.c_int(0)
    rc = _lib.jq_device_fault(1 if clear else 0, ctypes.byref(v))
    if rc not in (OK, ERR_TIMEOUT):
        check(rc)
    return int(v.value)


class DeviceHwInfo(ctypes.Structure):
    _fields_ = [
        ("name", ctypes.c_char * 256),
        ("device_id", _ci), ("cc_major", _ci), ("cc_minor", _ci), ("sm_count", _ci),
        ("sm_clock_khz", _ci), ("mem_clock_khz", _ci), ("mem_bus_width_bits", _ci),
        ("fp32_cores_per_sm", _ci), ("warp_schedulers_per_sm", _ci), ("max_warps_per_sm", _ci),
        ("smem_per_sm", _sz), ("smem_per_block_optin", _sz), ("l2_bytes", _sz), ("global_mem_bytes", _sz),
        ("peak_fp32_tflops", ctypes.c_double), ("peak_dram_gbs", ctypes.c_double),
        ("peak_int8_dense_tops", ctypes.c_double), ("peak_bf16_dense_tflops", ctypes.c_double),
        ("ridge_int8_ops_per_byte", ctypes.c_double),
    ]

    def as_dict(self) -> dict:
        d = {}
        for f, _ in self._fields_:
            v = getattr(self, f)
            d[f] = v.decode() if isinstance(v, bytes) else v
        return d


def query_device_hw_info(device: int = 0) -> dict:
    info = DeviceHwInfo()
    check(_lib.jq_query_device_hw_info(device, ctypes.byref(info)))
    return info.as_dict()


class ResidentWeights:
    """Host-facing linear with the weights uploaded once (``jq_weights_*`` of the C ABI)."""

    def __init__(self, w_q4_0_host, N: int, K: int):
        import numpy as np

        w = np.ascontiguousarray(w_q4_0_host, dtype=np.uint8)
        assert w.nbytes >= q4_0_bytes(N, K)
        self.N, self.K = N, K
        self._h = _vp()
        check(_lib.jq_weights_create(w.ctypes.data, N, K, ctypes.byref(self._h)))

    @property
    def device_ptr(self) -> int:
        return int(_lib.jq_weights_device_ptr(self._h) or 0)

    def linear(self, x_host_ptr: int, y_host_ptr: int, M: int, s_mode: int = S_D_SUM_Q, ws_host_ptr: int = 0) -> None:
        check(_lib.jq_linear_q4_0_host(self._h, x_host_ptr, ws_host_ptr or None, y_host_ptr, M, s_mode))

    def close(self) -> None:
        if self._h:
            _lib.jq_weights_destroy(self._h)
            self._h = _vp()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
