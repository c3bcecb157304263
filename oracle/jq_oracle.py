"""Loader for the C oracle (``jq_oracle.c``) plus an independent NumPy mirror of it.

TEST INFRASTRUCTURE ONLY: nothing in ``jjjetson_ops_b200`` imports this module.

Two restatements of the reference arithmetic live here on purpose: the C one (fast enough
for the large configurations and used as the timed CPU baseline) and a vectorised NumPy one
written separately, so that a slip in either shows up as a disagreement between them.
Reference lines are cited by their path inside the reference project.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libjq_oracle.so")

ORDER_KSUPER_COL = 0  # write order of quantize_q8_1_kernel, src/cuda/q8_1.cu:84-86
ORDER_COL_KSUPER = 1  # read order of the multiply, src/cuda/mm_q4_0_q8_1.cu:230,246
S_SUM_X = 0  # s = fp16(sum of the 32 floats), src/cuda/q8_1.cu:62-68,102
S_D_SUM_Q = 1  # s = fp16(fp16(d) * sum of the 32 int8)

Q4_BYTES = 18
Q8_BYTES = 144

_lib = None


def build(force: bool = False) -> str:
    """Compile ``libjq_oracle.so`` with the Makefile beside this file."""
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(
        os.path.join(_HERE, "jq_oracle.c")
    ):
        subprocess.run(["make", "-C", _HERE, "-s", "-B"], check=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        p = ctypes.c_void_p
        i64 = ctypes.c_int64
        ci = ctypes.c_int
        L.jqo_quantize_q4_0.argtypes = [p, i64, i64, p]
        L.jqo_dequantize_q4_0.argtypes = [p, i64, i64, p]
        L.jqo_quantize_q8_1_mmq.argtypes = [p, i64, i64, ci, ci, p]
        L.jqo_parse_q8_1.argtypes = [p, i64, p, p, p]
        L.jqo_block_sums.argtypes = [p, p, i64, i64, i64, ci, p]
        L.jqo_mul_mat_ref.argtypes = [p, p, i64, i64, i64, ci, p]
        L.jqo_dequantize_q8_1.argtypes = [p, i64, i64, ci, p]
        L.jqo_mul_mat_deq_f64.argtypes = [p, p, i64, i64, i64, ci, p]
        L.jqo_linear_cpu_baseline.argtypes = [p, p, p, i64, i64, i64, ci, p]
        L.jqo_rms_norm.argtypes = [p, p, p, p, i64, i64, ctypes.c_float]
        L.jqo_rms_norm.restype = None
        L.jqo_swiglu.argtypes = [p, p, p, i64]
        L.jqo_swiglu.restype = None
        L.jqo_num_threads.restype = ci
        L.jqo_set_num_threads.argtypes = [ci]
        L.jqo_set_num_threads.restype = None
        L.jqo_f32_to_f16.argtypes = [ctypes.c_float]
        L.jqo_f32_to_f16.restype = ctypes.c_uint16
        L.jqo_f16_to_f32.argtypes = [ctypes.c_uint16]
        L.jqo_f16_to_f32.restype = ctypes.c_float
        for name in (
            "jqo_quantize_q4_0 jqo_dequantize_q4_0 jqo_quantize_q8_1_mmq jqo_parse_q8_1 "
            "jqo_block_sums jqo_mul_mat_ref jqo_dequantize_q8_1 jqo_mul_mat_deq_f64 "
            "jqo_linear_cpu_baseline"
        ).split():
            getattr(L, name).restype = None
        _lib = L
    return _lib


def _ptr(a: np.ndarray) -> ctypes.c_void_p:
    assert a.flags["C_CONTIGUOUS"]
    return ctypes.c_void_p(a.ctypes.data)


def num_threads() -> int:
    return int(lib().jqo_num_threads())


def use_all_host_threads() -> int:
    """Let the OpenMP loops use every core this process may run on; returns the count."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().jqo_set_num_threads(n)
    return num_threads()


# ----------------------------------------------------------------------------- C wrappers
def quantize_q4_0(w: np.ndarray) -> np.ndarray:
    """fp32 ``[N, K]`` -> uint8 ``[N, K/32*18]`` (18-byte blocks, mm_q4_0_q8_1.cu:35-38)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    assert k % 32 == 0
    out = np.empty((n, k // 32 * Q4_BYTES), dtype=np.uint8)
    lib().jqo_quantize_q4_0(_ptr(w), n, k, _ptr(out))
    return out


def dequantize_q4_0(wq: np.ndarray, k: int) -> np.ndarray:
    wq = np.ascontiguousarray(wq, dtype=np.uint8).reshape(-1, k // 32 * Q4_BYTES)
    out = np.empty((wq.shape[0], k), dtype=np.float32)
    lib().jqo_dequantize_q4_0(_ptr(wq), wq.shape[0], k, _ptr(out))
    return out


def quantize_q8_1(x: np.ndarray, order: int = ORDER_COL_KSUPER, s_mode: int = S_SUM_X) -> np.ndarray:
    """fp32 ``[M, K]`` (K fastest) -> raw ``block_q8_1_mmq`` bytes, ``M*ceil(K/128)*144``."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    assert k % 32 == 0
    out = np.zeros(m * ((k + 127) // 128) * Q8_BYTES, dtype=np.uint8)
    lib().jqo_quantize_q8_1_mmq(_ptr(x), k, m, order, s_mode, _ptr(out))
    return out


def parse_q8_1(raw: np.ndarray, n_blocks: int):
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    qs = np.empty((n_blocks, 128), dtype=np.int8)
    d = np.empty((n_blocks, 4), dtype=np.float32)
    s = np.empty((n_blocks, 4), dtype=np.float32)
    lib().jqo_parse_q8_1(_ptr(raw), n_blocks, _ptr(qs), _ptr(d), _ptr(s))
    return qs, d, s


def block_sums(wq, xq, k, n, m, order=ORDER_COL_KSUPER) -> np.ndarray:
    """int32 ``[M, N, K/32]`` per-block integer dot products."""
    wq = np.ascontiguousarray(wq, dtype=np.uint8)
    xq = np.ascontiguousarray(xq, dtype=np.uint8)
    out = np.empty((m, n, k // 32), dtype=np.int32)
    lib().jqo_block_sums(_ptr(wq), _ptr(xq), k, n, m, order, _ptr(out))
    return out


def mul_mat_ref(wq, xq, k, n, m, order=ORDER_COL_KSUPER) -> np.ndarray:
    """Reference formula and accumulation order; fp32 ``[M, N]``."""
    wq = np.ascontiguousarray(wq, dtype=np.uint8)
    xq = np.ascontiguousarray(xq, dtype=np.uint8)
    out = np.empty((m, n), dtype=np.float32)
    lib().jqo_mul_mat_ref(_ptr(wq), _ptr(xq), k, n, m, order, _ptr(out))
    return out


def dequantize_q8_1(xq, k, m, order=ORDER_COL_KSUPER) -> np.ndarray:
    xq = np.ascontiguousarray(xq, dtype=np.uint8)
    out = np.empty((m, k), dtype=np.float32)
    lib().jqo_dequantize_q8_1(_ptr(xq), k, m, order, _ptr(out))
    return out


def mul_mat_deq_f64(wq, xq, k, n, m, order=ORDER_COL_KSUPER) -> np.ndarray:
    """Dequantise both operands, float64 accumulation; the 1e-3 accuracy yardstick."""
    wq = np.ascontiguousarray(wq, dtype=np.uint8)
    xq = np.ascontiguousarray(xq, dtype=np.uint8)
    out = np.empty((m, n), dtype=np.float32)
    lib().jqo_mul_mat_deq_f64(_ptr(wq), _ptr(xq), k, n, m, order, _ptr(out))
    return out


def linear_cpu_baseline(wq, x, k, n, m, s_mode=S_D_SUM_Q, y=None, ws=None) -> np.ndarray:
    """The timed CPU path: quantize X, dequantise W and X to fp32, fp32 matmul, all threads."""
    wq = np.ascontiguousarray(wq, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32)
    if y is None:
        y = np.empty((m, n), dtype=np.float32)
    if ws is None:
        ws = np.empty(m * (k // 128) * Q8_BYTES, dtype=np.uint8)
    lib().jqo_linear_cpu_baseline(_ptr(wq), _ptr(x), _ptr(ws), k, n, m, s_mode, _ptr(y))
    return y


def rms_norm(x: np.ndarray, weight: np.ndarray, epsilon: float, residual: np.ndarray = None):
    """RMSNorm of ``x`` ``[T, H]`` in the reference's operation order; with ``residual`` the fused-add form.
    Returns ``(normed, new_residual_or_None)``."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    weight = np.ascontiguousarray(weight, dtype=np.float32)
    t, h = x.shape
    res = None if residual is None else np.array(residual, dtype=np.float32, order="C", copy=True)
    out = np.empty_like(x)
    lib().jqo_rms_norm(_ptr(x), None if res is None else _ptr(res), _ptr(weight), _ptr(out), h, t, float(epsilon))
    return out, res


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    gate = np.ascontiguousarray(gate, dtype=np.float32)
    up = np.ascontiguousarray(up, dtype=np.float32)
    out = np.empty_like(gate)
    lib().jqo_swiglu(_ptr(gate), _ptr(up), _ptr(out), gate.size)
    return out


# ----------------------------------------------------------------------------- NumPy mirror
def np_quantize_q4_0(w: np.ndarray) -> np.ndarray:
    """Vectorised Q4_0 quantizer (same rule as ``jqo_quantize_q4_0``)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    blk = w.reshape(n, k // 32, 32)
    idx = np.argmax(np.abs(blk), axis=-1)  # first index of the largest magnitude
    mx = np.take_along_axis(blk, idx[..., None], axis=-1)[..., 0]
    d = (mx / np.float32(-8.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    q = np.minimum(15, ((blk * inv[..., None]).astype(np.float32) + np.float32(8.5)).astype(np.int8))
    q = q.astype(np.uint8)
    out = np.empty((n, k // 32, Q4_BYTES), dtype=np.uint8)
    out[..., 0:2] = d.astype(np.float16).view(np.uint8).reshape(n, k // 32, 2)
    out[..., 2:] = q[..., :16] | (q[..., 16:] << 4)
    return out.reshape(n, k // 32 * Q4_BYTES)


def np_unpack_q4_0(wq: np.ndarray, k: int):
    """-> (d fp32 ``[N, K/32]``, q uint8 ``[N, K/32, 32]`` in value order, 0..15)."""
    b = np.ascontiguousarray(wq, dtype=np.uint8).reshape(-1, k // 32, Q4_BYTES)
    d = b[..., 0:2].copy().view(np.float16)[..., 0].astype(np.float32)
    q = np.concatenate([b[..., 2:] & 0x0F, b[..., 2:] >> 4], axis=-1)
    return d, q


def np_quantize_q8_1(x: np.ndarray, order: int = ORDER_COL_KSUPER, s_mode: int = S_SUM_X) -> np.ndarray:
    """Vectorised activation quantizer following quantize_q8_1_kernel (src/cuda/q8_1.cu:20-104)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    assert k % 128 == 0
    g = x.reshape(m, k // 128, 4, 8, 4)  # [.., sub-block, thread, 4 floats per thread]
    amax = np.max(np.abs(g), axis=(-1, -2))
    t = ((g[..., 0] + g[..., 1]) + g[..., 2]) + g[..., 3]  # per-thread sum, q8_1.cu:63
    ssum = ((t[..., 0] + t[..., 4]) + (t[..., 2] + t[..., 6])) + (
        (t[..., 1] + t[..., 5]) + (t[..., 3] + t[..., 7])
    )  # xor butterfly 4,2,1 as seen by lane 0, q8_1.cu:65-68
    with np.errstate(divide="ignore"):
        d_inv = np.where(amax > 0, np.float32(127.0) / amax, np.float32(0.0)).astype(np.float32)
        d = np.where(amax > 0, np.float32(1.0) / d_inv, np.float32(0.0)).astype(np.float32)
    v = (g.reshape(m, k // 128, 4, 32) * d_inv[..., None]).astype(np.float32)
    q = (np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))).astype(np.int8)  # roundf: half away
    dh = d.astype(np.float16)
    if s_mode == S_SUM_X:
        sh = ssum.astype(np.float16)
    else:
        sh = (dh.astype(np.float32) * q.sum(axis=-1, dtype=np.int32).astype(np.float32)).astype(
            np.float16
        )
    blocks = np.zeros((m, k // 128, Q8_BYTES), dtype=np.uint8)
    ds = np.stack([dh, sh], axis=-1)  # [m, ks, 4, 2] halves
    blocks[..., :16] = ds.reshape(m, k // 128, 8).view(np.uint8).reshape(m, k // 128, 16)
    blocks[..., 16:] = q.reshape(m, k // 128, 128).view(np.uint8)
    if order == ORDER_KSUPER_COL:
        blocks = blocks.transpose(1, 0, 2)
    return np.ascontiguousarray(blocks).reshape(-1)


def np_unpack_q8_1(xq: np.ndarray, k: int, m: int, order: int = ORDER_COL_KSUPER):
    """-> (d ``[M, K/32]`` fp32, s ``[M, K/32]`` fp32, q ``[M, K/32, 32]`` int8)."""
    b = np.ascontiguousarray(xq, dtype=np.uint8)
    if order == ORDER_KSUPER_COL:
        b = b.reshape(k // 128, m, Q8_BYTES).transpose(1, 0, 2)
    else:
        b = b.reshape(m, k // 128, Q8_BYTES)
    b = np.ascontiguousarray(b)
    ds = b[..., :16].copy().view(np.float16).reshape(m, k // 128, 4, 2).astype(np.float32)
    q = b[..., 16:].copy().view(np.int8).reshape(m, k // 32, 32)
    return ds[..., 0].reshape(m, k // 32), ds[..., 1].reshape(m, k // 32), q


def np_block_sums(wq, xq, k, n, m, order=ORDER_COL_KSUPER) -> np.ndarray:
    _, q4 = np_unpack_q4_0(wq, k)
    _, _, q8 = np_unpack_q8_1(xq, k, m, order)
    return np.einsum("nbj,mbj->mnb", q4.astype(np.int32), q8.astype(np.int32))


def np_mul_mat_deq(wq, xq, k, n, m, order=ORDER_COL_KSUPER) -> np.ndarray:
    """float64 dequantise-then-matmul."""
    d4, q4 = np_unpack_q4_0(wq, k)
    d8, _, q8 = np_unpack_q8_1(xq, k, m, order)
    w = ((q4.astype(np.float64) - 8.0) * d4[..., None]).reshape(n, k)
    x = (q8.astype(np.float64) * d8[..., None]).reshape(m, k)
    return (x @ w.T).astype(np.float32)


def err_max_rel(y: np.ndarray, ref: np.ndarray) -> float:
    """max|y - ref| / max|ref|: the error metric every fp32 tolerance here is stated in."""
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.max(np.abs(np.asarray(y, dtype=np.float64) - ref)) / max(np.max(np.abs(ref)), 1e-30))
