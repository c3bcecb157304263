"""GPU test of ``jq_linear_q4_0_device_noalloc``, the entry point for callers that cannot allocate.

Some hosts of this library may not call ``cudaMalloc`` once they are running: a serving process that
gave the whole device to its own arena at start-up, or a decode loop that cannot take the
device-wide synchronisation an allocation implies.  For them the library carries its Q8_1 scratch
as a fixed array in its own image.  The test calls the new entry point through the C ABI twice in
a row, with different shapes so that the second call finds the first call's bytes in the shared
scratch, and compares each result with what the ordinary entry point (caller-owned workspace)
returns for the same inputs.  This file is named to be collected last.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _inputs(rng, K, N, M):
    w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    x = rng.standard_normal((M, K), dtype=np.float32)
    return w, x


def test_noalloc_entry_matches_workspace_entry_twice_in_a_row(native_lib, oracle, cuda_device):
    import torch

    c = native_lib
    rng = np.random.default_rng(2024)
    # first a batch that goes through the separate quantize kernel and leaves 8 * 32 blocks behind,
    # then a single row whose multiply quantizes in its own prologue, then a prefill-sized batch
    for K, N, M in ((4096, 1536, 8), (4096, 1024, 1), (2048, 640, 96)):
        w, x = _inputs(rng, K, N, M)
        d_w = c.quantize_q4_0(torch.from_numpy(w).to(cuda_device))
        d_x = torch.from_numpy(x).to(cuda_device)
        got = c.linear_q4_0_noalloc(d_w, d_x, N, c.S_D_SUM_Q)
        ws = torch.zeros(c.q8_1_bytes(K, M), dtype=torch.uint8, device=cuda_device)
        want = c.linear_q4_0(d_w, d_x, N, c.S_D_SUM_Q, ws=ws)
        torch.cuda.synchronize()
        got, want = got.cpu().numpy(), want.cpu().numpy()
        assert np.isfinite(got).all()
        assert oracle.err_max_rel(got, want) <= 1e-5  # the tolerance of the other multiply tests
        assert np.array_equal(got, want)  # same kernels on the same inputs: in fact the same bits
        # and against the CPU oracle, like every other parity test
        xq = oracle.quantize_q8_1(x, oracle.ORDER_COL_KSUPER, oracle.S_D_SUM_Q)
        # (64 columns and more take the fp16-operand GEMM, which the other tests hold to 1e-3 against the formula)
        assert oracle.err_max_rel(got, oracle.mul_mat_ref(d_w.cpu().numpy(), xq, K, N, M)) <= (1e-3 if M >= 64 else 1e-5)
    assert c.device_fault() == 0


def test_noalloc_entry_rejects_oversized_requests(native_lib, cuda_device):
    import torch

    c = native_lib
    K, M = 8192, 1024  # 1024 * 64 * 144 bytes = 9.4 MB of Q8_1 blocks > the 4 MiB array
    assert c.q8_1_bytes(K, M) > c.NOALLOC_WS_BYTES
    d_w = torch.zeros(c.q4_0_bytes(32, K), dtype=torch.uint8, device=cuda_device)
    d_x = torch.zeros((M, K), dtype=torch.float32, device=cuda_device)
    with pytest.raises(c.JqError) as ei:
        c.linear_q4_0_noalloc(d_w, d_x, 32, c.S_D_SUM_Q)
    assert ei.value.status == c.ERR_TOO_LARGE
    assert "4194304" in str(ei.value)
