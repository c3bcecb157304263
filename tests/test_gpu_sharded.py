"""GPU tests of the fused multiply + all-gather (``jq_linear_q4_0_allgather_device``).

On one GPU the kernel runs with world = 1 (its band staging, peer-store loop, completion counter
and flag logic all execute, with itself as the only peer).  With two or more GPUs a two-rank run
(one process per GPU, NCCL only for the rendezvous of the IPC handles) checks real peer stores.
One test lets a bounded wait run out on purpose: a wait for an all-gather that nobody performs, with the poll
limit set to a few thousand, must give up, report through the fault word and leave the device usable (the
kernel returns by itself; nothing hangs or faults).
"""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("K,N,M", [(4096, 11008, 1), (4096, 1000, 2), (8192, 4096, 1), (2048, 37, 1),
                                   (1024, 256, 64), (2048, 200, 130), (512, 96, 5), (4096, 4096, 512)])
def test_fused_allgather_single_rank(native_lib, oracle, cuda_device, K, N, M):
    import torch

    from jjjetson_ops_b200.sharded import PeerBands

    c = native_lib
    rng = np.random.default_rng(K + N + M)
    w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    wq = oracle.quantize_q4_0(w)
    d_w = torch.from_numpy(wq).to(cuda_device)
    ws = torch.zeros(c.q8_1_bytes(K, M), dtype=torch.uint8, device=cuda_device)
    bands = PeerBands(M, N, cuda_device)
    try:
        for step in range(3):  # alternates the two output buffers and advances the epoch
            x = rng.standard_normal((M, K), dtype=np.float32)
            bands.linear(d_w, torch.from_numpy(x).to(cuda_device), ws, 0, N)
            bands.wait()
            y = bands.latest().cpu().numpy()
            assert int(bands.epoch.item()) == step + 1
            xq = oracle.quantize_q8_1(x, oracle.ORDER_COL_KSUPER, oracle.S_D_SUM_Q)
            assert np.array_equal(ws.cpu().numpy(), xq)
            assert oracle.err_max_rel(y, oracle.mul_mat_ref(wq, xq, K, N, M)) <= 1e-5
            assert int(bands.counter.item()) == 0  # the completion counter re-arms itself
        assert c.device_fault() == 0
    finally:
        bands.close()


def test_fused_allgather_refuses_other_shapes(native_lib, cuda_device):
    import torch

    from jjjetson_ops_b200.sharded import PeerBands

    c = native_lib
    bands = PeerBands(4, 64, cuda_device)
    try:
        # K = 384 is not a multiple of 256: neither the streaming kernel nor the tensor-core GEMM takes it
        d_w = torch.zeros(c.q4_0_bytes(64, 384), dtype=torch.uint8, device=cuda_device)
        x = torch.zeros((4, 384), dtype=torch.float32, device=cuda_device)
        ws = torch.zeros(c.q8_1_bytes(384, 4), dtype=torch.uint8, device=cuda_device)
        with pytest.raises(c.JqError) as ei:
            bands.linear(d_w, x, ws, 0, 64)
        assert ei.value.status == c.ERR_UNSUPPORTED  # gather with NCCL instead
    finally:
        bands.close()


def test_bounded_wait_gives_up_and_reports(native_lib, oracle, cuda_device):
    """A wait whose bands never arrive: flag word zero, epoch 1, 4096 polls.  The kernel must return, the fault
    word must read 2 (and 0 after it was cleared), and an ordinary launch afterwards must be right."""
    import torch

    c = native_lib
    assert c.device_fault() == 0
    flags = torch.zeros(64, dtype=torch.int32, device=cuda_device)
    epoch = torch.ones(1, dtype=torch.int32, device=cuda_device)  # "one all-gather has been started"
    c.set_option(c.OPT_WAIT_POLL_LIMIT, 4096)
    try:
        c.allgather_wait(cuda_device, flags.data_ptr(), 1, epoch)
        torch.cuda.synchronize()
        v = c.ctypes.c_int(0)
        rc = c.lib().jq_device_fault(1, c.ctypes.byref(v))
        assert rc == c.ERR_TIMEOUT and v.value == 2, (rc, v.value, c.last_error())
    finally:
        c.set_option(c.OPT_WAIT_POLL_LIMIT, 0)
    assert c.device_fault() == 0  # cleared by the read above
    # the context is intact: a normal multiply gives the right answer
    K, N, M = 2048, 320, 1
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    x = rng.standard_normal((M, K), dtype=np.float32)
    wq = oracle.quantize_q4_0(w)
    y = c.linear_q4_0(torch.from_numpy(wq).to(cuda_device), torch.from_numpy(x).to(cuda_device), N).cpu().numpy()
    xq = oracle.quantize_q8_1(x, oracle.ORDER_COL_KSUPER, oracle.S_D_SUM_Q)
    assert oracle.err_max_rel(y, oracle.mul_mat_ref(wq, xq, K, N, M)) <= 1e-5
    assert c.device_fault() == 0


@pytest.mark.parametrize("K,N,M,K2,seg", [(4096, 11008, 1, 4096, None), (2048, 4096, 2, 1024, 256), (4096, 2080, 1, 2048, 512),
                                          (8192, 8192, 1, 8192, None), (4096, 11008, 1, 4096, -8), (2048, 4098, 2, 1024, 256)])
def test_tagged_allgather_single_rank(native_lib, oracle, cuda_device, K, N, M, K2, seg):
    """The decode form on one GPU (world = 1: ticket, tagged stores, polling loads and the reader all run,
    with itself as the only peer).  Layer 1 takes plain activations; layer 2 takes its activations from
    layer 1's tagged words (first K2 words, or runs of ``seg`` words spread over the row), three passes, so
    that both buffers of each pair and increasing tags are used."""
    import torch

    from jjjetson_ops_b200.sharded import TaggedBands, segments_of

    c = native_lib
    rng = np.random.default_rng(K + N + M)
    N2 = 512 + 32
    wq1 = oracle.quantize_q4_0((rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)).astype(np.float32))
    wq2 = oracle.quantize_q4_0((rng.standard_normal((N2, K2), dtype=np.float32) * np.float32(0.02)).astype(np.float32))
    d_w1, d_w2 = torch.from_numpy(wq1).to(cuda_device), torch.from_numpy(wq2).to(cuda_device)
    # a lane's eight words are read as two 32-byte loads when every run of words starts on a 32-byte boundary (the run
    # distance and the row length multiples of four words), else as four 16-byte loads: seg = -8 gives runs of eight
    # words every 18 words, and a row of 4098 words puts the second row of a batch of two off the boundary
    seg_len = K2 if seg is None else abs(seg)
    seg_stride = 0 if seg is None else (18 if seg < 0 else (N - seg_len) // (K2 // seg_len - 1) // 32 * 32)
    a = TaggedBands(M, N, cuda_device)
    b = TaggedBands(M, N2, cuda_device, share_with=a)
    try:
        for step in range(3):
            x = rng.standard_normal((M, K), dtype=np.float32)
            a.linear(d_w1, K, 0, N, x=torch.from_numpy(x).to(cuda_device))
            y1 = a.read().cpu().numpy()
            xq = oracle.quantize_q8_1(x, oracle.ORDER_COL_KSUPER, oracle.S_D_SUM_Q)
            assert oracle.err_max_rel(y1, oracle.mul_mat_ref(wq1, xq, K, N, M)) <= 1e-5
            b.linear(d_w2, K2, 0, N2, source=a, seg_len=seg_len, seg_stride=seg_stride)
            y2 = b.read().cpu().numpy()
            x2 = segments_of(torch.from_numpy(y1), K2, seg_len, seg_stride).numpy()
            xq2 = oracle.quantize_q8_1(x2, oracle.ORDER_COL_KSUPER, oracle.S_D_SUM_Q)
            assert oracle.err_max_rel(y2, oracle.mul_mat_ref(wq2, xq2, K2, N2, M)) <= 1e-5
            # the same bits as the single-GPU entry on the same activations
            y2_single = c.linear_q4_0(d_w2, torch.from_numpy(x2).to(cuda_device), N2).cpu().numpy()
            assert np.array_equal(y2, y2_single)
            # a second projection fed by the same output: its input is the all-gather before the one just ahead of it
            b.linear(d_w2, K2, 0, N2, source=a, seg_len=seg_len, seg_stride=seg_stride, back=1)
            assert np.array_equal(b.read().cpu().numpy(), y2)
            # the same pair back to back: nothing orders the second layer after the first but the words
            a.linear(d_w1, K, 0, N, x=torch.from_numpy(x).to(cuda_device))
            b.linear(d_w2, K2, 0, N2, source=a, seg_len=seg_len, seg_stride=seg_stride)
            assert np.array_equal(b.read().cpu().numpy(), y2)
            assert int(a.ticket.item()) == 5 * (step + 1) << 16
        assert c.device_fault() == 0
    finally:
        b.close()
        a.close()


def test_tagged_read_gives_up_and_reports(native_lib, cuda_device):
    """Words that never arrive: the count says one all-gather was launched, the buffers are still zero.  With a
    limit of a few thousand polls the reader must return by itself and report through the fault word."""
    import torch

    from jjjetson_ops_b200.sharded import TaggedBands

    c = native_lib
    assert c.device_fault() == 0
    bands = TaggedBands(1, 64, cuda_device)
    c.set_option(c.OPT_WAIT_POLL_LIMIT, 2048)
    try:
        bands.ticket.fill_(1 << 16)
        bands.read()
        torch.cuda.synchronize()
        v = c.ctypes.c_int(0)
        rc = c.lib().jq_device_fault(1, c.ctypes.byref(v))
        assert rc == c.ERR_TIMEOUT and v.value == 2, (rc, v.value, c.last_error())
    finally:
        c.set_option(c.OPT_WAIT_POLL_LIMIT, 0)
        bands.close()
    assert c.device_fault() == 0


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _two_rank_worker(rank: int, world: int, port: int, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist

    from jjjetson_ops_b200 import capi, synth
    from jjjetson_ops_b200.sharded import PeerBands
    from oracle import jq_oracle as O

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        K, N, M = 4096, 4096 + 64, 1
        rng = np.random.default_rng(77)
        w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        wq = O.quantize_q4_0(w)
        b, e = synth.shard_rows(N, world, rank)
        d_w = torch.from_numpy(np.ascontiguousarray(wq[b:e])).to(dev)
        ws = torch.zeros(capi.q8_1_bytes(K, M), dtype=torch.uint8, device=dev)
        bands = PeerBands(M, N, dev)
        ok = True
        for step in range(4):
            x = rng.standard_normal((M, K), dtype=np.float32)  # same stream of inputs on every rank
            bands.linear(d_w, torch.from_numpy(x).to(dev), ws, b, e - b)
            bands.wait()  # every rank's band has arrived before the buffer is read
            y = bands.latest().cpu().numpy()
            xq = O.quantize_q8_1(x, O.ORDER_COL_KSUPER, O.S_D_SUM_Q)
            ok = ok and O.err_max_rel(y, O.mul_mat_ref(wq, xq, K, N, M)) <= 1e-5  # all bands, not just ours
        bands.close()
        # a prefill batch through the tensor-core GEMM's all-gather epilogue (ragged last tile on both axes)
        M2, N2 = 200, 1000 + 24
        w2 = (rng.standard_normal((N2, K), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        wq2 = O.quantize_q4_0(w2)
        b2, e2 = synth.shard_rows(N2, world, rank)
        d_w2 = torch.from_numpy(np.ascontiguousarray(wq2[b2:e2])).to(dev)
        ws2 = torch.zeros(capi.q8_1_bytes(K, M2), dtype=torch.uint8, device=dev)
        bands2 = PeerBands(M2, N2, dev)
        for step in range(3):
            x = rng.standard_normal((M2, K), dtype=np.float32)
            bands2.linear(d_w2, torch.from_numpy(x).to(dev), ws2, b2, e2 - b2)
            bands2.wait()
            y = bands2.latest().cpu().numpy()
            xq = O.quantize_q8_1(x, O.ORDER_COL_KSUPER, O.S_D_SUM_Q)
            ok = ok and O.err_max_rel(y, O.mul_mat_ref(wq2, xq, K, N2, M2)) <= 1e-5
        bands2.close()
        # the decode form: tagged words, a chain of two sharded layers, the second fed by the first one's words
        # (K3 / world words from every rank's band), with no wait between them but the words themselves
        from jjjetson_ops_b200.sharded import TaggedBands, segments_of

        K3, N3 = 2048, 1024 + 64
        w3 = (rng.standard_normal((N3, K3), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        wq3 = O.quantize_q4_0(w3)
        b3, e3 = synth.shard_rows(N3, world, rank)
        d_w3 = torch.from_numpy(np.ascontiguousarray(wq3[b3:e3])).to(dev)
        ta = TaggedBands(1, N, dev)
        tb = TaggedBands(1, N3, dev, share_with=ta)
        seg_len, seg_stride = K3 // world, synth.shard_rows(N, world, 1)[0]
        for step in range(4):
            x = rng.standard_normal((1, K), dtype=np.float32)
            d_x = torch.from_numpy(x).to(dev)
            ta.linear(d_w, K, b, e - b, x=d_x)
            y1 = ta.read().cpu().numpy()  # the first layer's gathered output, to build the expectation from
            tb.linear(d_w3, K3, b3, e3 - b3, source=ta, seg_len=seg_len, seg_stride=seg_stride)
            y3 = tb.read().cpu().numpy()
            xq = O.quantize_q8_1(x, O.ORDER_COL_KSUPER, O.S_D_SUM_Q)
            ok = ok and O.err_max_rel(y1, O.mul_mat_ref(wq, xq, K, N, 1)) <= 1e-5
            x3 = segments_of(torch.from_numpy(y1), K3, seg_len, seg_stride).numpy()
            xq3 = O.quantize_q8_1(x3, O.ORDER_COL_KSUPER, O.S_D_SUM_Q)
            ok = ok and O.err_max_rel(y3, O.mul_mat_ref(wq3, xq3, K3, N3, 1)) <= 1e-5
            # the same pair back to back: nothing orders the second layer after the first but the words
            ta.linear(d_w, K, b, e - b, x=d_x)
            tb.linear(d_w3, K3, b3, e3 - b3, source=ta, seg_len=seg_len, seg_stride=seg_stride)
            ok = ok and np.array_equal(tb.read().cpu().numpy(), y3)
        tb.close()
        ta.close()
        ok = ok and capi.device_fault() == 0
        q.put((rank, bool(ok)))
    except Exception as ex:
        q.put((rank, repr(ex)))
        raise
    finally:
        dist.destroy_process_group()


def test_fused_allgather_two_ranks(native_lib, oracle):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_two_rank_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert results == [(0, True), (1, True)], results
