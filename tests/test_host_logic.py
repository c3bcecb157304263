"""CPU tests of the host-side logic: synthetic workloads, shard arithmetic, and the N-sharded
linear's plumbing on two gloo ranks (the compute step is injected, so no GPU is needed)."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_synth_is_deterministic_and_shaped():
    from jjjetson_ops_b200 import synth

    w1, x1, lin = synth.make_linear_case(1, rows=64)
    w2, x2, _ = synth.make_linear_case(1, rows=64)
    assert lin.K == 4096 and lin.N == 4096 and w1.shape == (64, 4096) and x1.shape == (1, 4096)
    assert np.array_equal(w1, w2) and np.array_equal(x1, x2)
    assert abs(float(w1.std()) - 0.02) < 2e-3 and abs(float(x1.std()) - 1.0) < 0.1
    # rows= only truncates: the activations do not depend on it
    w3, x3, _ = synth.make_linear_case(1, rows=8)
    assert np.array_equal(w3, w1[:8]) and np.array_equal(x3, x1)


def test_synth_outliers_and_batch_prefixes():
    from jjjetson_ops_b200 import synth

    _, x8, lin = synth.make_linear_case(2, M=8, rows=32)
    _, x2, _ = synth.make_linear_case(2, M=2, rows=32)
    assert np.array_equal(x8[:2], x2) and lin.N == 11008
    big = np.abs(x8).mean(axis=0) > 8.0
    assert 30 <= int(big.sum()) <= 41  # 41 channels scaled by 20, the same ones in every row


def test_algorithmic_bytes_of_the_five_configurations():
    from jjjetson_ops_b200 import synth

    assert synth.algorithmic_bytes(4096, 4096, 1, fused_quantize=False) == 9458176
    assert synth.algorithmic_bytes(4096, 11008, 1, fused_quantize=False) == 25411072
    assert synth.algorithmic_bytes(4096, 4096, 512, fused_quantize=False) == 20185088
    assert synth.algorithmic_bytes(8192, 28672, 1, fused_quantize=False) == 132244480
    assert synth.ops(4096, 4096, 512) == 17179869184


@pytest.mark.parametrize("N,world", [(28672, 8), (28672, 4), (11008, 8), (4096, 2), (100, 3), (31, 4)])
def test_shard_rows_partition(N, world):
    from jjjetson_ops_b200 import synth

    spans = [synth.shard_rows(N, world, r) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == N
    for (b0, e0), (b1, e1) in zip(spans, spans[1:]):
        assert e0 == b1 and b0 <= e0
    assert all(b % 32 == 0 for b, _ in spans)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _sharded_worker(rank: int, world: int, port: int, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    from jjjetson_ops_b200 import sharded
    from oracle import jq_oracle as O

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        K, N, M = 256, 160, 3
        rng = np.random.default_rng(21)
        w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        x = rng.standard_normal((M, K), dtype=np.float32)
        wq = O.quantize_q4_0(w)

        def cpu_compute(w_shard, x_t, n_rows):  # stand-in for the CUDA linear
            y = O.linear_cpu_baseline(w_shard.numpy(), x_t.numpy(), K, n_rows, M)
            return torch.from_numpy(y)

        lin = sharded.ShardedLinearQ4_0(torch.from_numpy(wq), N, K, compute=cpu_compute)
        b, e = lin.row_span
        assert lin.w_shard.shape[0] == e - b
        y = lin(torch.from_numpy(x))
        full = O.linear_cpu_baseline(wq, x, K, N, M)
        q.put((rank, bool(np.array_equal(y.numpy(), full)), tuple(y.shape), (b, e)))
    except Exception as ex:  # report instead of leaving the parent to time out
        q.put((rank, False, repr(ex), (-1, -1)))
        raise
    finally:
        dist.destroy_process_group()


def test_sharded_linear_gathers_on_two_gloo_ranks():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_sharded_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    assert all(r[1] for r in results) and all(r[2] == (3, 160) for r in results)
    assert sorted(r[3] for r in results) == [(0, 64), (64, 160)]  # 5 units of 32 rows: 2 + 3


@pytest.mark.parametrize("K,n_total,world", [(4096, 22016, 2), (4096, 88064, 8), (8192, 28672, 4), (4096, 4096, 8), (11008, 11008, 2)])
def test_segments_of_samples_every_band(K, n_total, world):
    """The activations a tagged sharded layer reads from the previous layer's gathered output: runs of 8 columns spread
    evenly over the row, as bench.py asks for them.  The mapping must stay inside the row, keep 16-byte alignment of the
    8-byte words in fours (offsets that are multiples of 4, so that a lane's eight words can be read as two 32-byte loads), take exactly K columns and touch every rank's band."""
    import torch

    from jjjetson_ops_b200.sharded import segments_of

    seg_len = 8
    stride = (n_total // (K // seg_len)) // 4 * 4
    assert stride >= seg_len and stride % 4 == 0
    assert (K // seg_len - 1) * stride + seg_len <= n_total
    y = torch.arange(2 * n_total, dtype=torch.float32).reshape(2, n_total)
    x = segments_of(y, K, seg_len, stride)
    assert x.shape == (2, K)
    cols = x[0].to(torch.int64)
    k = torch.arange(K)
    assert torch.equal(cols, (k // seg_len) * stride + k % seg_len)
    assert torch.equal(x[1], x[0] + n_total)
    band = n_total // world
    assert set((cols // band).tolist()) == set(range(world))
