"""Back-to-back calls with nothing between them, static weights on: every kernel of the path is launched with
programmatic dependent launch and starts (set-up, weight prefetch) while the call ahead of it is still running, and
all calls share one Q8_1 workspace.  Whatever a call reads or writes after its ``griddepcontrol.wait`` must be
ordered after the previous call; whatever it does before must not depend on it.  Each result of the queued sequence
is compared bit for bit with the same call made alone (device idle before and after).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SHAPES = [  # K, N
    (4096, 4096), (2048, 1000), (4096, 11008), (1024, 257), (8192, 2048), (11008, 512), (256, 64), (6144, 96), (4096, 300),
]
BATCHES = [1, 2, 3, 4, 8, 16, 33, 64, 128, 200]


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_queued_calls_equal_isolated_calls(native_lib, cuda_device, seed):
    import torch

    c = native_lib
    rng = np.random.default_rng(seed)
    gen = torch.Generator(device=cuda_device)
    gen.manual_seed(seed)
    weights = {}
    for K, N in SHAPES:
        w = torch.randint(0, 256, (N, K // 32 * 18), dtype=torch.uint8, device=cuda_device, generator=gen)
        blk = w.view(N, K // 32, 18)
        blk[:, :, 0] = torch.randint(0, 256, (N, K // 32), dtype=torch.uint8, device=cuda_device, generator=gen)
        blk[:, :, 1] = 0x1C  # scales between 2^-8 and 2^-7: finite
        weights[(K, N)] = w
    calls = []
    for _ in range(40):
        K, N = SHAPES[int(rng.integers(len(SHAPES)))]
        M = BATCHES[int(rng.integers(len(BATCHES)))]
        x = torch.randn((M, K), dtype=torch.float32, device=cuda_device, generator=gen)
        calls.append((K, N, M, x))
    ws = torch.zeros(max(c.q8_1_bytes(K, M) for K, _, M, _ in calls) + 16, dtype=torch.uint8, device=cuda_device)
    c.set_option(c.OPT_STATIC_WEIGHTS, 1)
    try:
        # alone: the device is idle before and after every call
        alone = []
        for K, N, M, x in calls:
            torch.cuda.synchronize()
            y = torch.empty((M, N), dtype=torch.float32, device=cuda_device)
            c.linear_q4_0(weights[(K, N)], x, N, c.S_D_SUM_Q, ws=ws, out=y)
            torch.cuda.synchronize()
            alone.append(y)
        # queued: nothing between the calls, one workspace for all of them
        for rep in range(3):
            outs = [torch.empty((M, N), dtype=torch.float32, device=cuda_device) for _, N, M, _ in calls]
            torch.cuda.synchronize()
            for (K, N, M, x), y in zip(calls, outs):
                c.linear_q4_0(weights[(K, N)], x, N, c.S_D_SUM_Q, ws=ws, out=y)
            torch.cuda.synchronize()
            for i, (y, ref) in enumerate(zip(outs, alone)):
                assert torch.equal(y, ref), (rep, i, calls[i][:3])
        # the same sequence replayed from one CUDA graph
        stream = torch.cuda.Stream()
        outs = [torch.empty((M, N), dtype=torch.float32, device=cuda_device) for _, N, M, _ in calls]
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            for (K, N, M, x), y in zip(calls, outs):  # warm-up outside the capture
                c.linear_q4_0(weights[(K, N)], x, N, c.S_D_SUM_Q, ws=ws, out=y)
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            for (K, N, M, x), y in zip(calls, outs):
                c.linear_q4_0(weights[(K, N)], x, N, c.S_D_SUM_Q, ws=ws, out=y)
        for rep in range(3):
            for y in outs:
                y.zero_()
            torch.cuda.synchronize()
            with torch.cuda.stream(stream):
                graph.replay()
            stream.synchronize()
            for i, (y, ref) in enumerate(zip(outs, alone)):
                assert torch.equal(y, ref), ("graph", rep, i, calls[i][:3])
        assert c.device_fault() == 0
    finally:
        c.set_option(c.OPT_STATIC_WEIGHTS, 0)
