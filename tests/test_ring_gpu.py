"""GPU test of the sequence-sharded ring (CUDA backend, NCCL): needs at least two GPUs, skipped otherwise.
Each rank holds a shard of a causal problem; the ring result is compared with the single-GPU kernels run on
the whole problem (rank 0) and with the CPU oracle on a subset of rows."""
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, layout, T, ret, transport="auto"):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import hyperkernels_b200 as hk
        from hyperkernels_b200.ring import RingAttention, segments_of

        g = torch.Generator(device="cuda").manual_seed(5)  # same seed on every rank: same global tensors
        B, H = 1, 4
        Q, K, V, dO = (torch.randn((B, H, T, 64), generator=g, device="cuda") for _ in range(4))
        K[:, :, ::64] *= 2.0
        segs = segments_of(rank, world, T, layout)
        shard = lambda x: torch.cat([x[:, :, s:s + n] for (s, n) in segs], dim=2).contiguous()
        ring = RingAttention(T, 0.125, True, layout=layout, transport=transport)
        assert (ring.native is not None) == (transport != "torch")
        O_l, L_l = ring.forward(shard(Q), shard(K), shard(V))
        dQ_l, dK_l, dV_l = ring.backward(shard(Q), shard(K), shard(V), O_l, L_l, shard(dO))
        torch.cuda.synchronize()
        assert hk.last_device_status() == 0
        O, LSE = hk.attention_forward(Q, K, V, 0.125, True)
        dQ, dK, dV, _ = hk.attention_backward(Q, K, V, O, dO, LSE, 0.125, True)
        errs = []
        for loc, full in ((O_l, O), (L_l, LSE), (dQ_l, dQ), (dK_l, dK), (dV_l, dV)):
            ref = shard(full)
            errs.append(float((loc - ref).abs().max()))
            errs.append(float((loc - ref).norm() / ref.norm()))
        ret.put((rank, errs))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("transport", ["native", "torch"])
@pytest.mark.parametrize("layout", ["contiguous", "zigzag"])
def test_ring_matches_single_gpu(layout, transport):
    """transport: the hop through libhk_ring.so (one native call per hop) or through torch.distributed."""
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = 29800 + (7 if layout == "zigzag" else 0) + (20 if transport == "torch" else 0)
    procs = [ctx.Process(target=_worker, args=(r, world, port, layout, 1024, ret, transport)) for r in range(world)]
    for p in procs:
        p.start()
    results = [ret.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, errs in results:
        # two TF32 evaluations of the same function with different tilings/merge order: both within the parity
        # gate of the oracle, so within twice that of each other
        for i in range(0, len(errs), 2):
            assert errs[i] <= 1e-2 and errs[i + 1] <= 2e-3, (rank, errs)


def _timeout_worker(rank, world, port, ret):
    """Rank 1 never posts its side of the hop; rank 0's host-side wait gives up after its limit, takes its
    communicator down (ncclCommAbort) and raises RingError.  Nobody dies and no rank leaves with work in flight."""
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from hyperkernels_b200.ring import NativeTransport, RingError

        tr = NativeTransport(None, rank, world)
        a = torch.ones(1 << 20, device="cuda")
        b = torch.zeros(1 << 20, device="cuda")
        comm = torch.cuda.Stream()
        # one good hop first: both sides post
        slot = tr.exchange(a, b, torch.cuda.current_stream(), comm)
        tr.finish(slot, torch.cuda.current_stream(), 30.0)
        torch.cuda.synchronize()
        assert float(b.sum()) == float(1 << 20)
        outcome = "idle"
        if rank == 0:
            slot = tr.exchange(a, b, torch.cuda.current_stream(), comm)
            try:
                tr.finish(slot, torch.cuda.current_stream(), 1.5)
                outcome = "completed"
            except RingError as e:
                outcome = "RingError: " + str(e)
            torch.cuda.synchronize()  # the aborted hop has left the stream: the context is usable
            assert float((a + 1).sum()) == float(2 << 20)
        ret.put((rank, outcome))
        ret.close()
        ret.join_thread()
        dist.barrier()  # rank 1 waits here, on the process group, while rank 0 times out
        tr.close(abort=True)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_native_hop_that_never_completes_raises_ring_error():
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_timeout_worker, args=(r, world, 29871, ret)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(ret.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results[0].startswith("RingError") and "did not complete in time" in results[0], results
    assert results[1] == "idle"


def _graph_worker(rank, world, port, ret):
    """The captured ring step (GraphedRingStep) gives what the call-by-call ring gives, also after the inputs were
    refilled in place; every rank replays the same number of times."""
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import hyperkernels_b200 as hk
        from hyperkernels_b200.ring import GraphedRingStep, RingAttention

        T, B, H = 2048, 1, 4
        g = torch.Generator(device="cuda").manual_seed(100 + rank)
        Q, K, V, dO = (torch.randn((B, H, T // world, 64), generator=g, device="cuda") for _ in range(4))
        ring = RingAttention(T, 0.125, True, layout="zigzag")
        gs = GraphedRingStep(ring, Q, K, V, dO)
        worst = 0.0
        for it in range(3):
            if it:
                for t in (Q, K, V, dO):
                    t.copy_(torch.randn(t.shape, generator=g, device="cuda"))
            gs.replay()
            torch.cuda.synchronize()
            O, LSE = ring.forward(Q, K, V)
            dQ, dK, dV = ring.backward(Q, K, V, O, LSE, dO)
            torch.cuda.synchronize()
            assert hk.last_device_status() == 0
            assert torch.equal(gs.O, O) and torch.equal(gs.LSE, LSE), it
            assert torch.equal(gs.dK, dK) and torch.equal(gs.dV, dV), it
            worst = max(worst, float((gs.dQ - dQ).abs().max()))
        ret.put((rank, worst))
        ret.close()
        ret.join_thread()
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_captured_ring_step_equals_the_call_by_call_ring():
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_graph_worker, args=(r, world, 29891, ret)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(ret.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(w <= 1e-4 for w in results.values()), results
