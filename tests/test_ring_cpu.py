"""CPU test of the sequence-sharded ring schedule (hyperkernels_b200/ring.py) on two gloo ranks.

The schedule (who computes which (query segment, key segment) pair at which step, the chaining of
the running forward result through the key blocks, the travelling gradient accumulators, the message order) is host logic and is what is tested here;
the per-pair compute is done by a stand-in backend built on the CPU oracle, which exists only in this test.
The same schedule with the CUDA backend is checked on GPUs in tests/test_ring_gpu.py.
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))


class OracleBackend:
    """Per-pair compute on the CPU oracle (test stand-in for the CUDA kernels)."""

    def __init__(self):
        import oracle_lib as ol

        self.ol = ol

    @staticmethod
    def _np(t):
        return np.ascontiguousarray(t.detach().cpu().numpy(), dtype=np.float32)

    def prepare(self, x, out=None):
        if out is None:
            return x.contiguous()
        out.copy_(x)
        return out

    def fwd_into(self, Q, K, V, scale, causal, q_pos0, k_pos0, O_acc, LSE_acc):
        """Attention over this key block, folded into the running (O_acc, LSE_acc): what the CUDA forward does with
        HK_FLAG_CONTINUE_SOFTMAX_STATE, restated with the oracle and a float64 merge."""
        O, L = self.ol.attn_forward(self._np(Q), self._np(K), self._np(V), scale, int(causal), None, q_pos0, k_pos0)
        O_part, LSE_part = torch.from_numpy(O), torch.from_numpy(L)
        la, lp = LSE_acc.double(), LSE_part.double()
        mx = torch.maximum(la, lp)
        safe = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
        ea, ep = torch.exp(la - safe), torch.exp(lp - safe)
        tot = ea + ep
        wa = torch.where(tot > 0, ea / tot, torch.zeros_like(tot))
        wp = torch.where(tot > 0, ep / tot, torch.zeros_like(tot))
        o_old = torch.where(torch.isinf(la).unsqueeze(-1), torch.zeros_like(O_part, dtype=torch.float64), O_acc.double())
        O_acc.copy_((o_old * wa[..., None] + O_part.double() * wp[..., None]).float())
        LSE_acc.copy_(torch.where(tot > 0, safe + torch.log(tot), torch.full_like(tot, float("-inf"))).float())

    def precompute_D(self, dO, O, out=None):
        D = torch.from_numpy(self.ol.precompute_D(self._np(dO), self._np(O)))
        if out is not None:
            out.copy_(D)
            return out
        return D

    def bwd(self, Q, K, V, O, dO, LSE, D, scale, causal, q_pos0, k_pos0, dQ, dK, dV):
        _, dq, dk, dv = self.ol.attn_backward(self._np(Q), self._np(K), self._np(V), self._np(O), self._np(dO),
                                              self._np(LSE), scale, int(causal), None, q_pos0, k_pos0)
        dQ.add_(torch.from_numpy(dq))
        dK.add_(torch.from_numpy(dk))
        dV.add_(torch.from_numpy(dv))


def _gather_seq(x_local, segs_all, T):
    """Reassemble a [B,H,T,...] tensor from every rank's shard (list over ranks) given each rank's segments."""
    out = torch.empty((x_local[0].shape[0], x_local[0].shape[1], T) + tuple(x_local[0].shape[3:]))
    for r, x in enumerate(x_local):
        off = 0
        for (s, n) in segs_all[r]:
            out[:, :, s:s + n] = x[:, :, off:off + n]
            off += n
    return out


def _worker(rank, world, port, layout, causal, T, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle_lib as ol
        from hyperkernels_b200.ring import RingAttention, segments_of

        rng = np.random.default_rng(7)
        B, H = 1, 2
        Q, K, V, dO = (torch.from_numpy(rng.standard_normal((B, H, T, 64)).astype(np.float32)) for _ in range(4))
        segs = segments_of(rank, world, T, layout)
        shard = lambda x: torch.cat([x[:, :, s:s + n] for (s, n) in segs], dim=2).contiguous()
        ring = RingAttention(T, 0.125, causal, layout=layout, backend=OracleBackend())
        O_l, L_l = ring.forward(shard(Q), shard(K), shard(V))
        dQ_l, dK_l, dV_l = ring.backward(shard(Q), shard(K), shard(V), O_l, L_l, shard(dO))
        outs = [O_l, L_l, dQ_l, dK_l, dV_l]
        gathered = []
        for x in outs:
            lst = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(lst, x.contiguous())
            gathered.append(lst)
        if rank == 0:
            segs_all = [segments_of(r, world, T, layout) for r in range(world)]
            O, L, dQ, dK, dV = (_gather_seq(g, segs_all, T).numpy() for g in gathered)
            O_ref, L_ref = ol.attn_forward(Q.numpy(), K.numpy(), V.numpy(), 0.125, int(causal))
            _, dQ_ref, dK_ref, dV_ref = ol.attn_backward(Q.numpy(), K.numpy(), V.numpy(), O_ref, dO.numpy(), L_ref, 0.125,
                                                         int(causal))
            errs = [float(np.abs(a - b).max()) for a, b in ((O, O_ref), (L, L_ref), (dQ, dQ_ref), (dK, dK_ref), (dV, dV_ref))]
            ret.put(errs)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("layout", ["contiguous", "zigzag"])
@pytest.mark.parametrize("causal", [False, True])
def test_ring_schedule_two_gloo_ranks(layout, causal):
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = 29600 + (hash((layout, causal)) % 200)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, layout, causal, 64, ret)) for r in range(2)]
    for p in procs:
        p.start()
    errs = ret.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # the oracle is fp32/fp64 throughout: only summation order differs from the one-piece computation
    assert max(errs) < 2e-5, errs


def test_ring_of_one_rank_needs_no_exchange():
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    p = ctx.Process(target=_worker, args=(0, 1, 29877, "zigzag", True, 64, ret))
    p.start()
    errs = ret.get(timeout=120)
    p.join(timeout=60)
    assert p.exitcode == 0 and max(errs) < 2e-5, errs


def _failing_worker(rank, world, port, ret):
    """Rank 1 leaves before the first hop (a peer that died between steps); rank 0 must get a RingError from its
    host-timed wait instead of hanging."""
    import datetime
    import time

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    from hyperkernels_b200.ring import RingAttention, RingError

    def leave():  # no clean shutdown of the process group: the process is simply gone
        ret.close()
        ret.join_thread()
        os._exit(0)

    if rank == 1:
        ret.put(("left", 1))
        leave()
    x = torch.zeros((1, 1, 32, 64))
    ring = RingAttention(64, 0.125, True, layout="zigzag", backend=OracleBackend(), timeout_s=3.0)
    t0 = time.time()
    try:
        ring.forward(x, x, x)
        ret.put(("no error", time.time() - t0))
    except RingError:
        ret.put(("RingError", time.time() - t0))
    leave()


def test_lost_peer_raises_ring_error_within_the_timeout():
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, 29911, ret)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict([ret.get(timeout=60), ret.get(timeout=60)])
    for p in procs:
        p.join(timeout=30)
    assert "RingError" in got, got
    assert got["RingError"] < 15.0, got


def test_segments_cover_sequence_once():
    from hyperkernels_b200.ring import segments_of, visible

    for layout in ("contiguous", "zigzag"):
        for G in (1, 2, 4, 8):
            T = 64 * G
            seen = np.zeros(T, int)
            for r in range(G):
                for (s, n) in segments_of(r, G, T, layout):
                    seen[s:s + n] += 1
            assert (seen == 1).all()
    assert visible((0, 8), (8, 8), False) and not visible((0, 8), (8, 8), True) and visible((8, 8), (0, 8), True)
    assert visible((0, 8), (7, 8), True)
