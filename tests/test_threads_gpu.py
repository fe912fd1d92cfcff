"""The C ABI driven from several host threads at once: four threads, each with its own stream, tensors and
workspace, call hk_attn_forward / hk_attn_backward concurrently (ctypes releases the interpreter lock during the
calls).  Every result must equal what the same call gives when made alone: the library keeps no per-call state
outside the argument block, and its per-device caches are filled once under a lock."""
import threading

import numpy as np
import pytest
import torch

import hyperkernels_b200 as hk

pytestmark = pytest.mark.gpu
SCALE = 0.125


def _problem(seed, B, H, T):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return [torch.randn((B, H, T, 64), generator=g, device="cuda") for _ in range(4)]


def _step(Q, K, V, dO, causal, stream, ws, **kw):
    O, LSE = hk.attention_forward(Q, K, V, SCALE, causal, workspace=ws, stream=stream, **kw)
    dQ, dK, dV, _ = hk.attention_backward(Q, K, V, O, dO, LSE, SCALE, causal, workspace=ws, reuse_fwd_rounded=True,
                                          stream=stream, **kw)
    return O, LSE, dQ, dK, dV


def test_four_host_threads_on_four_streams():
    shapes = [(2, 3, 384, True), (1, 4, 512, False), (3, 2, 200, True), (2, 2, 640, True)]
    drop = [dict(), dict(dropout_p=0.1, philox_seed=5, philox_offset=1), dict(), dict()]
    probs = [_problem(400 + i, B, H, T) for i, (B, H, T, _) in enumerate(shapes)]
    ws = [torch.empty(4 * B * H * T * 256 + 512, dtype=torch.uint8, device="cuda") for (B, H, T, _) in shapes]
    # alone, one after the other
    alone = []
    for i, (B, H, T, causal) in enumerate(shapes):
        alone.append(_step(*probs[i], causal, None, ws[i], **drop[i]))
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream() for _ in shapes]
    results, errors = [None] * len(shapes), []
    barrier = threading.Barrier(len(shapes))

    def work(i):
        try:
            torch.cuda.set_device(0)
            barrier.wait()
            out = None
            for _ in range(8):
                out = _step(*probs[i], shapes[i][3], streams[i], ws[i], **drop[i])
            streams[i].synchronize()
            results[i] = out
        except Exception as e:  # surfaced below, in the main thread
            errors.append((i, repr(e)))

    threads = [threading.Thread(target=work, args=(i,)) for i in range(len(shapes))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    torch.cuda.synchronize()
    assert not errors, errors
    assert hk.last_device_status() == 0
    for i in range(len(shapes)):
        O, LSE, dQ, dK, dV = results[i]
        O0, LSE0, dQ0, dK0, dV0 = alone[i]
        assert torch.equal(O, O0) and torch.equal(LSE, LSE0), i
        assert torch.equal(dK, dK0) and torch.equal(dV, dV0), i
        assert float((dQ - dQ0).abs().max()) <= 1e-4, i
