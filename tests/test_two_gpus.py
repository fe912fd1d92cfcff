"""Two GPUs driven from ONE process by one host thread each (the boundary keeps no per-call state and its per-device
caches are filled once under a lock): a batch of a dropout problem is split in two, each half runs on its own
device with bh_pos0 = its first (batch, head) slice, and the halves must equal the whole problem run on one
device bit for bit (O, LSE, dK, dV; dQ up to the order of its fp32 additions) -- same Philox mask however the
work is cut.  Skipped with fewer than two GPUs."""
import threading

import pytest
import torch

import hyperkernels_b200 as hk

pytestmark = pytest.mark.gpu
SCALE = 0.125


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_batch_split_over_two_devices_one_thread_each():
    B, H, T, p, seed, off = 4, 6, 512, 0.1, 0xC0FFEE, 2
    g = torch.Generator(device="cuda:0").manual_seed(77)
    Q, K, V, dO = (torch.randn((B, H, T, 64), generator=g, device="cuda:0") for _ in range(4))
    kw = dict(dropout_p=p, philox_seed=seed, philox_offset=off)
    torch.cuda.set_device(0)
    O, LSE = hk.attention_forward(Q, K, V, SCALE, True, **kw)
    dQ, dK, dV, _ = hk.attention_backward(Q, K, V, O, dO, LSE, SCALE, True, **kw)
    torch.cuda.synchronize()
    results, errors = {}, []

    def work(dev):
        try:
            torch.cuda.set_device(dev)
            sl = slice(dev * B // 2, (dev + 1) * B // 2)
            q, k, v, go = (t[sl].to(f"cuda:{dev}").contiguous() for t in (Q, K, V, dO))
            out = None
            for _ in range(4):
                o, l = hk.attention_forward(q, k, v, SCALE, True, bh_pos0=sl.start * H, **kw)
                dq, dk, dv, _ = hk.attention_backward(q, k, v, o, go, l, SCALE, True, bh_pos0=sl.start * H, **kw)
                out = (o, l, dq, dk, dv)
            torch.cuda.synchronize(dev)
            assert hk.last_device_status() == 0
            results[dev] = [t.to("cuda:0") for t in out]
        except Exception as e:  # surfaced in the main thread
            errors.append((dev, repr(e)))

    threads = [threading.Thread(target=work, args=(d,)) for d in (0, 1)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for dev in (0, 1):
        sl = slice(dev * B // 2, (dev + 1) * B // 2)
        o, l, dq, dk, dv = results[dev]
        assert torch.equal(o, O[sl]) and torch.equal(l, LSE[sl]), dev
        assert torch.equal(dk, dK[sl]) and torch.equal(dv, dV[sl]), dev
        assert float((dq - dQ[sl]).abs().max()) <= 1e-4, dev
