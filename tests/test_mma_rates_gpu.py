"""The tensor-pipe facts the attention kernels are built on, re-measured (GPU only).

tests/probes/umma_rate.cu issues one tcgen05.mma.kind::tf32 shape back to back from one warp per SM.  Two properties
are held here because the kernels' structure depends on them:

* issuing from a converged warp (instruction predicated on the elected lane) is faster than issuing from inside an
  `if (lane == 0)` region -- the kernels issue the first way;
* M64 shapes run at half the M128 rate, so splitting a tile into two M64 products buys nothing.

Run with `-s` to print the whole table (shape, issue style, TFLOP/s, cycles per instruction).
"""
import ctypes
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "probes", "libumma_rate.so")

MODES = [
    (0, "M128 N128 K8  SS  K-major A, K-major B   (S^T, dP^T shape)"),
    (1, "M128 N64  K8  TS  A in TMEM, MN-major B  (PV, dV, dK shape)"),
    (2, "M128 N64  K8  SS  MN-major A, MN-major B (dQ shape)"),
    (3, "M64  N128 K8  SS"),
    (4, "M64  N256 K8  SS"),
    (5, "M128 N256 K8  SS"),
    (6, "backward tile mix: 16 N128 + 48 N64 products in kernel order"),
]


@pytest.fixture(scope="module")
def probe():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    if not os.path.exists(LIB):
        subprocess.check_call(["make", "-C", os.path.dirname(LIB)])
    lib = ctypes.CDLL(LIB)
    lib.umma_rate_run.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_double),
                                  ctypes.POINTER(ctypes.c_int), ctypes.c_void_p]
    lib.umma_rate_run.restype = ctypes.c_int
    lib.umma_rate_status.restype = ctypes.c_int
    return lib


def _measure(lib, mode, converged, iters=2000):
    """(ms, TFLOP/s over the whole GPU, cycles per instruction at the clock nvidia-smi reports as maximum)"""
    import torch

    sms = torch.cuda.get_device_properties(0).multi_processor_count
    fl, ni = ctypes.c_double(), ctypes.c_int()
    st = torch.cuda.current_stream().cuda_stream
    best = None
    for rep in range(4):  # the first launch warms up; keep the fastest of the rest
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = lib.umma_rate_run(mode, iters, converged, sms, ctypes.byref(fl), ctypes.byref(ni), ctypes.c_void_p(st))
        e1.record()
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert lib.umma_rate_status() == 0
        ms = e0.elapsed_time(e1)
        if rep and (best is None or ms < best):
            best = ms
    tflops = fl.value * iters * sms / (best * 1e-3) / 1e12
    try:
        mhz = int(torch.cuda.clock_rate())  # the SM clock right after the run
    except Exception:
        mhz = 1965
    cyc = best * 1e-3 * mhz * 1e6 / (iters * ni.value)
    return best, tflops, cyc, mhz


def test_issue_from_a_converged_warp_and_shape_costs(probe):
    rows = {}
    for mode, name in MODES:
        for conv in (1, 0):
            rows[(mode, conv)] = _measure(probe, mode, conv)
    print()
    print(f"{'shape':<66} {'issue':<10} {'TFLOP/s':>8} {'cyc/instr':>10} {'SM MHz':>7}")
    for mode, name in MODES:
        for conv in (1, 0):
            ms, tf, cyc, mhz = rows[(mode, conv)]
            print(f"{name:<66} {'converged' if conv else 'lane-0 if':<10} {tf:8.1f} {cyc:10.1f} {mhz:7d}")
    # the N64 products and the tile mix are issue-bound from a divergent region
    assert rows[(1, 1)][1] > 1.15 * rows[(1, 0)][1]
    assert rows[(6, 1)][1] > 1.02 * rows[(6, 0)][1]
    # M64 runs at half rate: no more than 0.6 of the M128 throughput at the same N
    assert rows[(3, 1)][1] < 0.6 * rows[(0, 1)][1]
    assert rows[(4, 1)][1] < 0.6 * rows[(5, 1)][1]
    # the mix the backward kernel issues sustains well above the kernel's present rate: the kernel is not bound here
    assert rows[(6, 1)][1] > 700.0
