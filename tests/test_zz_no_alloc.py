"""GPU test of hk_attn_forward_static_scratch, the forward for callers that cannot allocate
device memory (a plug-in inside a framework that owns the GPU's memory pool, a serving loop
where cudaMalloc would stall the device).  The file name sorts last on purpose: a run that
stops at the first failure has then already run every other test.

The entry point must give what hk_attn_forward gives for the same block (it runs the same
kernels on the same rounded operands, so the results are required to be identical, which is
inside the tolerance every other forward test uses), on two calls in a row that share the
built-in scratch, and must refuse problems that do not fit in it.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import hyperkernels_b200 as hk

pytestmark = pytest.mark.gpu


def _block(Q, K, V, O, LSE, causal):
    B, H, T, _ = Q.shape
    p = hk.MemEfficientFwdParams()
    p.Q, p.K, p.V, p.O, p.LSE = (t.data_ptr() for t in (Q, K, V, O, LSE))
    p.B, p.nh, p.T, p.scale, p.is_causal = B, H, T, 0.125, causal
    for n in "qkvo":
        setattr(p, f"{n}_strideB", H * T * 64); setattr(p, f"{n}_strideH", T * 64); setattr(p, f"{n}_strideM", 64)
    p.lse_strideB, p.lse_strideH = H * T, T
    return p


def test_static_scratch_forward_matches_workspace_forward():
    L = hk.lib()
    L.hk_attn_forward_static_scratch.argtypes = [C.POINTER(hk.MemEfficientFwdParams), C.c_void_p]
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(123)
    for call, (B, H, T, causal) in enumerate([(2, 3, 333, True), (1, 4, 512, False), (2, 2, 640, True)]):
        Q, K, V = (torch.randn((B, H, T, 64), generator=g, device="cuda") for _ in range(3))
        O_ref, LSE_ref = hk.attention_forward(Q, K, V, 0.125, causal)      # existing entry point, caller workspace
        O = torch.full_like(O_ref, float("nan"))
        LSE = torch.full_like(LSE_ref, float("nan"))
        p = _block(Q, K, V, O, LSE, causal)                                # workspace fields left null on purpose
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]                         # cudaMemGetInfo
        rc = L.hk_attn_forward_static_scratch(C.byref(p), stream)
        torch.cuda.synchronize()
        free_after = torch.cuda.mem_get_info()[0]
        assert rc == 0, (call, L.hk_status_string(rc))
        if call > 0:
            # nothing was allocated or freed by the call (the first call on a device may make the driver load the
            # module that holds the array, which is when the 24 MiB become resident: it is exempt)
            assert free_after == free_before, (call, free_before, free_after)
        assert hk.last_device_status() == 0
        # same kernels, same rounded operands: identical results (tolerance of the other tests: 5e-3 / 1e-3)
        assert torch.equal(O, O_ref) and torch.equal(LSE, LSE_ref), call
        assert float((O - O_ref).abs().max()) <= 5e-3


def test_static_scratch_rejects_oversized_problem():
    L = hk.lib()
    L.hk_attn_forward_static_scratch.argtypes = [C.POINTER(hk.MemEfficientFwdParams), C.c_void_p]
    t = torch.zeros(64, device="cuda")
    B, H, T = 8, 12, 1024  # 3 * 96 * 1024 * 256 B = 72 MiB of rounded copies > 24 MiB
    p = hk.MemEfficientFwdParams()
    p.Q = p.K = p.V = p.O = p.LSE = t.data_ptr()
    p.B, p.nh, p.T, p.scale = B, H, T, 0.125
    for n in "qkvo":
        setattr(p, f"{n}_strideB", H * T * 64); setattr(p, f"{n}_strideH", T * 64); setattr(p, f"{n}_strideM", 64)
    rc = L.hk_attn_forward_static_scratch(C.byref(p), None)
    assert rc == -9
    assert b"24 MiB" in L.hk_status_string(rc)
