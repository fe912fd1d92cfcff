"""CPU tests of the C-ABI boundary: the library loads, exports every symbol the
header declares, the argument blocks have the reference's layout, and argument
validation answers with the documented status codes (no GPU work is launched)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import hyperkernels_b200 as hk
from hyperkernels_b200 import MemEfficientBwdParams as BP
from hyperkernels_b200 import MemEfficientFwdParams as FP

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_every_declared_symbol_is_exported():
    hdr = open(os.path.join(ROOT, "include", "hk_attention.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    names = re.findall(r"\b(hk_[a-z_A-Z0-9]+)\s*\(", hdr)
    assert len(names) >= 10
    L = hk.lib()
    for n in names:
        assert hasattr(L, n), n


def test_reference_block_layouts():
    # MemEfficientFwdParams, fused_attn_forward_kernel_tc_sm89.cu:8-29 (192 bytes)
    exp = dict(Q=0, K=8, V=16, O=24, LSE=32, B=40, nh=44, T=48, scale=56, is_causal=60, dropout_p=64,
               dropout_mask=72, q_strideB=80, q_strideM=88, q_strideH=96, k_strideB=104, v_strideB=128,
               o_strideB=152, lse_strideB=176, lse_strideH=184, dropout_seed=192)
    for k, v in exp.items():
        assert getattr(FP, k).offset == v, k
    assert C.sizeof(FP) == 256
    # MemEfficientBwdParams, mem_efficient_bwd_unified_kernel_exp12.cu:11-38 (328 bytes)
    exp = dict(Q=0, K=8, V=16, O=24, dO=32, LSE=40, D=48, dQ=56, dK=64, dV=72, B=80, nh=84, T=88, scale=92,
               is_causal=96, q_strideB=104, q_strideM=112, q_strideH=120, do_strideB=200, dq_strideB=224,
               dk_strideB=248, dv_strideB=272, lse_strideB=296, lse_strideH=304, d_strideB=312, d_strideH=320,
               dropout_p=328)
    for k, v in exp.items():
        assert getattr(BP, k).offset == v, k
    assert C.sizeof(BP) == 408
    # extension tails: the Philox (batch, head) base index
    assert FP.bh_pos0.offset == 252 and BP.bh_pos0.offset == 400


def _fwd_block():
    p = FP()
    p.Q = p.K = p.V = p.O = p.LSE = 0x1000
    p.B, p.nh, p.T, p.scale = 1, 1, 128, 0.125
    for n in "qkvo":
        setattr(p, f"{n}_strideB", 128 * 64); setattr(p, f"{n}_strideH", 128 * 64); setattr(p, f"{n}_strideM", 64)
    p.lse_strideB = p.lse_strideH = 128
    p.flags = hk.FLAG_OPERANDS_PREROUNDED
    return p


def test_forward_argument_validation():
    L = hk.lib()
    assert L.hk_attn_forward(None, None) == -1
    p = _fwd_block(); p.Q = None
    assert L.hk_attn_forward(C.byref(p), None) == -1          # null pointer
    p = _fwd_block(); p.T = 0
    assert L.hk_attn_forward(C.byref(p), None) == -2          # bad shape
    p = _fwd_block(); p.K = 0x1004
    assert L.hk_attn_forward(C.byref(p), None) == -3          # misaligned pointer
    p = _fwd_block(); p.q_strideM = 66
    assert L.hk_attn_forward(C.byref(p), None) == -3          # misaligned stride
    p = _fwd_block(); p.dropout_p = 1.0
    assert L.hk_attn_forward(C.byref(p), None) == -4          # p outside [0,1)
    p = _fwd_block(); p.dropout_p = 0.1; p.dropout_mask = 0x1000; p.flags |= hk.FLAG_PHILOX_DROPOUT
    assert L.hk_attn_forward(C.byref(p), None) == -4          # both mask sources
    p = _fwd_block(); p.flags = hk.FLAG_ROUND_IN_HBM
    assert L.hk_attn_forward(C.byref(p), None) == -5          # workspace missing (the HBM pre-pass needs one)
    p = _fwd_block(); p.flags = 0; p.T = 4096
    assert L.hk_attn_forward(C.byref(p), None) == -5          # long sequences are always rounded by the pre-pass
    p = _fwd_block(); p.dropout_p = 0.1; p.flags |= hk.FLAG_PHILOX_DROPOUT; p.k_pos0 = 2
    assert L.hk_attn_forward(C.byref(p), None) == -6          # unsupported Philox alignment


def _bwd_block():
    p = BP()
    p.Q = p.K = p.V = p.O = p.dO = p.LSE = p.D = p.dQ = p.dK = p.dV = 0x1000
    p.B, p.nh, p.T, p.scale = 1, 1, 128, 0.125
    for n in ("q", "k", "v", "o", "do", "dq", "dk", "dv"):
        setattr(p, f"{n}_strideB", 128 * 64); setattr(p, f"{n}_strideH", 128 * 64); setattr(p, f"{n}_strideM", 64)
    p.lse_strideB = p.lse_strideH = p.d_strideB = p.d_strideH = 128
    p.flags = hk.FLAG_OPERANDS_PREROUNDED
    return p


def test_backward_argument_validation():
    L = hk.lib()
    assert L.hk_attn_backward(None, None) == -1
    p = BP()
    assert L.hk_attn_backward(C.byref(p), None) == -1
    assert L.hk_attn_bwd_precompute_D(C.byref(p), None) == -1
    p = _bwd_block(); p.scale = 0.0
    assert L.hk_attn_backward(C.byref(p), None) == -2         # the same scale rule as the forward
    p = _fwd_block(); p.scale = 0.0
    assert L.hk_attn_forward(C.byref(p), None) == -2
    p = _bwd_block(); p.dq_strideM = 32
    assert L.hk_attn_backward(C.byref(p), None) == -2         # rows would overlap
    p = _bwd_block(); p.do_strideM = 32
    assert L.hk_attn_bwd_precompute_D(C.byref(p), None) == -2
    p = _bwd_block(); p.do_strideM = 32
    assert L.hk_attn_bwd_precompute_D_hd(C.byref(p), 64, None) == -2
    assert L.hk_attn_bwd_precompute_D_hd(C.byref(_bwd_block()), 72, None) == -6   # not one of the reference's ten


def test_broadcast_strides_are_refused():
    """A zero batch/head stride cannot be expressed by the TMA tensor maps: refused up front, not as a CUDA error."""
    L = hk.lib()
    p = _fwd_block(); p.nh = 4; p.k_strideH = 0
    assert L.hk_attn_forward(C.byref(p), None) == -6
    p = _fwd_block(); p.B = 2; p.v_strideB = 0
    assert L.hk_attn_forward(C.byref(p), None) == -6
    p = _bwd_block(); p.nh = 2; p.dk_strideH = 0
    assert L.hk_attn_backward(C.byref(p), None) == -6
    p = _fwd_block(); p.k_strideH = 0          # a single head may carry any stride
    assert L.hk_attn_forward(C.byref(p), None) != -6


def test_workspace_sizes():
    p = _fwd_block(); p.flags = hk.FLAG_ROUND_IN_HBM; p.B, p.nh, p.T = 2, 3, 100
    assert hk.fwd_workspace_bytes(p) == 3 * 2 * 3 * 100 * 256
    p.kv_len = 40
    assert hk.fwd_workspace_bytes(p) == 2 * 3 * 256 * (100 + 2 * 40)
    p.flags = hk.FLAG_OPERANDS_PREROUNDED
    assert hk.fwd_workspace_bytes(p) == 0
    # short sequences are rounded in shared memory: the forward needs no scratch at all
    p.flags = 0; p.kv_len = 0
    for T, causal, inside in ((100, False, False), (511, True, False), (512, False, True), (1024, False, True),
                              (1025, False, False), (2048, True, True), (2049, True, False)):
        p.T, p.is_causal = T, causal
        assert (hk.fwd_workspace_bytes(p) == 0) == inside, (T, causal)
        if not inside:
            assert hk.fwd_workspace_bytes(p) == 3 * 2 * 3 * T * 256
    b = BP(); b.B, b.nh, b.T = 2, 3, 100
    assert hk.bwd_workspace_bytes(b) == 4 * 2 * 3 * 100 * 256
    # deterministic dQ: one slab of B*nh*T*256 bytes per 128-key tile behind the rounded operands (alone if those are skipped)
    b.T, b.kv_len = 300, 500
    b.flags = hk.FLAG_DETERMINISTIC_DQ
    assert hk.bwd_workspace_bytes(b) == 2 * 3 * 256 * (2 * 300 + 2 * 500) + 4 * (2 * 3 * 300 * 256)
    b.flags = hk.FLAG_DETERMINISTIC_DQ | hk.FLAG_OPERANDS_PREROUNDED
    assert hk.bwd_workspace_bytes(b) == 4 * (2 * 3 * 300 * 256)


def test_status_strings_and_counters():
    L = hk.lib()
    for s in range(0, -9, -1):
        assert len(L.hk_status_string(s)) > 0
    assert hk.launch_count() == 0 or hk.launch_count() > 0


def test_host_mask_twin_matches_oracle():
    import oracle_lib as ol

    a = hk.dropout_keep_mask(2, 33, 70, 0.1, seed=42, offset=3, q_pos0=5, k_pos0=8)
    b = ol.dropout_mask(2, 33, 70, 0.1, 42, 3, 5, 8)
    assert np.array_equal(a, b)


def test_host_mask_twin_of_a_run_of_slices():
    """bh_pos0: the mask of (batch, head) slices 3..4 of a larger problem is rows 3..4 of the whole mask."""
    whole = hk.dropout_keep_mask(6, 17, 40, 0.3, seed=7, offset=1 << 33)
    part = hk.dropout_keep_mask(2, 17, 40, 0.3, seed=7, offset=1 << 33, bh_pos0=3)
    assert np.array_equal(part, whole[3:5])
    assert not np.array_equal(part, whole[0:2])


def test_missing_library_fails_loudly(monkeypatch):
    import hyperkernels_b200.attention as att

    monkeypatch.setattr(att, "_lib", None)
    monkeypatch.setattr(att, "_LIB_PATH", "/nonexistent/libhk_attention.so")
    with pytest.raises(ImportError):
        att.lib()


def test_ring_library_loads_and_exports_every_symbol():
    """libhk_ring.so (include/hk_ring.h): every declared function is exported; without a GPU the communicator cannot be
    made and the call says so with a status code instead of crashing."""
    import ctypes as C
    import re

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    header = open(os.path.join(root, "include", "hk_ring.h")).read()
    names = sorted(set(re.findall(r"\b(hk_ring_[a-z_]+)\s*\(", header)))
    assert len(names) >= 9
    L = C.CDLL(os.path.join(root, "hyperkernels_b200", "lib", "libhk_ring.so"))
    for n in names:
        assert hasattr(L, n), n
    L.hk_ring_error_string.restype = C.c_char_p
    assert L.hk_ring_error_string(0) == b"ok"
    assert L.hk_ring_get_unique_id(None) == -4
    ring = C.c_void_p()
    uid = C.create_string_buffer(128)
    assert L.hk_ring_create(C.byref(ring), uid, 3, 2) == -4  # rank outside the ring
    assert L.hk_ring_exchange(None, 0, None, 0, None, 0, 0, None, None) == -4
    assert L.hk_ring_wait(None, 0, C.c_double(0.1)) == -4
