"""Host-side mirror of the reference attention launch surface.

The reference (BlubridgeAI/HyperKernels) has no host API; a caller fills a
by-value argument block and launches a kernel:

* ``MemEfficientFwdParams`` + ``fused_attn_forward_kernel_tc_sm89<64,64,64,1>``
  (kernels/attention/fused_attn_forward_kernel_tc_sm89.cu:8-29, launch at
  kernels/tests/kernels_test.cu:520-530),
* ``MemEfficientBwdParams`` + ``mem_efficient_bwd_precompute_D_sm89<64>``
  (kernels/attention/mem_efficient_bwd_precompute_D_sm89.cu:7-33, launch at
  kernels/tests/kernels_test.cu:470-477),
* ``OwnTensor::MemEfficientBwdParams`` + ``mem_efficient_bwd_unified_kernel_exp12``
  (kernels/attention/mem_efficient_bwd_unified_kernel_exp12.cu:11-38, launch at
  kernels/tests/kernels_test.cu:566-584).

Here the same blocks are ``ctypes.Structure`` classes with the same field names
(plus the extension tail of ``include/hk_attention.h``) and the launches are the
functions ``fused_attn_forward``, ``mem_efficient_bwd_precompute_D`` and
``mem_efficient_bwd_unified``, which call the C ABI of ``libhk_attention.so``.
``attention_forward`` / ``attention_backward`` are conveniences that fill the
blocks from torch CUDA tensors; torch is used only to own device memory and
streams.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

# HK_ATTENTION_LIB overrides the location of the compiled library (e.g. an instrumented build).
_LIB_PATH = os.environ.get("HK_ATTENTION_LIB") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib",
                                                               "libhk_attention.so")

FLAG_PHILOX_DROPOUT = 1 << 0
FLAG_OPERANDS_PREROUNDED = 1 << 1
FLAG_ACCUM_DKDV = 1 << 2
FLAG_ACCUM_DQ = 1 << 3
FLAG_D_PRECOMPUTED = 1 << 4
FLAG_REUSE_FWD_ROUNDED = 1 << 5
FLAG_DROPOUT_SCALED = 1 << 6  # inverted dropout (kept terms / (1 - p), normaliser over all keys)
FLAG_CONTINUE_SOFTMAX_STATE = 1 << 7  # forward: O, LSE hold the result over earlier keys; fold this call's keys in
FLAG_ROUND_IN_HBM = 1 << 8  # always round operands with the HBM pre-pass (default: in shared memory for short sequences)
FLAG_DETERMINISTIC_DQ = 1 << 9  # backward: dQ through per-KV-tile slabs added in a fixed order (same bits on every run)

_f32p = C.POINTER(C.c_float)


class HKError(RuntimeError):
    """A call through the C ABI returned a negative hk_status."""

    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().hk_status_string(status).decode() if _lib is not None else "library not loaded"
        super().__init__(f"{where}: {msg} (status {status})")


class MemEfficientFwdParams(C.Structure):
    """Head = the reference's 192-byte MemEfficientFwdParams; tail = hk_attn_fwd_params extension."""

    _fields_ = [
        ("Q", C.c_void_p), ("K", C.c_void_p), ("V", C.c_void_p), ("O", C.c_void_p), ("LSE", C.c_void_p),
        ("B", C.c_int), ("nh", C.c_int), ("T", C.c_int64),
        ("scale", C.c_float), ("is_causal", C.c_bool), ("dropout_p", C.c_float), ("dropout_mask", C.c_void_p),
        ("q_strideB", C.c_int64), ("q_strideM", C.c_int64), ("q_strideH", C.c_int64),
        ("k_strideB", C.c_int64), ("k_strideM", C.c_int64), ("k_strideH", C.c_int64),
        ("v_strideB", C.c_int64), ("v_strideM", C.c_int64), ("v_strideH", C.c_int64),
        ("o_strideB", C.c_int64), ("o_strideM", C.c_int64), ("o_strideH", C.c_int64),
        ("lse_strideB", C.c_int64), ("lse_strideH", C.c_int64),
        # extension tail
        ("dropout_seed", C.c_uint64), ("dropout_offset", C.c_uint64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("kv_len", C.c_int64), ("q_pos0", C.c_int64), ("k_pos0", C.c_int64),
        ("flags", C.c_uint32), ("bh_pos0", C.c_uint32),
    ]


class MemEfficientBwdParams(C.Structure):
    """Head = the reference's 328-byte MemEfficientBwdParams; tail = hk_attn_bwd_params extension."""

    _fields_ = [
        ("Q", C.c_void_p), ("K", C.c_void_p), ("V", C.c_void_p), ("O", C.c_void_p), ("dO", C.c_void_p),
        ("LSE", C.c_void_p), ("D", C.c_void_p), ("dQ", C.c_void_p), ("dK", C.c_void_p), ("dV", C.c_void_p),
        ("B", C.c_int), ("nh", C.c_int), ("T", C.c_int), ("scale", C.c_float), ("is_causal", C.c_bool),
        ("q_strideB", C.c_int64), ("q_strideM", C.c_int64), ("q_strideH", C.c_int64),
        ("k_strideB", C.c_int64), ("k_strideM", C.c_int64), ("k_strideH", C.c_int64),
        ("v_strideB", C.c_int64), ("v_strideM", C.c_int64), ("v_strideH", C.c_int64),
        ("o_strideB", C.c_int64), ("o_strideM", C.c_int64), ("o_strideH", C.c_int64),
        ("do_strideB", C.c_int64), ("do_strideM", C.c_int64), ("do_strideH", C.c_int64),
        ("dq_strideB", C.c_int64), ("dq_strideM", C.c_int64), ("dq_strideH", C.c_int64),
        ("dk_strideB", C.c_int64), ("dk_strideM", C.c_int64), ("dk_strideH", C.c_int64),
        ("dv_strideB", C.c_int64), ("dv_strideM", C.c_int64), ("dv_strideH", C.c_int64),
        ("lse_strideB", C.c_int64), ("lse_strideH", C.c_int64),
        ("d_strideB", C.c_int64), ("d_strideH", C.c_int64),
        # extension tail
        ("dropout_p", C.c_float), ("flags", C.c_uint32), ("dropout_mask", C.c_void_p),
        ("dropout_seed", C.c_uint64), ("dropout_offset", C.c_uint64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("kv_len", C.c_int64), ("q_pos0", C.c_int64), ("k_pos0", C.c_int64),
        ("bh_pos0", C.c_uint32), ("reserved", C.c_uint32),
    ]


assert MemEfficientFwdParams.lse_strideH.offset == 184 and MemEfficientFwdParams.dropout_seed.offset == 192
assert MemEfficientBwdParams.d_strideH.offset == 320 and MemEfficientBwdParams.dropout_p.offset == 328

_lib = None


def lib() -> C.CDLL:
    """Load libhk_attention.so. Fails loudly if the CUDA extension has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise ImportError(
                f"{_LIB_PATH} is missing: build it with `make -C hyperkernels_b200/csrc` "
                "(or __graft_entry__.build()). There is no CPU fallback."
            )
        L = C.CDLL(_LIB_PATH)
        L.hk_status_string.restype = C.c_char_p
        L.hk_status_string.argtypes = [C.c_int]
        L.hk_attn_forward.argtypes = [C.POINTER(MemEfficientFwdParams), C.c_void_p]
        L.hk_attn_backward.argtypes = [C.POINTER(MemEfficientBwdParams), C.c_void_p]
        L.hk_attn_bwd_precompute_D.argtypes = [C.POINTER(MemEfficientBwdParams), C.c_void_p]
        L.hk_attn_bwd_precompute_D_hd.argtypes = [C.POINTER(MemEfficientBwdParams), C.c_int, C.c_void_p]
        L.hk_attn_fwd_workspace_bytes.restype = C.c_size_t
        L.hk_attn_fwd_workspace_bytes.argtypes = [C.POINTER(MemEfficientFwdParams)]
        L.hk_attn_bwd_workspace_bytes.restype = C.c_size_t
        L.hk_attn_bwd_workspace_bytes.argtypes = [C.POINTER(MemEfficientBwdParams)]
        L.hk_attn_merge_partial.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
        L.hk_attn_dropout_mask.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_float, C.c_uint64,
                                           C.c_uint64, C.c_int64, C.c_int64]
        L.hk_attn_dropout_mask_slices.argtypes = [C.c_void_p, C.c_uint32, C.c_int, C.c_int64, C.c_int64, C.c_float,
                                                  C.c_uint64, C.c_uint64, C.c_int64, C.c_int64]
        L.hk_attn_last_device_status.restype = C.c_int
        L.hk_attn_launch_count.restype = C.c_uint64
        L.hk_attn_round_tf32.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
        L.hk_attn_selftest.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        _lib = L
    return _lib


def _check(status: int, where: str) -> None:
    if status != 0:
        raise HKError(status, where)


def _stream_handle(stream) -> Optional[int]:
    if stream is None:
        import torch

        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


# ---- the three launches of the reference, through the C ABI -------------------
def fused_attn_forward(params: MemEfficientFwdParams, stream=None) -> None:
    """fused_attn_forward_kernel_tc_sm89<64,64,64,1><<<...>>>(params) -> hk_attn_forward."""
    _check(lib().hk_attn_forward(C.byref(params), _stream_handle(stream)), "hk_attn_forward")


def mem_efficient_bwd_precompute_D(params: MemEfficientBwdParams, stream=None, head_dim: int = 64) -> None:
    """mem_efficient_bwd_precompute_D_sm89<head_dim><<<...>>>(params) -> hk_attn_bwd_precompute_D[_hd];
    head_dim is the reference's template argument (16, 32, 64, 128 or 256)."""
    if head_dim == 64:
        _check(lib().hk_attn_bwd_precompute_D(C.byref(params), _stream_handle(stream)), "hk_attn_bwd_precompute_D")
    else:
        _check(lib().hk_attn_bwd_precompute_D_hd(C.byref(params), int(head_dim), _stream_handle(stream)),
               "hk_attn_bwd_precompute_D_hd")


def mem_efficient_bwd_unified(params: MemEfficientBwdParams, stream=None) -> None:
    """mem_efficient_bwd_unified_kernel_exp12<64,Causal><<<...>>>(params) -> hk_attn_backward."""
    _check(lib().hk_attn_backward(C.byref(params), _stream_handle(stream)), "hk_attn_backward")


def fwd_workspace_bytes(params: MemEfficientFwdParams) -> int:
    return int(lib().hk_attn_fwd_workspace_bytes(C.byref(params)))


def bwd_workspace_bytes(params: MemEfficientBwdParams) -> int:
    return int(lib().hk_attn_bwd_workspace_bytes(C.byref(params)))


def last_device_status() -> int:
    return int(lib().hk_attn_last_device_status())


def launch_count() -> int:
    return int(lib().hk_attn_launch_count())


def dropout_keep_mask(BH: int, Tq: int, Tk: int, p: float, seed: int, offset: int, q_pos0: int = 0, k_pos0: int = 0,
                      bh_pos0: int = 0):
    """Host twin of the in-kernel Philox mask, in the reference's dense format (numpy [BH,Tq,Tk] of 1.0/0.0);
    bh_pos0 = index of the first (batch, head) slice when the BH slices are a run out of a larger problem."""
    import numpy as np

    m = np.empty((BH, Tq, Tk), dtype=np.float32)
    _check(lib().hk_attn_dropout_mask_slices(m.ctypes.data, bh_pos0, BH, Tq, Tk, p, seed, offset, q_pos0, k_pos0),
           "hk_attn_dropout_mask_slices")
    return m


# ---- conveniences over torch tensors -----------------------------------------
def _strides_bmh(t):
    """(strideB, strideM, strideH) in elements of a [B, H, T, 64] tensor view."""
    assert t.dim() == 4 and t.shape[-1] == 64 and t.stride(-1) == 1, "expected [B,H,T,64] with unit last stride"
    return t.stride(0), t.stride(2), t.stride(1)


def _set3(p, name, t):
    sB, sM, sH = _strides_bmh(t)
    setattr(p, f"{name}_strideB", sB)
    setattr(p, f"{name}_strideM", sM)
    setattr(p, f"{name}_strideH", sH)


def _workspace(nbytes: int, like, workspace):
    import torch

    if nbytes == 0:
        return None
    if workspace is None:
        workspace = torch.empty(nbytes + 256, dtype=torch.uint8, device=like.device)
    base = workspace.data_ptr()
    off = (-base) % 256
    assert workspace.numel() - off >= nbytes, "workspace too small"
    return workspace, base + off


def attention_forward(Q, K, V, scale: float, causal: bool, *, dropout_p: float = 0.0, dropout_mask=None,
                      philox_seed: Optional[int] = None, philox_offset: int = 0, q_pos0: int = 0, k_pos0: int = 0,
                      bh_pos0: int = 0, prerounded: bool = False, dropout_scaled: bool = False, continue_state: bool = False,
                      round_in_hbm: bool = False, workspace=None, out=None, lse=None, stream=None):
    """O, LSE = fused attention forward of [B,H,Tq,64] Q against [B,H,Tk,64] K, V (fp32 CUDA tensors)."""
    import torch

    B, H, Tq, _ = Q.shape
    Tk = K.shape[2]
    O = out if out is not None else torch.empty((B, H, Tq, 64), dtype=torch.float32, device=Q.device)
    LSE = lse if lse is not None else torch.empty((B, H, Tq), dtype=torch.float32, device=Q.device)
    p = MemEfficientFwdParams()
    p.Q, p.K, p.V, p.O, p.LSE = Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), LSE.data_ptr()
    p.B, p.nh, p.T = B, H, Tq
    p.scale, p.is_causal, p.dropout_p = scale, bool(causal), dropout_p
    p.dropout_mask = dropout_mask.data_ptr() if dropout_mask is not None else None
    for name, t in (("q", Q), ("k", K), ("v", V), ("o", O)):
        _set3(p, name, t)
    p.lse_strideB, p.lse_strideH = LSE.stride(0), LSE.stride(1)
    p.kv_len = Tk if Tk != Tq else 0
    p.q_pos0, p.k_pos0, p.bh_pos0 = q_pos0, k_pos0, bh_pos0
    flags = 0
    if philox_seed is not None:
        flags |= FLAG_PHILOX_DROPOUT
        p.dropout_seed, p.dropout_offset = philox_seed, philox_offset
    if prerounded:
        flags |= FLAG_OPERANDS_PREROUNDED
    if dropout_scaled:
        flags |= FLAG_DROPOUT_SCALED
    if continue_state:
        assert out is not None and lse is not None, "continue_state folds new keys into the given out / lse"
        flags |= FLAG_CONTINUE_SOFTMAX_STATE
    if round_in_hbm:
        flags |= FLAG_ROUND_IN_HBM
    p.flags = flags
    need = fwd_workspace_bytes(p)
    if need == 0 and workspace is not None and not prerounded:
        # nothing is required (operands rounded in shared memory), but a workspace that is given receives the rounded
        # Q for a backward call with reuse_fwd_rounded
        base = workspace.data_ptr()
        off = (-base) % 256
        p.workspace, p.workspace_bytes = base + off, workspace.numel() - off
    else:
        ws = _workspace(need, Q, workspace)
        if ws is not None:
            p.workspace, p.workspace_bytes = ws[1], need
    fused_attn_forward(p, stream)
    return O, LSE


def attention_backward(Q, K, V, O, dO, LSE, scale: float, causal: bool, *, dropout_p: float = 0.0, dropout_mask=None,
                       philox_seed: Optional[int] = None, philox_offset: int = 0, q_pos0: int = 0, k_pos0: int = 0,
                       bh_pos0: int = 0, prerounded: bool = False, D=None, d_precomputed: bool = False, accum_dkdv: bool = False,
                       accum_dq: bool = False, reuse_fwd_rounded: bool = False, dropout_scaled: bool = False,
                       round_in_hbm: bool = False, deterministic_dq: bool = False, workspace=None, dQ=None, dK=None, dV=None,
                       stream=None):
    """dQ, dK, dV, D = fused attention backward (fp32 CUDA tensors, [B,H,T,64])."""
    import torch

    B, H, Tq, _ = Q.shape
    Tk = K.shape[2]
    dev = Q.device
    dQ = dQ if dQ is not None else torch.empty((B, H, Tq, 64), dtype=torch.float32, device=dev)
    dK = dK if dK is not None else torch.empty((B, H, Tk, 64), dtype=torch.float32, device=dev)
    dV = dV if dV is not None else torch.empty((B, H, Tk, 64), dtype=torch.float32, device=dev)
    D = D if D is not None else torch.empty((B, H, Tq), dtype=torch.float32, device=dev)
    p = MemEfficientBwdParams()
    p.Q, p.K, p.V, p.dO, p.LSE = Q.data_ptr(), K.data_ptr(), V.data_ptr(), dO.data_ptr(), LSE.data_ptr()
    p.O = O.data_ptr() if O is not None else None
    p.D, p.dQ, p.dK, p.dV = D.data_ptr(), dQ.data_ptr(), dK.data_ptr(), dV.data_ptr()
    p.B, p.nh, p.T = B, H, Tq
    p.scale, p.is_causal = scale, bool(causal)
    for name, t in (("q", Q), ("k", K), ("v", V), ("do", dO), ("dq", dQ), ("dk", dK), ("dv", dV)):
        _set3(p, name, t)
    if O is not None:
        _set3(p, "o", O)
    p.lse_strideB, p.lse_strideH = LSE.stride(0), LSE.stride(1)
    p.d_strideB, p.d_strideH = D.stride(0), D.stride(1)
    p.dropout_p = dropout_p
    p.dropout_mask = dropout_mask.data_ptr() if dropout_mask is not None else None
    p.kv_len = Tk if Tk != Tq else 0
    p.q_pos0, p.k_pos0, p.bh_pos0 = q_pos0, k_pos0, bh_pos0
    flags = 0
    if philox_seed is not None:
        flags |= FLAG_PHILOX_DROPOUT
        p.dropout_seed, p.dropout_offset = philox_seed, philox_offset
    if prerounded:
        flags |= FLAG_OPERANDS_PREROUNDED
    if d_precomputed:
        flags |= FLAG_D_PRECOMPUTED
    if accum_dkdv:
        flags |= FLAG_ACCUM_DKDV
    if accum_dq:
        flags |= FLAG_ACCUM_DQ
    if dropout_scaled:
        flags |= FLAG_DROPOUT_SCALED
    if reuse_fwd_rounded:
        assert workspace is not None, "reuse_fwd_rounded needs the workspace the forward used"
        flags |= FLAG_REUSE_FWD_ROUNDED
    if round_in_hbm:
        flags |= FLAG_ROUND_IN_HBM
    if deterministic_dq:
        flags |= FLAG_DETERMINISTIC_DQ
    p.flags = flags
    ws = _workspace(bwd_workspace_bytes(p), Q, workspace)
    if ws is not None:
        p.workspace, p.workspace_bytes = ws[1], bwd_workspace_bytes(p)
    mem_efficient_bwd_unified(p, stream)
    return dQ, dK, dV, D


def round_tf32(x, out=None, stream=None):
    """TF32-round a contiguous [..., 64] fp32 CUDA tensor the way the kernels' pre-pass does."""
    import torch

    assert x.is_contiguous() and x.shape[-1] == 64
    out = out if out is not None else torch.empty_like(x)
    _check(lib().hk_attn_round_tf32(x.data_ptr(), out.data_ptr(), x.numel() // 64, _stream_handle(stream)),
           "hk_attn_round_tf32")
    return out


def merge_partial(O_acc, LSE_acc, O_part, LSE_part, stream=None) -> None:
    """In-place softmax merge of two forward results over disjoint key blocks (contiguous tensors)."""
    assert O_acc.is_contiguous() and O_part.is_contiguous() and LSE_acc.is_contiguous() and LSE_part.is_contiguous()
    rows = LSE_acc.numel()
    _check(lib().hk_attn_merge_partial(O_acc.data_ptr(), LSE_acc.data_ptr(), O_part.data_ptr(), LSE_part.data_ptr(),
                                       rows, _stream_handle(stream)), "hk_attn_merge_partial")
