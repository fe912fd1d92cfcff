"""ctypes access to the CPU checkers under oracle/ (test infrastructure only).

``oracle()`` is our plain-C restatement (oracle/attn_oracle.c); ``reference()``
is the reference's own host code compiled from its sources (oracle/_ref), or
None when it has not been built.  Both are built by ``make -C oracle``.
"""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
_f32p = C.POINTER(C.c_float)
_oracle = None
_ref = False


def _p(a):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_f32p)


def oracle():
    global _oracle
    if _oracle is None:
        path = os.path.join(ORACLE_DIR, "liboracle.so")
        if not os.path.exists(path):
            subprocess.check_call(["make", "-C", ORACLE_DIR, "liboracle.so"], stdout=subprocess.DEVNULL)
        _oracle = C.CDLL(path)
    return _oracle


def reference():
    global _ref
    if _ref is False:
        path = os.path.join(ORACLE_DIR, "_ref", "libhkref.so")
        _ref = C.CDLL(path) if os.path.exists(path) else None
    return _ref


def rand_vec(n, seed, lo=-1.0, hi=1.0):
    """kernels_test.cu:48-54 (mt19937_64 + uniform_real_distribution<float>)."""
    out = np.empty(n, np.float32)
    oracle().hk_oracle_rand_vec(_p(out), C.c_size_t(n), C.c_uint64(seed), C.c_float(lo), C.c_float(hi))
    return out


def dropout_mask(BH, Tq, Tk, p, seed, offset, q_pos0=0, k_pos0=0):
    m = np.empty((BH, Tq, Tk), np.float32)
    oracle().hk_oracle_dropout_mask(_p(m), BH, Tq, Tk, C.c_float(p), C.c_uint64(seed), C.c_uint64(offset),
                                    C.c_int64(q_pos0), C.c_int64(k_pos0))
    return m


def attn_forward(Q, K, V, scale, causal, mask=None, q_pos0=0, k_pos0=0):
    """Q [B,H,Tq,Hd], K/V [B,H,Tk,Hd] float32 numpy -> O, LSE."""
    B, H, Tq, Hd = Q.shape
    Tk = K.shape[2]
    Q, K, V = (np.ascontiguousarray(x, np.float32) for x in (Q, K, V))
    O = np.empty((B, H, Tq, Hd), np.float32)
    LSE = np.empty((B, H, Tq), np.float32)
    mp = _p(np.ascontiguousarray(mask, np.float32)) if mask is not None else None
    oracle().hk_oracle_attn_forward(_p(Q), _p(K), _p(V), B, H, Tq, Tk, Hd, C.c_float(scale), int(causal),
                                    C.c_int64(q_pos0), C.c_int64(k_pos0), mp, _p(O), _p(LSE))
    return O, LSE


def attn_backward(Q, K, V, O, dO, LSE, scale, causal, mask=None, q_pos0=0, k_pos0=0):
    B, H, Tq, Hd = Q.shape
    Tk = K.shape[2]
    Q, K, V, O, dO, LSE = (np.ascontiguousarray(x, np.float32) for x in (Q, K, V, O, dO, LSE))
    D = np.empty((B, H, Tq), np.float32)
    dQ = np.empty((B, H, Tq, Hd), np.float32)
    dK = np.empty((B, H, Tk, Hd), np.float32)
    dV = np.empty((B, H, Tk, Hd), np.float32)
    mp = _p(np.ascontiguousarray(mask, np.float32)) if mask is not None else None
    oracle().hk_oracle_attn_backward(_p(Q), _p(K), _p(V), _p(O), _p(dO), _p(LSE), B, H, Tq, Tk, Hd, C.c_float(scale),
                                     int(causal), C.c_int64(q_pos0), C.c_int64(k_pos0), mp, _p(D), _p(dQ), _p(dK),
                                     _p(dV))
    return D, dQ, dK, dV


def attn_forward_scaled(Q, K, V, scale, causal, mask, p, q_pos0=0, k_pos0=0):
    """Inverted dropout (mask / (1 - p), no renormalisation): see oracle/attn_oracle.c."""
    B, H, Tq, Hd = Q.shape
    Tk = K.shape[2]
    Q, K, V = (np.ascontiguousarray(x, np.float32) for x in (Q, K, V))
    O = np.empty((B, H, Tq, Hd), np.float32)
    LSE = np.empty((B, H, Tq), np.float32)
    mp = _p(np.ascontiguousarray(mask, np.float32)) if mask is not None else None
    oracle().hk_oracle_attn_forward_scaled_dropout(_p(Q), _p(K), _p(V), B, H, Tq, Tk, Hd, C.c_float(scale), int(causal),
                                                   C.c_int64(q_pos0), C.c_int64(k_pos0), mp,
                                                   C.c_float(1.0 / (1.0 - p)), _p(O), _p(LSE))
    return O, LSE


def attn_backward_scaled(Q, K, V, O, dO, LSE, scale, causal, mask, p, q_pos0=0, k_pos0=0):
    B, H, Tq, Hd = Q.shape
    Tk = K.shape[2]
    Q, K, V, O, dO, LSE = (np.ascontiguousarray(x, np.float32) for x in (Q, K, V, O, dO, LSE))
    D = np.empty((B, H, Tq), np.float32)
    dQ = np.empty((B, H, Tq, Hd), np.float32)
    dK = np.empty((B, H, Tk, Hd), np.float32)
    dV = np.empty((B, H, Tk, Hd), np.float32)
    mp = _p(np.ascontiguousarray(mask, np.float32)) if mask is not None else None
    oracle().hk_oracle_attn_backward_scaled_dropout(_p(Q), _p(K), _p(V), _p(O), _p(dO), _p(LSE), B, H, Tq, Tk, Hd,
                                                    C.c_float(scale), int(causal), C.c_int64(q_pos0), C.c_int64(k_pos0),
                                                    mp, C.c_float(1.0 / (1.0 - p)), _p(D), _p(dQ), _p(dK), _p(dV))
    return D, dQ, dK, dV


def precompute_D(dO, O):
    Hd = dO.shape[-1]
    dO, O = (np.ascontiguousarray(x, np.float32) for x in (dO, O))
    D = np.empty(dO.shape[:-1], np.float32)
    oracle().hk_oracle_precompute_D(_p(dO), _p(O), C.c_int64(D.size), Hd, _p(D))
    return D


# ---- the reference's own host functions (only where oracle/_ref is built) ----
def ref_rand_vec(n, seed, lo=-1.0, hi=1.0):
    out = np.empty(n, np.float32)
    reference().hkref_rand_vec(_p(out), C.c_size_t(n), C.c_uint64(seed), C.c_float(lo), C.c_float(hi))
    return out


def ref_attn_forward(Q, K, V, scale, causal):
    B, H, T, Hd = Q.shape
    O = np.empty((B, H, T, Hd), np.float32)
    LSE = np.empty((B, H, T), np.float32)
    reference().hkref_attn_forward(_p(Q), _p(K), _p(V), B, H, T, Hd, C.c_float(scale), int(causal), _p(O), _p(LSE))
    return O, LSE


def ref_attn_backward(Q, K, V, O, dO, LSE, scale, causal):
    B, H, T, Hd = Q.shape
    D = np.empty((B, H, T), np.float32)
    dQ, dK, dV = (np.empty((B, H, T, Hd), np.float32) for _ in range(3))
    reference().hkref_attn_backward(_p(Q), _p(K), _p(V), _p(O), _p(dO), _p(LSE), B, H, T, Hd, C.c_float(scale),
                                    int(causal), _p(D), _p(dQ), _p(dK), _p(dV))
    return D, dQ, dK, dV


# ---- error metrics of the parity gate ----------------------------------------
def max_abs(a, b):
    return float(np.max(np.abs(a.astype(np.float64) - b.astype(np.float64)))) if a.size else 0.0


def rel_l2(a, b):
    """||a - b||_2 / ||b||_2 with b the oracle."""
    den = float(np.linalg.norm(b.astype(np.float64)))
    num = float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)))
    return num / den if den > 0 else num


# ---- per-head parallel drivers (ctypes releases the GIL; one (b,h) slice per call) ----
def _pool():
    import concurrent.futures as cf

    return cf.ThreadPoolExecutor(max_workers=max(1, os.cpu_count() or 1))


def attn_forward_mt(Q, K, V, scale, causal, mask=None, q_pos0=0, k_pos0=0):
    B, H, Tq, Hd = Q.shape
    O = np.empty((B, H, Tq, Hd), np.float32)
    LSE = np.empty((B, H, Tq), np.float32)

    def one(i):
        b, h = divmod(i, H)
        m = mask[i:i + 1] if mask is not None else None
        o, l = attn_forward(Q[b:b + 1, h:h + 1], K[b:b + 1, h:h + 1], V[b:b + 1, h:h + 1], scale, causal, m, q_pos0, k_pos0)
        O[b, h], LSE[b, h] = o[0, 0], l[0, 0]

    with _pool() as ex:
        list(ex.map(one, range(B * H)))
    return O, LSE


def attn_backward_mt(Q, K, V, O, dO, LSE, scale, causal, mask=None, q_pos0=0, k_pos0=0):
    B, H, Tq, Hd = Q.shape
    Tk = K.shape[2]
    D = np.empty((B, H, Tq), np.float32)
    dQ = np.empty((B, H, Tq, Hd), np.float32)
    dK = np.empty((B, H, Tk, Hd), np.float32)
    dV = np.empty((B, H, Tk, Hd), np.float32)

    def one(i):
        b, h = divmod(i, H)
        m = mask[i:i + 1] if mask is not None else None
        s = (slice(b, b + 1), slice(h, h + 1))
        d, dq, dk, dv = attn_backward(Q[s], K[s], V[s], O[s], dO[s], LSE[s], scale, causal, m, q_pos0, k_pos0)
        D[b, h], dQ[b, h], dK[b, h], dV[b, h] = d[0, 0], dq[0, 0], dk[0, 0], dv[0, 0]

    with _pool() as ex:
        list(ex.map(one, range(B * H)))
    return D, dQ, dK, dV
