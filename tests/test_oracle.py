"""CPU tests: the oracle (oracle/attn_oracle.c) against the golden vectors made
from the reference's own host code, and against that code itself where it is built."""
import hashlib
import json
import os

import numpy as np
import pytest

import oracle_lib as ol

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _inputs(B, H, T, seeds):
    n = B * H * T * 64
    return [ol.rand_vec(n, s).reshape(B, H, T, 64) for s in seeds]


@pytest.mark.parametrize("name", ["attn_ref_T256", "attn_ref_T77"])
@pytest.mark.parametrize("causal", [0, 1])
def test_oracle_matches_golden_bit_exact(name, causal):
    g = np.load(os.path.join(GOLD, name + ".npz"))
    B, H, T, Hd, *seeds = [int(x) for x in g["meta"]]
    Q, K, V, dO = _inputs(B, H, T, seeds)
    O, LSE = ol.attn_forward(Q, K, V, 0.125, causal)
    D, dQ, dK, dV = ol.attn_backward(Q, K, V, O, dO, LSE, 0.125, causal)
    for k, v in dict(O=O, LSE=LSE, D=D, dQ=dQ, dK=dK, dV=dV).items():
        assert np.array_equal(v, g[f"{k}_causal{causal}"]), k


def test_oracle_matches_reference_test_shape_checksums():
    """B=2,H=6,T=256, seeds 101..104: the shape of kernels_test.cu:491-499,545."""
    sums = json.load(open(os.path.join(GOLD, "checksums.json")))
    for s, head in sums["rand_vec_head"].items():
        assert ol.rand_vec(8, int(s)).tolist() == head
    Q, K, V, dO = _inputs(2, 6, 256, (101, 102, 103, 104))
    for causal in (0, 1):
        O, LSE = ol.attn_forward(Q, K, V, 0.125, causal)
        D, dQ, dK, dV = ol.attn_backward(Q, K, V, O, dO, LSE, 0.125, causal)
        for k, v in dict(O=O, LSE=LSE, D=D, dQ=dQ, dK=dK, dV=dV).items():
            assert hashlib.sha256(v.tobytes()).hexdigest() == sums[f"B2H6T256_{k}_causal{causal}"], (k, causal)


@pytest.mark.skipif(ol.reference() is None, reason="oracle/_ref not built (reference sources absent)")
@pytest.mark.parametrize("causal", [0, 1])
def test_oracle_matches_reference_host_code(causal):
    B, H, T = 2, 3, 100
    n = B * H * T * 64
    for s in (3, 101):
        assert np.array_equal(ol.rand_vec(n, s), ol.ref_rand_vec(n, s))
    Q, K, V, dO = _inputs(B, H, T, (21, 22, 23, 24))
    O, LSE = ol.attn_forward(Q, K, V, 0.2, causal)
    O2, LSE2 = ol.ref_attn_forward(Q, K, V, 0.2, causal)
    assert np.array_equal(O, O2) and np.array_equal(LSE, LSE2)
    outs = ol.attn_backward(Q, K, V, O, dO, LSE, 0.2, causal)
    outs2 = ol.ref_attn_backward(Q, K, V, O, dO, LSE, 0.2, causal)
    for a, b in zip(outs, outs2):
        assert np.array_equal(a, b)


def test_precompute_D_matches_reference_formula():
    """kernels_test.cu:465: refD[r] = (float) sum_k (double)(dO*O) with float products."""
    rng = np.random.default_rng(0)
    dO = rng.uniform(-1, 1, (50, 64)).astype(np.float32)
    O = rng.uniform(-1, 1, (50, 64)).astype(np.float32)
    D = ol.precompute_D(dO, O)
    ref = (dO.astype(np.float64) * O.astype(np.float64)).sum(-1)
    assert np.max(np.abs(D - ref)) < 1e-5


def test_philox_known_answers():
    """Random123 known-answer vectors for philox4x32-10, through the keep-mask threshold path."""
    import ctypes as C
    import subprocess
    import tempfile

    src = r'''
#include <stdio.h>
#include "philox.h"
int main(void) {
  hk_philox4_t a = hk_philox4x32_10(0,0,0,0,0,0);
  printf("%08x %08x %08x %08x\n", a.v[0], a.v[1], a.v[2], a.v[3]);
  a = hk_philox4x32_10(~0u,~0u,~0u,~0u,~0u,~0u);
  printf("%08x %08x %08x %08x\n", a.v[0], a.v[1], a.v[2], a.v[3]);
  a = hk_philox4x32_10(0x243f6a88,0x85a308d3,0x13198a2e,0x03707344,0xa4093822,0x299f31d0);
  printf("%08x %08x %08x %08x\n", a.v[0], a.v[1], a.v[2], a.v[3]);
  return 0; }
'''
    inc = os.path.join(ol.ROOT, "hyperkernels_b200", "csrc")
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, "k.c"), "w").write(src)
        subprocess.check_call(["gcc", "-I", inc, os.path.join(d, "k.c"), "-o", os.path.join(d, "k")])
        out = subprocess.check_output([os.path.join(d, "k")]).decode().split("\n")
    assert out[0] == "6627e8d5 e169c58d bc57ac4c 9b00dbd8"
    assert out[1] == "408f276d 41c83b0e a20bc7c6 6d5451fd"
    assert out[2] == "d16cfe09 94fdcceb 5001e420 24126ea1"


def test_dropout_mask_properties():
    m = ol.dropout_mask(3, 40, 52, 0.25, seed=1234, offset=77)
    assert set(np.unique(m)) <= {0.0, 1.0}
    assert abs(m.mean() - 0.75) < 0.03
    # position-addressed: a shifted window reproduces the same bits
    w = ol.dropout_mask(3, 10, 12, 0.25, seed=1234, offset=77, q_pos0=8, k_pos0=16)
    assert np.array_equal(w, m[:, 8:18, 16:28])
    assert not np.array_equal(m, ol.dropout_mask(3, 40, 52, 0.25, seed=1235, offset=77))
    assert ol.dropout_mask(1, 4, 8, 0.0, 1, 1).min() == 1.0


def _fd_check(mask):
    """Finite-difference check of the oracle backward (incl. dropout) in float64 re-implementation."""
    rng = np.random.default_rng(5)
    T, Hd = 9, 64
    Q, K, V, dO = (rng.standard_normal((1, 1, T, Hd)).astype(np.float32) for _ in range(4))
    scale, causal = 0.125, 1

    def f64(Qd):
        S = (Qd[0, 0].astype(np.float64) @ K[0, 0].astype(np.float64).T) * scale
        S = np.where(np.tril(np.ones((T, T), bool)), S, -np.inf)
        E = np.exp(S - S.max(-1, keepdims=True))
        if mask is not None:
            E = E * mask[0]
        P = E / E.sum(-1, keepdims=True)
        return float(((P @ V[0, 0].astype(np.float64)) * dO[0, 0]).sum())

    O, LSE = ol.attn_forward(Q, K, V, scale, causal, mask=mask)
    _, dQ, _, _ = ol.attn_backward(Q, K, V, O, dO, LSE, scale, causal, mask=mask)
    eps = 1e-3
    for (i, k) in [(0, 0), (3, 5), (8, 63)]:
        Qp = Q.astype(np.float64).copy(); Qm = Qp.copy()
        Qp[0, 0, i, k] += eps; Qm[0, 0, i, k] -= eps
        fd = (f64(Qp) - f64(Qm)) / (2 * eps)
        assert abs(fd - dQ[0, 0, i, k]) < 2e-4 * max(1.0, abs(fd)), (i, k, fd, dQ[0, 0, i, k])


def test_oracle_backward_finite_difference_no_dropout():
    _fd_check(None)


def test_oracle_backward_finite_difference_dropout():
    m = ol.dropout_mask(1, 9, 9, 0.3, seed=9, offset=0)
    m[0, np.arange(9), np.arange(9)] = 1.0  # keep the diagonal so no row is fully dropped
    _fd_check(m)


def test_oracle_fully_dropped_row():
    rng = np.random.default_rng(1)
    Q, K, V, dO = (rng.standard_normal((1, 1, 4, 64)).astype(np.float32) for _ in range(4))
    mask = np.ones((1, 4, 4), np.float32)
    mask[0, 0, :] = 0.0  # row 0 sees only key 0 under the causal mask, and it is dropped
    O, LSE = ol.attn_forward(Q, K, V, 0.125, 1, mask=mask)
    assert np.all(O[0, 0, 0] == 0) and LSE[0, 0, 0] == -np.inf
    D, dQ, dK, dV = ol.attn_backward(Q, K, V, O, dO, LSE, 0.125, 1, mask=mask)
    assert np.all(np.isfinite(dQ)) and np.all(dQ[0, 0, 0] == 0)


def test_oracle_shifted_window_equals_full():
    """q_pos0/k_pos0: a block of queries against a block of keys equals the same slice of the full causal problem
    once partial results are merged (here: one block containing every visible key)."""
    rng = np.random.default_rng(2)
    T = 48
    Q, K, V = (rng.standard_normal((1, 2, T, 64)).astype(np.float32) for _ in range(3))
    O, LSE = ol.attn_forward(Q, K, V, 0.125, 1)
    Ob, Lb = ol.attn_forward(Q[:, :, 16:32], K[:, :, :32], V[:, :, :32], 0.125, 1, q_pos0=16, k_pos0=0)
    assert np.array_equal(Ob, O[:, :, 16:32]) and np.array_equal(Lb, LSE[:, :, 16:32])


def test_oracle_scaled_dropout_finite_difference():
    """Inverted dropout (mask/(1-p), no renormalisation): float64 restatement + finite differences."""
    rng = np.random.default_rng(8)
    T, Hd, p = 9, 64, 0.3
    Q, K, V, dO = (rng.standard_normal((1, 1, T, Hd)).astype(np.float32) for _ in range(4))
    mask = ol.dropout_mask(1, T, T, p, seed=4, offset=0)
    scale = 0.125

    def f64(Qd):
        S = (Qd[0, 0].astype(np.float64) @ K[0, 0].astype(np.float64).T) * scale
        S = np.where(np.tril(np.ones((T, T), bool)), S, -np.inf)
        P = np.exp(S - S.max(-1, keepdims=True))
        P = P / P.sum(-1, keepdims=True)
        return float((((P * mask[0] / (1 - p)) @ V[0, 0].astype(np.float64)) * dO[0, 0]).sum())

    O, LSE = ol.attn_forward_scaled(Q, K, V, scale, 1, mask, p)
    O0, LSE0 = ol.attn_forward(Q, K, V, scale, 1)
    assert np.array_equal(LSE, LSE0)  # the mask does not enter the normaliser
    _, dQ, _, _ = ol.attn_backward_scaled(Q, K, V, O, dO, LSE, scale, 1, mask, p)
    eps = 1e-3
    for (i, k) in [(0, 0), (3, 5), (8, 63)]:
        Qp = Q.astype(np.float64).copy(); Qm = Qp.copy()
        Qp[0, 0, i, k] += eps; Qm[0, 0, i, k] -= eps
        fd = (f64(Qp) - f64(Qm)) / (2 * eps)
        assert abs(fd - dQ[0, 0, i, k]) < 2e-4 * max(1.0, abs(fd)), (i, k, fd, dQ[0, 0, i, k])
    # without a mask it is the plain attention
    O1, _ = ol.attn_forward_scaled(Q, K, V, scale, 1, None, 0.0)
    assert np.allclose(O1, O0, atol=1e-7)
