"""GPU comparison with the reference's OWN kernels: the three sm_89 attention kernels of
BlubridgeAI/HyperKernels, unmodified, recompiled for the local GPU into oracle/_ref/libhkref.so (only where the
reference sources were available at build time; skipped otherwise).  They are fed the very argument block that
hk_attn_forward / hk_attn_backward receive (the first 192 / 328 bytes are the reference layout), which shows the
drop-in property, and their error against the CPU oracle is the accuracy ceiling: ours must be no worse."""
import ctypes as C
import time

import numpy as np
import pytest
import torch

import hyperkernels_b200 as hk
import oracle_lib as ol

pytestmark = pytest.mark.gpu
SCALE = 0.125


def _blocks(Q, K, V, O, LSE, dO, D, dQ, dK, dV, causal):
    B, H, T, _ = Q.shape
    f = hk.MemEfficientFwdParams()
    f.Q, f.K, f.V, f.O, f.LSE = (t.data_ptr() for t in (Q, K, V, O, LSE))
    f.B, f.nh, f.T, f.scale, f.is_causal = B, H, T, SCALE, causal
    b = hk.MemEfficientBwdParams()
    b.Q, b.K, b.V, b.O, b.dO, b.LSE, b.D, b.dQ, b.dK, b.dV = (t.data_ptr() for t in (Q, K, V, O, dO, LSE, D, dQ, dK, dV))
    b.B, b.nh, b.T, b.scale, b.is_causal = B, H, T, SCALE, causal
    for blk, names in ((f, "qkvo"), (b, ("q", "k", "v", "o", "do", "dq", "dk", "dv"))):
        for n in names:
            setattr(blk, f"{n}_strideB", H * T * 64); setattr(blk, f"{n}_strideH", T * 64); setattr(blk, f"{n}_strideM", 64)
        blk.lse_strideB, blk.lse_strideH = H * T, T
    b.d_strideB, b.d_strideH = H * T, T
    return f, b


@pytest.mark.skipif(ol.reference() is None, reason="oracle/_ref not built (reference sources absent at build time)")
@pytest.mark.parametrize("causal,stress", [(False, False), (True, False), (True, True)])
def test_no_worse_than_the_reference_kernels(causal, stress):
    """stress: every 64th key row scaled x8 as in the long-sequence config, where |scores| reach ~60 and plain TF32
    cannot meet the absolute gate -- neither kernel does; the applicable bound there is the reference kernel's own
    error."""
    ref = ol.reference()
    B, H, T = 2, 4, 512
    rng = np.random.default_rng(21)
    Q, K, V, dO = (rng.standard_normal((B, H, T, 64)).astype(np.float32) for _ in range(4))
    if stress:
        K[:, :, ::64] *= 8.0
    O_or, L_or = ol.attn_forward_mt(Q, K, V, SCALE, int(causal))
    D_or, dQ_or, dK_or, dV_or = ol.attn_backward_mt(Q, K, V, O_or, dO, L_or, SCALE, int(causal))
    t = {k: torch.from_numpy(v).cuda() for k, v in dict(Q=Q, K=K, V=V, dO=dO).items()}
    mk = lambda: torch.empty((B, H, T, 64), device="cuda")
    O, dQ, dK, dV = mk(), torch.zeros((B, H, T, 64), device="cuda"), mk(), mk()
    LSE, D = torch.empty((B, H, T), device="cuda"), torch.empty((B, H, T), device="cuda")
    f, b = _blocks(t["Q"], t["K"], t["V"], O, LSE, t["dO"], D, dQ, dK, dV, causal)
    # --- the reference kernels, launched with the reference test's geometry (kernels_test.cu:509-530,475-477,580-584)
    assert ref.hkref_gpu_forward(C.byref(f), None) == 0
    assert ref.hkref_gpu_precompute_D(C.byref(b), None) == 0
    assert ref.hkref_gpu_backward(C.byref(b), None) == 0
    torch.cuda.synchronize()
    ref_err = {k: (ol.max_abs(v.cpu().numpy(), o), ol.rel_l2(v.cpu().numpy(), o))
               for k, v, o in (("O", O, O_or), ("dQ", dQ, dQ_or), ("dK", dK, dK_or), ("dV", dV, dV_or))}
    # --- ours, same argument blocks plus a workspace
    O2, dQ2, dK2, dV2 = mk(), mk(), mk(), mk()
    LSE2, D2 = torch.empty((B, H, T), device="cuda"), torch.empty((B, H, T), device="cuda")
    f2, b2 = _blocks(t["Q"], t["K"], t["V"], O2, LSE2, t["dO"], D2, dQ2, dK2, dV2, causal)
    ws = torch.empty(4 * B * H * T * 256 + 256, dtype=torch.uint8, device="cuda")
    base = ws.data_ptr() + (-ws.data_ptr()) % 256
    f2.workspace, f2.workspace_bytes = base, hk.fwd_workspace_bytes(f2)
    b2.workspace, b2.workspace_bytes = base, hk.bwd_workspace_bytes(b2)
    hk.fused_attn_forward(f2)
    hk.mem_efficient_bwd_unified(b2)
    torch.cuda.synchronize()
    assert hk.last_device_status() == 0
    our_err = {k: (ol.max_abs(v.cpu().numpy(), o), ol.rel_l2(v.cpu().numpy(), o))
               for k, v, o in (("O", O2, O_or), ("dQ", dQ2, dQ_or), ("dK", dK2, dK_or), ("dV", dV2, dV_or))}
    print("reference kernels:", ref_err)
    print("sm_100a kernels:  ", our_err)
    for k in ref_err:
        # same rounding of every MMA operand, same fp32 accumulation: errors of the same size (25 % slack for the
        # different summation order and exp2 approximation), and inside the absolute gate
        assert our_err[k][1] <= max(1.25 * ref_err[k][1], 2e-4), (k, our_err[k], ref_err[k])
        if stress:
            assert our_err[k][0] <= max(1.25 * ref_err[k][0], 5e-3), (k, our_err[k], ref_err[k])
        else:
            assert our_err[k][0] <= 5e-3 and our_err[k][1] <= 1e-3


@pytest.mark.skipif(ol.reference() is None, reason="oracle/_ref not built (reference sources absent at build time)")
@pytest.mark.parametrize("causal", [False, True])
def test_dropout_forward_pinned_to_the_reference_kernel(causal):
    """The only implementation of the reference's dropout semantics is its GPU forward fed a dense mask
    (fused_attn_forward_kernel_tc_sm89.cu:321-334: e *= mask before the row sum; :412 O = 0 and :424 LSE = -inf for
    a row with nothing kept).  Feed it the mask the Philox generator draws, and compare: the reference kernel, ours
    with the same dense mask, and ours generating the mask in the kernel, each against the CPU oracle's dropout
    extension; ours may not be worse than the reference kernel, and must agree with it directly."""
    ref = ol.reference()
    B, H, T, p, seed, off = 2, 4, 512, 0.2, 0x5EED5EED, 9
    rng = np.random.default_rng(33)
    Q, K, V = (rng.standard_normal((B, H, T, 64)).astype(np.float32) for _ in range(3))
    mask = hk.dropout_keep_mask(B * H, T, T, p, seed, off)
    O_or, L_or = ol.attn_forward_mt(Q, K, V, SCALE, int(causal), mask)
    tQ, tK, tV = (torch.from_numpy(x).cuda() for x in (Q, K, V))
    dmask = torch.from_numpy(mask).cuda()
    mk = lambda: torch.full((B, H, T, 64), float("nan"), device="cuda")
    dummy = mk()
    outs = {}
    for name in ("reference", "ours_dense", "ours_philox"):
        O, LSE = mk(), torch.full((B, H, T), float("nan"), device="cuda")
        f, _ = _blocks(tQ, tK, tV, O, LSE, dummy, LSE, dummy, dummy, dummy, causal)
        f.dropout_p = p
        if name != "ours_philox":
            f.dropout_mask = dmask.data_ptr()
        if name == "reference":
            assert ref.hkref_gpu_forward(C.byref(f), None) == 0
        else:
            if name == "ours_philox":
                f.flags = hk.FLAG_PHILOX_DROPOUT
                f.dropout_seed, f.dropout_offset = seed, off
            ws = torch.empty(3 * B * H * T * 256 + 256, dtype=torch.uint8, device="cuda")
            f.workspace, f.workspace_bytes = ws.data_ptr() + (-ws.data_ptr()) % 256, hk.fwd_workspace_bytes(f)
            hk.fused_attn_forward(f)
        torch.cuda.synchronize()
        outs[name] = (O.cpu().numpy(), LSE.cpu().numpy())
    assert hk.last_device_status() == 0
    err = {k: (ol.max_abs(v[0], O_or), ol.rel_l2(v[0], O_or)) for k, v in outs.items()}
    print("dropout forward errors vs oracle:", err)
    fin = np.isfinite(L_or)
    if causal:
        assert (~fin).any(), "expected at least one fully dropped row (row 0 of a causal head)"
    for k, (O, LSE) in outs.items():
        # fully dropped rows: O = 0, LSE = -inf, exactly (reference :412, :424)
        assert np.array_equal(np.isfinite(LSE), fin), k
        assert np.all(O[~fin] == 0.0), k
        assert ol.max_abs(LSE[fin], L_or[fin]) <= 2e-3, k
    for k in ("ours_dense", "ours_philox"):
        assert err[k][0] <= 5e-3 and err[k][1] <= 1e-3, (k, err[k])
        assert err[k][1] <= max(1.25 * err["reference"][1], 2e-4), (k, err[k], err["reference"])
        assert ol.rel_l2(outs[k][0], outs["reference"][0]) <= 1e-3
    # the in-kernel generator and the dense mask are the same mask: the same result up to the order of the row sums
    assert np.allclose(outs["ours_dense"][0], outs["ours_philox"][0], rtol=1e-5, atol=1e-6)
    assert np.allclose(outs["ours_dense"][1][fin], outs["ours_philox"][1][fin], rtol=0, atol=1e-5)


def _per_head_errors(got, ref):
    """(max abs, relative L2) of every (b, h) slice, computed on the device."""
    d = (got.double() - ref.double()).flatten(2)
    r = ref.double().flatten(2)
    return d.abs().amax(-1), d.norm(dim=-1) / r.norm(dim=-1).clamp_min(1e-30)


def _every_head_against_reference_kernels(B, H, T, causal, sigma, stress, seed, rel_gate, abs_gate):
    """Full-size run of both kernel sets on the same device tensors; every head of O, dQ, dK, dV compared."""
    ref = ol.reference()
    g = torch.Generator(device="cuda").manual_seed(seed)
    Q, K, V = (torch.randn((B, H, T, 64), generator=g, device="cuda") * sigma for _ in range(3))
    dO = torch.randn((B, H, T, 64), generator=g, device="cuda")
    if stress:
        K[:, :, ::64] *= 8.0
    mk = lambda: torch.empty((B, H, T, 64), device="cuda")
    O, dQ, dK, dV = mk(), torch.zeros((B, H, T, 64), device="cuda"), mk(), mk()
    LSE, D = torch.empty((B, H, T), device="cuda"), torch.empty((B, H, T), device="cuda")
    f, b = _blocks(Q, K, V, O, LSE, dO, D, dQ, dK, dV, causal)
    assert ref.hkref_gpu_forward(C.byref(f), None) == 0
    assert ref.hkref_gpu_precompute_D(C.byref(b), None) == 0
    assert ref.hkref_gpu_backward(C.byref(b), None) == 0
    O2, LSE2 = hk.attention_forward(Q, K, V, SCALE, causal)
    dQ2, dK2, dV2, _ = hk.attention_backward(Q, K, V, O2, dO, LSE2, SCALE, causal)
    torch.cuda.synchronize()
    assert hk.last_device_status() == 0
    worst, bad = {}, {}
    for name, a, r in (("O", O2, O), ("dQ", dQ2, dQ), ("dK", dK2, dK), ("dV", dV2, dV)):
        ma, rl = _per_head_errors(a, r)
        worst[name] = (float(ma.max()), float(rl.max()))
        scale_abs = max(1.0, float(r.abs().max()) / 5.0)  # the absolute gate is stated for outputs of magnitude <= 5
        over = torch.nonzero((rl > rel_gate) | (ma > abs_gate * scale_abs)).tolist()
        if over:
            bad[name] = over
    lse_gate = 2e-2 if stress else 2e-3
    lse_err = (LSE2 - LSE).abs().amax(-1)  # per head
    worst["LSE"] = float(lse_err.max())
    if torch.nonzero(lse_err > lse_gate).numel():
        bad["LSE"] = torch.nonzero(lse_err > lse_gate).tolist()
    print(f"every head of B{B} H{H} T{T} vs the reference kernels (worst max-abs, worst rel-L2):", worst)
    if bad and T <= 4096:
        # The two kernel sets disagree on some head: float64 attention of that head (autograd) says which one is off.
        # The reference's sm_89 forward, recompiled for this GPU, is not always reproducible at the B32 H25 shape (a few
        # heads of O come out 1e-2 off from run to run, and D, hence dQ, with them); a head where the reference is
        # the one that deviates is reported and skipped, a head where OURS deviates fails the test.
        heads = sorted({(bi, hi) for hs in bad.values() for (bi, hi) in hs})
        assert len(heads) <= 16, ("too many disagreeing heads to arbitrate", worst)
        report = []
        for (bi, hi) in heads:
            ex = _exact_head(Q, K, V, dO, bi, hi, causal)
            for name, mine_t, theirs_t in (("O", O2, O), ("dQ", dQ2, dQ), ("dK", dK2, dK), ("dV", dV2, dV)):
                mine, theirs = mine_t[bi, hi].double(), theirs_t[bi, hi].double()
                e_mine = float((mine - ex[name]).norm() / ex[name].norm())
                e_theirs = float((theirs - ex[name]).norm() / ex[name].norm())
                report.append((name, bi, hi, e_mine, e_theirs))
                assert e_mine <= 1e-3, ("ours deviates from float64", name, bi, hi, e_mine, e_theirs)
            e_mine = float((LSE2[bi, hi].double() - ex["LSE"]).abs().max())
            e_theirs = float((LSE[bi, hi].double() - ex["LSE"]).abs().max())
            report.append(("LSE", bi, hi, e_mine, e_theirs))
            assert e_mine <= 2e-3, ("ours deviates from float64", "LSE", bi, hi, e_mine, e_theirs)
        print("heads where the reference kernels deviate (tensor, b, h, ours vs float64, reference vs float64):",
              [r for r in report if r[4] > 1e-3])
    else:
        assert not bad, (bad, worst)


def _exact_head(Q, K, V, dO, b, h, causal):
    """float64 attention forward and backward of one (b, h) slice on the device (autograd)."""
    q, k, v = (t[b, h].double().clone().requires_grad_(True) for t in (Q, K, V))
    s = (q @ k.T) * SCALE
    if causal:
        n = s.shape[0]
        s = s.masked_fill(torch.triu(torch.ones(n, n, device=s.device, dtype=torch.bool), 1), float("-inf"))
    o = torch.softmax(s, -1) @ v
    o.backward(dO[b, h].double())
    return {"O": o.detach(), "dQ": q.grad, "dK": k.grad, "dV": v.grad, "LSE": torch.logsumexp(s.detach(), -1)}


# Two TF32 kernels with different summation orders differ from each other by up to the sum of their own errors against
# the exact result: gates = twice the single-kernel gates (max abs 5e-3, relative L2 1e-3).
@pytest.mark.skipif(ol.reference() is None, reason="oracle/_ref not built (reference sources absent at build time)")
def test_config3_shape_every_head_against_reference_kernels():
    """B=16, H=16, N=2048 non-causal, sigma 0.5, p = 0 (the reference backward has no dropout)."""
    _every_head_against_reference_kernels(16, 16, 2048, False, 0.5, False, 31, 2e-3, 1e-2)


@pytest.mark.skipif(ol.reference() is None, reason="oracle/_ref not built (reference sources absent at build time)")
def test_config4_shape_every_head_against_reference_kernels():
    """B=32, H=25, N=1024 causal, p = 0."""
    _every_head_against_reference_kernels(32, 25, 1024, True, 1.0, False, 41, 2e-3, 1e-2)


@pytest.mark.skipif(ol.reference() is None, reason="oracle/_ref not built (reference sources absent at build time)")
def test_config5_shape_every_head_against_reference_kernels():
    """B=1, H=32, N=32768 causal with every 64th key x8: |scores| reach ~60, where plain TF32 cannot meet the absolute
    gate (neither kernel does); the bound is agreement with the reference kernel on every head."""
    _every_head_against_reference_kernels(1, 32, 32768, True, 1.0, True, 51, 1e-2, 5e-2)


@pytest.mark.skipif(ol.reference() is None, reason="oracle/_ref not built (reference sources absent at build time)")
@pytest.mark.parametrize("T,causal,sigma,p", [(2048, False, 0.5, 0.1), (1024, True, 1.0, 0.1)])
def test_dropout_forward_slice_of_configs_3_and_4_against_reference_kernel(T, causal, sigma, p):
    """B=1, H=8 slice of the two dropout configs: the reference forward fed the dense Philox mask against ours
    generating it in the kernel, every head."""
    ref = ol.reference()
    B, H, seed, off = 1, 8, 0x1234ABCD5678, 42
    g = torch.Generator(device="cuda").manual_seed(61)
    Q, K, V = (torch.randn((B, H, T, 64), generator=g, device="cuda") * sigma for _ in range(3))
    mask = torch.from_numpy(hk.dropout_keep_mask(B * H, T, T, p, seed, off)).cuda()
    O, LSE = torch.empty((B, H, T, 64), device="cuda"), torch.empty((B, H, T), device="cuda")
    f, _ = _blocks(Q, K, V, O, LSE, O, LSE, O, O, O, causal)
    f.dropout_p, f.dropout_mask = p, mask.data_ptr()
    assert ref.hkref_gpu_forward(C.byref(f), None) == 0
    O2, LSE2 = hk.attention_forward(Q, K, V, SCALE, causal, dropout_p=p, philox_seed=seed, philox_offset=off)
    torch.cuda.synchronize()
    assert hk.last_device_status() == 0
    ma, rl = _per_head_errors(O2, O)
    print("worst head:", float(ma.max()), float(rl.max()))
    assert float(rl.max()) <= 2e-3 and float(ma.max()) <= 1e-2
    fin = torch.isfinite(LSE)
    assert torch.equal(torch.isfinite(LSE2), fin)
    assert float((LSE2[fin] - LSE[fin]).abs().max()) <= 2e-3


@pytest.mark.skipif(ol.reference() is None, reason="oracle/_ref not built (reference sources absent at build time)")
def test_speed_against_the_reference_kernels_on_this_gpu(capsys):
    """Not a gate: prints the time of the reference's kernels and ours at the GPT-2-small shape on this GPU."""
    ref = ol.reference()
    B, H, T = 8, 12, 1024
    g = torch.Generator(device="cuda").manual_seed(3)
    Q, K, V, dO = (torch.randn((B, H, T, 64), generator=g, device="cuda") for _ in range(4))
    mk = lambda: torch.empty((B, H, T, 64), device="cuda")
    O, dQ, dK, dV = mk(), mk(), mk(), mk()
    LSE, D = torch.empty((B, H, T), device="cuda"), torch.empty((B, H, T), device="cuda")
    f, b = _blocks(Q, K, V, O, LSE, dO, D, dQ, dK, dV, True)

    def timed(fn, n=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        e.record()
        torch.cuda.synchronize()
        return a.elapsed_time(e) / n

    def ref_step():
        ref.hkref_gpu_forward(C.byref(f), None)
        ref.hkref_gpu_precompute_D(C.byref(b), None)
        dQ.zero_()
        ref.hkref_gpu_backward(C.byref(b), None)

    ws = torch.empty(4 * B * H * T * 256 + 256, dtype=torch.uint8, device="cuda")

    def our_step():
        hk.attention_forward(Q, K, V, SCALE, True, workspace=ws, out=O, lse=LSE)
        hk.attention_backward(Q, K, V, O, dO, LSE, SCALE, True, workspace=ws, D=D, dQ=dQ, dK=dK, dV=dV, reuse_fwd_rounded=True)

    t_ref, t_our = timed(ref_step), timed(our_step)
    flop = 14 * B * H * T * T * 64 / 2
    with capsys.disabled():
        print(f"\n[B200, B8 H12 N1024 causal fwd+bwd] reference sm_89 kernels recompiled: {t_ref:.3f} ms "
              f"({flop / t_ref / 1e9:.1f} TFLOP/s); sm_100a kernels: {t_our:.3f} ms ({flop / t_our / 1e9:.1f} TFLOP/s); "
              f"ratio {t_ref / t_our:.2f}x")
    assert hk.last_device_status() == 0
