#!/usr/bin/env python
"""Benchmark driver: fused attention forward + backward (fp32 I/O, TF32 tensor cores).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config C] [--impl ours|reference]

A "step" is one forward + one backward over one batch of the chosen BASELINE
config (default config 2, the GPT-2-small shape B=8, H=12, N=1024, d=64, causal,
p=0).  With N GPUs every rank runs its own batch of that shape (the work is
partitioned by batch x head, which needs no collective): weak scaling, value =
total algorithmic FLOP/s over all ranks, time = max over ranks.  A line printed
at N > 1 also carries the two multi-GPU configs: `strong_cfg4` (config 4, its
batch split over the ranks) and `ring_cfg5` (config 5, heads split over N/2
groups, the sequence of each group sharded over a 2-rank KV ring), each with its
efficiency against the same config measured on one GPU in the same run.

FLOP convention (the reference's, README.md:148-151 of BlubridgeAI/HyperKernels):
forward 4*B*H*N^2*d, backward 10*B*H*N^2*d, causal counts half.

Printed line (rank 0): metric/value as above with inputs resident in HBM;
`e2e` = the same metric through the C ABI with HOST (pinned) inputs and outputs,
host<->device copies inside the timed region; `roofline` for the dominant kernel
(the backward), timed with CUDA events around the kernel launches inside the
timed region; `cpu_baseline` = the reference's own fp32 host attention timed on
this box's cores (N = 1 only).
"""
import argparse
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    1: dict(B=2, H=4, N=256, causal=True, p=0.0, sigma=1.0, name="cfg1 B2 H4 N256 d64 causal p0"),
    2: dict(B=8, H=12, N=1024, causal=True, p=0.0, sigma=1.0, name="cfg2 GPT-2-small B8 H12 N1024 d64 causal p0"),
    3: dict(B=16, H=16, N=2048, causal=False, p=0.1, sigma=0.5, name="cfg3 B16 H16 N2048 d64 non-causal p0.1"),
    4: dict(B=32, H=25, N=1024, causal=True, p=0.1, sigma=1.0, name="cfg4 GPT-2-XL B32 H25 N1024 d64 causal p0.1"),
    5: dict(B=1, H=32, N=32768, causal=True, p=0.0, sigma=1.0, name="cfg5 B1 H32 N32768 d64 causal p0 (every 64th key x8)"),
}
METRIC = "attn fwd+bwd TF32 TFLOP/s"


def ncu_traffic(kernel, config_id):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of `kernel` at config `config_id`, from the capture
    record committed with the profiles (one line per capture: `<kernel> cfg<id> read_bytes=.. write_bytes=..`);
    None when no capture of that kernel at that config exists."""
    path = os.path.join(ROOT, "profiles", "ncu_dram_traffic.txt")
    try:
        for line in open(path):
            f = line.split()
            if len(f) >= 4 and f[0] == kernel and f[1] == f"cfg{config_id}":
                kv = dict(x.split("=", 1) for x in f[2:] if "=" in x)
                return float(kv["read_bytes"]) + float(kv["write_bytes"])
    except OSError:
        pass
    return None


def flops(cfg, heads=None, fwd=True, bwd=True):
    heads = cfg["B"] * cfg["H"] if heads is None else heads
    f = (4.0 if fwd else 0.0) + (10.0 if bwd else 0.0)
    return f * heads * cfg["N"] ** 2 * 64 * (0.5 if cfg["causal"] else 1.0)


# bare tcgen05.mma.kind::tf32 rate of the backward kernel's own instruction mix (S^T, dP^T at M128 N128; dV, dK, dQ at
# M128 N64), one issuing warp, measured on this pool's B200: a tighter ceiling than half the bf16 GEMM rate
MMA_MIX_PROBE_TFLOPS = 1005.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        # dense TF32 runs at half the dense bf16 rate on the same tensor cores
        return dict(tf32_tflops=p["bf16_tflops"] / 2.0, hbm_gbs=p["hbm_gbs"], source="measured (bf16 burst / 2)")
    return dict(tf32_tflops=1590.0 / 2.0, hbm_gbs=6650.0, source="fallback (1.59 PF bf16 / 2)")


# ---------------------------------------------------------------------------
# reference CPU arm / cpu_baseline
# ---------------------------------------------------------------------------
def _cpu_lib():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol

    if ol.reference() is not None:
        return ol, "reference"
    return ol, "port"


def _cpu_head(ol, kind, cfg, seed):
    """One (b,h) slice, forward + backward, on one thread."""
    import numpy as np

    rng = np.random.default_rng(seed)
    N = cfg["N"]
    Q, K, V, dO = ((rng.standard_normal((1, 1, N, 64)) * s).astype(np.float32)
                   for s in (cfg["sigma"], cfg["sigma"], cfg["sigma"], 1.0))
    t0 = time.perf_counter()
    if kind == "reference":
        O, L = ol.ref_attn_forward(Q, K, V, 0.125, int(cfg["causal"]))
        ol.ref_attn_backward(Q, K, V, O, dO, L, 0.125, int(cfg["causal"]))
    else:
        O, L = ol.attn_forward(Q, K, V, 0.125, int(cfg["causal"]))
        ol.attn_backward(Q, K, V, O, dO, L, 0.125, int(cfg["causal"]))
    return time.perf_counter() - t0


def cpu_batch(ol, kind, cfg, heads, cores, seed0=0):
    """`heads` independent (b,h) slices over `cores` threads; returns wall seconds."""
    import concurrent.futures as cf

    t0 = time.perf_counter()
    with cf.ThreadPoolExecutor(max_workers=cores) as ex:
        list(ex.map(lambda i: _cpu_head(ol, kind, cfg, seed0 + i), range(heads)))
    return time.perf_counter() - t0


def cpu_baseline(cfg, budget_core_s=12.0):
    ol, kind = _cpu_lib()
    cores = os.cpu_count() or 1
    BH = cfg["B"] * cfg["H"]
    heads_done, wall = 0, 0.0
    while heads_done < BH and wall * cores < budget_core_s:
        n = min(cores, BH - heads_done)
        wall += cpu_batch(ol, kind, cfg, n, cores, seed0=heads_done)
        heads_done += n
    return dict(value=flops(cfg, heads_done) / wall / 1e12, unit="TFLOP/s", cores=cores, kind=kind,
                sample=f"{heads_done} of {BH} (b,h) slices of {cfg['name']}, fwd+bwd, one slice per thread, "
                       f"{wall:.2f} s wall" + ("" if heads_done == BH else " (bounded sample; slices are independent and equal-cost)"))


def run_reference(args, cfg, rank, world):
    if rank != 0:
        return
    ol, kind = _cpu_lib()
    cores = os.cpu_count() or 1
    BH = cfg["B"] * cfg["H"]
    heads = min(cores, BH)
    # keep a step near a second of wall time on long sequences
    for _ in range(args.warmup):
        cpu_batch(ol, kind, cfg, heads, cores)
    t = [cpu_batch(ol, kind, cfg, heads, cores, seed0=17 * i) for i in range(args.steps)]
    wall = sum(t)
    value = flops(cfg, heads) * args.steps / wall / 1e12
    sample = f"each step = {heads} of {BH} (b,h) slices of {cfg['name']}, fwd+bwd, one slice per thread"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": wall / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 (f64 accumulate)", "data": "synthetic",
        "config": {"workload": cfg["name"], "config_id": args.config},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and clock-event reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml as nv

            nv.nvmlInit()
            self.nv, self.h = nv, nv.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.001)

    def start(self):
        if self.nv is not None:
            self._t = threading.Thread(target=self._loop, daemon=True)
            self._t.start()

    def stop(self):
        self._stop.set()
        if self._t is not None:
            self._t.join()
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
def _median(xs):
    s = sorted(xs)
    n = len(s)
    return s[n // 2] if n % 2 else 0.5 * (s[n // 2 - 1] + s[n // 2])


class Problem:
    """Device tensors of one rank's batch of a config, the two C-ABI calls on them, and the same step captured in
    a CUDA graph."""

    def __init__(self, cfg, config_id, seed, bh_pos0=0, dropout_seed=0x5EED0000):
        import torch

        import hyperkernels_b200 as hk

        self.hk, self.torch, self.cfg = hk, torch, cfg
        B, H, N = cfg["B"], cfg["H"], cfg["N"]
        g = torch.Generator(device="cuda").manual_seed(seed)
        self.shape = (B, H, N, 64)
        self.Q, self.K, self.V = (torch.randn(self.shape, generator=g, device="cuda") * cfg["sigma"] for _ in range(3))
        self.dO = torch.randn(self.shape, generator=g, device="cuda")
        if config_id == 5:
            self.K[:, :, ::64] *= 8.0
        self.O, self.dQ, self.dK, self.dV = (torch.empty(self.shape, device="cuda") for _ in range(4))
        self.LSE, self.D = (torch.empty((B, H, N), device="cuda") for _ in range(2))
        self.ws = torch.empty(4 * B * H * N * 256 + 512, dtype=torch.uint8, device="cuda")
        # one Philox stream for the whole job: a rank that holds a slice of the batch passes the index of its first
        # (batch, head) slice, so that any partition draws the mask of the unpartitioned problem
        self.drop = (dict(dropout_p=cfg["p"], philox_seed=dropout_seed, philox_offset=0, bh_pos0=bh_pos0)
                     if cfg["p"] > 0 else {})
        self.graph = None

    def forward(self):
        self.hk.attention_forward(self.Q, self.K, self.V, 0.125, self.cfg["causal"], workspace=self.ws, out=self.O,
                                  lse=self.LSE, **self.drop)

    def backward(self):
        self.hk.attention_backward(self.Q, self.K, self.V, self.O, self.dO, self.LSE, 0.125, self.cfg["causal"],
                                   workspace=self.ws, D=self.D, dQ=self.dQ, dK=self.dK, dV=self.dV, reuse_fwd_rounded=True,
                                   **self.drop)

    def step(self):
        self.forward()
        self.backward()

    def capture(self):
        drop = {k: v for k, v in self.drop.items() if k != "bh_pos0"}
        # GraphedAttentionStep captures exactly these two calls on its own output buffers
        self.graph = self.hk.GraphedAttentionStep(self.Q, self.K, self.V, self.dO, 0.125, self.cfg["causal"],
                                                  bh_pos0=self.drop.get("bh_pos0", 0), **drop)
        return self.graph


def timed_samples(fn, n, flush, stream, torch):
    """n samples of fn() in ms, a 256 MiB write (untimed) before each so that the inputs come from HBM."""
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
    for a, b in ev:
        flush.zero_()
        a.record(stream)
        fn()
        b.record(stream)
    torch.cuda.synchronize()
    return [a.elapsed_time(b) for a, b in ev]


def kernel_times(L, C):
    kt = {}
    for kind, name in ((0, "fwd"), (1, "bwd")):
        tot, n = C.c_double(), C.c_int()
        L.hk_attn_kernel_timing_read(kind, C.byref(tot), C.byref(n))
        kt[name] = (tot.value, n.value)
    return kt


def run_ours(args, cfg, rank, local_rank, world):
    import ctypes as C

    import torch

    import hyperkernels_b200 as hk

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the attention kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_

        dist = dist_
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    L = hk.lib()
    stream = torch.cuda.current_stream()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # > 126 MB of L2
    strong = args.scaling == "strong" and world > 1
    prob = Problem(cfg, args.config, 1000 + rank, bh_pos0=(rank * cfg["B"] * cfg["H"] if strong else 0),
                   dropout_seed=0x5EED0000 + (0 if strong else rank))
    B, H, N = cfg["B"], cfg["H"], cfg["N"]

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    warm = max(args.warmup, 3)
    for _ in range(warm):
        flush.zero_()
        prob.step()
    barrier()
    assert hk.last_device_status() == 0, "a bounded wait inside a kernel gave up during warm-up"

    # ---- device-resident timing -------------------------------------------------
    # The step = the launches of hk_attn_forward + hk_attn_backward, captured once in a CUDA graph
    # (hyperkernels_b200.GraphedAttentionStep) and replayed: the same four kernels without the gaps between
    # dependent launches.  Every driver step is `inner` replays, each timed by its own pair of events after an
    # untimed L2 flush, so that the timed region covers at least ~0.2 s of kernels; the step time is the MEDIAN of
    # all samples (the mean is reported beside it).
    gstep = prob.capture()
    est = _median(timed_samples(gstep.replay, 5, flush, stream, torch))
    inner = args.inner if args.inner > 0 else max(1, min(200, int(math.ceil(0.2 / max(args.steps * est * 1e-3, 1e-9)))))
    barrier()
    clocks = ClockSampler(local_rank)
    clocks.start()  # sampled from here to the end of the end-to-end loop
    t_wall = time.perf_counter()
    samples = timed_samples(gstep.replay, args.steps * inner, flush, stream, torch)
    barrier()
    t_wall = time.perf_counter() - t_wall
    launches_per_step = int(gstep.launches_per_replay)
    launches = launches_per_step * args.steps * inner
    ms, ms_mean = _median(samples), sum(samples) / len(samples)
    assert hk.last_device_status() == 0, "a bounded wait inside a kernel gave up"

    # the same steps issued launch by launch: forward call and backward call timed separately (bwd = everything
    # hk_attn_backward launches: D pre-pass with dO rounding and dQ zeroing + the main kernel; fwd = the rounding
    # pre-pass of Q, K, V + the main kernel), and the library's own events round the two tensor-core kernels
    n_e = max(args.steps, 10)
    L.hk_attn_kernel_timing_enable(1)
    fwd_s = timed_samples(prob.forward, n_e, flush, stream, torch)
    bwd_s = []
    for _ in range(n_e):
        flush.zero_()
        prob.forward()
        bwd_s += timed_samples(prob.backward, 1, torch.empty(0, dtype=torch.uint8, device="cuda"), stream, torch)
    L.hk_attn_kernel_timing_enable(0)
    kt = kernel_times(L, C)
    k_fwd, k_bwd = kt["fwd"][0] / max(kt["fwd"][1], 1), kt["bwd"][0] / max(kt["bwd"][1], 1)
    ms_fwd_call, ms_bwd_call = _median(fwd_s), _median(bwd_s)
    ms_eager = _median(timed_samples(prob.step, n_e, flush, stream, torch))
    # back to back, no flush (the reference reports flushed numbers; this one is extra)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(n_e):
        gstep.replay()
    e1.record(stream)
    torch.cuda.synchronize()
    ms_hot = e0.elapsed_time(e1) / n_e
    assert hk.last_device_status() == 0, "a bounded wait inside a kernel gave up"

    # ---- end to end through the C ABI with host buffers ----------------------------
    Q, K, V, dO, O, LSE, dQ, dK, dV = prob.Q, prob.K, prob.V, prob.dO, prob.O, prob.LSE, prob.dQ, prob.dK, prob.dV
    hQ, hK, hV, hdO = (t.cpu().pin_memory() for t in (Q, K, V, dO))
    hO, hdQ, hdK, hdV = (torch.empty(prob.shape).pin_memory() for _ in range(4))
    hLSE = torch.empty((B, H, N)).pin_memory()
    h2d = 4 * Q.numel() * 4
    d2h = 4 * Q.numel() * 4 + LSE.numel() * 4

    def e2e_sequential():
        Q.copy_(hQ, non_blocking=True); K.copy_(hK, non_blocking=True)
        V.copy_(hV, non_blocking=True); dO.copy_(hdO, non_blocking=True)
        prob.step()
        hO.copy_(O, non_blocking=True); hLSE.copy_(LSE, non_blocking=True)
        hdQ.copy_(dQ, non_blocking=True); hdK.copy_(dK, non_blocking=True); hdV.copy_(dV, non_blocking=True)

    # the host-buffer call of the package: batch chunks, copies of one chunk under the kernels of another
    host_step = hk.HostAttentionStep(B, H, N, 0.125, cfg["causal"],
                                     **({"dropout_p": cfg["p"], "philox_seed": prob.drop["philox_seed"]} if cfg["p"] > 0 else {}))

    def e2e_pipelined():
        host_step.step(hQ, hK, hV, hdO, hO, hLSE, hdQ, hdK, hdV)

    def time_e2e(fn):
        for _ in range(2):
            fn()
        barrier()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for a, b in evs:
            a.record(stream)
            fn()
            b.record(stream)
        barrier()
        return _median([a.elapsed_time(b) for a, b in evs])

    ms_e2e_seq = time_e2e(e2e_sequential)
    ms_e2e = time_e2e(e2e_pipelined)
    assert hk.last_device_status() == 0, "a bounded wait inside a kernel gave up"
    clk = clocks.stop()
    del hQ, hK, hV, hdO, hO, hdQ, hdK, hdV, hLSE, host_step

    # ---- the two multi-GPU configs, measured in the same run -------------------------
    extra = {}
    if dist is not None and not args.no_multi_gpu_configs:
        del prob, gstep
        torch.cuda.empty_cache()
        extra["strong_cfg4"] = strong_cfg4(args, rank, world, dist, flush, stream)
        extra["ring_cfg5"] = ring_cfg5(args, rank, local_rank, world, dist, flush, stream)

    if dist is not None:
        t = torch.tensor([ms, ms_e2e, k_fwd, k_bwd, ms_e2e_seq, ms_eager, ms_fwd_call, ms_bwd_call, ms_mean], device="cuda",
                         dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e, k_fwd, k_bwd, ms_e2e_seq, ms_eager, ms_fwd_call, ms_bwd_call, ms_mean = (float(x) for x in t.tolist())
    if rank == 0:
        peaks = measured_peaks()
        total = flops(cfg) * world
        f_fwd, f_bwd = flops(cfg, bwd=False), flops(cfg, fwd=False)
        achieved = f_bwd / (k_bwd * 1e-3) / 1e12 if k_bwd > 0 else None
        line = {
            "metric": METRIC, "value": total / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "tf32", "data": "synthetic",
            "config": {"workload": cfg["name"] + (" per GPU" if world > 1 and args.scaling == "weak" else ""),
                       "config_id": args.config,
                       "l2": "256 MiB buffer written before every timed sample (untimed)",
                       "step": "hk_attn_forward + hk_attn_backward with every launch they make (operand rounding to TF32: in shared memory inside the kernels for 512 <= N <= 2048 causal / 1024 otherwise, else one HBM pre-pass per step; D pre-pass with dO rounding and dQ zeroing; the two main kernels), captured in a CUDA graph and replayed",
                       "launches_per_step": launches_per_step,
                       "timing": f"median of {len(samples)} samples ({args.steps} steps x {inner} replays), one CUDA-event pair per replay",
                       "partition": "batch x head across GPUs, no collective"},
            "ms_per_step_mean": ms_mean,
            "pct_of_tf32_peak": total / world / (ms * 1e-3) / 1e12 / peaks["tf32_tflops"],
            "fwd_tflops": f_fwd / (ms_fwd_call * 1e-3) / 1e12, "bwd_tflops": f_bwd / (ms_bwd_call * 1e-3) / 1e12,
            "call_ms": {"hk_attn_forward": ms_fwd_call, "hk_attn_backward": ms_bwd_call,
                        "note": "every launch of the call: fwd = Q/K/V rounding pre-pass (if the config takes the HBM path) + forward kernel; bwd = D pre-pass (dO rounding, dQ zeroing) + backward kernel"},
            "kernel_ms": {"fwd_kernel": k_fwd, "bwd_kernel": k_bwd,
                          "fwd_kernel_tflops": f_fwd / (k_fwd * 1e-3) / 1e12 if k_fwd else None,
                          "bwd_kernel_tflops": achieved},
            "roofline": {"bound": "tensor", "kernel": "attn_bwd_kernel", "achieved": achieved,
                         "peak": peaks["tf32_tflops"], "unit": "TFLOP/s",
                         "frac": (achieved / peaks["tf32_tflops"]) if achieved else None,
                         "peak_source": peaks["source"],
                         "peak_mma_probe": MMA_MIX_PROBE_TFLOPS,
                         "frac_of_mma_probe": (achieved / MMA_MIX_PROBE_TFLOPS) if achieved else None,
                         "traffic": ncu_traffic("attn_bwd_kernel", args.config)},
            "e2e": {"value": total / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e,
                    "call": "hyperkernels_b200.HostAttentionStep.step: pinned host tensors in and out, chunks of (batch, head) slices, "
                            "H2D / kernels / D2H of different chunks overlapped on three streams",
                    "sequential": {"value": total / (ms_e2e_seq * 1e-3) / 1e12, "ms_per_step": ms_e2e_seq,
                                   "call": "copy in, hk_attn_forward + hk_attn_backward, copy out on one stream"}},
            "gpu_launches": int(launches),
            "clocks": clk,
            "wall_s_timed_region": t_wall,
            "ms_per_step_launch_by_launch": ms_eager,
            "ms_per_step_back_to_back_no_flush": ms_hot,
        }
        line.update(extra)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(cfg)
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def _single_gpu_reference(cfg, config_id, flush, stream, n=5):
    """ms per step of the WHOLE config on this one GPU (graph replay, median), for the efficiency of a sharded run."""
    import torch

    prob = Problem(cfg, config_id, 4242)
    for _ in range(2):
        prob.step()
    g = prob.capture()
    ms = _median(timed_samples(g.replay, n, flush, stream, torch))
    del prob, g
    torch.cuda.empty_cache()
    return ms


def strong_cfg4(args, rank, world, dist, flush, stream):
    """Config 4 (B=32, H=25, N=1024, causal, p=0.1), its batch split evenly over the ranks: no collective, one Philox
    stream for the whole job (bh_pos0 = the rank's first slice).  Efficiency = (whole config on one GPU) / (N x this)."""
    import torch

    import hyperkernels_b200 as hk

    full = dict(CONFIGS[4])
    assert full["B"] % world == 0
    cfg = dict(full, B=full["B"] // world)
    prob = Problem(cfg, 4, 4000 + rank, bh_pos0=rank * cfg["B"] * cfg["H"])
    for _ in range(3):
        prob.step()
    g = prob.capture()
    torch.cuda.synchronize()
    dist.barrier()
    ms = _median(timed_samples(g.replay, 15, flush, stream, torch))
    del prob, g
    torch.cuda.empty_cache()
    ms1 = _single_gpu_reference(full, 4, flush, stream) if rank == 0 else 0.0
    t = torch.tensor([ms, ms1], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms1 = (float(x) for x in t.tolist())
    assert hk.last_device_status() == 0
    return {"workload": full["name"] + f", batch split over {world} GPUs", "scaling": "strong",
            "value": flops(full) / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms,
            "single_gpu_ms_per_step": ms1, "single_gpu_value": flops(full) / (ms1 * 1e-3) / 1e12,
            "efficiency": ms1 / (world * ms), "collective": "none", "timing": "median of 15 graph replays, max over ranks"}


# --ring-graph: replay the ring step from a CUDA graph.  Off by default: on 2- and 4-rank rings the captured step
# measured the same as the call-by-call one (14.51 against 14.54 ms on a 4-rank ring: the step is bound by the GPU side)
RING_GRAPH = False


def _captured_ring_step(ring, Q, K, V, dO, eager_step, dist, torch):
    """The ring step as one CUDA-graph launch per rank (hyperkernels_b200.ring.GraphedRingStep) if every rank could
    capture it, else the call-by-call step on every rank."""
    from hyperkernels_b200.ring import GraphedRingStep

    gs, ok = None, 1
    try:
        if not RING_GRAPH:
            raise RuntimeError("--ring-graph not given")
        gs = GraphedRingStep(ring, Q, K, V, dO)
    except Exception as e:  # capture is all-or-nothing over the ranks: NCCL operations must match
        if RING_GRAPH:
            print(f"bench: ring step not captured ({e}); issuing it call by call", file=sys.stderr)
        ok = 0
    flag = torch.tensor([ok], device="cuda", dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if int(flag.item()) == 1:
        return gs.replay, "one CUDA-graph launch per rank and step (kernels, NCCL hops and their ordering captured)"
    return eager_step, "call by call from Python"


def ring_cfg5(args, rank, local_rank, world, dist, flush, stream, Gs=2):
    """Config 5 (B=1, H=32, N=32768, causal, every 64th key x8): heads split over world/Gs groups, the sequence of each
    group sharded over a Gs-rank KV ring (zigzag chunks, NCCL send/recv on a side stream under the compute)."""
    import ctypes as C

    import torch

    import hyperkernels_b200 as hk
    from hyperkernels_b200.ring import RingAttention, segments_of

    L = hk.lib()
    full = dict(CONFIGS[5])
    Gh = world // Gs
    assert world % Gs == 0 and full["H"] % Gh == 0
    groups = [dist.new_group(list(range(g * Gs, (g + 1) * Gs))) for g in range(Gh)]
    group, srank = groups[rank // Gs], rank % Gs
    Hl, N = full["H"] // Gh, full["N"]
    segs = segments_of(srank, Gs, N, "zigzag")
    gen = torch.Generator(device="cuda").manual_seed(2000 + rank)
    shape = (full["B"], Hl, N // Gs, 64)
    Q, K, V, dO = (torch.randn(shape, generator=gen, device="cuda") for _ in range(4))
    off = 0
    for (s0, n) in segs:  # every 64th key of the GLOBAL sequence scaled x8
        K[:, :, off + ((-s0) % 64):off + n:64] *= 8.0
        off += n
    ring = RingAttention(N, 0.125, True, group=group, layout="zigzag")
    out = {}

    def step():
        out["O"], out["LSE"] = ring.forward(Q, K, V)
        out["dQ"], out["dK"], out["dV"] = ring.backward(Q, K, V, out["O"], out["LSE"], dO)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    n0 = hk.launch_count()
    step()
    launches = hk.launch_count() - n0
    run, how = _captured_ring_step(ring, Q, K, V, dO, step, dist, torch)
    for _ in range(2):
        run()
    torch.cuda.synchronize()
    dist.barrier()
    samples = timed_samples(run, 8, flush, stream, torch)
    ms = _median(samples)
    # second pass with the library's kernel events on: how much of the step the two tensor-core kernels are busy
    L.hk_attn_kernel_timing_enable(1)
    timed_samples(step, 3, flush, stream, torch)
    L.hk_attn_kernel_timing_enable(0)
    kt = kernel_times(L, C)
    busy = (kt["fwd"][0] + kt["bwd"][0]) / 3.0
    assert hk.last_device_status() == 0
    del Q, K, V, dO, out, ring
    torch.cuda.empty_cache()
    ms1 = _single_gpu_reference(full, 5, flush, stream, n=3) if rank == 0 else 0.0
    t = torch.tensor([ms, ms1, busy], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms1, busy = (float(x) for x in t.tolist())
    return {"workload": full["name"], "scaling": "strong", "mesh": f"{Gh} head groups x {Gs}-rank KV ring (zigzag)",
            "value": flops(full) / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms,
            "single_gpu_ms_per_step": ms1, "single_gpu_value": flops(full) / (ms1 * 1e-3) / 1e12,
            "efficiency": ms1 / (world * ms), "kernels_busy_frac": busy / ms, "launches_per_step": int(launches),
            "issue": how,
            "collective": "NCCL send/recv of K/V blocks and of the travelling dK/dV accumulators, one hop per ring step",
            "timing": "median of 8 steps (CUDA events), max over ranks"}


def run_ours_ring(args, cfg, rank, local_rank, world):
    """Config 5 on N > 1 GPUs: heads split over N / ring groups, the sequence of each group sharded over `ring`
    ranks with the KV ring of hyperkernels_b200/ring.py (NCCL send/recv overlapped with compute).  Strong scaling:
    the problem is the one config-5 problem whatever N is."""
    import ctypes as C

    import torch
    import torch.distributed as dist

    import hyperkernels_b200 as hk
    from hyperkernels_b200.ring import RingAttention, segments_of

    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    L = hk.lib()
    Gs = args.ring
    assert world % Gs == 0 and cfg["H"] % (world // Gs) == 0
    Gh = world // Gs
    groups = [dist.new_group(list(range(g * Gs, (g + 1) * Gs))) for g in range(Gh)]
    group = groups[rank // Gs]
    srank = rank % Gs
    Hl, N = cfg["H"] // Gh, cfg["N"]
    segs = segments_of(srank, Gs, N, "zigzag")
    gen = torch.Generator(device="cuda").manual_seed(2000 + rank)
    shape = (cfg["B"], Hl, N // Gs, 64)
    Q, K, V, dO = (torch.randn(shape, generator=gen, device="cuda") for _ in range(4))
    off = 0
    for (s0, n) in segs:  # every 64th key of the GLOBAL sequence scaled x8
        first = (-s0) % 64
        K[:, :, off + first:off + n:64] *= 8.0
        off += n
    ring = RingAttention(N, 0.125, True, group=group, layout="zigzag")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream()
    out = {}

    def step():
        out["O"], out["LSE"] = ring.forward(Q, K, V)
        out["dQ"], out["dK"], out["dV"] = ring.backward(Q, K, V, out["O"], out["LSE"], dO)

    def barrier():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    assert hk.last_device_status() == 0
    clocks = ClockSampler(local_rank)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    n0 = hk.launch_count()
    step()
    launches = (hk.launch_count() - n0) * args.steps
    run, how = _captured_ring_step(ring, Q, K, V, dO, step, dist, torch)
    for _ in range(2):
        run()
    barrier()
    clocks.start()
    for a, b in ev:
        flush.zero_()
        a.record(stream)
        run()
        b.record(stream)
    barrier()
    ms = sum(a.elapsed_time(b) for a, b in ev) / args.steps
    # second, untimed pass with the library's kernel events on (they cost two event creations per launch, which do
    # not belong in the timed region): how long the two tensor-core kernels run per step
    n_k = 2
    L.hk_attn_kernel_timing_enable(1)
    for _ in range(n_k):
        step()
    barrier()
    L.hk_attn_kernel_timing_enable(0)
    kt = {}
    for kind, name in ((0, "fwd"), (1, "bwd")):
        tot, n = C.c_double(), C.c_int()
        L.hk_attn_kernel_timing_read(kind, C.byref(tot), C.byref(n))
        kt[name] = tot.value / n_k  # all kernel launches of that kind in one step, summed
    hQ, hK, hV, hdO = (t.cpu().pin_memory() for t in (Q, K, V, dO))
    hout = {k: torch.empty(v.shape).pin_memory() for k, v in out.items()}

    def e2e_step():
        Q.copy_(hQ, non_blocking=True); K.copy_(hK, non_blocking=True)
        V.copy_(hV, non_blocking=True); dO.copy_(hdO, non_blocking=True)
        step()
        for k in hout:
            hout[k].copy_(out[k], non_blocking=True)

    e2e_step()
    barrier()
    ev2 = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for a, b in ev2:
        a.record(stream)
        e2e_step()
        b.record(stream)
    barrier()
    ms_e2e = sum(a.elapsed_time(b) for a, b in ev2) / args.steps
    clk = clocks.stop()
    t = torch.tensor([ms, ms_e2e, kt["fwd"], kt["bwd"]], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e, kt["fwd"], kt["bwd"] = (float(x) for x in t.tolist())
    if rank == 0:
        peaks = measured_peaks()
        total = flops(cfg)
        achieved = flops(cfg, fwd=False) / world / (kt["bwd"] * 1e-3) / 1e12 if kt["bwd"] > 0 else None
        print(json.dumps({
            "metric": METRIC, "value": total / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "tf32", "data": "synthetic",
            "config": {"workload": cfg["name"], "config_id": args.config, "mesh": f"{Gh} head groups x {Gs}-rank KV ring (zigzag)",
                       "l2": "256 MiB buffer written between timed steps (untimed)",
                       "step": "ring forward + ring backward (hk_attn_forward/backward per segment pair, NCCL send/recv)",
                       "issue": how},
            "pct_of_tf32_peak": total / world / (ms * 1e-3) / 1e12 / peaks["tf32_tflops"],
            "kernel_ms": {"fwd_kernels_per_step": kt["fwd"], "bwd_kernels_per_step": kt["bwd"]},
            "roofline": {"bound": "tensor", "kernel": "attn_bwd_kernel", "achieved": achieved, "peak": peaks["tf32_tflops"],
                         "unit": "TFLOP/s", "frac": (achieved / peaks["tf32_tflops"]) if achieved else None,
                         "peak_source": peaks["source"], "traffic": None},
            "e2e": {"value": total / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": 4 * Q.numel() * 4,
                    "d2h_bytes_per_step": sum(v.numel() for v in out.values()) * 4, "ms_per_step": ms_e2e},
            "gpu_launches": int(launches), "clocks": clk,
        }))
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", type=int, default=2, choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--inner", type=int, default=0,
                    help="graph replays per driver step (0: as many as make the timed region ~0.2 s); 1 for profiler runs")
    ap.add_argument("--no-multi-gpu-configs", action="store_true",
                    help="N > 1: skip the strong_cfg4 and ring_cfg5 sub-records")
    ap.add_argument("--ring", type=int, default=2, help="config 5 on N > 1 GPUs: ranks per sequence ring")
    ap.add_argument("--ring-graph", action="store_true", help="replay the ring step from a CUDA graph (GraphedRingStep)")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: every rank runs a whole batch of the config; strong: the config's batch is split over the ranks")
    args = ap.parse_args()
    global RING_GRAPH
    RING_GRAPH = bool(args.ring_graph)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cfg = dict(CONFIGS[args.config])
    if args.scaling == "strong" and world > 1 and args.config != 5:
        assert cfg["B"] % world == 0, "strong scaling splits the batch dimension evenly"
        cfg["B"] //= world
        cfg["name"] += f" split over {world} GPUs by batch"
    if args.impl == "reference":
        run_reference(args, cfg, rank, world)
    elif args.config == 5 and world > 1:
        run_ours_ring(args, cfg, rank, local_rank, world)
    else:
        run_ours(args, cfg, rank, local_rank, world)


if __name__ == "__main__":
    main()
