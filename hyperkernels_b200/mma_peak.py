"""Measures the TF32 tensor-pipe ceilings of this GPU for the MMA shapes the attention
kernels issue (C ABI: hk_attn_mma_peak), plus the library GEMM rates for scale.

    python -m hyperkernels_b200.mma_peak
"""
import ctypes as C

import torch

from . import lib, last_device_status

MODES = {
    0: "8 x M128 N128 K8, A and B K-major smem (S = Q K^T)",
    3: "same, alternating two accumulators",
    4: "M128 N256 K8, K-major smem",
    1: "16 x M128 N64 K8, A tensor memory, B MN-major smem (O = P V)",
    2: "16 x M128 N64 K8, A and B MN-major smem (dQ = dS K)",
}


def measure(mode: int, iters: int = 2000, ctas: int = 148) -> float:
    """TFLOP/s of `ctas` CTAs each issuing `iters` MMA groups of `mode`."""
    L = lib()
    L.hk_attn_mma_peak.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.POINTER(C.c_double), C.c_void_p]
    A = torch.randn(128, 64, device="cuda")
    B = torch.randn(128, 64, device="cuda")
    fl = C.c_double()
    s = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        L.hk_attn_mma_peak(mode, iters, ctas, A.data_ptr(), B.data_ptr(), C.byref(fl), s)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    rc = L.hk_attn_mma_peak(mode, iters, ctas, A.data_ptr(), B.data_ptr(), C.byref(fl), s)
    b.record()
    torch.cuda.synchronize()
    assert rc == 0 and last_device_status() == 0
    return fl.value / a.elapsed_time(b) / 1e9


def main():
    for mode, name in MODES.items():
        print(f"mode {mode}: {measure(mode, ctas=148):7.1f} / {measure(mode, ctas=296):7.1f} TFLOP/s (148 / 296 CTAs)  {name}")
    torch.backends.cuda.matmul.allow_tf32 = True
    for dt, label in ((torch.float32, "cuBLAS TF32"), (torch.bfloat16, "cuBLAS bf16")):
        x = torch.randn(8192, 8192, device="cuda", dtype=dt)
        y = torch.randn(8192, 8192, device="cuda", dtype=dt)
        for _ in range(3):
            x @ y
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(10):
            x @ y
        b.record()
        torch.cuda.synchronize()
        print(f"{label} 8192^3 (library, for scale): {2 * 8192 ** 3 * 10 / a.elapsed_time(b) / 1e9:7.1f} TFLOP/s")


if __name__ == "__main__":
    main()
