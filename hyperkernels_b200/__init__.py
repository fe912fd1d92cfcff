"""B200-native (sm_100a) fused attention forward/backward behind the launch
surface of BlubridgeAI/HyperKernels' ``kernels/attention``.

The compute lives in ``lib/libhk_attention.so`` (built from ``csrc/``); this
package is the thin host-side mirror of the reference's by-value argument blocks
and launches.  There is no CPU fallback: importing works anywhere, but every
compute call needs the compiled library and a CUDA device.
"""
from .attention import (  # noqa: F401
    HKError,
    MemEfficientBwdParams,
    MemEfficientFwdParams,
    attention_backward,
    attention_forward,
    bwd_workspace_bytes,
    dropout_keep_mask,
    fused_attn_forward,
    fwd_workspace_bytes,
    last_device_status,
    launch_count,
    lib,
    mem_efficient_bwd_precompute_D,
    mem_efficient_bwd_unified,
    merge_partial,
    round_tf32,
    FLAG_PHILOX_DROPOUT,
    FLAG_OPERANDS_PREROUNDED,
    FLAG_ACCUM_DKDV,
    FLAG_ACCUM_DQ,
    FLAG_D_PRECOMPUTED,
    FLAG_REUSE_FWD_ROUNDED,
    FLAG_DROPOUT_SCALED,
    FLAG_CONTINUE_SOFTMAX_STATE,
    FLAG_ROUND_IN_HBM,
    FLAG_DETERMINISTIC_DQ,
)
from .graph_step import GraphedAttentionStep  # noqa: F401
from .host_step import HostAttentionStep  # noqa: F401
