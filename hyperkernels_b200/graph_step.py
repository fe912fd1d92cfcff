"""Forward + backward captured once in a CUDA graph and replayed.

A training step of the attention path is four launches (TF32 rounding pre-pass,
forward, D pre-pass with dO rounding and dQ zeroing, backward).  At small sizes
the gaps between dependent launches are a large part of the step (B=2, H=4,
T=256: 0.064 ms issued launch by launch, 0.033 ms replayed from a graph); at
B=8, H=12, T=1024 the graph saves about 2 %.  The graph holds exactly the
launches the two C-ABI calls make: capture goes through ``hk_attn_forward`` and
``hk_attn_backward`` on a side stream after one eager warm-up step (which sets
the kernels' attributes and resolves the library's device symbols -- neither is
allowed during capture).
"""
from __future__ import annotations

from typing import Optional

from . import attention as att


class GraphedAttentionStep:
    """``O, LSE = fwd(Q, K, V)`` and ``dQ, dK, dV = bwd(dO)`` on fixed device buffers.

    The graph reads ``Q, K, V, dO`` (the tensors given here: refill them in place between replays) and writes
    ``self.O, self.LSE, self.dQ, self.dK, self.dV, self.D``.  With Philox dropout the seed and offset are frozen
    into the graph: every replay draws the same mask; capture again for a new one.
    """

    def __init__(self, Q, K, V, dO, scale: float, causal: bool, *, dropout_p: float = 0.0,
                 philox_seed: Optional[int] = None, philox_offset: int = 0, dropout_scaled: bool = False,
                 bh_pos0: int = 0):
        import torch

        B, H, T, _ = Q.shape
        Tk = K.shape[2]
        dev = Q.device
        self.Q, self.K, self.V, self.dO = Q, K, V, dO
        self.O = torch.empty((B, H, T, 64), dtype=torch.float32, device=dev)
        self.dQ = torch.empty((B, H, T, 64), dtype=torch.float32, device=dev)
        self.dK = torch.empty((B, H, Tk, 64), dtype=torch.float32, device=dev)
        self.dV = torch.empty((B, H, Tk, 64), dtype=torch.float32, device=dev)
        self.LSE = torch.empty((B, H, T), dtype=torch.float32, device=dev)
        self.D = torch.empty((B, H, T), dtype=torch.float32, device=dev)
        self._ws = torch.empty(2 * B * H * (T + Tk) * 256 + 1024, dtype=torch.uint8, device=dev)
        drop = {}
        if dropout_p > 0:
            if philox_seed is None:
                raise ValueError("dropout in a captured step uses the Philox mask: give philox_seed")
            drop = dict(dropout_p=dropout_p, philox_seed=philox_seed, philox_offset=philox_offset,
                        dropout_scaled=dropout_scaled, bh_pos0=bh_pos0)

        def step():
            att.attention_forward(Q, K, V, scale, causal, workspace=self._ws, out=self.O, lse=self.LSE, **drop)
            att.attention_backward(Q, K, V, self.O, dO, self.LSE, scale, causal, workspace=self._ws, D=self.D,
                                   dQ=self.dQ, dK=self.dK, dV=self.dV, reuse_fwd_rounded=True, **drop)

        n0 = att.launch_count()
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            step()  # eager: first-call set-up happens here, outside the capture
            self.launches_per_replay = att.launch_count() - n0
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                step()
        torch.cuda.current_stream(dev).wait_stream(side)

    def replay(self) -> None:
        """Enqueue one step on the current stream."""
        self.graph.replay()
