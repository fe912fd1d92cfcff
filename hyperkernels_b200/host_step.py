"""Forward + backward of HOST-resident tensors, with the copies overlapped.

The reference keeps its tensors on the host between launches
(``kernels/tests/kernels_test.cu:491-507`` copies Q, K, V in, ``:533-534`` copies
O and LSE out, around every kernel it tests).  A caller in that position pays
the PCIe transfer of four [B, H, T, 64] inputs and five outputs per training
step, which at these sizes is an order of magnitude more than the kernels.  The
(batch, head) slices of the problem are independent, so this helper cuts the
batch into chunks and runs three queues: chunk i+1 travels to the device while
the kernels work on chunk i and the results of chunk i-1 travel back (the two
copy directions use different DMA engines and the link is full duplex).  The
chunks are runs of consecutive (batch, head) slices, so a single-batch problem
with many heads is pipelined too; small problems (under 2 MB per tensor and
chunk) are not cut, the extra launches would cost more than the overlap gains.
The whole step -- every copy, every launch, the dependencies between the three
queues -- is captured in a CUDA graph the second time it is called with the same
host tensors and replayed from then on, so the host issues one call per step.

Everything on the device goes through the C ABI (``hk_attn_forward`` and
``hk_attn_backward`` per chunk, with preallocated buffers and workspace); torch
is used for pinned host memory, streams and events only.
"""
from __future__ import annotations

from typing import Optional

from . import attention as att


class HostAttentionStep:
    """One training step of attention for tensors that live in pinned host memory.

    ``step(hQ, hK, hV, hdO, hO, hLSE, hdQ, hdK, hdV)``: inputs and outputs are pinned fp32 host tensors,
    [B, H, T, 64] (LSE: [B, H, T]).  The call enqueues everything and returns; the caller's current stream waits for
    the last result copy, so a ``torch.cuda.synchronize()`` (or an event on that stream) marks completion.

    With Philox dropout every chunk passes the index of its first (batch, head) slice (``bh_pos0``) with the same
    seed and offset, so the keep-mask of a chunked step is the one a single call over the whole batch draws.
    """

    def __init__(self, B: int, H: int, T: int, scale: float, causal: bool, *, chunks: Optional[int] = None,
                 n_slots: int = 3, graph: bool = True, device=None, dropout_p: float = 0.0, philox_seed: Optional[int] = None, philox_offset: int = 0):
        import torch

        self.torch = torch
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        n = B * H  # independent slices; a chunk is a run of them, handed to the kernels as a batch of one-head items
        # chunk sizes in slices: by default up to eight equal chunks of at least 2 MB per tensor (every copy costs a fixed
        # ~10 us on its engine; schedules with small chunks at both ends and large ones in the middle measured slower
        # than equal chunks: 2.92-3.02 against 2.61 ms at B8 H12 T1024)
        if chunks is None:
            c = next(c for c in (8, 4, 2, 1) if n % c == 0 and (c == 1 or n // c * T * 256 >= (2 << 20)))
            sizes = [n // c] * c
        elif isinstance(chunks, int):
            if chunks <= 0 or n % chunks != 0:
                raise ValueError("batch x heads must divide into equal chunks")
            sizes = [n // chunks] * chunks
        else:
            sizes = [int(x) for x in chunks]
            if any(x <= 0 for x in sizes) or sum(sizes) != n:
                raise ValueError("chunk sizes must be positive and add up to batch x heads")
        self.B, self.H, self.T, self.scale, self.causal = B, H, T, float(scale), bool(causal)
        self.sizes = sizes
        self.starts = [sum(sizes[:i]) for i in range(len(sizes))]
        chunks = len(sizes)
        self.chunks, self.cb = chunks, max(sizes)
        self.drop = {}
        if dropout_p > 0:
            if philox_seed is None:
                raise ValueError("dropout on this path uses the Philox mask: give philox_seed")
            self.drop = dict(dropout_p=dropout_p, philox_seed=philox_seed)
        self.philox_offset = philox_offset
        shp, lshp = (self.cb, 1, T, 64), (self.cb, 1, T)
        n_slots = max(1, min(n_slots, chunks))
        self.slots = []
        for _ in range(n_slots):
            s = {k: torch.empty(shp, dtype=torch.float32, device=self.device)
                 for k in ("Q", "K", "V", "dO", "O", "dQ", "dK", "dV")}
            s["LSE"] = torch.empty(lshp, dtype=torch.float32, device=self.device)
            s["D"] = torch.empty(lshp, dtype=torch.float32, device=self.device)
            s["ws"] = torch.empty(4 * self.cb * T * 256 + 512, dtype=torch.uint8, device=self.device)
            self.slots.append(s)
        self.s_in, self.s_cmp, self.s_out = (torch.cuda.Stream(device=self.device) for _ in range(3))
        self.ev_start = torch.cuda.Event()
        self.ev_in = [torch.cuda.Event() for _ in range(chunks)]
        self.ev_cmp = [torch.cuda.Event() for _ in range(chunks)]
        self.ev_out = [torch.cuda.Event() for _ in range(chunks)]
        self.use_graph = bool(graph)
        self._seen_key = None    # host tensors of the last eager step
        self._graph_key = None   # host tensors the captured graph copies from / to
        self._graph = None
        self.h2d_bytes = 4 * B * H * T * 64 * 4
        self.d2h_bytes = 4 * B * H * T * 64 * 4 + B * H * T * 4

    def step(self, hQ, hK, hV, hdO, hO, hLSE, hdQ, hdK, hdV) -> None:
        torch = self.torch
        args = (hQ, hK, hV, hdO, hO, hLSE, hdQ, hdK, hdV)
        if not self.use_graph:
            return self._enqueue(*args)
        key = tuple(int(t.data_ptr()) for t in args)
        if key == self._graph_key:
            self._graph.replay()  # on the caller's current stream
            return
        if key != self._seen_key:
            # first step with these tensors: issue it call by call (first-call set-up of the library happens here)
            self._seen_key = key
            return self._enqueue(*args)
        # second step with the same tensors: capture it, then run the capture
        cur = torch.cuda.current_stream(self.device)
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(cur)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                self._enqueue(*args)
        cur.wait_stream(side)
        self._graph, self._graph_key = g, key
        self._keep = args  # the graph holds raw pointers into these tensors
        g.replay()

    def _enqueue(self, hQ, hK, hV, hdO, hO, hLSE, hdQ, hdK, hdV) -> None:
        torch = self.torch
        n = self.B * self.H
        # [B, H, ...] contiguous == [B*H, 1, ...]
        hQ, hK, hV, hdO, hO, hdQ, hdK, hdV = (x.view(n, 1, self.T, 64) for x in (hQ, hK, hV, hdO, hO, hdQ, hdK, hdV))
        hLSE = hLSE.view(n, 1, self.T)
        cur = torch.cuda.current_stream(self.device)
        self.ev_start.record(cur)
        for s in (self.s_in, self.s_cmp, self.s_out):
            s.wait_event(self.ev_start)
        n_slots = len(self.slots)
        for i in range(self.chunks):
            full = self.slots[i % n_slots]
            m = self.sizes[i]
            d = {k: (v if k == "ws" else v[:m]) for k, v in full.items()}  # this chunk's part of the slot's buffers
            sl = slice(self.starts[i], self.starts[i] + m)
            with torch.cuda.stream(self.s_in):
                if i >= n_slots:  # the kernels of the chunk that used this slot have read its inputs
                    self.s_in.wait_event(self.ev_cmp[i - n_slots])
                d["Q"].copy_(hQ[sl], non_blocking=True)
                d["K"].copy_(hK[sl], non_blocking=True)
                d["V"].copy_(hV[sl], non_blocking=True)
                d["dO"].copy_(hdO[sl], non_blocking=True)
                self.ev_in[i].record(self.s_in)
            with torch.cuda.stream(self.s_cmp):
                self.s_cmp.wait_event(self.ev_in[i])
                if i >= n_slots:  # the results of the chunk that used this slot have left
                    self.s_cmp.wait_event(self.ev_out[i - n_slots])
                drop = dict(self.drop, philox_offset=self.philox_offset, bh_pos0=self.starts[i]) if self.drop else {}
                att.attention_forward(d["Q"], d["K"], d["V"], self.scale, self.causal, workspace=d["ws"], out=d["O"],
                                      lse=d["LSE"], stream=self.s_cmp, **drop)
                att.attention_backward(d["Q"], d["K"], d["V"], d["O"], d["dO"], d["LSE"], self.scale, self.causal,
                                       workspace=d["ws"], D=d["D"], dQ=d["dQ"], dK=d["dK"], dV=d["dV"],
                                       reuse_fwd_rounded=True, stream=self.s_cmp, **drop)
                self.ev_cmp[i].record(self.s_cmp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_cmp[i])
                hO[sl].copy_(d["O"], non_blocking=True)
                hLSE[sl].copy_(d["LSE"], non_blocking=True)
                hdQ[sl].copy_(d["dQ"], non_blocking=True)
                hdK[sl].copy_(d["dK"], non_blocking=True)
                hdV[sl].copy_(d["dV"], non_blocking=True)
                self.ev_out[i].record(self.s_out)
        cur.wait_event(self.ev_out[self.chunks - 1])
        cur.wait_event(self.ev_cmp[self.chunks - 1])
