"""CUDA graphs for decode steps.

A decode step launches a few hundred small kernels; launched one by one from
the host they take several times longer than they run.  For each batch-size
bucket (powers of two) the whole forward pass of a one-token-per-sequence step
is captured once into a CUDA graph over fixed input buffers (token ids,
positions, slots) and replayed afterwards.  Everything that changes from step
to step is read by the kernels from device memory: positions and slots from
the input buffers, pages from the cache's block tables.  Rows beyond the live
batch are padding (slot -1): they write nothing to the cache and their
outputs are dropped.

Upstream launches every kernel from the host and allocates inside the loop
(src/models/qwen3/qwen3.cpp:263-288, src/src-cuda/simple-ops/simple-ops.cu:58).
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..ops import counters, kernels
from ..parts import StepContext


def bucket_for(n: int, largest: int) -> Optional[int]:
    b = 1
    while b < n:
        b *= 2
    return b if b <= largest else None


class _Captured:
    def __init__(self, size: int, device):
        self.size = size
        self.ints = torch.zeros(3 * size, dtype=torch.int32, device=device)      # tokens | positions | slots
        self.ints[2 * size:] = -1
        self.host = torch.zeros(3 * size, dtype=torch.int32).pin_memory()        # the same, staged
        self.host_np = self.host.numpy()
        self.want = torch.arange(size, dtype=torch.int32, device=device)
        self.event: Optional[torch.cuda.Event] = None
        self.graph = torch.cuda.CUDAGraph()
        self.logits: Optional[torch.Tensor] = None
        self.n_kernels = 0

    @property
    def tokens(self):
        return self.ints[:self.size]

    def context(self, status) -> StepContext:
        s = self.size
        return StepContext(n_tokens=s, tokens=self.ints[:s], tok_pos=self.ints[s:2 * s], tok_slot=self.ints[2 * s:],
                           seq_slots=[], seq_starts=[], seq_lens=[], seq_past=[], all_single=True, max_kv_len=0,
                           status=status, captured=True)


class DecodeGraphs:
    """Captured decode steps of one engine, one per batch-size bucket."""

    def __init__(self, model, cache, largest_bucket: int = 256):
        self.model, self.cache = model, cache
        self.largest = largest_bucket
        self._graphs: dict[int, _Captured] = {}
        self._pool = None
        self.bytes_uploaded = 0

    def _capture(self, size: int) -> _Captured:
        cap = _Captured(size, self.cache.device)
        ctx = cap.context(self.cache.status)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):                    # all rows are padding: the cache is not touched
            for _ in range(2):
                self.model.forward(ctx, self.cache, cap.want)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        before = counters.launches
        # a recorded step lets each kernel be launched while the one before it still runs: what a kernel reads
        # that no kernel of the step writes (weights, positions, the cache of earlier steps) is on its way by then
        kernels.set_dependent_launch(True)
        try:
            with torch.cuda.graph(cap.graph, pool=self._pool):
                cap.logits = self.model.forward(ctx, self.cache, cap.want)
        finally:
            kernels.set_dependent_launch(False)
        cap.n_kernels = counters.launches - before
        counters.launches = before                        # capturing launches nothing
        return cap

    def run(self, slots: list[int], past: list[int], tokens_host: Optional[np.ndarray],
            tokens_dev: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Replay the bucket's graph for these slots; returns logits [len(slots), vocab] (a copy), or None
        when the batch is larger than the largest bucket."""
        n = len(slots)
        size = bucket_for(n, self.largest)
        if size is None:
            return None
        cap = self._graphs.get(size)
        if cap is None:
            cap = self._graphs[size] = self._capture(size)
        if cap.event is not None:
            cap.event.synchronize()
        h = cap.host_np
        h[size:size + n] = past
        h[size + n:2 * size] = 0
        h[2 * size:2 * size + n] = slots
        h[2 * size + n:] = -1
        if tokens_dev is None:
            h[:n] = tokens_host
            h[n:size] = 0
            cap.ints.copy_(cap.host, non_blocking=True)
            self.bytes_uploaded += 12 * size
        else:
            cap.ints[size:].copy_(cap.host[size:], non_blocking=True)
            cap.ints[:n].copy_(tokens_dev)
            self.bytes_uploaded += 8 * size
        cap.event = torch.cuda.Event()
        cap.event.record()
        cap.graph.replay()
        counters.launches += cap.n_kernels
        return cap.logits[:n].clone()
