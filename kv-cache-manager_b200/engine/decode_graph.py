"""CUDA graphs for decode-only steps.

A decode step of a small model is a few hundred short kernels; launched one by one their launch
cost exceeds their run time.  A step in which every request brings exactly one token is therefore
captured once per shape and replayed.  The shape of a captured step is (batch bucket, context
bucket, greedy or not): the batch is padded to the bucket with rows that read and write nothing,
the bucket of the longest context fixes how the decode attention kernel splits the keys, and a
step in which some request samples with a temperature ends in the sampling kernel (fed from the
sampler's device buffers) instead of the argmax.  The integer arrays of the batch live in a
buffer owned by the graph; a replay is one host-to-device copy into that buffer (plus the
sampling parameters where there are any) and one graph launch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Tuple

import torch

BATCH_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256, 512)
MIN_CTX_BUCKET = 256


def batch_bucket(n: int) -> int:
    for b in BATCH_BUCKETS:
        if n <= b:
            return b
    return ((n + 255) // 256) * 256


def ctx_bucket(n: int) -> int:
    b = MIN_CTX_BUCKET
    while b < n:
        b *= 2
    return b


@dataclass
class _Captured:
    graph: torch.cuda.CUDAGraph
    ints: torch.Tensor
    sampled: torch.Tensor     # [status pair | one token per row of the bucket]
    total_ints: int
    kernels: int = 0          # launches of this engine's kernels inside one replay


class DecodeGraphs:
    def __init__(self, runner, sampler) -> None:
        self.runner, self.sampler = runner, sampler
        self.captured: Dict[Tuple[int, int], _Captured] = {}
        self.pool = None
        self.replays = 0
        self.kernels_last = 0

    def run(self, sched, n: int, timer=None, sampling=None) -> torch.Tensor:
        """Runs the scheduler's current plan (n single-row entries).  ``sampling``: None when every
        entry samples greedily, else (request ids, positions, temperatures, seeds) of the entries.
        Returns [status pair | sampled tokens] on the device; the first n tokens are real."""
        r = self.runner
        b = min(batch_bucket(n), max(r.max_seqs, n))
        layout = r.build_from_scheduler(sched, pad_rows=b, pad_seqs=b, pad_logit_rows=b)
        key = (b, ctx_bucket(layout.max_decode_ctx), sampling is not None)
        if sampling is not None:
            self.sampler.stage(*sampling, rows=b)            # before a first capture too: its eager run reads them
        cap = self.captured.get(key)
        if cap is None:
            # The capture's warm-up ran THIS step eagerly (a capture itself runs nothing) and left
            # its tokens in the graph's buffer.  The step must not run a second time: writing a page
            # twice is harmless, advancing a mixer's per-request state twice is not.
            cap = self._capture(layout, key)
            self.kernels_last = cap.kernels
            return cap.sampled
        if int(layout.total_ints) != cap.total_ints:
            raise RuntimeError("decode graph: batch layout changed for a captured shape")
        r.upload(layout, into=cap.ints, sync_follows=True)    # the engine reads the sampled tokens back
        if timer is not None:
            timer.start()
        cap.graph.replay()
        if timer is not None:
            timer.stop()
        self.replays += 1
        self.kernels_last = cap.kernels
        return cap.sampled

    def _capture(self, layout, key) -> _Captured:
        r = self.runner
        n_ints = int(layout.total_ints)
        ints = torch.zeros(n_ints, dtype=torch.int32, device=r.device)
        sampled = torch.zeros(2 + key[0], dtype=torch.int32, device=r.device)
        r.upload(layout, into=ints)
        ctx = r.context(layout, ints=ints)
        ctx.max_decode_ctx = key[1]
        ctx.max_ctx = key[1]
        from ..kernels import library as K

        def body():
            logits = r.forward(ctx)
            if key[2]:
                self.sampler.sample_staged(logits, sampled[2:], sampled[:2])   # temperatures, seeds ... in the sampler's buffers
            else:
                K.argmax(logits, sampled[2:], sampled[:2])

        # One eager run on a side stream first: lazy initialisation (library handles, kernel
        # attributes) must not happen inside a capture.  It is the real run of the step at hand.
        side = torch.cuda.Stream(device=r.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            body()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = K.launch_count()
        with torch.cuda.graph(graph, pool=self.pool):
            body()
        kernels = K.launch_count() - before
        if self.pool is None:
            self.pool = graph.pool()
        cap = _Captured(graph, ints, sampled, n_ints, kernels)
        self.captured[key] = cap
        return cap
