"""Next-token choice on the device: greedy (the reference's only mode, first index among equal
maxima, ``src/cuda/kernels.cu:90-119``) and temperature sampling with a per-request seed.

The random number of a draw depends only on (seed, request id, position of the drawn token), so
what a request generates does not depend on batching, on how its prompt was cut, or on being
preempted and computed again.  ``uniform_for`` restates the device formula on the host.
"""
from __future__ import annotations

from typing import Sequence

import torch

from ..kernels import library as K

_M64 = (1 << 64) - 1


def uniform_for(seed: int, request_id: int, position: int) -> float:
    """The uniform number in [0, 1) the sampling kernel uses for this draw."""
    z = (seed ^ (request_id * 0x9E3779B97F4A7C15) ^ (position * 0xBF58476D1CE4E5B9)) & _M64
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    z ^= z >> 31
    return (z >> 40) / 16777216.0


def _signed64(v: int) -> int:
    v &= _M64
    return v - (1 << 64) if v >= (1 << 63) else v


class Sampler:
    def __init__(self, device, max_rows: int) -> None:
        self.device = torch.device(device)
        self.max_rows = max_rows
        # [status pair | sampled tokens]: one buffer, so that the copy that brings the tokens to the
        # host also brings the word that says whether a kernel of the step gave up a bounded wait
        self.packed = torch.zeros(2 + max_rows, dtype=torch.int32, device=self.device)
        self.status, self.out = self.packed[:2], self.packed[2:]
        # [temperature (as float bits) | position] int32 and [seed | request id] int64, pinned
        self.h_f = torch.zeros(max_rows, dtype=torch.float32, pin_memory=True)
        self.h_i = torch.zeros(max_rows, dtype=torch.int32, pin_memory=True)
        self.h_l = torch.zeros(2 * max_rows, dtype=torch.int64, pin_memory=True)
        self.d_f = torch.zeros(max_rows, dtype=torch.float32, device=self.device)
        self.d_i = torch.zeros(max_rows, dtype=torch.int32, device=self.device)
        self.d_l = torch.zeros(2 * max_rows, dtype=torch.int64, device=self.device)
        self.h2d_bytes_last = 0

    def greedy(self, logits: torch.Tensor) -> torch.Tensor:
        n = logits.shape[0]
        K.argmax(logits, self.out, self.status)
        self.h2d_bytes_last = 0
        return self.out[:n]

    def sample(self, logits: torch.Tensor, request_ids: Sequence[int], positions: Sequence[int],
               temperatures: Sequence[float], seeds: Sequence[int]) -> torch.Tensor:
        """One token per row of ``logits`` (int32, on the device).  Rows with temperature 0 are
        greedy.  ``positions``: index the drawn token will have in its request."""
        n = logits.shape[0]
        if not any(t > 0 for t in temperatures):
            return self.greedy(logits)
        self.stage(request_ids, positions, temperatures, seeds)
        self.sample_staged(logits, self.out, self.status)
        return self.out[:n]

    def stage(self, request_ids: Sequence[int], positions: Sequence[int], temperatures: Sequence[float],
              seeds: Sequence[int], rows: int = 0) -> None:
        """Copies the per-row sampling parameters to the device buffers that ``sample_staged`` (and
        a captured graph) reads.  ``rows`` > len(...): the rows beyond get temperature 0."""
        n = len(temperatures)
        rows = max(rows, n)
        if rows > self.max_rows:
            raise RuntimeError(f"sampler sized for {self.max_rows} rows, got {rows}")
        self.h_f[:n] = torch.tensor(list(temperatures), dtype=torch.float32)
        self.h_f[n:rows] = 0.0
        self.h_i[:n] = torch.tensor(list(positions), dtype=torch.int32)
        self.h_l[:n] = torch.tensor([_signed64(s) for s in seeds], dtype=torch.int64)
        self.h_l[self.max_rows:self.max_rows + n] = torch.tensor([_signed64(r) for r in request_ids], dtype=torch.int64)
        self.d_f[:rows].copy_(self.h_f[:rows], non_blocking=True)
        self.d_i[:n].copy_(self.h_i[:n], non_blocking=True)
        self.d_l[:n].copy_(self.h_l[:n], non_blocking=True)
        self.d_l[self.max_rows:self.max_rows + n].copy_(self.h_l[self.max_rows:self.max_rows + n], non_blocking=True)
        self.h2d_bytes_last = n * (4 + 4 + 16) + (rows - n) * 4

    def sample_staged(self, logits: torch.Tensor, out: torch.Tensor, status=None) -> None:
        """The sampling kernel on the staged parameters; only enqueues device work."""
        K.sample(logits, self.d_f, self.d_l[:self.max_rows], self.d_l[self.max_rows:], self.d_i, out, status)
