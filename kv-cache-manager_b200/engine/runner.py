"""The step function: runs one batch of (request, its next tokens) through the model, from the
cache, and returns float32 logits at the wanted places.

A batch may hold portions of prompts beside single decoded tokens, cut anywhere.  The step runs
only the tokens it is given.  Generation (``engine.Engine``), trace replay (``bin/trace_run``)
and the tests all call this one function; there is no second forward pass anywhere.

Per step (as the reference's forward, ``src/model/llama.cpp:54-141``): the batch's integer arrays
are packed into one pinned buffer by the C++ ``BatchBuilder`` and reach the device in ONE copy;
embedding; the layers in the model's run order; final norm and output head on the wanted rows
only.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence as Seq, Tuple

import torch

from ..cache import core
from ..cache.pools import CachePlan, CachePools, bytes_per_block, plan_cache
from ..models.spec import ModelSpec
from ..parts.base import GroupView, StepContext

PREFILL_TILE_ROWS = 64      # query rows per work item of the prefill attention kernel


class ModelRunner:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device, *, num_blocks: int,
                 block_size: int, max_seq_len: int, num_slots: int, max_rows: int, max_seqs: int,
                 max_logit_rows: int, options: Optional[dict] = None) -> None:
        self.spec, self.dtype, self.device = spec, dtype, torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("this engine runs on a CUDA device only (no CPU path)")
        self.options = dict(options or {})
        self.block_size, self.num_blocks, self.max_seq_len = block_size, num_blocks, max_seq_len
        self.max_blocks = (max_seq_len + block_size - 1) // block_size
        self.max_rows, self.max_seqs, self.max_logit_rows = max_rows, max_seqs, max_logit_rows
        self.plan: CachePlan = plan_cache(spec)
        self.pools = CachePools(self.plan, num_blocks, block_size, num_slots, dtype, self.device)
        self.num_groups = max(1, len(self.plan.groups))
        self.windows = self.plan.windows or [0]
        self.builder = core.BatchBuilder(block_size, self.max_blocks, self.num_groups, PREFILL_TILE_ROWS)
        cap = int(self.builder.capacity_for(max_rows, max_seqs, max_logit_rows))
        self.capacity = cap
        self.host_ints = torch.empty(cap, dtype=torch.int32, pin_memory=True)
        self.dev_ints = torch.zeros(cap, dtype=torch.int32, device=self.device)
        self._copied = torch.cuda.Event()
        self._copy_pending = False
        self._views = {}                  # (buffer, length) -> (device view, pinned view) of an upload
        self.h2d_bytes_last = 0
        # The standard arrangement of parts runs its layer loop in C++ (engine/native_forward.py).
        from .native_forward import NativeForward
        self.native = NativeForward.plan(spec, self) if self.options.get("native_forward", True) else None

    # ------------------------------------------------------------------ batch -> device
    def build(self, entries: Seq[Tuple[object, int, int, Seq[int]]], pad_rows: int = 0,
              pad_seqs: int = 0):
        """entries: (Sequence, start, num_tokens, wanted places).  Returns the BatchLayout."""
        self._wait_copy()
        layout = self.builder.build([(s, int(a), int(n), [int(w) for w in want])
                                     for s, a, n, want in entries],
                                    self.host_ints.data_ptr(), self.capacity, pad_rows, pad_seqs)
        self._check_limits(layout)
        return layout

    def build_from_scheduler(self, sched, pad_rows: int = 0, pad_seqs: int = 0,
                             pad_logit_rows: int = 0):
        self._wait_copy()
        layout = sched.build_batch(self.builder, self.host_ints.data_ptr(), self.capacity,
                                   pad_rows, pad_seqs, pad_logit_rows)
        self._check_limits(layout)
        return layout

    def _check_limits(self, layout) -> None:
        if layout.rows > self.max_rows or layout.seqs > self.max_seqs or \
                layout.logit_rows > self.max_logit_rows:
            raise RuntimeError(
                f"step of {layout.rows} rows / {layout.seqs} requests / {layout.logit_rows} logit rows "
                f"exceeds the limits {self.max_rows} / {self.max_seqs} / {self.max_logit_rows}")

    def _wait_copy(self) -> None:
        if self._copy_pending:
            self._copied.synchronize()      # the pinned buffer is free again
            self._copy_pending = False

    def upload(self, layout, into: Optional[torch.Tensor] = None, sync_follows: bool = False) -> torch.Tensor:
        """One host-to-device copy of the step's packed integer arrays.  ``sync_follows``: the caller
        synchronises with the device before the next batch is built (a step that reads its sampled
        tokens back does), so the pinned buffer needs no event of its own."""
        n = int(layout.total_ints)
        dst = self.dev_ints if into is None else into
        key = (dst.data_ptr(), n)
        views = self._views.get(key)
        if views is None:
            if len(self._views) > 64:
                self._views.clear()
            views = self._views[key] = (dst[:n], self.host_ints[:n])
        views[0].copy_(views[1], non_blocking=True)
        if sync_follows:
            self._copy_pending = False
        else:
            self._copied.record()
            self._copy_pending = True
        self.h2d_bytes_last = 4 * n
        return dst

    def context(self, layout, ints: Optional[torch.Tensor] = None) -> StepContext:
        d = self.dev_ints if ints is None else ints
        T, S, G, MB = layout.rows, layout.seqs, layout.groups, layout.max_blocks

        def view(off: int, n: int) -> torch.Tensor:
            return d[off:off + n]

        groups: List[GroupView] = []
        for g in range(G):
            bt = view(layout.off_block_tables + g * S * MB, S * MB).view(S, MB)
            sm = view(layout.off_slot_mapping + g * T, T)
            groups.append(GroupView(bt, sm, self.block_size, self.windows[g] if g < len(self.windows) else 0))
        return StepContext(
            rows=T, seqs=S, decode_seqs=layout.decode_seqs + (layout.seqs - layout.real_seqs),
            prefill_rows=layout.prefill_rows, prefill_tiles=layout.prefill_tiles,
            tile_rows=layout.tile_rows, max_ctx=layout.max_ctx, max_decode_ctx=layout.max_decode_ctx,
            max_q_len=layout.max_q_len,
            tokens=view(layout.off_tokens, T), positions=view(layout.off_positions, T),
            row_seq=view(layout.off_row_seq, T), seq_q_start=view(layout.off_seq_q_start, S),
            seq_q_len=view(layout.off_seq_q_len, S), seq_ctx_len=view(layout.off_seq_ctx_len, S),
            seq_state_slot=view(layout.off_seq_state_slot, S),
            tile_seq=view(layout.off_tile_seq, max(layout.prefill_tiles, 0)),
            tile_q0=view(layout.off_tile_q0, max(layout.prefill_tiles, 0)),
            logit_rows=view(layout.off_logit_rows, layout.logit_rows),
            groups=groups, dtype=self.dtype, workspace=self, options=self.options)

    # ------------------------------------------------------------------------- forward
    def forward(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """Hidden states through every layer; float32 logits [wanted rows, vocab] (None when no
        row is wanted: the step then only fills the cache)."""
        spec = self.spec
        if self.native is not None and self.native.takes(ctx):
            return self.native.run(ctx)
        x = spec.embedding.forward(ctx)
        pending = None
        for k, call in enumerate(spec.order):
            pending = spec.blocks[call.layer].forward(x, pending, ctx, self.pools.sites[k])
        n = ctx.logit_rows.numel()
        if n == 0:
            return None
        h_last = torch.empty((n, x.shape[1]), dtype=self.dtype, device=x.device)
        spec.final_norm.forward(x, pending, h_last, rows=ctx.logit_rows)
        return spec.lm_head.forward(h_last, ctx)

    def step(self, entries: Seq[Tuple[object, int, int, Seq[int]]]) -> Optional[torch.Tensor]:
        """Builds, uploads and runs one batch.  Logits rows follow the order of ``entries`` and of
        each entry's wanted places."""
        layout = self.build(entries)
        self.upload(layout)
        return self.forward(self.context(layout))

    # --------------------------------------------------------------------------- sizes
    def bytes_per_block(self) -> int:
        return bytes_per_block(self.plan, self.block_size, self.dtype)
