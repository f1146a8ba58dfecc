"""The loop of trace replay: given token ids go through the model step by step, as the caller cuts
them.  One object owns what a replay needs -- the model runner (step function, pools), a cache
manager, state slots, the live requests -- and ``bin/trace_run`` and the tests both drive it, so
there is one replay driver, as there is one forward pass.

It bypasses the scheduler's *choice* of portions and nothing else: requests are admitted by the
cache manager on first appearance (with prefix caching that is where matching pages are taken over),
pages are taken per portion (``ensure``), completed pages are registered after the step
(``commit``), and everything is given back when the caller says a request has ended.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..cache import core, manager_from_config
from ..config import KVManagerConfig
from .model_io import torch_dtype
from .runner import ModelRunner


class ReplayError(RuntimeError):
    pass


class ReplaySession:
    def __init__(self, spec, dtype: str, max_tokens: int, block_size: int = 16, max_live: int = 64,
                 policy: str = "paged", prefix_caching: bool = False, max_seq_len: int = 0,
                 options: Optional[dict] = None, device: str = "cuda:0") -> None:
        B = block_size
        num_blocks = (max_tokens + B - 1) // B
        if max_seq_len <= 0:
            # paged: one request may fill the pool; contiguous: every request reserves its longest
            # length up front, so leave room for four
            max_seq_len = num_blocks * B if policy == "paged" else max(B, (num_blocks // 4) * B)
        self.spec, self.block_size, self.max_live, self.max_tokens = spec, B, max_live, max_tokens
        self.max_seq_len = max_seq_len
        rows = num_blocks * B
        self.runner = ModelRunner(spec, torch_dtype(dtype), device, num_blocks=num_blocks, block_size=B,
                                  max_seq_len=max_seq_len, num_slots=max_live, max_rows=rows, max_seqs=max_live,
                                  max_logit_rows=rows, options=options or {})
        self.kv = manager_from_config(KVManagerConfig(policy=policy, num_blocks=num_blocks, block_size=B,
                                                      max_seq_len=max_seq_len, prefix_caching=prefix_caching,
                                                      watermark_blocks=0), self.runner.windows)
        self.slots = core.StateSlots(max_live)
        self.vocab = spec.lm_head.vocab
        self.live: Dict[object, object] = {}
        self._next_id = 0
        self.cached_tokens_last: Dict[object, int] = {}     # per request of the last step: tokens a prefix hit skipped

    def release(self, rid) -> None:
        seq = self.live.pop(rid)
        self.kv.release(seq)
        if seq.state_slot >= 0:
            self.slots.give_back(seq.state_slot)

    def step(self, entries: Sequence[dict], end: Sequence = (), tag=None) -> Optional[torch.Tensor]:
        """entries: {"id", "tokens", "want"}.  Returns float32 logits [wanted, vocab] on the device in
        the order of the entries and of ``want`` (None when nothing is wanted).  Raises ReplayError
        with one line for what the step cannot do."""
        where = f"step {tag}: " if tag is not None else ""
        batch: List[Tuple[object, int, int, List[int]]] = []
        self.cached_tokens_last = {}
        for e in entries:
            rid, toks = e["id"], [int(t) for t in e["tokens"]]
            want = [int(w) for w in e.get("want", [])]
            if not toks:
                raise ReplayError(f"{where}request {rid!r} brings no tokens")
            bad = [t for t in toks if t < 0 or t >= self.vocab]
            if bad:
                raise ReplayError(f"{where}token {bad[0]} outside the vocabulary of {self.vocab}")
            bad = [w for w in want if w < 0 or w >= len(toks)]
            if bad:
                raise ReplayError(f"{where}request {rid!r} wants place {bad[0]} of a portion of {len(toks)} tokens")
            seq = self.live.get(rid)
            skipped = 0
            if seq is None:
                seq = core.Sequence()
                seq.id = self._next_id
                self._next_id += 1
                seq.state_slot = self.slots.take()
                if seq.state_slot < 0:
                    raise ReplayError(f"{where}more than {self.max_live} live requests")
                seq.extend_tokens(toks)             # the manager matches cached pages against these
                seq.prompt_len = len(toks)
                if not self.kv.can_admit(seq):
                    self.slots.give_back(seq.state_slot)
                    raise ReplayError(f"{where}request {rid!r} of {len(toks)} tokens does not fit the cache "
                                      f"(pool made for --max-tokens {self.max_tokens}, longest request "
                                      f"{self.max_seq_len})")
                self.kv.admit(seq)
                self.runner.pools.reset_slot(seq.state_slot)
                self.live[rid] = seq
                start, skipped = 0, seq.num_computed        # a prefix hit: these rows lie in shared pages
            else:
                start = seq.length()
                seq.extend_tokens(toks)
            if seq.length() > self.max_seq_len:
                raise ReplayError(f"{where}request {rid!r} would hold {seq.length()} tokens, more than the "
                                  f"longest request of {self.max_seq_len}")
            if not self.kv.ensure(seq, seq.length()):
                raise ReplayError(f"{where}out of cache pages for request {rid!r} ({seq.length()} tokens; pool "
                                  f"made for --max-tokens {self.max_tokens})")
            if skipped:
                below = [w for w in want if w < skipped]
                if below:
                    self.release(rid)               # the request is not taken
                    raise ReplayError(f"{where}request {rid!r} wants place {below[0]}, which lies in the "
                                      f"{skipped} tokens taken over from the prefix cache (they are not computed)")
                want = [w - skipped for w in want]
                self.cached_tokens_last[rid] = skipped
            batch.append((seq, start + skipped, len(toks) - skipped, want))
        logits = self.runner.step(batch) if batch else None
        for seq, first, n, _ in batch:
            seq.num_computed = first + n
            self.kv.commit(seq)
        for rid in end:
            if rid in self.live:
                self.release(rid)
        return logits
