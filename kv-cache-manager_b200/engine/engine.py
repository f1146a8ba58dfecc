"""The request loop: scheduler + cache manager + step function + sampler behind one object.

API after the reference's ``Engine`` (``src/engine/engine.h:29-52``): ``add_request`` (its
``add``), ``step`` -> ``StepInfo``, ``take_finished``, ``idle``, ``score``.  One ``step()`` =
schedule (C++), build the batch (C++, one pinned buffer, one host-to-device copy), run the model
on the batch, sample on the device, read the sampled tokens back (the step's only
synchronisation), update the scheduler (``src/engine/engine.cpp:73-90``).
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..cache import core, manager_from_config
from ..cache.pools import bytes_per_block, plan_cache
from ..config.engine_config import EngineConfig, canonical_dtype
from ..models.spec import ModelSpec
from ..kernels import library as K
from ..sampling import Sampler
from .decode_graph import DecodeGraphs
from .model_io import load_model, torch_dtype
from .runner import ModelRunner


@dataclass
class StepInfo:
    rows: int = 0
    seqs: int = 0
    prefill_tokens: int = 0
    decode_seqs: int = 0
    sampled: int = 0
    ms: float = 0.0
    h2d_bytes: int = 0
    d2h_bytes: int = 0
    graph: bool = False


class DeviceTimer:
    """CUDA events around the device work of each step (after the step's host-to-device copy,
    up to and including sampling).  ``total_ms()`` synchronises and sums."""

    def __init__(self) -> None:
        self.pairs = []

    def start(self) -> None:
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self._open = e

    def stop(self) -> None:
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.pairs.append((self._open, e))

    def total_ms(self) -> float:
        torch.cuda.synchronize()
        own = sum(a.elapsed_time(b) for a, b in self.pairs)
        return own + (self.native.device_ms_total() if getattr(self, "native", None) is not None else 0.0)

    def reset(self) -> None:
        self.pairs = []


class _NativeGraphs:
    """What callers read of the decode graphs when the C++ loop owns them."""

    def __init__(self, native) -> None:
        self._native = native
        self.kernels_last = 0

    @property
    def replays(self) -> int:
        return int(self._native.graph_replays())

    @property
    def captured(self) -> dict:
        return {(b, c, bool(t)): None for b, c, t in self._native.graph_shapes()}


class Engine:
    def __init__(self, spec: ModelSpec, cfg: Optional[EngineConfig] = None) -> None:
        self.cfg = cfg = cfg or EngineConfig()
        self.spec = spec
        self.dtype_name = canonical_dtype(cfg.dtype)
        dtype = torch_dtype(self.dtype_name)
        plan = plan_cache(spec)
        kv = cfg.kv
        if kv.num_blocks <= 0:       # pool size given in GB (src/engine/engine.cpp:19-27)
            per_block = max(1, bytes_per_block(plan, kv.block_size, dtype))
            kv.num_blocks = int(cfg.pool_gb * float(1 << 30) / per_block)
        if kv.policy == "contiguous":
            kv.prefix_caching = False
        if kv.prefix_caching and plan.has_state:
            raise ValueError("prefix caching skips tokens whose fixed-size state would be missing; "
                             "it cannot be used with a model that keeps per-request state")
        sc = cfg.sched
        max_rows = sc.max_batched_tokens if sc.chunked_prefill else max(sc.max_batched_tokens, kv.max_seq_len)
        max_rows = max(max_rows, sc.max_num_seqs)
        self.max_logit_rows = cfg.max_logit_rows or max(sc.max_num_seqs, 512)
        self.runner = ModelRunner(
            spec, dtype, cfg.device, num_blocks=kv.num_blocks, block_size=kv.block_size,
            max_seq_len=kv.max_seq_len, num_slots=sc.max_num_seqs,
            max_rows=max(max_rows, kv.max_seq_len), max_seqs=sc.max_num_seqs,
            max_logit_rows=max(self.max_logit_rows, kv.max_seq_len),
            options={"attn_version": cfg.attn, "gemm": cfg.gemm, "fuse_norms": cfg.fuse_norms})
        self.kv = manager_from_config(kv, self.runner.windows)
        s = core.SchedulerConfig()
        s.max_num_seqs, s.max_batched_tokens = sc.max_num_seqs, sc.max_batched_tokens
        s.prefill_chunk, s.chunked_prefill, s.eos_token_id = sc.prefill_chunk, sc.chunked_prefill, cfg.eos_token_id
        self.sched = core.Scheduler(self.kv, s)
        self.sampler = Sampler(cfg.device, max(self.max_logit_rows, sc.max_num_seqs))
        capturable = all(part.capturable for _, top in spec.parts() for _, part in top.named_parts())
        self.graphs = DecodeGraphs(self.runner, self.sampler) if cfg.cuda_graphs and capturable else None
        self.vocab = spec.lm_head.vocab
        self._next_id = 0
        self._t0 = time.perf_counter()
        self._has_state = plan.has_state
        self._device_timer = None         # a DeviceTimer brackets the device work of every step
        # The standard arrangement of parts with default options: the whole request loop runs in C++
        # (csrc/core/native_engine.cpp) over the same scheduler, cache manager and pools.
        self.native = None
        nf = self.runner.native
        if cfg.native_loop and nf is not None and cfg.gemm == "auto" and cfg.attn == "auto" and not plan.has_state:
            torch.cuda.synchronize(self.runner.device)         # weights and pools are in place
            scratch = 0 if nf.f32 else min(sc.max_num_seqs, 1024) * nf.nh * 64 * (nf.hd + 2)
            self.native = core.NativeEngine(
                self.kv, self.sched, nf.model_for_core(),
                dict(block_size=kv.block_size, max_seq_len=kv.max_seq_len, num_groups=self.runner.num_groups,
                     max_rows=max(max_rows, kv.max_seq_len), max_seqs=sc.max_num_seqs, graphs=bool(cfg.cuda_graphs),
                     attn_scratch_floats=scratch,
                     # one step of lookahead, unless a token's value matters to the host at once
                     fuse_norms=bool(cfg.fuse_norms),
                     lookahead=bool(cfg.lookahead and cfg.eos_token_id < 0 and not kv.prefix_caching)),
                K.device_backend_address())
            self.graphs = _NativeGraphs(self.native) if cfg.cuda_graphs else None

    @classmethod
    def from_folder(cls, folder: str, cfg: Optional[EngineConfig] = None) -> "Engine":
        cfg = cfg or EngineConfig()
        return cls(load_model(folder, cfg.dtype, cfg.device), cfg)

    # -------------------------------------------------------------------------- clock
    def now(self) -> float:
        return self.native.now() if self.native is not None else time.perf_counter() - self._t0

    def reset_clock(self) -> None:
        self._t0 = time.perf_counter()
        if self.native is not None:
            self.native.reset_clock()

    @property
    def device_timer(self):
        return self._device_timer

    @device_timer.setter
    def device_timer(self, timer) -> None:
        """A ``DeviceTimer`` (or None): device time of every step from now on.  With the C++ loop the
        events are its own and the timer is handed their sum."""
        self._device_timer = timer
        if self.native is not None:
            self.native.set_timing(timer is not None)
            self.native.reset_device_ms()
            if timer is not None:
                timer.native = self.native

    # ----------------------------------------------------------------------- requests
    def add_request(self, tokens: Sequence[int], max_new_tokens: int, temperature: float = 0.0,
                    seed: Optional[int] = None, request_id: Optional[int] = None,
                    arrival: Optional[float] = None) -> int:
        toks = [int(t) for t in tokens]
        if not toks:
            raise ValueError("a request needs at least one token")
        bad = [t for t in toks if t < 0 or t >= self.vocab]
        if bad:
            raise ValueError(f"token id {bad[0]} outside the vocabulary of {self.vocab}")
        rid = self._next_id if request_id is None else int(request_id)
        self._next_id = max(self._next_id, rid) + 1
        self.sched.add_request(rid, toks, int(max_new_tokens), float(temperature),
                               int(self.cfg.sampling_seed if seed is None else seed) & ((1 << 64) - 1),
                               self.now() if arrival is None else arrival)
        return rid

    def idle(self) -> bool:
        return self.sched.idle()

    def take_finished(self):
        return self.sched.take_finished()

    # --------------------------------------------------------------------------- step
    def step(self) -> StepInfo:
        if self.native is not None and not K.profiling():
            return self._native_step()
        info = StepInfo()
        t_start = self.now()
        self.sched.schedule(t_start)
        rows, entries, wants, prefill, singles, tempered = self.sched.plan_summary()
        if entries == 0:
            return info
        if self._has_state:
            for p in self.sched.plan():
                if p.start == 0:
                    self.runner.pools.reset_slot(p.seq.state_slot)
        greedy_only = tempered == 0
        if wants and not greedy_only:
            ids, pos, temps, seeds = self.sched.plan_sampling()
        timed = self.device_timer is not None
        if self.graphs is not None and singles == entries and wants == entries:
            packed = self.graphs.run(self.sched, entries, self.device_timer,
                                     None if greedy_only else (ids, pos, temps, seeds))
            info.graph = True
        else:
            layout = self.runner.build_from_scheduler(self.sched)
            self.runner.upload(layout, sync_follows=wants > 0)
            if timed:
                self.device_timer.start()
            logits = self.runner.forward(self.runner.context(layout))
            if wants:
                if greedy_only:
                    self.sampler.greedy(logits)
                else:
                    self.sampler.sample(logits, ids, pos, temps, seeds)
            packed = self.sampler.packed
            if timed:
                self.device_timer.stop()
        info.h2d_bytes = self.runner.h2d_bytes_last + (self.sampler.h2d_bytes_last if wants else 0)
        sampled: List[int] = []
        if wants:
            # The step's one synchronisation: the sampled tokens and, in front of them, the status
            # pair that the sampling kernel gathered from the kernels' error words.
            got = packed[:2 + wants].tolist()
            K.raise_on_status(got[0], got[1])
            sampled = got[2:]
        info.d2h_bytes = 4 * (2 + wants) if wants else 0
        t_end = self.now()
        self.sched.update(sampled, t_end)
        info.rows, info.seqs, info.prefill_tokens = rows, entries, prefill
        info.decode_seqs, info.sampled = singles, wants
        info.ms = (t_end - t_start) * 1e3
        return info

    def _native_step(self) -> StepInfo:
        try:
            n = self.native.step()
        except RuntimeError as e:
            if "a bounded wait ran out" in str(e):
                raise K.KernelError(str(e)) from None
            raise
        K.add_launches(n.launches)
        if self.graphs is not None:
            self.graphs.kernels_last = n.launches
        return StepInfo(rows=n.rows, seqs=n.seqs, prefill_tokens=n.prefill_tokens, decode_seqs=n.decode_seqs,
                        sampled=n.sampled, ms=n.ms, h2d_bytes=n.h2d_bytes, d2h_bytes=n.d2h_bytes, graph=n.graph)

    def run_until_idle(self, max_steps: int = 1 << 30) -> int:
        n = 0
        while not self.idle() and n < max_steps:
            self.step()
            n += 1
        return n

    # -------------------------------------------------------------------------- score
    def score(self, tokens: Sequence[int]) -> torch.Tensor:
        """Teacher-forced float32 logits [n, vocab] at every position of ``tokens``, through the
        real cache path (``src/engine/engine.cpp:92-108``).  Not with prefix caching: computing
        every position again would write pages that other requests share."""
        if self.cfg.kv.prefix_caching:
            raise RuntimeError("score: disable prefix caching")
        if self.native is not None:
            self.native.drain()               # a step still on the device ends first (its result comes with the next step())
        torch.cuda.synchronize()              # the C++ loop runs on a stream of its own
        s = core.Sequence()
        s.id = -1
        s.tokens = [int(t) for t in tokens]
        s.prompt_len = len(s.tokens)
        if not self.kv.can_admit(s):
            raise RuntimeError("score: sequence does not fit in the KV pool")
        self.kv.admit(s)
        try:
            if not self.kv.ensure(s, s.length()):
                raise RuntimeError("score: out of cache pages")
            if self._has_state:
                raise RuntimeError("score: models with per-request state are scored through add_request")
            logits = self.runner.step([(s, 0, s.length(), list(range(s.length())))])
            torch.cuda.synchronize()
            K.check_errors()
        finally:
            self.kv.release(s)
        return logits


def generate(engine: Engine, prompts: Sequence[Sequence[int]], max_new_tokens: int,
             temperature: float = 0.0, seed: Optional[int] = None) -> List[List[int]]:
    """Runs the prompts to completion and returns the generated tokens in the prompts' order
    (host tokens in, host tokens out)."""
    ids = [engine.add_request(p, max_new_tokens, temperature, seed) for p in prompts]
    done = {}
    while not engine.idle():
        engine.step()
        for f in engine.take_finished():
            done[f.id] = f
    for f in engine.take_finished():
        done[f.id] = f
    out = []
    for i in ids:
        f = done.get(i)
        out.append([] if f is None or f.rejected else f.generated())
    return out
