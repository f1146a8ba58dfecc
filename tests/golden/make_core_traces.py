#!/usr/bin/env python3
"""Golden traces of the reference's CPU core, and the replay of the same scripts through this
repository's own core.

    python tests/golden/make_core_traces.py [--reference DIR]     # rewrites core_traces.json

The reference's ``src/core/*.cpp`` (block allocator, prefix cache, paged and contiguous managers,
scheduler) is plain C++17 and compiles on a CPU in a few seconds.  ``reference_core_trace.cpp``
(beside this file) is compiled against it and fed scripts of operations; what it prints is stored
in ``core_traces.json`` together with the scripts.  ``replay`` below runs a script through
``kvcm_core`` and produces lines of the same form; ``tests/test_reference_core.py`` compares the two.

Scripts are drawn at random with fixed seeds.  The generator asks this repository's core which
operations are legal next (a request is admitted only after ``can_admit`` said yes), so a script is
valid for both sides exactly when they agree -- and where they do not, the lines differ.

Where the two cores differ on purpose, the scripts stay inside what both do alike:
* this core takes pages per portion (``ensure``), the reference takes all pages of the prompt at
  admission (src/core/paged_manager.cpp:26-36): ``admit`` here is ``admit`` + ``ensure(length)``;
* chunked prefill is switched off (the reference has none: src/core/scheduler.cpp:68-69);
* no script drives the scheduler into preemption: the reference may take the evicted request back
  in the same call (src/core/scheduler.cpp:22,50-76), this core admits nothing in a step that
  evicted.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import subprocess
import sys
import tempfile
from typing import Dict, List

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "core_traces.json")
REFERENCE_CORE = ["block_allocator.cpp", "prefix_cache.cpp", "kv_manager.cpp", "paged_manager.cpp",
                  "contiguous_manager.cpp", "scheduler.cpp"]


def next_token(rid: int, length: int) -> int:
    return (rid * 7919 + length * 104729) % 1000 + 3


# ------------------------------------------------------------------ this repository's core

class Replay:
    """Runs a script through kvcm_core and returns the lines the reference driver would print."""

    def __init__(self) -> None:
        if ROOT not in sys.path:
            sys.path.insert(0, ROOT)
        from kvcm.cache import core
        self.core = core
        self.kv = None
        self.sched = None
        self.seqs: Dict[int, object] = {}
        self.admitted: Dict[int, bool] = {}

    def run(self, ops: List[str]) -> List[dict]:
        return [self.one(op) for op in ops]

    def one(self, line: str) -> dict:
        core = self.core
        f = line.split()
        op, a = f[0], f[1:]
        if op == "manager":
            c = core.KVManagerConfig()
            c.policy, c.num_blocks, c.block_size, c.max_seq_len = a[0], int(a[1]), int(a[2]), int(a[3])
            c.prefix_caching, c.watermark_blocks = bool(int(a[4])), int(a[5])
            self.sched, self.seqs, self.admitted = None, {}, {}
            self.kv = core.make_kv_manager(c)
            return {"op": "manager"}
        if op == "sched":
            c = core.SchedulerConfig()
            c.max_num_seqs, c.max_batched_tokens, c.chunked_prefill = int(a[0]), int(a[1]), False
            self.sched = core.Scheduler(self.kv, c)
            return {"op": "sched"}
        if op == "new":
            rid, n = int(a[0]), int(a[1])
            s = core.Sequence()
            s.id, s.tokens, s.prompt_len = rid, [int(t) for t in a[2:2 + n]], n
            self.seqs[rid], self.admitted[rid] = s, False
            return {"op": "new", "id": rid}
        if op == "can":
            rid = int(a[0])
            return {"op": "can", "id": rid, "ok": int(self.kv.can_admit(self.seqs[rid]))}
        if op == "admit":
            rid = int(a[0])
            s = self.seqs[rid]
            self.kv.admit(s)
            if not self.kv.ensure(s, s.length()):
                raise RuntimeError("ensure failed after can_admit said yes")
            self.admitted[rid] = True
            return {"op": "admit", "id": rid, "table": list(s.table(0)), "num_computed": s.num_computed,
                    "cached": s.cached_tokens}
        if op == "grow":
            rid = int(a[0])
            s = self.seqs[rid]
            s.append_token(int(a[1]))
            ok = self.kv.ensure(s, s.length())
            return {"op": "grow", "id": rid, "ok": int(ok), "table": list(s.table(0))}
        if op == "commit":
            rid = int(a[0])
            s = self.seqs[rid]
            s.num_computed = int(a[1])
            self.kv.commit(s)
            return {"op": "commit", "id": rid, "hashes": len(s.page_hashes)}
        if op == "release":
            rid = int(a[0])
            self.kv.release(self.seqs[rid])
            self.admitted[rid] = False
            return {"op": "release", "id": rid}
        if op == "stats":
            live = self.sched.live() if self.sched else [s for i, s in sorted(self.seqs.items()) if self.admitted[i]]
            st = self.kv.stats(live)
            p = st.prefix
            return {"op": "stats", "in_use": st.blocks_in_use, "cached_free": st.blocks_cached_free,
                    "allocated": st.allocated_slots, "used": st.used_slots, "tail_waste": st.tail_waste_slots,
                    "reserved_unused": st.reserved_unused_slots, "entries": st.block_table_entries,
                    "seqs": st.num_seqs, "queried": p.queried_blocks, "hits": p.hit_blocks,
                    "inserted": p.inserted_blocks, "evictions": p.evictions, "duplicates": p.duplicate_inserts}
        if op == "add":
            rid, max_new, n = int(a[0]), int(a[1]), int(a[2])
            self.sched.add_request(rid, [int(t) for t in a[3:3 + n]], max_new)
            return {"op": "add", "id": rid}
        if op == "step":
            plan = self.sched.schedule(0.0)
            rows, nxt = [], []
            for p in plan:
                rows.append([p.seq.id, p.start, p.num_tokens, int(p.is_prefill), list(p.seq.table(0))])
                if not p.wants_logits:
                    raise RuntimeError("a portion of a prompt in a script without chunked prefill")
                nxt.append(next_token(p.seq.id, p.seq.length()))
            self.sched.update(nxt, 1.0)
            done = [(-f.id - 1 if f.first_token < 0 else f.id) for f in self.sched.take_finished()]
            return {"op": "step", "plan": rows, "finished": done, "running": self.sched.num_running(),
                    "waiting": self.sched.num_waiting()}
        if op == "counters":
            c = self.sched.counters()
            return {"op": "counters", "steps": c.steps, "preemptions": c.preemptions, "admissions": c.admissions,
                    "blocked": c.admission_blocked_steps, "rejected": c.rejected, "prefill": c.prefill_tokens,
                    "decode": c.decode_tokens, "saved": c.prefill_tokens_saved, "batch_sum": c.batch_size_sum,
                    "max_running": c.max_running}
        raise ValueError(f"unknown operation {op}")


def replay(ops: List[str]) -> List[dict]:
    return Replay().run(ops)


# ------------------------------------------------------------------ script generators

def manager_script(seed: int, policy: str, prefix: bool, num_blocks: int, block_size: int, max_seq_len: int,
                   watermark: int, n_ops: int) -> List[str]:
    """Random admit / grow / commit / release / stats against one manager, with shared prefixes."""
    rng = random.Random(seed)
    r = Replay()
    ops = [f"manager {policy} {num_blocks} {block_size} {max_seq_len} {int(prefix)} {watermark}"]
    r.one(ops[0])
    prefixes = [[rng.randrange(3, 500) for _ in range(block_size * rng.randint(1, 4))] for _ in range(3)]
    next_id = 0
    live: List[int] = []        # admitted
    idle: List[int] = []        # created or released, not admitted

    def emit(line: str) -> dict:
        ops.append(line)
        return r.one(line)

    for _ in range(n_ops):
        roll = rng.random()
        if roll < 0.22 or (not live and not idle):
            n = rng.randint(1, min(max_seq_len + 3, 5 * block_size))
            toks = (rng.choice(prefixes) if rng.random() < 0.6 else []) + [rng.randrange(3, 500) for _ in range(n)]
            toks = toks[:max_seq_len + 2]
            emit(f"new {next_id} {len(toks)} " + " ".join(map(str, toks)))
            idle.append(next_id)
            next_id += 1
        elif roll < 0.45 and idle:
            rid = rng.choice(idle)
            if emit(f"can {rid}")["ok"]:
                emit(f"admit {rid}")
                idle.remove(rid)
                live.append(rid)
        elif roll < 0.65 and live:
            rid = rng.choice(live)
            s = r.seqs[rid]
            if s.length() < max_seq_len and s.num_computed >= s.length() - 1:
                emit(f"commit {rid} {s.length()}")
                emit(f"grow {rid} {rng.randrange(3, 500)}")
            else:
                emit(f"commit {rid} {rng.randint(s.num_computed, s.length())}")
        elif roll < 0.8 and live:
            rid = rng.choice(live)
            s = r.seqs[rid]
            emit(f"commit {rid} {rng.randint(s.num_computed, s.length())}")
        elif roll < 0.93 and live:
            rid = rng.choice(live)
            emit(f"release {rid}")
            live.remove(rid)
            idle.append(rid)
        else:
            emit("stats")
    emit("stats")
    return ops


def scheduler_script(seed: int, prefix: bool, num_blocks: int, block_size: int, max_seq_len: int, watermark: int,
                     max_num_seqs: int, max_batched_tokens: int, requests: int, max_prompt: int,
                     max_new: int) -> List[str]:
    """Requests arriving over time into the scheduler; runs until it is idle.  Sized so that running
    requests never exhaust the pool (no preemption): the watermark keeps more pages spare than the
    running requests can still grow by."""
    assert watermark >= max_num_seqs * ((max_new + block_size - 1) // block_size + 1)
    rng = random.Random(seed)
    r = Replay()
    ops = [f"manager paged {num_blocks} {block_size} {max_seq_len} {int(prefix)} {watermark}",
           f"sched {max_num_seqs} {max_batched_tokens}"]
    for o in ops:
        r.one(o)
    prefixes = [[rng.randrange(3, 900) for _ in range(block_size * rng.randint(1, 3))] for _ in range(2)]

    def emit(line: str) -> dict:
        ops.append(line)
        return r.one(line)

    added = 0
    while added < requests or not r.sched.idle():
        for _ in range(rng.choice([0, 0, 1, 1, 2, 3])):
            if added >= requests:
                break
            n = rng.randint(1, max_prompt)
            if rng.random() < 0.08:
                n = max_seq_len + rng.randint(1, 5)             # can never fit: rejected
            toks = (rng.choice(prefixes) if prefix and rng.random() < 0.6 else []) \
                + [rng.randrange(3, 900) for _ in range(n)]
            emit(f"add {added} {rng.randint(1, max_new)} {len(toks)} " + " ".join(map(str, toks)))
            added += 1
        emit("step")
        if rng.random() < 0.15:
            emit("stats")
    emit("counters")
    emit("stats")
    assert r.sched.counters().preemptions == 0, "the script must stay clear of preemption"
    return ops


def scenarios() -> Dict[str, List[str]]:
    return {
        "paged_plain": manager_script(11, "paged", False, 24, 4, 40, 0, 260),
        "paged_watermark": manager_script(12, "paged", False, 30, 8, 64, 3, 220),
        "paged_prefix": manager_script(13, "paged", True, 28, 4, 48, 1, 420),
        "paged_prefix_tight": manager_script(14, "paged", True, 14, 4, 40, 0, 420),
        "contiguous": manager_script(15, "contiguous", False, 40, 4, 36, 0, 260),
        "scheduler_plain": scheduler_script(21, False, 64, 4, 40, 20, 6, 64, 40, 24, 6),
        "scheduler_budget": scheduler_script(22, False, 80, 8, 80, 16, 5, 48, 40, 44, 16),
        "scheduler_prefix": scheduler_script(23, True, 72, 4, 48, 21, 6, 96, 50, 20, 8),
    }


# ------------------------------------------------------------------ the reference's side

def build_reference_driver(reference: str, workdir: str) -> str:
    exe = os.path.join(workdir, "reference_core_trace")
    src = [os.path.join(reference, "src", "core", f) for f in REFERENCE_CORE]
    cmd = ["g++", "-std=c++17", "-O1", "-I", os.path.join(reference, "src"),
           os.path.join(HERE, "reference_core_trace.cpp"), *src, "-o", exe]
    subprocess.run(cmd, check=True)
    return exe


def run_reference(exe: str, ops: List[str]) -> List[dict]:
    r = subprocess.run([exe], input="\n".join(ops) + "\n", stdout=subprocess.PIPE, text=True, check=True)
    return [json.loads(line) for line in r.stdout.splitlines()]


def reference_source() -> str | None:
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            p = json.load(f).get("reference_path")
    except (OSError, ValueError):
        return None
    return p if p and os.path.isfile(os.path.join(p, "src", "core", "scheduler.cpp")) else None


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=reference_source())
    args = ap.parse_args()
    if not args.reference:
        print("the reference's source tree is not on this machine", file=sys.stderr)
        return 1
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        exe = build_reference_driver(args.reference, tmp)
        for name, ops in scenarios().items():
            out[name] = {"ops": ops, "reference": run_reference(exe, ops)}
            print(f"{name}: {len(ops)} operations")
    with open(OUT, "w") as f:
        json.dump(out, f, separators=(",", ":"))
    print(f"wrote {OUT} ({os.path.getsize(OUT)} bytes)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
