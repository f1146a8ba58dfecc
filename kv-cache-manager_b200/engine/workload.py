"""Synthetic requests: Poisson arrivals, lognormal prompt and output lengths, optional shared
prefixes, deterministic random tokens.  Flags, defaults and clamping as the reference's generator
(``src/sim/workload.cpp:12-125``); the random streams are numpy's, so draws differ from the
reference's ``mt19937_64`` while the distributions are the same."""
from __future__ import annotations

import csv
import math
from dataclasses import dataclass
from typing import List

import numpy as np


@dataclass
class WorkloadConfig:
    num_requests: int = 1000
    arrival_rate: float = 0.0            # requests per second; <= 0: all arrive at t = 0
    prompt_mu: float = 5.0
    prompt_sigma: float = 1.0            # lognormal of the prompt length (median ~148)
    output_mu: float = 5.3
    output_sigma: float = 0.9            # lognormal of the output length (median ~200)
    min_prompt: int = 4
    max_prompt: int = 1024
    min_output: int = 4
    max_output: int = 1024
    max_seq_len: int = 2048
    shared_frac: float = 0.0             # fraction of requests that start with a shared prefix
    shared_len: int = 0
    num_shared_prefixes: int = 1
    lengths_csv: str = ""                # optional "prompt_len,output_len" rows, drawn with replacement
    vocab: int = 32000
    seed: int = 1

    @classmethod
    def from_args(cls, a) -> "WorkloadConfig":
        c = cls()
        c.num_requests = a.i32("requests", c.num_requests)
        c.arrival_rate = a.f64("rate", c.arrival_rate)
        c.prompt_mu = a.f64("prompt-mu", c.prompt_mu)
        c.prompt_sigma = a.f64("prompt-sigma", c.prompt_sigma)
        c.output_mu = a.f64("output-mu", c.output_mu)
        c.output_sigma = a.f64("output-sigma", c.output_sigma)
        c.min_prompt = a.i32("min-prompt", c.min_prompt)
        c.max_prompt = a.i32("max-prompt", c.max_prompt)
        c.min_output = a.i32("min-output", c.min_output)
        c.max_output = a.i32("max-output", c.max_output)
        c.max_seq_len = a.i32("max-seq-len", c.max_seq_len)
        c.shared_frac = a.f64("shared-frac", c.shared_frac)
        c.shared_len = a.i32("shared-len", c.shared_len)
        c.num_shared_prefixes = a.i32("num-prefixes", c.num_shared_prefixes)
        c.lengths_csv = a.str("lengths-csv", c.lengths_csv)
        c.seed = a.i64("seed", c.seed)
        if a.has("prompt-len"):                       # fixed lengths override the distributions
            n = a.i32("prompt-len", 0)
            c.prompt_sigma, c.prompt_mu, c.min_prompt, c.max_prompt = 0.0, math.log(max(n, 1)), n, n
        if a.has("output-len"):
            n = a.i32("output-len", 0)
            c.output_sigma, c.output_mu, c.min_output, c.max_output = 0.0, math.log(max(n, 1)), n, n
        return c

    def describe(self) -> str:
        return (f"requests={self.num_requests} rate={self.arrival_rate} prompt~LN({self.prompt_mu},"
                f"{self.prompt_sigma}) output~LN({self.output_mu},{self.output_sigma}) "
                f"shared_frac={self.shared_frac} shared_len={self.shared_len} "
                f"max_seq_len={self.max_seq_len} seed={self.seed}")


@dataclass
class Request:
    id: int
    arrival: float
    prompt_len: int          # total, shared prefix included
    output_len: int
    prefix_id: int           # -1: no shared prefix


def generate_workload(c: WorkloadConfig) -> List[Request]:
    rng = np.random.default_rng(c.seed)
    table = []
    if c.lengths_csv:
        with open(c.lengths_csv) as f:
            for row in csv.reader(f):
                try:
                    p, o = int(row[0]), int(row[1])
                except (ValueError, IndexError):
                    continue
                if p > 0 and o > 0:
                    table.append((p, o))
        if not table:
            raise ValueError(f"no rows in lengths csv: {c.lengths_csv}")
    out, t, next_prefix = [], 0.0, 0
    for i in range(c.num_requests):
        if c.arrival_rate > 0:
            t += rng.exponential(1.0 / c.arrival_rate)
        if table:
            p, o = table[rng.integers(len(table))]
        else:
            p = int(round(rng.lognormal(c.prompt_mu, max(c.prompt_sigma, 1e-9))))
            o = int(round(rng.lognormal(c.output_mu, max(c.output_sigma, 1e-9))))
        p = min(max(p, c.min_prompt), c.max_prompt)
        o = min(max(o, c.min_output), c.max_output)
        prefix = -1
        if c.shared_len > 0 and rng.random() < c.shared_frac:
            prefix = next_prefix % max(1, c.num_shared_prefixes)
            next_prefix += 1
            p += c.shared_len
        p = min(p, c.max_seq_len - 1)
        o = max(1, min(o, c.max_seq_len - p))
        out.append(Request(i, t, p, o, prefix))
    return out


def make_prompt_tokens(r: Request, c: WorkloadConfig) -> List[int]:
    """Tokens in [3, vocab); the tokens of a shared prefix depend only on (seed, prefix id)."""
    toks: List[int] = []
    if r.prefix_id >= 0:
        pr = np.random.default_rng([c.seed, 0xABCDEF, r.prefix_id])
        toks = pr.integers(3, c.vocab, size=min(c.shared_len, r.prompt_len)).tolist()
    rr = np.random.default_rng([c.seed, 0x1234567, r.id])
    toks += rr.integers(3, c.vocab, size=r.prompt_len - len(toks)).tolist()
    return toks
