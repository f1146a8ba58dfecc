"""This repository's CPU core against the reference's own: the same scripts of operations give
the same page tables, plans, statistics and counters.

``tests/golden/core_traces.json`` holds the scripts and what the reference's ``src/core`` printed
for them (made by ``tests/golden/make_core_traces.py``, which compiles the reference's sources with
``reference_core_trace.cpp``).  Where the reference's source tree and a C++ compiler are on this
machine, the reference side is built and run again, so the stored lines cannot go stale.
"""
import json
import os
import shutil
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_core_traces as mct  # noqa: E402

with open(os.path.join(HERE, "golden", "core_traces.json")) as f:
    GOLDEN = json.load(f)


def first_difference(ours, theirs, ops):
    for i, (a, b) in enumerate(zip(ours, theirs)):
        if a != b:
            return f"operation {i} '{ops[i][:60]}': ours {a} reference {b}"
    if len(ours) != len(theirs):
        return f"{len(ours)} lines against {len(theirs)}"
    return None


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_same_script_same_lines_as_the_reference(name):
    ops, reference = GOLDEN[name]["ops"], GOLDEN[name]["reference"]
    ours = mct.replay(ops)
    assert first_difference(ours, reference, ops) is None, first_difference(ours, reference, ops)


def test_scripts_cover_what_they_claim():
    """Prefix hits, evictions of parked pages, refused growth, blocked admissions and rejections all
    occur in the stored scripts (a script that never reaches them would prove nothing)."""
    last_stats = {n: [l for l in g["reference"] if l["op"] == "stats"][-1] for n, g in GOLDEN.items()}
    assert last_stats["paged_prefix"]["hits"] > 20 and last_stats["paged_prefix_tight"]["evictions"] > 10
    assert last_stats["paged_prefix"]["duplicates"] + last_stats["paged_prefix_tight"]["duplicates"] > 0
    grows = [l for g in GOLDEN.values() for l in g["reference"] if l["op"] == "grow"]
    assert any(l["ok"] == 0 for l in grows) and any(l["ok"] == 1 for l in grows)
    cans = [l for g in GOLDEN.values() for l in g["reference"] if l["op"] == "can"]
    assert any(l["ok"] == 0 for l in cans)
    counters = {n: g["reference"][-2] for n, g in GOLDEN.items() if n.startswith("scheduler")}
    assert all(c["preemptions"] == 0 for c in counters.values())
    assert sum(c["blocked"] for c in counters.values()) > 5 and sum(c["rejected"] for c in counters.values()) > 2
    assert counters["scheduler_prefix"]["saved"] > 0


def test_the_generator_still_makes_the_stored_scripts():
    """The scripts are a pure function of their seeds and of this core's answers."""
    for name, ops in mct.scenarios().items():
        assert ops == GOLDEN[name]["ops"], f"{name}: the generator no longer makes the stored script"


@pytest.mark.skipif(mct.reference_source() is None or shutil.which("g++") is None,
                    reason="the reference's source tree or g++ is not on this machine")
def test_stored_lines_are_what_the_reference_prints_now(tmp_path):
    exe = mct.build_reference_driver(mct.reference_source(), str(tmp_path))
    for name, g in GOLDEN.items():
        assert mct.run_reference(exe, g["ops"]) == g["reference"], name
