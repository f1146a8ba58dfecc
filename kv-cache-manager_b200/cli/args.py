"""Command-line flags in the reference's manner (``src/common/args.h:12-58``): ``--key=value``,
``--key value`` or a bare ``--flag`` (= "1"); typed getters with the default at the call site;
``warn_unused()`` names every flag nobody read, which catches typos."""
from __future__ import annotations

import sys
from typing import Dict, List, Optional, Set


class Args:
    def __init__(self, argv: Optional[List[str]] = None) -> None:
        argv = list(sys.argv[1:] if argv is None else argv)
        self.kv: Dict[str, str] = {}
        self.used: Set[str] = set()
        i = 0
        while i < len(argv):
            a = argv[i]
            if not a.startswith("--"):
                raise ValueError(f"bad argument: {a}")
            a = a[2:]
            if "=" in a:
                k, v = a.split("=", 1)
                self.kv[k] = v
            elif i + 1 < len(argv) and not argv[i + 1].startswith("--"):
                self.kv[a] = argv[i + 1]
                i += 1
            else:
                self.kv[a] = "1"
            i += 1

    def has(self, k: str) -> bool:
        self.used.add(k)
        return k in self.kv

    def str(self, k: str, default: str) -> str:
        self.used.add(k)
        return self.kv.get(k, default)

    def i64(self, k: str, default: int) -> int:
        s = self.str(k, "")
        return int(s) if s else default

    i32 = i64

    def f64(self, k: str, default: float) -> float:
        s = self.str(k, "")
        return float(s) if s else default

    def flag(self, k: str, default: bool = False) -> bool:
        s = self.str(k, "")
        return s in ("1", "true", "on", "yes") if s else default

    def ints(self, k: str, default: str) -> List[int]:
        return [int(x) for x in self.str(k, default).split(",") if x]

    def warn_unused(self) -> None:
        for k in self.kv:
            if k not in self.used:
                print(f"warning: unused flag --{k}", file=sys.stderr)
