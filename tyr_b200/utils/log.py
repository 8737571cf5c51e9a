"""Log handlers: library code stays silent unless handlers are supplied (Tyr/Log.lean, Pipeline.LogHandlers)."""
from __future__ import annotations

import sys
import time
from dataclasses import dataclass
from typing import Callable

_noop = lambda msg: None


@dataclass
class Handlers:
    on_info: Callable[[str], None] = _noop
    on_warn: Callable[[str], None] = _noop
    on_error: Callable[[str], None] = _noop

    def combine(self, other: "Handlers") -> "Handlers":
        def both(a, b):
            def f(m):
                a(m)
                b(m)
            return f
        return Handlers(both(self.on_info, other.on_info), both(self.on_warn, other.on_warn), both(self.on_error, other.on_error))

    @staticmethod
    def stdout(prefix: str = "") -> "Handlers":
        return Handlers(lambda m: print(prefix + m, flush=True), lambda m: print(prefix + "WARN " + m, flush=True),
                        lambda m: print(prefix + "ERROR " + m, file=sys.stderr, flush=True))

    @staticmethod
    def to_file(path: str) -> "Handlers":
        def w(tag):
            def f(m):
                with open(path, "a", encoding="utf-8") as fh:
                    fh.write(f"{time.strftime('%H:%M:%S')} {tag}{m}\n")
            return f
        return Handlers(w(""), w("WARN "), w("ERROR "))

    def master_only(self, rank: int) -> "Handlers":
        return self if rank == 0 else Handlers()


LogHandlers = Handlers
