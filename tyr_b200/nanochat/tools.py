"""Tool execution for the generation engine: a safe arithmetic calculator (recursive-descent parser, no ``eval``)
and placeholder prover / eval tools (Examples/NanoChat/Generator/Tools.lean)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Tuple


@dataclass
class ExecResult:
    success: bool
    output: str = ""
    error: Optional[str] = None
    timed_out: bool = False

    @staticmethod
    def ok(output: str) -> "ExecResult":
        return ExecResult(True, output)

    @staticmethod
    def fail(error: str) -> "ExecResult":
        return ExecResult(False, "", error)

    @staticmethod
    def timeout() -> "ExecResult":
        return ExecResult(False, "", "timed out", True)


CALC_SAFE_CHARS = "0123456789+-*/.()^ "


def is_calc_safe(s: str) -> bool:
    return all(c in CALC_SAFE_CHARS for c in s)


class _Parser:
    """expr := term (('+'|'-') term)* ; term := factor (('*'|'/') factor)* ; factor := base ('^' factor)? ;
    base := number | '(' expr ')' | '-' base"""

    def __init__(self, text: str):
        self.s, self.i = text, 0

    def _ws(self):
        while self.i < len(self.s) and self.s[self.i] == " ":
            self.i += 1

    def _peek(self) -> Optional[str]:
        self._ws()
        return self.s[self.i] if self.i < len(self.s) else None

    def number(self) -> float:
        self._ws()
        j, dot = self.i, False
        while j < len(self.s) and (self.s[j].isdigit() or (self.s[j] == "." and not dot)):
            dot |= self.s[j] == "."
            j += 1
        if j == self.i or self.s[self.i:j] == ".":
            raise ValueError(f"expected a number at position {self.i}")
        v = float(self.s[self.i:j])
        self.i = j
        return v

    def base(self) -> float:
        c = self._peek()
        if c == "(":
            self.i += 1
            v = self.expr()
            if self._peek() != ")":
                raise ValueError("expected ')'")
            self.i += 1
            return v
        if c == "-":
            self.i += 1
            return -self.base()
        return self.number()

    def factor(self) -> float:
        b = self.base()
        if self._peek() == "^":
            self.i += 1
            return math.pow(b, self.factor())
        return b

    def term(self) -> float:
        v = self.factor()
        while self._peek() in ("*", "/"):
            op = self.s[self.i]
            self.i += 1
            r = self.factor()
            if op == "/":
                if r == 0.0:
                    raise ValueError("division by zero")
                v /= r
            else:
                v *= r
        return v

    def expr(self) -> float:
        v = self.term()
        while self._peek() in ("+", "-"):
            op = self.s[self.i]
            self.i += 1
            r = self.term()
            v = v + r if op == "+" else v - r
        return v


def eval_calc(text: str) -> float:
    p = _Parser(text)
    v = p.expr()
    if p._peek() is not None:
        raise ValueError(f"unexpected character {p._peek()!r} at position {p.i}")
    return v


def format_float(f: float) -> str:
    if f == math.floor(f) and abs(f) < 1e15:
        return str(int(f))
    return repr(f)


@dataclass
class Tool:
    name: str
    can_execute: Callable[[str], bool]
    execute: Callable[[str], ExecResult]


def _calc(inp: str) -> ExecResult:
    try:
        return ExecResult.ok(format_float(eval_calc(inp.strip())))
    except (ValueError, OverflowError) as e:
        return ExecResult.fail(str(e))


calculator_tool = Tool("calculator", lambda s: is_calc_safe(s) and "**" not in s, _calc)
lean_prover_tool = Tool("prover", lambda s: any(w in s for w in ("theorem", "lemma", "by")), lambda s: ExecResult.fail("Prover not yet implemented"))
lean_eval_tool = Tool("eval", lambda s: s.startswith("#eval") or s.startswith("#reduce"), lambda s: ExecResult.fail("Eval not yet implemented"))


@dataclass
class ToolRegistry:
    tools: List[Tool] = field(default_factory=lambda: [calculator_tool, lean_prover_tool, lean_eval_tool])

    def execute(self, tool_name: str, inp: str) -> ExecResult:
        for t in self.tools:
            if t.name == tool_name:
                return t.execute(inp)
        return ExecResult.fail(f"Unknown tool: {tool_name}")

    def dispatch(self, inp: str) -> ExecResult:
        for t in self.tools:
            if t.can_execute(inp):
                return t.execute(inp)
        return ExecResult.fail("No tool matched input")
