"""Plain-ASCII report helpers shared by the cost-model modules: a column-spec table renderer and
a ledger of named checks.  Every report of the package is text a terminal without Unicode can
show (the reference's CLI tests require ASCII output, ``tests/test_cli_ascii.py``)."""
from __future__ import annotations

from typing import Callable, Iterable, Sequence


class Column:
    """One column: header, ``%``-style cell format (applied to ``get(row)``) and header format."""

    def __init__(self, header: str, cell: str, get: Callable, head: str | None = None):
        self.header, self.cell, self.get = header, cell, get
        width = "".join(ch for ch in cell.split(".")[0] if ch.isdigit() or ch == "-")
        self.head = head or ("%" + width + "s")

    def title(self) -> str:
        return self.head % self.header

    def render(self, row) -> str:
        return self.cell % self.get(row)


def render_table(columns: Sequence[Column], rows: Iterable, rule: int | None = None,
                 sep: str = " ") -> list:
    """Header line, a dashed rule (``rule`` characters, default the header's length) and one line
    per row."""
    head = sep.join(c.title() for c in columns)
    out = [head, "-" * (rule if rule is not None else len(head))]
    out.extend(sep.join(c.render(r) for c in columns) for r in rows)
    return out


class Ledger:
    """Named pass/fail checks with the message to show when one fails; ``ok`` is their
    conjunction.  Keeps insertion order so that reports and tests read the same sequence."""

    def __init__(self):
        self.items: list = []

    def add(self, name: str, passed: bool, detail: str = "") -> bool:
        self.items.append((name, bool(passed), detail))
        return bool(passed)

    @property
    def ok(self) -> bool:
        return all(p for _, p, _ in self.items)

    def failures(self) -> list:
        return [(n, d) for n, p, d in self.items if not p]

    def as_dict(self) -> dict:
        return {n: p for n, p, _ in self.items}

    def lines(self, mark=("ok  ", "FAIL")) -> list:
        return ["  [%s] %s%s" % (mark[0] if p else mark[1], n, (" -- " + d) if d and not p else "")
                for n, p, d in self.items]
