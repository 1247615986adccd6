"""Optional runtime integration points (ft-runtime/src/lib.rs:199-220, behind the reference's
``asupersync-integration`` and ``frankentui-integration`` features).

``asupersync_infinite_budget`` gives the budget a caller passes to a structured-concurrency region when the
helper itself should impose no limit (offline inference, batch orchestration): no deadline, no poll quota,
no cost quota, lowest priority.  ``frankentui_default_style`` gives the baseline style of the text dashboard
that ``render_ledger_panel`` draws from a session's evidence ledger.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .ledger import EvidenceKind, EvidenceLedger


@dataclass(frozen=True)
class Budget:
    """Limits of a cancellable region: wall-clock deadline (unix ms), polls, abstract cost, priority."""
    deadline_unix_ms: Optional[int] = None
    poll_quota: Optional[int] = None
    cost_quota: Optional[int] = None
    priority: int = 0

    def is_infinite(self) -> bool:
        return self.deadline_unix_ms is None and self.poll_quota is None and self.cost_quota is None

    def exhausted(self, now_unix_ms: int, polls: int = 0, cost: int = 0) -> bool:
        return ((self.deadline_unix_ms is not None and now_unix_ms >= self.deadline_unix_ms)
                or (self.poll_quota is not None and polls >= self.poll_quota)
                or (self.cost_quota is not None and cost >= self.cost_quota))

    def meet(self, other: "Budget") -> "Budget":
        """The tighter of two budgets, field by field (a child region never outlives its parent)."""
        def tight(a, b):
            return b if a is None else (a if b is None else min(a, b))
        return Budget(tight(self.deadline_unix_ms, other.deadline_unix_ms), tight(self.poll_quota, other.poll_quota),
                      tight(self.cost_quota, other.cost_quota), max(self.priority, other.priority))


Budget.INFINITE = Budget()


def asupersync_infinite_budget() -> Budget:
    return Budget.INFINITE


@dataclass(frozen=True)
class Style:
    """Presentation of a dashboard panel: colours as names (``None`` = terminal default) and text attributes."""
    fg: Optional[str] = None
    bg: Optional[str] = None
    bold: bool = False
    dim: bool = False
    border: str = "plain"          # plain | rounded | none
    width: int = 100


def frankentui_default_style() -> Style:
    return Style()


_BORDERS = {"plain": ("+", "-", "|"), "rounded": (".", "-", "|"), "none": ("", "", "")}


def render_ledger_panel(ledger: EvidenceLedger, style: Optional[Style] = None, last: int = 10, title: str = "evidence") -> str:
    """Text panel with the ledger's totals per kind and its latest ``last`` entries, clipped to ``style.width``."""
    st = style or frankentui_default_style()
    corner, hbar, vbar = _BORDERS[st.border]
    inner = max(20, st.width - 2 * len(vbar))
    entries = ledger.entries()
    counts = {k: 0 for k in EvidenceKind}
    for e in entries:
        counts[e.kind] += 1
    lines = [f"{title}: {ledger.total_recorded} recorded, {len(entries)} kept  " +
             "  ".join(f"{k.name}={v}" for k, v in counts.items() if v)]
    lines += [f"{e.kind.name:<10} {e.summary}" for e in entries[-last:]]
    body = [vbar + ln[:inner].ljust(inner) + vbar for ln in lines]
    if not corner:
        return "\n".join(b.rstrip() for b in body)
    bar = corner + hbar * inner + corner
    return "\n".join([bar] + body + [bar])
