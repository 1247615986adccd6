"""When the arms are sampled: interleaved, in a balanced order, with an A/A null.

Behaviour of ft-api/src/harness_interleave.rs: the incumbent runs as a request / response
co-process (:42 ``PT_READY``, ``SAMPLE <lane>`` -> ``PT_SAMPLE <lane> <ms> <checksum>``, ``QUIT``), one
round has eight slots in the balanced-square order (:60: each arm sits twice in each half and
equally often at every position, so drift is common-mode), a fixed number of incumbent samples is
spread evenly over the rounds (``incumbent_sample_rounds``), both arms must time the same region
(``PT_TIMED_STEPS``), and a ratio is quoted only when each arm's first-half / second-half null
interval is narrow and contains 1 (``adjudicate_null``).
"""
from __future__ import annotations

import enum
import math
import statistics
import subprocess
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

READY_MARKER = "PT_READY"
SAMPLE_MARKER = "PT_SAMPLE "
REQUEST_PREFIX = "SAMPLE "
QUIT_REQUEST = "QUIT"
TIMED_STEPS_MARKER = "PT_TIMED_STEPS "
# incumbent (True) / ours (False): two of each in either half, every position taken equally often
BALANCED_SQUARE: Tuple[bool, ...] = (True, False, False, True, True, False, False, True)
MAX_NULL_CI_WIDTH = 0.60


@dataclass(frozen=True)
class IncumbentSample:
    lane: str
    milliseconds: float
    gradient_checksum: float


class NullVerdict(enum.Enum):
    Calm = "PASS"
    TooWide = "WIDE"
    OffCentre = "FAIL"

    @property
    def is_quotable(self) -> bool:
        return self is NullVerdict.Calm


def incumbent_sample_rounds(rounds: int, samples: int) -> List[int]:
    """Exactly ``min(samples, rounds)`` round indices spread evenly over ``range(rounds)``."""
    if rounds <= 0 or samples <= 0:
        return []
    samples = min(samples, rounds)
    return [r for r in range(rounds) if (r * samples) // rounds != ((r + 1) * samples) // rounds]


def sample_request(lane: str) -> str:
    return REQUEST_PREFIX + lane


def parse_sample_line(line: str) -> Optional[IncumbentSample]:
    """A well-formed ``PT_SAMPLE <lane> <ms> <checksum>`` line, else None (negative or non-finite
    durations are broken measurements, not slow ones)."""
    t = line.strip()
    if not t.startswith(SAMPLE_MARKER):
        return None
    f = t[len(SAMPLE_MARKER):].split()
    if len(f) < 3:
        return None
    try:
        ms, ck = float(f[1]), float(f[2])
    except ValueError:
        return None
    if not math.isfinite(ms) or ms < 0.0:
        return None
    return IncumbentSample(f[0], ms, ck)


def parse_timed_steps(stdout: str) -> Optional[List[str]]:
    for line in stdout.splitlines():
        t = line.strip()
        if t.startswith(TIMED_STEPS_MARKER):
            v = t[len(TIMED_STEPS_MARKER):].strip()
            if v:
                return [s.strip() for s in v.split(",")]
    return None


def timed_region_disagreement(ours: Sequence[str], incumbent: Sequence[str]) -> Optional[str]:
    if list(ours) == list(incumbent):
        return None
    only_ours = [s for s in ours if s not in incumbent]
    only_theirs = [s for s in incumbent if s not in ours]
    return (f"the two arms did not time the same region: ours {list(ours)}, incumbent {list(incumbent)} "
            f"(only ours: {only_ours}; only theirs: {only_theirs}); no ratio from this run is quotable")


def adjudicate_null(low: float, high: float, max_width: float = MAX_NULL_CI_WIDTH) -> NullVerdict:
    if not (math.isfinite(low) and math.isfinite(high)) or high < low or high - low > max_width:
        return NullVerdict.TooWide
    return NullVerdict.Calm if low <= 1.0 <= high else NullVerdict.OffCentre


NULL_RESOLUTION = 0.01      # a half-to-half shift below 1 % is under what a handful of samples can resolve


def aa_null(samples: Sequence[float], resolution: float = NULL_RESOLUTION) -> Tuple[float, float, NullVerdict]:
    """First-half / second-half null of one arm's samples (taken in time order): the interval spanned
    by the ratios of paired samples (i-th of the first half over i-th of the second), widened by the
    measurement resolution on either side, and its verdict.  An arm that drifted between the halves
    (thermal state, a neighbour's load) fails it, and no ratio involving that arm is quoted."""
    n = len(samples) // 2
    if n == 0:
        return float("nan"), float("nan"), NullVerdict.TooWide
    ratios = [samples[i] / samples[n + i] for i in range(n) if samples[n + i] > 0]
    if not ratios:
        return float("nan"), float("nan"), NullVerdict.TooWide
    lo, hi = min(ratios) - resolution, max(ratios) + resolution
    return lo, hi, adjudicate_null(lo, hi)


@dataclass
class HeadToHead:
    """Result of an interleaved comparison: per-arm samples (ms), the ratio of medians
    (incumbent / ours: above 1 means ours is faster) and whether it may be quoted."""
    ours_ms: List[float] = field(default_factory=list)
    incumbent_ms: List[float] = field(default_factory=list)
    order: str = "balanced-square"
    null_ours: Tuple[float, float, str] = (float("nan"), float("nan"), "WIDE")
    null_incumbent: Tuple[float, float, str] = (float("nan"), float("nan"), "WIDE")
    refused: Optional[str] = None

    @property
    def ratio(self) -> Optional[float]:
        if self.refused or not self.ours_ms or not self.incumbent_ms:
            return None
        return statistics.median(self.incumbent_ms) / statistics.median(self.ours_ms)

    @property
    def quotable(self) -> bool:
        return self.refused is None and self.null_ours[2] == "PASS" and self.null_incumbent[2] == "PASS"

    def as_dict(self) -> Dict:
        return {"ratio_incumbent_over_ours": self.ratio, "quotable": self.quotable, "order": self.order,
                "ours_ms_median": statistics.median(self.ours_ms) if self.ours_ms else None,
                "incumbent_ms_median": statistics.median(self.incumbent_ms) if self.incumbent_ms else None,
                "samples_per_arm": len(self.ours_ms),
                "aa_null_ours": list(self.null_ours), "aa_null_incumbent": list(self.null_incumbent),
                "refused": self.refused}


def run_balanced_square(ours: Callable[[], float], incumbent: Callable[[], float], rounds: int = 1,
                        ours_steps: Sequence[str] = (), incumbent_steps: Sequence[str] = ()) -> HeadToHead:
    """Sample the two arms in the balanced-square slot order, ``rounds`` times.  Each callable returns
    one timed sample in milliseconds.  If both step lists are given and differ, the ratio is refused."""
    res = HeadToHead()
    if ours_steps and incumbent_steps:
        res.refused = timed_region_disagreement(ours_steps, incumbent_steps)
    for _ in range(max(1, rounds)):
        for slot_is_incumbent in BALANCED_SQUARE:
            (res.incumbent_ms if slot_is_incumbent else res.ours_ms).append(float((incumbent if slot_is_incumbent else ours)()))
    lo, hi, v = aa_null(res.ours_ms)
    res.null_ours = (lo, hi, v.value)
    lo, hi, v = aa_null(res.incumbent_ms)
    res.null_incumbent = (lo, hi, v.value)
    return res


class CoProcessArm:
    """The incumbent as a request / response child process: blocks until ``PT_READY``, then returns
    one ``PT_SAMPLE`` per ``SAMPLE <lane>`` request.  The child's version line is mandatory."""

    def __init__(self, argv: Sequence[str], timeout_s: float = 600.0):
        from .provenance import require_reported_version
        self.proc = subprocess.Popen(list(argv), stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
        head = []
        while True:
            line = self.proc.stdout.readline()
            if not line:
                raise RuntimeError("the incumbent co-process exited before announcing " + READY_MARKER)
            head.append(line)
            if line.strip() == READY_MARKER:
                break
        self.preamble = "".join(head)
        self.version = require_reported_version(self.preamble)
        self.timed_steps = parse_timed_steps(self.preamble)

    def sample(self, lane: str) -> IncumbentSample:
        self.proc.stdin.write(sample_request(lane) + "\n")
        self.proc.stdin.flush()
        while True:
            line = self.proc.stdout.readline()
            if not line:
                raise RuntimeError("the incumbent co-process died while a sample was pending")
            s = parse_sample_line(line)
            if s is not None:
                if s.lane != lane:
                    raise RuntimeError(f"sample for lane '{s.lane}' answered a request for '{lane}'")
                return s

    def close(self) -> None:
        try:
            self.proc.stdin.write(QUIT_REQUEST + "\n")
            self.proc.stdin.flush()
            self.proc.wait(timeout=30)
        except Exception:
            self.proc.kill()
