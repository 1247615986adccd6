"""Who was measured: the incumbent reports its own version, or there is no ratio.

Behaviour of ft-api/src/harness_provenance.rs (:37 ``VERSION_MARKER``, :55
``parse_reported_version``, :79 ``require_reported_version``, :90 ``payload_line``, :107
``version_disagreement``, :206 ``incumbent_provenance_block``): the benchmark's PyTorch arm prints
``PT_TORCH_VERSION <version>`` itself, from inside the interpreter that produced the timings; the
harness never fills the version in from its own environment, because the arm may run under another
interpreter.  A payload without the marker is an unattributed measurement and is refused.
"""
from __future__ import annotations

from typing import Optional, Tuple

VERSION_MARKER = "PT_TORCH_VERSION "
VERSION_PROBE_PY = "print('PT_TORCH_VERSION %s' % torch.__version__, flush=True)"


class MissingIncumbentVersion(RuntimeError):
    def __init__(self):
        super().__init__("the incumbent arm did not report its version (no 'PT_TORCH_VERSION <v>' line): "
                         "a ratio against an unidentified incumbent is not quotable")


def parse_reported_version(stdout: str) -> Optional[str]:
    """The version on the first well-formed marker line, or None."""
    for line in stdout.splitlines():
        line = line.strip()
        if line.startswith(VERSION_MARKER):
            v = line[len(VERSION_MARKER):].strip()
            if v and not any(c.isspace() for c in v):
                return v
    return None


def require_reported_version(stdout: str) -> str:
    v = parse_reported_version(stdout)
    if v is None:
        raise MissingIncumbentVersion()
    return v


def payload_line(stdout: str) -> Optional[str]:
    """The last non-empty line that is not a marker line (the arm's JSON payload)."""
    for line in reversed(stdout.splitlines()):
        t = line.strip()
        if t and not t.startswith("PT_"):
            return t
    return None


def version_disagreement(first: Tuple[str, str], observed: Tuple[str, str]) -> Optional[str]:
    """``(lane, version)`` pairs of two lanes of one run: a message when the versions differ."""
    if first[1] == observed[1]:
        return None
    return (f"incumbent version moved inside one run: lane '{first[0]}' reported {first[1]}, lane "
            f"'{observed[0]}' reported {observed[1]}; ratios of this run are not comparable")


def incumbent_provenance_block(version: str, threads: int = 0, extra: Optional[dict] = None) -> dict:
    """The provenance record that accompanies every quoted ratio."""
    out = {"incumbent": "pytorch", "incumbent_version": version, "version_source": "self-reported by the arm"}
    if threads:
        out["incumbent_threads"] = int(threads)
    if extra:
        out.update(extra)
    return out
