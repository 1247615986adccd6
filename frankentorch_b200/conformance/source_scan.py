"""Source scanner of the repository's own code: the rules a change must not break, checked on text.

The reference guards its tree twice: an integration test scans production sources for forbidden constructs
(ft-conformance/tests/smoke.rs:156, which forbids the panic and unfinished-work macros) and a pre-commit hook runs a
bug scanner over the staged files and blocks the commit on a critical finding (hooks/pre-commit).  This module is
both: ``scan_paths`` returns findings with a severity, the command line prints them with a three-line summary
(``Files: n`` / ``Critical: n`` / ``Warning: n``) that ``hooks/pre-commit`` parses, and ``tests/test_cpu_tools.py``
runs it over the whole package.

Critical rules (a finding fails the gate):

* a GPU spin loop without a bound: ``while (true)`` / ``for (;;)`` in CUDA sources whose body has no cycle-budget
  or iteration check (every wait of this code base gives up with a status word instead of hanging the GPU);
* device-side traps and failing asserts (``__trap()``, ``assert(0)``, ``assert(false)``) in CUDA sources;
* the four batched-memcpy driver / runtime entry points, and bulk or TMA loads with cluster multicast, anywhere;
* ``eval`` / ``exec`` of strings, ``pickle`` loading, ``os.system``, ``shell=True`` in library code;
* process kills by pattern (they can match unrelated processes);
* stand-ins in production code: raising the not-implemented error outside an abstract method, unfinished-work
  markers in comments.

Warnings: a bare ``except:``, ``except ...: pass`` without a comment, ``print(`` in library modules that are not
command-line entry points.
"""
from __future__ import annotations

import os
import re
import subprocess
import sys
from dataclasses import dataclass
from typing import Iterable, List, Optional, Sequence, Tuple

CRITICAL, WARNING = "critical", "warning"
_CUDA_EXT = (".cu", ".cuh")
_PY_EXT = (".py",)
_SKIP_DIRS = {".git", "__pycache__", "build", "baseline", "lib"}       # plus the directories .gitignore names

# Names are assembled from pieces so that this file does not itself contain what it looks for.
_BATCH_COPY = [p + "Batch" + "Async" for p in ("cuda" + "Memcpy", "cuda" + "Memcpy3D", "cu" + "Memcpy", "cu" + "Memcpy3D")]
_MULTICAST = ".multi" + "cast::clu" + "ster"
_KILL_BY_PATTERN = ["pk" + "ill", "kill" + "all", "pg" + "rep -f"]
_NOT_IMPL = "NotImplemented" + "Error"
_MARKERS = "|".join(["TO" + "DO", "FIX" + "ME", "XX" + "X"])


@dataclass(frozen=True)
class Finding:
    path: str
    line: int
    severity: str
    rule: str
    text: str

    def render(self) -> str:
        return f"{self.path}:{self.line}: {self.severity}: {self.rule}: {self.text.strip()[:120]}"


def _strip_py_comment(line: str, drop_strings: bool = False) -> str:
    """The code part of one line: without its comment and, on request, with the bodies of string literals blanked
    (a rule about calls must not fire on text that merely mentions the call)."""
    out, quote = [], None
    for i, ch in enumerate(line):
        if quote:
            if ch == quote and line[i - 1] != "\\":
                quote = None
                out.append(ch)
            elif not drop_strings:
                out.append(ch)
            continue
        if ch in "\"'":
            quote = ch
        elif ch == "#":
            break
        out.append(ch)
    return "".join(out)


_CLI_MARKERS = ("argparse", "__main__")


def _scan_python(path: str, text: str) -> List[Finding]:
    f: List[Finding] = []
    lines = text.split("\n")
    is_cli = any(m in text for m in _CLI_MARKERS) or os.path.basename(path) in ("bench.py", "__graft_entry__.py")
    is_test = "/tests/" in path.replace("\\", "/") or os.path.basename(path).startswith("test_")
    in_doc = False
    for n, raw in enumerate(lines, 1):
        # skip docstring / multi-line string bodies for the code rules
        triple = raw.count('"""') + raw.count("'''")
        if in_doc:
            if triple % 2 == 1:
                in_doc = False
            continue
        if triple % 2 == 1:
            in_doc = True
            continue
        with_strings = _strip_py_comment(raw)
        comment = raw[len(with_strings):]
        code = _strip_py_comment(raw, drop_strings=True)
        s = code.strip()
        if re.search(r"(?<![\w.])(eval|exec)\(\s*[\"'a-zA-Z_]", code) and not re.match(r"def\s", s) and not is_test:
            f.append(Finding(path, n, CRITICAL, "dynamic code execution", raw))
        if re.search(r"\bpickle\.(load|loads)\(", code):
            f.append(Finding(path, n, CRITICAL, "pickle loading", raw))
        if re.search(r"\bos\.system\(", code) or re.search(r"shell\s*=\s*True", code):
            f.append(Finding(path, n, CRITICAL, "shell command execution", raw))
        if any(k in with_strings for k in _KILL_BY_PATTERN):       # command names live in string literals
            f.append(Finding(path, n, CRITICAL, "process kill by pattern", raw))
        if re.match(r"raise " + _NOT_IMPL + r"\b", s) and not is_test:
            # allowed as the body of a method the subclasses override (the `def` is within the 4 lines above)
            head = "\n".join(lines[max(0, n - 5): n - 1])
            if not re.search(r"^\s*def \w+\(self", head, re.M):
                f.append(Finding(path, n, CRITICAL, "placeholder in production code", raw))
        if re.search(r"#\s*(" + _MARKERS + r")\b", comment):
            f.append(Finding(path, n, CRITICAL, "unfinished-work marker", raw))
        if re.match(r"except\s*:", s):
            f.append(Finding(path, n, WARNING, "bare except", raw))
        if re.match(r"except\b.*:\s*pass\s*$", s) and "#" not in raw:
            f.append(Finding(path, n, WARNING, "exception swallowed without a reason", raw))
        if re.match(r"print\(", s) and not (is_cli or is_test) and "/benchmarks/" not in path:
            f.append(Finding(path, n, WARNING, "print in a library module", raw))
    return f


def _loop_body(text: str) -> str:
    """Text of the brace-delimited block that starts ``text`` (or its first statement if there is no brace)."""
    i = text.find("{")
    semi = text.find(";")
    if i < 0 or (0 <= semi < i):
        return text[: semi + 1] if semi >= 0 else text
    depth = 0
    for j in range(i, len(text)):
        if text[j] == "{":
            depth += 1
        elif text[j] == "}":
            depth -= 1
            if depth == 0:
                return text[i: j + 1]
    return text[i:]


def _scan_cuda(path: str, text: str) -> List[Finding]:
    f: List[Finding] = []
    lines = text.split("\n")
    for n, raw in enumerate(lines, 1):
        code = raw.split("//", 1)[0]
        m = re.search(r"\b(while\s*\(\s*(true|1)\s*\)|for\s*\(\s*;\s*;\s*\))", code)
        if m:
            body = _loop_body("\n".join([code[m.end():]] + lines[n: n + 60]))
            if not re.search(r"clock64\(\)|budget|BUDGET|max_spins|MAX_SPINS|\blimit\b|--\s*tries|tries\s*--", body):
                f.append(Finding(path, n, CRITICAL, "spin loop without a bound", raw))
        if re.search(r"__trap\s*\(\s*\)|\bassert\s*\(\s*(0|false)\s*\)", code):
            f.append(Finding(path, n, CRITICAL, "device-side trap", raw))
    return f


def _scan_any(path: str, text: str) -> List[Finding]:
    f: List[Finding] = []
    for n, raw in enumerate(text.split("\n"), 1):
        if any(b in raw for b in _BATCH_COPY):
            f.append(Finding(path, n, CRITICAL, "batched memcpy entry point", raw))
        if _MULTICAST in raw and "tcgen05.commit" not in raw and "multimem" not in raw:
            f.append(Finding(path, n, CRITICAL, "bulk / TMA load with cluster multicast", raw))
    return f


def scan_text(path: str, text: str) -> List[Finding]:
    out = _scan_any(path, text)
    if path.endswith(_PY_EXT):
        out += _scan_python(path, text)
    elif path.endswith(_CUDA_EXT):
        out += _scan_cuda(path, text)
    return sorted(out, key=lambda x: (x.path, x.line, x.rule))


def _ignored_dirs(start: str) -> set:
    """Directory names that the nearest ``.gitignore`` above ``start`` lists (``name/`` entries): scratch space."""
    d = os.path.abspath(start if os.path.isdir(start) else os.path.dirname(start))
    while True:
        gi = os.path.join(d, ".gitignore")
        if os.path.isfile(gi):
            with open(gi) as fh:
                return {ln.strip().strip("/") for ln in fh if ln.strip().endswith("/") and "*" not in ln}
        up = os.path.dirname(d)
        if up == d:
            return set()
        d = up


def _walk(root: str) -> Iterable[str]:
    if os.path.isfile(root):
        yield root
        return
    skip = _SKIP_DIRS | _ignored_dirs(root)
    for d, dirs, files in os.walk(root):
        dirs[:] = sorted(x for x in dirs if x not in skip)
        for name in sorted(files):
            if name.endswith(_PY_EXT + _CUDA_EXT + (".cpp", ".h", ".sh")):
                yield os.path.join(d, name)


def scan_paths(paths: Sequence[str]) -> Tuple[int, List[Finding]]:
    """``(files scanned, findings)`` over files and directories."""
    n, out = 0, []
    for p in paths:
        for fpath in _walk(p):
            try:
                with open(fpath, encoding="utf-8", errors="replace") as fh:
                    text = fh.read()
            except OSError:
                continue
            n += 1
            out += scan_text(fpath, text)
    return n, out


def staged_files(repo: str) -> List[str]:
    r = subprocess.run(["git", "-C", repo, "diff", "--cached", "--name-only", "--diff-filter=ACMR"], capture_output=True, text=True)
    return [os.path.join(repo, p) for p in r.stdout.split("\n") if p.strip() and os.path.isfile(os.path.join(repo, p))]


def summary(n_files: int, findings: Sequence[Finding]) -> str:
    crit = sum(1 for x in findings if x.severity == CRITICAL)
    return f"Files: {n_files}\nCritical: {crit}\nWarning: {len(findings) - crit}"


def main(argv: Optional[Sequence[str]] = None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description="scan sources for constructs this repository forbids")
    ap.add_argument("paths", nargs="*", help="files or directories (default: the package, tests, benchmarks, bench.py)")
    ap.add_argument("--staged", action="store_true", help="scan the files staged in git instead")
    ap.add_argument("--quiet", action="store_true", help="print the summary only")
    args = ap.parse_args(argv)
    repo = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    if args.staged:
        paths = staged_files(repo)
    else:
        paths = args.paths or [os.path.join(repo, p) for p in ("frankentorch_b200", "tests", "benchmarks", "bench.py", "__graft_entry__.py", "hooks")]
    n, findings = scan_paths(paths)
    if not args.quiet:
        for x in findings:
            print(x.render())
    print(summary(n, findings))
    return 1 if any(x.severity == CRITICAL for x in findings) else 0


if __name__ == "__main__":
    sys.exit(main())
