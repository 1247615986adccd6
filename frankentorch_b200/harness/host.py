"""What the machine looked like while a head-to-head number was taken (ft-api/src/harness_provenance.rs:140-830,
harness_interleave.rs:299-365).

A ratio of two arms is only as good as the window it was measured in, so every quoted row carries: which code
ran (a digest of the kernel library and of this package, so an A/B whose rebuild never reached the loaded file
is caught), which host and GPU, whether another measurement announced itself or is visible in the process table
at the same time, how far apart the CPU cores' clocks were, and whether the load average drifted during the run.
All of it reports and none of it waits or refuses by itself: callers decide what is quotable with the
``*_is_quotable`` predicates, which fail closed on a missing reading.
"""
from __future__ import annotations

import enum
import glob
import hashlib
import math
import os
import platform
from typing import Callable, List, Optional, Sequence, Tuple

MAX_LOAD_DRIFT = 1.25                 # largest max/min of the 1-minute load average (floored at 1) within a run
CONTENTION_ACTIVE_FLOOR = 0.25        # CPU share (cores) above which a foreign measurement counts as active
LEGACY_BLOCK_ARMS_ENV = "FT_H2H_LEGACY_BLOCK_ARMS"
SLOT_DIR_ENV = "FT_H2H_SLOT_DIR"
_MEASUREMENT_MARKS = ("bench.py", "kernel_bench", "collective_bench", "ops_bench", "torch_baseline", "encoder_bench", "_h2h")


def _first_line(path: str) -> str:
    try:
        with open(path) as f:
            return f.readline().strip()
    except OSError:
        return ""


# ------------------------------------------------------------------------------------ which code ran
def executing_code_sha256() -> str:
    """Digest of what this process executes: the built kernel and host libraries plus the package sources.  Two
    arms of an A/B that print the same digest ran the same code, whatever the build log said."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    h = hashlib.sha256()
    paths = sorted(glob.glob(os.path.join(root, "lib", "*.so"))) + sorted(glob.glob(os.path.join(root, "**", "*.py"), recursive=True))
    for p in paths:
        h.update(os.path.relpath(p, root).encode())
        try:
            with open(p, "rb") as f:
                h.update(f.read())
        except OSError:
            h.update(b"<unreadable>")
    return h.hexdigest()


executing_elf_sha256 = executing_code_sha256     # the reference's name (it hashes its one executable)


def identical_arm_digests(before: str, after: str) -> Optional[str]:
    """``None`` when the two arms of an A/B ran different code; otherwise the message to fail with."""
    if before.strip() != after.strip() or not before.strip():
        return None
    return (f"both A/B arms executed the SAME code (executing_code_sha256={before.strip()}): the rebuild did not reach "
            "the files that were loaded, so one build was measured twice and any delta is noise")


# ------------------------------------------------------------------------------------ arm ordering
class ArmOrdering(enum.Enum):
    Interleaved = "interleaved"
    LegacyBlock = "legacy_block"

    def label(self) -> str:
        return ("INTERLEAVED per round (default)" if self is ArmOrdering.Interleaved
                else "LEGACY BLOCK - whole incumbent arm first (NOT quotable)")

    def is_quotable(self) -> bool:
        return self is ArmOrdering.Interleaved


def arm_ordering_from_env(value: Optional[str] = None) -> ArmOrdering:
    """``FT_H2H_LEGACY_BLOCK_ARMS`` = 1 / true / yes selects the block order kept for comparisons with old rows."""
    v = os.environ.get(LEGACY_BLOCK_ARMS_ENV) if value is None else value
    return ArmOrdering.LegacyBlock if (v or "").strip().lower() in ("1", "true", "yes") else ArmOrdering.Interleaved


def interpreter_args(script: str) -> List[str]:
    """Arguments that make an interpreter run ``script`` given inline (the co-process arm is started this way, so
    the arm's source is part of the command line and of the provenance)."""
    return ["-c", script]


# ------------------------------------------------------------------------------------ host, clocks, load
def measurement_host_block(cpu_threads: int = 0) -> str:
    host = _first_line("/proc/sys/kernel/hostname") or platform.node() or "unknown"
    cpu = "unknown"
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name"):
                    cpu = line.split(":", 1)[1].strip()
                    break
    except OSError:
        pass
    governor = _first_line("/sys/devices/system/cpu/cpu0/cpufreq/scaling_governor") or "unknown"
    gpu = "none"
    try:
        import torch
        if torch.cuda.is_available():
            p = torch.cuda.get_device_properties(0)
            gpu = f"{p.name} sm_{p.major}{p.minor} x{torch.cuda.device_count()} ({p.multi_processor_count} SMs)"
    except Exception:       # a host block must never take a measurement down
        gpu = "unknown"
    return (f"measurement_host={host} cpu={cpu!r} isa={platform.machine()} governor={governor} cpu_threads={cpu_threads} "
            f"online_cpus={os.cpu_count() or 'unknown'} gpu={gpu!r}\n"
            "host_rule=both arms are sampled in ONE invocation on THIS machine; a row measured elsewhere is not "
            "comparable to this one, A/A PASS or not")


def cpu_mhz_sorted() -> List[float]:
    """Instantaneous per-core clocks in MHz, ascending (cpufreq sysfs, else /proc/cpuinfo); empty if unknown."""
    out: List[float] = []
    cpu = 0
    while True:
        v = _first_line(f"/sys/devices/system/cpu/cpu{cpu}/cpufreq/scaling_cur_freq")
        if not v:
            break
        try:
            out.append(float(v) / 1000.0)
        except ValueError:
            break
        cpu += 1
    if not out:
        try:
            with open("/proc/cpuinfo") as f:
                for line in f:
                    if line.lower().startswith("cpu mhz"):
                        out.append(float(line.split(":", 1)[1]))
        except (OSError, ValueError):
            pass
    return sorted(out)


def cpu_mhz_stats() -> Optional[Tuple[float, float, float, float]]:
    """``(min, median, max, max / min)`` of the per-core clocks."""
    mhz = cpu_mhz_sorted()
    if not mhz:
        return None
    lo, hi = mhz[0], mhz[-1]
    return lo, mhz[len(mhz) // 2], hi, (hi / lo if lo > 0 else math.nan)


def cpu_clock_block(pinned: Optional[str] = None) -> str:
    st = cpu_mhz_stats()
    if st is None:
        return ("cpu_mhz=UNAVAILABLE (no cpufreq sysfs and no /proc/cpuinfo MHz); this host cannot show whether the two "
                "arms ran at comparable clocks")
    lo, med, hi, spread = st
    how = (f"arms pinned to the SAME core set [{pinned}], so both saw the same clock domain" if pinned else
           "arms NOT pinned: host threads of the two arms land wherever the scheduler puts them, so their CPU parts are "
           "NOT known to have run at comparable clocks (the GPU clocks of the timed region are in the bench line)")
    return f"cpu_mhz min={lo:.0f} median={med:.0f} max={hi:.0f} spread={spread:.3f}x; {how}"


def load_average_1m() -> Optional[float]:
    try:
        return float(_first_line("/proc/loadavg").split()[0])
    except (IndexError, ValueError):
        return None


def _floored_range(samples: Sequence[float]) -> Optional[Tuple[float, float]]:
    lo, hi = math.inf, 0.0
    for s in samples:
        if s is None or not math.isfinite(s) or s < 0:
            return None                    # a malformed reading fails closed instead of being skipped
        v = max(float(s), 1.0)             # 0.2 -> 0.5 on an idle host is 2.5x and means nothing
        lo, hi = min(lo, v), max(hi, v)
    return lo, hi


def load_drift_is_quotable(start: Optional[float], end: Optional[float]) -> bool:
    """Steady load is measurable at any level; what disqualifies a run is drift.  Unknown drift is not quotable."""
    if start is None or end is None:
        return False
    r = _floored_range([start, end])
    return r is not None and r[1] / r[0] <= MAX_LOAD_DRIFT


def load_series_is_quotable(samples: Sequence[float]) -> bool:
    """As ``load_drift_is_quotable`` over readings taken during the run (a spike in the middle counts)."""
    if len(samples) < 2:
        return False
    r = _floored_range(samples)
    return r is not None and r[1] / r[0] <= MAX_LOAD_DRIFT


def load_series_drift(samples: Sequence[float]) -> Optional[float]:
    if len(samples) < 2:
        return None
    r = _floored_range(samples)
    return None if r is None else r[1] / r[0]


# ------------------------------------------------------------------------------------ other measurements on the host
def _cmdline(pid: int) -> str:
    try:
        with open(f"/proc/{pid}/cmdline", "rb") as f:
            return f.read().replace(b"\0", b" ").decode(errors="replace").strip()
    except OSError:
        return ""


def _is_measurement(cmdline: str) -> bool:
    return any(m in cmdline for m in _MEASUREMENT_MARKS)


def _cpu_share(pid: int) -> float:
    """Average number of cores the process has used since it started (utime + stime over its age)."""
    try:
        with open(f"/proc/{pid}/stat") as f:
            fields = f.read().rsplit(")", 1)[1].split()
        ticks = os.sysconf("SC_CLK_TCK")
        used = (int(fields[11]) + int(fields[12])) / ticks
        uptime = float(_first_line("/proc/uptime").split()[0])
        age = uptime - int(fields[19]) / ticks
        return used / age if age > 0 else 0.0
    except (OSError, IndexError, ValueError):
        return 0.0


def concurrent_measurement_processes(exclude: Sequence[int] = ()) -> List[Tuple[int, str, float]]:
    """``(pid, command line, CPU share)`` of other processes that look like measurements (this process, its
    ancestors and its children are not "other")."""
    mine = {os.getpid(), *exclude}
    pid = os.getpid()
    for _ in range(16):                     # ancestors: the shell or launcher that started this run
        try:
            with open(f"/proc/{pid}/stat") as f:
                pid = int(f.read().rsplit(")", 1)[1].split()[1])
        except (OSError, ValueError, IndexError):
            break
        if pid <= 1:
            break
        mine.add(pid)
    out = []
    for d in glob.glob("/proc/[0-9]*"):
        p = int(os.path.basename(d))
        if p in mine:
            continue
        try:
            with open(f"{d}/stat") as f:
                ppid = int(f.read().rsplit(")", 1)[1].split()[1])
        except (OSError, ValueError, IndexError):
            continue
        if ppid in mine:                    # this run's own ranks / co-process arm
            continue
        c = _cmdline(p)
        if c and _is_measurement(c):
            out.append((p, c[:120], _cpu_share(p)))
    return sorted(out)


def concurrent_measurement_block() -> str:
    """A report, never a refusal or a wait: which other measurement-shaped processes were alive at the start."""
    others = concurrent_measurement_processes()
    if not others:
        return "concurrent_measurements=none of the shapes this scan knows (that is not the same as a quiet host)"
    active = [o for o in others if o[2] >= CONTENTION_ACTIVE_FLOOR]
    idle = [o for o in others if o[2] < CONTENTION_ACTIVE_FLOOR]
    def fmt(rows):
        return " | ".join(f"pid={p} cpu={s:.2f} {c}" for p, c, s in rows)
    parts = [f"concurrent_measurements={len(others)} ({len(active)} active, {len(idle)} idle)"]
    if active:
        parts.append("ACTIVE: " + fmt(active) + " - rows from this window share the machine with them and are not quotable")
    if idle:
        parts.append("idle: " + fmt(idle))
    return "; ".join(parts)


class MeasurementSlot:
    """An announcement that this process is measuring; removed by ``release()`` or when the object goes away."""

    def __init__(self, path: str):
        self.path = path

    def release(self) -> None:
        try:
            os.remove(self.path)
        except OSError:
            pass

    __del__ = release

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.release()


def _slot_holder_is_live(pid: int) -> bool:
    """A bare /proc/<pid> check would accept a recycled pid of something else and strand the slot for ever."""
    return _is_measurement(_cmdline(pid))


def announce_measurement(label: str, is_live: Callable[[int], bool] = _slot_holder_is_live) -> Tuple[Optional[MeasurementSlot], str]:
    """Write ``<pid>.slot`` into the slot directory (``FT_H2H_SLOT_DIR``, default under the system temp directory) and
    report every other live announcement.  Advisory: it never waits.  Slots of dead or recycled pids are removed
    on sight, so the directory heals itself.  Keep the returned slot bound for the length of the run."""
    import tempfile
    d = os.environ.get(SLOT_DIR_ENV) or os.path.join(tempfile.gettempdir(), "ft-h2h-slots")
    try:
        os.makedirs(d, exist_ok=True)
    except OSError:
        return None, (f"measurement_slot=UNAVAILABLE (cannot create {d}); overlap with another harness cannot be detected "
                      "in advance, only afterwards by the process scan")
    me = os.getpid()
    others = []
    for p in sorted(glob.glob(os.path.join(d, "*.slot"))):
        try:
            pid = int(os.path.basename(p)[:-5])
        except ValueError:
            continue
        if pid == me:
            continue
        if not is_live(pid):
            try:
                os.remove(p)
            except OSError:
                pass
            continue
        others.append(_first_line(p) or f"pid={pid}")
    digest = executing_code_sha256()[:16]
    record = f"pid={me} host={_first_line('/proc/sys/kernel/hostname') or platform.node()} code={digest} lanes={label}"
    path = os.path.join(d, f"{me}.slot")
    try:
        with open(path, "w") as f:
            f.write(record + "\n")
        slot = MeasurementSlot(path)
    except OSError:
        slot = None
    if not others:
        return slot, f"measurement_slot=held [{record}]; no other live announcement"
    return slot, (f"measurement_slot=OVERLAPPED [{record}]; {len(others)} other live announcement(s): {' | '.join(others)} - "
                  "those runs and this one sample the same machine at the same time; no row from an overlapped window "
                  "is quotable")
