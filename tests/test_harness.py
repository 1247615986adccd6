"""Measurement harness: provenance refusal, interleaving order, A/A null, co-process protocol
(ft-api/src/harness_provenance.rs, ft-api/src/harness_interleave.rs)."""
import sys
import textwrap

import pytest

from frankentorch_b200 import harness as H


def test_version_must_be_self_reported():
    out = "warming up\nPT_TORCH_VERSION 2.11.0+cu128\n{\"ms\": 1.0}\n"
    assert H.parse_reported_version(out) == "2.11.0+cu128" and H.require_reported_version(out) == "2.11.0+cu128"
    assert H.payload_line(out) == '{"ms": 1.0}'
    for bad in ("", "{\"ms\": 1.0}", "PT_TORCH_VERSION \n", "PT_TORCH_VERSION 2.1 extra words\n"):
        with pytest.raises(H.MissingIncumbentVersion):
            H.require_reported_version(bad)
    assert H.version_disagreement(("a", "2.11"), ("b", "2.11")) is None
    assert "moved" in H.version_disagreement(("a", "2.11"), ("b", "2.12"))
    assert H.incumbent_provenance_block("2.11", 8)["incumbent_threads"] == 8


def test_balanced_square_is_balanced():
    sq = H.BALANCED_SQUARE
    assert len(sq) == 8 and sum(sq) == 4
    assert sum(sq[:4]) == 2 and sum(sq[4:]) == 2                     # two of each arm in either half
    pos_inc = [i for i, s in enumerate(sq) if s]
    pos_our = [i for i, s in enumerate(sq) if not s]
    assert sum(pos_inc) == sum(pos_our)                               # a linear drift cancels in the means


def test_linear_drift_is_common_mode_and_a_step_change_fails_the_null():
    t = [0]

    def drifting(base):
        def f():
            t[0] += 1
            return base * (1.0 + 0.0005 * t[0])                        # both arms slow down 0.05 % per slot
        return f
    res = H.run_balanced_square(drifting(10.0), drifting(20.0), rounds=2)
    assert res.quotable and abs(res.ratio - 2.0) < 0.02
    t[0] = 0

    def stepping():
        t[0] += 1
        return 20.0 if t[0] <= 4 else 26.0                            # the incumbent got 30 % slower half way

    res = H.run_balanced_square(lambda: 10.0, stepping, rounds=2)
    assert not res.quotable and res.null_incumbent[2] == "FAIL" and res.null_ours[2] == "PASS"


def test_null_adjudication_and_region_agreement():
    assert H.adjudicate_null(0.98, 1.03) is H.NullVerdict.Calm
    assert H.adjudicate_null(1.02, 1.10) is H.NullVerdict.OffCentre
    assert H.adjudicate_null(0.5, 1.5) is H.NullVerdict.TooWide
    assert H.adjudicate_null(float("nan"), 1.0) is H.NullVerdict.TooWide
    assert H.timed_region_disagreement(["forward", "backward"], ["forward", "backward"]) is None
    msg = H.timed_region_disagreement(["forward", "backward"], ["forward", "backward", "checksum"])
    assert "only theirs: ['checksum']" in msg
    res = H.run_balanced_square(lambda: 1.0, lambda: 1.0, ours_steps=["forward"], incumbent_steps=["forward", "x"])
    assert res.ratio is None and not res.quotable and res.refused
    assert H.parse_timed_steps("x\nPT_TIMED_STEPS forward, backward\n") == ["forward", "backward"]


_CHILD = textwrap.dedent('''
    import sys
    print("PT_TORCH_VERSION 9.9.9", flush=True)
    print("PT_TIMED_STEPS forward,backward", flush=True)
    print("PT_READY", flush=True)
    n = 0
    for line in sys.stdin:
        line = line.strip()
        if line == "QUIT":
            break
        if line.startswith("SAMPLE "):
            n += 1
            print("noise line", flush=True)
            print("PT_SAMPLE %s %.3f %.1f" % (line[7:], 2.0 + 0.001 * n, 42.0), flush=True)
''')


def test_incumbent_co_process_protocol(tmp_path):
    script = tmp_path / "arm.py"
    script.write_text(_CHILD)
    arm = H.CoProcessArm([sys.executable, str(script)])
    try:
        assert arm.version == "9.9.9" and arm.timed_steps == ["forward", "backward"]
        s1 = arm.sample("mlp")
        assert s1.lane == "mlp" and abs(s1.milliseconds - 2.001) < 1e-9 and s1.gradient_checksum == 42.0
        res = H.run_balanced_square(lambda: 1.0, lambda: arm.sample("mlp").milliseconds, rounds=1)
        assert res.quotable and 1.9 < res.ratio < 2.1
    finally:
        arm.close()
    assert arm.proc.poll() is not None

    silent = tmp_path / "silent.py"
    silent.write_text("print('PT_READY', flush=True)\n")
    with pytest.raises(H.MissingIncumbentVersion):
        H.CoProcessArm([sys.executable, str(silent)])
