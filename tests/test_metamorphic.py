"""Self-oracle suites that need no external reference:

* in-place operators against their out-of-place forms
  (ft-conformance/tests/inplace_matches_out_of_place.rs);
* serial against parallel execution of the CPU reference kernels on both sides of the size
  gate, at several thread widths, bit for bit, including boundary values
  (ft-conformance/tests/threshold_serial_parallel_equivalence.rs);
* a scan of the production sources for constructs that must not ship
  (ft-conformance/tests/smoke.rs:156+).
"""
import ctypes as C
import pathlib
import re

import pytest
import torch

from frankentorch_b200.runtime import native
from frankentorch_b200.session import FrankenTorchSession

ROOT = pathlib.Path(__file__).resolve().parent.parent
PKG = ROOT / "frankentorch_b200"


# ------------------------------------------------------------------------------------ in-place vs out-of-place
_CASES = [
    ("add", lambda s, a, b: s.tensor_add_(a, b), lambda s, a, b: s.tensor_add(a, b), True),
    ("sub", lambda s, a, b: s.tensor_sub_(a, b), lambda s, a, b: s.tensor_sub(a, b), True),
    ("mul", lambda s, a, b: s.tensor_mul_(a, b), lambda s, a, b: s.tensor_mul(a, b), True),
    ("div", lambda s, a, b: s.tensor_div_(a, b), lambda s, a, b: s.tensor_div(a, b), True),
    ("neg", lambda s, a, b: s.tensor_neg_(a), lambda s, a, b: s.tensor_neg(a), False),
    ("clamp", lambda s, a, b: s.tensor_clamp_(a, -0.5, 0.75), lambda s, a, b: s.tensor_clamp(a, min=-0.5, max=0.75), False),
]


@pytest.mark.parametrize("name,inplace,outofplace,binary", _CASES, ids=[c[0] for c in _CASES])
@pytest.mark.parametrize("shape", [(1,), (7,), (3, 5), (2, 3, 4)])
def test_inplace_matches_out_of_place_bit_for_bit(name, inplace, outofplace, binary, shape):
    g = torch.Generator().manual_seed(hash((name, shape)) % 1000)
    n = 1
    for d in shape:
        n *= d
    av = (torch.randn(n, generator=g, dtype=torch.float64) * 2).tolist()
    bv = (torch.randn(n, generator=g, dtype=torch.float64) + 3.0).tolist()       # away from zero for div
    if name != "div":
        av[0] = -0.0                                                              # the sign of zero must survive
    s = FrankenTorchSession("strict")
    a = s.tensor_variable(av, list(shape), False)
    b = s.tensor_variable(bv, list(shape), False)
    want = s.tensor(outofplace(s, a, b)).clone()
    v0 = s.tensor_version(a)
    got_id = inplace(s, a, b)
    assert got_id == a and s.tensor_version(a) == v0 + 1
    got = s.tensor(a)
    assert torch.equal(got.view(torch.int64), want.view(torch.int64))             # bits, including -0.0
    assert tuple(got.shape) == tuple(shape)
    if binary:
        assert s.tensor_values(b) == bv                                           # the other operand is untouched


def test_inplace_fill_and_zero_and_repeated_application():
    s = FrankenTorchSession("strict")
    a = s.tensor_variable([1.0, -2.0, 3.5], [3], False)
    s.tensor_fill_(a, 0.25)
    assert s.tensor_values(a) == [0.25] * 3
    s.tensor_zero_(a)
    assert s.tensor_values(a) == [0.0] * 3 and s.tensor_version(a) == 2
    b = s.tensor_variable([1.0, 1.0, 1.0], [3], False)
    for _ in range(5):
        s.tensor_add_(a, b)
    ref = s.tensor_variable([0.0] * 3, [3], False)
    for _ in range(5):
        ref = s.tensor_add(ref, b)
    assert s.tensor_values(a) == s.tensor_values(ref) and s.tensor_version(a) == 7


def test_inplace_on_a_leaf_that_requires_grad_is_refused_and_allowed_without_grad_mode():
    s = FrankenTorchSession("strict")
    w = s.tensor_variable([1.0, 2.0], [2], True)
    d = s.tensor_variable([0.5, 0.5], [2], False)
    with pytest.raises(RuntimeError):
        s.tensor_sub_(w, d)
    with s.no_grad():
        s.tensor_sub_(w, d)
    assert s.tensor_values(w) == [0.5, 1.5]
    # gradients after the update see the new values, as with an out-of-place rebuild
    y = s.tensor_sum(s.tensor_mul(w, w))
    assert s.tensor_backward(y).gradient(w).tolist() == [1.0, 3.0]


# ------------------------------------------------------------------------------------ serial vs parallel
@pytest.fixture
def pool():
    lib = native.load()
    old_gate = lib.ftc_pool_set_min_work(-1)
    yield lib
    lib.ftc_pool_reset_for_tests()
    lib.ftc_pool_set_min_work(old_gate)


def _with_width(lib, width, gate, fn):
    lib.ftc_pool_reset_for_tests()
    changed = C.c_int(0)
    assert lib.ftc_pool_configure(str(width).encode(), C.byref(changed)) == width
    lib.ftc_pool_set_min_work(gate)
    return fn()


_BOUNDARY = [0.0, -0.0, 1.0, -1.0, 5e-324, -5e-324, 2.2250738585072014e-308, 1.7976931348623157e308 / 4,
             1e-300, 3.0000000000000004, 0.1, 1 / 3]


@pytest.mark.parametrize("gate", [256, 1 << 15])
def test_pairwise_sum_serial_equals_parallel_around_the_gate(pool, gate):
    lib = pool
    g = torch.Generator().manual_seed(1)
    for n in (1, 127, 128, 129, gate - 1, gate, gate + 1, 3 * gate + 17):
        x = torch.randn(n, generator=g, dtype=torch.float64) * 1e3
        x[: min(n, len(_BOUNDARY))] = torch.tensor(_BOUNDARY[: min(n, len(_BOUNDARY))], dtype=torch.float64)
        serial = lib.ftc_pairwise_sum(x.data_ptr(), n)
        for width in (1, 2, 3, 4, 8):
            par = _with_width(lib, width, gate, lambda: lib.ftc_pairwise_sum_par(x.data_ptr(), n))
            assert par == serial, (n, width)
            # chunked-below-gate vs whole-above-gate: the tree is cut at the midpoint, so summing the
            # two halves separately and adding is the same computation
            if n > 128:
                mid = n // 2
                halves = lib.ftc_pairwise_sum(x.data_ptr(), mid) + lib.ftc_pairwise_sum(x.data_ptr() + 8 * mid, n - mid)
                assert halves == serial


def test_row_parallel_kernels_are_bitwise_serial_at_every_width_and_gate(pool):
    lib = pool
    g = torch.Generator().manual_seed(2)
    m, k, n = 37, 29, 23
    x = torch.randn(m, k, generator=g, dtype=torch.float64)
    x.view(-1)[: len(_BOUNDARY)] = torch.tensor(_BOUNDARY, dtype=torch.float64).clamp(-1e3, 1e3)
    w = torch.randn(n, k, generator=g, dtype=torch.float64)
    b = torch.randn(n, generator=g, dtype=torch.float64)
    gam, bet = torch.rand(k, generator=g, dtype=torch.float64) + 0.5, torch.randn(k, generator=g, dtype=torch.float64)
    y0 = torch.empty(m, n, dtype=torch.float64)
    lib.ftc_linear_f64(x.data_ptr(), w.data_ptr(), b.data_ptr(), y0.data_ptr(), m, k, n)
    ln0 = torch.empty(m, k, dtype=torch.float64)
    lib.ftc_layer_norm_f64(x.data_ptr(), gam.data_ptr(), bet.data_ptr(), ln0.data_ptr(), None, None, m, k, 1e-5)
    work = m * k * n
    for width in (1, 2, 5, 8, 64):                       # more threads than rows included
        for gate in (0, work - 1, work, work + 1, 1 << 30):
            def run():
                y = torch.full((m, n), float("nan"), dtype=torch.float64)
                lib.ftc_linear_f64_par(x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), m, k, n)
                ln = torch.full((m, k), float("nan"), dtype=torch.float64)
                lib.ftc_layer_norm_f64_par(x.data_ptr(), gam.data_ptr(), bet.data_ptr(), ln.data_ptr(), m, k, 1e-5)
                return y, ln
            y, ln = _with_width(lib, width, gate, run)
            assert torch.equal(y.view(torch.int64), y0.view(torch.int64)), (width, gate)
            assert torch.equal(ln.view(torch.int64), ln0.view(torch.int64)), (width, gate)


def test_chunk_target_of_row_parallel_kernels_changes_scheduling_not_results(pool):
    """``set_parallel_target_workers`` (ft-kernel-cpu/src/lib.rs:2758): the number of chunks of the row split is a
    measurement lever that returns the previous value; every row is computed by one thread whatever the split."""
    from frankentorch_b200.runtime import cpu_pool
    lib = pool
    g = torch.Generator().manual_seed(3)
    m, k, n = 37, 64, 48
    x, w, b = (torch.randn(*s, generator=g, dtype=torch.float64) for s in ((m, k), (n, k), (n,)))
    y0 = torch.empty(m, n, dtype=torch.float64)
    lib.ftc_linear_f64(x.data_ptr(), w.data_ptr(), b.data_ptr(), y0.data_ptr(), m, k, n)

    def run():
        y = torch.full((m, n), float("nan"), dtype=torch.float64)
        lib.ftc_linear_f64_par(x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), m, k, n)
        return y
    assert cpu_pool.parallel_target_workers() == 0
    try:
        prev = 0
        for target in (1, 3, 7, 37, 100, 0):
            assert cpu_pool.set_parallel_target_workers(target) == prev
            prev = target
            for width in (1, 4):
                y = _with_width(lib, width, 0, run)
                assert torch.equal(y.view(torch.int64), y0.view(torch.int64)), (target, width)
        assert cpu_pool.set_parallel_target_workers(-5) == 0 and cpu_pool.parallel_target_workers() == 0   # out of range: ignored
        old_gate = cpu_pool.set_par_min_work(123)
        assert cpu_pool.set_par_min_work(old_gate) == 123
    finally:
        cpu_pool.set_parallel_target_workers(0)


def test_pool_policy_auto_caps_at_sixteen_and_is_decided_once(pool):
    from frankentorch_b200.runtime.cpu_pool import configure_cpu_threads
    lib = pool
    lib.ftc_pool_reset_for_tests()
    assert lib.ftc_pool_width() == 1                                            # unset means serial
    assert 1 <= lib.ftc_pool_auto_width() <= 16 and lib.ftc_pool_auto_width() <= lib.ftc_pool_physical_cores()
    with pytest.raises(ValueError):
        configure_cpu_threads("many")
    first = configure_cpu_threads("auto")
    assert first.changed and first.width == lib.ftc_pool_auto_width()
    second = configure_cpu_threads("3")
    assert not second.changed and second.width == first.width                  # the first decision stands
    assert "cpu pool width=" in first.summary()


def test_session_echoes_the_pool_policy_into_the_ledger(pool, monkeypatch):
    pool.ftc_pool_reset_for_tests()
    monkeypatch.setenv("FT_CPU_THREADS", "2")
    s = FrankenTorchSession("strict")
    assert any("cpu pool width=2" in e.summary for e in s.evidence())


# ------------------------------------------------------------------------------------ source scan
def _sources(*suffixes):
    for p in sorted(PKG.rglob("*")):
        if p.suffix in suffixes and "build" not in p.parts and "__pycache__" not in p.parts:
            yield p, p.read_text(errors="replace")


def test_kernels_carry_no_traps_asserts_or_prints():
    """A release kernel reports through the status word; it never traps, asserts or prints."""
    bad = []
    trap, dev_assert, dev_print = "__tr" + "ap", re.compile(r"(?<![_A-Za-z])assert\s*\("), re.compile(r"(?<![_A-Za-z])printf\s*\(")
    for p, text in _sources(".cu", ".cuh"):
        code = re.sub(r"//[^\n]*", "", text)
        code = re.sub(r"/\*.*?\*/", "", code, flags=re.S)
        for ln, line in enumerate(code.splitlines(), 1):
            if trap in line or dev_assert.search(line.replace("static_assert", "")) or dev_print.search(line):
                bad.append(f"{p.name}:{ln}: {line.strip()}")
    assert not bad, "\n".join(bad)


def test_every_spin_wait_in_the_kernels_is_bounded():
    """A loop that polls a flag or an mbarrier must consult a clock (or a spin budget) inside it."""
    bad = []
    for p, text in _sources(".cu", ".cuh"):
        for m in re.finditer(r"while\s*\(([^)]*(?:ld_acquire|ld_acq|try_wait|volatile)[^)]*)\)\s*\{(.*?)\n\s*\}", text, flags=re.S):
            body = m.group(2)
            if not re.search(r"clock64|globaltimer|spins|budget|BUDGET", body):
                bad.append(f"{p.name}: unbounded wait: while ({m.group(1).strip()[:60]})")
        for m in re.finditer(r"while\s*\(\s*(?:true|1)\s*\)\s*\{(.*?)\n  \}", text, flags=re.S):
            if not re.search(r"clock64|globaltimer|spins|budget|return|break", m.group(1)):
                bad.append(f"{p.name}: while(true) without an exit")
    assert not bad, "\n".join(bad)


def test_no_load_of_any_kind_uses_cluster_multicast():
    """Bulk / tensor loads never carry the cluster-multicast qualifier (only the tcgen05 commit does)."""
    qual = ".multi" + "cast::cluster"
    bad = []
    for p, text in _sources(".cu", ".cuh"):
        for ln, line in enumerate(text.splitlines(), 1):
            if qual in line and "cp.async.bulk" in line:
                bad.append(f"{p.name}:{ln}")
    assert not bad, bad


def test_production_python_has_no_placeholders():
    marks = re.compile(r"\b(TO" + r"DO|FIX" + r"ME|XX" + r"X|HA" + r"CK)\b|unimplemented|not implemented yet|place" + "holder hash")
    bad = []
    for p, text in _sources(".py"):
        for ln, line in enumerate(text.splitlines(), 1):
            if marks.search(line):
                bad.append(f"{p.relative_to(ROOT)}:{ln}: {line.strip()[:80]}")
            if re.search(r"raise NotImplementedError", line):
                ctx = "\n".join(text.splitlines()[max(0, ln - 6): ln])
                if "def " not in ctx:                      # allowed only as the body of an abstract method
                    bad.append(f"{p.relative_to(ROOT)}:{ln}: NotImplementedError outside a method body")
            if re.search(r"det64:0{16}|sha256:0{8}", line):
                bad.append(f"{p.relative_to(ROOT)}:{ln}: placeholder digest")
    assert not bad, "\n".join(bad)


def test_committed_files_name_no_closed_call_and_no_machine_path():
    closed = ["cudaMemcpy" + "BatchAsync", "cudaMemcpy3D" + "BatchAsync", "cuMemcpy" + "BatchAsync",
              "cuMemcpy3D" + "BatchAsync"]
    machine = re.compile(r"/ro" + r"ot/(repo|reference)|gpu" + r"run_out|\bgpu" + r"run\b")
    bad = []
    for base in (PKG, ROOT / "tests", ROOT / "benchmarks"):
        for p in sorted(base.rglob("*")):
            if p.suffix not in (".py", ".cu", ".cuh", ".h", ".cpp") or "__pycache__" in p.parts or "build" in p.parts:
                continue
            text = p.read_text(errors="replace")
            for c in closed:
                if c in text:
                    bad.append(f"{p.relative_to(ROOT)} names {c}")
            if machine.search(text):
                bad.append(f"{p.relative_to(ROOT)} names a path or tool of the build machine")
    for p in (ROOT / "bench.py", ROOT / "__graft_entry__.py"):
        if machine.search(p.read_text()):
            bad.append(f"{p.name} names a path or tool of the build machine")
    assert not bad, "\n".join(bad)


def test_cpu_attention_tile_is_a_scheduling_knob_only():
    """The query-row tile of the blocked CPU attention kernel (``set_sdpa_br``, ``FT_SDPA_BR``) and the pool width
    never change a bit of the result; the adaptive rule coarsens only while heads x blocks keeps the pool busy."""
    import math

    import torch

    from frankentorch_b200.runtime import cpu_pool, native
    lib = native.load()
    g = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn(3, 2, 150, 16, generator=g, dtype=torch.float64) for _ in range(3))
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    old_br = cpu_pool.sdpa_br()
    lib.ftc_pool_reset_for_tests()
    lib.ftc_pool_set_min_work(1)
    try:
        outs = []
        for width in ("1", "3", "8"):
            lib.ftc_pool_reset_for_tests()
            assert lib.ftc_pool_configure(width.encode(), None) == int(width)
            for br in (8, 64, 100, 512, 0):
                cpu_pool.set_sdpa_br(br)
                outs.append(cpu_pool.sdpa_blocked(q, k, v, causal=True))
        assert all(torch.equal(outs[0], o) for o in outs)
        assert torch.allclose(outs[0], ref, atol=1e-12)
        # one (batch, head) problem at a time through the serial oracle gives the same bits
        one = torch.empty(150, 16, dtype=torch.float64)
        lib.ftc_sdpa_f64(q[1, 0].contiguous().data_ptr(), k[1, 0].contiguous().data_ptr(),
                         v[1, 0].contiguous().data_ptr(), one.data_ptr(), 150, 150, 16, 1.0 / math.sqrt(16), 1)
        assert torch.equal(one, outs[0][1, 0])
        # setter clamps; adaptive rule
        assert cpu_pool.set_sdpa_br(3) == 8 and cpu_pool.set_sdpa_br(4096) == 512
        cpu_pool.set_sdpa_br_auto()
        lib.ftc_pool_reset_for_tests()
        lib.ftc_pool_configure(b"8", None)
        assert cpu_pool.sdpa_br_for(1500, 8) == 128          # heads fill the pool
        assert cpu_pool.sdpa_br_for(1500, 4) == 128          # 4 x 12 blocks >= 4 x 8
        assert cpu_pool.sdpa_br_for(300, 2) == 64            # 2 x 3 blocks would starve the pool
    finally:
        cpu_pool.set_sdpa_br(old_br)
        lib.ftc_pool_reset_for_tests()
        lib.ftc_pool_set_min_work(1 << 15)
