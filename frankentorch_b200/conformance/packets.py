"""Packet contract artifacts: for each porting packet (``FT-P2C-001`` .. ``009``) a contract table, a
fixture manifest and a parity report, generated from the code and the golden suite and checked by
``validate_phase2c_artifacts``.

The reference ships one directory per packet under ``artifacts/phase2c/FT-P2C-00X/`` with
``contract_table.md``, ``fixture_manifest.json``, ``parity_report.json`` and ``parity_gate.yaml``
(e.g. artifacts/phase2c/FT-P2C-004/contract_table.md).  Here the tables state the contracts THIS
implementation enforces, each with the module that enforces it and the test that checks it; the
manifest pins the golden cases by hash and the parity report is produced by running them in both
modes when the artifacts are emitted.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, List

from ..runtime.ledger import ExecutionMode
from .runner_more import FAMILIES, run_family

SCHEMA = "ft-packet-contract-v1"

# packet -> (scope, fixture families, [(contract id, statement, enforced in, checked by)])
CONTRACTS: Dict[str, tuple] = {
    "FT-P2C-001": ("tensor metadata: shape / stride / offset validation, linear indexing, views", ["tensor_meta"], [
        ("META-001", "rank, shape, strides and storage offset are validated on construction; a view that could index "
                     "outside the storage fails closed", "core/meta.py TensorMeta", "tests/test_cpu_contract.py tensor_meta family"),
        ("META-002", "contiguous strides are derived from the shape; overflowing products are an error, not a wrap",
         "core/meta.py contiguous_strides", "tests/test_properties.py meta properties"),
        ("META-003", "the FNV-1a fingerprint of a tensor's metadata is a pure function of (dtype, device, shape, strides, offset)",
         "csrc/core/ftcore.cpp ftc_fnv*", "tests/test_cpu_contract.py fingerprints"),
    ]),
    "FT-P2C-002": ("dispatch keys, key sets and mode-split resolution", ["dispatch_key"], [
        ("DISPATCH-001", "the dispatch key set is a bit set with a fixed priority order; the highest type key wins",
         "dispatch/keys.py DispatchKeySet", "tests/test_cpu_contract.py dispatch_key family"),
        ("DISPATCH-002", "strict mode refuses a composite / backend-select fallback; hardened mode takes it and records "
                         "fallback_path=true under the allow-listed deviation id", "dispatch/keys.py decide",
         "tests/test_cpu_contract.py dispatch_key family, tests/test_gpu_session.py"),
        ("DISPATCH-003", "on the CUDA backend the decision names the kernel that was launched (ftk::...) or, for an "
                         "allow-listed hardened fallback, torch::<op>; an operator with neither is refused",
         "dispatch/sm100.py", "tests/test_gpu_session.py"),
    ]),
    "FT-P2C-003": ("operator schema parsing and registry", ["op_schema"], [
        ("SCHEMA-001", "a schema string parses into (name, overload, arguments, returns, alias sets) or fails with a "
                       "position; parse(print(x)) == x", "dispatch/schema.py", "tests/test_properties.py schema properties"),
        ("SCHEMA-002", "in-place overloads carry a write alias on self; out= variants on their out arguments",
         "dispatch/schema.py", "tests/test_cpu_contract.py op_schema family"),
    ]),
    "FT-P2C-004": ("deterministic autograd scheduler", ["autograd_scheduler", "scalar_autograd"], [
        ("AUTOGRAD-001", "reachability, dependency counts and the ready queue (max-heap on node id) give one execution "
                         "order per graph; it is replayed bit for bit", "csrc/core/ftcore.cpp ftc_schedule, autograd/tape.py",
         "tests/test_cpu_contract.py autograd_scheduler family, tests/test_properties.py scheduler properties"),
        ("AUTOGRAD-002", "reentrant depth overflow fails closed in strict mode and takes the bounded fallback, flagged in "
                         "telemetry, in hardened mode", "autograd/tape.py", "tests/test_cpu_contract.py autograd_scheduler family"),
        ("AUTOGRAD-003", "the backward report carries execution order, queue pushes / pops, dependency snapshot and the "
                         "fallback flags", "autograd/tape.py BackwardReport", "tests/test_cpu_contract.py telemetry golden"),
        ("AUTOGRAD-004", "create_graph records the backward pass itself, so gradients of gradients follow the same order rules",
         "autograd/double_backward.py", "tests/test_double_backward.py"),
    ]),
    "FT-P2C-005": ("CPU kernels (the f64 / f32 reference path) and their GPU counterparts", sorted(
        f for f in FAMILIES if f.startswith("tensor_") and f != "tensor_meta"), [
        ("KERNEL-001", "every operator of the golden suite reproduces the recorded outputs and gradients in both modes",
         "autograd/functions*.py, csrc/core/ftcore.cpp oracles", "tests/test_cpu_contract.py golden families"),
        ("KERNEL-002", "serial and pool-parallel CPU oracles are bit-identical for every thread width",
         "csrc/core/cpu_pool.cpp", "tests/test_metamorphic.py serial/parallel suite"),
        ("KERNEL-003", "in-place operators match their out-of-place forms and bump the version counter",
         "autograd/tape.py, _session_ops.py", "tests/test_metamorphic.py in-place suite"),
        ("KERNEL-004", "sm_100a kernels agree with an fp32 PyTorch restatement per 128x128 tile and replay bit for bit",
         "csrc/*.cu", "tests/test_gpu_*.py"),
    ]),
    "FT-P2C-006": ("serialization: state-dict bytes, checkpoint envelope, repair sidecar", ["serialization"], [
        ("SERIALIZE-001", "the FTSV state-dict encoding is byte-exact and the loader fails closed on any malformed field",
         "serialize/state_dict.py", "tests/test_cpu_contract.py serialization family, tests/test_properties.py loader fuzz"),
        ("SERIALIZE-002", "strict decode rejects unknown fields, hardened decode reports them; version and hash mismatches "
                          "are errors in both", "serialize/checkpoint.py", "tests/test_cpu_contract.py serialization family"),
        ("SERIALIZE-003", "a repair sidecar recovers the payload after the loss of up to its repair-symbol count of source "
                          "symbols and says recovered=false otherwise", "serialize/checkpoint.py (RLF-256 code)",
         "tests/test_cpu_tools.py, tests/test_properties.py sidecar property"),
    ]),
    "FT-P2C-007": ("device guard and device-mismatch policy", ["dispatch_key"], [
        ("DEVICE-001", "operands on different devices fail before any kernel runs", "core/meta.py ensure_same_device",
         "tests/test_cpu_contract.py"),
        ("DEVICE-002", "a device guard restores the previous device on every exit path", "core/meta.py DeviceGuard",
         "tests/test_cpu_contract.py"),
    ]),
    "FT-P2C-008": ("nn module state: parameters, buffers, prefixes, strict loading", ["nn_state"], [
        ("NNSTATE-001", "state_dict keys are '<prefix>.<name>' in registration order; buffers marked non-persistent are left out",
         "nn/module.py", "tests/test_cpu_contract.py nn_state family"),
        ("NNSTATE-002", "load_state_dict(strict=True) reports missing and unexpected keys and refuses shape mismatches",
         "nn/module.py", "tests/test_cpu_contract.py nn_state family"),
    ]),
    "FT-P2C-009": ("optimizers and schedulers", ["optimizer"], [
        ("OPTIM-001", "each optimizer's update reproduces the recorded trajectories (SGD variants, Adam family, RMSprop, ...)",
         "optim/optimizers.py", "tests/test_cpu_contract.py optimizer family"),
        ("OPTIM-002", "the fused / sharded AdamW kernels follow the same update formula and are replayable bit for bit",
         "csrc/elementwise.cu, csrc/dp_fused.cu", "tests/test_gpu_rowops.py, tests/_dp_worker.py"),
    ]),
}


def _suite_slice_hash(family: str) -> Dict[str, object]:
    from .runner import load_suite
    cases = load_suite()[family]
    blob = json.dumps(cases, sort_keys=True, separators=(",", ":")).encode()
    return {"family": family, "cases": len(cases), "sha256": hashlib.sha256(blob).hexdigest()}


def emit(root: str) -> List[str]:
    """Write ``<root>/FT-P2C-00X/{contract_table.md, fixture_manifest.json, parity_report.json}``; returns the paths."""
    written = []
    for packet, (scope, fams, rows) in sorted(CONTRACTS.items()):
        d = os.path.join(root, packet)
        os.makedirs(d, exist_ok=True)
        md = [f"# {packet} - contract table", "", f"Scope: {scope}", "",
              "| Contract | Statement | Enforced in | Checked by |", "|---|---|---|---|"]
        md += [f"| `{cid}` | {text} | `{where}` | `{test}` |" for cid, text, where, test in rows]
        md += ["", "Strict and hardened mode may differ only through the deviation ids of "
               "`frankentorch_b200/conformance/HARDENED_DEVIATION_ALLOWLIST_V1.json`.", ""]
        manifest = {"schema_version": SCHEMA, "packet": packet, "fixtures": [_suite_slice_hash(f) for f in fams]}
        parity = {"schema_version": SCHEMA, "packet": packet, "modes": {}}
        for mode in (ExecutionMode.Strict, ExecutionMode.Hardened):
            tot = ok = 0
            for f in fams:
                res = run_family(f, mode).results
                tot += len(res)
                ok += sum(1 for r in res if r.passed)
            parity["modes"][mode.value] = {"cases": tot, "passed": ok}
        parity["passed"] = all(v["cases"] == v["passed"] and v["cases"] > 0 for v in parity["modes"].values())
        for name, text in (("contract_table.md", "\n".join(md)), ("fixture_manifest.json", json.dumps(manifest, indent=2) + "\n"),
                           ("parity_report.json", json.dumps(parity, indent=2) + "\n")):
            path = os.path.join(d, name)
            with open(path, "w") as fh:
                fh.write(text)
            written.append(path)
    return written


def validate(root: str) -> List[str]:
    """Problems found in the packet artifacts under ``root`` (empty list = valid): a missing file, a parity report
    that is not all-pass, or a manifest whose hashes no longer match the golden suite."""
    bad = []
    for packet, (_, fams, rows) in sorted(CONTRACTS.items()):
        d = os.path.join(root, packet)
        if not os.path.isdir(d):
            continue                      # packets are validated where they have been emitted
        for name in ("contract_table.md", "fixture_manifest.json", "parity_report.json"):
            if not os.path.exists(os.path.join(d, name)):
                bad.append(f"{packet}: {name} missing")
        try:
            man = json.load(open(os.path.join(d, "fixture_manifest.json")))
            for fx in man["fixtures"]:
                if _suite_slice_hash(fx["family"]) != fx:
                    bad.append(f"{packet}: fixture family {fx['family']} changed since the manifest was written")
            par = json.load(open(os.path.join(d, "parity_report.json")))
            if not par.get("passed"):
                bad.append(f"{packet}: parity report is not all-pass")
            table = open(os.path.join(d, "contract_table.md")).read()
            for cid, *_ in rows:
                if f"`{cid}`" not in table:
                    bad.append(f"{packet}: contract {cid} missing from the table")
        except (OSError, ValueError, KeyError) as e:
            bad.append(f"{packet}: unreadable artifact ({e})")
    return bad
