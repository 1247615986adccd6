"""Measurement discipline for head-to-head numbers (the reference keeps these helpers next to its
session API: ft-api/src/harness_provenance.rs, ft-api/src/harness_interleave.rs).

* :mod:`.provenance`: the incumbent arm must report its own version (``PT_TORCH_VERSION``); a
  ratio without it, or across arms that report different versions, is refused.
* :mod:`.host`: what the machine looked like (code digest, host and GPU, other measurements, CPU clock spread, load
  drift) and the predicates that say whether a window is quotable.
* :mod:`.interleave`: arms are sampled alternately in a balanced-square slot order, the incumbent
  may run as a request / response co-process, and each arm's first-half / second-half A/A null
  has to be calm before a ratio is quoted.
"""
from .interleave import (BALANCED_SQUARE, MAX_NULL_CI_WIDTH, QUIT_REQUEST, READY_MARKER, REQUEST_PREFIX,
                         SAMPLE_MARKER, TIMED_STEPS_MARKER, CoProcessArm, HeadToHead, IncumbentSample, NullVerdict,
                         adjudicate_null, aa_null, incumbent_sample_rounds, parse_sample_line, parse_timed_steps,
                         run_balanced_square, sample_request, timed_region_disagreement)
from .host import (LEGACY_BLOCK_ARMS_ENV, MAX_LOAD_DRIFT, ArmOrdering, MeasurementSlot, announce_measurement,
                   arm_ordering_from_env, concurrent_measurement_block, concurrent_measurement_processes, cpu_clock_block,
                   cpu_mhz_sorted, cpu_mhz_stats, executing_code_sha256, executing_elf_sha256, identical_arm_digests,
                   interpreter_args, load_average_1m, load_drift_is_quotable, load_series_drift, load_series_is_quotable,
                   measurement_host_block)
from .provenance import (VERSION_MARKER, MissingIncumbentVersion, incumbent_provenance_block, parse_reported_version,
                         payload_line, require_reported_version, version_disagreement)

__all__ = [n for n in dir() if not n.startswith("_")]
