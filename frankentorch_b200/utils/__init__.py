"""Configuration, metrics and profiling helpers shared by the engine, the benches and the tests."""
from .config import (ENV_FLAGS, EnvFlag, ModelSpec, OptimSpec, ParallelSpec, PrecisionSpec, RunConfig,
                     echo_to_ledger, env_flag, env_snapshot, reset_flags, set_flag)
from .metrics import (FALLBACK_PEAKS, Peaks, StepTimer, gpt_step_flops, load_peaks, max_over_ranks,
                      percentile_nearest_rank, roofline_fraction, summarize)
from .profiling import StageProfile, install_tape_ranges, nvtx_range

__all__ = [n for n in dir() if not n.startswith("_")]
