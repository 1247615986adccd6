#!/usr/bin/env python
"""Headline benchmark: GPT training tokens/sec on N B200s of one node.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

Metric and config follow the repository baseline: train tokens/sec (whole job, max over
ranks) for a GPT-2 decoder in bf16 with fp32 master weights, micro-batch 8 per GPU at
sequence length 1024 (GPT-2 small, data parallel) by default; ``--model`` selects the other
named configs.  Data is synthetic (tokens uniform over the vocabulary), weights are
random-init.

``vs_torch`` is a head-to-head with stock PyTorch (``benchmarks/torch_baseline.py``: DDP for the
data-parallel config, FSDP for the ZeRO-3 one) sampled in the same invocation, the two arms
interleaved in a balanced-square slot order, each arm's first-half / second-half null checked,
the incumbent's version reported by the arm itself.  On more than one GPU ``multi_gpu_check``
holds the fused gradient reduction against an NCCL all-reduce of the same gradients and against
its own replay (a failure makes the exit code non-zero), and ``exposed_comm_ms_per_step`` is the
time the compute stream waited for communication in the last step (GPU timer marks).

Two numbers are reported.  ``value`` times K optimizer steps with CUDA events on the
launching stream (inputs already on the device).  ``e2e`` times K calls of the public
``TrainEngine.step(ids, targets)`` API, which every step copies that step's tokens and
targets from pinned host memory to the device and reads the loss back to the host.

``--impl reference`` would run the unmodified reference; it is a Rust workspace with no
Python package and no Rust toolchain exists on this machine, so that arm reports itself
unavailable.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

MODELS = {
    # name: (preset, micro_batch_per_gpu, seq_len, default parallelism)
    "gpt2-small": ("gpt2-small", 8, 1024, "dp"),       # data parallel, fused reduce-scatter + AdamW
    "gpt2-medium": ("gpt2-medium", 4, 2048, "zero3"),  # block weights sharded, gathers fused into GEMMs
    "gpt-1.3b": ("gpt-1.3b", 4, 2048, "tp"),           # tensor + sequence parallel over all GPUs
    "moe-12l": ("moe-12l", 4, 2048, "ep"),             # 8 experts top-2, expert parallel
    "gpt-tiny": ("gpt-tiny", 4, 128, "dp"),
    "moe-tiny": ("moe-tiny", 4, 128, "ep"),
    # CPU single-process MLP 784-256-128-10 (f32, ReLU, cross-entropy, AdamW 1e-3, batch 64): no GPU involved
    "mlp-cpu": ("mlp-cpu", 64, 784, "cpu"),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="gpt2-small", choices=sorted(MODELS))
    ap.add_argument("--micro-batch", type=int, default=0)
    ap.add_argument("--seq-len", type=int, default=0)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-torch-arm", action="store_true",
                    help="skip the interleaved stock-PyTorch arm (DDP for dp, FSDP for zero3, Megatron-style TP for tp, "
                         "all_to_all + bmm experts for ep) that fills vs_torch")
    ap.add_argument("--h2h-steps", type=int, default=5, help="optimizer steps per head-to-head sample")
    ap.add_argument("--log-jsonl", default="", help="append a structured ft-conformance-log-v1 record of this run")
    ap.add_argument("--parallelism", default="", choices=["", "dp", "tp", "zero3", "ep"],
                    help="default: the one the named config asks for")
    ap.add_argument("--dp-impl", default=os.environ.get("FT_DP_IMPL", "fused"), choices=["fused", "nccl"],
                    help="multi-GPU gradient path: in-kernel NVLink reduce-scatter+AdamW+all-gather, or NCCL all-reduce")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, uuid: str = ""):
        self.gpu = gpu_index
        self.uuid = uuid
        self.proc = None
        self.path = None
        self.thread = None
        self.stop_flag = None
        self.rows = []

    def _start_nvml(self) -> bool:
        """Preferred sampler: NVML in a thread of this process, one reading every 20 ms (a
        spawned nvidia-smi needs longer to enumerate eight GPUs than a short timed region lasts).
        Read-only queries; nothing on the GPU is changed."""
        try:
            import threading

            import pynvml as nv
            nv.nvmlInit()
            h = None
            if self.uuid:
                for cand in (self.uuid, self.uuid.encode()):
                    try:
                        h = nv.nvmlDeviceGetHandleByUUID(cand)
                        break
                    except Exception:
                        h = None
            if h is None:
                h = nv.nvmlDeviceGetHandleByIndex(self.gpu)
            reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
            mx = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            self.stop_flag = threading.Event()

            def loop():
                while not self.stop_flag.is_set():
                    try:
                        self.rows.append((float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)), mx, int(reasons_fn(h))))
                    except Exception:
                        pass
                    self.stop_flag.wait(0.02)
            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return True
        except Exception:
            self.thread = None
            return False

    def start(self):
        if self._start_nvml():
            return
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            if self.rows:
                # NVML clocks-event-reason bits
                bits = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
                        0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}
                seen = 0
                for _, _, r in self.rows:
                    seen |= r
                out.update(sm_mhz=statistics.median(r[0] for r in self.rows), sm_max_mhz=self.rows[0][1],
                           samples=len(self.rows), reasons=sorted(n for b, n in bits.items() if seen & b),
                           source="nvml")
            return out
        if self.proc is None:
            return out
        try:
            self.proc.terminate()
            self.proc.wait(timeout=5)
        except Exception:
            pass
        try:
            sm, mx, reasons = [], [], set()
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
                for name, val in zip(names, f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            if sm:
                out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), samples=len(sm),
                           reasons=sorted(reasons))
            os.unlink(self.path)
        except Exception:
            pass
        return out


def multi_gpu_check(engine, dp, dist, torch):
    """Outside the timed region, on the gradients of one more step: the fused reduce-scatter against an
    NCCL all-reduce of the same gradients, and a second run of the reduction against the first, bit for bit."""
    from frankentorch_b200.ops import kernels as K
    engine.step_device(read_loss=False)
    torch.cuda.synchronize()
    a = engine.model.arena
    fused = dp._gather(dp.gshard)                        # reduced gradients, arena order, fp32
    ref = a.grads.detach().clone()
    dist.all_reduce(ref, op=dist.ReduceOp.AVG)
    scale = float(ref.abs().max().clamp_min(1e-30))
    diff = float((fused[: ref.numel()] - ref).abs().max()) / scale
    first = dp.gshard.clone()
    dp.begin_step()                                      # applies the pending update, advances the sequence
    for b in reversed(range(len(dp.buckets))):
        dp._launch_bucket(b)
    torch.cuda.current_stream().wait_stream(dp.comm_stream)
    torch.cuda.synchronize()
    K.check_status()
    same = torch.tensor([1 if torch.equal(first, dp.gshard) else 0], device=first.device)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    tol = 8e-3 if dp.wire == "bf16" else 1e-5
    return {"reduced_grad_max_abs_diff_over_max": diff, "tolerance": tol, "wire": dp.wire,
            "bit_identical_replay": bool(int(same)), "buckets": len(dp.buckets),
            "ok": bool(diff <= tol and int(same) == 1)}


def run_mlp_cpu(args):
    """Config 1: the public session API end to end on the CPU reference path, with deterministic-replay and
    state-dict round-trip checks, and the stock-PyTorch arm as an interleaved co-process."""
    import tempfile as _tmp

    import torch

    from frankentorch_b200 import harness as H
    from frankentorch_b200 import nn, optim, serialize
    from frankentorch_b200.core.dtype import DType
    from frankentorch_b200.session import FrankenTorchSession
    dims, batch = (784, 256, 128, 10), 64
    steps, warmup = max(args.steps, 1), max(args.warmup, 3)

    class MLP(nn.Module):
        def __init__(self, s):
            super().__init__()
            self.l1, self.l2, self.l3 = (nn.Linear(s, dims[i], dims[i + 1]) for i in range(3))

        def forward(self, s, x):
            return self.l3(s, s.tensor_relu(self.l2(s, s.tensor_relu(self.l1(s, x)))))

    def build():
        s = FrankenTorchSession(default_dtype=DType.F32)
        m = MLP(s)
        for _, p in m.named_parameters():
            s.tensor(p).data = s.tensor(p).to(torch.float32)
        return s, m, optim.AdamW(m.parameters(), 1e-3), s.autograd_graph_len()

    def train(state, n):
        s, m, opt, boundary = state
        losses, orders = [], []
        for _ in range(n):
            x = s.tensor_variable_from_storage(s.tensor(s.randn([batch, dims[0]])).to(torch.float32))
            y = s.randint(0, dims[-1], [batch])
            loss = s.tensor_cross_entropy(m(s, x), y)
            opt.zero_grad(s)
            rep = s.tensor_backward(loss)
            opt.step(s, rep)
            losses.append(s.tensor_item(loss))
            orders.append(tuple(rep.telemetry.execution_order))
            s.truncate_autograd_graph(boundary)
        return losses, orders
    # replay: two sessions from the same seed give the same loss bits and execution orders for 100 steps
    a, b = build(), build()
    la, oa = train(a, 100)
    lb, ob = train(b, 100)
    replay_ok = la == lb and oa == ob
    with _tmp.TemporaryDirectory() as td:
        path = os.path.join(td, "mlp.ftsv")
        serialize.save_state_dict(a[1].state_dict(a[0]), path)
        c = build()
        c[1].load_state_dict(c[0], serialize.load_state_dict(path), strict=True)
        probe = torch.randn(4, dims[0])
        pa = a[0].tensor(a[1](a[0], a[0].tensor_variable_from_storage(probe)))
        pc = c[0].tensor(c[1](c[0], c[0].tensor_variable_from_storage(probe)))
        round_trip_ok = bool(torch.equal(pa, pc))
    # timed: K steps after W warm-up steps (wall clock: everything is host work)
    st = build()
    train(st, warmup)
    t0 = time.perf_counter()
    train(st, steps)
    ms = (time.perf_counter() - t0) * 1e3
    # head to head: the incumbent as a co-process, interleaved in the balanced-square order
    hs = max(1, args.h2h_steps * 2)
    vs = None
    if not args.no_torch_arm:
        try:
            arm = H.CoProcessArm([sys.executable, os.path.join(REPO, "benchmarks", "torch_mlp_arm.py"),
                                  "--steps", str(hs)])
            try:
                def ours():
                    t = time.perf_counter()
                    train(st, hs)
                    return (time.perf_counter() - t) * 1e3 / hs
                res = H.run_balanced_square(ours, lambda: arm.sample("mlp").milliseconds / hs, rounds=2,
                                            ours_steps=("batch", "forward", "loss", "backward", "optimizer"),
                                            incumbent_steps=arm.timed_steps or ())
                vs = dict(res.as_dict(), impl="stock pytorch CPU (nn.Sequential, AdamW), co-process",
                          steps_per_sample=hs, **H.incumbent_provenance_block(arm.version, torch.get_num_threads()))
            finally:
                arm.close()
        except H.MissingIncumbentVersion as e:
            vs = {"refused": str(e)}
    out = {"metric": "train steps/sec (CPU, single process)", "value": steps / (ms / 1e3), "unit": "steps/s",
           "n_gpus": 0, "steps": steps, "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True,
           "scaling": "none", "vs_baseline": None, "dtype": "f32 (f64 gradient space)",
           "data": "synthetic (inputs N(0,1), labels uniform in [0,10), session PRNG)", "impl": "ours",
           "config": {"model": "mlp 784-256-128-10", "batch": batch, "optimizer": "AdamW lr 1e-3",
                      "api": "FrankenTorchSession + ft.nn + ft.optim on the CPU reference path"},
           "deterministic_replay_100_steps": replay_ok, "state_dict_round_trip_exact": round_trip_ok,
           "final_loss": la[-1], "gpu_launches": 0, "vs_torch": vs,
           "e2e": {"value": steps / (ms / 1e3), "unit": "steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                   "note": "host-only workload: the timed region is already the public API end to end"}}
    print(json.dumps(out))
    return 0 if (replay_ok and round_trip_ok) else 3


def run_reference(args):
    print(json.dumps({
        "impl": "reference",
        "unavailable": "the reference is a Rust 2024 nightly workspace with no Python package "
                       "(pip: \"neither setup.py nor pyproject.toml found\"), no cargo/rustc on this "
                       "image, no CUDA backend and no distributed training, so it cannot run this metric",
    }))
    return 0


def main():
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.model == "mlp-cpu":
        return run_mlp_cpu(args)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from frankentorch_b200.autograd.tape import TensorTape
    from frankentorch_b200.models.gpt import GPT, GPTConfig
    from frankentorch_b200.ops import kernels as K
    from frankentorch_b200.training.engine import OptimConfig, TrainEngine
    from frankentorch_b200.utils.metrics import percentile_nearest_rank

    preset, mb, seq, par = MODELS[args.model]
    par = args.parallelism or par
    mb = args.micro_batch or mb
    seq = args.seq_len or seq
    group = dist.group.WORLD if world > 1 else None
    tape = TensorTape(grad_dtype=None)
    tape.accumulate_fn = lambda a, b: K.add(a, b) if (a.dtype == torch.bfloat16 and a.is_cuda) else a + b
    if par == "ep":
        from frankentorch_b200.models.gpt_moe import MoEConfig, MoEGPT
        cfg = MoEConfig.gpt_preset(preset)
        cfg.max_seq = max(seq, 1) if seq < cfg.max_seq else cfg.max_seq
        model = MoEGPT(cfg, MoEConfig(), tape, dev, group=group, micro_batch=mb, seq_len=seq, seed=1234)
    else:
        cfg = GPTConfig.preset(preset)
        cfg.max_seq = max(seq, 1) if seq < cfg.max_seq else cfg.max_seq
        if par == "tp":
            from frankentorch_b200.models.gpt_tp import TensorParallelGPT
            model = TensorParallelGPT(cfg, tape, dev, group=group, micro_batch=mb, seq_len=seq, seed=1234)
        elif par == "zero3":
            from frankentorch_b200.models.gpt_zero3 import Zero3GPT
            model = Zero3GPT(cfg, tape, dev, group=group, seed=1234)
        else:
            model = GPT(cfg, tape, device=dev, seed=1234, group=group)
    n_params = model.param_count() if hasattr(model, "param_count") else cfg.param_count()
    dp = None
    if world > 1:
        from frankentorch_b200.parallel.data_parallel import FusedDataParallel, NcclDataParallel
        dp = (NcclDataParallel if args.dp_impl == "nccl" else FusedDataParallel)(model.arena, dist.group.WORLD, dev)
    if dp is not None and hasattr(dp, "record_stamps"):
        dp.record_stamps = True      # four one-thread time-mark kernels per step: the exposed-communication figure
    from frankentorch_b200.runtime.ledger import EvidenceLedger
    ledger = EvidenceLedger()        # the eager step before graph capture is written down here, once
    engine = TrainEngine(model, mb, seq, OptimConfig(lr=3e-4, grad_clip=1.0), use_cuda_graph=not args.no_graph, dp=dp,
                         ledger=ledger)

    # synthetic data: tokens uniform over the vocabulary, a fresh pinned batch per step
    g = torch.Generator().manual_seed(1000 + rank)
    n_batches = max(4, min(16, args.steps))
    batches = []
    for _ in range(n_batches):
        tok = torch.randint(0, cfg.vocab_size, (mb, seq + 1), generator=g, dtype=torch.int64)
        batches.append((tok[:, :-1].contiguous().pin_memory(), tok[:, 1:].contiguous().pin_memory()))

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---------------- warm-up (also captures the CUDA graph)
    losses = []
    for i in range(max(args.warmup, 3)):
        ids, tg = batches[i % n_batches]
        losses.append(engine.step(ids, tg))
    K.check_status()

    # ---------------- device-timed region: K steps, CUDA events, inputs resident on the device
    sampler = ClockSampler(local_rank, "GPU-" + str(getattr(torch.cuda.get_device_properties(dev), "uuid", "")))
    sampler.start()
    sync_all()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps - 1)]
    ev0.record()
    for i in range(args.steps):
        engine.step_device(read_loss=False)
        if i + 1 < args.steps:
            marks[i].record()          # step boundaries for the p50 / p99 figures (no synchronisation)
    ev1.record()
    sync_all()
    dev_ms = ev0.elapsed_time(ev1)
    edges = [ev0] + marks + [ev1]
    step_ms = [edges[i].elapsed_time(edges[i + 1]) for i in range(args.steps)]

    # ---------------- end-to-end region: public API, H2D inputs + D2H loss every step
    e2e_ms = None
    if not args.no_e2e:
        sync_all()
        t0 = time.perf_counter()
        for i in range(args.steps):
            ids, tg = batches[i % n_batches]
            losses.append(engine.step(ids, tg, read_loss=True))
        sync_all()
        e2e_ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop()          # the clock record covers the two timed regions above, nothing else
    exposed_ms = dp.exposed_ms() if (dp is not None and hasattr(dp, "exposed_ms")) else None
    if hasattr(engine, "sync_parameters"):
        engine.sync_parameters()
    K.check_status()

    # ---------------- head to head with stock PyTorch, interleaved in the balanced-square slot order
    vs_torch = None
    if not args.no_torch_arm and preset in ("gpt2-small", "gpt2-medium", "gpt-1.3b", "gpt-tiny", "moe-12l", "moe-tiny"):
        from benchmarks.torch_baseline import TorchArm
        from frankentorch_b200 import harness as H
        try:
            arm = TorchArm(preset, dev, world, rank, micro_batch=mb, seq_len=seq,
                           parallel={"dp": "ddp", "zero3": "fsdp", "tp": "tp", "ep": "ep"}[par])
            version = H.require_reported_version(arm.version_line())     # the arm reports it; no ratio without it
            for _ in range(3):
                arm.step()
            hs = max(1, args.h2h_steps)
            load_start = H.load_average_1m()
            h2h_sampler = ClockSampler(local_rank, "GPU-" + str(getattr(torch.cuda.get_device_properties(dev), "uuid", "")))
            h2h_sampler.start()

            def _max_ms(ms):
                t = torch.tensor([ms], dtype=torch.float64, device=dev)
                if world > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                return float(t) / hs

            def ours_sample():
                sync_all()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(hs):
                    engine.step_device(read_loss=False)
                b.record()
                torch.cuda.synchronize()
                return _max_ms(a.elapsed_time(b))

            def torch_sample():
                sync_all()
                return _max_ms(arm.timed_block(hs))
            res = H.run_balanced_square(ours_sample, torch_sample, rounds=2,
                                        ours_steps=("forward", "backward", "clip", "optimizer"),
                                        incumbent_steps=H.parse_timed_steps(arm.timed_steps_line()) or ())
            vs_torch = dict(res.as_dict(), impl=arm.impl, steps_per_sample=hs, clocks=h2h_sampler.stop(),
                            **H.incumbent_provenance_block(version))
            try:            # the window the ratio was taken in; a host record must never take the bench down
                load_end = H.load_average_1m()
                vs_torch["host"] = {
                    "code_sha256": H.executing_code_sha256()[:16], "arm_ordering": H.arm_ordering_from_env().label(),
                    "load_1m": [load_start, load_end], "load_drift_quotable": H.load_drift_is_quotable(load_start, load_end),
                    "concurrent": H.concurrent_measurement_block(), "host": H.measurement_host_block().split("\n")[0]}
            except Exception as e:      # noqa: BLE001
                vs_torch["host"] = {"error": f"{type(e).__name__}: {e}"}
            arm.release()
            if hasattr(engine, "sync_parameters"):
                engine.sync_parameters()
        except H.MissingIncumbentVersion as e:
            vs_torch = {"refused": str(e)}
    K.check_status()

    mgc = None
    if world > 1 and dp is not None and hasattr(dp, "gshard"):
        mgc = multi_gpu_check(engine, dp, dist, torch)

    times = torch.tensor([dev_ms, e2e_ms if e2e_ms is not None else 0.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_max = float(times[0]), float(times[1])

    tokens_per_step = mb * seq * world
    value = tokens_per_step * args.steps / (dev_ms / 1e3)
    h2d = 2 * mb * seq * 8
    out = {
        "metric": "train tokens/sec (box, max over ranks)",
        "value": value,
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": max(args.warmup, 3),
        "ms_per_step": dev_ms / args.steps,
        "step_ms_p50": percentile_nearest_rank(step_ms, 50),
        "step_ms_p99": percentile_nearest_rank(step_ms, 99),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic (tokens uniform over the vocabulary, random-init weights)",
        "impl": "ours",
        "config": {
            "model": cfg.name, "n_layer": cfg.n_layer, "d_model": cfg.d_model, "n_head": cfg.n_head,
            "vocab": cfg.vocab_size, "params": n_params,
            "micro_batch_per_gpu": mb, "global_batch": mb * world, "seq_len": seq,
            "parallelism": ({"dp": "dp", "tp": "tp+sp", "zero3": "zero3-dp", "ep": "ep+dp"}[par] + str(world))
            if world > 1 else f"single ({par} code path)",
            "dp_impl": (args.dp_impl if world > 1 else None),
            "dp_param_allgather": (("multimem stores through NVSwitch" if getattr(dp, "nvls_params", False)
                                    else "peer stores") if dp is not None else None),
            "optimizer": "AdamW fp32 master + bf16 compute copy, grad clip 1.0",
            "cuda_graph": engine.use_graph,
            "l2": "no flush: one step streams >3 GB of activations, weights and optimizer state (L2 is 126 MB)",
        },
        "clocks": clocks,
        "ledger_entries": len(ledger),
        "gpu_launches": engine.launches_per_step * args.steps,
        "gpu_launches_per_step": engine.launches_per_step,
        "final_loss": losses[-1] if losses and losses[-1] is not None else None,
        "vs_torch": vs_torch,
    }
    if exposed_ms is not None:
        out["exposed_comm_ms_per_step"] = exposed_ms
        parts = getattr(dp, "exposed_parts_ms", None)
        if parts:
            out["exposed_comm_parts_ms"] = {"before_first_parameters": parts[0], "after_backward": parts[1]}
    if mgc is not None:
        out["multi_gpu_check"] = mgc
    if e2e_ms is not None:
        out["e2e"] = {
            "value": tokens_per_step * args.steps / (e2e_max / 1e3),
            "unit": "tokens/s",
            "ms_per_step": e2e_max / args.steps,
            "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": 4,
        }
    if rank == 0:
        print(json.dumps(out))
        if args.log_jsonl:
            from frankentorch_b200.utils.metrics import training_log_record
            with open(args.log_jsonl, "a") as f:
                f.write(json.dumps(training_log_record(out), sort_keys=True) + "\n")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if mgc is not None and not mgc["ok"]:
        return 3
    return 0


if __name__ == "__main__":
    sys.exit(main())
