"""Multi-GPU paths (run as child processes, one rank per GPU; skipped with fewer than 2 GPUs)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _run_workers(script, nproc, port, timeout=300):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, script)]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)


def test_collective_fused_gemms(cuda_device):
    """all-gather -> GEMM (A and B operand) and GEMM -> reduce-scatter against fp32 references."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    nproc = 2 if n < 4 else 4
    p = _run_workers("_comm_worker.py", nproc, 29633)
    assert p.returncode == 0 and "COMM_WORKER_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


def test_expert_parallel_moe(cuda_device):
    """Dispatch / combine all-to-alls over peer memory with experts split over the ranks."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    nproc = 2 if n < 4 else 4
    p = _run_workers("_moe_worker.py", nproc, 29635)
    assert p.returncode == 0 and "MOE_WORKER_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


def test_tensor_parallel_gpt_follows_unsharded_model(cuda_device):
    """Tensor + sequence parallel GPT (fused all-gather->GEMM / GEMM->reduce-scatter blocks)."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    p = _run_workers("_tp_worker.py", 2, 29637)
    assert p.returncode == 0 and "TP_WORKER_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


def test_zero3_gpt_follows_unsharded_model(cuda_device):
    """Block weights sharded by rows: gather fused into fwd / dgrad GEMMs, wgrad reduce-scattered."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    p = _run_workers("_zero3_worker.py", 2, 29639)
    assert p.returncode == 0 and "ZERO3_WORKER_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


def test_fused_data_parallel_matches_nccl_and_replays(cuda_device):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    nproc = 2 if n < 4 else 4
    p = _run_workers("_dp_worker.py", nproc, 29631)
    assert p.returncode == 0 and "DP_WORKER_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


def test_pipeline_stages_over_nccl_match_a_single_process_run(cuda_device):
    """GPipe and 1F1B on two GPUs over NCCL send / recv (NVLS off, 60 s process-group timeout): the
    posting order that the host-side replay accepted really completes, gradients and loss match."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    p = _run_workers("_pp_worker.py", 2, 29641, timeout=240)
    assert p.returncode == 0 and "PP_WORKER_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


def test_multicast_collectives_match_nccl(cuda_device):
    """multimem.st all-gather (bit-exact) and multimem.ld_reduce all-reduce (tolerance, same bits on every
    rank and run) over a symmetric allocation bound to an NVSwitch multicast object."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    nproc = 2 if n < 4 else 4
    p = _run_workers("_nvls_worker.py", nproc, 29643, timeout=240)
    if "NVLS_WORKER_SKIP" in p.stdout:
        pytest.skip("no multicast support on this system")
    assert p.returncode == 0 and "NVLS_WORKER_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]
