#!/usr/bin/env python
"""Stock-PyTorch arm of the CPU MLP benchmark (config 1) as a request / response co-process.

Protocol (the one of the reference's head-to-head harness, ft-api/src/harness_interleave.rs): the
arm prints ``PT_TORCH_VERSION <v>`` and ``PT_TIMED_STEPS <steps>``, sets up, warms up, prints
``PT_READY``, then answers every ``SAMPLE <lane>`` line on stdin with one
``PT_SAMPLE <lane> <milliseconds> <checksum>`` line (one timed block of training steps) until ``QUIT``.
MLP 784-256-128-10, ReLU, cross-entropy, AdamW lr 1e-3, batch 64, f32, inputs N(0,1), labels uniform.
"""
import argparse
import sys
import time

import torch
import torch.nn as nn
import torch.nn.functional as F


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10, help="training steps per sample")
    ap.add_argument("--threads", type=int, default=0)
    a = ap.parse_args()
    if a.threads:
        torch.set_num_threads(a.threads)
    print("PT_TORCH_VERSION %s" % torch.__version__, flush=True)
    print("PT_TIMED_STEPS batch,forward,loss,backward,optimizer", flush=True)
    torch.manual_seed(42)
    model = nn.Sequential(nn.Linear(784, 256), nn.ReLU(), nn.Linear(256, 128), nn.ReLU(), nn.Linear(128, 10))
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)

    def block(n):
        loss = None
        for _ in range(n):
            x = torch.randn(64, 784)
            y = torch.randint(0, 10, (64,))
            loss = F.cross_entropy(model(x), y)
            opt.zero_grad(set_to_none=True)
            loss.backward()
            opt.step()
        return float(loss)
    block(5)
    print("PT_READY", flush=True)
    for line in sys.stdin:
        line = line.strip()
        if line == "QUIT":
            break
        if line.startswith("SAMPLE "):
            t0 = time.perf_counter()
            ck = block(a.steps)
            ms = (time.perf_counter() - t0) * 1e3
            print("PT_SAMPLE %s %.6f %.6f" % (line[7:], ms, ck), flush=True)


if __name__ == "__main__":
    main()
