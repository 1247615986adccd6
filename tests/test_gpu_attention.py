"""Flash attention (tcgen05) forward/backward against an fp32 PyTorch reference."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, k, v, causal):
    # q,k,v: [B,S,H,hd] fp32
    B, S, H, hd = q.shape
    qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    s = qh @ kh.transpose(-1, -2) / math.sqrt(hd)
    if causal:
        mask = torch.triu(torch.ones(S, S, dtype=torch.bool, device=q.device), 1)
        s = s.masked_fill(mask, float("-inf"))
    p = torch.softmax(s, -1)
    return (p @ vh).permute(0, 2, 1, 3)


@pytest.mark.parametrize("B,S,H,hd,causal", [
    (1, 128, 1, 64, True),
    (1, 128, 1, 64, False),
    (2, 256, 3, 64, True),
    (1, 512, 2, 64, True),
    (1, 200, 2, 64, True),      # ragged sequence
    (1, 256, 2, 128, True),
    (1, 384, 1, 128, False),
    (1, 200, 2, 64, False),     # ragged, non-causal (encoder inference)
    (1, 328, 1, 128, True),     # ragged, head_dim 128
    (2, 1024, 2, 64, True),     # eight key blocks: every ring slot is reused
])
def test_attention_fwd_bwd(cuda_device, B, S, H, hd, causal):
    from frankentorch_b200.ops import kernels as k
    torch.manual_seed(0)
    d = H * hd
    # packed QKV activations, exactly the layout the model uses
    qkv = (torch.randn(B, S, 3 * d) * 0.8).to(torch.bfloat16).to(cuda_device)
    q = qkv[:, :, 0 * d:1 * d].view(B, S, H, hd)
    kk = qkv[:, :, 1 * d:2 * d].view(B, S, H, hd)
    v = qkv[:, :, 2 * d:3 * d].view(B, S, H, hd)
    o, lse = k.attention_fwd(q, kk, v, causal=causal)
    k.check_status()
    qf, kf, vf = (t.float().detach().requires_grad_(True) for t in (q, kk, v))
    ref = _ref(qf, kf, vf, causal)
    err = (o.float() - ref).abs().max().item()
    assert err < 3e-2, f"fwd max err {err}"
    # log-sum-exp is stored in the log2 domain of the scaled scores
    s = (qf.permute(0, 2, 1, 3) @ kf.permute(0, 2, 3, 1)) / math.sqrt(hd)
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device=s.device), 1), float("-inf"))
    lse_ref = torch.logsumexp(s, -1) / math.log(2.0)
    assert (lse - lse_ref).abs().max().item() < 2e-2

    d_o = (torch.randn(B, S, H, hd) * 0.5).to(torch.bfloat16).to(cuda_device)
    dqkv = torch.zeros_like(qkv)
    dq = dqkv[:, :, 0 * d:1 * d].view(B, S, H, hd)
    dk = dqkv[:, :, 1 * d:2 * d].view(B, S, H, hd)
    dv = dqkv[:, :, 2 * d:3 * d].view(B, S, H, hd)
    k.attention_bwd(q, kk, v, o, lse, d_o, causal=causal, dq=dq, dk=dk, dv=dv)
    k.check_status()
    ref.backward(d_o.float())
    for name, got, want in (("dq", dq, qf.grad), ("dk", dk, kf.grad), ("dv", dv, vf.grad)):
        e = (got.float() - want).abs().max().item()
        scale = want.abs().max().item() + 1e-6
        assert e / scale < 4e-2, f"{name}: max err {e} (ref max {scale})"
        # per (batch, head, 128-row block): error relative to that block's own magnitude, so that a
        # wrong block of small values (late query rows of dq, early key rows of dk) cannot hide
        gb, wb = got.float().permute(0, 2, 1, 3), want.permute(0, 2, 1, 3)
        pad = (-S) % 128
        gb, wb = torch.nn.functional.pad(gb, (0, 0, 0, pad)), torch.nn.functional.pad(wb, (0, 0, 0, pad))
        eb = (gb - wb).abs().reshape(B, H, -1, 128 * hd).amax(-1)
        mb = wb.abs().reshape(B, H, -1, 128 * hd).amax(-1).clamp_min(scale * 1e-3)
        assert (eb / mb).max().item() < 0.12, f"{name}: worst block is off by {(eb / mb).max().item():.3g} of its own magnitude"


def test_attention_bitwise_replay(cuda_device):
    from frankentorch_b200.ops import kernels as k
    torch.manual_seed(1)
    B, S, H, hd = 2, 512, 4, 64
    q, kk, v, d_o = ((torch.randn(B, S, H, hd) * 0.7).to(torch.bfloat16).to(cuda_device) for _ in range(4))
    outs = []
    for _ in range(2):
        o, lse = k.attention_fwd(q, kk, v)
        dq, dk, dv = k.attention_bwd(q, kk, v, o, lse, d_o)
        outs.append((o.clone(), dq.clone(), dk.clone(), dv.clone()))
    k.check_status()
    for a, b in zip(*outs):
        assert torch.equal(a, b)
