"""Out-of-bounds write detection with canary-padded outputs on shapes that are not multiples of a tile."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _k():
    from frankentorch_b200.ops import kernels as k
    return k


def _bf(shape, dev, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * 0.5).to(torch.bfloat16).to(dev)


def test_canary_detects_a_stray_write(cuda_device):
    from frankentorch_b200.utils.canary import Canary, CanaryError
    c = Canary(cuda_device)
    t = c.empty((7, 9), torch.float32, "victim")
    t.fill_(1.0)
    c.check()
    flat = t.view(-1)
    torch.as_strided(flat, (flat.numel() + 1,), (1,))[-1] = 2.0          # one element past the end
    with pytest.raises(CanaryError, match="victim.*after"):
        c.check()


def test_kernels_keep_inside_their_outputs_on_ragged_shapes(cuda_device):
    from frankentorch_b200.utils.canary import Canary
    k, c = _k(), Canary(cuda_device)
    # GEMMs: M, N off the 128 x {128,192,256} tiles, fp32 and bf16 outputs, bias + GELU epilogue, split-K
    for (M, N, Kd) in ((200, 328, 192), (129, 136, 64), (1000, 776, 320)):
        a, b = _bf((M, Kd), cuda_device, 1), _bf((N, Kd), cuda_device, 2)
        bias = _bf((N,), cuda_device, 3)
        k.gemm(a, b, out=c.empty((M, N), torch.bfloat16, f"gemm bf16 {M}x{N}"))
        k.gemm(a, b, bias=bias, epi=k.EPI_GELU_TANH, out=c.empty((M, N), torch.bfloat16, f"gemm gelu {M}x{N}"))
        k.gemm(a, b, out=c.empty((M, N), torch.float32, f"gemm fp32 {M}x{N}"))
    dy, x = _bf((4096, 264), cuda_device, 4), _bf((4096, 200), cuda_device, 5)
    k.gemm(dy, x, a_mn=True, b_mn=True, out=c.empty((264, 200), torch.float32, "wgrad split-k"), split_k=4)
    # row kernels: 1000 x 264 (264 = 33 vectors of 8)
    rows, cols = 1000, 264
    xr, g, b = _bf((rows, cols), cuda_device, 6), _bf((cols,), cuda_device, 7), _bf((cols,), cuda_device, 8)
    lib = k._lib.load()
    y = c.empty((rows, cols), torch.bfloat16, "layernorm y")
    mean, rstd = c.empty((rows,), torch.float32, "ln mean"), c.empty((rows,), torch.float32, "ln rstd")
    k._chk(lib.ftk_layernorm_fwd(xr.data_ptr(), None, None, g.data_ptr(), b.data_ptr(), y.data_ptr(), mean.data_ptr(),
                                 rstd.data_ptr(), rows, cols, 1e-5, k._stream()), "ln fwd")
    dx = c.empty((rows, cols), torch.bfloat16, "layernorm dx")
    dg, db = c.empty((cols,), torch.float32, "ln dgamma"), c.empty((cols,), torch.float32, "ln dbeta")
    nblk = max(lib.ftk_layernorm_bwd_blocks(rows), (rows + 31) // 32)
    part = c.empty((2 * nblk * cols,), torch.float32, "ln partials")
    k._chk(lib.ftk_layernorm_bwd(xr.data_ptr(), xr.data_ptr(), g.data_ptr(), mean.data_ptr(), rstd.data_ptr(), None,
                                 dx.data_ptr(), dg.data_ptr(), db.data_ptr(), part.data_ptr(), rows, cols, 0,
                                 k._stream()), "ln bwd")
    out = c.empty((cols,), torch.float32, "colsum out")
    k.colsum(xr, out=out)
    ids = torch.randint(0, 50, (3, 7), device=cuda_device)
    wte = _bf((50, 72), cuda_device, 9)
    dwte = c.empty((50, 72), torch.float32, "dwte")
    dwte.zero_()
    k.embedding_bwd(ids, _bf((21, 72), cuda_device, 10), dwte, None, 7)
    # attention, ragged sequence length
    B, S, H, hd = 2, 200, 3, 64
    qkv = _bf((B, S, 3 * H * hd), cuda_device, 11)
    q, kk, v = (qkv[:, :, i * H * hd:(i + 1) * H * hd].view(B, S, H, hd) for i in range(3))
    o, lse = k.attention_fwd(q, kk, v, causal=True)
    dqkv = c.empty((B, S, 3 * H * hd), torch.bfloat16, "dqkv")
    dq, dk, dv = (dqkv[:, :, i * H * hd:(i + 1) * H * hd].view(B, S, H, hd) for i in range(3))
    k.attention_bwd(q, kk, v, o, lse, _bf((B, S, H, hd), cuda_device, 12), causal=True, dq=dq, dk=dk, dv=dv)
    k.check_status()
    torch.cuda.synchronize()
    c.check()
