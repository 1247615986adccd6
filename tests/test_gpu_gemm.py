"""tcgen05 GEMM numerics against a plain PyTorch fp32 reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ops():
    from frankentorch_b200.ops import kernels
    return kernels


def _rand(shape, dev, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).to(dev)


def _tile_rel_err(out, ref, tile=128):
    """Max over ``tile x tile`` output tiles of (max abs error in the tile) / (max abs reference in the
    tile): one wrong tile of small values cannot hide behind large values elsewhere in the matrix."""
    import torch.nn.functional as F
    g, w = out.float().reshape(-1, out.shape[-1]), ref.float().reshape(-1, ref.shape[-1])
    R, C = g.shape
    pr, pc = (-R) % tile, (-C) % tile
    g, w = F.pad(g, (0, pc, 0, pr)), F.pad(w, (0, pc, 0, pr))
    e = (g - w).abs().view((R + pr) // tile, tile, (C + pc) // tile, tile).amax((1, 3))
    m = w.abs().view((R + pr) // tile, tile, (C + pc) // tile, tile).amax((1, 3))
    return (e / m.clamp_min(w.abs().max() * 1e-3)).max().item()


def _check(out, ref, tol, what):
    err = (out.float() - ref).abs().max().item()
    denom = ref.abs().max().item() + 1e-6
    assert err / denom < tol, f"{what}: max abs err {err:.4g} vs ref max {denom:.4g}"
    if out.dim() >= 2:
        t = _tile_rel_err(out, ref)
        assert t < 3 * tol, f"{what}: worst 128x128 tile is off by {t:.3g} of its own magnitude"


@pytest.mark.parametrize("M,N,K,bn", [
    (128, 128, 64, 128),      # one tile, one k-block
    (128, 256, 64, 256),
    (128, 128, 256, 128),     # k loop
    (256, 512, 512, 256),     # multiple tiles per CTA ring
    (1024, 768, 768, 0),
    (200, 136, 72, 0),        # ragged M, N, K (TMA zero fill + guarded stores)
    (4096, 2304, 768, 0),     # more tiles than SMs: persistent loop + accumulator ping-pong
])
def test_gemm_kmajor(cuda_device, M, N, K, bn):
    k = _ops()
    a = _rand((M, K), cuda_device, seed=1)
    b = _rand((N, K), cuda_device, seed=2)
    out = k.gemm(a, b, force_bn=bn)
    k.check_status()
    ref = a.float() @ b.float().t()
    _check(out, ref, 2e-2, f"gemm {M}x{N}x{K}")


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (384, 512, 320), (520, 264, 200)])
def test_gemm_mn_major(cuda_device, a_mn, b_mn, M, N, K):
    k = _ops()
    a = _rand((K, M) if a_mn else (M, K), cuda_device, seed=3)
    b = _rand((K, N) if b_mn else (N, K), cuda_device, seed=4)
    out = k.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    k.check_status()
    af = a.float().t() if a_mn else a.float()
    bf = b.float().t() if b_mn else b.float()
    _check(out, af @ bf.t(), 2e-2, f"gemm a_mn={a_mn} b_mn={b_mn} {M}x{N}x{K}")


def test_gemm_epilogues(cuda_device):
    k = _ops()
    M, N, K = 512, 768, 256
    a = _rand((M, K), cuda_device, 0.5, 5)
    w = _rand((N, K), cuda_device, 0.1, 6)
    bias = _rand((N,), cuda_device, 1.0, 7)
    resid = _rand((M, N), cuda_device, 1.0, 8)
    pre = a.float() @ w.float().t() + bias.float()
    out = k.gemm(a, w, bias=bias)
    _check(out, pre, 2e-2, "bias")
    aux = torch.empty((M, N), dtype=torch.bfloat16, device=cuda_device)
    out = k.gemm(a, w, bias=bias, epi=k.EPI_GELU_TANH, aux=aux)
    _check(out, torch.nn.functional.gelu(pre, approximate="tanh"), 2e-2, "gelu_tanh")
    _check(aux, pre, 2e-2, "aux pre-activation")
    out = k.gemm(a, w, bias=bias, epi=k.EPI_GELU_ERF)
    _check(out, torch.nn.functional.gelu(pre), 2e-2, "gelu_erf")
    out = k.gemm(a, w, bias=bias, resid=resid)
    _check(out, pre + resid.float(), 2e-2, "bias+residual")
    # dgelu epilogue: acc * gelu'(u)
    u = _rand((M, N), cuda_device, 1.0, 9)
    uf = u.float().requires_grad_(True)
    torch.nn.functional.gelu(uf, approximate="tanh").sum().backward()
    out = k.gemm(a, w, resid=u, epi=k.EPI_MUL_DGELU_TANH)
    _check(out, (a.float() @ w.float().t()) * uf.grad, 2e-2, "mul_dgelu_tanh")
    # fp32 output with accumulation (weight gradients)
    acc = torch.ones((M, N), dtype=torch.float32, device=cuda_device)
    k.gemm(a, w, out=acc, accumulate=True)
    _check(acc, a.float() @ w.float().t() + 1.0, 1e-2, "fp32 accumulate")
    k.check_status()


def test_linear_grads(cuda_device):
    k = _ops()
    M, N, K = 1024, 3072, 768
    x = _rand((M, K), cuda_device, 1.0, 10)
    w = _rand((N, K), cuda_device, 0.05, 11)
    dy = _rand((M, N), cuda_device, 1.0, 12)
    dx = k.linear_dgrad(dy, w)
    dw = k.linear_wgrad(dy, x)
    k.check_status()
    _check(dx, dy.float() @ w.float(), 2e-2, "dgrad")
    _check(dw, dy.float().t() @ x.float(), 2e-2, "wgrad")


def test_gemm_deterministic(cuda_device):
    k = _ops()
    a = _rand((2048, 1024), cuda_device, seed=13)
    b = _rand((1536, 1024), cuda_device, seed=14)
    o1 = k.gemm(a, b, force_bn=256)
    o2 = k.gemm(a, b, force_bn=256, max_ctas=37)   # different grid, same bits: one CTA reduces all of K
    k.check_status()
    assert torch.equal(o1, o2)
    # run-to-run: the default configuration (whatever tile/split it picks) replays bit for bit
    assert torch.equal(k.gemm(a, b), k.gemm(a, b))


def test_gemm_split_k_deterministic_and_correct(cuda_device):
    k = _ops()
    # weight-gradient shape: small output, long reduction -> split-K with fixed-order reduce
    M, N, Kd = 768, 768, 8192
    dy = _rand((Kd, M), cuda_device, 0.5, 21)
    x = _rand((Kd, N), cuda_device, 0.5, 22)
    ref = dy.float().t() @ x.float()
    outs = []
    for split in (0, 1, 4, 6):
        o = k.gemm(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32, split_k=split)
        _check(o, ref, 5e-3, f"split_k={split}")
        outs.append(o)
    again = k.gemm(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32, split_k=6)
    assert torch.equal(outs[3], again)
    acc = torch.ones((M, N), dtype=torch.float32, device=cuda_device)
    k.gemm(dy, x, a_mn=True, b_mn=True, out=acc, accumulate=True, split_k=4)
    _check(acc, ref + 1.0, 5e-3, "split-k accumulate")
    k.check_status()


def test_gemm_grouped_weight_gradients(cuda_device):
    """Four weight gradients of different extents in one launch: each against its fp32 reference per 128 x 128
    tile, with accumulation into one of them, on ragged extents, identical on a smaller grid and run to run."""
    k = _ops()
    T = 2048
    shapes = ((2304, 768), (768, 768), (3072, 768), (768, 3072), (200, 136))
    dys = [_rand((T, m), cuda_device, 0.5, 40 + i) for i, (m, n) in enumerate(shapes)]
    xs = [_rand((T, n), cuda_device, 0.5, 50 + i) for i, (m, n) in enumerate(shapes)]
    refs = [dy.float().t() @ x.float() for dy, x in zip(dys, xs)]

    def run(max_ctas=0):
        outs = [torch.full((m, n), 3.0 if i == 1 else float("nan"), dtype=torch.float32, device=cuda_device)
                for i, (m, n) in enumerate(shapes)]
        k.gemm_grouped([(dy, x, o, i == 1) for i, (dy, x, o) in enumerate(zip(dys, xs, outs))], max_ctas=max_ctas)
        return outs
    outs = run()
    k.check_status()
    for i, (o, r) in enumerate(zip(outs, refs)):
        want = r + 3.0 if i == 1 else r
        _check(o, want, 5e-3, f"grouped problem {i}")     # includes the per-tile check
    again, small = run(), run(max_ctas=37)
    for a, b, c in zip(outs, again, small):
        assert torch.equal(a, b) and torch.equal(a, c)
    # one problem alone equals the plain GEMM without split-K, bit for bit (same k-block order)
    solo = torch.empty((768, 768), dtype=torch.float32, device=cuda_device)
    k.gemm_grouped([(dys[1], xs[1], solo, False)])
    plain = k.gemm(dys[1], xs[1], a_mn=True, b_mn=True, out_dtype=torch.float32, split_k=1, force_bn=192)
    assert torch.equal(solo, plain)
    k.check_status()


def test_gemm_batched(cuda_device):
    k = _ops()
    L0, L1, M, N, K = 3, 2, 256, 128, 64
    a = _rand((L1, L0, M, K), cuda_device, seed=15)
    b = _rand((L1, L0, N, K), cuda_device, seed=16)
    out = torch.empty((L1, L0, M, N), dtype=torch.bfloat16, device=cuda_device)
    k.gemm_batched(a, b, out, M=M, N=N, K=K, L0=L0, L1=L1,
                   a_strides=(K, M * K, L0 * M * K), b_strides=(K, N * K, L0 * N * K),
                   d_strides=(N, M * N, L0 * M * N), alpha=0.5)
    k.check_status()
    ref = 0.5 * torch.einsum("xymk,xynk->xymn", a.float(), b.float())
    _check(out, ref, 2e-2, "batched")


# ------------------------------------------------------------------ CTA-pair kernel (force_bn = 512)
@pytest.mark.parametrize("M,N,K", [
    (256, 256, 64),           # one pair tile, one k-block
    (256, 256, 512),          # k loop over the 6-stage ring
    (512, 768, 320),          # several tiles, ragged K
    (520, 264, 200),          # ragged M / N: the peer CTA's rows and columns run off the edge
    (4096, 2304, 768),        # more tiles than clusters: persistent loop + accumulator ping-pong
])
def test_gemm_pair_kmajor(cuda_device, M, N, K):
    k = _ops()
    a = _rand((M, K), cuda_device, seed=11)
    b = _rand((N, K), cuda_device, seed=12)
    out = k.gemm(a, b, force_bn=512)
    k.check_status()
    _check(out, a.float() @ b.float().t(), 2e-2, f"pair gemm {M}x{N}x{K}")


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
def test_gemm_pair_mn_major_and_epilogues(cuda_device, a_mn, b_mn):
    k = _ops()
    M, N, K = 512, 640, 384
    a = _rand((K, M) if a_mn else (M, K), cuda_device, seed=13)
    b = _rand((K, N) if b_mn else (N, K), cuda_device, seed=14)
    bias = _rand((N,), cuda_device, seed=15)
    resid = _rand((M, N), cuda_device, seed=16)
    out = k.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, resid=resid, force_bn=512)
    k.check_status()
    af = a.float().t() if a_mn else a.float()
    bf = b.float() if b_mn else b.float().t()
    _check(out, af @ bf + bias.float() + resid.float(), 2e-2, f"pair gemm a_mn={a_mn} b_mn={b_mn}")


def test_gemm_pair_split_k_and_determinism(cuda_device):
    k = _ops()
    a = _rand((4096, 768), cuda_device, seed=17)       # wgrad shape: dW = dy^T x
    b = _rand((4096, 768), cuda_device, seed=18)
    ref = a.float().t() @ b.float()
    o1 = k.gemm(a, b, a_mn=True, b_mn=True, out_dtype=torch.float32, force_bn=512, split_k=4)
    o2 = k.gemm(a, b, a_mn=True, b_mn=True, out_dtype=torch.float32, force_bn=512, split_k=4, max_ctas=36)
    k.check_status()
    _check(o1, ref, 2e-2, "pair split-k")
    assert torch.equal(o1, o2), "the pair kernel's result must not depend on the grid"


def test_gemm_skips_tiles_without_rows_in_use(cuda_device):
    """Ragged rows (expert batches): rows come in segments of which only a prefix is in use; tiles of
    128 rows that hold no row in use are skipped (their output is left alone), every other row is exact."""
    k = _ops()
    seg_rows, segs, N, K = 640, 3, 256, 192          # 5 tiles per segment
    counts = torch.tensor([200, 0, 513], dtype=torch.int32, device=cuda_device)
    a = _rand((seg_rows * segs, K), cuda_device, seed=7)
    w = _rand((N, K), cuda_device, 0.2, 8)
    bias = _rand((N,), cuda_device, 0.5, 9)
    out = torch.full((seg_rows * segs, N), 7.0, dtype=torch.bfloat16, device=cuda_device)
    k.gemm(a, w, bias=bias, out=out, seg_counts=counts, seg_rows=seg_rows)
    k.check_status()
    ref = a.float() @ w.float().t() + bias.float()
    for s, c in enumerate(counts.tolist()):
        lo = s * seg_rows
        used_hi = lo + -(-c // 128) * 128                      # rows of tiles that hold a used row are computed
        if c:
            _check(out[lo:lo + c], ref[lo:lo + c], 2e-2, f"segment {s} rows in use")
        assert torch.all(out[used_hi:lo + seg_rows].float() == 7.0), f"segment {s}: a skipped tile was written"
    dense = k.gemm(a, w, bias=bias)
    assert torch.equal(dense[:200], out[:200])                 # the same kernel arithmetic, bit for bit
