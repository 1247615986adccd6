"""GPU-resident encoder stack: oracle on CPU, kernels against the oracle on a GPU."""
import pytest
import torch

from frankentorch_b200.models.encoder import EncoderGpu, EncoderLayerWeights, reference_forward


def _layers(n, d, ff, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [EncoderLayerWeights.random(d, ff, g) for _ in range(n)]


def test_reference_forward_matches_torch_modules():
    torch.manual_seed(0)
    d, H, S = 64, 1, 10
    (l,) = _layers(1, d, 128)
    x = torch.randn(S, d, dtype=torch.float64)
    got = reference_forward([l], x, H)
    # the same layer from torch building blocks (pre-norm, key projection without bias)
    w = {k: getattr(l, k).double() for k in l.__dataclass_fields__}
    n1 = torch.nn.functional.layer_norm(x, (d,), w["ln1_g"], w["ln1_b"], 1e-5)
    q, k, v = n1 @ w["wq"].T + w["bq"], n1 @ w["wk"].T, n1 @ w["wv"].T + w["bv"]
    a = torch.nn.functional.scaled_dot_product_attention(q[None, None], k[None, None], v[None, None])[0, 0]
    x1 = x + a @ w["wo"].T + w["bo"]
    n2 = torch.nn.functional.layer_norm(x1, (d,), w["ln2_g"], w["ln2_b"], 1e-5)
    want = x1 + torch.nn.functional.gelu(n2 @ w["w1"].T + w["b1"], approximate="tanh") @ w["w2"].T + w["b2"]
    assert torch.allclose(got, want, atol=1e-10)


def test_encoder_rejects_bad_shapes():
    with pytest.raises(ValueError):
        EncoderGpu([], 1, device="cpu")
    with pytest.raises(ValueError):
        EncoderGpu(_layers(1, 96, 128), 2, device="cpu")      # head size 48


@pytest.mark.gpu
@pytest.mark.parametrize("seq,d,heads,n_layers,chunk", [(200, 256, 4, 3, 2), (384, 256, 2, 2, 8)])
def test_encoder_gpu_matches_the_fp32_oracle(seq, d, heads, n_layers, chunk):
    layers = _layers(n_layers, d, 4 * d, seed=3)
    torch.manual_seed(1)
    x = torch.randn(seq, d)
    want = reference_forward(layers, x.to("cuda", torch.float32), heads).cpu()
    enc = EncoderGpu(layers, heads, chunk=chunk)
    got = enc.forward(x, seq)
    err = (got - want).abs().max() / want.abs().max()
    assert err < 4e-2, float(err)
    again = enc.forward(x, seq)                       # graph replay
    assert torch.equal(got, again)
    eager = EncoderGpu(layers, heads, chunk=1, use_cuda_graph=False).forward(x, seq)
    assert torch.equal(got, eager)                    # chunking and graphs do not change the bits
    assert len(enc.chunks()) == -(-n_layers // chunk)


def test_reference_stem_is_two_strided_convolutions_plus_positions():
    from frankentorch_b200.models.encoder import StemWeights, reference_stem, stem_out_rows
    g = torch.Generator().manual_seed(4)
    n_mels, d, t_in = 8, 16, 11
    stem = StemWeights.random(n_mels, d, 32, g)
    mel = torch.randn(t_in, n_mels, generator=g, dtype=torch.float64)
    got = reference_stem(stem, mel)
    assert got.shape == (stem_out_rows(t_in), d) and stem_out_rows(t_in) == 6 and stem_out_rows(12) == 6
    # the gather the GPU path uses (column index ci * 3 + kk, zero padding) times the [cin*3, d] weight
    def im2col(x, stride):
        t, c = x.shape
        t_out = (t + 2 - 3) // stride + 1
        y = torch.zeros(t_out, c * 3, dtype=x.dtype)
        for o in range(t_out):
            for ci in range(c):
                for kk in range(3):
                    p = o * stride + kk - 1
                    if 0 <= p < t:
                        y[o, ci * 3 + kk] = x[p, ci]
        return y
    from frankentorch_b200.models.encoder import _gelu_tanh_clamped
    h1 = _gelu_tanh_clamped(im2col(mel, 1) @ stem.conv1_wt.double() + stem.conv1_b.double())
    h2 = _gelu_tanh_clamped(im2col(h1, 2) @ stem.conv2_wt.double() + stem.conv2_b.double())
    assert torch.allclose(got, h2 + stem.pos_emb.double()[: h2.shape[0]], atol=1e-10)


@pytest.mark.gpu
def test_forward_from_mel_matches_the_fp32_oracle():
    from frankentorch_b200.models.encoder import StemWeights, reference_stem, stem_out_rows
    d, heads, n_mels, t_in = 256, 4, 80, 301
    layers = _layers(2, d, 4 * d, seed=5)
    g = torch.Generator().manual_seed(6)
    stem = StemWeights.random(n_mels, d, 1500, g)
    mel = torch.randn(t_in, n_mels, generator=g)
    enc = EncoderGpu(layers, heads, chunk=8)
    with pytest.raises(RuntimeError):
        enc.forward_from_mel(mel)
    enc.attach_stem(stem, n_mels, 1500)
    assert enc.has_stem()
    got, rows = enc.forward_from_mel(mel, t_in)
    assert rows == stem_out_rows(t_in) == 151 and got.shape == (151, d)
    x0 = reference_stem(stem, mel.to("cuda", torch.float32))
    want = reference_forward(layers, x0, heads).cpu()
    err = (got - want).abs().max() / want.abs().max()
    assert err < 4e-2, float(err)
    again, _ = enc.forward_from_mel(mel, t_in)
    assert torch.equal(got, again)
    with pytest.raises(ValueError):
        enc.forward_from_mel(torch.randn(4000, n_mels))          # more rows than positional embeddings
