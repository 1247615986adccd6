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
