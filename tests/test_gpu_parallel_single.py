"""The sharded model variants on ONE GPU (world = 1): every collective-fused kernel runs with
itself as the only peer, so the code paths of the multi-GPU models are exercised on any box."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tape():
    from frankentorch_b200.autograd.tape import TensorTape
    from frankentorch_b200.ops import kernels as K
    t = TensorTape(grad_dtype=None)
    t.accumulate_fn = lambda a, b: K.add(a, b) if a.dtype == torch.bfloat16 else a + b
    return t


def _batch(cfg, bs, S, seed=5):
    g = torch.Generator().manual_seed(seed)
    tok = torch.randint(0, cfg.vocab_size, (bs, S + 1), generator=g)
    return tok[:, :-1].contiguous().pin_memory(), tok[:, 1:].contiguous().pin_memory()


@pytest.mark.parametrize("kind", ["tp", "zero3"])
def test_sharded_gpt_on_one_rank_matches_plain_gpt(cuda_device, kind):
    from frankentorch_b200.models.gpt import GPT, GPTConfig
    from frankentorch_b200.models.gpt_tp import TensorParallelGPT
    from frankentorch_b200.models.gpt_zero3 import Zero3GPT
    from frankentorch_b200.ops import kernels as K
    from frankentorch_b200.training.engine import OptimConfig, TrainEngine
    cfg = GPTConfig(n_layer=2, d_model=256, n_head=4, d_ff=1024, vocab_size=1000, max_seq=128, name="gpt-test")
    bs, S = 2, 128
    ids, tgt = _batch(cfg, bs, S)
    opt = OptimConfig(lr=1e-3, grad_clip=None)
    ref = GPT(cfg, _tape(), device=cuda_device, seed=3)
    sd = ref.state_dict()
    ref_losses = [TrainEngine(ref, bs, S, opt, use_cuda_graph=False).step(ids, tgt) for _ in range(1)]
    eng_ref = TrainEngine(ref, bs, S, opt, use_cuda_graph=False)
    ref_losses += [eng_ref.step(ids, tgt) for _ in range(3)]
    for graph in (False, True):
        if kind == "tp":
            m = TensorParallelGPT(cfg, _tape(), cuda_device, group=None, micro_batch=bs, seq_len=S, seed=3)
        else:
            m = Zero3GPT(cfg, _tape(), cuda_device, group=None, seed=3)
        m.load_full_state_dict(sd)
        eng = TrainEngine(m, bs, S, opt, use_cuda_graph=graph)
        losses = [eng.step(ids, tgt) for _ in range(4)]
        K.check_status()
        for a, b in zip(losses, ref_losses):
            assert abs(a - b) < 3e-2 * max(1.0, abs(b)), (kind, graph, losses, ref_losses)
        assert losses[-1] < losses[0]


def test_moe_gpt_trains_on_one_rank(cuda_device):
    from frankentorch_b200.models.gpt_moe import MoEConfig, MoEGPT
    from frankentorch_b200.ops import kernels as K
    from frankentorch_b200.training.engine import OptimConfig, TrainEngine
    cfg = MoEConfig.gpt_preset("moe-tiny")
    bs, S = 4, 128
    ids, tgt = _batch(cfg, bs, S)
    for graph in (False, True):
        m = MoEGPT(cfg, MoEConfig(), _tape(), cuda_device, group=None, micro_batch=bs, seq_len=S, seed=3)
        eng = TrainEngine(m, bs, S, OptimConfig(lr=2e-3, grad_clip=1.0), use_cuda_graph=graph)
        losses = [eng.step(ids, tgt) for _ in range(8)]
        K.check_status()
        assert all(torch.isfinite(torch.tensor(losses))), losses
        assert losses[-1] < losses[0] - 0.05, losses
        # replay determinism: a second engine from the same seed gives the same losses bit for bit
        m2 = MoEGPT(cfg, MoEConfig(), _tape(), cuda_device, group=None, micro_batch=bs, seq_len=S, seed=3)
        eng2 = TrainEngine(m2, bs, S, OptimConfig(lr=2e-3, grad_clip=1.0), use_cuda_graph=graph)
        assert [eng2.step(ids, tgt) for _ in range(8)] == losses


def test_training_state_checkpoint_resumes_bit_identically(cuda_device, tmp_path):
    from frankentorch_b200.models.gpt import GPT, GPTConfig
    from frankentorch_b200.serialize.state_dict import load_state_dict
    from frankentorch_b200.training.checkpoint import load_training_state, save_training_state
    from frankentorch_b200.training.engine import OptimConfig, TrainEngine
    cfg = GPTConfig.preset("gpt-tiny")
    bs, S = 2, 128
    batches = [_batch(cfg, bs, S, seed=100 + i) for i in range(6)]
    opt = OptimConfig(lr=1e-3, grad_clip=1.0)

    def engine(seed):
        return TrainEngine(GPT(cfg, _tape(), device=cuda_device, seed=seed), bs, S, opt, use_cuda_graph=True)
    full = engine(3)
    ref = [full.step(*b) for b in batches]
    first = engine(3)
    head = [first.step(*b) for b in batches[:3]]
    stem = str(tmp_path / "ckpt")
    path = save_training_state(first, stem)
    sd = load_state_dict(path)
    assert "optim.master" in sd and "rank0.step" in sd and float(sd["rank0.step"][0]) == 3.0
    resumed = engine(77)                      # different initial weights: everything must come from the file
    resumed.step(*batches[0])                 # capture its graph first; the load below must still take effect
    load_training_state(resumed, stem)
    tail = [resumed.step(*b) for b in batches[3:]]
    assert head == ref[:3]
    assert tail == ref[3:], (tail, ref[3:])
