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


@pytest.mark.parametrize("kind", ["tp", "zero3"])
def test_clip_norm_of_a_sharded_model_covers_every_parameter(cuda_device, kind):
    """The clip factor of the sharded models comes from the norm of ALL gradients (replicated arena +
    rank-local shards): with clipping active the reported norm and the trajectory follow the plain model."""
    from frankentorch_b200.models.gpt import GPT, GPTConfig
    from frankentorch_b200.models.gpt_tp import TensorParallelGPT
    from frankentorch_b200.models.gpt_zero3 import Zero3GPT
    from frankentorch_b200.training.engine import OptimConfig, TrainEngine
    cfg = GPTConfig(n_layer=2, d_model=256, n_head=4, d_ff=1024, vocab_size=1000, max_seq=128, name="gpt-test")
    bs, S = 2, 128
    ids, tgt = _batch(cfg, bs, S)
    opt = OptimConfig(lr=1e-3, grad_clip=0.05)                 # far below the gradient norm: always active
    ref = GPT(cfg, _tape(), device=cuda_device, seed=3)
    sd = ref.state_dict()
    eng_ref = TrainEngine(ref, bs, S, opt, use_cuda_graph=False)
    ref_losses, ref_norms = [], []
    for _ in range(3):
        ref_losses.append(eng_ref.step(ids, tgt))
        ref_norms.append(float(eng_ref.grad_norm))
    assert ref_norms[0] > 0.5                                  # the clip really bites
    m = (TensorParallelGPT(cfg, _tape(), cuda_device, group=None, micro_batch=bs, seq_len=S, seed=3) if kind == "tp"
         else Zero3GPT(cfg, _tape(), cuda_device, group=None, seed=3))
    m.load_full_state_dict(sd)
    eng = TrainEngine(m, bs, S, opt, use_cuda_graph=True)
    for step in range(3):
        loss = eng.step(ids, tgt)
        assert abs(float(eng.grad_norm) - ref_norms[step]) < 2e-2 * ref_norms[step], (kind, step, float(eng.grad_norm), ref_norms)
        assert abs(loss - ref_losses[step]) < 3e-2 * max(1.0, abs(ref_losses[step]))
    K.check_status()


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


from frankentorch_b200.ops import kernels as K  # noqa: E402


def _dp_engine(cuda_device, seed, *, graph, clip, wire="fp32", bucket_elems=None, overlap=True, dp=True,
               defer=None):
    from frankentorch_b200.models.gpt import GPT, GPTConfig
    from frankentorch_b200.parallel.data_parallel import FusedDataParallel
    from frankentorch_b200.training.engine import OptimConfig, TrainEngine
    cfg = GPTConfig.preset("gpt-tiny")
    model = GPT(cfg, _tape(), device=cuda_device, seed=seed, peer_visible=dp)
    d = FusedDataParallel(model.arena, None, cuda_device, wire=wire, bucket_elems=bucket_elems,
                          overlap=overlap, defer_update=defer) if dp else None
    eng = TrainEngine(model, 2, 128, OptimConfig(lr=1e-3, grad_clip=clip), use_cuda_graph=graph, dp=d)
    return cfg, model, eng, d


def test_bucketed_data_parallel_on_one_rank_matches_plain_engine(cuda_device):
    """The peer-memory path with a world of one (every "peer" is this GPU) against the single-GPU
    optimizer: with fp32 on the wire and no clipping the two are the same arithmetic, bit for bit,
    whatever the bucket size and whether or not buckets start under the backward pass."""
    from frankentorch_b200.models.gpt import GPTConfig
    cfg = GPTConfig.preset("gpt-tiny")
    batches = [_batch(cfg, 2, 128, seed=200 + i) for i in range(4)]
    _, m0, e0, _ = _dp_engine(cuda_device, 5, graph=False, clip=None, dp=False)
    ref_losses = [e0.step(*b) for b in batches]
    ref = m0.arena.params.clone()
    for graph, bucket_elems, overlap, defer in ((False, None, True, True), (True, 40_000, True, True),
                                                (True, 40_000, False, True), (True, 40_000, True, False),
                                                (False, 40_000, True, False)):
        _, m, e, d = _dp_engine(cuda_device, 5, graph=graph, clip=None, bucket_elems=bucket_elems, overlap=overlap,
                                defer=defer)
        losses = [e.step(*b) for b in batches]
        e.sync_parameters()
        K.check_status()
        assert d.step_ok()
        assert losses == ref_losses, (graph, bucket_elems, losses, ref_losses)
        assert torch.equal(m.arena.params, ref)
        if bucket_elems:
            assert len(d.buckets) > 3
            if overlap:
                # the last layers' bucket goes first, the embeddings' bucket (arena start) last
                assert set(d.launch_order[-2:]) == {0, 1} and d.launch_order[0] == len(d.buckets) - 1, d.launch_order
        assert torch.equal(d.gather_master()[: ref.numel()].to(torch.bfloat16), ref)


def test_bucketed_data_parallel_bf16_wire_and_clip_replay(cuda_device):
    """bf16 on the wire + global-norm clipping: close to the single-GPU path, and bit-identical
    between eager execution and CUDA-graph replay and between bucket sizes (sums are per element;
    only the norm's partial sums depend on the buckets, so that part is compared with clipping off)."""
    from frankentorch_b200.models.gpt import GPTConfig
    cfg = GPTConfig.preset("gpt-tiny")
    batches = [_batch(cfg, 2, 128, seed=300 + i) for i in range(5)]
    _, m0, e0, _ = _dp_engine(cuda_device, 9, graph=True, clip=1.0, dp=False)
    for b in batches:
        e0.step(*b)
    outs = {}
    for key, graph, be, clip, defer in (("eager", False, 40_000, 1.0, True), ("graph", True, 40_000, 1.0, True),
                                        ("now", True, 40_000, 1.0, False),
                                        ("nc_small", True, 40_000, None, True), ("nc_big", True, None, None, False)):
        _, m, e, d = _dp_engine(cuda_device, 9, graph=graph, clip=clip, wire="bf16", bucket_elems=be, defer=defer)
        for b in batches:
            e.step(*b)
        e.sync_parameters()
        K.check_status()
        outs[key] = m.arena.params.clone()
    assert torch.equal(outs["eager"], outs["graph"])
    assert torch.equal(outs["now"], outs["graph"])        # deferring the update does not change it
    assert torch.equal(outs["nc_small"], outs["nc_big"])
    diff = (outs["graph"].float() - m0.arena.params.float()).abs().max().item()
    assert diff < 2e-2, diff


def test_sharded_checkpoint_of_bucketed_optimizer_state_resumes(cuda_device, tmp_path):
    from frankentorch_b200.models.gpt import GPTConfig
    from frankentorch_b200.serialize.state_dict import consolidate_shards
    from frankentorch_b200.training.checkpoint import load_training_state, save_training_state
    cfg = GPTConfig.preset("gpt-tiny")
    batches = [_batch(cfg, 2, 128, seed=400 + i) for i in range(6)]
    _, _, full, _ = _dp_engine(cuda_device, 3, graph=True, clip=1.0, wire="bf16", bucket_elems=40_000)
    ref = [full.step(*b) for b in batches]
    _, _, first, d1 = _dp_engine(cuda_device, 3, graph=True, clip=1.0, wire="bf16", bucket_elems=40_000)
    head = [first.step(*b) for b in batches[:3]]
    stem = str(tmp_path / "ck")
    save_training_state(first, stem)
    merged = consolidate_shards(stem, 1)
    assert torch.equal(merged["optim.master"], d1.gather_master().cpu())
    _, _, resumed, _ = _dp_engine(cuda_device, 77, graph=True, clip=1.0, wire="bf16", bucket_elems=40_000)
    resumed.step(*batches[0])
    load_training_state(resumed, stem)
    tail = [resumed.step(*b) for b in batches[3:]]
    assert head + tail == ref


def test_symmetric_buffer_close_frees_the_local_allocation(cuda_device):
    """``close()`` unmaps the peers, then frees the rank's own ``cudaMalloc`` block; a second call is a no-op."""
    from frankentorch_b200.parallel.symm import SymmetricBuffer
    before = torch.cuda.mem_get_info(cuda_device)[0]
    buf = SymmetricBuffer(64 << 20, None, cuda_device)
    t = buf.tensor(torch.float32, 1024)
    t.fill_(3.0)
    assert float(t.sum()) == 3.0 * 1024 and buf.peer_ptrs[0] == buf.local_ptr != 0
    held = torch.cuda.mem_get_info(cuda_device)[0]
    assert before - held >= 60 << 20
    del t
    buf.close()
    assert buf.local_ptr == 0 and buf.bytes is None
    assert torch.cuda.mem_get_info(cuda_device)[0] - held >= 60 << 20     # the block went back to the driver
    buf.close()
