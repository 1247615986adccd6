"""Row-sparse gradients: ``index_select_sparse`` / ``Embedding(sparse=True)`` -> ``SparseAdam``
(ft-autograd/src/lib.rs:582-587, :8204, :15680-15750; ft-optim/src/lib.rs:5519)."""
import torch

from frankentorch_b200 import nn, optim
from frankentorch_b200.session import FrankenTorchSession


def _setup(sparse):
    s = FrankenTorchSession("strict")
    emb = nn.Embedding(s, 50, 4, sparse=sparse)
    w = emb._parameters["weight"]
    ids = s.tensor_variable([3.0, 7.0, 3.0, 49.0, 0.0, 7.0], [2, 3], False)      # float-valued ids, repeats
    proj = s.tensor_variable([0.5, -1.0, 2.0, 0.25], [4], False)
    return s, emb, w, ids, proj


def test_sparse_route_emits_coo_rows_and_equals_the_dense_gradient():
    s, emb, w, ids, proj = _setup(True)
    loss = s.tensor_sum(s.tensor_mul(emb.forward(s, ids), proj))
    rep = s.tensor_backward(loss)
    coo = rep.sparse_gradient(w)
    assert coo is not None and coo.indices.tolist() == [[0, 3, 7, 49]] and coo.nnz == 4
    assert tuple(coo.values.shape) == (4, 4) and coo.shape == (50, 4)
    s2, emb2, w2, ids2, proj2 = _setup(False)
    rep2 = s2.tensor_backward(s2.tensor_sum(s2.tensor_mul(emb2.forward(s2, ids2), proj2)))
    assert rep2.sparse_gradient(w2) is None
    assert torch.equal(rep.gradient(w), rep2.gradient(w2))                       # same values, bit for bit
    assert torch.equal(coo.to_dense(), rep2.gradient(w2))
    assert torch.equal(s.tensor_tape.accumulated_gradient(w), rep2.gradient(w2))
    assert any(st.rule == "d(index_select(x))/dx=scatter_add_grad [row-sparse]" for st in rep.steps)


def test_sparse_gradients_accumulate_over_backward_calls_and_clear():
    s, emb, w, ids, proj = _setup(True)
    for _ in range(2):
        s.tensor_backward(s.tensor_sum(s.tensor_mul(emb.forward(s, ids), proj)))
    sg = s.tensor_tape.accumulated_sparse_gradient(w)
    assert sg.rows.tolist() == [0, 3, 7, 49]
    assert torch.allclose(sg.values[1], 2 * 2 * torch.tensor([0.5, -1.0, 2.0, 0.25], dtype=torch.float64))
    s.tensor_zero_grad(w)
    assert s.tensor_tape.accumulated_sparse_gradient(w) is None and s.tensor_tape.accumulated_gradient(w) is None


def test_sparse_adam_touches_only_the_rows_that_were_read():
    outs = []
    for sparse in (True, False):
        s, emb, w, ids, proj = _setup(sparse)
        opt = optim.SparseAdam([w], lr=0.1)
        before = s.tensor(w).clone()
        for _ in range(3):
            opt.zero_grad(s)
            rep = s.tensor_backward(s.tensor_sum(s.tensor_mul(emb.forward(s, ids), proj)))
            opt.step(s, rep)
        after = s.tensor(w).clone()
        changed = (after != before).any(1).nonzero().reshape(-1).tolist()
        assert changed == [0, 3, 7, 49]
        outs.append(after)
    assert torch.equal(outs[0], outs[1])          # sparse route == dense gradient scanned for its rows


def test_mixed_dense_and_sparse_use_of_one_table_falls_back_to_dense():
    s, emb, w, ids, proj = _setup(True)
    a = s.tensor_sum(s.tensor_mul(emb.forward(s, ids), proj))
    b = s.tensor_sum(s.tensor_mul(w, w))                                        # a dense use of the same leaf
    rep = s.tensor_backward(s.tensor_add(a, b))
    assert rep.sparse_gradient(w) is None
    g = rep.gradient(w)
    want = 2 * s.tensor(w)
    want[[0, 49]] += torch.tensor([0.5, -1.0, 2.0, 0.25], dtype=torch.float64)
    want[[3, 7]] += 2 * torch.tensor([0.5, -1.0, 2.0, 0.25], dtype=torch.float64)
    assert torch.allclose(g, want)
