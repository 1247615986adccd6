"""Layers, part 2: attention, transformer stacks, recurrent layers, loss modules.

Reference: ft-nn/src/lib.rs - MultiheadAttention :4685 (separate ``q_proj/k_proj/v_proj/
out_proj`` Linear children, heads split by reshape [N,S,H,hd] -> permute [0,2,1,3] ->
[N*H,S,hd] :5145-5167, one SDPA call :5178), TransformerEncoderLayer :14581 (post-norm
default, ``norm_first`` pre-norm, ReLU|GELU, children ``self_attn, linear1, linear2, norm1,
norm2, dropout, dropout1, dropout2`` :14765-14776), TransformerEncoder :14796,
TransformerDecoderLayer :14947, TransformerDecoder :15228, Transformer :15381,
``generate_square_subsequent_mask`` :15558, RNNCell/LSTMCell/GRUCell and RNN/LSTM/GRU
:13172-14158, loss modules :15577-17024.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch

from .layers import Dropout, LayerNorm, Linear, _param
from .module import Module, ModuleList


def generate_square_subsequent_mask(session, size: int) -> int:
    """Additive causal mask: 0 on and below the diagonal, -inf above."""
    m = torch.triu(torch.full((size, size), float("-inf"), dtype=torch.float64), 1)
    return session.tensor_tape.leaf(m.to(session.device), False)


class MultiheadAttention(Module):
    def __init__(self, session, embed_dim: int, num_heads: int, dropout: float = 0.0, bias: bool = True):
        super().__init__()
        if embed_dim % num_heads:
            raise ValueError("embed_dim must be divisible by num_heads")
        self.embed_dim, self.num_heads, self.head_dim = embed_dim, num_heads, embed_dim // num_heads
        self.q_proj = Linear(session, embed_dim, embed_dim, bias)
        self.k_proj = Linear(session, embed_dim, embed_dim, bias)
        self.v_proj = Linear(session, embed_dim, embed_dim, bias)
        self.out_proj = Linear(session, embed_dim, embed_dim, bias)
        self.dropout = Dropout(dropout)

    def _split(self, session, x):
        n, s, _ = session.tensor_shape(x)
        x = session.tensor_reshape(x, shape=(n, s, self.num_heads, self.head_dim))
        x = session.tensor_permute(x, dims=(0, 2, 1, 3))
        return session.tensor_reshape(x, shape=(n * self.num_heads, s, self.head_dim))

    def forward_qkv(self, session, q, k, v, attn_mask: Optional[int] = None, is_causal: bool = False,
                    key_padding_mask: Optional[int] = None):
        n, sq, _ = session.tensor_shape(q)
        sk = session.tensor_shape(k)[1]
        qh = self._split(session, self.q_proj(session, q))
        kh = self._split(session, self.k_proj(session, k))
        vh = self._split(session, self.v_proj(session, v))
        mask = attn_mask
        if mask is not None and session.tensor(mask).dtype == torch.bool:
            # module convention (as torch.nn.MultiheadAttention): True = this key is blocked for this query
            m = session.tensor(mask)
            mask = session.tensor_tape.leaf(torch.zeros_like(m, dtype=session.tensor(q).dtype).masked_fill(m, float("-inf")), False)
        if key_padding_mask is not None:
            kp = session.tensor(key_padding_mask).bool()            # [N, Sk], True = ignore
            add = torch.zeros(n, 1, 1, sk, dtype=session.tensor(q).dtype, device=session.device)
            add.masked_fill_(kp[:, None, None, :], float("-inf"))
            add = add.expand(n, self.num_heads, sq, sk).reshape(n * self.num_heads, sq, sk)
            if mask is not None:
                add = add + session.tensor(mask)
            mask = session.tensor_tape.leaf(add.contiguous(), False)
        scale = 1.0 / math.sqrt(self.head_dim)
        o = session.tensor_sdpa(qh, kh, vh, mask, is_causal=is_causal, scale=scale)
        o = session.tensor_reshape(o, shape=(n, self.num_heads, sq, self.head_dim))
        o = session.tensor_permute(o, dims=(0, 2, 1, 3))
        o = session.tensor_reshape(o, shape=(n, sq, self.embed_dim))
        return self.out_proj(session, o)

    def forward(self, session, x, attn_mask: Optional[int] = None, is_causal: bool = False,
                key_padding_mask: Optional[int] = None):
        return self.forward_qkv(session, x, x, x, attn_mask, is_causal, key_padding_mask)

    def forward_qkv_with_weights(self, session, q, k, v, attn_mask: Optional[int] = None, is_causal: bool = False,
                                 average_attn_weights: bool = True):
        """Attention output and the attention probabilities (ft-nn/src/lib.rs:5212): ``[N, Sq, Sk]`` averaged over
        the heads, or ``[N, heads, Sq, Sk]`` per head.  The probabilities are formed explicitly (scores, mask,
        softmax) out of session operators, so both results are differentiable; the output equals ``forward_qkv``."""
        n, sq, _ = session.tensor_shape(q)
        sk = session.tensor_shape(k)[1]
        qh = self._split(session, self.q_proj(session, q))
        kh = self._split(session, self.k_proj(session, k))
        vh = self._split(session, self.v_proj(session, v))
        scores = session.tensor_mul_scalar(session.tensor_bmm(qh, session.tensor_transpose(kh, dim0=1, dim1=2)),
                                           c=1.0 / math.sqrt(self.head_dim))
        add = None
        if is_causal:
            add = torch.triu(torch.full((sq, sk), float("-inf"), dtype=session.tensor(q).dtype, device=session.device), 1)
        if attn_mask is not None:
            m = session.tensor(attn_mask)
            m = torch.zeros_like(m, dtype=session.tensor(q).dtype).masked_fill(m, float("-inf")) if m.dtype == torch.bool else m
            add = m if add is None else add + m
        if add is not None:
            scores = session.tensor_add(scores, session.tensor_tape.leaf(add.expand(n * self.num_heads, sq, sk).contiguous(), False))
        probs = session.tensor_softmax(scores, dim=-1)
        o = session.tensor_bmm(session.functional_dropout(probs, self.dropout.p, self.training) if self.dropout.p else probs, vh)
        o = session.tensor_reshape(o, shape=(n, self.num_heads, sq, self.head_dim))
        o = session.tensor_permute(o, dims=(0, 2, 1, 3))
        o = session.tensor_reshape(o, shape=(n, sq, self.embed_dim))
        w = session.tensor_reshape(probs, shape=(n, self.num_heads, sq, sk))
        if average_attn_weights:
            w = session.tensor_mean_dim(w, dim=1)
        return self.out_proj(session, o), w

    def forward_qkv_causal(self, session, q, k, v):
        return self.forward_qkv(session, q, k, v, None, True)

    def forward_qkv_key_padding(self, session, q, k, v, key_padding_mask):
        return self.forward_qkv(session, q, k, v, None, False, key_padding_mask)

    def forward_qkv_masked(self, session, q, k, v, attn_mask):
        return self.forward_qkv(session, q, k, v, attn_mask, False)


class TransformerEncoderLayer(Module):
    def __init__(self, session, d_model: int, nhead: int, dim_feedforward: int = 2048, dropout: float = 0.1,
                 activation: str = "relu", norm_first: bool = False, layer_norm_eps: float = 1e-5):
        super().__init__()
        self.self_attn = MultiheadAttention(session, d_model, nhead, dropout)
        self.linear1 = Linear(session, d_model, dim_feedforward)
        self.linear2 = Linear(session, dim_feedforward, d_model)
        self.norm1 = LayerNorm(session, d_model, layer_norm_eps)
        self.norm2 = LayerNorm(session, d_model, layer_norm_eps)
        self.dropout = Dropout(dropout)
        self.dropout1 = Dropout(dropout)
        self.dropout2 = Dropout(dropout)
        if activation not in ("relu", "gelu"):
            raise ValueError("activation must be 'relu' or 'gelu'")
        self.activation, self.norm_first = activation, norm_first

    def _ff(self, session, x):
        h = self.linear1(session, x)
        h = session.tensor_relu(h) if self.activation == "relu" else session.tensor_gelu(h)
        return self.dropout2(session, self.linear2(session, self.dropout(session, h)))

    def forward(self, session, x, src_mask: Optional[int] = None, is_causal: bool = False,
                src_key_padding_mask: Optional[int] = None):
        """``src_mask`` is ``[S, S]`` (bool: True = blocked, or additive); ``src_key_padding_mask`` is ``[N, S]``
        with True at padded keys, which no query attends to."""
        sa = lambda t: self.self_attn(session, t, src_mask, is_causal, src_key_padding_mask)   # noqa: E731
        if self.norm_first:
            x = session.tensor_add(x, self.dropout1(session, sa(self.norm1(session, x))))
            return session.tensor_add(x, self._ff(session, self.norm2(session, x)))
        x = self.norm1(session, session.tensor_add(x, self.dropout1(session, sa(x))))
        return self.norm2(session, session.tensor_add(x, self._ff(session, x)))

    def forward_layer(self, session, src):
        """ft-nn/src/lib.rs:14696."""
        return self.forward(session, src)

    def forward_layer_masked(self, session, src, src_mask=None, src_key_padding_mask=None, is_causal: bool = False):
        """ft-nn/src/lib.rs:14709 (the reference's argument order)."""
        return self.forward(session, src, src_mask, is_causal, src_key_padding_mask)


class TransformerEncoder(Module):
    def __init__(self, session, layer_factory, num_layers: int, norm: Optional[Module] = None):
        super().__init__()
        self.layers = ModuleList([layer_factory() for _ in range(num_layers)])
        if norm is not None:
            self.norm = norm
        self._has_norm = norm is not None

    def forward(self, session, x, mask: Optional[int] = None, is_causal: bool = False,
                src_key_padding_mask: Optional[int] = None):
        for l in self.layers:
            x = l(session, x, mask, is_causal, src_key_padding_mask)
        return self.norm(session, x) if self._has_norm else x

    def forward_masked(self, session, src, mask=None, src_key_padding_mask=None, is_causal: bool = False):
        """ft-nn/src/lib.rs:14856."""
        return self.forward(session, src, mask, is_causal, src_key_padding_mask)


class TransformerDecoderLayer(Module):
    def __init__(self, session, d_model: int, nhead: int, dim_feedforward: int = 2048, dropout: float = 0.1,
                 activation: str = "relu", norm_first: bool = False, layer_norm_eps: float = 1e-5):
        super().__init__()
        self.self_attn = MultiheadAttention(session, d_model, nhead, dropout)
        self.multihead_attn = MultiheadAttention(session, d_model, nhead, dropout)
        self.linear1 = Linear(session, d_model, dim_feedforward)
        self.linear2 = Linear(session, dim_feedforward, d_model)
        self.norm1 = LayerNorm(session, d_model, layer_norm_eps)
        self.norm2 = LayerNorm(session, d_model, layer_norm_eps)
        self.norm3 = LayerNorm(session, d_model, layer_norm_eps)
        self.dropout = Dropout(dropout)
        self.dropout1, self.dropout2, self.dropout3 = Dropout(dropout), Dropout(dropout), Dropout(dropout)
        self.activation, self.norm_first = activation, norm_first

    def _ff(self, session, x):
        h = self.linear1(session, x)
        h = session.tensor_relu(h) if self.activation == "relu" else session.tensor_gelu(h)
        return self.dropout3(session, self.linear2(session, self.dropout(session, h)))

    def forward(self, session, tgt, memory, tgt_mask: Optional[int] = None, memory_mask: Optional[int] = None,
                tgt_is_causal: bool = False, tgt_key_padding_mask: Optional[int] = None,
                memory_key_padding_mask: Optional[int] = None, memory_is_causal: bool = False):
        add = session.tensor_add
        sa = lambda t: self.self_attn(session, t, tgt_mask, tgt_is_causal, tgt_key_padding_mask)   # noqa: E731
        ca = lambda t: self.multihead_attn.forward_qkv(session, t, memory, memory, memory_mask, memory_is_causal,   # noqa: E731
                                                       memory_key_padding_mask)
        if self.norm_first:
            x = add(tgt, self.dropout1(session, sa(self.norm1(session, tgt))))
            x = add(x, self.dropout2(session, ca(self.norm2(session, x))))
            return add(x, self._ff(session, self.norm3(session, x)))
        x = self.norm1(session, add(tgt, self.dropout1(session, sa(tgt))))
        x = self.norm2(session, add(x, self.dropout2(session, ca(x))))
        return self.norm3(session, add(x, self._ff(session, x)))

    def forward_layer(self, session, tgt, memory):
        """ft-nn/src/lib.rs:15066."""
        return self.forward(session, tgt, memory)

    def forward_layer_masked(self, session, tgt, memory, tgt_mask=None, memory_mask=None, tgt_key_padding_mask=None,
                             memory_key_padding_mask=None, tgt_is_causal: bool = False, memory_is_causal: bool = False):
        """ft-nn/src/lib.rs:15082 (the reference's argument order)."""
        return self.forward(session, tgt, memory, tgt_mask, memory_mask, tgt_is_causal, tgt_key_padding_mask,
                            memory_key_padding_mask, memory_is_causal)


class TransformerDecoder(Module):
    def __init__(self, session, layer_factory, num_layers: int, norm: Optional[Module] = None):
        super().__init__()
        self.layers = ModuleList([layer_factory() for _ in range(num_layers)])
        if norm is not None:
            self.norm = norm
        self._has_norm = norm is not None

    def forward(self, session, tgt, memory, tgt_mask=None, memory_mask=None, tgt_is_causal=False,
                tgt_key_padding_mask=None, memory_key_padding_mask=None, memory_is_causal=False):
        x = tgt
        for l in self.layers:
            x = l(session, x, memory, tgt_mask, memory_mask, tgt_is_causal, tgt_key_padding_mask,
                  memory_key_padding_mask, memory_is_causal)
        return self.norm(session, x) if self._has_norm else x

    def forward_decoder(self, session, tgt, memory):
        """ft-nn/src/lib.rs:15277."""
        return self.forward(session, tgt, memory)

    def forward_decoder_masked(self, session, tgt, memory, tgt_mask=None, memory_mask=None, tgt_key_padding_mask=None,
                               memory_key_padding_mask=None, tgt_is_causal: bool = False, memory_is_causal: bool = False):
        """ft-nn/src/lib.rs:15292."""
        return self.forward(session, tgt, memory, tgt_mask, memory_mask, tgt_is_causal, tgt_key_padding_mask,
                            memory_key_padding_mask, memory_is_causal)


class Transformer(Module):
    def __init__(self, session, d_model: int = 512, nhead: int = 8, num_encoder_layers: int = 6,
                 num_decoder_layers: int = 6, dim_feedforward: int = 2048, dropout: float = 0.1,
                 activation: str = "relu", norm_first: bool = False):
        super().__init__()
        enc = lambda: TransformerEncoderLayer(session, d_model, nhead, dim_feedforward, dropout, activation, norm_first)
        dec = lambda: TransformerDecoderLayer(session, d_model, nhead, dim_feedforward, dropout, activation, norm_first)
        self.encoder = TransformerEncoder(session, enc, num_encoder_layers, LayerNorm(session, d_model))
        self.decoder = TransformerDecoder(session, dec, num_decoder_layers, LayerNorm(session, d_model))

    def forward(self, session, src, tgt, src_mask=None, tgt_mask=None, memory_mask=None, src_key_padding_mask=None,
                tgt_key_padding_mask=None, memory_key_padding_mask=None, tgt_is_causal: bool = False):
        memory = self.encoder(session, src, src_mask, False, src_key_padding_mask)
        return self.decoder(session, tgt, memory, tgt_mask, memory_mask, tgt_is_causal, tgt_key_padding_mask,
                            memory_key_padding_mask)

    def forward_transformer(self, session, src, tgt):
        """ft-nn/src/lib.rs:15449."""
        return self.forward(session, src, tgt)

    def forward_transformer_masked(self, session, src, tgt, src_mask=None, tgt_mask=None, memory_mask=None,
                                   src_key_padding_mask=None, tgt_key_padding_mask=None, memory_key_padding_mask=None,
                                   tgt_is_causal: bool = False):
        """ft-nn/src/lib.rs:15469."""
        return self.forward(session, src, tgt, src_mask, tgt_mask, memory_mask, src_key_padding_mask,
                            tgt_key_padding_mask, memory_key_padding_mask, tgt_is_causal)


# -------------------------------------------------------------------------------------- recurrent
class _CellBase(Module):
    def __init__(self, session, input_size: int, hidden_size: int, gates: int, bias: bool = True):
        super().__init__()
        self.input_size, self.hidden_size = input_size, hidden_size
        k = 1.0 / math.sqrt(hidden_size)
        self.register_parameter("weight_ih", _param(session, (gates * hidden_size, input_size), "uniform", k))
        self.register_parameter("weight_hh", _param(session, (gates * hidden_size, hidden_size), "uniform", k))
        self.register_parameter("bias_ih", _param(session, (gates * hidden_size,), "uniform", k) if bias else None)
        self.register_parameter("bias_hh", _param(session, (gates * hidden_size,), "uniform", k) if bias else None)

    def _gates(self, session, x, h):
        P = self._parameters
        return (session.tensor_linear(x, P["weight_ih"], P["bias_ih"]),
                session.tensor_linear(h, P["weight_hh"], P["bias_hh"]))

    def forward_cell(self, session, x, hx):
        """One step under the reference's name (ft-nn/src/lib.rs:12576, :12738); ``hx`` is the hidden state, or the
        ``(h, c)`` pair of an LSTM cell."""
        return self.forward(session, x, hx)


class RNNCell(_CellBase):
    def __init__(self, session, input_size, hidden_size, bias=True, nonlinearity="tanh"):
        super().__init__(session, input_size, hidden_size, 1, bias)
        self.nonlinearity = nonlinearity

    def forward(self, session, x, h):
        gi, gh = self._gates(session, x, h)
        s = session.tensor_add(gi, gh)
        return session.tensor_tanh(s) if self.nonlinearity == "tanh" else session.tensor_relu(s)


class LSTMCell(_CellBase):
    def __init__(self, session, input_size, hidden_size, bias=True):
        super().__init__(session, input_size, hidden_size, 4, bias)

    def forward(self, session, x, state: Tuple[int, int]):
        h, c = state
        gi, gh = self._gates(session, x, h)
        g = session.tensor_add(gi, gh)
        H = self.hidden_size
        i, f, gg, o = (session.tensor_narrow(g, dim=-1 % len(session.tensor_shape(g)), start=k * H, length=H) for k in range(4))
        i, f, o = session.tensor_sigmoid(i), session.tensor_sigmoid(f), session.tensor_sigmoid(o)
        gg = session.tensor_tanh(gg)
        c2 = session.tensor_add(session.tensor_mul(f, c), session.tensor_mul(i, gg))
        return session.tensor_mul(o, session.tensor_tanh(c2)), c2


class GRUCell(_CellBase):
    def __init__(self, session, input_size, hidden_size, bias=True):
        super().__init__(session, input_size, hidden_size, 3, bias)

    def forward(self, session, x, h):
        gi, gh = self._gates(session, x, h)
        H, d = self.hidden_size, len(session.tensor_shape(gi)) - 1
        ir, iz, inn = (session.tensor_narrow(gi, dim=d, start=k * H, length=H) for k in range(3))
        hr, hz, hn = (session.tensor_narrow(gh, dim=d, start=k * H, length=H) for k in range(3))
        r = session.tensor_sigmoid(session.tensor_add(ir, hr))
        z = session.tensor_sigmoid(session.tensor_add(iz, hz))
        n = session.tensor_tanh(session.tensor_add(inn, session.tensor_mul(r, hn)))
        one_minus_z = session.tensor_add_scalar(session.tensor_neg(z), c=1.0)
        return session.tensor_add(session.tensor_mul(one_minus_z, n), session.tensor_mul(z, h))


class _Recurrent(Module):
    """Multi-layer recurrent stack built from cells, one cell per (layer, direction).

    Reference: ft-nn/src/lib.rs:13195 (``LSTM::new``: ``bidirectional``, ``dropout`` between layers,
    ``batch_first``), :13271 ``forward_lstm``, :13778 ``forward_gru``, :14245 ``forward_rnn``.  A bidirectional
    layer runs a second cell over the reversed sequence and concatenates the two outputs on the feature axis,
    so the next layer reads ``2 * hidden_size`` features.  States are ordered ``layer * num_directions +
    direction``, as in torch.  ``forward`` takes and returns per-cell lists of ``[N, H]`` nodes;
    ``forward_rnn / forward_gru / forward_lstm`` take and return the stacked ``[L * D, N, H]`` form."""

    cell_cls = RNNCell
    has_cell_state = False

    def __init__(self, session, input_size: int, hidden_size: int, num_layers: int = 1, bias: bool = True,
                 dropout: float = 0.0, bidirectional: bool = False, batch_first: bool = True):
        super().__init__()
        if num_layers < 1:
            raise ValueError(f"{type(self).__name__} num_layers must be >= 1")
        if not (math.isfinite(dropout) and 0.0 <= dropout <= 1.0):
            raise ValueError(f"{type(self).__name__} dropout probability must be finite and in [0, 1]")
        self.input_size, self.hidden_size, self.num_layers = input_size, hidden_size, num_layers
        self.bidirectional, self.batch_first = bool(bidirectional), bool(batch_first)
        d = self.num_directions
        self.cells = ModuleList([self.cell_cls(session, input_size if l == 0 else hidden_size * d, hidden_size, bias)
                                 for l in range(num_layers) for _ in range(d)])
        self.drop = Dropout(dropout)

    @property
    def num_directions(self) -> int:
        return 2 if self.bidirectional else 1

    def is_bidirectional(self) -> bool:
        return self.bidirectional

    def _run_cell(self, session, cell, steps, h, c):
        outs = []
        for t in steps:
            if self.has_cell_state:
                h, c = cell(session, t, (h, c))
            else:
                h = cell(session, t, h)
            outs.append(h)
        return outs, h, c

    def forward(self, session, x, state=None):
        time_dim = 1 if self.batch_first else 0
        shape = session.tensor_shape(x)
        if len(shape) != 3:
            raise ValueError(f"{type(self).__name__} expects a 3-D input, got shape {tuple(shape)}")
        n = shape[0] if self.batch_first else shape[1]
        steps = session.tensor_unbind(x, dim=time_dim)
        d, dt = self.num_directions, session.tensor_dtype(x)
        if state is not None and len(state[0]) != self.num_layers * d:
            raise ValueError(f"initial state has {len(state[0])} entries, the stack has {self.num_layers * d} cells")
        finals: List = []
        for l in range(self.num_layers):
            per_dir = []
            for k in range(d):
                idx = l * d + k
                h = session.zeros([n, self.hidden_size], dtype=dt) if state is None else state[0][idx]
                c = (session.zeros([n, self.hidden_size], dtype=dt) if state is None else state[1][idx]) \
                    if self.has_cell_state else None
                seq = steps if k == 0 else steps[::-1]
                outs, h, c = self._run_cell(session, self.cells[idx], seq, h, c)
                per_dir.append(outs if k == 0 else outs[::-1])
                finals.append((h, c))
            outs = per_dir[0] if d == 1 else [session.tensor_cat([f, r], dim=1) for f, r in zip(*per_dir)]
            steps = [self.drop(session, o) for o in outs] if l + 1 < self.num_layers else outs
        out = session.tensor_stack(steps, dim=time_dim)
        if self.has_cell_state:
            return out, ([h for h, _ in finals], [c for _, c in finals])
        return out, [h for h, _ in finals]

    def _split_state(self, session, packed):
        return None if packed is None else list(session.tensor_unbind(packed, dim=0))

    def _forward_packed(self, session, x, h_0=None, c_0=None):
        hs = self._split_state(session, h_0)
        if self.has_cell_state:
            if (h_0 is None) != (c_0 is None):
                raise ValueError("LSTM takes both initial states or neither")
            state = None if hs is None else (hs, self._split_state(session, c_0))
        else:
            state = None if hs is None else (hs, None)
        out, fin = _Recurrent.forward(self, session, x, state)
        if self.has_cell_state:
            return out, session.tensor_stack(fin[0], dim=0), session.tensor_stack(fin[1], dim=0)
        return out, session.tensor_stack(fin, dim=0), None


class RNN(_Recurrent):
    cell_cls = RNNCell

    def forward(self, session, x, state=None):
        return super().forward(session, x, None if state is None else (state, None))

    def forward_rnn(self, session, x, h_0=None):
        from .extra import RNNOutput
        out, h_n, _ = self._forward_packed(session, x, h_0)
        return RNNOutput(out, h_n)


class GRU(_Recurrent):
    cell_cls = GRUCell

    def forward(self, session, x, state=None):
        return super().forward(session, x, None if state is None else (state, None))

    def forward_gru(self, session, x, h_0=None):
        from .extra import GRUOutput
        out, h_n, _ = self._forward_packed(session, x, h_0)
        return GRUOutput(out, h_n)


class LSTM(_Recurrent):
    cell_cls = LSTMCell
    has_cell_state = True

    def forward_lstm(self, session, x, h_0=None, c_0=None):
        from .extra import LSTMOutput
        out, h_n, c_n = self._forward_packed(session, x, h_0, c_0)
        return LSTMOutput(out, h_n, c_n)


# -------------------------------------------------------------------------------------- losses
class LossModule(Module):
    op = "mse_loss"

    def __init__(self, reduction: str = "mean", **kw):
        super().__init__()
        self.kw = dict(kw)
        if reduction is not None:
            self.kw["reduction"] = reduction

    def forward(self, session, *inputs):
        return getattr(session, "tensor_" + self.op)(*inputs, **self.kw)


def _loss(op_name: str, reduction_default: Optional[str] = "mean"):
    class _L(LossModule):
        op = op_name

        def __init__(self, reduction: Optional[str] = reduction_default, **kw):
            super().__init__(reduction, **kw)
    _L.__name__ = op_name
    return _L


MSELoss, L1Loss = _loss("mse_loss"), _loss("l1_loss")
CrossEntropyLoss, NLLLoss = _loss("cross_entropy"), _loss("nll_loss")
BCELoss, BCEWithLogitsLoss = _loss("bce_loss"), _loss("bce_with_logits_loss")
SmoothL1Loss, HuberLoss = _loss("smooth_l1_loss"), _loss("huber_loss")
KLDivLoss = _loss("kl_div", "batchmean")
CosineEmbeddingLoss = _loss("cosine_embedding_loss", None)
TripletMarginLoss = _loss("triplet_margin_loss", None)
MultiMarginLoss = _loss("multi_margin_loss", None)
GaussianNLLLoss, PoissonNLLLoss = _loss("gaussian_nll_loss", None), _loss("poisson_nll_loss", None)
HingeEmbeddingLoss, SoftMarginLoss = _loss("hinge_embedding_loss", None), _loss("soft_margin_loss", None)
MarginRankingLoss, CTCLoss = _loss("margin_ranking_loss", None), _loss("ctc_loss", None)
FocalLoss, DiceLoss = _loss("focal_loss", None), _loss("dice_loss", None)
