"""GPU-resident transformer encoder stack for inference (the counterpart of the reference's
``EncoderGpu``, crates/ft-kernel-metal/src/fused.rs:1033-1189).

The reference uploads the six big matrices of every layer once (as f16), uploads the activation,
encodes 12 kernels per layer (LN, Wq, Wk, Wv, MHA, Wo, add, LN, W1, GELU, W2, add) into one
command buffer per chunk of layers (``FT_METAL_ENC_CHUNK``, default 8) and synchronises once per
chunk.  Here the weights live on the GPU in bf16, a layer is 7 launches of the sm_100a kernels

    LayerNorm -> [Wq;Wk;Wv] GEMM + bias -> flash attention (non-causal) -> Wo GEMM + bias + residual
    -> LayerNorm -> W1 GEMM + bias + GELU -> W2 GEMM + bias + residual

(the adds and the GELU ride in GEMM epilogues, q/k/v come from one GEMM and are read in place by
the attention kernel through strided tensor maps), and a chunk of layers is one CUDA graph that
is captured on first use for a sequence length and replayed afterwards.  ``FT_ENC_CHUNK`` plays
the role of ``FT_METAL_ENC_CHUNK``: it bounds the intermediates that are live at once and sets
the number of graph launches per forward to ``ceil(layers / chunk)``.

As in the reference the key projection has no bias (Whisper-style encoder), the GELU is the
clamped tanh form and the output is the stack output before any final LayerNorm.

``attach_stem`` + ``forward_from_mel`` run the encoder front as well (fused.rs:1060-1132): two
1-D convolutions over time (kernel 3, padding 1; stride 1, then stride 2) as im2col + GEMM with
the bias and the GELU in the epilogue, the positional embedding added as the second GEMM's
residual, then the layer stack.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

LN_EPS = 1e-5


@dataclass
class EncoderLayerWeights:
    """fp32 host-side weights of one layer, ``[out, in]`` matrices like ``nn.Linear``."""
    ln1_g: torch.Tensor
    ln1_b: torch.Tensor
    wq: torch.Tensor
    bq: torch.Tensor
    wk: torch.Tensor
    wv: torch.Tensor
    bv: torch.Tensor
    wo: torch.Tensor
    bo: torch.Tensor
    ln2_g: torch.Tensor
    ln2_b: torch.Tensor
    w1: torch.Tensor
    b1: torch.Tensor
    w2: torch.Tensor
    b2: torch.Tensor

    @staticmethod
    def random(d_model: int, d_ff: int, gen: torch.Generator) -> "EncoderLayerWeights":
        def mat(o, i):
            return torch.randn(o, i, generator=gen) * (1.0 / i ** 0.5)

        def vec(n, s=0.02):
            return torch.randn(n, generator=gen) * s
        return EncoderLayerWeights(
            1.0 + vec(d_model, 0.05), vec(d_model), mat(d_model, d_model), vec(d_model), mat(d_model, d_model),
            mat(d_model, d_model), vec(d_model), mat(d_model, d_model), vec(d_model), 1.0 + vec(d_model, 0.05),
            vec(d_model), mat(d_ff, d_model), vec(d_ff), mat(d_model, d_ff), vec(d_model))


def _gelu_tanh_clamped(x: torch.Tensor) -> torch.Tensor:
    # x >= 10 -> x, x <= -10 -> 0 (crates/ft-kernel-metal/src/fused.rs:302-313)
    y = torch.nn.functional.gelu(x, approximate="tanh")
    return torch.where(x >= 10, x, torch.where(x <= -10, torch.zeros_like(x), y))


def reference_forward(layers: Sequence[EncoderLayerWeights], x: torch.Tensor, n_heads: int) -> torch.Tensor:
    """The same stack in plain fp32/fp64 torch ops on any device (oracle for the GPU path)."""
    S, d = x.shape
    hd = d // n_heads
    for l in layers:
        w = {k: getattr(l, k).to(x) for k in l.__dataclass_fields__}
        n1 = torch.nn.functional.layer_norm(x, (d,), w["ln1_g"], w["ln1_b"], LN_EPS)
        q = n1 @ w["wq"].T + w["bq"]
        k = n1 @ w["wk"].T
        v = n1 @ w["wv"].T + w["bv"]
        qh, kh, vh = (t.view(S, n_heads, hd).transpose(0, 1) for t in (q, k, v))
        p = torch.softmax((qh @ kh.transpose(1, 2)) / hd ** 0.5, -1)
        attn = (p @ vh).transpose(0, 1).reshape(S, d)
        x1 = x + attn @ w["wo"].T + w["bo"]
        n2 = torch.nn.functional.layer_norm(x1, (d,), w["ln2_g"], w["ln2_b"], LN_EPS)
        x = x1 + _gelu_tanh_clamped(n2 @ w["w1"].T + w["b1"]) @ w["w2"].T + w["b2"]
    return x


@dataclass
class StemWeights:
    """Conv stem in the reference's upload layout (fused.rs:1064-1081): ``conv*_wt`` is
    ``[cin * 3, d_model]`` with row index ``ci * 3 + kk``; ``pos_emb`` is ``[n_ctx_cap, d_model]``."""
    conv1_wt: torch.Tensor
    conv1_b: torch.Tensor
    conv2_wt: torch.Tensor
    conv2_b: torch.Tensor
    pos_emb: torch.Tensor

    @staticmethod
    def random(n_mels: int, d_model: int, n_ctx_cap: int, gen: torch.Generator) -> "StemWeights":
        r = lambda *sh, s=1.0: torch.randn(*sh, generator=gen) * s
        return StemWeights(r(n_mels * 3, d_model, s=(n_mels * 3) ** -0.5), r(d_model, s=0.02),
                           r(d_model * 3, d_model, s=(d_model * 3) ** -0.5), r(d_model, s=0.02),
                           r(n_ctx_cap, d_model, s=0.1))


def stem_out_rows(t_in: int) -> int:
    """Rows after conv1 (k3, s1, p1: unchanged) and conv2 (k3, s2, p1: halved, rounded up)."""
    t1 = (t_in + 2 - 3) + 1
    return (t1 + 2 - 3) // 2 + 1


def reference_stem(stem: StemWeights, mel: torch.Tensor) -> torch.Tensor:
    """conv1 + GELU -> conv2 + GELU -> + pos_emb in plain torch (oracle); ``mel`` is ``[t_in, n_mels]``."""
    d = stem.conv1_b.shape[0]

    def conv(x, wt, b, stride):
        cin = x.shape[1]
        w = wt.to(x).T.reshape(d, cin, 3)                                  # [out, cin, k]
        y = torch.nn.functional.conv1d(x.T.unsqueeze(0), w, b.to(x), stride=stride, padding=1)
        return _gelu_tanh_clamped(y.squeeze(0).T)
    h = conv(conv(mel, stem.conv1_wt, stem.conv1_b, 1), stem.conv2_wt, stem.conv2_b, 2)
    return h + stem.pos_emb.to(mel)[: h.shape[0]]


class _GpuLayer:
    def __init__(self, l: EncoderLayerWeights, dev):
        bf = lambda t: t.to(dev, torch.bfloat16).contiguous()
        self.ln1_g, self.ln1_b, self.ln2_g, self.ln2_b = bf(l.ln1_g), bf(l.ln1_b), bf(l.ln2_g), bf(l.ln2_b)
        self.w_qkv = bf(torch.cat([l.wq, l.wk, l.wv], 0))                       # [3d, d]
        self.b_qkv = bf(torch.cat([l.bq, torch.zeros_like(l.bq), l.bv], 0))     # the key bias is zero
        self.wo, self.bo = bf(l.wo), bf(l.bo)
        self.w1, self.b1, self.w2, self.b2 = bf(l.w1), bf(l.b1), bf(l.w2), bf(l.b2)


class EncoderGpu:
    """Weights resident on the GPU; ``forward`` takes and returns host tensors."""

    def __init__(self, layers: Sequence[EncoderLayerWeights], n_heads: int, device="cuda:0",
                 chunk: Optional[int] = None, use_cuda_graph: bool = True):
        if not layers:
            raise ValueError("an encoder needs at least one layer")
        self.device = torch.device(device)
        self.d_model = int(layers[0].wq.shape[0])
        self.d_ff = int(layers[0].w1.shape[0])
        self.n_heads = int(n_heads)
        if self.d_model % self.n_heads or self.d_model // self.n_heads not in (64, 128):
            raise ValueError("head size must be 64 or 128")
        env = os.environ.get("FT_ENC_CHUNK")
        self.chunk = int(chunk if chunk is not None else (env if env and int(env) >= 1 else 8))
        if self.chunk < 1:
            raise ValueError("chunk must be at least 1")
        self.use_graph = use_cuda_graph
        self.layers = [_GpuLayer(l, self.device) for l in layers]
        self._graphs: Dict[int, Tuple[list, torch.Tensor, torch.Tensor]] = {}
        self.launches_per_layer = 7
        self.stem = None

    # ------------------------------------------------------------------ conv stem
    def attach_stem(self, stem: StemWeights, n_mels: int, n_ctx_cap: int) -> None:
        """Upload the conv stem and the positional embedding (bf16, resident)."""
        d = self.d_model
        if tuple(stem.conv1_wt.shape) != (n_mels * 3, d) or tuple(stem.conv2_wt.shape) != (d * 3, d):
            raise ValueError("conv weights must be [cin * 3, d_model]")
        if tuple(stem.pos_emb.shape) != (n_ctx_cap, d):
            raise ValueError("pos_emb must be [n_ctx_cap, d_model]")
        if (n_mels * 3) % 8:
            raise ValueError("n_mels * 3 must be a multiple of 8 (16-byte operand rows)")
        bf = lambda t: t.to(self.device, torch.bfloat16).contiguous()
        self.stem = dict(n_mels=n_mels, n_ctx_cap=n_ctx_cap, conv1_wt=bf(stem.conv1_wt), conv1_b=bf(stem.conv1_b),
                         conv2_wt=bf(stem.conv2_wt), conv2_b=bf(stem.conv2_b), pos_emb=bf(stem.pos_emb))

    def has_stem(self) -> bool:
        return self.stem is not None

    def _run_stem(self, mel_dev: torch.Tensor) -> torch.Tensor:
        """``mel_dev``: fp32 ``[t_in, n_mels]`` on the device -> bf16 ``[t2, d_model]``; 8 launches."""
        from ..ops import kernels as K
        st = self.stem
        c1 = K.cast_f32_to_bf16(K.im2col_1d(mel_dev, 3, 1, 1))
        g1 = K.gemm(c1, st["conv1_wt"], b_mn=True, bias=st["conv1_b"], epi=K.EPI_GELU_TANH)
        c2 = K.cast_f32_to_bf16(K.im2col_1d(K.cast_bf16_to_f32(g1), 3, 2, 1))
        t2 = c2.shape[0]
        return K.gemm(c2, st["conv2_wt"], b_mn=True, bias=st["conv2_b"], epi=K.EPI_GELU_TANH,
                      resid=st["pos_emb"][:t2])

    def forward_from_mel(self, mel: torch.Tensor, t_in: Optional[int] = None):
        """The whole encoder front from the mel spectrogram ``[t_in, n_mels]`` (host or device floats):
        conv1 (k3, s1, p1) + GELU -> conv2 (k3, s2, p1) + GELU -> + pos_emb -> layer stack.
        Returns ``(activations before any final LayerNorm as fp32 on the host, rows)``."""
        from ..ops import kernels as K
        if self.stem is None:
            raise RuntimeError("no conv stem attached (attach_stem)")
        n_mels = self.stem["n_mels"]
        t_in = int(mel.numel() // n_mels) if t_in is None else int(t_in)
        if t_in == 0 or mel.numel() != t_in * n_mels:
            raise ValueError(f"forward_from_mel input {mel.numel()} != {t_in}x{n_mels}")
        t2 = stem_out_rows(t_in)
        if t2 > self.stem["n_ctx_cap"]:
            raise ValueError(f"forward_from_mel: conv output {t2} rows > positional capacity {self.stem['n_ctx_cap']}")
        m = mel.reshape(t_in, n_mels).to(self.device, torch.float32, non_blocking=True).contiguous()
        x = self._run_stem(m)
        K.check_status()
        return self.forward_stack(x).to("cpu", torch.float32), t2

    # ------------------------------------------------------------------ one chunk, eager
    def _run_layers(self, x: torch.Tensor, layers: List[_GpuLayer]) -> torch.Tensor:
        from ..ops import kernels as K
        S, d, H = x.shape[0], self.d_model, self.n_heads
        hd = d // H
        for l in layers:
            n1 = K.layernorm_fwd(x, l.ln1_g, l.ln1_b, LN_EPS)[0]
            qkv = K.gemm(n1, l.w_qkv, bias=l.b_qkv)                          # [S, 3d]
            q, k, v = (qkv[:, i * d:(i + 1) * d].view(1, S, H, hd) for i in range(3))
            attn, _ = K.attention_fwd(q, k, v, causal=False)
            x1 = K.gemm(attn.view(S, d), l.wo, bias=l.bo, resid=x)
            n2 = K.layernorm_fwd(x1, l.ln2_g, l.ln2_b, LN_EPS)[0]
            h = K.gemm(n2, l.w1, bias=l.b1, epi=K.EPI_GELU_TANH)
            x = K.gemm(h, l.w2, bias=l.b2, resid=x1)
        return x

    def chunks(self) -> List[List[_GpuLayer]]:
        return [self.layers[i:i + self.chunk] for i in range(0, len(self.layers), self.chunk)]

    # ------------------------------------------------------------------ the chunked stack
    def forward_stack(self, x: torch.Tensor) -> torch.Tensor:
        """``x``: bf16 ``[seq, d_model]`` on the device.  One graph launch (or one eager pass) per
        chunk of layers; intermediates of a chunk are released before the next one runs."""
        from ..ops import kernels as K
        if not self.use_graph:
            for ch in self.chunks():
                x = self._run_layers(x, ch)
            K.check_status()
            return x
        S = int(x.shape[0])
        if S not in self._graphs:
            x_in = torch.empty_like(x)
            x_in.copy_(x)
            side = torch.cuda.Stream(self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):               # warm-up outside capture (lazy kernel attributes)
                y = x_in
                for ch in self.chunks():
                    y = self._run_layers(y, ch)
            torch.cuda.current_stream(self.device).wait_stream(side)
            torch.cuda.synchronize(self.device)
            graphs, cur = [], x_in
            for ch in self.chunks():
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    cur = self._run_layers(cur, ch)
                graphs.append(g)
            self._graphs[S] = (graphs, x_in, cur)
        graphs, x_in, out = self._graphs[S]
        x_in.copy_(x)
        for g in graphs:
            g.replay()
        K.check_status()
        return out

    def forward(self, inp: torch.Tensor, seq: Optional[int] = None) -> torch.Tensor:
        """``inp``: host (or device) ``[seq, d_model]`` floats; returns fp32 on the host."""
        inp = inp.reshape(-1, self.d_model) if seq is None else inp.reshape(seq, self.d_model)
        x = inp.to(self.device, torch.bfloat16, non_blocking=True).contiguous()     # the upload
        return self.forward_stack(x).to("cpu", torch.float32)                       # the download
