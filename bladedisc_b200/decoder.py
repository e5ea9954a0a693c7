"""Llama-shaped W8A8 decoder harness: the column-parallel configuration.

Shapes of the 7B configuration: 32 layers, hidden 4096, 32 heads, SwiGLU FFN
11008, RMSNorm, RoPE; int8 per-channel weights, per-token dynamic int8
activations; prefill, then decode steps.  Every linear is split by output
channels over the ranks of a :class:`bladedisc_b200.tp.Communicator` and
followed by an all-gather, except where the consumer works on the local columns
anyway (attention on the rank's own heads, the SwiGLU product).  With one rank
the same code runs without collectives.

Per layer and rank (g ranks, M tokens, H hidden, F ffn):

    rmsnorm + residual + per-token quantize          own kernel (reads gathered fp16 slabs)
    QKV linear  [M,H] -> [M, 3H/g] fp16              own kernel (local heads, no gather)
    RoPE, KV cache, attention on H/g columns         torch (SDPA: a library call, as the
                                                     reference's batched ral_gemm is)
    row scales: local max -> max over ranks          own kernel + NCCL all-reduce
    quantize into slot r of [g,M,H/g] int8           own kernel, NCCL all-gather in place
    O linear (gathered int8 in) -> slot r of [g,M,H/g] fp16, all-gather
    rmsnorm + residual + per-token quantize
    gate-up linear [M,H] -> [M, 2F/g] fp16           own kernel (local)
    silu(gate)*up row scales / quantize -> slot r of [g,M,F/g] int8, all-gather
    down linear (gathered int8 in) -> slot r of [g,M,H/g] fp16, all-gather

Weights are random (~N(0, 0.02)), generated from a seed on the device, the full
matrix on every rank and then cut, so that any number of ranks computes the
same model.
"""
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F
from torch.nn.attention import SDPBackend, sdpa_kernel

from . import ops
from .tp import ColumnParallelQLinear, Communicator, column_share, quantize_rows_gathered


@dataclass
class DecoderConfig:
    layers: int = 32
    hidden: int = 4096
    heads: int = 32
    ffn: int = 11008
    vocab: int = 32000
    rope_theta: float = 10000.0
    eps: float = 1e-5

    @staticmethod
    def llama7b(layers: int = 32) -> "DecoderConfig":
        return DecoderConfig(layers=layers)

    @staticmethod
    def tiny() -> "DecoderConfig":
        return DecoderConfig(layers=2, hidden=256, heads=4, ffn=512, vocab=1000)

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads


def _quantize_weight(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-output-channel symmetric int8, the offline rule of the reference's
    QuantizeOp::fold (double precision, round half to even)."""
    scale = (w.abs().amax(dim=1) / 127.0).clamp_min(torch.finfo(torch.float32).eps)
    q = torch.round(w.double() / scale.double()[:, None]).clamp_(-128, 127).to(torch.int8)
    return q, scale.float()


_SDPA_BACKENDS = [SDPBackend.FLASH_ATTENTION, SDPBackend.EFFICIENT_ATTENTION, SDPBackend.MATH]


class _Layer:
    pass


class QuantDecoder:
    def __init__(self, cfg: DecoderConfig, comm: Optional[Communicator] = None, seed: int = 1238,
                 device: str = "cuda"):
        self.cfg, self.comm = cfg, comm
        self.world = comm.world if comm else 1
        self.rank = comm.rank if comm else 0
        self.device = torch.device(device)
        if cfg.heads % self.world:
            raise ValueError("heads must split evenly over the ranks")
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed)

        def rnd(*shape, std=0.02):
            return torch.randn(*shape, generator=gen, device=self.device) * std

        H, Fn = cfg.hidden, cfg.ffn
        self.embed = rnd(cfg.vocab, H).half()
        self.layers: List[_Layer] = []
        hb, he = column_share(H, self.world, self.rank)
        fb, fe = column_share(Fn, self.world, self.rank)
        for _ in range(cfg.layers):
            L = _Layer()
            wq, wk, wv, wo = rnd(H, H), rnd(H, H), rnd(H, H), rnd(H, H)
            wg, wu, wd = rnd(Fn, H), rnd(Fn, H), rnd(H, Fn)
            L.g1 = (1.0 + rnd(H, std=0.1)).half()
            L.g2 = (1.0 + rnd(H, std=0.1)).half()
            # the rank's heads of q, k, v side by side; its gate and up channels side by side
            qkv = [_quantize_weight(w[hb:he]) for w in (wq, wk, wv)]
            L.qkv = self._linear(torch.cat([q for q, _ in qkv]), torch.cat([s for _, s in qkv]))
            gu = [_quantize_weight(w[fb:fe]) for w in (wg, wu)]
            L.gate_up = self._linear(torch.cat([q for q, _ in gu]), torch.cat([s for _, s in gu]))
            L.o = self._linear(*_quantize_weight(wo[hb:he]))
            L.down = self._linear(*_quantize_weight(wd[hb:he]))
            self.layers.append(L)
            del wq, wk, wv, wo, wg, wu, wd
        self.g_final = (1.0 + rnd(H, std=0.1)).half()
        torch.cuda.synchronize(self.device)  # the weights are final: linears may fetch them early
        for L in self.layers:
            for lin in (L.qkv, L.o, L.gate_up, L.down):
                lin.weights_static = True
        self.kv: Optional[List[Tuple[torch.Tensor, torch.Tensor]]] = None
        self.pos = 0
        self._cos = self._sin = None

    def _linear(self, wq: torch.Tensor, scale: torch.Tensor) -> ColumnParallelQLinear:
        return ColumnParallelQLinear(wq, scale, None, self.comm, rows=(0, wq.shape[0]))

    # ------------------------------------------------------------------ pieces
    def _rope_tables(self, upto: int) -> None:
        half = self.cfg.head_dim // 2
        inv = self.cfg.rope_theta ** (-torch.arange(half, device=self.device, dtype=torch.float32) / half)
        ang = torch.arange(upto, device=self.device, dtype=torch.float32)[:, None] * inv[None, :]
        self._cos, self._sin = ang.cos(), ang.sin()

    def _rope(self, x: torch.Tensor, pos0: int) -> torch.Tensor:
        """x [B, S, h, d]; rotates pairs (i, i + d/2) by position * theta^(-2i/d)."""
        b, s, h, d = x.shape
        half = d // 2
        if getattr(self, "_cos", None) is None or self._cos.shape[0] < pos0 + s:
            self._rope_tables(max(pos0 + s, 256))
        cos = self._cos[pos0:pos0 + s][None, :, None, :]
        sin = self._sin[pos0:pos0 + s][None, :, None, :]
        xf = x.float()
        x1, x2 = xf[..., :half], xf[..., half:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).half()

    def _attention(self, L: _Layer, idx: int, qkv: torch.Tensor, batch: int, seq: int) -> torch.Tensor:
        cfg = self.cfg
        hl, d = cfg.heads // self.world, cfg.head_dim
        kc, vc = self.kv[idx]
        # q and k rotated, k and v appended to the cache: one pass over the QKV output
        ops.rope_kv_append(qkv, kc, vc, self._cos, self._sin, batch, seq, self.pos)
        q = qkv.view(batch, seq, 3, hl, d)[:, :, 0]
        end = self.pos + seq
        # Library attention, without the backend that builds a new plan for every
        # cache length (tens of milliseconds on the host per decode step).
        with sdpa_kernel(_SDPA_BACKENDS):
            if self.pos == 0:
                o = F.scaled_dot_product_attention(q.transpose(1, 2), kc[:, :, :end], vc[:, :, :end], is_causal=True)
            else:  # decode: the new tokens see the whole cache
                o = F.scaled_dot_product_attention(q.transpose(1, 2), kc[:, :, :end], vc[:, :, :end])
        return o.transpose(1, 2).reshape(batch * seq, hl * d)

    def start(self, batch: int, max_seq: int) -> None:
        cfg = self.cfg
        hl, d = cfg.heads // self.world, cfg.head_dim
        self.kv = [(torch.zeros(batch, hl, max_seq, d, dtype=torch.float16, device=self.device),
                    torch.zeros(batch, hl, max_seq, d, dtype=torch.float16, device=self.device))
                   for _ in range(cfg.layers)]
        self.pos = 0
        self._rope_tables(max_seq)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [B, S] (prefill when the cache is empty, else S new tokens per
        sequence) -> final hidden states [B * S, H] fp16."""
        cfg = self.cfg
        batch, seq = ids.shape
        if self.kv is None:
            raise RuntimeError("call start(batch, max_seq) first")
        h = self.embed[ids.reshape(-1)]  # [M, H] residual stream, replicated
        prev = None  # gathered fp16 output of the previous sublayer
        for idx, L in enumerate(self.layers):
            if prev is None:
                xq, xs, _ = ops.rmsnorm_dynamic_quant(h, L.g1, cfg.eps)
            else:
                xq, xs, h = ops.rmsnorm_dynamic_quant(prev, L.g1, cfg.eps, residual=h, x_gathered=True)
            qkv = L.qkv.forward(xq, xs, gather=False)
            att = self._attention(L, idx, qkv, batch, seq)
            aq, a_s = quantize_rows_gathered(self.comm, att)
            o = L.o.forward(aq, a_s, a_gathered=True)
            xq, xs, h = ops.rmsnorm_dynamic_quant(o, L.g2, cfg.eps, residual=h, x_gathered=True)
            gu = L.gate_up.forward(xq, xs, gather=False)
            fl = gu.shape[1] // 2
            hq, h_s = quantize_rows_gathered(self.comm, gu[:, :fl], gu[:, fl:])
            prev = L.down.forward(hq, h_s, a_gathered=True)
        self.pos += seq
        # final norm straight from the gathered output of the last layer
        return ops.rmsnorm(prev, self.g_final, cfg.eps, residual=h, x_gathered=True)

    def launches_per_layer(self) -> int:
        """Kernels of this library per layer and rank (collectives and torch ops not counted)."""
        return 2 + 4 + 4  # two norms, four linears, two two-pass quantizations


def reference_forward(dec: QuantDecoder, ids: torch.Tensor) -> torch.Tensor:
    """The same model in plain torch on ONE GPU from a world-1 decoder's
    weights: fp32 math with the quantization points of the kernel path restated
    as fake-quant (per-token scale s = max|x| / 127, level = x * fl(1 / s)
    rounded once, half to even: the reciprocal form of the row kernels).  Used by
    the tests as the end-to-end oracle; no cache (prefill only)."""
    if dec.world != 1:
        raise ValueError("reference_forward takes an unsharded decoder")
    cfg = dec.cfg
    batch, seq = ids.shape

    def fq_rows(x):
        s = (x.abs().amax(dim=1, keepdim=True) / 127.0).clamp_min(torch.finfo(torch.float32).eps)
        inv = (1.0 / s).double()  # fl(1 / s); the product in double is exact, so one rounding as in a fused multiply-add
        return torch.round(x.double() * inv).clamp(-128, 127).float() * s

    def lin(layer: ColumnParallelQLinear, x):
        w = layer.wq.float() * layer.w_scale[:, None]
        return (x @ w.t()).half().float()

    def rms(x, g):  # the normalized row exists in fp16 before it is quantized
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(dim=1, keepdim=True) + cfg.eps) * g.float()).half().float()

    h = dec.embed[ids.reshape(-1)]
    prev = None
    for L in dec.layers:
        if prev is not None:
            h = (h.float() + prev).half()
        x = fq_rows(rms(h, L.g1))
        qkv = lin(L.qkv, x).half()
        hl, d = cfg.heads, cfg.head_dim
        q, k, v = qkv.view(batch, seq, 3, hl, d).unbind(dim=2)
        save = dec.pos
        dec.pos = 0
        q, k = dec._rope(q, 0), dec._rope(k, 0)
        dec.pos = save
        # the same library call as the kernel path: attention is not one of the kernels under test
        with sdpa_kernel(_SDPA_BACKENDS):
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2).contiguous(),
                                               v.transpose(1, 2).contiguous(), is_causal=True)
        att = o.transpose(1, 2).reshape(batch * seq, hl * d).float()
        o = lin(L.o, fq_rows(att))
        h = (h.float() + o).half()
        x = fq_rows(rms(h, L.g2))
        gu = lin(L.gate_up, x)
        fl = gu.shape[1] // 2
        act = F.silu(gu[:, :fl]) * gu[:, fl:]
        prev = lin(L.down, fq_rows(act))
    h = (h.float() + prev).half()
    return rms(h, dec.g_final).half()
