"""W8A8 transformer-encoder harness built from the quantized-path kernels.

This is what a torch_quant-quantized, DISC-compiled BERT-shaped encoder
executes at run time, written as a sequence of the library's calls: every
Linear is an int8 `qgemm` (per-channel weight scales, static per-tensor
activation scales from calibration), LayerNorm / softmax / quantize are the
row kernels, and the epilogues carry the fusions the reference needs separate
generated kernels for (dequantize + bias [+ GELU] [+ quantize]).

Sequences are packed: the rows of every linear, LayerNorm and quantize are
the real tokens of the batch, one sequence after the other, without padding
rows.  Self-attention is one fused kernel per layer (`ops.attention`: Q K^T,
masked softmax, P V and the quantize of the context, scores kept on chip); in
the reference the two products are `ral_gemm` = cuBLAS through StreamExecutor
(tao_compiler/mlir/ral/context/stream_executor_based_impl.cc:551-637) with a
generated softmax between them.  The embedding gather is torch indexing.
Everything else is this library.

Weights are random (N(0, 0.02)) and token ids synthetic: there is no network
for checkpoints or datasets.
"""
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from . import ops, quant


@dataclass
class EncoderConfig:
    layers: int = 12
    hidden: int = 768
    heads: int = 12
    ffn: int = 3072
    vocab: int = 30522
    max_len: int = 512
    eps: float = 1e-12

    @staticmethod
    def bert_base():
        return EncoderConfig()

    @staticmethod
    def bert_large():
        return EncoderConfig(layers=24, hidden=1024, heads=16, ffn=4096)

    @staticmethod
    def tiny():
        return EncoderConfig(layers=2, hidden=128, heads=2, ffn=256, vocab=1000, max_len=64)


@dataclass
class LayerWeights:
    wqkv: torch.Tensor
    bqkv: torch.Tensor
    wo: torch.Tensor
    bo: torch.Tensor
    w1: torch.Tensor
    b1: torch.Tensor
    w2: torch.Tensor
    b2: torch.Tensor
    ln1_g: torch.Tensor
    ln1_b: torch.Tensor
    ln2_g: torch.Tensor
    ln2_b: torch.Tensor


@dataclass
class FloatEncoder:
    """fp32 master weights (what a checkpoint would hold)."""
    cfg: EncoderConfig
    word: torch.Tensor
    pos: torch.Tensor
    emb_g: torch.Tensor
    emb_b: torch.Tensor
    layers: List[LayerWeights] = field(default_factory=list)


def init_float_encoder(cfg: EncoderConfig, seed: int = 1234, device="cuda") -> FloatEncoder:
    g = torch.Generator(device="cpu").manual_seed(seed)

    def rnd(*shape, std=0.02):
        return (torch.randn(*shape, generator=g) * std).to(device)

    H, Fd = cfg.hidden, cfg.ffn
    enc = FloatEncoder(cfg, rnd(cfg.vocab, H), rnd(cfg.max_len, H), torch.ones(H, device=device),
                       torch.zeros(H, device=device))
    for _ in range(cfg.layers):
        enc.layers.append(LayerWeights(
            wqkv=rnd(3 * H, H), bqkv=rnd(3 * H, std=0.01), wo=rnd(H, H), bo=rnd(H, std=0.01),
            w1=rnd(Fd, H), b1=rnd(Fd, std=0.01), w2=rnd(H, Fd), b2=rnd(H, std=0.01),
            ln1_g=torch.ones(H, device=device), ln1_b=torch.zeros(H, device=device),
            ln2_g=torch.ones(H, device=device), ln2_b=torch.zeros(H, device=device)))
    return enc


def _attention_fp(q, k, v, lens, heads):
    B, L, H = q.shape
    d = H // heads
    q = q.view(B, L, heads, d).transpose(1, 2)
    k = k.view(B, L, heads, d).transpose(1, 2)
    v = v.view(B, L, heads, d).transpose(1, 2)
    s = torch.matmul(q, k.transpose(-1, -2)) / math.sqrt(d)
    mask = torch.arange(L, device=q.device)[None, :] >= lens[:, None]
    s = s.masked_fill(mask[:, None, None, :], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, v).transpose(1, 2).reshape(B, L, H)


def float_forward(enc: FloatEncoder, ids: torch.Tensor, lens: torch.Tensor,
                  scales: Optional[Dict[str, torch.Tensor]] = None, observe: Optional[Dict[str, float]] = None):
    """Eager fp32 forward.  With `scales` it is the fake-quant model (the functional
    golden the reference's e2e tests use: fake_quantize on every Linear input and
    per-channel on every weight); with `observe` it records max|x| at the same
    points for calibration."""
    cfg = enc.cfg
    B, L = ids.shape

    def point(name, x):
        if observe is not None:
            observe[name] = max(observe.get(name, 0.0), float(x.abs().max()))
        if scales is not None:
            return torch.fake_quantize_per_tensor_affine(x, float(scales[name]), 0, -128, 127)
        return x

    def weight(w):
        if scales is None:
            return w
        s = quant.per_channel_scale(w)
        return torch.fake_quantize_per_channel_affine(w, s, torch.zeros_like(s, dtype=torch.int32), 0, -128, 127)

    x = enc.word[ids] + enc.pos[:L][None]
    x = F.layer_norm(x, (cfg.hidden,), enc.emb_g, enc.emb_b, cfg.eps)
    for i, lw in enumerate(enc.layers):
        xin = point(f"l{i}.attn_in", x)
        qkv = F.linear(xin, weight(lw.wqkv), lw.bqkv)
        q, k, v = qkv.split(cfg.hidden, dim=-1)
        ctx = _attention_fp(q, k, v, lens, cfg.heads)
        ctx = point(f"l{i}.ctx", ctx)
        attn = F.linear(ctx, weight(lw.wo), lw.bo)
        h1 = F.layer_norm(attn + x, (cfg.hidden,), lw.ln1_g, lw.ln1_b, cfg.eps)
        mid = F.gelu(F.linear(point(f"l{i}.ffn_in", h1), weight(lw.w1), lw.b1))
        mid = point(f"l{i}.ffn_mid", mid)
        ffn = F.linear(mid, weight(lw.w2), lw.b2)
        x = F.layer_norm(ffn + h1, (cfg.hidden,), lw.ln2_g, lw.ln2_b, cfg.eps)
    return x


def synthetic_batch(cfg: EncoderConfig, batch: int, min_len: int, max_len: int, seed: int, device="cuda"):
    """Token ids uniform over the vocabulary, one length per sequence uniform in [min_len, max_len]."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    lens = torch.randint(min_len, max_len + 1, (batch,), generator=g)
    L = int(lens.max())
    ids = torch.randint(0, cfg.vocab, (batch, L), generator=g)
    return ids.to(device), lens.to(device=device, dtype=torch.int32)


def calibrate(enc: FloatEncoder, batches: Sequence[Tuple[torch.Tensor, torch.Tensor]]) -> Dict[str, torch.Tensor]:
    """Activation scales max|x| / 127 at every Linear input, over calibration batches."""
    seen: Dict[str, float] = {}
    with torch.no_grad():
        for ids, lens in batches:
            float_forward(enc, ids, lens, observe=seen)
    dev = enc.word.device
    return {k: torch.tensor([max(v / 127.0, 1e-8)], dtype=torch.float32, device=dev) for k, v in seen.items()}


class QuantEncoder:
    """int8 weights + scales on the device; forward() runs the quantized path."""

    def __init__(self, enc: FloatEncoder, scales: Dict[str, torch.Tensor]):
        self.cfg = enc.cfg
        self.scales = scales
        h = torch.float16
        self.word = enc.word.to(h)
        self.pos = enc.pos.to(h)
        self.emb_g, self.emb_b = enc.emb_g.to(h), enc.emb_b.to(h)
        self.layers = []
        for lw in enc.layers:
            d = {}
            for name in ("wqkv", "wo", "w1", "w2"):
                wq, ws = quant.quantize_linear(getattr(lw, name), per_channel=True)
                d[name], d[name + "_s"] = wq.contiguous(), ws
            for name in ("bqkv", "bo", "b1", "b2"):
                d[name] = getattr(lw, name).float().contiguous()
            for name in ("ln1_g", "ln1_b", "ln2_g", "ln2_b"):
                d[name] = getattr(lw, name).to(h)
            self.layers.append(d)
        self.kernel_launches = 0
        self.rows_processed = 0

    # ------------------------------------------------------------------ batch plan
    def prepare(self, ids: torch.Tensor, lens: torch.Tensor) -> None:
        """Host-side plan for one batch shape: where every real token sits in the padded `ids`, the work list
        of the attention kernel, and the first token of every sequence.  Reads `lens` on the host (one
        synchronisation), so it is called once per batch shape, outside any stream capture; `forward_packed`
        then only launches kernels."""
        lens_h = [int(v) for v in lens.cpu().tolist()]
        B, L = ids.shape
        if len(lens_h) != B or any(n < 1 or n > L for n in lens_h):
            raise ValueError("lens must hold one length in 1..L per sequence")
        dev = ids.device
        flat = torch.cat([torch.arange(n, dtype=torch.int64) + b * L for b, n in enumerate(lens_h)])
        pos = torch.cat([torch.arange(n, dtype=torch.int64) for n in lens_h])
        starts = torch.tensor([0] + lens_h[:-1], dtype=torch.int64).cumsum(0)
        self._plan = {
            "key": (B, L, tuple(lens_h)), "flat": flat.to(dev), "pos": pos.to(dev), "first": starts.to(dev),
            "blocks": self._pick_attention_blocks(lens_h, dev), "tokens": int(sum(lens_h)), "lens": lens_h,
        }
        self.rows_processed = self._plan["tokens"]

    def _pick_attention_blocks(self, lens_h, dev) -> torch.Tensor:
        """Work list of the attention kernel for this batch: items of four, two or one query blocks -- the largest
        that still gives two thread blocks per SM.  Whole-sequence items fetch keys and values once and win when the
        batch has many more items than the GPU has SMs (34 against 43 us on 32 sequences of up to 512 tokens); on a
        rank's small share one block per item does (9 against 28 us on 4 sequences)."""
        heads = self.cfg.heads
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        for g in (4, 2):
            b = ops.attention_blocks(lens_h, heads, group=g)
            if b.shape[0] * heads >= 2 * sms:
                return b.to(dev)
        return ops.attention_blocks(lens_h, heads, group=1).to(dev)

    def _plan_for(self, ids, lens):
        plan = getattr(self, "_plan", None)
        if plan is None or plan["key"][:2] != tuple(ids.shape):
            self.prepare(ids, lens)
        return self._plan

    def describe(self) -> str:
        return ("sequences packed (rows of the linears = real tokens); self-attention is this library's fused "
                "kernel (tcgen05 kind::f16, scores in TMEM, int8 context out); embedding gather by torch indexing; "
                "every other kernel is this library's")

    def first_tokens(self, packed: torch.Tensor) -> torch.Tensor:
        """Row of the first token of every sequence ([CLS]) of a packed result."""
        return packed[self._plan["first"]]

    def forward_packed(self, ids: torch.Tensor, lens: torch.Tensor) -> torch.Tensor:
        """[tokens, hidden] f16, sequences one after the other."""
        cfg = self.cfg
        plan = self._plan_for(ids, lens)
        H, heads = cfg.hidden, cfg.heads
        sc = self.scales
        n = 0
        emb = self.word[ids.reshape(-1)[plan["flat"]]] + self.pos[plan["pos"]]
        x, xq = ops.layernorm_quant(emb, self.emb_g, self.emb_b, sc["l0.attn_in"], eps=cfg.eps)
        n += 1
        inv_sqrt_d = 1.0 / math.sqrt(H // heads)
        for i, lw in enumerate(self.layers):
            qkv = ops.qgemm(xq, lw["wqkv"], x_scale=sc[f"l{i}.attn_in"], w_scale=lw["wqkv_s"], bias=lw["bqkv"],
                            out_dtype=torch.float16)
            ctxq = ops.attention(qkv, plan["blocks"], heads, inv_sqrt_d, out_scale=sc[f"l{i}.ctx"])
            attn = ops.qgemm(ctxq, lw["wo"], x_scale=sc[f"l{i}.ctx"], w_scale=lw["wo_s"], bias=lw["bo"],
                             out_dtype=torch.float16)
            h1, h1q = ops.layernorm_quant(attn, lw["ln1_g"], lw["ln1_b"], sc[f"l{i}.ffn_in"], eps=cfg.eps, residual=x)
            midq = ops.qgemm(h1q, lw["w1"], x_scale=sc[f"l{i}.ffn_in"], w_scale=lw["w1_s"], bias=lw["b1"], act="gelu",
                             out_scale=sc[f"l{i}.ffn_mid"])
            ffn = ops.qgemm(midq, lw["w2"], x_scale=sc[f"l{i}.ffn_mid"], w_scale=lw["w2_s"], bias=lw["b2"],
                            out_dtype=torch.float16)
            nxt = sc[f"l{i + 1}.attn_in"] if i + 1 < len(self.layers) else sc[f"l{i}.attn_in"]
            x, xq = ops.layernorm_quant(ffn, lw["ln2_g"], lw["ln2_b"], nxt, eps=cfg.eps, residual=h1)
            n += 7
        self.kernel_launches += n
        return x

    def forward(self, ids: torch.Tensor, lens: torch.Tensor) -> torch.Tensor:
        """[B, L, hidden] f16 with the packed result scattered back to the padded layout (padding rows zero)."""
        B, L = ids.shape
        self.prepare(ids, lens)
        packed = self.forward_packed(ids, lens)
        out = torch.zeros((B * L, self.cfg.hidden), dtype=packed.dtype, device=packed.device)
        out[self._plan["flat"]] = packed
        return out.view(B, L, self.cfg.hidden)


def build_quant_encoder(cfg: EncoderConfig, seed: int = 1234, device="cuda", calib_batches: int = 4,
                        calib_batch: int = 8, min_len: int = 16, max_len: Optional[int] = None):
    """Random-init encoder, calibrated on `calib_batches` seeded synthetic batches."""
    max_len = max_len or cfg.max_len
    enc = init_float_encoder(cfg, seed, device)
    batches = [synthetic_batch(cfg, calib_batch, min_len, max_len, seed + 100 + i, device) for i in range(calib_batches)]
    scales = calibrate(enc, batches)
    return enc, QuantEncoder(enc, scales), scales


def shard_batch(ids: torch.Tensor, lens: torch.Tensor, world: int, rank: int):
    """This rank's sequences (balanced by packed work, see sharding.balance_packed), re-padded to its own longest."""
    from .sharding import balance_packed
    assign = balance_packed(lens.tolist(), world)[rank]
    if not assign:
        return ids[:0, :1], lens[:0], assign
    idx = torch.tensor(assign, device=ids.device)
    my_lens = lens[idx]
    L = int(my_lens.max())
    mine = ids[idx][:, :L]
    if mine.shape[1] < L:
        mine = torch.nn.functional.pad(mine, (0, L - mine.shape[1]))
    return mine.contiguous(), my_lens.contiguous(), assign
