"""Ninelix: a decoder-only design of post-normed sub-layers over a 32-bit residual stream, with a different token mixer
per layer -- recurrent ones (RWKV-style time mixing, lightning attention, Mamba-2) and softmax attention.

    x = embed[token] + bigram[hash(previous token, token)]            (32-bit from here on)
    layer:   x <- x + norm1(mixer(x)) ;  x <- x + norm2(ffn(x))       the sub-layers read x itself; the norm
                                                                      rms_div(y) * (1 + w) sits on their OUTPUT
    mixers:  "wkv" | "lightning" | "parallel" (biased attention beside Mamba-2, normed and averaged)   -> models/mixers.py
    ffn:     dense (erf-GELU) | routed experts (gated SiLU, softmax over the chosen logits) | none    -> mixers / blocks
    logits = head (rms_div(x) * (1 + final.norm)) * logit_scale

config.json keys: architecture, vocab, width, norm.eps, logit_scale, embedding.bigram{buckets, mul_prev, mul_cur},
layers[i].{type, mixer{...}, mlp{kind, ff | expert.ff, router{experts, top}} | null}.  Tensor names: embed, bigram,
head, final.norm, l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.* (listed with each loader below).

The model is a graph over the framework's ops.  What a sequence carries between steps lives in the engine's
HybridCache: pages for the attention layers' keys / values, one state slot for recurrent states, convolution tails,
the token-shift row and the previous token.  Runner, block and slot allocators, batching and sampler drive it like the
other families.  It runs unsharded (TP = 1).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch
from torch import nn

from .. import ops
from ..engine.batch import BatchInput
from ..engine.kv_cache import HybridCache
from ..ops import ACT_SILU
from ..parallel.comm import comm_for
from ..utils.tracing import trace
from .blocks import RoutedExperts
from .mixers import (BiasedAttention, DenseFFN, LayerCacheView, LightningMixer, ParallelPair, SsdMixer, WkvMixer)

MIXER_TYPES = ("wkv", "lightning", "parallel")
FFN_KINDS = ("dense", "moe")


@dataclass
class NinelixSpec:
    hidden: int
    vocab: int
    eps: float
    logit_scale: float
    buckets: int
    mul_prev: int
    mul_cur: int
    layers: List[dict] = field(default_factory=list)      # the config's layer entries, checked
    model_type: str = "ninelix"
    max_pos: int = 1 << 30       # positions enter only through relative distances: no limit of its own
    default_seq_len: int = 4096  # block-table width when the caller names neither a length nor a pool
    learned_pos: bool = False

    @property
    def n_layers(self) -> int:
        return len(self.layers)


def ninelix_spec(config) -> NinelixSpec:
    c = config.raw if hasattr(config, "raw") else dict(config)
    bg = c["embedding"]["bigram"]
    for i, lc in enumerate(c["layers"]):
        if lc["type"] not in MIXER_TYPES:
            raise ValueError(f"ninelix: layer {i} has unknown mixer type {lc['type']!r}; have {MIXER_TYPES}")
        f = lc.get("mlp")
        if f is not None and f.get("kind") not in FFN_KINDS:
            raise ValueError(f"ninelix: layer {i} has unknown feed-forward kind {f.get('kind')!r}; have {FFN_KINDS}")
    return NinelixSpec(int(c["width"]), int(c["vocab"]), float(c["norm"]["eps"]), float(c.get("logit_scale", 1.0)),
                       int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"]), list(c["layers"]))


def _build_mixer(kind: str, m: dict, width: int, eps: float):
    if kind == "wkv":
        return WkvMixer(width, int(m["heads"]), int(m["dim"]), eps)
    if kind == "lightning":
        return LightningMixer(width, int(m["heads"]), int(m["dim"]), int(m["vdim"]), m["decay"], eps)
    a, s = m["left"], m["right"]
    qt = a.get("q_temp") or {"coef": 0.0, "every": 1}
    left = BiasedAttention(width, int(a["heads"]), int(a["kv_heads"]), int(a["dim"]), int(a["vdim"]), int(a["conv"]),
                           float(a["scale"]), float(qt["coef"]), int(qt["every"]), int(a["bias_max"]), eps)
    right = SsdMixer(width, int(s["heads"]), int(s["vdim"]), int(s["state"]), int(s["groups"]), int(s["norm_groups"]),
                     int(s["conv"]), eps)
    return ParallelPair(left, right)


class NinelixLayer:
    __slots__ = ("kind", "mixer", "ffn", "norm1", "norm2")


class NinelixLM(nn.Module):
    """The decoder core the engine drives (same surface as DecoderLM: forward / forward_hidden / logits / make_cache)."""

    needs_state = True     # the runner gives every sequence a state slot, and neither shares nor evicts its pages

    def __init__(self, spec: NinelixSpec, process_group, device, dtype):
        super().__init__()
        self.spec = spec
        self.comm = comm_for(process_group, device)
        self.tp, self.rank = self.comm.size, self.comm.rank
        if self.tp != 1:
            raise NotImplementedError("ninelix runs unsharded: start it with one rank")
        self.device, self.dtype = torch.device(device), dtype
        self.vocab_blk = spec.vocab
        self.layers: List[NinelixLayer] = []
        for lc in spec.layers:
            L = NinelixLayer()
            L.kind = lc["type"]
            L.mixer = _build_mixer(lc["type"], lc["mixer"], spec.hidden, spec.eps)
            f = lc.get("mlp")
            if f is None:
                L.ffn = None
            elif f["kind"] == "dense":
                L.ffn = DenseFFN()
            else:
                r = f["router"]
                L.ffn = RoutedExperts(int(r["experts"]), int(r["top"]), 1, 1, 1.0, int(f["expert"]["ff"]), act=ACT_SILU, gated=True)
            L.norm1 = L.norm2 = None
            self.layers.append(L)
        self.wte = self.bigram = self.w_head = self.final_w = None

    # ------------------------------------------------------------------ cache
    def default_block_size(self) -> int:
        return 64 if self.device.type == "cuda" else 16

    def make_cache(self, num_blocks: int, block_size: int, max_seqs: Optional[int] = None) -> HybridCache:
        kv, states = {}, {("embed", "prev_token"): ((), torch.int32)}
        for i, L in enumerate(self.layers):
            shape = L.mixer.kv_shape()
            if shape is not None:
                kv[i] = shape
            for name, sd in L.mixer.state_shapes().items():
                states[(i, name)] = sd
        return HybridCache(kv, states, num_blocks, block_size, max_seqs or 1, self.dtype, self.device)

    def num_parameters_local(self) -> int:
        ts = [self.wte, self.bigram, self.w_head, self.final_w]
        for L in self.layers:
            ts += [L.norm1, L.norm2] + L.mixer.weights()
            if L.ffn is not None:
                ts += [L.ffn.w_up, L.ffn.w_down] + ([L.ffn.w_router] if isinstance(L.ffn, RoutedExperts) else [])
        return sum(t.numel() for t in ts if t is not None)

    def finalize(self):
        for L in self.layers:
            if isinstance(L.mixer, ParallelPair):
                L.mixer.finalize()
        return self

    # ------------------------------------------------------------------ forward
    def forward_hidden(self, batch: BatchInput, kv: HybridCache, taps: Optional[list] = None) -> torch.Tensor:
        """Final-normed hidden states [T, width] of every packed token.  ``taps``: a list that receives the 32-bit
        residual stream after every layer (debugging / tests)."""
        s, dt = self.spec, self.dtype
        assert batch.state_slots is not None, "ninelix: the batch names no state slots"
        with trace("embed"):
            x = ops.embed_bigram(batch.tokens, self.wte, self.bigram, s.mul_prev, s.mul_cur, s.buckets, batch,
                                 kv.state("embed", "prev_token"))
        h = x if dt == torch.float32 else x.to(dt)
        for i, L in enumerate(self.layers):
            lc = LayerCacheView(kv, i)
            if isinstance(L.mixer, ParallelPair):
                a, b = L.mixer.forward_pair(x, h, batch, lc, dt)
                with trace("postnorm_residual"):
                    h, x = ops.postnorm_residual(a, L.norm1, s.eps, resid=x, y2=b, w_a=L.mixer.w_left, w_b=L.mixer.w_right,
                                                 out_dtype=dt)
            else:
                y = L.mixer.forward(x, h, batch, lc, dt)
                with trace("postnorm_residual"):
                    h, x = ops.postnorm_residual(y, L.norm1, s.eps, resid=x, out_dtype=dt)
            if L.ffn is not None:
                y = L.ffn.forward(h)
                with trace("postnorm_residual"):
                    h, x = ops.postnorm_residual(y, L.norm2, s.eps, resid=x, out_dtype=dt)
            if taps is not None:
                taps.append(x.clone())
        with trace("final_norm"):
            return ops.postnorm_residual(x, self.final_w, s.eps, out_dtype=dt)[0]

    def logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        with trace("lm_head"):
            z = ops.linear(hidden_rows, self.w_head, out_dtype=torch.float32)
            return z.mul_(self.spec.logit_scale) if self.spec.logit_scale != 1.0 else z

    local_logits = logits

    def forward(self, batch: BatchInput, kv, last_only: bool = True, gather_logits: bool = True) -> torch.Tensor:
        h = self.forward_hidden(batch, kv)
        if last_only:
            h = h.index_select(0, batch.last_idx)
        return self.logits(h)


# ---------------------------------------------------------------------------------------------------- weights
def _f32(t):
    """Small per-channel parameters are kept in 32-bit whatever the compute type (the checkpoint's values are exact in it)."""
    return t.float().contiguous()


def _load_wkv(mx: WkvMixer, get, p):
    """<p>.mu.{r,k,v,g,w} [W]; <p>.{r,k,v,g} [heads*dim, W]; <p>.w1 [lora, W]; <p>.w2 [heads*dim, lora]; <p>.w0 [heads*dim];
    <p>.u [heads, dim]; <p>.norm [heads*dim]; <p>.o [W, heads*dim]."""
    mx.mu = _f32(torch.stack([get(f"{p}.mu.{s}") for s in "rkvgw"]))
    mx.w_r, mx.w_k, mx.w_v, mx.w_g = (get(f"{p}.{s}").contiguous() for s in "rkvg")
    mx.w_w1, mx.w_w2, mx.w0 = get(f"{p}.w1").contiguous(), get(f"{p}.w2").contiguous(), get(f"{p}.w0")
    mx.u, mx.norm_w, mx.w_o = _f32(get(f"{p}.u")), _f32(get(f"{p}.norm")), get(f"{p}.o").contiguous()


def _load_lightning(mx: LightningMixer, get, p):
    """<p>.{q,k} [heads*dim, W]; <p>.{v,g} [heads*vdim, W]; <p>.norm [heads*vdim]; <p>.o [W, heads*vdim]."""
    mx.set_weights(get(f"{p}.q"), get(f"{p}.k"), get(f"{p}.v"), get(f"{p}.g"), _f32(get(f"{p}.norm")), get(f"{p}.o"))


def _load_parallel(mx: ParallelPair, get, p):
    """left: <p>.left.{q,k,v} + .b + .conv [channels, taps]; .q.norm / .k.norm [dim]; .rel [buckets, heads]; .g [heads, W];
    .o [W, heads*vdim].  right: <p>.right.in; .conv [channels, taps] + .conv.b; .dt_bias / .A_log / .D [heads]; .norm
    [inner]; .o [W, inner].  <p>.left.out / <p>.right.out [W]."""
    a, b = mx.left, mx.right
    lp, rp = f"{p}.left", f"{p}.right"
    a.set_weights(get(f"{lp}.q"), get(f"{lp}.q.b"), get(f"{lp}.k"), get(f"{lp}.k.b"), get(f"{lp}.v"), get(f"{lp}.v.b"),
                  _f32(get(f"{lp}.q.conv")), _f32(get(f"{lp}.k.conv")), _f32(get(f"{lp}.v.conv")), _f32(get(f"{lp}.q.norm")),
                  _f32(get(f"{lp}.k.norm")), get(f"{lp}.rel"), get(f"{lp}.g"), get(f"{lp}.o"))
    b.w_rows, b.conv_w, b.conv_b = get(f"{rp}.in"), _f32(get(f"{rp}.conv")), _f32(get(f"{rp}.conv.b"))
    b.dt_bias, b.a_log, b.d = _f32(get(f"{rp}.dt_bias")), _f32(get(f"{rp}.A_log")), _f32(get(f"{rp}.D"))
    b.norm_w, b.w_o = _f32(get(f"{rp}.norm")), get(f"{rp}.o").contiguous()
    mx.w_left, mx.w_right = _f32(get(f"{lp}.out")), _f32(get(f"{rp}.out"))


_LOADERS = {"wkv": _load_wkv, "lightning": _load_lightning, "parallel": _load_parallel}


def load_ninelix(m: NinelixLM, w):
    get = w.get_tensor
    m.wte, m.bigram, m.w_head, m.final_w = get("embed"), get("bigram"), get("head").contiguous(), _f32(get("final.norm"))
    for i, L in enumerate(m.layers):
        p = f"l{i}"
        L.norm1 = _f32(get(f"{p}.norm1"))
        _LOADERS[L.kind](L.mixer, get, f"{p}.mix")
        if L.ffn is None:
            continue
        L.norm2 = _f32(get(f"{p}.norm2"))
        if isinstance(L.ffn, DenseFFN):
            L.ffn.w_up, L.ffn.w_down = get(f"{p}.mlp.up").contiguous(), get(f"{p}.mlp.down").contiguous()
        else:
            ff, E = L.ffn, L.ffn.experts
            ff.w_router = get(f"{p}.mlp.router").contiguous()
            # gate and up rows interleaved (gate_0, up_0, gate_1, ...): the layout of the GEMM's gated epilogue
            ff.w_up = torch.stack([torch.stack([get(f"{p}.mlp.e{e}.gate"), get(f"{p}.mlp.e{e}.up")], dim=1).flatten(0, 1)
                                   for e in range(E)]).contiguous()                                        # [E, 2 F, W]
            ff.w_down = torch.cat([get(f"{p}.mlp.e{e}.down") for e in range(E)], dim=1).contiguous()         # [W, E * F]
