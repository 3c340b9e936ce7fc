"""Bedovik: a decoder-only design of parallel blocks over a 32-bit residual stream.

    x  = embed[token] + pos[position]                       (32-bit from here on; x0 = this embedding output)
    layer:  h = DyT(x);  x <- x + ls1 * mixer(h) + ls2 * ffn(h)      one norm feeds both branches
    mixer:  latent attention (optionally with a per-head sigmoid output gate)      -> models/blocks.LatentAttention
    ffn:    routed experts, squared-ReLU, group-limited top-k, or none             -> models/blocks.RoutedExperts
    loop:   layers [start, stop) run `times` times with shared weights; before each pass
            x <- W_in [x ; x0] + step[pass]      (re-injection of the embedding; every pass has its own cache plane)
    logits = head DyT_final(x)

config.json keys: architecture, vocab, width, max_positions, norm.eps, layers[i].{type, mixer{heads, dim, vdim,
kv_rank, scale}, mlp{kind, expert.ff, router{experts, top, scale, groups{count, keep}}} | null},
loop{start, stop, times} (optional).  Tensor names: embed, pos, loop.in, loop.step, head, final.norm{,.b,.alpha},
l<i>.norm1{,.b,.alpha}, l<i>.ls1, l<i>.ls2, l<i>.mix.{q, dkv, dkv.norm, uk, uv, g, o}, l<i>.mlp.router,
l<i>.mlp.e<j>.{up, down}.

The model is a graph over the framework's ops; the engine's runner, paged block allocator (a LatentCache with one
plane per layer run), batching and sampler drive it like the multi-head families.  It runs unsharded (TP = 1).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
from torch import nn

from .. import ops
from ..engine.batch import BatchInput
from ..engine.kv_cache import LatentCache
from ..parallel.comm import comm_for
from ..utils.tracing import trace
from .blocks import LatentAttention, RoutedExperts

_MIXERS = {"latent_attention": True, "latent_attention_2": False}    # type -> has the output gate


@dataclass
class MixerSpec:
    kind: str
    heads: int
    dim: int
    vdim: int
    rank: int
    scale: float

    @property
    def gated(self) -> bool:
        return _MIXERS[self.kind]


@dataclass
class ExpertsSpec:
    experts: int
    top: int
    groups: int
    keep: int
    route_scale: float
    ff: int


@dataclass
class BedovikSpec:
    hidden: int
    vocab: int
    max_pos: int
    eps: float
    mixers: List[MixerSpec]
    ffns: List[Optional[ExpertsSpec]]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0          # 0: no loop (and no re-injection)
    model_type: str = "bedovik"
    learned_pos: bool = True     # absolute position table: no sliding window past max_pos

    @property
    def n_weight_layers(self) -> int:
        return len(self.mixers)

    def schedule(self):
        """[(layer index, pass number if the run opens a loop pass else None)] in execution order."""
        n = self.n_weight_layers
        if not self.loop_times:
            return [(i, None) for i in range(n)]
        runs = [(i, None) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            runs += [(i, t if i == self.loop_start else None) for i in range(self.loop_start, self.loop_stop)]
        return runs + [(i, None) for i in range(self.loop_stop, n)]

    @property
    def n_layers(self) -> int:    # layer runs = cache planes
        return len(self.schedule())


def bedovik_spec(config) -> BedovikSpec:
    c = config.raw if hasattr(config, "raw") else dict(config)
    mixers, ffns = [], []
    for i, lc in enumerate(c["layers"]):
        if lc["type"] not in _MIXERS:
            raise ValueError(f"bedovik: layer {i} has unknown mixer type {lc['type']!r}; have {sorted(_MIXERS)}")
        m = lc["mixer"]
        mixers.append(MixerSpec(lc["type"], int(m["heads"]), int(m["dim"]), int(m["vdim"]), int(m["kv_rank"]),
                                float(m.get("scale", int(m["dim"]) ** -0.5))))
        f = lc.get("mlp")
        if f is None:
            ffns.append(None)
            continue
        if f.get("kind", "moe") != "moe":
            raise ValueError(f"bedovik: layer {i} has unknown feed-forward kind {f.get('kind')!r}")
        r = f["router"]
        g = r.get("groups") or {"count": 1, "keep": 1}
        ffns.append(ExpertsSpec(int(r["experts"]), int(r["top"]), int(g["count"]), int(g["keep"]), float(r.get("scale", 1.0)),
                                int(f["expert"]["ff"])))
    lp = c.get("loop")
    spec = BedovikSpec(int(c["width"]), int(c["vocab"]), int(c["max_positions"]), float(c["norm"]["eps"]), mixers, ffns)
    if lp:
        spec.loop_start, spec.loop_stop, spec.loop_times = int(lp["start"]), int(lp["stop"]), int(lp["times"])
        if not (0 <= spec.loop_start < spec.loop_stop <= len(mixers)) or spec.loop_times < 1:
            raise ValueError(f"bedovik: bad loop {lp}")
    return spec


class BedovikLayer:
    __slots__ = ("alpha", "norm_w", "norm_b", "ls1", "ls2", "mixer", "ffn", "w_in")


class BedovikLM(nn.Module):
    """The decoder core the engine drives (same surface as DecoderLM: forward / forward_hidden / logits / make_cache)."""

    def __init__(self, spec: BedovikSpec, process_group, device, dtype):
        super().__init__()
        self.spec = spec
        self.comm = comm_for(process_group, device)
        self.tp, self.rank = self.comm.size, self.comm.rank
        if self.tp != 1:
            raise NotImplementedError("bedovik runs unsharded: start it with one rank")
        self.device, self.dtype = torch.device(device), dtype
        self.runs = spec.schedule()
        self.vocab_blk = spec.vocab
        self.layers: List[BedovikLayer] = []
        self.wte = self.wpe = self.w_loop_in = self.loop_step = self.w_head = None
        self.final_alpha, self.final_w, self.final_b = 1.0, None, None

    # ------------------------------------------------------------------ cache
    def default_block_size(self) -> int:
        return 64 if self.device.type == "cuda" else 16

    def make_cache(self, num_blocks: int, block_size: int, max_seqs=None) -> LatentCache:
        return LatentCache([self.spec.mixers[i].rank for i, _ in self.runs], num_blocks, block_size, self.dtype, self.device)

    def num_parameters_local(self) -> int:
        n = sum(t.numel() for t in (self.wte, self.wpe, self.w_loop_in, self.loop_step, self.w_head, self.final_w, self.final_b)
                if t is not None)
        for L in self.layers:
            ts = [L.norm_w, L.norm_b, L.ls1, L.ls2, L.w_in, L.mixer.norm_w, L.mixer.w_uk, L.mixer.w_uv, L.mixer.w_o]
            if L.ffn is not None:
                ts += [L.ffn.w_up, L.ffn.w_down]
            n += sum(t.numel() for t in ts if t is not None)
        return n

    def finalize(self):
        """Stack the rows of everything that reads the normed input into one projection per layer."""
        for L in self.layers:
            blocks = [L.mixer] + ([L.ffn] if L.ffn is not None else [])
            L.w_in = torch.cat([b.in_rows() for b in blocks], dim=0).contiguous()
            col = 0
            for b in blocks:
                col = b.bind(col)
            assert col == L.w_in.shape[0]
        return self

    # ------------------------------------------------------------------ forward
    def forward_hidden(self, batch: BatchInput, kv: LatentCache, taps: Optional[list] = None) -> torch.Tensor:
        """Final-normed hidden states [T, width] of every packed token.  ``taps``: a list that receives the 32-bit
        residual stream after every layer run (debugging / tests)."""
        s, dt = self.spec, self.dtype
        x = ops.embed(batch.tokens, self.wte, batch.positions, self.wpe, 0, out_dtype=torch.float32)
        x0 = x
        pend = (None, None, None, None)     # branch outputs of the previous layer, folded in by the next kernel
        for run, (li, opens_pass) in enumerate(self.runs):
            L = self.layers[li]
            if opens_pass is not None:
                if pend[0] is not None:
                    _, x = ops.dyt_residual(x, 1.0, L.norm_w, None, *pend, out_dtype=dt, want_norm=False)
                    pend = (None, None, None, None)
                with trace("loop_reinject"):
                    x = ops.linear(ops.cast_concat(x, x0, dt), self.w_loop_in, self.loop_step[opens_pass], out_dtype=torch.float32)
            with trace("dyt_residual"):
                h, x = ops.dyt_residual(x, L.alpha, L.norm_w, L.norm_b, *pend, out_dtype=dt)
            with trace("gemm_in"):
                y = ops.linear(h, L.w_in, out_dtype=torch.float32)
            a = L.mixer.forward(y, batch, kv.latent(run), dt)
            m = L.ffn.forward(h, y) if L.ffn is not None else None
            pend = (a, L.ls1, m, L.ls2)
            if taps is not None:
                taps.append(ops.dyt_residual(x, 1.0, L.norm_w, None, *pend, out_dtype=dt, want_norm=False)[1].clone())
        h, _ = ops.dyt_residual(x, self.final_alpha, self.final_w, self.final_b, *pend, out_dtype=dt)
        return h

    def logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        with trace("lm_head"):
            return ops.linear(hidden_rows, self.w_head, out_dtype=torch.float32)

    local_logits = logits

    def forward(self, batch: BatchInput, kv, last_only: bool = True, gather_logits: bool = True) -> torch.Tensor:
        h = self.forward_hidden(batch, kv)
        if last_only:
            h = h.index_select(0, batch.last_idx)
        return self.logits(h)


def load_bedovik(m: BedovikLM, w):
    s = m.spec
    get = w.get_tensor
    m.wte, m.wpe, m.w_head = get("embed"), get("pos"), get("head")
    if s.loop_times:
        m.w_loop_in, m.loop_step = get("loop.in").contiguous(), get("loop.step").contiguous()
    m.final_alpha, m.final_w, m.final_b = float(get("final.norm.alpha").float()), get("final.norm"), get("final.norm.b")
    for i, (ms, fs) in enumerate(zip(s.mixers, s.ffns)):
        p, L = f"l{i}", BedovikLayer()
        L.alpha, L.norm_w, L.norm_b = float(get(f"{p}.norm1.alpha").float()), get(f"{p}.norm1"), get(f"{p}.norm1.b")
        L.ls1 = get(f"{p}.ls1")
        L.ls2 = get(f"{p}.ls2") if fs is not None else None
        mx = LatentAttention(ms.heads, ms.dim, ms.vdim, ms.rank, ms.scale, ms.gated, s.eps)
        mx.w_q, mx.w_dkv, mx.norm_w = get(f"{p}.mix.q"), get(f"{p}.mix.dkv"), get(f"{p}.mix.dkv.norm")
        mx.w_uk, mx.w_uv, mx.w_o = get(f"{p}.mix.uk").contiguous(), get(f"{p}.mix.uv").contiguous(), get(f"{p}.mix.o").contiguous()
        if ms.gated:
            mx.w_g = get(f"{p}.mix.g")
        L.mixer, L.ffn, L.w_in = mx, None, None
        if fs is not None:
            ff = RoutedExperts(fs.experts, fs.top, fs.groups, fs.keep, fs.route_scale, fs.ff)
            ff.w_router = get(f"{p}.mlp.router")
            ff.w_up = torch.stack([get(f"{p}.mlp.e{e}.up") for e in range(fs.experts)]).contiguous()          # [E, F, W]
            ff.w_down = torch.cat([get(f"{p}.mlp.e{e}.down") for e in range(fs.experts)], dim=1).contiguous()  # [W, E * F]
            L.ffn = ff
        m.layers.append(L)
