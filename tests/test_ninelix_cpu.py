"""Ninelix through the engine (CPU: the 32-bit PyTorch ops) against the plain float64 oracle in ninelix_oracle.py.

Own small configurations and random weights; the same cases run on CUDA in test_gpu_ninelix.py.
"""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch
from safetensors.torch import load_file, save_file

import ninelix_oracle as oracle
from llmss_b200 import ops
from llmss_b200.engine.batch import BatchInput
from llmss_b200.engine.engine import Engine
from llmss_b200.engine.runner import SamplingParams
from llmss_b200.utils.checkpoint import ninelix_config, write_random_checkpoint

ROOT = Path(__file__).resolve().parents[1]
TOL = 2e-4


def attn(heads=3, kv_heads=1, dim=10, vdim=6, conv=3, bias_max=24, buckets=8, scale=None, q_temp=None):
    d = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, bias_max=bias_max, buckets=buckets)
    if scale is not None:
        d["scale"] = scale
    if q_temp is not None:
        d["q_temp"] = q_temp
    return d


def ssd(heads=4, vdim=6, state=10, groups=2, norm_groups=2, conv=4):
    return dict(heads=heads, vdim=vdim, state=state, groups=groups, norm_groups=norm_groups, conv=conv)


DENSE, MOE = {"kind": "dense", "ff": 40}, {"kind": "moe", "experts": 5, "top": 2, "ff": 12}
CONFIGS = {
    # one layer of each kind, to see each mechanism alone
    "wkv": ninelix_config(32, 61, [{"type": "wkv", "heads": 3, "dim": 10, "lora": 5, "mlp": None}], buckets=17),
    "lightning": ninelix_config(32, 61, [{"type": "lightning", "heads": 3, "dim": 10, "vdim": 14, "mlp": None}], buckets=17),
    "parallel": ninelix_config(32, 61, [{"type": "parallel", "left": attn(), "right": ssd(), "mlp": None}], buckets=17),
    "dense": ninelix_config(32, 61, [{"type": "lightning", "heads": 1, "dim": 8, "vdim": 8, "mlp": DENSE}], buckets=17),
    "moe": ninelix_config(32, 61, [{"type": "lightning", "heads": 1, "dim": 8, "vdim": 8, "mlp": MOE}], buckets=17),
    # all kinds in an order of their own, sizes that are neither equal nor powers of two
    "mixed": ninelix_config(48, 97, [
        {"type": "wkv", "heads": 2, "dim": 12, "lora": 6, "mlp": MOE},
        {"type": "parallel", "left": attn(heads=4, kv_heads=2, dim=12, vdim=8, conv=3, bias_max=30, buckets=10),
         "right": ssd(heads=6, vdim=4, state=14, groups=3, norm_groups=2, conv=4), "mlp": DENSE},
        {"type": "lightning", "heads": 3, "dim": 8, "vdim": 12, "mlp": None},
        {"type": "parallel", "left": attn(heads=2, kv_heads=2, dim=16, vdim=16, conv=2, bias_max=9, buckets=6,
                                          q_temp={"coef": 0.5, "every": 7}),
         "right": ssd(heads=2, vdim=10, state=6, groups=1, norm_groups=1, conv=2), "mlp": MOE}],
        buckets=23, mul_prev=5, mul_cur=3, logit_scale=0.7),
    # values that are often 1 or equal: one head, one key/value head, every query head its own, one tap, top = 1 and
    # top = all experts, groups = heads, one norm group per channel pair, temperature step of one position
    "edges": ninelix_config(40, 53, [
        {"type": "parallel", "left": attn(heads=1, kv_heads=1, dim=20, vdim=4, conv=1, bias_max=5, buckets=4,
                                          q_temp={"coef": 0.2, "every": 1}),
         "right": ssd(heads=3, vdim=8, state=5, groups=3, norm_groups=12, conv=1),
         "mlp": {"kind": "moe", "experts": 3, "top": 1, "ff": 16}},
        {"type": "wkv", "heads": 1, "dim": 24, "lora": 3, "mlp": {"kind": "moe", "experts": 2, "top": 2, "ff": 8}},
        {"type": "parallel", "left": attn(heads=5, kv_heads=5, dim=6, vdim=10, conv=4, bias_max=64, buckets=16),
         "right": ssd(heads=1, vdim=12, state=20, groups=1, norm_groups=3, conv=5), "mlp": None},
        {"type": "lightning", "heads": 5, "dim": 4, "vdim": 4, "decay": [1.0, 0.5, 0.9, 0.99, 0.25], "mlp": DENSE}],
        buckets=1, mul_prev=1, mul_cur=1),
}


def write_ckpt(tmp_path, cfg, seed=0, tweak=None):
    path = write_random_checkpoint(Path(tmp_path) / f"ckpt{seed}", cfg, dtype=torch.bfloat16, device="cpu", seed=seed)
    if tweak is not None:
        for f in sorted(path.glob("*.safetensors")):
            t = load_file(str(f))
            tweak(t)
            save_file({k: v.contiguous() for k, v in t.items()}, str(f), metadata={"format": "pt"})
    return path


def decisive_router(t):
    """16-bit runs: router logits spread out, so that rounding seldom changes which experts are chosen (a changed choice
    moves the position by a whole expert's output, and every later one through the recurrent states)."""
    for k in list(t):
        if k.endswith(".mlp.router"):
            t[k] = (t[k].float() * 6.0).to(t[k].dtype)


def build(tmp_path, name, device="cpu", dtype=torch.float32, seed=0, tweak=None, **kw):
    cfg = CONFIGS[name] if isinstance(name, str) else name
    tweaks = [f for f in (tweak, decisive_router if dtype != torch.float32 else None) if f is not None]
    path = write_ckpt(tmp_path, cfg, seed, (lambda t: [f(t) for f in tweaks]) if tweaks else None)
    kw.setdefault("max_batch", 4)
    kw.setdefault("max_seq_len", 512)
    eng = Engine.from_pretrained(str(path), dtype=dtype, device=torch.device(device), use_cuda_graph=kw.pop("graph", False), **kw)
    return json.loads((path / "config.json").read_text()), oracle.load_weights(path), eng


def tokens_for(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def close(got, want, tol, rows_over=0.0):
    """Largest difference per row relative to the spread of the expected values.  ``rows_over``: share of rows that may
    exceed ``tol`` (a 16-bit run flips a routing decision now and then where two router logits nearly tie, which moves that
    position by a whole expert's output); the 32-bit runs allow none."""
    got, want = got.double().cpu(), want.double().cpu()
    spread = max(want.std().item(), 1e-6)
    d = (got - want).abs().reshape(got.shape[0], -1).max(-1).values / spread
    ok = d < tol
    over = (~ok).sum().item()
    rms = ((got - want)[ok].pow(2).mean().sqrt().item() / spread) if ok.any() else 0.0
    assert over <= rows_over * d.numel() and rms < tol / 3, \
        f"relative error max {d.max().item():.3g} rms {rms:.3g}, {over} of {d.numel()} rows over {tol}"


def flips(dtype):
    """Share of rows a 16-bit run may have over the tolerance: a router choice that rounding flips moves its position by a whole
    expert's output and, through the recurrent states, every later position of that request.  32-bit runs allow none."""
    return 0.0 if dtype == torch.float32 else 0.15


def feed_in_portions(eng, key, toks, sizes):
    """Feed ``toks`` cut into ``sizes`` (the last size repeats); returns the logits of every position."""
    out, at, i = [], 0, 0
    while at < len(toks):
        n = min(sizes[min(i, len(sizes) - 1)], len(toks) - at)
        out.append(eng.feed([(key, toks[at:at + n], list(range(n)))], [key] if at + n == len(toks) else []))
        at, i = at + n, i + 1
    return torch.cat(out)


def fake_batch(lens, ctxs, slots, device="cpu", bs=16):
    tables = [[1 + i * 8 + j for j in range(8)] for i in range(len(lens))]
    return BatchInput.build([[0] * n for n in lens], ctxs, tables, bs, device, state_slots=slots)


# ----------------------------------------------------------------------------- mechanisms alone (ops)
@pytest.mark.parametrize("taps", [1, 2, 3, 4, 6])
def test_causal_conv_op(taps, device="cpu"):
    """Convolution over portions of 1, 2 and more rows with the tail carried in the state, two sequences in a batch."""
    torch.manual_seed(taps)
    C, n = 7, 23
    w, b = torch.randn(C, taps), torch.randn(C)
    seqs = [torch.randn(n, C), torch.randn(n - 5, C)]
    want = [oracle.silu(oracle.causal_conv(u.double(), w.double(), b.double())) for u in seqs]
    state = torch.full((3, max(taps - 1, 1), C), 7.0).to(device) if taps > 1 else None     # slots hold rubbish at the start
    got, at = [[], []], [0, 0]
    for sizes in ([1, 5], [2, 1], [1, 1], [6, 2], [3, 9], [10, 0]):
        live = [i for i in (0, 1) if sizes[i] > 0 and at[i] < len(seqs[i])]
        lens = [min(sizes[i], len(seqs[i]) - at[i]) for i in live]
        batch = fake_batch(lens, [at[i] for i in live], [2 - i for i in live], device)
        u = torch.cat([seqs[i][at[i]:at[i] + k] for i, k in zip(live, lens)])
        wide = torch.cat([torch.randn(u.shape[0], 2), u], dim=1).to(device)      # a column view of a wider projection
        y = ops.causal_conv(wide[:, 2:], w.to(device), b.to(device), ops.ACT_SILU, batch, state).cpu()
        o = 0
        for i, k in zip(live, lens):
            got[i].append(y[o:o + k])
            at[i] += k
            o += k
    for i in (0, 1):
        g = torch.cat(got[i])
        close(g, want[i][:g.shape[0]], 1e-5)
        assert g.shape[0] >= 17


def test_distance_table_follows_the_bucket_rule():
    for B, D in [(16, 120), (8, 24), (4, 5), (6, 9), (32, 512), (7, 33)]:
        rel = torch.randn(B, 3)
        tab = ops.distance_bias_table(rel, D)
        assert tab.shape == (3, D + 1)
        for n in range(D + 1):
            assert torch.equal(tab[:, n], rel[oracle.distance_bucket(n, B, D)])
        assert torch.equal(tab[:, D], rel[B - 1])


@pytest.mark.parametrize("E,top", [(8, 2), (5, 1), (3, 3), (64, 6)])
def test_router_is_softmax_over_the_chosen_logits(E, top, device="cpu"):
    torch.manual_seed(E)
    z = (2.0 * torch.randn(19, E)).to(device)
    ids, wts = ops.moe_route(z, E, top, 1, 1, 1.0)
    want_ids, want_w = oracle.route(z.double().cpu(), top)
    for t in range(z.shape[0]):
        got = dict(zip(ids[t].tolist(), wts[t].tolist()))
        assert sorted(got) == sorted(want_ids[t])
        for e, x in zip(want_ids[t], want_w[t]):
            assert abs(got[e] - float(x)) < 1e-5


def test_gated_experts_op(device="cpu", dtype=torch.float32, tol=1e-5):
    torch.manual_seed(5)
    T, W, F, E, top = 9, 24, 10, 4, 2
    h = torch.randn(T, W).to(dtype)
    gate, up, down = torch.randn(E, F, W).to(dtype) * 0.3, torch.randn(E, F, W).to(dtype) * 0.3, torch.randn(E, W, F).to(dtype) * 0.3
    ids = torch.stack([torch.randperm(E)[:top] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, top)
    w_up = torch.stack([gate, up], dim=2).flatten(1, 2).contiguous()          # rows (gate_0, up_0, gate_1, ...)
    w_down = torch.cat([down[e] for e in range(E)], dim=1).contiguous()
    got = ops.moe_experts(h.to(device), ids.to(device), wts.to(device), w_up.to(device), w_down.to(device), ops.ACT_SILU, True)
    want = torch.zeros(T, W, dtype=torch.float64)
    for t in range(T):
        for k in range(top):
            e = int(ids[t, k])
            a = oracle.silu(gate[e].double() @ h[t].double()) * (up[e].double() @ h[t].double())
            want[t] += wts[t, k].double() * (down[e].double() @ a)
    close(got, want, tol)


# ----------------------------------------------------------------------------- the model, whole prompts
def residual_stream(eng, toks):
    """The 32-bit residual stream after every layer for one whole prompt, through the core's own forward."""
    r = eng.runner
    n = -(-len(toks) // r.block_size)
    batch = BatchInput.build([toks], [0], [list(range(1, n + 1))], r.block_size, r.device, max_blocks=r.max_blocks_per_seq,
                             state_slots=[0])
    taps = []
    with torch.no_grad():
        eng.core.forward_hidden(batch, r.kv, taps)
    return taps


@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_and_residual_stream(tmp_path, name, device="cpu", dtype=torch.float32, tol=TOL):
    cfg, W, eng = build(tmp_path, name, device, dtype)
    toks = tokens_for(cfg, 45, 1)
    taps = []
    want = oracle.forward(toks, W, cfg, taps)
    for i, (g, w) in enumerate(zip(residual_stream(eng, toks), taps)):
        close(g, w, tol * (1 + i), rows_over=flips(dtype))
    close(eng.feed([("a", toks, list(range(len(toks))))], ["a"]), want, tol * 2, rows_over=flips(dtype))


# ----------------------------------------------------------------------------- decoding, portions, batches
@pytest.mark.parametrize("name", ["mixed", "edges"])
def test_decode_token_by_token_and_portions(tmp_path, name, device="cpu", dtype=torch.float32, tol=TOL):
    """Prefill against token-by-token decoding, and portions down to two tokens that cut pages and convolution tails."""
    cfg, W, eng = build(tmp_path, name, device, dtype)
    toks = tokens_for(cfg, 70, 2)
    want = oracle.forward(toks, W, cfg)
    for sizes in ([1], [2], [3, 1, 2, 7, 1, 1, 16, 5], [15, 1, 1, 17, 2], [33, 31, 1], [64, 1]):
        close(feed_in_portions(eng, "s", toks, sizes), want, tol * 2, rows_over=flips(dtype))


def test_unequal_batches_against_each_alone(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    """Portions of some requests beside single tokens of others in one step; every request equals itself alone."""
    cfg, W, eng = build(tmp_path, "mixed", device, dtype)
    reqs = {k: tokens_for(cfg, n, 10 + i) for i, (k, n) in enumerate([("a", 61), ("b", 9), ("c", 33), ("d", 1), ("e", 20)])}
    want = {k: oracle.forward(t, W, cfg) for k, t in reqs.items()}
    plan = [[("a", 20), ("b", 1)], [("a", 1), ("b", 1), ("c", 17)], [("a", 2), ("c", 1), ("d", 1), ("b", 3)],
            [("a", 30), ("b", 1), ("c", 2), ("e", 5)], [("b", 3), ("c", 13), ("e", 1)], [("a", 8), ("e", 14)]]
    at, got = {k: 0 for k in reqs}, {k: [] for k in reqs}
    for step in plan:
        entries, end = [], []
        for k, n in step:
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
            at[k] += n
            if at[k] == len(reqs[k]):
                end.append(k)
        out = eng.feed(entries, end)
        o = 0
        for k, n in step:
            got[k].append(out[o:o + n])
            o += n
    for k in reqs:
        assert at[k] == len(reqs[k])
        close(torch.cat(got[k]), want[k], tol * 2, rows_over=flips(dtype))


def test_pages_and_slots_are_used_again(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    """Two state slots and a pool of a few pages serve six requests one after another and overlapping; what a slot or a
    page held before must not show.  A third live request, and a request beyond the pool, are errors."""
    cfg, W, eng = build(tmp_path, "mixed", device, dtype, max_batch=2)
    bs = eng.runner.block_size
    cfg2, W2, small = build(tmp_path / "p", "mixed", device, dtype, max_batch=2, pool_tokens=4 * bs)
    for e in (eng, small):
        lens = [bs + 3, 2 * bs, 5, bs - 1, bs + 1, 7]
        reqs = [tokens_for(cfg, n, 30 + i) for i, n in enumerate(lens)]
        want = [oracle.forward(t, W, cfg) for t in reqs]
        # r0 and r1 live together; r1 ends, r2 takes its slot and pages while r0 goes on; and so on
        a = e.feed([(0, reqs[0][:5], list(range(5))), (1, reqs[1], list(range(lens[1])))], [1])
        close(a[5:], want[1], tol * 2, rows_over=flips(dtype))
        b = e.feed([(0, reqs[0][5:], list(range(lens[0] - 5))), (2, reqs[2], list(range(5)))], [0, 2])
        close(torch.cat([a[:5], b[:lens[0] - 5]]), want[0], tol * 2, rows_over=flips(dtype))
        close(b[lens[0] - 5:], want[2], tol * 2, rows_over=flips(dtype))
        for i in (3, 4, 5):
            close(feed_in_portions(e, i, reqs[i], [4, 1]), want[i], tol * 2, rows_over=flips(dtype))
        assert e.runner.slots.num_free == 2 and e.runner.alloc.num_free == e.runner.alloc.num_blocks - 1
    eng.feed([("x", [1, 2], []), ("y", [3], [])])
    with pytest.raises(RuntimeError):
        eng.feed([("z", [4], [])])
    eng.feed([], ["x", "y"])
    with pytest.raises(MemoryError):
        small.feed([("big", tokens_for(cfg, 5 * bs, 1), [])])


def far_and_peaky(t):
    """Attention that is decided by single keys far back: a steep softmax, and a distance table that prefers the last
    buckets, so that a far key lost, a bucket edge moved by one or a page read wrongly changes the result at once."""
    for k in list(t):
        if k.endswith(".left.rel"):
            B = t[k].shape[0]
            t[k] = (t[k].float() + torch.linspace(-3.0, 4.0, B)[:, None]).to(t[k].dtype)


def test_far_keys_bucket_edges_and_page_borders(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    """bias_max and the half-way bucket lie inside the context; prompts, portions and decoded tokens ask across them and across
    page borders."""
    cfg = ninelix_config(32, 71, [
        {"type": "parallel", "left": attn(heads=2, kv_heads=1, dim=8, vdim=8, conv=2, bias_max=37, buckets=10, scale=3.0 * 8 ** -0.5),
         "right": ssd(heads=2, vdim=4, state=4, groups=1, norm_groups=1, conv=2), "mlp": None},
        {"type": "parallel", "left": attn(heads=4, kv_heads=4, dim=8, vdim=4, conv=3, bias_max=130, buckets=6, scale=3.0 * 8 ** -0.5,
                                          q_temp={"coef": 0.4, "every": 16}),
         "right": ssd(heads=2, vdim=4, state=4, groups=2, norm_groups=2, conv=3), "mlp": None}], buckets=13)
    cfg, W, eng = build(tmp_path, cfg, device, dtype, tweak=far_and_peaky)
    toks = tokens_for(cfg, 150, 4)
    want = oracle.forward(toks, W, cfg)
    close(feed_in_portions(eng, "w", toks, [150]), want, tol * 3)
    close(feed_in_portions(eng, "p", toks, [31, 2, 36, 1, 1, 59, 2, 1]), want, tol * 3)
    close(feed_in_portions(eng, "d", toks, [100, 1]), want, tol * 3)
    # the far keys decide: without the table's preference for far buckets the logits differ by far more than the tolerance
    W0 = dict(W)
    for k in W0:
        if k.endswith(".left.rel"):
            W0[k] = torch.zeros_like(W0[k])
    assert (oracle.forward(toks, W0, cfg) - want).abs().max() > want.std()


def test_first_tokens(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    """One-token and two-token requests, and the first tokens one by one: the bigram's start row, the convolutions'
    zeros before the start, the zero states -- in slots that another request has just left."""
    cfg, W, eng = build(tmp_path, "mixed", device, dtype)
    feed_in_portions(eng, "warm", tokens_for(cfg, 40, 7), [40])          # leaves states and pages behind
    for n in (1, 2, 3, 6):
        toks = tokens_for(cfg, n, 50 + n)
        want = oracle.forward(toks, W, cfg)
        close(feed_in_portions(eng, "f", toks, [n]), want, tol * 2, rows_over=flips(dtype))
        close(feed_in_portions(eng, "g", toks, [1]), want, tol * 2, rows_over=flips(dtype))


def test_long_decoding(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    cfg, W, eng = build(tmp_path, "mixed", device, dtype)
    toks = tokens_for(cfg, 160, 8)
    want = oracle.forward(toks, W, cfg)
    close(feed_in_portions(eng, "l", toks, [12, 1]), want, tol * 4, rows_over=flips(dtype))


# ----------------------------------------------------------------------------- generation through the public entry points
def oracle_greedy(W, cfg, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(oracle.forward(toks, W, cfg)[-1].argmax()))
    return toks[len(prompt):]


def test_greedy_generation_through_engine_and_cli(tmp_path, device="cpu", dtype=torch.float32, graph=False):
    """Engine.generate: admission of more requests than slots, packed prefill, decode steps, the sampler; then generate.py."""
    cfg, W, eng = build(tmp_path, "mixed", device, dtype, max_batch=2, graph=graph)
    prompts = [tokens_for(cfg, n, 60 + n) for n in (9, 1, 14)]
    got = eng.generate(prompts, SamplingParams(max_new_tokens=7, is_greedy=True))
    if dtype == torch.float32:
        assert got == [oracle_greedy(W, cfg, p, 7) for p in prompts]
    else:   # 16-bit: teacher-forced, every chosen token is the oracle's best or within rounding of it
        for p, g in zip(prompts, got):
            lg = oracle.forward(p + g, W, cfg)[len(p) - 1:-1]
            for row, tok in zip(lg, g):
                assert row[tok] >= row.max() - 0.15 * lg.std()
    assert eng.runner.slots.num_free == 2
    if device == "cpu":
        path = tmp_path / "ckpt0"
        r = subprocess.run([sys.executable, str(ROOT / "generate.py"), "--pretrained_model_path", str(path), "--prompt_ids",
                            " ".join(map(str, prompts[0])), "--max_new_tokens", "5", "--is_greedy", "--use_cache"],
                           capture_output=True, text=True, timeout=300, cwd=str(ROOT),
                           env={**__import__("os").environ, "CUDA_VISIBLE_DEVICES": ""})
        assert r.returncode == 0, r.stderr[-2000:]
        assert " ".join(map(str, got[0][:5])) in r.stdout.replace(",", " ").replace("  ", " "), r.stdout[-1000:]


def test_model_call_with_a_past(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    """The HF-shaped call: a prompt, then single tokens, with the cache object handed back."""
    from llmss_b200.models import MODEL_REGISTRY
    from llmss_b200.utils.config import load_config
    from llmss_b200.utils.dist import FakeGroup
    from llmss_b200.utils.hub import weight_files
    from llmss_b200.utils.weights import Weights

    path = write_ckpt(tmp_path, CONFIGS["mixed"], 0, decisive_router if dtype != torch.float32 else None)
    cfg, W = json.loads((path / "config.json").read_text()), oracle.load_weights(path)
    config = load_config(str(path))
    weights = Weights(weight_files(str(path)), device=torch.device(device), dtype=dtype, process_group=FakeGroup(0, 1))
    model = MODEL_REGISTRY[config.model_type](config, weights).eval()
    seqs = [tokens_for(cfg, 30, 3), tokens_for(cfg, 30, 4)]
    ids = torch.tensor(seqs)
    out = model(ids[:, :21], use_cache=True)
    rows = [out.logits]
    for t in range(21, 30):
        out = model(ids[:, t:t + 1], past_key_values=out.past_key_values, use_cache=True)
        rows.append(out.logits)
    got = torch.cat(rows, dim=1)
    for b in (0, 1):
        close(got[b], oracle.forward(seqs[b], W, cfg), tol * 2, rows_over=flips(dtype))


def test_unknown_kinds_are_refused(tmp_path):
    from llmss_b200.models.ninelix import ninelix_spec

    cfg = json.loads(json.dumps(CONFIGS["wkv"]))
    cfg["layers"][0]["type"] = "other"
    with pytest.raises(ValueError):
        ninelix_spec(cfg)
    cfg = json.loads(json.dumps(CONFIGS["dense"]))
    cfg["layers"][0]["mlp"]["kind"] = "other"
    with pytest.raises(ValueError):
        ninelix_spec(cfg)
