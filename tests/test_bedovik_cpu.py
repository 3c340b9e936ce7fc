"""Bedovik through the engine (CPU: fp32 ops) against the plain float64 oracle in bedovik_oracle.py.

Own small configurations and random weights; the same cases run on CUDA in test_gpu_bedovik.py.
"""

import pytest
import torch

import bedovik_oracle as oracle
from llmss_b200 import ops
from llmss_b200.engine.batch import BatchInput
from llmss_b200.engine.engine import Engine
from llmss_b200.engine.runner import SamplingParams
from llmss_b200.utils.checkpoint import bedovik_config, write_random_checkpoint


def L(gated, heads, dim, vdim, rank, experts=0, top=0, groups=1, keep=1, ff=0, route_scale=1.5, scale=None):
    d = dict(gated=gated, heads=heads, dim=dim, vdim=vdim, kv_rank=rank)
    if scale is not None:
        d["scale"] = scale
    if experts:
        d.update(experts=experts, top=top, groups=groups, keep=keep, ff=ff, route_scale=route_scale)
    return d


CONFIGS = {
    # loop in the middle, a layer without feed-forward, one head, top = 1, one group, sizes that are no powers of two
    "mid_loop": bedovik_config(64, 97, 160, [L(True, 3, 8, 12, 24, 8, 3, 4, 2, 16), L(False, 2, 16, 8, 40),
                                             L(True, 1, 8, 8, 16, 4, 1, 1, 1, 8, scale=0.5)], loop=(1, 3, 2)),
    # no loop at all; keep = every group; top = a whole group
    "no_loop": bedovik_config(48, 61, 96, [L(False, 4, 8, 8, 32, 6, 2, 3, 3, 12), L(True, 2, 12, 4, 20, 6, 3, 2, 1, 10)]),
    # the loop covers every layer and runs three times; and a loop of one pass (re-injection only)
    "all_loop": bedovik_config(32, 50, 96, [L(True, 2, 8, 8, 16, 4, 2, 2, 1, 8), L(False, 2, 8, 16, 24, 4, 2, 2, 2, 8)], loop=(0, 2, 3)),
    "one_pass": bedovik_config(32, 50, 96, [L(False, 2, 8, 8, 16, 4, 2, 1, 1, 8), L(True, 2, 8, 8, 16)], loop=(0, 1, 1)),
}


def build(tmp_path, name, device="cpu", dtype=torch.float32, seed=0, **kw):
    cfg = CONFIGS[name] if isinstance(name, str) else name
    path = write_random_checkpoint(tmp_path / f"ckpt{seed}", cfg, dtype=torch.bfloat16, device="cpu", seed=seed)
    kw.setdefault("max_batch", 4)
    eng = Engine.from_pretrained(str(path), dtype=dtype, device=torch.device(device), use_cuda_graph=kw.pop("graph", False), **kw)
    return cfg, oracle.load_weights(path), eng


def tokens_for(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def close(got, want, tol, rows_over=0.0):
    """Largest difference, and root mean square difference, relative to the spread of the expected values.  `rows_over`: share
    of rows that may exceed `tol`: a 16-bit run flips a routing decision now and then where two expert scores nearly tie,
    which moves that one position by a whole expert's output; those rows are then left out of the root mean square.  The true
    32-bit runs allow none, and the 16-bit kernels are held to `tol` on every row where no router is involved."""
    got, want = got.double().cpu(), want.double().cpu()
    spread = max(want.std().item(), 1e-6)
    d = (got - want).abs().reshape(got.shape[0], -1).max(-1).values / spread
    ok = d < tol
    over = (~ok).sum().item()
    rms = ((got - want)[ok].pow(2).mean().sqrt().item() / spread) if ok.any() else 0.0
    assert over <= rows_over * d.numel() and rms < tol / 4, \
        f"relative error max {d.max().item():.3g} rms {rms:.3g}, {over} of {d.numel()} rows over {tol}"


def feed_in_portions(eng, key, toks, sizes):
    """Feed `toks` cut into `sizes` (the last size repeats); returns the logits of every position."""
    out, at, i = [], 0, 0
    while at < len(toks):
        n = min(sizes[min(i, len(sizes) - 1)], len(toks) - at)
        out.append(eng.feed([(key, toks[at:at + n], list(range(n)))], [key] if at + n == len(toks) else []))
        at, i = at + n, i + 1
    return torch.cat(out)


TOL = 2e-4


# ----------------------------------------------------------------------------- mechanisms alone
def test_dyt_residual_op():
    torch.manual_seed(0)
    r, a, b = torch.randn(5, 24), torch.randn(5, 24), torch.randn(5, 24)
    w, bias, s1, s2 = torch.randn(24), torch.randn(24), torch.rand(24), torch.rand(24)
    y, r2 = ops.dyt_residual(r, 0.6, w, bias, a, s1, b, s2, out_dtype=torch.float32)
    want_r = r.double() + s1.double() * a.double() + s2.double() * b.double()
    close(r2, want_r, 1e-5)
    close(y, oracle.dyt(want_r, 0.6, w.double(), bias.double()), 1e-5)
    y, r3 = ops.dyt_residual(r, 1.3, w, None, a, None, None, None, out_dtype=torch.float32)
    close(r3, r.double() + a.double(), 1e-5)
    close(y, torch.tanh(1.3 * (r.double() + a.double())) * w.double(), 1e-5)


@pytest.mark.parametrize("E,top,groups,keep", [(8, 3, 4, 2), (6, 2, 3, 3), (6, 3, 2, 1), (4, 1, 1, 1), (12, 4, 3, 2), (5, 5, 1, 1),
                                               (64, 6, 8, 3), (96, 8, 4, 1)])
def test_router_op(E, top, groups, keep, device="cpu"):
    torch.manual_seed(E + top)
    z = (2.0 * torch.randn(33, E)).to(device)
    ids, wts = ops.moe_route(z, E, top, groups, keep, 2.5)
    for t in range(z.shape[0]):
        chosen, w = oracle.route(z[t].double().cpu(), top, groups, keep, 2.5)
        assert sorted(ids[t].tolist()) == sorted(chosen)
        got = dict(zip(ids[t].tolist(), wts[t].tolist()))
        for e, x in zip(chosen, w):
            assert abs(got[e] - float(x)) < 1e-5


def test_router_group_limit_is_applied():
    """The two largest scores sit in one group, the third largest in another: with keep = 1 the third must not be chosen."""
    z = torch.full((1, 8), -4.0)
    z[0, 0], z[0, 1], z[0, 6], z[0, 2] = 3.0, 2.0, 2.5, 0.5     # groups of 4: {0..3}, {4..7}
    ids, wts = ops.moe_route(z, 8, 3, 2, 1, 1.0)
    assert sorted(ids[0].tolist()) == [0, 1, 2]
    assert abs(wts.sum().item() - 1.0) < 1e-5
    ids, _ = ops.moe_route(z, 8, 3, 2, 2, 1.0)
    assert sorted(ids[0].tolist()) == [0, 1, 6]


def test_experts_op(device="cpu", dtype=torch.float32, tol=1e-5):
    torch.manual_seed(3)
    T, W, F, E, top = 7, 24, 10, 5, 2
    h = torch.randn(T, W).to(dtype)
    ups = [(torch.randn(F, W) * W ** -0.5).to(dtype) for _ in range(E)]
    downs = [(torch.randn(W, F) * F ** -0.5).to(dtype) for _ in range(E)]
    ids = torch.stack([torch.randperm(E)[:top] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, top)
    got = ops.moe_experts(h.to(device), ids.to(device), wts.to(device), torch.stack(ups).to(device),
                          torch.cat(downs, dim=1).contiguous().to(device), ops.ACT_RELU2)
    want = torch.stack([oracle.experts(h[t].double(), ids[t].tolist(), wts[t].double(), [u.double() for u in ups],
                                       [d.double() for d in downs]) for t in range(T)])
    close(got, want, tol)


def latent_pipeline(h, w, heads, d, dv, R, scale, eps, gated, chunks, block_size, device, dtype):
    """The product's op sequence for one sequence fed in `chunks`, over a paged cache whose pages are handed out in
    reverse order (so that a wrong page lookup shows)."""
    T, W = h.shape
    nblk = -(-T // block_size)
    cache = torch.zeros(nblk + 1, block_size, R, dtype=dtype, device=device)
    table = list(range(nblk, 0, -1))
    w_in = torch.cat([w["q"], w["dkv"]] + ([w["g"]] if gated else [])).to(device=device, dtype=dtype)
    outs, at = [], 0
    for n in chunks:
        batch = BatchInput.build([[0] * n], [at], [table], block_size, device)
        y = ops.linear(h[at:at + n].to(device=device, dtype=dtype), w_in, out_dtype=torch.float32)
        q, gate = ops.latent_prep(y, 0, heads * d, heads * d + R if gated else -1, heads * d, R, heads,
                                  w["norm"].to(device=device, dtype=dtype), eps, batch.slot_mapping, cache, dtype)
        qa = ops.heads_matmul(q, w["uk"].to(device=device, dtype=dtype), heads, d, R, True,
                              out_dtype=ops.latent_query_dtype(cache, heads, R))
        o = ops.latent_attention(qa, cache, batch, heads, R, scale, dtype)
        ctx = ops.heads_matmul(o, w["uv"].to(device=device, dtype=dtype), heads, R, dv, False, row_scale=gate, out_dtype=dtype)
        outs.append(ops.linear(ctx, w["o"].to(device=device, dtype=dtype), out_dtype=torch.float32))
        at += n
    return torch.cat(outs)


def latent_weights(W, heads, d, dv, R, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: (torch.randn(*s, generator=g) * s[-1] ** -0.5).to(dtype).float()
    return dict(q=r(heads * d, W), dkv=r(R, W), norm=1 + 0.1 * r(R), uk=r(heads * d, R), uv=r(heads * dv, R), g=r(heads, W),
                o=r(W, heads * dv))


@pytest.mark.parametrize("gated", [True, False])
@pytest.mark.parametrize("chunks", [[37], [1] * 37, [5, 2, 17, 1, 1, 9, 2], [16, 16, 5]])
def test_latent_attention_ops(gated, chunks, device="cpu", dtype=torch.float32, tol=1e-4, sizes=(40, 3, 8, 12, 24)):
    W, heads, d, dv, R = sizes
    T = sum(chunks)
    w = latent_weights(W, heads, d, dv, R, 5, dtype if dtype != torch.float32 else torch.float32)
    h = torch.randn(T, W, generator=torch.Generator().manual_seed(1)).to(dtype).float()
    got = latent_pipeline(h, w, heads, d, dv, R, 0.3, 1e-5, gated, chunks, 16, device, dtype)
    wd = {k: v.double() for k, v in w.items()}
    want = oracle.latent_attention(h.double(), wd["q"], wd["dkv"], wd["norm"], wd["uk"], wd["uv"], wd["o"],
                                   wd["g"] if gated else None, heads, d, dv, 0.3, 1e-5)
    close(got, want, tol)


@pytest.mark.parametrize("far", [0, 3, 15, 16, 31, 32, 63, 64, 200, 255, 256, 399])
@pytest.mark.parametrize("q_len", [1, 2, 9])
def test_one_key_stands_out(far, q_len, device="cpu", dtype=torch.float32, R=24, block_size=16, tol=1e-3, ctx=400):
    """Random latents in the cache; the query of the last token is a large multiple of ONE cached latent, so that key takes
    (almost) all of the softmax: the output must be that latent.  The key sits far back, on page borders, first in the
    sequence; the query is decoded alone or is the end of a portion.  A kernel that skips or misreads the key returns a blend
    of other latents instead."""
    far = min(far, ctx - 1)
    g = torch.Generator().manual_seed(far)
    lat = torch.randn(ctx, R, generator=g)
    lat = lat / lat.norm(dim=-1, keepdim=True)
    nblk = -(-ctx // block_size)
    table = torch.randperm(nblk, generator=g).add(1).tolist()
    cache = torch.zeros(nblk + 1, block_size, R, dtype=dtype)
    for p in range(ctx):
        cache[table[p // block_size], p % block_size] = lat[p].to(dtype)
    cache = cache.to(device)
    heads = 3
    batch = BatchInput.build([[0] * q_len], [ctx - q_len], [table], block_size, device)
    q = torch.zeros(q_len, heads, R)
    q[-1, :] = 60.0 * lat[far]                       # unit latents: score 60 for the chosen key, |score| < ~20 elsewhere
    q[-1, 1] = 60.0 * lat[(far * 7 + 5) % ctx]      # the middle head asks for another key
    qd = ops.latent_query_dtype(cache, heads, R)
    out = ops.latent_attention(q.reshape(q_len, heads * R).to(device=device, dtype=qd), cache, batch, heads, R, 1.0, dtype)
    out = out.float().cpu().view(q_len, heads, R)
    for hd, j in ((0, far), (1, (far * 7 + 5) % ctx), (2, far)):
        s = (lat @ lat[j]) * 60.0
        want = torch.softmax(s.double(), 0) @ lat.double()
        assert (out[-1, hd].double() - want).abs().max().item() < tol
        assert (out[-1, hd] - cache.float().cpu()[table[j // block_size], j % block_size]).abs().max().item() < 0.05


def test_window_edges_of_causality(device="cpu", dtype=torch.float32, tol=2e-3):
    """The only visibility rule is causal: token i of a portion must see key i and must not see key i + 1.  Make key i + 1
    the one that would win."""
    R, bs, ctx, n = 16, 16, 30, 5
    g = torch.Generator().manual_seed(9)
    lat = torch.randn(ctx + n, R, generator=g)
    lat = lat / lat.norm(dim=-1, keepdim=True)
    table = [2, 1, 3]
    cache = torch.zeros(4, bs, R, dtype=dtype)
    for p in range(ctx + n):
        cache[table[p // bs], p % bs] = lat[p].to(dtype)
    batch = BatchInput.build([[0] * n], [ctx], [table], bs, device)
    q = torch.stack([50.0 * lat[ctx + i + 1] if i + 1 < n else 50.0 * lat[ctx + i] for i in range(n)])   # asks for the NEXT key
    cache = cache.to(device)
    out = ops.latent_attention(q.to(device=device, dtype=ops.latent_query_dtype(cache, 1, R)), cache, batch, 1, R, 1.0, dtype)
    out = out.float().cpu()
    for i in range(n):
        vis = ctx + i + 1
        s = (lat[:vis] @ q[i].float())
        want = torch.softmax(s.double(), 0) @ lat[:vis].double()
        assert (out[i].double() - want).abs().max().item() < tol


# ----------------------------------------------------------------------------- the model through the engine
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt_and_residual_stream(tmp_path, name, device="cpu", dtype=torch.float32, tol=TOL):
    cfg, W, eng = build(tmp_path, name, device, dtype)
    toks = tokens_for(cfg, 41, 1)
    want, taps = oracle.forward(cfg, W, toks)
    got = eng.feed([("a", toks, list(range(len(toks))))], ["a"])
    close(got, want, tol)
    # residual stream after every layer run, straight from the model's step function
    core, r = eng.core, eng.runner
    blocks = r.alloc.alloc(r.blocks_needed(len(toks)))
    batch = BatchInput.build([toks], [0], [blocks], r.block_size, core.device, max_blocks=r.max_blocks_per_seq)
    mine = []
    core.forward_hidden(batch, r.kv, taps=mine)
    r.alloc.release(blocks)
    assert len(mine) == len(taps) == len(oracle.run_order(cfg))
    for a, b in zip(mine, taps):
        close(a, b, tol)


def test_decode_token_by_token_and_portions(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    cfg, W, eng = build(tmp_path, "mid_loop", device, dtype)
    toks = tokens_for(cfg, 70, 2)
    want, _ = oracle.forward(cfg, W, toks)
    close(feed_in_portions(eng, "one", toks, [1]), want, tol)                 # every token decoded alone, across pages
    close(feed_in_portions(eng, "dec", toks, [38, 1]), want, tol)            # a prompt, then decoding
    for sizes in ([2], [3, 2, 7, 2, 16, 5, 2, 2, 31], [17, 15, 2, 1, 1, 33], [64, 6]):
        close(feed_in_portions(eng, tuple(sizes), toks, sizes), want, tol)
    assert eng.runner.alloc.num_free == eng.runner.alloc.num_blocks - 1       # every page came back


def test_first_tokens(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    cfg, W, eng = build(tmp_path, "no_loop", device, dtype)
    for n in (1, 2, 3):
        toks = tokens_for(cfg, n, 10 + n)
        close(eng.feed([("f", toks, list(range(n)))], ["f"]), oracle.forward(cfg, W, toks)[0], tol)


def test_unequal_batch_equals_each_alone(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    cfg, W, eng = build(tmp_path, "mid_loop", device, dtype)
    reqs = {k: tokens_for(cfg, n, 20 + n) for k, n in (("a", 53), ("b", 1), ("c", 18), ("d", 34))}
    want = {k: oracle.forward(cfg, W, t)[0] for k, t in reqs.items()}
    # step 1: a portion of a, all of b, a portion of c; step 2: rest of a beside single tokens of c, d starts; ...
    plan = [[("a", 20), ("b", 1), ("c", 9)], [("a", 33), ("c", 1), ("d", 2)], [("c", 1), ("d", 30)], [("c", 7), ("d", 1)], [("d", 1)]]
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
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
        close(torch.cat(got[k]), want[k], tol)


def test_pages_and_slots_are_reused(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    """A pool of a few pages and two slots: later requests run in pages and slots that earlier ones dirtied."""
    cfg, W, _ = build(tmp_path, "all_loop", device, dtype)
    _, _, eng = build(tmp_path, "all_loop", device, dtype, max_batch=2, pool_tokens=96, block_size=16)
    assert eng.runner.alloc.num_blocks == 1 + 6
    seqs = [tokens_for(cfg, n, 40 + i) for i, n in enumerate((45, 33, 48, 17, 40, 31))]
    want = [oracle.forward(cfg, W, t)[0] for t in seqs]
    close(eng.feed([(0, seqs[0], list(range(45))), (1, seqs[1], list(range(33)))], [0, 1]), torch.cat(want[:2]), tol)
    with pytest.raises(RuntimeError):           # both slots are taken
        eng.feed([(2, seqs[2][:8], []), (3, seqs[3][:4], [])], [])
        eng.feed([(4, seqs[4][:2], [])], [])
    eng.feed([], [2, 3])
    # pool exhaustion is an error, not a silent overwrite
    with pytest.raises(MemoryError):
        eng.feed([(2, seqs[2], []), (4, seqs[2] + seqs[4], [])], [])
    eng.feed([], [2, 4])
    for rnd in range(2):                        # the same pages again and again, interleaved lifetimes
        a, b = 2 + 2 * rnd, 3 + 2 * rnd
        o1 = eng.feed([(a, seqs[a][:20], list(range(20))), (b, seqs[b][:9], list(range(9)))], [])
        o2 = eng.feed([(a, seqs[a][20:], list(range(len(seqs[a]) - 20))), (b, seqs[b][9:10], [0])], [a])
        o3 = eng.feed([(b, seqs[b][10:], list(range(len(seqs[b]) - 10)))], [b])
        na, nb = len(seqs[a]), len(seqs[b])
        close(torch.cat([o1[:20], o2[:na - 20]]), want[a], tol)
        close(torch.cat([o1[20:], o2[na - 20:], o3]), want[b], tol)
    assert eng.runner.alloc.num_free == 6


def test_long_decode(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    cfg, W, eng = build(tmp_path, "one_pass", device, dtype)
    toks = tokens_for(cfg, 90, 3)
    want, _ = oracle.forward(cfg, W, toks)
    close(feed_in_portions(eng, "x", toks, [3, 1]), want, tol)


@pytest.mark.parametrize("name", ["mid_loop", "no_loop"])
def test_greedy_generation_through_the_scheduler(tmp_path, name, device="cpu", dtype=torch.float32, graph=False):
    cfg, W, eng = build(tmp_path, name, device, dtype, graph=graph, max_seq_len=96)
    prompts = [tokens_for(cfg, n, 60 + n) for n in (5, 1, 19, 12, 3)]    # five requests, four slots: one waits
    params = SamplingParams(max_new_tokens=12, is_greedy=True)
    got = eng.generate(prompts, params)
    for p, g in zip(prompts, got):
        assert g == oracle.greedy(cfg, W, p, 12)
    assert eng.generate_no_cache(prompts[:2], params) == got[:2]
    assert eng.runner.alloc.num_free == eng.runner.alloc.num_blocks - 1


def test_config_is_read_not_assumed(tmp_path):
    from llmss_b200.models.bedovik import bedovik_spec
    from llmss_b200.utils.config import NativeConfig

    s = bedovik_spec(NativeConfig(CONFIGS["mid_loop"]))
    assert [i for i, _ in s.schedule()] == [0, 1, 2, 1, 2] and [t for _, t in s.schedule()] == [None, 0, None, 1, None]
    assert s.n_layers == 5 and s.mixers[2].scale == 0.5 and s.ffns[1] is None and s.ffns[0].keep == 2
    assert [i for i, _ in bedovik_spec(NativeConfig(CONFIGS["no_loop"])).schedule()] == [0, 1]
    bad = dict(CONFIGS["no_loop"], layers=[dict(CONFIGS["no_loop"]["layers"][0], type="windowed")])
    with pytest.raises(ValueError):
        bedovik_spec(NativeConfig(bad))


def test_command_line_generation_with_token_ids(tmp_path):
    """generate.py serves a checkpoint that ships no tokenizer: prompts and continuations are token ids."""
    import generate

    cfg = CONFIGS["no_loop"]
    path = write_random_checkpoint(tmp_path / "cli", cfg, dtype=torch.bfloat16, device="cpu", seed=4)
    W = oracle.load_weights(path)
    prompts = [tokens_for(cfg, 6, 70), tokens_for(cfg, 2, 71)]
    out = generate.main(["--pretrained_model_path", str(path), "--prompt_ids", *[" ".join(map(str, p)) for p in prompts],
                         "--max_new_tokens", "6", "--is_greedy", "--use_cache", "--dtype", "float32"])
    assert out == [oracle.greedy(cfg, W, p, 6) for p in prompts]


def run_trace_runner(tmp_path, device_env, dtype, tol):
    """bin/trace_run as a user starts it: steps on standard input, `done <n>` lines back, logits files in --out."""
    import json
    import os
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np

    cfg = CONFIGS["mid_loop"]
    path = write_random_checkpoint(tmp_path / "m", cfg, dtype=torch.bfloat16, device="cpu", seed=2)
    W = oracle.load_weights(path)
    a, b = tokens_for(cfg, 70, 80), tokens_for(cfg, 9, 81)
    want = {"a": oracle.forward(cfg, W, a)[0], "b": oracle.forward(cfg, W, b)[0]}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:33], "want": [0, 5, 32]}, {"id": "b", "tokens": b[:2], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[33:34], "want": [0]}], "end": []},                      # b sits this one out
        {"step": 2, "entries": [{"id": "b", "tokens": b[2:], "want": [0, 6]}, {"id": "a", "tokens": a[34:66], "want": [31]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": a[66:], "want": [0, 1, 2, 3]}], "end": ["a"]},
        {"step": 4, "entries": [{"id": "c", "tokens": b, "want": [8]}], "end": ["c"]},                          # b's pages and slot again
    ]
    expect = {0: [("a", 0), ("a", 5), ("a", 32)], 1: [("a", 33)], 2: [("b", 2), ("b", 8), ("a", 65)],
              3: [("a", 66), ("a", 67), ("a", 68), ("a", 69)], 4: [("b", 8)]}
    root = Path(__file__).resolve().parents[1]
    out = tmp_path / "out"
    env = dict(os.environ, **device_env)
    # --max-tokens 192: 70 and 9 tokens are live at once, each rounded up to whole 64-token pages
    p = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(path), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "192"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True,
                       text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(5)]
    for n, rows in expect.items():
        got = torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(len(rows), cfg["vocab"]))
        close(got, torch.stack([want[k][i] for k, i in rows]), tol)


def test_trace_runner_on_cpu(tmp_path):
    run_trace_runner(tmp_path, {"LLMSS_TRACE_CPU": "1", "CUDA_VISIBLE_DEVICES": ""}, "float32", TOL)


def test_model_call_with_past_state(tmp_path):
    """The registry class called like the other families' classes: model(input_ids, past_key_values) -> logits [B, S, V]."""
    cfg, W, eng = build(tmp_path, "no_loop")
    toks = tokens_for(cfg, 30, 90)
    want, _ = oracle.forward(cfg, W, toks)
    ids = torch.tensor([toks])
    out = eng.model(ids[:, :21], use_cache=True)
    out2 = eng.model(ids[:, 21:], past_key_values=out.past_key_values, use_cache=True)
    close(torch.cat([out.logits[0], out2.logits[0]]), want, TOL)
