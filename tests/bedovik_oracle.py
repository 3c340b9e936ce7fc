"""Plain, slow float64 implementation of the Bedovik design, one function per mechanism.

Written from the equations only: no import from llmss_b200, no cache, no batching, no absorbed products --
every call recomputes whole sequences with explicit loops over tokens, heads and experts.  The product path
(engine + ops, CPU or CUDA) is compared with this.

Notation: W = width, H = heads, d = query / key size per head, dv = value size per head, R = latent rank,
E = experts, F = expert hidden size.  Linear weights are [out, in].
"""

import torch

F64 = torch.float64


def dyt(x, alpha, w, b):
    """Dynamic Tanh: tanh(alpha * x) * w + b, element-wise."""
    return torch.tanh(alpha * x) * w + b


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def latent_attention(h, w_q, w_dkv, norm_w, w_uk, w_uv, w_o, w_g, heads, d, dv, scale, eps):
    """h: [T, W] of ONE sequence from position 0.  Keys and values are rebuilt from the normed latent per head."""
    T = h.shape[0]
    q = h @ w_q.T                                # [T, H * d]
    c = rms_norm(h @ w_dkv.T, norm_w, eps)       # [T, R]
    k = c @ w_uk.T                               # [T, H * d]
    v = c @ w_uv.T                               # [T, H * dv]
    out = torch.zeros(T, heads * dv, dtype=F64)
    for t in range(T):
        for hd in range(heads):
            qh = q[t, hd * d:(hd + 1) * d]
            s = torch.stack([qh @ k[j, hd * d:(hd + 1) * d] for j in range(t + 1)]) * scale
            p = torch.softmax(s, 0)
            o = sum(p[j] * v[j, hd * dv:(hd + 1) * dv] for j in range(t + 1))
            if w_g is not None:
                o = o * torch.sigmoid(w_g[hd] @ h[t])
            out[t, hd * dv:(hd + 1) * dv] = o
    return out @ w_o.T


def route(z, top, groups, keep, route_scale):
    """z: [E] router logits of one token -> (chosen expert indices, their weights)."""
    E = z.shape[0]
    s = torch.softmax(z, 0)
    size = E // groups
    gscore = [max(float(s[g * size + i]) for i in range(size)) for g in range(groups)]
    best_groups = sorted(range(groups), key=lambda g: (-gscore[g], g))[:keep]
    eligible = [e for e in range(E) if e // size in best_groups]
    chosen = sorted(eligible, key=lambda e: (-float(s[e]), e))[:top]
    total = sum(s[e] for e in chosen) + 1e-20
    return chosen, [s[e] / total * route_scale for e in chosen]


def experts(h_t, chosen, weights, ups, downs):
    """Weighted sum of the chosen experts for one token; expert = W_down relu(W_up h)^2."""
    out = torch.zeros(downs[0].shape[0], dtype=F64)
    for e, w in zip(chosen, weights):
        out = out + w * (downs[e] @ torch.relu(ups[e] @ h_t) ** 2)
    return out


def run_order(cfg):
    """[(layer, pass number if this run opens a pass of the loop else None)]."""
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(lp["start"])]
    for t in range(lp["times"]):
        for i in range(lp["start"], lp["stop"]):
            order.append((i, t if i == lp["start"] else None))
    return order + [(i, None) for i in range(lp["stop"], n)]


def forward(cfg, W, tokens):
    """Whole sequence from position 0.  W: name -> float64 tensor.  Returns (logits [T, vocab], residual after each run)."""
    T = len(tokens)
    eps = cfg["norm"]["eps"]
    x = W["embed"][tokens] + W["pos"][:T]
    x0 = x.clone()
    taps = []
    for li, opens in run_order(cfg):
        if opens is not None:
            x = torch.cat([x, x0], -1) @ W["loop.in"].T + W["loop.step"][opens]
        L, p = cfg["layers"][li], f"l{li}"
        h = dyt(x, W[f"{p}.norm1.alpha"], W[f"{p}.norm1"], W[f"{p}.norm1.b"])
        m = L["mixer"]
        gate = W[f"{p}.mix.g"] if L["type"] == "latent_attention" else None
        y = W[f"{p}.ls1"] * latent_attention(h, W[f"{p}.mix.q"], W[f"{p}.mix.dkv"], W[f"{p}.mix.dkv.norm"], W[f"{p}.mix.uk"],
                                              W[f"{p}.mix.uv"], W[f"{p}.mix.o"], gate, m["heads"], m["dim"], m["vdim"],
                                              m["scale"], eps)
        if L.get("mlp"):
            r = L["mlp"]["router"]
            ups = [W[f"{p}.mlp.e{e}.up"] for e in range(r["experts"])]
            downs = [W[f"{p}.mlp.e{e}.down"] for e in range(r["experts"])]
            ff = torch.zeros_like(x)
            for t in range(T):
                chosen, wts = route(W[f"{p}.mlp.router"] @ h[t], r["top"], r["groups"]["count"], r["groups"]["keep"], r["scale"])
                ff[t] = experts(h[t], chosen, wts, ups, downs)
            y = y + W[f"{p}.ls2"] * ff
        x = x + y
        taps.append(x.clone())
    logits = dyt(x, W["final.norm.alpha"], W["final.norm"], W["final.norm.b"]) @ W["head"].T
    return logits, taps


def greedy(cfg, W, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, W, toks)[0][-1].argmax()))
    return toks[len(prompt):]


def load_weights(path):
    """All tensors of a checkpoint folder as float64."""
    from pathlib import Path

    from safetensors import safe_open

    out = {}
    for f in sorted(Path(path).glob("*.safetensors")):
        with safe_open(str(f), framework="pytorch") as h:
            for k in h.keys():
                out[k] = h.get_tensor(k).to(F64)
    return out
