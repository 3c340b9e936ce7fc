"""Plain float64 implementation of the Ninelix design: one function per mechanism, whole sequences, explicit loops
over tokens, no cache, no state objects, nothing imported from the package.  Slow on purpose.

``W`` maps tensor names to float64 tensors, ``cfg`` is the parsed config.json.
"""
import math

import torch

F64 = torch.float64


def rms_div(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x, w, eps):
    """The layer norm of the design: unit root mean square, weight stored around zero."""
    return rms_div(x, eps) * (1.0 + w)


def silu(x):
    return x / (1.0 + torch.exp(-x))


def sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def softplus(x):
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def gelu_erf(x):
    return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))


def embedding(tokens, W, cfg):
    bg = cfg["embedding"]["bigram"]
    rows = []
    for t, tok in enumerate(tokens):
        if t == 0:
            r = bg["buckets"]
        else:
            r = (tokens[t - 1] * bg["mul_prev"] + tok * bg["mul_cur"]) % bg["buckets"]
        rows.append(W["embed"][tok] + W["bigram"][r])
    return torch.stack(rows)


def causal_conv(u, w, bias=None):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
        if bias is not None:
            y[t] += bias
    return y


def distance_bucket(n, B, D):
    half = B // 2
    if n < half:
        return n
    return min(B - 1, half + int(math.floor(math.log(n / half) / math.log(D / half) * (B - half))))


# ----------------------------------------------------------------------------------------------------- mixers
def mixer_wkv(h, W, p, m, eps):
    T, width = h.shape
    H, D = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros(1, width, dtype=F64), h[:-1]])
    mix = {s: h + (prev - h) * W[f"{p}.mu.{s}"] for s in "rkvgw"}
    r = (mix["r"] @ W[f"{p}.r"].T).view(T, H, D)
    k = (mix["k"] @ W[f"{p}.k"].T).view(T, H, D)
    v = (mix["v"] @ W[f"{p}.v"].T).view(T, H, D)
    gate = silu(mix["g"] @ W[f"{p}.g"].T)
    w = torch.exp(-torch.exp(torch.tanh(mix["w"] @ W[f"{p}.w1"].T) @ W[f"{p}.w2"].T + W[f"{p}.w0"])).view(T, H, D)
    u = W[f"{p}.u"]
    out = torch.zeros(T, H, D, dtype=F64)
    for hd in range(H):
        S = torch.zeros(D, D, dtype=F64)
        for t in range(T):
            kv = torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = (S + u[hd][:, None] * kv).T @ r[t, hd]
            S = w[t, hd][:, None] * S + kv
    out = rms_div(out, eps).reshape(T, H * D) * W[f"{p}.norm"] * gate
    return out @ W[f"{p}.o"].T


def mixer_lightning(h, W, p, m, eps):
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ W[f"{p}.q"].T).view(T, H, D)
    k = silu(h @ W[f"{p}.k"].T).view(T, H, D)
    v = silu(h @ W[f"{p}.v"].T).view(T, H, Dv)
    out = torch.zeros(T, H, Dv, dtype=F64)
    for hd in range(H):
        S = torch.zeros(D, Dv, dtype=F64)
        for t in range(T):
            S = m["decay"][hd] * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    out = rms_div(out.reshape(T, H * Dv), eps) * W[f"{p}.norm"] * sigmoid(h @ W[f"{p}.g"].T)
    return out @ W[f"{p}.o"].T


def attention_left(h, W, p, m, eps):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    proj = {}
    for s in "qkv":
        u = h @ W[f"{p}.{s}"].T + W[f"{p}.{s}.b"]
        proj[s] = causal_conv(u, W[f"{p}.{s}.conv"])
    q = rms_div(proj["q"].view(T, H, D), eps) * W[f"{p}.q.norm"]
    k = rms_div(proj["k"].view(T, G, D), eps) * W[f"{p}.k.norm"]
    v = proj["v"].view(T, G, Dv)
    qt = m["q_temp"]
    rel = W[f"{p}.rel"]
    B = rel.shape[0]
    gate = sigmoid(h @ W[f"{p}.g"].T)
    out = torch.zeros(T, H, Dv, dtype=F64)
    for i in range(T):
        temp = 1.0 + qt["coef"] * math.log((i + 1) // qt["every"] + 1)
        for hd in range(H):
            g = hd // (H // G)
            s = (k[:i + 1, g] @ (q[i, hd] * temp)) * m["scale"]
            s = s + torch.stack([rel[distance_bucket(i - j, B, m["bias_max"]), hd] for j in range(i + 1)])
            a = torch.softmax(s, dim=0)
            out[i, hd] = (a[:, None] * v[:i + 1, g]).sum(0) * gate[i, hd]
    return out.reshape(T, H * Dv) @ W[f"{p}.o"].T


def mamba_right(h, W, p, m, eps):
    T = h.shape[0]
    H, Dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * Dv
    y = h @ W[f"{p}.in"].T
    z, xbc, dt = y[:, :inner], y[:, inner:2 * inner + 2 * G * N], y[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[f"{p}.conv"], W[f"{p}.conv.b"]))
    x = xbc[:, :inner].view(T, H, Dv)
    Bm = xbc[:, inner:inner + G * N].view(T, G, N)
    Cm = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + W[f"{p}.dt_bias"])
    out = torch.zeros(T, H, Dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(N, Dv, dtype=F64)
        a = torch.exp(W[f"{p}.A_log"][hd])
        for t in range(T):
            S = torch.exp(-a * dt[t, hd]) * S + dt[t, hd] * torch.outer(Bm[t, g], x[t, hd])
            out[t, hd] = S.T @ Cm[t, g] + W[f"{p}.D"][hd] * x[t, hd]
    out = out.reshape(T, inner) * silu(z)
    ng = m["norm_groups"]
    out = rms_div(out.view(T, ng, inner // ng), eps).reshape(T, inner) * W[f"{p}.norm"]
    return out @ W[f"{p}.o"].T


def mixer_parallel(h, W, p, m, eps):
    a = rms_div(attention_left(h, W, f"{p}.left", m["left"], eps), eps) * W[f"{p}.left.out"]
    b = rms_div(mamba_right(h, W, f"{p}.right", m["right"], eps), eps) * W[f"{p}.right.out"]
    return 0.5 * (a + b)


MIXERS = {"wkv": mixer_wkv, "lightning": mixer_lightning, "parallel": mixer_parallel}


# ----------------------------------------------------------------------------------------------------- feed-forward
def ff_dense(h, W, p, f):
    return gelu_erf(h @ W[f"{p}.up"].T) @ W[f"{p}.down"].T


def route(z, top):
    """Per token: the ``top`` largest logits (lower index first on a tie) and the softmax over just those."""
    ids, wts = [], []
    for row in z:
        order = sorted(range(len(row)), key=lambda e: (-float(row[e]), e))[:top]
        sel = torch.stack([row[e] for e in order])
        ids.append(order)
        wts.append(torch.softmax(sel, dim=0))
    return ids, wts


def ff_moe(h, W, p, f):
    z = h @ W[f"{p}.router"].T
    ids, wts = route(z, f["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(ids[t], wts[t]):
            a = silu(W[f"{p}.e{e}.gate"] @ h[t]) * (W[f"{p}.e{e}.up"] @ h[t])
            out[t] += wt * (W[f"{p}.e{e}.down"] @ a)
    return out


# ----------------------------------------------------------------------------------------------------- model
def forward(tokens, W, cfg, taps=None):
    """Logits [T, vocab] of a whole sequence; ``taps`` receives the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = embedding(list(tokens), W, cfg)
    for i, lc in enumerate(cfg["layers"]):
        p = f"l{i}"
        x = x + layer_norm(MIXERS[lc["type"]](x, W, f"{p}.mix", lc["mixer"], eps), W[f"{p}.norm1"], eps)
        f = lc.get("mlp")
        if f is not None:
            y = ff_dense(x, W, f"{p}.mlp", f) if f["kind"] == "dense" else ff_moe(x, W, f"{p}.mlp", f)
            x = x + layer_norm(y, W[f"{p}.norm2"], eps)
        if taps is not None:
            taps.append(x.clone())
    return (layer_norm(x, W["final.norm"], eps) @ W["head"].T) * cfg["logit_scale"]


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
