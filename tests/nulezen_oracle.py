"""A plain, slow restatement of the Nulezen design in float64 torch, one function per mechanism, from its equations.  No cache, no
batch, no kernels: every function sees one whole sequence.  Shares no code with the package; `cfg` is the dictionary of a
``config.json``, `W` a dictionary of float64 tensors by checkpoint name.

    x0 = E[token] * embedding.scale
    layer:   h = dyt(x);  x <- x + ls1 * mixer(h) + ls2 * ff(h)                 dyt(x) = tanh(alpha x) * w + b
    loop:    layers start .. stop - 1 run `times` times; pass t begins with  x <- W_in [x ; x0] + step[t]
    logits = (E dyt_final(x)) * logit_scale
"""
from __future__ import annotations

import torch

F64 = torch.float64


def dyt(x, W, name):
    """dynamic tanh: no statistics, one scalar inside the tanh, a weight and an offset outside"""
    return torch.tanh(W[name + ".alpha"] * x) * W[name] + W[name + ".b"]


def rotate_half_split(x, pos, dims, base):
    """x (T, heads, dim): the pair (i, i + dims / 2), i < dims / 2, turns by pos * base^(-2 i / dims); dimensions past `dims` stay"""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = pos.to(F64)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def windowed_softmax_attention(q, k, v, scale, window, penalty=None):
    """q (T, H, dk), k (T, G, dk), v (T, G, dv) -> (T, H, dv).  Row i sees j with 0 <= i - j < window.  penalty(h, dist) is taken off
    the scaled score (dist = i - j as float64 tensor)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for i in range(T):
        lo = max(0, i - window + 1)
        dist = torch.arange(i - lo, -1, -1, dtype=F64)          # distance of keys lo .. i
        for h in range(H):
            g = h // (H // G)
            s = (k[lo : i + 1, g] @ q[i, h]) * scale
            if penalty is not None:
                s = s - penalty(h, dist)
            p = torch.softmax(s, dim=0)
            out[i, h] = p @ v[lo : i + 1, g]
    return out


def attention(h, W, p, m, kind):
    """Either mixer on the normed rows h (T, width).  kind "attention": no biases, no rotation, distance penalty r1 ln(1 + r2 dist),
    sigmoid gate per output number; kind "attention_2": biased q / k / v, rotation of half-split pairs, sigmoid gate per head."""
    T = h.shape[0]
    H, G = m["heads"], m.get("kv_heads", m["heads"])
    dk, dv = m["dim"], m.get("vdim", m["dim"])
    second = kind == "attention_2"
    q, k, v = h @ W[p + "q"].T, h @ W[p + "k"].T, h @ W[p + "v"].T
    if second:
        q, k, v = q + W[p + "q.b"], k + W[p + "k.b"], v + W[p + "v.b"]
    q, k, v = q.view(T, H, dk), k.view(T, G, dk), v.view(T, G, dv)
    penalty = None
    if second:
        rot = m.get("rot")
        if rot and rot["dims"] > 0:
            pos = torch.arange(T)
            q, k = rotate_half_split(q, pos, rot["dims"], rot["base"]), rotate_half_split(k, pos, rot["dims"], rot["base"])
    else:
        r1, r2 = W[p + "r1"], W[p + "r2"]
        penalty = lambda hh, dist: r1[hh] * torch.log(1.0 + r2[hh] * dist)   # noqa: E731
    o = windowed_softmax_attention(q, k, v, m["scale"], m["mask"]["size"], penalty)
    gate = torch.sigmoid(h @ W[p + "g"].T)
    o = o * gate[:, :, None] if second else o * gate.view(T, H, dv)
    return o.reshape(T, H * dv) @ W[p + "o"].T


def xielu(z, p, q):
    sp = lambda t: torch.log1p(torch.exp(t))   # noqa: E731
    pos = sp(p) * z * z + 0.5 * z
    neg = (0.5 + sp(q)) * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def dense_ff(h, W, p):
    return xielu(h @ W[p + "up"].T, W[p + "act"][0], W[p + "act"][1]) @ W[p + "down"].T


def clamped_expert(h, W, p, limit, alpha=1.702):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(alpha * g) * (u + 1.0)) @ W[p + "down"].T


def route(h, W, p, top):
    """-> (ids (T, top), weights (T, top)): the largest biased logits, softmax among those few"""
    z = h @ W[p + "router"].T + W[p + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def sparse_ff(h, W, p, ml):
    E, top = ml["router"]["experts"], ml["router"]["top"]
    idx, wts = route(h, W, p, top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += wts[t, j] * clamped_expert(h[t : t + 1], W, f"{p}e{e}.", ml["expert"]["limit"])[0]
    if ml.get("shared"):
        out = out + clamped_expert(h, W, p + "shared.", ml["shared"]["limit"])
    return out


def feed_forward(h, W, p, ml):
    return dense_ff(h, W, p) if ml["kind"] == "dense" else sparse_ff(h, W, p, ml)


def layer(x, W, i, spec):
    h = dyt(x, W, f"l{i}.norm1")
    y = attention(h, W, f"l{i}.mix.", spec["mixer"], spec["type"]) * W[f"l{i}.ls1"]
    if spec.get("mlp") is not None:
        y = y + feed_forward(h, W, f"l{i}.mlp.", spec["mlp"]) * W[f"l{i}.ls2"]
    return x + y


def forward(cfg, weights, tokens, trace=None):
    """logits (T, vocab) of one whole sequence; `trace` receives the stream after every layer run"""
    W = {k: v.to(F64) for k, v in weights.items()}
    x0 = W["embed"][torch.tensor(list(tokens))] * cfg.get("embedding", {}).get("scale", 1.0)
    x, L, loop = x0, cfg["layers"], cfg.get("loop")

    def run(i, x):
        x = layer(x, W, i, L[i])
        if trace is not None:
            trace.append(x.clone())
        return x

    if loop and loop["stop"] > loop["start"]:
        for i in range(loop["start"]):
            x = run(i, x)
        for t in range(loop["times"]):
            x = torch.cat([x, x0], dim=-1) @ W["loop.in"].T + W["loop.step"][t]
            for i in range(loop["start"], loop["stop"]):
                x = run(i, x)
        for i in range(loop["stop"], len(L)):
            x = run(i, x)
    else:
        for i in range(len(L)):
            x = run(i, x)
    return (dyt(x, W, "final.norm") @ W["embed"].T) * cfg.get("logit_scale", 1.0)


def greedy(cfg, weights, prompt, new_tokens):
    seq = list(prompt)
    for _ in range(new_tokens):
        seq.append(int(forward(cfg, weights, seq)[-1].argmax()))
    return seq

