"""Plain, slow restatement of the Fizadra design in torch, one function per mechanism, for the tests to compare the
framework against.  It shares no code with the package: it takes the parsed ``config.json`` dictionary and a
``{tensor name: tensor}`` dictionary and recomputes every position from the whole token list (no cache, no batch).

Everything runs in float64 on the CPU: the comparison tolerances of the tests are what the framework's bfloat16 / float32
arithmetic may lose against exact arithmetic.

Notation: ``T`` tokens, ``d`` width, ``H`` query heads, ``G`` key / value heads, ``dn`` unrotated and ``dr`` rotated query / key
sizes of a latent head, ``dk`` / ``dv`` key / value sizes, ``r`` latent size.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F64 = torch.float64


# ---- norms ------------------------------------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def group_norm(x: torch.Tensor, w: torch.Tensor, eps: float, groups: int) -> torch.Tensor:
    """x (T, d): every one of `groups` equal consecutive pieces of a row is brought to unit RMS on its own, then x * w."""
    T, d = x.shape
    return unit_rms(x.reshape(T, groups, d // groups), eps).reshape(T, d) * w


# ---- rotary positions -------------------------------------------------------------------------------------------
def rotary_frequencies(rot: dict) -> Tuple[torch.Tensor, float]:
    """Angular frequency per pair and the factor on cos / sin."""
    dims, base = rot["dims"], rot["base"]
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def index_of(turns: float) -> float:
        return dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(index_of(sc["fast"])), 0)
    hi = min(math.ceil(index_of(sc["slow"])), dims - 1)
    i = torch.arange(dims // 2, dtype=F64)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
    return f / sc["factor"] * ramp + f * (1 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x: torch.Tensor, rot: dict, interleaved: bool) -> torch.Tensor:
    """x (T, heads, n): the first rot.dims dimensions of every head turn by position * frequency; pairs are (2i, 2i + 1) when
    `interleaved`, else (i, i + dims / 2).  Row t is position t."""
    dims = rot["dims"]
    if dims == 0:
        return x
    f, mag = rotary_frequencies(rot)
    T = x.shape[0]
    ang = torch.arange(T, dtype=F64)[:, None] * f[None, :]
    cos, sin = (ang.cos() * mag)[:, None, :], (ang.sin() * mag)[:, None, :]
    part = x[..., :dims]
    if interleaved:
        u, v = part[..., 0::2], part[..., 1::2]
        turned = torch.stack([u * cos - v * sin, v * cos + u * sin], dim=-1).reshape(part.shape)
    else:
        u, v = part[..., : dims // 2], part[..., dims // 2 :]
        turned = torch.cat([u * cos - v * sin, v * cos + u * sin], dim=-1)
    return torch.cat([turned, x[..., dims:]], dim=-1)


# ---- attention over explicit keys and values ------------------------------------------------------------------
def causal_probabilities(scores: torch.Tensor, sink: Optional[torch.Tensor]) -> torch.Tensor:
    """scores (H, T, T) -> probabilities over keys j <= i; `sink` (H,) joins the denominator as exp(sink_h) and nothing else."""
    H, T, _ = scores.shape
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    p = torch.zeros_like(scores)
    for h in range(H):
        for i in range(T):
            s = scores[h, i, : i + 1]
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            den = e.sum() + (torch.exp(sink[h] - m) if sink is not None else 0.0)
            p[h, i, : i + 1] = e / den
    return p * mask


def latent_mixer(h: torch.Tensor, mx: dict, w: Dict[str, torch.Tensor], p: str, eps: float, second: bool,
                 shared: Optional[Tuple[torch.Tensor, torch.Tensor]]) -> Tuple[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    """Latent attention with one rotated key part shared by the heads.  `second`: the variant with half-split rotation pairs,
    no sink and one gate per head; otherwise interleaved pairs, a sink per head and a gate per output number.  `shared`:
    (latents, rotated key part) of the layer this one borrows from, or None.  Returns the output and what it attends over."""
    T = h.shape[0]
    H, dn, dr, dv, r = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    rot = dict(mx["rot"])
    cq = unit_rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(T, H, dn + dr)
    q_rot = rotate(q[..., dn:], rot, interleaved=not second)
    if shared is None:
        down = h @ w[p + "dkv"].T
        c = unit_rms(down[:, :r], eps) * w[p + "dkv.norm"]
        k_rot = rotate(down[:, None, r:], rot, interleaved=not second)[:, 0]
    else:
        c, k_rot = shared
    k = (c @ w[p + "uk"].T).reshape(T, H, dn)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q[..., :dn], k) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * mx["scale"]
    prob = causal_probabilities(scores, None if second else w[p + "sink"])
    o = torch.einsum("hij,jhd->ihd", prob, v)
    gate = torch.sigmoid(h @ w[p + "g"].T)
    o = o * (gate[:, :, None] if second else gate.reshape(T, H, dv))
    return o.reshape(T, H * dv) @ w[p + "o"].T, (c, k_rot)


def talking_mixer(h: torch.Tensor, mx: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    """Grouped-head attention with biased projections, a weighted RMS norm on every query and key head, half-split rotation,
    scores mixed over the heads by a matrix, and a softmax whose denominator holds an extra 1."""
    T = h.shape[0]
    H, G, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, dk)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, dk)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    q = rotate(unit_rms(q, eps) * w[p + "q.norm"], mx["rot"], interleaved=False)
    k = rotate(unit_rms(k, eps) * w[p + "k.norm"], mx["rot"], interleaved=False)
    per = H // G
    kv_of = [g // per for g in range(H)]
    raw = torch.einsum("ihd,jhd->hij", q, k[:, kv_of]) * mx["scale"]
    mixed = torch.einsum("hg,gij->hij", w[p + "talk"], raw)
    prob = causal_probabilities(mixed, torch.zeros(H, dtype=F64))
    o = torch.einsum("hij,jhd->ihd", prob, v[:, kv_of])
    return o.reshape(T, H * dv) @ w[p + "o"].T


def feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return torch.relu(h @ w[p + "up"].T) ** 2 @ w[p + "down"].T


# ---- the model --------------------------------------------------------------------------------------------------
def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], streams: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits (T, vocab) of a token list.  `streams` receives what leaves each layer (after the average over depth)."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    x = w["embed"][torch.tensor(tokens)]
    outs = [x]
    kept: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
    for i, layer in enumerate(cfg["layers"]):
        p, mx, kind = f"l{i}.", layer["mixer"], layer["type"]
        h = group_norm(x, w[p + "norm1"], eps, groups)
        if kind == "attention":
            y = talking_mixer(h, mx, w, p + "mix.", eps)
        elif kind in ("latent_attention", "latent_attention_2"):
            src = mx.get("kv_from")
            y, kept[i] = latent_mixer(h, mx, w, p + "mix.", eps, kind == "latent_attention_2", None if src is None else kept[src])
        else:
            raise ValueError(kind)
        x = x + group_norm(y, w[p + "norm1b"], eps, groups)
        if layer.get("mlp") is not None:
            x = x + group_norm(feed_forward(group_norm(x, w[p + "norm2"], eps, groups), w, p + "mlp."), w[p + "norm2b"], eps, groups)
        outs.append(x)
        x = sum(w[p + "dwa"][j] * outs[j] for j in range(i + 2))
        if streams is not None:
            streams.append(x)
    return group_norm(x, w["final.norm"], eps, groups) @ w["head"].T


def greedy(cfg: dict, weights: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    out = list(prompt)
    for _ in range(n_new):
        out.append(int(forward(cfg, weights, out)[-1].argmax()))
    return out
