"""Plain, slow implementation of the Lonasun decoder: whole sequences, no cache,
one function per mechanism.  It shares no code with the product package; it
reads a raw ``config.json`` dictionary and a ``{tensor name: tensor}`` dict.

Lonasun in this file's notation.  A layer is pre-norm: x += mixer(n1(x)), then
x += ff(n2(x)), with n(x) = x / sqrt(mean(x^2) + eps) * (1 + w).  The mixer is
attention with a short causal convolution over time on every channel of q, k and
v, a rotation of the first ``rot.dims`` dimensions of each q and k head, keys
visible only inside the query's own chunk of ``mask.size`` positions, and a
sigmoid gate on the concatenated heads.  The feed-forward is a mixture of small
relu^2 experts with identity experts at the end of the router's outputs and a
shared expert.  A span of layers runs several times with the same weights; each
pass starts by mixing the embedding output back in.

The arithmetic dtype is a parameter (float64 by default).
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def unit_offset_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * (1 + w): the checkpoint holds the gain's offset from one."""
    ms = x.pow(2).mean(-1, keepdim=True)
    return x / torch.sqrt(ms + eps) * (1.0 + w)


def short_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Causal convolution over time per channel.  u [S, C], w [C, taps]:
    y[t] = sum_j w[:, j] * u[t - (taps - 1) + j], zeros before the start."""
    S, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(S):
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                y[t] += w[:, j] * u[src]
    return y


def partial_rotation(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [S, heads, d].  The first ``dims`` dimensions of each head are rotated,
    dimension i paired with i + dims/2; the angle of pair i at position p is
    p * base^(-2i/dims).  The other dimensions pass unchanged."""
    half = dims // 2
    out = x.clone()
    for i in range(half):
        f = base ** (-2.0 * i / dims)
        a = positions.to(torch.float64) * f
        c, s = torch.cos(a).to(x.dtype)[:, None], torch.sin(a).to(x.dtype)[:, None]
        u, v = x[:, :, i], x[:, :, i + half]
        out[:, :, i] = u * c - v * s
        out[:, :, i + half] = v * c + u * s
    return out


def chunk_visible(i: int, j: int, size: int) -> bool:
    """Query position i sees key position j: causal and in the same chunk."""
    return j <= i and (i // size) == (j // size)


def chunked_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, size: int) -> torch.Tensor:
    """q [S, H, d], k [S, G, d], v [S, G, dv] -> [S, H, dv]; query head h reads
    key/value head h // (H / G); ordinary softmax over the visible keys."""
    S, H, d = q.shape
    G = k.shape[1]
    per = H // G
    out = torch.zeros((S, H, v.shape[2]), dtype=q.dtype)
    for h in range(H):
        g = h // per
        for i in range(S):
            js = [j for j in range(S) if chunk_visible(i, j, size)]
            sc = torch.stack([(q[i, h] * k[j, g]).sum() * scale for j in js])
            p = torch.softmax(sc, dim=0)
            out[i, h] = (p[:, None] * v[js, g]).sum(0)
    return out


def chunked_attention_fast(q, k, v, scale, size):
    """The same as ``chunked_attention`` with the mask as a matrix (for long sequences)."""
    S, H, d = q.shape
    G = k.shape[1]
    per = H // G
    pos = torch.arange(S)
    vis = (pos[None, :] <= pos[:, None]) & ((pos[None, :] // size) == (pos[:, None] // size))
    out = torch.zeros((S, H, v.shape[2]), dtype=q.dtype)
    for h in range(H):
        g = h // per
        sc = (q[:, h] @ k[:, g].T) * scale
        sc = sc.masked_fill(~vis, float("-inf"))
        out[:, h] = torch.softmax(sc, dim=-1) @ v[:, g]
    return out


def attention_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, fast: bool = True) -> torch.Tensor:
    """The whole mixer on h [S, width]; ``p`` is the layer's tensor prefix, ``m`` its 'mixer' dictionary."""
    S = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    dt = h.dtype
    q = short_conv(h @ W[f"{p}.mix.q"].to(dt).T, W[f"{p}.mix.q.conv"].to(dt))
    k = short_conv(h @ W[f"{p}.mix.k"].to(dt).T, W[f"{p}.mix.k.conv"].to(dt))
    v = short_conv(h @ W[f"{p}.mix.v"].to(dt).T, W[f"{p}.mix.v.conv"].to(dt))
    pos = torch.arange(S)
    q, k = q.view(S, H, d), k.view(S, G, d)
    if m.get("rot"):                                   # no 'rot': nothing is rotated
        q = partial_rotation(q, pos, m["rot"]["dims"], m["rot"]["base"])
        k = partial_rotation(k, pos, m["rot"]["dims"], m["rot"]["base"])
    size = m["mask"]["size"] if m.get("mask") else S   # no 'mask': one chunk holds the whole sequence
    att = (chunked_attention_fast if fast else chunked_attention)(q, k, v.view(S, G, dv), m["scale"], size)
    gate = torch.sigmoid(h @ W[f"{p}.mix.g"].to(dt).T)
    return (att.reshape(S, H * dv) * gate) @ W[f"{p}.mix.o"].to(dt).T


def relu2_expert(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """down( relu(up h)^2 )."""
    return torch.relu(h @ up.T).pow(2) @ down.T


def route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, top: int):
    """(chosen [S, top], weights [S, top]): scores are a softmax over all router outputs;
    the choice is by score + correction, the weights are the chosen scores over their sum."""
    s = torch.softmax(h @ router.T, dim=-1)
    chosen = torch.topk(s + correction, top, dim=-1).indices
    w = torch.gather(s, 1, chosen)
    return chosen, w / (w.sum(-1, keepdim=True) + 1e-20)


def moe_feed_forward(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    dt = h.dtype
    r = m["router"]
    E, top = r["experts"], r["top"]
    chosen, w = route(h, W[f"{p}.mlp.router"].to(dt), W[f"{p}.mlp.correction"].to(dt), top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(chosen[t, c])
            if e >= E:                                   # an identity expert
                y = h[t]
            else:
                y = relu2_expert(h[t], W[f"{p}.mlp.e{e}.up"].to(dt), W[f"{p}.mlp.e{e}.down"].to(dt))
            out[t] += w[t, c] * y
    if m.get("shared"):
        out = out + relu2_expert(h, W[f"{p}.mlp.shared.up"].to(dt), W[f"{p}.mlp.shared.down"].to(dt))
    return out


def layer_runs(cfg: dict) -> List[tuple]:
    """[(layer index, starts a pass)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        runs += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, False) for i in range(loop["stop"], n)]


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            fast: bool = True, trace: Optional[list] = None) -> torch.Tensor:
    """Logits [S, vocab] of one whole sequence.  ``trace`` (a list) receives the
    residual stream after every layer run."""
    eps = cfg["norm"]["eps"]
    x0 = W["embed"].to(dtype)[torch.tensor(tokens)]
    x = x0
    for i, starts_pass in layer_runs(cfg):
        if starts_pass:
            x = torch.cat([x, x0], dim=-1) @ W["loop.in"].to(dtype).T
        L, p = cfg["layers"][i], f"l{i}"
        if L["type"] != "attention":
            raise ValueError(L["type"])
        x = x + attention_mixer(unit_offset_rmsnorm(x, W[f"{p}.norm1"].to(dtype), eps), W, p, L["mixer"], fast)
        if L.get("mlp"):
            x = x + moe_feed_forward(unit_offset_rmsnorm(x, W[f"{p}.norm2"].to(dtype), eps), W, p, L["mlp"])
        if trace is not None:
            trace.append(x.clone())
    return unit_offset_rmsnorm(x, W["final.norm"].to(dtype), eps) @ W["head"].to(dtype).T
