"""Plain, slow implementation of the Nizazen decoder: whole sequences, no cache,
one function per mechanism.  It shares no code with the product package; it
reads a raw ``config.json`` dictionary and a ``{tensor name: tensor}`` dict.

Nizazen in this file's notation.  The residual stream has ``streams`` lanes
X[0..S-1], all equal to the token embedding at the start.  A sub-layer f (a
mixer or a feed-forward) with its norm n, its per-channel output scale ls and
its lane weights (a [S], M [S, S], b [S]) does

    u      = sum_s a[s] X[s]
    y      = ls * f(n(u))                      n(u) = u / sqrt(mean(u^2) + eps) * w
    X'[t]  = sum_s M[s, t] X[s] + b[t] * y     (all lanes from the old ones)

and at the end the lanes are added, normed, sent through the head, and the
logits are squashed to cap * tanh(logits / cap).  Without ``streams`` in the
configuration there is one lane and x' = x + y.

Mixers: windowed attention (grouped heads, no rotation, q and k each normed over
their whole projection before the heads are split, a window of ``mask.size``
positions that includes the query's own) and latent attention (keys and values
of every head are made from one normed low-rank vector per position; causal).
Feed-forwards: a dense gated one with biases and the tanh form of GELU, and a
mixture of clamped gated experts chosen by the largest router logits.

The arithmetic dtype is a parameter (float64 by default).
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w over the last dimension."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                      window: Optional[int]) -> torch.Tensor:
    """q [S, H, d], k [S, G, d], v [S, G, dv] -> [S, H, dv].  Query head h reads key/value head h // (H / G).
    The query at position i sees j <= i, and with a window only those with i - j < window."""
    S, H, _ = q.shape
    G = k.shape[1]
    per = H // G
    out = torch.zeros((S, H, v.shape[2]), dtype=q.dtype)
    for h in range(H):
        g = h // per
        for i in range(S):
            lo = 0 if window is None else max(0, i - window + 1)
            sc = (k[lo:i + 1, g] @ q[i, h]) * scale
            p = torch.softmax(sc, dim=0)
            out[i, h] = p @ v[lo:i + 1, g]
    return out


def windowed_attention(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """The 'attention' mixer on a whole sequence h [S, width]."""
    S = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rmsnorm(h @ t[f"{p}.q"].T, t[f"{p}.q.norm"], eps)          # over all heads' rows at once
    k = rmsnorm(h @ t[f"{p}.k"].T, t[f"{p}.k.norm"], eps)
    v = h @ t[f"{p}.v"].T
    window = m["mask"]["size"] if m.get("mask") else None
    a = softmax_attention(q.view(S, H, d), k.view(S, G, d), v.view(S, G, dv), m["scale"], window)
    return a.reshape(S, H * dv) @ t[f"{p}.o"].T


def latent_attention(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """The 'latent_attention' mixer on a whole sequence: every head's keys and values come from one
    normed vector c of ``kv_rank`` dimensions per position."""
    S = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ t[f"{p}.q"].T).view(S, H, d)
    c = rmsnorm(h @ t[f"{p}.dkv"].T, t[f"{p}.dkv.norm"], eps)
    k = (c @ t[f"{p}.uk"].T).view(S, H, d)
    v = (c @ t[f"{p}.uv"].T).view(S, H, dv)
    window = m["mask"]["size"] if m.get("mask") else None
    a = softmax_attention(q, k, v, m["scale"], window)
    return a.reshape(S, H * dv) @ t[f"{p}.o"].T


def dense_ff(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    g = h @ t[f"{p}.gate"].T + t[f"{p}.gate.b"]
    u = h @ t[f"{p}.up"].T + t[f"{p}.up.b"]
    return (gelu_tanh(g) * u) @ t[f"{p}.down"].T + t[f"{p}.down.b"]


def clamped_expert(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ t[f"{p}.gate"].T, max=limit)
    u = torch.clamp(h @ t[f"{p}.up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ t[f"{p}.down"].T


def route(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str, top: int):
    """(chosen experts [S, top], weights [S, top]): the largest logits, softmax over them alone."""
    z = h @ t[f"{p}.router"].T + t[f"{p}.router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def expert_mixture(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str, f: dict) -> torch.Tensor:
    idx, w = route(h, t, p, f["router"]["top"])
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        for e, we in zip(idx[i].tolist(), w[i]):
            out[i] += we * clamped_expert(h[i:i + 1], t, f"{p}.e{e}", f["expert"]["limit"])[0]
    return out


def lane_sublayer(X: torch.Tensor, f, norm_w: torch.Tensor, eps: float, ls: torch.Tensor,
                  a: Optional[torch.Tensor], M: Optional[torch.Tensor], b: Optional[torch.Tensor]) -> torch.Tensor:
    """X [S_lanes, T, width] -> the new lanes.  a, M, b None: one lane, plain residual sum."""
    if a is None:
        return X + (ls * f(rmsnorm(X[0], norm_w, eps)))[None]
    u = torch.einsum("s,stw->tw", a, X)
    y = ls * f(rmsnorm(u, norm_w, eps))
    return torch.einsum("sr,stw->rtw", M, X) + b[:, None, None] * y[None]


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            layer_states: Optional[list] = None) -> torch.Tensor:
    """Logits [len(tokens), vocab].  ``layer_states``: a list that receives the sum of the lanes after every layer."""
    t = {k: (v.to(dtype) if v.dtype.is_floating_point else v) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    lanes = cfg.get("streams")
    x = t["embed"][torch.tensor(tokens, dtype=torch.long)]
    X = torch.stack([x] * (lanes or 1))
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}"
        mixer = {"attention": windowed_attention, "latent_attention": latent_attention}[L["type"]]
        hc = (lambda q: (t[f"{p}.hc{q}.in"], t[f"{p}.hc{q}.mix"], t[f"{p}.hc{q}.out"])) if lanes else (lambda q: (None,) * 3)
        X = lane_sublayer(X, lambda z: mixer(z, t, f"{p}.mix", L["mixer"], eps), t[f"{p}.norm1"], eps, t[f"{p}.ls1"], *hc(1))
        f = L.get("mlp")
        if f is not None:
            if f["kind"] == "dense":
                ff = lambda z: dense_ff(z, t, f"{p}.mlp")
            else:
                ff = lambda z: expert_mixture(z, t, f"{p}.mlp", f)
            X = lane_sublayer(X, ff, t[f"{p}.norm2"], eps, t[f"{p}.ls2"], *hc(2))
        if layer_states is not None:
            layer_states.append(X.sum(0))
    logits = rmsnorm(X.sum(0), t["final.norm"], eps) @ t["head"].T
    cap = cfg.get("logit_softcap")
    return logits if not cap else cap * torch.tanh(logits / cap)
