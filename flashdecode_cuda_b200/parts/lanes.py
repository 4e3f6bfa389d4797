"""A residual stream of several lanes, and the pre-norm layer on it.

The stream of a step is ``resid`` [T, lanes * H] float32 (``ModelBlueprint.lanes``).  A sub-layer f with its
connection (read weights a [S], mixing matrix M [S, S] indexed [from, to], write-back weights b [S], a gain g [H]
per channel and a norm weight w [H]) does

    u     = sum_s a[s] X[s]
    y     = f(u / sqrt(mean(u^2) + eps) * w)
    X'[t] = sum_s M[s, t] X[s] + b[t] * (g * y)         (all lanes from the old ones)

The update is left pending, as the deferred residual add of the one-lane layers is: whoever norms next - the next
connection, or the final norm - applies it in the same kernel that reads the lanes (``csrc/lanes.cu``).  A connection
without a, M and b is a plain sum over one lane: x' = x + g * y.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.spec import TensorSpec
from .base import Block, LayerCache, Norm, Runtime
from .linear import GEMV_MAX_ROWS


@dataclass
class PendingLanes:
    """A sub-layer's output that is not in the lanes yet, with the weights that put it there."""
    y: torch.Tensor                     # [T, H] in the activation dtype, or float32 partial sums [parts, T, H]
    gain: Optional[torch.Tensor]        # [H] float32, or None
    mix: Optional[torch.Tensor]         # [S, S] float32 (from, to), or None: every lane keeps itself
    back: Optional[torch.Tensor]        # [S] float32, or None: ones


@register_part("norm", "lanes_rmsnorm")
class LanesRMSNorm(Norm):
    """A sub-layer's connection to a stream of ``lanes`` lanes: applies the update pending from the sub-layer before,
    reads its own mixture of the lanes and norms it (RMS norm, plain weight ``tensor``).  ``read`` / ``mix`` /
    ``back`` / ``gain``: full names of its tensors ([S], [S, S], [S], [H]); None: ones (``mix``: the unit matrix).  A
    connection that only reads - the final norm, whose ``read`` is None: the lanes added up - has no others."""

    accepts_parts = True

    def __init__(self, prefix: str, size: int, eps: float, lanes: int = 1, tensor: Optional[str] = None,
                 read: Optional[str] = None, mix: Optional[str] = None, back: Optional[str] = None,
                 gain: Optional[str] = None):
        if not (1 <= lanes <= 8):
            raise ValueError(f"{prefix or tensor}: {lanes} lanes: the kernel takes 1 to 8")
        self.name = tensor or f"{prefix}.weight"
        self.size, self.eps, self.lanes = size, float(eps), lanes
        self.names = {"read": read, "mix": mix, "back": back, "gain": gain}

    def tensor_specs(self) -> List[TensorSpec]:
        S = self.lanes
        shapes = {"read": (S,), "mix": (S, S), "back": (S,), "gain": (self.size,)}
        inits = {"read": "lane_read", "mix": "lane_mix", "back": "norm", "gain": "norm"}
        specs = [TensorSpec(self.name, (self.size,), "vector", init="norm")]
        specs += [TensorSpec(n, shapes[k], "vector", init=inits[k]) for k, n in self.names.items() if n is not None]
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        f32 = lambda n: None if n is None else tensors[n].float().contiguous()
        self.weight = f32(self.name)
        self.read, self.mix, self.back, self.gain = (f32(self.names[k]) for k in ("read", "mix", "back", "gain"))

    def pending(self, y: torch.Tensor) -> PendingLanes:
        """The output of this connection's sub-layer, to be put into the lanes by whoever norms next."""
        return PendingLanes(y, self.gain, self.mix, self.back)

    def forward(self, ctx, delta: Optional[PendingLanes], resid: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None, n_out: Optional[int] = None, write_resid: bool = True) -> None:
        d = delta
        K.lanes_norm(None if d is None else d.y, None if d is None else d.gain, None if d is None else d.mix,
                     None if d is None else d.back, resid, self.read, self.weight, self.eps, out, self.lanes,
                     rows=rows, n_out=n_out, write_lanes=write_resid)


@register_part("block", "lanes_prenorm")
class LanesPreNormBlock(Block):
    """Pre-norm layer on a stream of lanes: mixer, then feed-forward (or none), each behind its connection
    (``norm1`` / ``norm2``, parts of the kind ``lanes_rmsnorm``).  Takes and returns the pending update of the last
    sub-layer instead of a plain delta."""

    def __init__(self, norm1, mixer, norm2=None, feed_forward=None):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward
        if feed_forward is not None and norm2 is None:
            raise ValueError("a layer with a feed-forward needs the feed-forward's connection to the lanes")
        for n in (norm1, norm2):
            if n is not None and not hasattr(n, "pending"):
                raise TypeError("the connections of a layer on lanes are parts of the kind norm/lanes_rmsnorm")

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    def first_weights(self) -> Optional[torch.Tensor]:
        return self.mixer.first_weights()

    @property
    def accepts_parts(self) -> bool:
        return bool(getattr(self.norm1, "accepts_parts", False))

    def forward(self, ctx, resid: torch.Tensor, delta: Optional[PendingLanes], lc: LayerCache) -> PendingLanes:
        xn = ctx.ws.get("normed", (ctx.T, self.norm1.size), ctx.rt.dtype)
        after_block = ctx.upcoming
        self.norm1.forward(ctx, delta, resid, xn)
        if self.feed_forward is None:
            return self.norm1.pending(self.mixer.forward(ctx, xn, lc))
        ctx.upcoming = self.feed_forward.first_weights()
        d1 = self.norm1.pending(self.mixer.forward(ctx, xn, lc))
        self.norm2.forward(ctx, d1, resid, xn)
        ctx.upcoming = after_block
        if ctx.delta_parts_ok and ctx.T <= GEMV_MAX_ROWS and getattr(self.feed_forward, "offers_parts", False):
            return self.norm2.pending(self.feed_forward.forward(ctx, xn, parts_ok=True))
        return self.norm2.pending(self.feed_forward.forward(ctx, xn))

    def stream_state(self, resid: torch.Tensor, delta: Optional[PendingLanes]) -> torch.Tensor:
        """The lanes added up, with the pending update applied."""
        S = self.norm1.lanes
        out = torch.empty((resid.shape[0], resid.shape[1] // S), dtype=torch.float32, device=resid.device)
        if delta is None:
            K.lanes_sum(None, None, None, None, resid, out, S)
        else:
            y = delta.y if delta.y.dim() == 2 else delta.y.sum(0)
            K.lanes_sum(y.contiguous(), delta.gain, delta.mix, delta.back, resid, out, S)
        return out
