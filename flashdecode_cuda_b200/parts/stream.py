"""Operations on the whole residual stream between layers."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.spec import TensorSpec
from .base import Part, Runtime
from .linear import matmul


class StreamOp(Part):
    """``forward(ctx, resid, delta, embedded) -> delta``: ``resid`` [T, H] float32 is the residual stream,
    ``delta`` the output of the last sub-layer that has not been added to it yet (or None), ``embedded`` the
    embedding output of the step.  The operation leaves the new stream in ``resid`` and returns what is still to
    be added to it (None: nothing)."""
    kind = "stream_op"
    accepts_parts = False


@register_part("stream_op", "reinject_embedding")
class ReinjectEmbedding(StreamOp):
    """x <- W [x ; x0]: the stream and the embedding output side by side through one matrix ``<tensor>``
    [H, 2H] (x's columns first).  The sum that completes x and the result are float32; the product runs in the
    model's dtype."""

    def __init__(self, prefix: str, hidden_size: int, tensor: Optional[str] = None):
        self.name = tensor or f"{prefix}.weight"
        self.hidden_size = hidden_size

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.hidden_size, 2 * self.hidden_size), init="unit")]

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.weight = tensors[self.name]

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def first_weights(self) -> Optional[torch.Tensor]:
        return self.weight

    def forward(self, ctx, resid: torch.Tensor, delta: Optional[torch.Tensor], embedded: torch.Tensor):
        both = ctx.ws.get("reinject_in", (ctx.T, 2 * self.hidden_size), self.rt.dtype)
        K.add_concat(delta, resid, embedded, both)
        matmul(both, self.weight, None, resid, status=self.rt.status)
        return None
