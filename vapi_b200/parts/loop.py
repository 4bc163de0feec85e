"""What a looped stack does to the residual stream between passes."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch

from .. import ops
from .base import Part, ScaledPair, TensorSpec


class StreamInjection(Part):
    """``x <- W [x; x0]``: the stream, with the embedding's output x0 beside it, through one matrix
    [hidden, 2 * hidden] (x first).  A model whose layers run several passes puts this in front of a pass's first
    layer, so that every pass starts from what the pass before left and from the input itself.

    It is not a layer: it has no cache, it replaces the stream instead of adding to it, and the run order names
    it by a key of ``ModelPlan.stream_parts`` (``LayerCall.before``).  Whatever is pending for the stream (the
    outputs of the layer before) is folded in by the kernel that lays x out for the product, in float32; the
    product's float32 result is the new stream.  x0 is laid out once per step, in the right half of a buffer
    whose left half every pass refills.
    """

    #: the runner keeps the embedding's output of the step for parts that say so
    needs_embedding_output = True

    def __init__(self, hidden: int, name: str = "loop.in"):
        self.hidden, self.name = int(hidden), name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str = "") -> List[TensorSpec]:
        return [TensorSpec(f"{prefix}{self.name}", (self.hidden, 2 * self.hidden))]

    def bind(self, tensors: Dict[str, torch.Tensor], prefix: str, dtype: torch.dtype) -> None:
        self.weight = tensors[f"{prefix}{self.name}"].contiguous()

    def forward(self, x: torch.Tensor, delta: Any, ctx: Any) -> Tuple[torch.Tensor, None]:
        """Returns the new stream and what is pending for it (nothing)."""
        H = self.hidden
        key = ("stream_injection", id(self))
        both = ctx.extras.get(key)
        if both is None:
            x0 = ctx.extras["embedding_output"]
            both = torch.empty((x.shape[0], 2 * H), dtype=ctx.dtype, device=x.device)
            ops.scaled_add_rmsnorm(x0, None, None, None, None, None, 0.0, ctx.dtype, copy=True, out=both[:, H:])
            ctx.extras[key] = both
        if isinstance(delta, ScaledPair):
            a, sa, b, sb = delta.a, delta.scale_a, delta.b, delta.scale_b
        elif delta is None or isinstance(delta, torch.Tensor):
            a, sa, b, sb = delta, None, None, None
        else:
            raise TypeError(f"a stream injection cannot fold in a pending {type(delta).__name__}")
        ops.scaled_add_rmsnorm(x, a, sa, b, sb, None, 0.0, ctx.dtype, copy=True, out=both[:, :H])
        return ops.linear(both, self.weight, None, torch.float32), None
