"""RMSNorm with the residual add folded in."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from .base import Norm, NormedStream, PostNormed, ScaledPair, TensorSpec, register_norm


def _raw_branches(y):
    """A sublayer's output as the post-norm kernel takes it.  Mixers side by side may hand on their raw outputs
    (``outs``, ``weights``, ``eps``, ``scale``): two of them ride on the kernel that norms the sublayer into the
    stream, any other number is normed and averaged by a kernel of its own first."""
    if not hasattr(y, "outs"):
        return y, None
    if len(y.outs) == 2:
        return y.outs[0], (y.outs[1], y.weights[0], y.weights[1], y.eps, y.scale)
    return y.tensor(), None


class RMSNorm(Norm):
    """``y = x * rsqrt(mean(x^2) + eps) * w``: the weight multiplies as it is (no ``1 + w``)
    (crates/vapi-backend-candle/src/models/lfm2.rs:626-628).  Mean, rsqrt and the residual
    sum are float32 whatever the activation dtype."""

    #: what the kernels that norm on a reader's behalf call this norm
    kind = "rms"

    def __init__(self, dim: int, eps: float, weight_name: str = "weight"):
        self.dim, self.eps, self.weight_name = int(dim), float(eps), weight_name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(f"{prefix}{self.weight_name}", (self.dim,), role="vector", init="ones")]

    def bind(self, tensors: Dict[str, torch.Tensor], prefix: str, dtype: torch.dtype) -> None:
        self.weight = tensors[f"{prefix}{self.weight_name}"].contiguous()

    def apply(self, x, delta, dtype, rows=None):
        if isinstance(delta, PostNormed):
            y, branches = _raw_branches(delta.y)
            return ops.postnorm_add_rmsnorm(x, y, delta.weight, delta.eps, delta.mult, self.weight, self.eps,
                                            dtype, rows, branches=branches)
        if isinstance(delta, ScaledPair):
            return ops.scaled_add_rmsnorm(x, delta.a, delta.scale_a, delta.b, delta.scale_b, self.weight, self.eps, dtype, rows)
        return ops.add_rmsnorm(x, delta, self.weight, self.eps, dtype, rows)

    def stream_weight(self):
        return self.weight

    def deferred(self, state):
        return NormedStream(state.xw, state.ss, self.eps)


class LayerNorm(Norm):
    """``y = (x - mean) / sqrt(var + eps) * w`` with a weight and no bias; the variance is the mean of the
    squared deviations.  Mean, variance and the residual sum are float32 whatever the activation dtype.

    The stream it reads may be a single one, [n, H], with a plain delta pending, or several copies side by
    side, [n, S, H], with a :class:`~vapi_b200.parts.hyper.HyperPending` pending; it then norms the sum of
    the copies (that is how a model with several streams ends)."""

    kind = "layer"

    def __init__(self, dim: int, eps: float, weight_name: str = "weight"):
        self.dim, self.eps, self.weight_name = int(dim), float(eps), weight_name
        self.weight: Optional[torch.Tensor] = None
        self._one: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(f"{prefix}{self.weight_name}", (self.dim,), role="vector", init="ones")]

    def bind(self, tensors: Dict[str, torch.Tensor], prefix: str, dtype: torch.dtype) -> None:
        self.weight = tensors[f"{prefix}{self.weight_name}"].contiguous()
        self._one = torch.ones(1, dtype=torch.float32, device=self.weight.device)

    def apply(self, x, delta, dtype, rows=None):
        from .hyper import HyperPending
        if x.dim() == 2:                         # one stream: a plain delta is a write with weight one
            y = delta.y if isinstance(delta, HyperPending) else delta
            return ops.hyper_read_norm(x.unsqueeze(1), y, self._one if y is not None else None,
                                       self._one if y is not None else None, None, self.weight, self.eps, dtype, rows,
                                       self.kind, delta.branch if isinstance(delta, HyperPending) else None)
        if delta is not None and not isinstance(delta, HyperPending):
            raise TypeError("several streams take a sublayer's output with its mix matrix and write vector")
        y, mix, write = (delta.y, delta.mix, delta.write) if delta is not None else (None, None, None)
        return ops.hyper_read_norm(x, y, mix, write, None, self.weight, self.eps, dtype, rows, self.kind,
                                   delta.branch if delta is not None else None)


class NoNorm(Norm):
    """No norm at all, for a sublayer that reads the residual stream as it is: ``apply`` folds in what is pending
    (a plain delta, or a :class:`PostNormed` that is normed on its way into the stream) and hands the rows on in
    the activation dtype.  It has no tensors."""

    kind = "none"

    def __init__(self, dim: int = 0):
        self.dim = int(dim)
        self.weight = None

    def apply(self, x, delta, dtype, rows=None):
        if isinstance(delta, PostNormed):
            y, branches = _raw_branches(delta.y)
            return ops.postnorm_add_rmsnorm(x, y, delta.weight, delta.eps, delta.mult, None, 0.0, dtype, rows, copy=True,
                                            branches=branches)
        if delta is not None:
            if rows is not None:
                raise ValueError("a plain delta is added to every row or to none")
            ops.add_residual(x, delta)
        if rows is None and x.dtype == dtype:
            return x                      # the sublayers only read it
        return ops.postnorm_add_rmsnorm(x, None, None, 0.0, 1.0, None, 0.0, dtype, rows, copy=True)


register_norm("none", NoNorm)
register_norm("rmsnorm", RMSNorm)
register_norm("layernorm", LayerNorm)
