"""The arrangement of parts in a layer."""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional

import torch

from .base import CacheView, FeedForward, Mixer, Norm, Part, PostNormed, ScaledPair, StreamState, TensorSpec

BLOCKS: Dict[str, Callable[..., "Part"]] = {}


def register_block(name: str, ctor: Callable[..., "Part"], *, replace: bool = False) -> None:
    if name in BLOCKS and not replace and BLOCKS[name] is not ctor:
        raise ValueError(f"block `{name}` is already registered")
    BLOCKS[name] = ctor


class PreNormBlock(Part):
    """``x <- x + mixer(norm_m(x))``; ``x <- x + ffn(norm_f(x))``
    (crates/vapi-backend-candle/src/models/lfm2.rs:633-648).

    The residual stream ``x`` is float32.  A layer's output is not added right away: it is
    handed on as ``delta`` and the next norm adds it while it reads the row, so each add
    costs no pass of its own.  ``forward`` therefore takes the pending delta of the layer
    before and returns its own.

    ``sub`` gives the checkpoint sub-prefix of each part, e.g. ``{"mixer": "conv.",
    "mixer_norm": "operator_norm.", "ffn": "feed_forward.", "ffn_norm": "ffn_norm."}``.
    """

    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, ffn: FeedForward,
                 sub: Dict[str, str]):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn, self.sub = mixer_norm, mixer, ffn_norm, ffn, dict(sub)

    def _parts(self):
        return (("mixer_norm", self.mixer_norm), ("mixer", self.mixer),
                ("ffn_norm", self.ffn_norm), ("ffn", self.ffn))

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        out: List[TensorSpec] = []
        for key, part in self._parts():
            out += part.tensor_specs(prefix + self.sub[key])
        return out

    def bind(self, tensors, prefix, dtype):
        for key, part in self._parts():
            part.bind(tensors, prefix + self.sub[key], dtype)

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor], ctx: Any,
                cache: CacheView) -> torch.Tensor:
        a = self.mixer_norm.apply(x, delta, ctx.dtype)
        d1 = self.mixer.forward(a, ctx, cache)
        f = self.ffn_norm.apply(x, d1, ctx.dtype)
        return self.ffn.forward(f, ctx)

    def first_norm(self) -> Norm:
        """The norm that reads the stream first in this block (its producer works for it)."""
        return self.mixer_norm

    def forward_stream(self, x: torch.Tensor, state: StreamState, ctx: Any, cache: CacheView,
                       next_weight: torch.Tensor) -> StreamState:
        """The same block for steps of a few rows: a norm is not run but handed, as a
        description, to its consumer's first product; each part's last product adds into ``x``
        and leaves the :class:`StreamState` the following norm needs (``next_weight`` is the
        weight of the norm that reads the stream after this block).  A part without a stream
        form is run the ordinary way between two small kernels."""
        from .. import ops
        mid_weight = self.ffn_norm.stream_weight()
        a = self.mixer_norm.deferred(state) if state is not None else None
        out = self.mixer.forward_stream(a, ctx, cache, x, mid_weight) if (a is not None and mid_weight is not None) else NotImplemented
        if out is NotImplemented:
            delta = self.mixer.forward(self.mixer_norm.apply(x, None, ctx.dtype), ctx, cache)
            out = self._add(ops, x, delta, mid_weight)
        f = self.ffn_norm.deferred(out) if out is not None else None
        out2 = self.ffn.forward_stream(f, ctx, x, next_weight) if (f is not None and next_weight is not None) else NotImplemented
        if out2 is NotImplemented:
            delta = self.ffn.forward(self.ffn_norm.apply(x, None, ctx.dtype), ctx)
            out2 = self._add(ops, x, delta, next_weight)
        return out2

    @staticmethod
    def _add(ops, x, delta, weight):
        if weight is None:
            ops.add_residual(x, delta)
            return None
        ss, xw = ops.add_residual_ss(x, delta, weight)
        return StreamState(xw, ss)


class SandwichBlock(Part):
    """A norm before and after each sublayer, and a multiplier on what the sublayer adds:

        x <- x + mult * post_m(mixer(pre_m(x)));   x <- x + mult * post_f(ffn(pre_f(x)))

    ``ffn`` may be None: the block then has only the first sublayer.  A sublayer's output is not
    normed and added by a kernel of its own: it is handed on as a :class:`PostNormed`, and the norm
    that reads the stream next (this block's second pre-norm, the next block's first, or the
    model's final norm) norms, scales and adds it while it reads the row.

    ``sub`` gives the checkpoint sub-prefix of each part (``mixer_norm``, ``mixer_post``, ``mixer``,
    ``ffn_norm``, ``ffn_post``, ``ffn``).  The post-norms must be RMS norms (their weight and eps are
    what is handed on).
    """

    def __init__(self, mixer_norm: Norm, mixer: Mixer, mixer_post: Norm, ffn_norm: Optional[Norm],
                 ffn: Optional[FeedForward], ffn_post: Optional[Norm], sub: Dict[str, str], mult: float = 1.0):
        if (ffn is None) != (ffn_norm is None) or (ffn is None) != (ffn_post is None):
            raise ValueError("a feed-forward comes with both of its norms or not at all")
        self.mixer_norm, self.mixer, self.mixer_post = mixer_norm, mixer, mixer_post
        self.ffn_norm, self.ffn, self.ffn_post = ffn_norm, ffn, ffn_post
        self.sub, self.mult = dict(sub), float(mult)

    def _parts(self):
        out = [("mixer_norm", self.mixer_norm), ("mixer", self.mixer), ("mixer_post", self.mixer_post)]
        if self.ffn is not None:
            out += [("ffn_norm", self.ffn_norm), ("ffn", self.ffn), ("ffn_post", self.ffn_post)]
        return out

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        out: List[TensorSpec] = []
        for key, part in self._parts():
            out += part.tensor_specs(prefix + self.sub.get(key, ""))
        return out

    def bind(self, tensors, prefix, dtype):
        for key, part in self._parts():
            part.bind(tensors, prefix + self.sub.get(key, ""), dtype)

    def first_norm(self) -> Norm:
        return self.mixer_norm

    def forward(self, x: torch.Tensor, delta, ctx: Any, cache: CacheView) -> PostNormed:
        a = self.mixer_norm.apply(x, delta, ctx.dtype)
        pending = PostNormed(self.mixer.forward(a, ctx, cache), self.mixer_post.weight, self.mixer_post.eps, self.mult)
        if self.ffn is None:
            return pending
        f = self.ffn_norm.apply(x, pending, ctx.dtype)
        return PostNormed(self.ffn.forward(f, ctx), self.ffn_post.weight, self.ffn_post.eps, self.mult)


class ParallelBlock(Part):
    """One norm, and both sublayers read its output: ``h = norm(x)``; ``x <- x + s_m * mixer(h) + s_f * ffn(h)``.

    ``s_m`` and ``s_f`` are vectors over the width (layer scale), named by ``scales = (mixer's, feed-forward's)``
    under the block's prefix; a name None means no scale.  ``ffn`` may be None: the block then has the mixer alone.
    Neither output is added by a kernel of its own: the block hands both on as a :class:`ScaledPair`, and the norm
    that reads the stream next (the next block's, or the model's final norm) scales and adds them while it reads
    the row.  ``sub`` gives the checkpoint sub-prefix of ``norm``, ``mixer`` and ``ffn``.
    """

    def __init__(self, norm: Norm, mixer: Mixer, ffn: Optional[FeedForward], sub: Dict[str, str],
                 scales=(None, None), hidden: Optional[int] = None):
        self.norm, self.mixer, self.ffn, self.sub = norm, mixer, ffn, dict(sub)
        self.scale_names = (scales[0], scales[1] if ffn is not None else None)
        self.hidden = int(hidden) if hidden is not None else int(getattr(norm, "dim", 0))
        if any(self.scale_names) and self.hidden <= 0:
            raise ValueError("a layer scale needs the width")
        self.s_m = self.s_f = None

    def _parts(self):
        out = [("norm", self.norm), ("mixer", self.mixer)]
        if self.ffn is not None:
            out.append(("ffn", self.ffn))
        return out

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        out: List[TensorSpec] = []
        for key, part in self._parts():
            out += part.tensor_specs(prefix + self.sub.get(key, ""))
        out += [TensorSpec(prefix + name, (self.hidden,), role="vector", init="ones") for name in self.scale_names if name]
        return out

    def bind(self, tensors, prefix, dtype):
        for key, part in self._parts():
            part.bind(tensors, prefix + self.sub.get(key, ""), dtype)
        self.s_m = tensors[prefix + self.scale_names[0]].contiguous() if self.scale_names[0] else None
        self.s_f = tensors[prefix + self.scale_names[1]].contiguous() if self.scale_names[1] else None

    def first_norm(self) -> Norm:
        return self.norm

    def forward(self, x: torch.Tensor, delta, ctx: Any, cache: CacheView) -> ScaledPair:
        h = self.norm.apply(x, delta, ctx.dtype)
        a = self.mixer.forward(h, ctx, cache)
        b = self.ffn.forward(h, ctx) if self.ffn is not None else None
        return ScaledPair(a, self.s_m, b, self.s_f)


register_block("prenorm", PreNormBlock)
register_block("parallel", ParallelBlock)
register_block("sandwich", SandwichBlock)
