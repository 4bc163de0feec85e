"""A mixture of small feed-forward experts with a shared expert and identity experts."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from .. import ops
from .base import FeedForward, TensorSpec, register_feed_forward


class SparseMoE(FeedForward):
    """Each token uses ``top`` of ``experts`` feed-forward layers ``W_down relu(W_up f)^2`` (no biases).

    The router's logits ``W_r f`` are float32 and cover ``experts + identity`` outputs; the scores are their
    softmax over all outputs.  An output is chosen by its score plus a stored correction; the weights use the
    score without it, divided by the sum of the chosen scores (+ 1e-20).  The outputs form ``groups`` equal groups
    of neighbours; a group's score is its largest corrected score, and only outputs of the ``keep`` best groups
    can be chosen.  The last ``identity`` outputs have no tensors: their output is the token's input itself.  A
    shared expert of the same form (``shared_ff`` wide; None: absent) runs for every token and is added.

    Options: ``gated`` (an expert is ``W_down (silu(W_gate f) * (W_up f))``, three matrices), ``router_bias`` (a
    stored vector added to the router's logits) and ``score`` "chosen" (the ``top`` largest logits win and the
    weights are the softmax over the chosen logits only; there is then no correction tensor and no grouping),
    ``route`` "table" (no router at all: a stored integer table [``vocab``, top] names the experts of each token id,
    each with weight ``1 / top``; the step's token ids choose) and, for gated experts, ``act`` = (limit, alpha,
    shift): ``g' * sigmoid(alpha g') * (u' + shift)`` with ``g' = min(W_gate f, limit)`` and
    ``u' = clamp(W_up f, -limit, limit)`` when ``limit`` > 0 (the default (0, 1, 0) is SiLU gating).

    The experts' matrices are stacked at bind time ([experts, ff, hidden] and [experts, hidden, ff]); a step's
    tokens are grouped by expert on the device (see ``csrc/moe.cu``), so nothing about the routing reaches the host.
    """

    def __init__(self, hidden: int, ff: int, experts: int, top: int, *, identity: int = 0, groups: int = 1, keep: int = 1,
                 shared_ff: Optional[int] = None, names: Optional[Dict[str, str]] = None, weight_suffix: str = ".weight",
                 gated: bool = False, router_bias: bool = False, score: str = "softmax", route: str = "router",
                 vocab: int = 0, act=(0.0, 1.0, 0.0)):
        outputs = int(experts) + int(identity)
        if experts < 0 or identity < 0 or outputs <= 0 or not 1 <= top <= outputs:
            raise ValueError(f"{experts} experts + {identity} identity experts, top {top}")
        if groups < 1 or outputs % groups or not 1 <= keep <= groups or (outputs // groups) * keep < top:
            raise ValueError(f"{outputs} router outputs in {groups} groups, {keep} kept, top {top}")
        self.hidden, self.ff, self.E, self.I, self.top = int(hidden), int(ff), int(experts), int(identity), int(top)
        self.groups, self.keep, self.shared_ff, self.sfx = int(groups), int(keep), shared_ff, weight_suffix
        if score not in ("softmax", "chosen"):
            raise ValueError(f"score `{score}` is not one of softmax, chosen")
        if score == "chosen" and (groups != 1 or identity):
            raise ValueError("weights from the chosen logits come without groups and identity experts")
        if route not in ("router", "table"):
            raise ValueError(f"route `{route}` is not one of router, table")
        if route == "table" and (identity or groups != 1 or router_bias or vocab <= 0 or experts <= 0):
            raise ValueError("a table over the token ids chooses among real experts, without groups or a bias, and needs the vocabulary's size")
        self.by_table, self.vocab = route == "table", int(vocab)
        self.act = tuple(float(v) for v in act)
        if len(self.act) != 3 or (self.act != (0.0, 1.0, 0.0) and not gated):
            raise ValueError("the activation's constants (limit, alpha, shift) belong to gated experts")
        self.gated, self.router_bias, self.score = bool(gated), bool(router_bias), score
        self.names = {"expert": "experts.{}.", "up": "up_proj", "down": "down_proj", "gate": "gate_proj", "router": "router",
                      "correction": "correction", "router_bias": "router.bias", "shared": "shared.", "table": "table"}
        if names:
            self.names.update(names)
        self.router = self.correction = self.bias = self.w_up = self.w_down = self.s_up = self.s_down = self.s_gate = None
        self.table = None

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        n, h, x = self.names, self.hidden, self.sfx
        specs = []
        for e in range(self.E):
            ep = prefix + n["expert"].format(e)
            if self.gated:
                specs.append(TensorSpec(f"{ep}{n['gate']}{x}", (self.ff, h)))
            specs += [TensorSpec(f"{ep}{n['up']}{x}", (self.ff, h)), TensorSpec(f"{ep}{n['down']}{x}", (h, self.ff))]
        if self.by_table:
            # (the random-weights writer draws rows of distinct expert indices)
            specs.append(TensorSpec(f"{prefix}{n['table']}", (self.vocab, self.top), role="table", init=f"distinct:{self.E}"))
        else:
            # the router works in float32 whatever the activation dtype
            specs.append(TensorSpec(f"{prefix}{n['router']}{x}", (self.E + self.I, h), role="vector"))
        if self.score == "softmax" and not self.by_table:
            specs.append(TensorSpec(f"{prefix}{n['correction']}", (self.E + self.I,), role="vector", init="zeros"))
        if self.router_bias:
            specs.append(TensorSpec(f"{prefix}{n['router_bias']}", (self.E + self.I,), role="vector"))
        if self.shared_ff is not None:
            sp = prefix + n["shared"]
            if self.gated:
                specs.append(TensorSpec(f"{sp}{n['gate']}{x}", (self.shared_ff, h)))
            specs += [TensorSpec(f"{sp}{n['up']}{x}", (self.shared_ff, h)), TensorSpec(f"{sp}{n['down']}{x}", (h, self.shared_ff))]
        return specs

    def bind(self, tensors, prefix, dtype):
        n, x = self.names, self.sfx
        if self.E > 0:
            ups = [tensors[f"{prefix}{n['expert'].format(e)}{n['up']}{x}"] for e in range(self.E)]
            downs = [tensors[f"{prefix}{n['expert'].format(e)}{n['down']}{x}"] for e in range(self.E)]
            self.w_up = torch.stack([t.to(dtype) for t in ups], 0).contiguous()
            if self.gated:
                # rows alternate gate_j, up_j, so that a thread of the product holds a pair and applies the gate itself
                gates = torch.stack([tensors[f"{prefix}{n['expert'].format(e)}{n['gate']}{x}"].to(dtype) for e in range(self.E)], 0)
                self.w_up = torch.stack([gates, self.w_up], 2).reshape(self.E, 2 * self.ff, self.hidden).contiguous()
            self.w_down = torch.stack([t.to(dtype) for t in downs], 0).contiguous()
        if self.by_table:
            self.table = tensors[f"{prefix}{n['table']}"].to(torch.int32).contiguous()
        else:
            self.router = tensors[f"{prefix}{n['router']}{x}"].contiguous()
        self.correction = tensors[f"{prefix}{n['correction']}"].contiguous() if self.score == "softmax" and not self.by_table else None
        self.bias = tensors[f"{prefix}{n['router_bias']}"].contiguous() if self.router_bias else None
        if self.shared_ff is not None:
            sp = prefix + n["shared"]
            self.s_up = tensors[f"{sp}{n['up']}{x}"].contiguous()
            self.s_down = tensors[f"{sp}{n['down']}{x}"].contiguous()
            if self.gated:
                g = tensors[f"{sp}{n['gate']}{x}"]
                self.s_gate = torch.cat([g.to(self.s_up.dtype), self.s_up], 0).contiguous()      # gate | up, one product

    def forward(self, f: torch.Tensor, ctx: Any) -> torch.Tensor:
        if self.by_table:
            ids, wts, plan = ops.moe_table_route(ctx.tokens, self.table, self.E, ctx.status)
        else:
            ids, wts, plan = ops.moe_route(f, self.router, self.correction, self.E, self.top, self.groups, self.keep,
                                           bias=self.bias, score=self.score)
        shared = None
        if self.s_gate is not None:
            shared = ops.linear(ops.linear_swiglu(f, self.s_gate), self.s_down)
        elif self.s_up is not None:
            shared = ops.linear(ops.relu_squared(ops.linear(f, self.s_up)), self.s_down)
        return ops.moe_experts(f, ids, wts, plan, self.w_up, self.w_down, shared, gated=self.gated, act=self.act)


register_feed_forward("sparse_moe", SparseMoE)
