"""Mixers whose state is a matrix per head that every token decays and adds an outer product to: the matrix
memory of the xLSTM (mLSTM) and gated linear attention.

Both keep their matrices in the request's state slot as one float32 row, and their kernel
(``csrc/linear_memory.cu``) walks each sequence of the step in order from the state that earlier steps left, so
a prompt may be cut anywhere and a decode step is the same call with one token per sequence.  Gates, decays, their
logarithms and exponentials, the normalizer and the state are float32 whatever the activation dtype; the gates'
pre-activations leave their products in float32.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from .. import ops
from .base import CacheView, Mixer, StateSpec, TensorSpec, register_mixer


class MatrixMemoryMixer(Mixer):
    """The matrix memory of the xLSTM (Beck et al., "xLSTM: Extended Long Short-Term Memory").

    ``q = W_q x * head_dim^-1/2``, ``k = W_k x`` (``n_heads`` of ``head_dim``), ``v = W_v x`` (``n_heads`` of
    ``v_head_dim``).  Per head a log input gate ``li = cap tanh((W_i x + b_i) / cap)`` and a log forget gate
    ``lf = logsigmoid(cap tanh((W_f x + b_f) / cap))``; with a running maximum m that starts at 0 (like S and n):

        m' = max(lf + m, li);   S <- exp(lf + m - m') S + exp(li - m') k v^T;   n likewise with k alone
        o = S^T q / (max(|n . q|, exp(-m')) + floor_eps)

    Each head's o is divided by its root mean square (``norm_eps`` inside the root), the heads are concatenated and
    multiplied by a weight as wide as all heads and by ``sigmoid(W_g x)``, and ``W_o`` projects the result.  q, k, v
    and the output gate are one product; the two gates are a second one whose result stays float32.
    """

    def __init__(self, hidden: int, n_heads: int, head_dim: int, v_head_dim: int, gate_cap: float, norm_eps: float, *,
                 floor_eps: float = 1e-6, names: Optional[Dict[str, str]] = None, weight_suffix: str = ".weight",
                 bias_suffix: str = ".bias"):
        if n_heads <= 0 or not 1 <= head_dim <= 256 or v_head_dim <= 0:
            raise ValueError(f"{n_heads} heads of {head_dim} x {v_head_dim} (keys up to 256)")
        if not gate_cap > 0:
            raise ValueError("the gates' cap must be positive")
        self.hidden, self.nh, self.dk, self.dv = int(hidden), int(n_heads), int(head_dim), int(v_head_dim)
        self.cap, self.eps, self.floor_eps = float(gate_cap), float(norm_eps), float(floor_eps)
        self.sfx, self.bsfx = weight_suffix, bias_suffix
        self.names = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "g": "g_proj", "o": "o_proj", "i": "igate", "f": "fgate",
                      "norm": "norm"}
        if names:
            self.names.update(names)
        self.w_in = self.w_gates = self.b_gates = self.norm_w = self.w_o = None

    def cache_spec(self):
        return StateSpec("matrix_memory", (self.nh * self.dk * self.dv + self.nh * self.dk + self.nh,), torch.float32)

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        n, h, x, b = self.names, self.hidden, self.sfx, self.bsfx
        qk, vv = self.nh * self.dk, self.nh * self.dv
        return [TensorSpec(f"{prefix}{n['q']}{x}", (qk, h)), TensorSpec(f"{prefix}{n['k']}{x}", (qk, h)),
                TensorSpec(f"{prefix}{n['v']}{x}", (vv, h)), TensorSpec(f"{prefix}{n['g']}{x}", (vv, h)),
                TensorSpec(f"{prefix}{n['o']}{x}", (h, vv)),
                TensorSpec(f"{prefix}{n['norm']}", (vv,), role="vector", init="ones"),
                TensorSpec(f"{prefix}{n['i']}{x}", (self.nh, h)), TensorSpec(f"{prefix}{n['i']}{b}", (self.nh,), role="vector"),
                TensorSpec(f"{prefix}{n['f']}{x}", (self.nh, h)), TensorSpec(f"{prefix}{n['f']}{b}", (self.nh,), role="vector")]

    def bind(self, tensors, prefix, dtype):
        n, x, b = self.names, self.sfx, self.bsfx
        parts = [tensors[f"{prefix}{n[r]}{x}"] for r in ("q", "k", "v", "g")]
        wd = parts[0].dtype if all(p.dtype == parts[0].dtype for p in parts) else torch.float32
        self.w_in = torch.cat([p.to(wd) for p in parts], 0).contiguous()                  # q | k | v | g
        gi, gf = tensors[f"{prefix}{n['i']}{x}"], tensors[f"{prefix}{n['f']}{x}"]
        gd = gi.dtype if gi.dtype == gf.dtype else torch.float32
        self.w_gates = torch.cat([gi.to(gd), gf.to(gd)], 0).contiguous()                  # input gates | forget gates
        self.b_gates = torch.cat([tensors[f"{prefix}{n['i']}{b}"], tensors[f"{prefix}{n['f']}{b}"]], 0).contiguous()
        self.norm_w = tensors[f"{prefix}{n['norm']}"].contiguous()
        self.w_o = tensors[f"{prefix}{n['o']}{x}"].contiguous()

    def forward(self, a: torch.Tensor, ctx: Any, cache: CacheView) -> torch.Tensor:
        nh, dk, dv = self.nh, self.dk, self.dv
        h = ops.linear(a, self.w_in)
        gates = ops.linear(a, self.w_gates, None, torch.float32)
        o = ops.matrix_memory(h, gates, self.b_gates, self.cap, cache.tensor, ctx.state_slots, ctx.cu_q, ctx.positions,
                              nh, dk, dv, dk ** -0.5, self.floor_eps, ctx.status, max_q=ctx.max_q)
        off = 2 * nh * dk + nh * dv
        y = ops.gated_group_rmsnorm(o, h[:, off:off + nh * dv], self.norm_w, self.eps, dv, False, h.dtype, gate="sigmoid")
        return ops.linear(y, self.w_o)


class GatedLinearAttentionMixer(Mixer):
    """Gated linear attention (Yang et al., "Gated Linear Attention Transformers with Hardware-Efficient Training").

    ``q = W_q x * head_dim^-1/2``, ``k = W_k x`` (``n_heads`` of ``head_dim``), ``v = W_v x`` (``n_heads`` of
    ``v_head_dim``).  A decay per key channel through a low-rank pair: ``z = W_a2 (W_a1 x) + b_a2`` laid out heads x
    head_dim, ``alpha = sigmoid(z)^(1/tau)``.  Per head ``S <- diag(alpha) S + k v^T`` and ``o = S^T q``.  Each
    head's o is RMS-normed over ``v_head_dim`` with one weight shared by the heads, the heads are concatenated and
    multiplied by ``silu(W_g x)``, and ``W_o`` projects the result.  q, k, v and the gate are one product.
    """

    def __init__(self, hidden: int, n_heads: int, head_dim: int, v_head_dim: int, tau: float, norm_eps: float, *,
                 names: Optional[Dict[str, str]] = None, weight_suffix: str = ".weight", bias_suffix: str = ".bias"):
        if n_heads <= 0 or not 1 <= head_dim <= 256 or v_head_dim <= 0:
            raise ValueError(f"{n_heads} heads of {head_dim} x {v_head_dim} (keys up to 256)")
        if not tau > 0:
            raise ValueError("tau must be positive")
        self.hidden, self.nh, self.dk, self.dv = int(hidden), int(n_heads), int(head_dim), int(v_head_dim)
        self.tau, self.eps, self.sfx, self.bsfx = float(tau), float(norm_eps), weight_suffix, bias_suffix
        self.names = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "g": "g_proj", "o": "o_proj", "a1": "gk_proj.0",
                      "a2": "gk_proj.1", "norm": "g_norm"}
        if names:
            self.names.update(names)
        self.rank: Optional[int] = None
        self.w_in = self.w_a1 = self.w_a2 = self.b_a2 = self.norm_w = self.w_o = None

    def cache_spec(self):
        return StateSpec("gated_linear_attention", (self.nh * self.dk * self.dv,), torch.float32)

    def with_rank(self, rank: int) -> "GatedLinearAttentionMixer":
        """The width of the decay's low-rank pair (a size that only the checkpoint's shapes give)."""
        self.rank = int(rank)
        return self

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        n, h, x, b = self.names, self.hidden, self.sfx, self.bsfx
        qk, vv = self.nh * self.dk, self.nh * self.dv
        r = self.rank if self.rank is not None else -1          # -1: any size, as long as the pair agrees
        return [TensorSpec(f"{prefix}{n['q']}{x}", (qk, h)), TensorSpec(f"{prefix}{n['k']}{x}", (qk, h)),
                TensorSpec(f"{prefix}{n['v']}{x}", (vv, h)), TensorSpec(f"{prefix}{n['g']}{x}", (vv, h)),
                TensorSpec(f"{prefix}{n['o']}{x}", (h, vv)),
                TensorSpec(f"{prefix}{n['norm']}", (self.dv,), role="vector", init="ones"),
                TensorSpec(f"{prefix}{n['a1']}{x}", (r, h)), TensorSpec(f"{prefix}{n['a2']}{x}", (qk, r)),
                TensorSpec(f"{prefix}{n['a2']}{b}", (qk,), role="vector")]

    def bind(self, tensors, prefix, dtype):
        n, x, b = self.names, self.sfx, self.bsfx
        parts = [tensors[f"{prefix}{n[r]}{x}"] for r in ("q", "k", "v", "g")]
        wd = parts[0].dtype if all(p.dtype == parts[0].dtype for p in parts) else torch.float32
        self.w_in = torch.cat([p.to(wd) for p in parts], 0).contiguous()                  # q | k | v | g
        self.w_a1 = tensors[f"{prefix}{n['a1']}{x}"].contiguous()
        self.w_a2 = tensors[f"{prefix}{n['a2']}{x}"].contiguous()
        if self.w_a1.shape[0] != self.w_a2.shape[1]:
            raise ValueError(f"the decay's pair does not fit: {tuple(self.w_a1.shape)} and {tuple(self.w_a2.shape)}")
        self.b_a2 = tensors[f"{prefix}{n['a2']}{b}"].contiguous()
        self.norm_w = tensors[f"{prefix}{n['norm']}"].contiguous()
        self.w_o = tensors[f"{prefix}{n['o']}{x}"].contiguous()

    def forward(self, a: torch.Tensor, ctx: Any, cache: CacheView) -> torch.Tensor:
        nh, dk, dv = self.nh, self.dk, self.dv
        h = ops.linear(a, self.w_in)
        z = ops.linear(ops.linear(a, self.w_a1), self.w_a2, self.b_a2, torch.float32)
        o = ops.gated_linear_attention(h, z, self.tau, cache.tensor, ctx.state_slots, ctx.cu_q, ctx.positions, nh, dk, dv,
                                       dk ** -0.5, ctx.status, max_q=ctx.max_q)
        off = 2 * nh * dk + nh * dv
        y = ops.gated_group_rmsnorm(o, h[:, off:off + nh * dv], self.norm_w, self.eps, dv, False, h.dtype)
        return ops.linear(y, self.w_o)


register_mixer("matrix_memory", MatrixMemoryMixer)
register_mixer("gated_linear_attention", GatedLinearAttentionMixer)
